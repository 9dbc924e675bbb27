"""Parity of one rank of a (possibly expert-parallel) layer against the CPU oracle, at any size.

Used by the multi-GPU tests and by bench.py's parity leg (checker only; nothing here is timed). The oracle never
sees more than one expert's weights at a time, so the Mixtral- and DeepSeek-shaped configurations fit in host
memory: routing is recomputed for every token of the rank (gate logits, top-k, dispatch: bit-exact), the output for
a sample of token rows (per expert: the oracle's expert FFN over the sampled rows that use it; then the weighted
combine in increasing j, fp32, as the oracle's combine does).
"""
from __future__ import annotations

import numpy as np

from oracle import moe_oracle as O

TOL_MAX, TOL_MEAN = 2e-2, 1e-2      # 16-bit / fp8 outputs: max-relative and mean-relative against the fp32 oracle


def global_expert_weights(cfg, e: int):
    """Host fp32 copies of expert e's weights as the synthetic generator of cuplayground_b200.layer makes them
    (expert e draws from its own Philox streams, so any rank can regenerate any expert on its GPU). For
    torch_dtype 4 the weights are quantised to e4m3 with 128x128-block scales exactly as the layer's inputs are and
    de-quantised here."""
    import torch
    import cuplayground_b200.layer as layer
    fp8 = cfg.torch_dtype == 4
    H, I = cfg.hidden_size, cfg.intermediate_size
    dt = layer._TORCH_DTYPE[cfg.torch_dtype]

    def one(rows, cols, which):
        w = layer.fill_normal(torch.empty((rows, cols), dtype=dt, device="cuda"), 0.0, 0.02, cfg.seed,
                              16 * (e + 1) + which)
        if not fp8:
            return w.float().cpu().numpy()
        q, s = layer.quantize_fp8(w, 128)
        return O.dequantize_fp8(q.cpu().numpy(), s.cpu().numpy(), 128)

    w1 = one(I, H, 2)
    w3 = one(I, H, 3) if cfg.hidden_act == 2 else None
    w2 = one(H, I, 4)
    return w1, w3, w2


def check_rank(cfg, L, x, wg, out, *, n_rows: int = 64, seed: int = 0, expert_weights=None, gate_bias=None) -> dict:
    """x, wg, out: this rank's device tensors of the forward that just ran on layer L. expert_weights(e) returns
    the host fp32 (w1, w3, w2) of GLOBAL expert e (default: regenerate the synthetic weights). Raises
    AssertionError on a routing mismatch; returns dict(rows, max_rel, mean_rel, kept, routing='bit-exact')."""
    import torch
    import cuplayground_b200.layer as layer
    if expert_weights is None:
        expert_weights = lambda e: global_expert_weights(cfg, e)
    S, H, E, k = cfg.S, cfg.hidden_size, cfg.num_experts, cfg.expert_top_k
    cap = cfg.capacity
    fp8 = cfg.torch_dtype == 4
    r = L.routing()
    xh = x.float().cpu().numpy()
    bias = gate_bias
    if bias is None and cfg.gate_bias_zipf_s > 0:
        bias = O.zipf_bias(E, cfg.gate_bias_zipf_s)
    logits = O.gate_logits(xh, wg.float().cpu().numpy(), bias)
    idx, w = O.gate_topk(logits, k, cfg.gate_fn, cfg.renorm_topk)
    count, slot_of, tos = O.dispatch(idx, E, cap)
    assert np.array_equal(r["topk_idx"].numpy(), idx), "top-k expert indices differ from the oracle"
    assert np.array_equal(r["count"].numpy(), count), "per-expert counts differ from the oracle"
    assert np.array_equal(r["slot_of"].numpy(), slot_of), "slot assignment (drops, token order) differs from the oracle"
    assert np.array_equal(r["token_of_slot"].numpy(), tos), "token lists differ from the oracle"
    assert np.allclose(r["topk_w"].numpy(), w, rtol=1e-5, atol=1e-7), "gate weights differ from the oracle"

    rows = np.sort(np.random.default_rng(seed).choice(S, size=min(n_rows, S), replace=False)).astype(np.int64)
    x_ffn = xh[rows]
    if fp8:       # the experts see the quantised tokens
        xq, sx = layer.quantize_fp8(x[torch.from_numpy(rows).cuda()].contiguous(), 1)
        x_ffn = O.dequantize_fp8(xq.cpu().numpy(), sx.cpu().numpy(), 1)
    ref = np.zeros((rows.size, H), dtype=np.float32)
    sel_e = idx[rows]                                   # (n, k)
    kept = slot_of[rows] >= 0
    y_of = np.zeros((rows.size, k, H), dtype=np.float32)
    for e in np.unique(sel_e[kept]):
        ii, jj = np.nonzero((sel_e == e) & kept)
        w1, w3, w2 = expert_weights(int(e))
        xg = np.ascontiguousarray(x_ffn[ii])[None]
        y = O.expert_ffn(xg, np.array([ii.size], dtype=np.int32), w1[None], None if w3 is None else w3[None], w2[None],
                         cfg.hidden_act, round_h=2 if fp8 else 0)
        y_of[ii, jj] = y[0]
    for j in range(k):                                  # the oracle's combine: increasing j, fp32 fmaf per element
        wj = np.where(kept[:, j], w[rows, j], 0.0).astype(np.float32)[:, None]
        ref = (ref.astype(np.float64) + wj.astype(np.float64) * y_of[:, j].astype(np.float64)).astype(np.float32)
    got = out[torch.from_numpy(rows).cuda()].float().cpu().numpy()
    d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    max_rel = float(d.max() / max(np.abs(ref).max(), 1e-30))
    mean_rel = float(d.mean() / max(np.abs(ref).mean(), 1e-30))
    return dict(rows=int(rows.size), max_rel=max_rel, mean_rel=mean_rel, kept=int(kept.sum()), routing="bit-exact",
                ok=bool(max_rel < TOL_MAX and mean_rel < TOL_MEAN))
