"""FP8 (e4m3, fp32 block scales) path: quantisation, the two-level-accumulation expert GEMM and the layer
(torch_dtype 4), against the fp32 oracle run on the SAME quantised operands (de-quantised on the host)."""
import numpy as np
import pytest

from helpers import TOL_BF16_MAX, TOL_BF16_MEAN, make_inputs, rel_errors, to_dev

pytestmark = pytest.mark.gpu


def _mods():
    import torch
    import cuplayground_b200 as cp
    import cuplayground_b200.layer as layer
    return torch, cp, layer


def test_e4m3_tables_roundtrip(oracle):
    codes = np.arange(256, dtype=np.uint8)
    vals = oracle.e4m3_decode(codes)
    finite = ~np.isnan(vals)
    assert finite.sum() == 254 and np.nanmax(vals) == 448.0 and vals[0x08] == 2.0 ** -6
    back = oracle.e4m3_encode(vals[finite])
    ok = (back == codes[finite]) | (vals[finite] == 0)           # +0 / -0 both decode to zero
    assert ok.all()
    assert oracle.e4m3_encode(np.array([1e9, -1e9, 0.0625 + 1e-9], np.float32)).tolist()[:2] == [0x7E, 0xFE]


def test_quantize_fp8_matches_committed_golden_codes():
    """A row whose largest magnitude is 448 gets scale 1, so its codes are the raw e4m3 encoding: compared with the
    committed probe of rounding ties, subnormals and the saturation edge (tests/golden/case2_oracle.npz)."""
    import os
    import torch
    import cuplayground_b200.layer as layer
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "case2_oracle.npz"))
    keep = np.abs(g["e4m3_probe"]) <= 448.0
    row = np.zeros((1, 128), np.float32)
    row[0, :keep.sum()] = g["e4m3_probe"][keep]
    q, s = layer.quantize_fp8(torch.from_numpy(row).cuda(), 1)
    assert float(s[0, 0]) == 1.0
    np.testing.assert_array_equal(q.cpu().numpy()[0, :keep.sum()], g["e4m3_codes"][keep])


@pytest.mark.parametrize("block_rows,shape", [(1, (300, 512)), (128, (3, 200, 384)), (128, (2, 256, 256))])
def test_quantize_fp8_matches_numpy(oracle, block_rows, shape):
    torch, cp, layer = _mods()
    rng = np.random.default_rng(5)
    src = oracle.round_bf16((rng.standard_normal(shape) * rng.uniform(0.01, 3.0, size=shape[:-1] + (1,))).astype(np.float32))
    src.reshape(-1)[::97] = 0.0
    q, s = layer.quantize_fp8(to_dev(src, torch.bfloat16), block_rows)
    q, s = q.cpu().numpy(), s.cpu().numpy()
    # reference: amax per block / 448 in fp32, codes = round-to-nearest-even of x * (1 / scale)
    rows, cols = shape[-2], shape[-1]
    a = np.abs(src).reshape(-1, rows, cols)
    if block_rows == 1:
        amax = a.reshape(-1, rows, cols // 128, 128).max(-1)
        ref_s = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32).reshape(s.shape)
        full = np.repeat(ref_s.reshape(-1, rows, cols // 128), 128, axis=-1)
    else:
        pad = (-rows) % 128
        ap = np.pad(a, ((0, 0), (0, pad), (0, 0)))
        amax = ap.reshape(-1, (rows + pad) // 128, 128, cols // 128, 128).max((2, 4))
        ref_s = np.where(amax > 0, amax / np.float32(448.0), np.float32(1.0)).astype(np.float32).reshape(s.shape)
        full = np.repeat(np.repeat(ref_s.reshape(-1, (rows + pad) // 128, cols // 128), 128, axis=1)[:, :rows], 128, axis=2)
    np.testing.assert_array_equal(s, ref_s)
    inv = (np.float32(1.0) / full).astype(np.float32)
    ref_q = oracle.e4m3_encode((src.reshape(-1, rows, cols) * inv).astype(np.float32)).reshape(q.shape)
    zero = src == 0
    assert ((q == ref_q) | zero).all()
    dq = oracle.dequantize_fp8(q, s, block_rows)
    assert np.abs(dq - src).max() <= np.abs(src).max() * 2.0 ** -4 * 1.01       # 3 mantissa bits


@pytest.mark.parametrize("E,rows,H,I,act,counts", [
    (1, 128, 128, 128, 0, [128]),                         # one tile, one K block
    (2, 200, 512, 256, 1, [200, 77]),                     # GELU, 4 K blocks, ragged rows
    (3, 300, 256, 384, 2, [300, 0, 129]),                 # SwiGLU (64 + 64 column tiles), an empty expert
    (4, 160, 1024, 512, 2, [160, 1, 128, 33]),
])
def test_expert_ffn_fp8_parity(oracle, E, rows, H, I, act, counts):
    torch, cp, layer = _mods()
    x, _, w1, w3, w2 = make_inputs(E * rows, H, I, E, seed=61, swiglu=(act == 2), w_std=0.05)
    dt = torch.bfloat16
    xq, sx = layer.quantize_fp8(to_dev(x.reshape(E, rows, H), dt), 1)
    w1q, s1 = layer.quantize_fp8(to_dev(w1, dt), 128)
    w2q, s2 = layer.quantize_fp8(to_dev(w2, dt), 128)
    w3q, s3 = layer.quantize_fp8(to_dev(w3, dt), 128) if act == 2 else (None, None)
    count = np.array(counts, np.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = layer.expert_ffn_fp8(xq, sx, torch.from_numpy(count).cuda(), w1q, s1, w3q, s3, w2q, s2, act, dev_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    host = lambda t: None if t is None else t.cpu().numpy()
    dq = lambda q, s, b: None if q is None else oracle.dequantize_fp8(host(q), host(s), b)
    # fp32 recomputation of the same pipeline: same quantised operands, hidden activations rounded to bf16 and
    # re-quantised to e4m3 per 128 values before the down projection
    ref = oracle.expert_ffn(dq(xq, sx, 1), count, dq(w1q, s1, 128), dq(w3q, s3, 128), dq(w2q, s2, 128), act, round_h=2)
    got = y.float().cpu().numpy()
    for e in range(E):
        n = counts[e]
        assert (got[e, n:] == 0).all(), "rows past the group's count are not written"
        if n:
            mx, mean = rel_errors(got[e, :n], ref[e, :n])
            assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (e, mx, mean)


def _fp8_layer_case(oracle, cfg, seed, n_sample=None):
    torch, cp, layer = _mods()
    S, H, I, E = cfg.S, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    dt = torch.bfloat16
    mk = lambda shape, std, sid: layer.fill_normal(torch.empty(shape, dtype=dt, device="cuda"), 0.0, std, seed, sid)
    x, wg = mk((S, H), 1.0, 0), mk((E, H), 0.02, 1)
    swiglu = cfg.hidden_act == 2
    w1q, s1 = layer.quantize_fp8(mk((E, I, H), 0.02, 2), 128)
    w3q, s3 = layer.quantize_fp8(mk((E, I, H), 0.02, 3), 128) if swiglu else (None, None)
    w2q, s2 = layer.quantize_fp8(mk((E, H, I), 0.02, 4), 128)
    scales = torch.cat([t.reshape(-1) for t in (s1, s3, s2) if t is not None]).contiguous()
    L = layer.MoELayer(cfg)
    out = L.forward(x, wg, w1q, w3q, w2q, scales=scales)
    L.status()
    out2 = L.forward(x, wg, w1q, w3q, w2q, scales=scales)
    L.status()
    assert torch.equal(out, out2)
    r = L.routing()
    xq, sx = layer.quantize_fp8(x, 1)                     # the same quantiser the layer runs on the tokens
    host = lambda t: None if t is None else t.cpu().numpy()
    dq = lambda q, s, b: None if q is None else oracle.dequantize_fp8(host(q), host(s), b)
    rows = None if n_sample is None else np.random.default_rng(1).choice(S, size=n_sample, replace=False).astype(np.int32)
    ref = oracle.moe_forward(x.float().cpu().numpy(), wg.float().cpu().numpy(), dq(w1q, s1, 128), dq(w3q, s3, 128),
                             dq(w2q, s2, 128), k=cfg.expert_top_k, cap=cfg.capacity, gate_fn=cfg.gate_fn,
                             renorm=cfg.renorm_topk, hidden_act=cfg.hidden_act, only_rows=rows, x_ffn=dq(xq, sx, 1),
                             round_h=2)
    for name in ("topk_idx", "count", "slot_of", "token_of_slot"):
        np.testing.assert_array_equal(r[name].numpy(), ref[name])
    got = out.float().cpu().numpy() if rows is None else out[torch.from_numpy(rows.astype(np.int64)).cuda()].float().cpu().numpy()
    mx, mean = rel_errors(got, ref["out"])
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mx, mean)
    L.close()


def test_layer_fp8_small(oracle):
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(drop_tokens=0, expert_top_k=4, hidden_act=2, hidden_size=512, intermediate_size=256,
                           num_experts=16, torch_dtype=4, tokens=384, gate_fn=1, renorm_topk=1)
    _fp8_layer_case(oracle, cfg, seed=3)


def test_layer_fp8_with_drops_gelu(oracle):
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(capacity_factor=1.0, drop_tokens=1, expert_top_k=2, hidden_act=1, hidden_size=512,
                           intermediate_size=384, num_experts=8, torch_dtype=4, tokens=640)
    _fp8_layer_case(oracle, cfg, seed=9)


def test_config4_rank_shape(oracle):
    """DeepSeek-V3-shaped case at the size one of eight ranks computes: H=7168, I=2048, SwiGLU, top-8 sigmoid gate
    normalised over the selected experts, no drops, FP8 weights with 128x128 block scales - with the 32 experts a rank
    owns (the full layer has 256) and 4096 tokens. Routing on every token, outputs on a 64-token sample."""
    torch, cp, layer = _mods()
    cfg = cp.baseline_config(4)
    cfg.num_experts = 32
    _fp8_layer_case(oracle, cfg, seed=3, n_sample=64)


def test_config4_full_layer_on_one_gpu(oracle):
    """The whole DeepSeek-V3-shaped layer on one GPU: all 256 experts, 4096 tokens, H 7168, top-8 sigmoid gate
    normalised over the selected experts, no drops, FP8 operands. With E = 256 the layer's gate is the tensor-core
    screen + exact candidates, so this is the screened gate checked through the layer at the shape with the longest
    accumulation chains: routing bit-exact on every token, 8 sampled output rows (up to 64 experts' weights
    regenerated and de-quantised on the host) against the oracle."""
    torch, cp, layer = _mods()
    import parity
    cfg = cp.baseline_config(4, world=1)
    assert cfg.num_experts == 256 and cfg.S == 4096
    x, wg, w1, w3, w2, scales = layer.synthetic_tensors(cfg, 0, 1)
    L = layer.MoELayer(cfg)
    out = L.forward(x, wg, w1, w3, w2, scales=scales)
    L.status()
    out2 = L.forward(x, wg, w1, w3, w2, scales=scales)
    L.status()
    assert torch.equal(out, out2)
    res = parity.check_rank(cfg, L, x, wg, out, n_rows=8, seed=4)
    assert res["ok"], res
    L.close()


_FFN_HASH = r"""
import hashlib, sys
import numpy as np, torch
import cuplayground_b200.layer as layer
out = []
for (E, rows, H, I, act) in [(4, 640, 1024, 1536, 1), (3, 384, 512, 512, 2), (2, 256, 2048, 1024, 0)]:
    g = torch.Generator(device="cuda").manual_seed(7)
    mk = lambda shape, std: (torch.randn(shape, device="cuda", generator=g) * std).to(torch.bfloat16)
    x, w1, w3, w2 = mk((E, rows, H), 1.0), mk((E, I, H), 0.05), mk((E, I, H), 0.05), mk((E, H, I), 0.05)
    xq, sx = layer.quantize_fp8(x, 1)
    w1q, s1 = layer.quantize_fp8(w1, 128)
    w3q, s3 = layer.quantize_fp8(w3, 128) if act == 2 else (None, None)
    w2q, s2 = layer.quantize_fp8(w2, 128)
    cnt = np.array([rows - (37 * e) % rows if e % 3 else rows for e in range(E)], dtype=np.int32)
    if E == 3: cnt[1] = 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = layer.expert_ffn_fp8(xq, sx, torch.from_numpy(cnt).cuda(), w1q, s1, w3q, s3, w2q, s2, act, dev_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    yh = y.float().cpu().numpy()
    for e in range(E): yh[e, cnt[e]:] = 0
    assert np.isfinite(yh).all() and np.abs(yh).max() > 0
    out.append(hashlib.sha256(yh.tobytes()).hexdigest())
print("HASHES", *out)
"""


def test_hidden_activations_quantised_in_the_epilogue_give_the_same_bits():
    """The up projection quantises its own output rows; with ARISTOS_FP8_FUSED_QUANT=0 it writes bf16 and a kernel
    of its own quantises that. Both must give bit-identical expert outputs (ragged counts, an empty expert,
    ReLU / GELU / SwiGLU)."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    got = {}
    for fused in ("1", "0"):
        env = dict(os.environ, ARISTOS_FP8_FUSED_QUANT=fused, PYTHONPATH=root)
        r = subprocess.run([sys.executable, "-c", _FFN_HASH], cwd=root, env=env, capture_output=True, text=True,
                           timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        got[fused] = [l for l in r.stdout.splitlines() if l.startswith("HASHES")][-1]
    assert got["1"] == got["0"]
