"""GPU parity of every stage against the CPU oracle, called through the C ABI (ctypes)."""
import numpy as np
import pytest

from helpers import TOL_BF16_MAX, TOL_BF16_MEAN, TOL_F32_MAX, make_inputs, rel_errors, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cp():
    import cuplayground_b200.layer as layer
    return layer


def _torch():
    import torch
    return torch


@pytest.mark.parametrize("S,H,E,k,gate_fn,renorm,bf16,bias", [
    (128, 256, 8, 1, 0, 0, False, False),      # the fp32 reference case
    (333, 320, 8, 2, 0, 1, True, False),       # ragged S, H with a partial 32-chunk sweep
    (512, 2048, 64, 2, 0, 1, True, False),     # gate of the single-GPU case
    (256, 4096, 8, 2, 0, 0, True, False),      # gate of the Mixtral-shaped case
    (200, 1024, 128, 4, 0, 0, True, True),     # skewed case: Zipf prior on the logits
    (96, 448, 256, 8, 1, 1, True, False),      # sigmoid gate, many experts
    (64, 64, 3, 3, 0, 0, True, False),         # k == E, E not a multiple of the register tile
])
def test_gate_parity(cp, oracle, S, H, E, k, gate_fn, renorm, bf16, bias):
    torch = _torch()
    x, wg, *_ = make_inputs(S, H, 64, E, seed=11, bf16=bf16)
    wg = wg * 8.0 if bf16 else wg      # spread the logits a little (still exact in bf16)
    b = oracle.zipf_bias(E, 1.2) if bias else None
    dt = torch.bfloat16 if bf16 else torch.float32
    idx, w, logits = cp.gate_topk(to_dev(x, dt), to_dev(wg, dt), k, gate_fn, renorm,
                                  gate_bias=to_dev(b, torch.float32), want_logits=True)
    ref_logits = oracle.gate_logits(x, wg, b)
    ref_idx, ref_w = oracle.gate_topk(ref_logits, k, gate_fn, renorm)
    np.testing.assert_array_equal(logits.cpu().numpy().view(np.uint32), ref_logits.view(np.uint32))  # bit-exact
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx)
    np.testing.assert_allclose(w.cpu().numpy(), ref_w, rtol=2e-5, atol=1e-7)


def test_gate_ties_go_to_lower_index(cp, oracle):
    torch = _torch()
    S, H, E, k = 40, 64, 16, 3
    x = np.ones((S, H), np.float32)
    wg = np.zeros((E, H), np.float32)
    wg[3] = wg[7] = wg[11] = 0.5     # three exact ties above the rest, the rest tie at zero
    idx, w = cp.gate_topk(to_dev(x, torch.bfloat16), to_dev(wg, torch.bfloat16), k)
    ref_idx, _ = oracle.gate_topk(oracle.gate_logits(x, wg), k)
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx)
    assert (idx.cpu().numpy() == np.array([3, 7, 11])).all()
    idx5, _ = cp.gate_topk(to_dev(x, torch.bfloat16), to_dev(wg, torch.bfloat16), 5)
    assert (idx5.cpu().numpy() == np.array([3, 7, 11, 0, 1])).all()


@pytest.mark.parametrize("S,H,E,k,gate_fn,renorm,f16,bias", [
    (512, 2048, 64, 2, 0, 1, False, False),    # gate of the single-GPU case
    (777, 1024, 128, 4, 0, 0, False, True),    # skewed case (Zipf prior), ragged S
    (96, 448, 256, 8, 1, 1, False, False),     # sigmoid gate, H not a multiple of the 64-element K block
    (300, 7168, 256, 8, 1, 1, False, False),   # gate of the fine-grained case: long rows, H split over CTAs
    (260, 512, 36, 3, 0, 0, True, False),      # fp16, E not a multiple of 16
    (1, 64, 32, 1, 0, 0, False, False),        # one token
])
def test_gate_screened_parity(cp, oracle, S, H, E, k, gate_fn, renorm, f16, bias):
    """Tensor-core screen + exact candidates: routing identical to the all-experts contract, weights to rounding,
    and the screen's error bound holds on every candidate (status word stays 0)."""
    torch = _torch()
    x, wg, *_ = make_inputs(S, H, 64, E, seed=23, bf16=not f16, f16=f16)
    wg = wg * 8.0
    b = oracle.zipf_bias(E, 1.2) if bias else None
    dt = torch.float16 if f16 else torch.bfloat16
    idx, w, status = cp.gate_topk_screened(to_dev(x, dt), to_dev(wg, dt), k, gate_fn, renorm,
                                           gate_bias=to_dev(b, torch.float32))
    ref_idx, ref_w = oracle.gate_topk(oracle.gate_logits(x, wg, b), k, gate_fn, renorm)
    assert int(status.item()) == 0
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx)
    np.testing.assert_allclose(w.cpu().numpy(), ref_w, rtol=2e-5, atol=1e-7)
    idx2, w2 = cp.gate_topk(to_dev(x, dt), to_dev(wg, dt), k, gate_fn, renorm, gate_bias=to_dev(b, torch.float32))
    assert torch.equal(idx, idx2)
    if gate_fn == 1:
        assert torch.equal(w, w2)          # sigmoid weights depend on the selected (exact) logits only


def test_gate_screened_ties_and_near_ties(cp, oracle):
    """Experts that tie exactly (duplicated rows) or differ in one element by one bf16 step lie inside the screen's
    error interval: all of them must become candidates and the exact logits decide, ties to the lower index."""
    torch = _torch()
    S, H, E, k = 256, 1024, 64, 4
    x, wg, *_ = make_inputs(S, H, 64, E, seed=29, bf16=True)
    wg = wg * 8.0
    wg[32:] = wg[:32]                              # expert e + 32 ties with expert e on every token
    wg = oracle.round_bf16(wg)
    for e, h in ((41, 7), (50, 300), (63, 1023)):  # about one bf16 step away from rows 9, 18, 31 in one element
        wg[e, h] = oracle.round_bf16(np.array([wg[e, h] * (1.0 + 2.0 ** -7)], np.float32))[0]
    idx, w, status = cp.gate_topk_screened(to_dev(x, torch.bfloat16), to_dev(wg, torch.bfloat16), k)
    ref_idx, ref_w = oracle.gate_topk(oracle.gate_logits(x, wg), k)
    assert int(status.item()) == 0
    np.testing.assert_array_equal(idx.cpu().numpy(), ref_idx)
    np.testing.assert_allclose(w.cpu().numpy(), ref_w, rtol=2e-5, atol=1e-7)
    first = idx.cpu().numpy()[:, 0]
    assert ((first < 32) | np.isin(first, (41, 50, 63))).all()     # an exact tie goes to the lower index


def _random_topk(rng, S, E, k, skew):
    p = 1.0 / np.arange(1, E + 1) ** skew
    p /= p.sum()
    return np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(S)]).astype(np.int32)


@pytest.mark.parametrize("S,E,k,cap,skew", [
    (128, 8, 1, 16, 0.0),
    (1000, 8, 2, 250, 0.5),       # ragged: not a multiple of the 2048-assignment chunk
    (8192, 64, 2, 320, 0.3),
    (16384, 8, 2, 5120, 0.2),
    (8192, 128, 4, 256, 1.2),     # Zipf-skewed: several experts overflow
    (4096, 256, 8, 4096, 0.5),    # dropless (cap = S)
    (5, 4, 2, 1, 0.0),            # tiny, capacity 1
    (3000, 1, 1, 100, 0.0),       # one expert, heavy overflow
])
def test_dispatch_parity(cp, oracle, S, E, k, cap, skew):
    torch = _torch()
    rng = np.random.default_rng(S * 31 + E)
    topk = _random_topk(rng, S, E, k, skew)
    count, slot_of, tos = cp.dispatch(torch.from_numpy(topk).cuda(), E, cap)
    rc, rs, rt = oracle.dispatch(topk, E, cap)
    np.testing.assert_array_equal(count.cpu().numpy(), rc)
    np.testing.assert_array_equal(slot_of.cpu().numpy(), rs)
    np.testing.assert_array_equal(tos.cpu().numpy(), rt)


def test_dispatch_empty(cp):
    torch = _torch()
    count, slot_of, tos = cp.dispatch(torch.empty((0, 2), dtype=torch.int32, device="cuda"), 8, 4)
    assert count.cpu().numpy().sum() == 0 and (tos.cpu().numpy() == -1).all()


@pytest.mark.parametrize("bf16", [True, False])
def test_permute_and_combine_parity(cp, oracle, bf16):
    torch = _torch()
    S, H, E, k, cap = 777, 320, 16, 4, 150
    rng = np.random.default_rng(5)
    x, *_ = make_inputs(S, H, 64, E, seed=3, bf16=bf16)
    topk = _random_topk(rng, S, E, k, 0.8)
    count, slot_of, tos = oracle.dispatch(topk, E, cap)
    dt = torch.bfloat16 if bf16 else torch.float32
    xg = cp.permute(to_dev(x, dt), torch.from_numpy(slot_of).cuda(), E * cap, zero=True)
    np.testing.assert_array_equal(xg.float().cpu().numpy(), oracle.permute(x, tos))       # pure copy: exact
    # combine on synthetic expert outputs
    y = oracle.round_bf16(rng.standard_normal((E * cap, H)).astype(np.float32)) if bf16 else \
        rng.standard_normal((E * cap, H)).astype(np.float32)
    w = rng.random((S, k)).astype(np.float32)
    out = cp.combine(to_dev(y, dt), torch.from_numpy(slot_of).cuda(), torch.from_numpy(w).cuda())
    ref = oracle.combine(y, slot_of, w)
    if bf16:
        np.testing.assert_array_equal(out.float().cpu().numpy(), oracle.round_bf16(ref))   # same fma order
    else:
        np.testing.assert_array_equal(out.cpu().numpy(), ref)


def test_combine_identity_fixture(cp):
    """The reference's hostCombine fixture (auditorium/combine.cuh:219-231): identity indices, row i filled with
    i + 1 -> activations row i == i + 1."""
    torch = _torch()
    M, N = 128, 64
    y = torch.arange(1, M + 1, dtype=torch.float32, device="cuda")[:, None].expand(M, N).contiguous()
    slot_of = torch.arange(M, dtype=torch.int32, device="cuda")[:, None].contiguous()
    w = torch.ones((M, 1), dtype=torch.float32, device="cuda")
    out = cp.combine(y.to(torch.bfloat16), slot_of, w)
    assert torch.equal(out.float(), y)


@pytest.mark.parametrize("E,rows,H,I,act,counts", [
    (1, 128, 64, 256, 0, [128]),                       # one full tile, one k-block
    (1, 128, 256, 256, 3, [128]),                      # identity epilogue, 4 k-blocks
    (2, 200, 128, 512, 1, [200, 77]),                  # GELU, ragged rows, row tile tail
    (3, 320, 256, 384, 2, [320, 0, 129]),              # SwiGLU, an empty expert, I not a multiple of 128*2
    (4, 40, 2048, 1024, 1, [40, 1, 17, 33]),           # fewer rows than one tile, long K
    (8, 300, 512, 1024, 2, [300, 256, 128, 127, 129, 5, 0, 299]),
])
def test_expert_ffn_bf16_parity(cp, oracle, E, rows, H, I, act, counts):
    torch = _torch()
    x, _, w1, w3, w2 = make_inputs(E * rows, H, I, E, seed=21, swiglu=(act == 2), w_std=0.05)
    xg = x.reshape(E, rows, H)
    count = np.array(counts, np.int32)
    hidden_act = act if act != 3 else 0
    dt = torch.bfloat16
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if act == 3:
        # identity is the epilogue of the down-projection: check it through a ReLU layer whose first GEMM is
        # positive by construction (|x|, |w1|)
        xg, w1 = np.abs(xg), np.abs(w1)
    y = cp.expert_ffn(to_dev(xg, dt), torch.from_numpy(count).cuda(), to_dev(w1, dt), to_dev(w3, dt), to_dev(w2, dt),
                      hidden_act, dev_status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = oracle.expert_ffn(xg, count, w1, w3, w2, hidden_act, round_h=1)
    got = y.float().cpu().numpy()
    for e in range(E):
        n = counts[e]
        assert (got[e, -(-n // 128) * 128:] == 0).all(), "rows past the last valid 128-row tile must not be written"
        if n:
            mx, mean = rel_errors(got[e, :n], ref[e, :n])
            assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (e, mx, mean)


def test_expert_ffn_row_window_and_groups(cp, oracle):
    """Row windows (what the chunked expert-parallel pipeline calls) and group -> expert = g % experts."""
    torch = _torch()
    experts, groups, rows, H, I = 2, 4, 384, 128, 256
    x, _, w1, w3, w2 = make_inputs(groups * rows, H, I, experts, seed=5, swiglu=True, w_std=0.05)
    xg = x.reshape(groups, rows, H)
    count = np.array([384, 130, 0, 257], np.int32)
    dt = torch.bfloat16
    dev = [to_dev(a, dt) for a in (xg, w1, w3, w2)]
    cnt = torch.from_numpy(count).cuda()
    y = torch.zeros((groups, rows, H), dtype=dt, device="cuda")
    h = torch.empty((groups, rows, I), dtype=dt, device="cuda")
    for r0, r1 in ((0, 128), (128, 384)):
        cp.expert_ffn(dev[0], cnt, dev[1], dev[2], dev[3], 2, experts=experts, row_begin=r0, row_end=r1, y=y, h=h)
    got = y.float().cpu().numpy()
    w1g, w3g, w2g = (np.concatenate([w, w]) for w in (w1, w3, w2))     # expert of group g is g % 2
    ref = oracle.expert_ffn(xg, count, w1g, w3g, w2g, 2, round_h=1)
    for g in range(groups):
        n = count[g]
        assert (got[g, -(-n // 128) * 128:] == 0).all()
        if n:
            mx, mean = rel_errors(got[g, :n], ref[g, :n])
            assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (g, mx, mean)


def test_expert_tile_reference_fixture(cp, oracle):
    """The reference's testCollective fixture (mma.cuh:399-411, bias left out: the MoE experts have none):
    A[0:2,0:2] = [[0,1],[2,3]], B[0:2,0:2] = [[4,5],[6,7]], everything else zero, ReLU ->
    C[0:2,0:2] = [[5,7],[23,33]]. The down-projection is an identity matrix so the layer output shows C."""
    torch = _torch()
    M, K, N = 128, 64, 64
    A = np.zeros((1, M, K), np.float32); A[0, :2, :2] = [[0, 1], [2, 3]]
    B = np.zeros((1, N, K), np.float32); B[0, :2, :2] = [[4, 5], [6, 7]]
    W2 = np.eye(N, dtype=np.float32)[None]
    count = torch.tensor([M], dtype=torch.int32, device="cuda")
    for dt in (torch.bfloat16, torch.float32):
        y = cp.expert_ffn(to_dev(A, dt), count, to_dev(B, dt), None, to_dev(W2, dt), 0)
        got = y.float().cpu().numpy()[0]
        assert (got[:2, :2] == np.array([[5, 7], [23, 33]], np.float32)).all()
        assert np.count_nonzero(got) == 4      # all 128 rows are valid here


@pytest.mark.parametrize("act", [0, 1, 2])
def test_expert_ffn_f32_parity(cp, oracle, act):
    torch = _torch()
    E, rows, H, I = 3, 70, 96, 160
    x, _, w1, w3, w2 = make_inputs(E * rows, H, I, E, seed=9, swiglu=(act == 2), bf16=False, w_std=0.05)
    xg = x.reshape(E, rows, H)
    count = np.array([70, 0, 33], np.int32)
    dt = torch.float32
    y = cp.expert_ffn(to_dev(xg, dt), torch.from_numpy(count).cuda(), to_dev(w1, dt), to_dev(w3, dt), to_dev(w2, dt), act)
    ref = oracle.expert_ffn(xg, count, w1, w3, w2, act)
    got = y.cpu().numpy()
    for e in range(E):
        n = count[e]
        assert (got[e, n:] == 0).all()
        if n:
            mx, _ = rel_errors(got[e, :n], ref[e, :n])
            assert mx < TOL_F32_MAX


def test_fill_normal_matches_oracle_generator(cp, oracle):
    torch = _torch()
    n = 100003
    t = torch.empty(n, dtype=torch.float32, device="cuda")
    cp.fill_normal(t, 0.5, 2.0, seed=0x1234567890, stream_id=7)
    ref = oracle.fill_normal(n, 0.5, 2.0, 0x1234567890, 7)
    np.testing.assert_allclose(t.cpu().numpy(), ref, rtol=0, atol=2e-5)
    assert abs(float(t.mean()) - 0.5) < 0.05 and abs(float(t.std()) - 2.0) < 0.05


def test_expert_tile_reference_fixture_with_bias(cp):
    """The reference's testCollective fixture with its bias (mma.cuh:399-411): bias[0:2] = [1,2] ->
    C[0:2,0:2] = [[6,9],[24,35]], and every other row shows ReLU(0 + bias) = [1,2] in its first two columns."""
    torch = _torch()
    M, K, N = 128, 64, 64
    A = np.zeros((1, M, K), np.float32); A[0, :2, :2] = [[0, 1], [2, 3]]
    B = np.zeros((1, N, K), np.float32); B[0, :2, :2] = [[4, 5], [6, 7]]
    bias = np.zeros((1, N), np.float32); bias[0, :2] = [1, 2]
    W2 = np.eye(N, dtype=np.float32)[None]
    count = torch.tensor([M], dtype=torch.int32, device="cuda")
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        y = cp.expert_ffn(to_dev(A, dt), count, to_dev(B, dt), None, to_dev(W2, dt), 0, b1=to_dev(bias, dt))
        got = y.float().cpu().numpy()[0]
        assert (got[:2, :2] == np.array([[6, 9], [24, 35]], np.float32)).all()
        assert (got[2:, :2] == np.array([1, 2], np.float32)).all() and np.count_nonzero(got[:, 2:]) == 0


@pytest.mark.parametrize("act,dtype", [(2, "bf16"), (1, "bf16"), (2, "f16"), (0, "f32"), (2, "f32")])
def test_expert_ffn_bias_parity(cp, oracle, act, dtype):
    """act(acc + bias) in both projections (and on the SwiGLU up branch) against the oracle."""
    torch = _torch()
    from helpers import round_f16
    E, rows, H, I = 3, 200, 128, 384
    bf16, f16 = dtype == "bf16", dtype == "f16"
    x, _, w1, w3, w2 = make_inputs(E * rows, H, I, E, seed=31, swiglu=(act == 2), bf16=bf16, f16=f16, w_std=0.05)
    rnd = oracle.round_bf16 if bf16 else (round_f16 if f16 else (lambda a: a))
    rng = np.random.default_rng(7)
    b1, b3, b2 = (rnd(rng.standard_normal(s).astype(np.float32) * 0.5) for s in ((E, I), (E, I), (E, H)))
    if act != 2:
        b3 = None
    xg = x.reshape(E, rows, H)
    count = np.array([200, 64, 129], np.int32)
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    y = cp.expert_ffn(to_dev(xg, dt), torch.from_numpy(count).cuda(), to_dev(w1, dt), to_dev(w3, dt), to_dev(w2, dt),
                      act, b1=to_dev(b1, dt), b3=to_dev(b3, dt), b2=to_dev(b2, dt))
    ref = oracle.expert_ffn(xg, count, w1, w3, w2, act, round_h=0 if dtype == "f32" else 1, b1=b1, b3=b3, b2=b2)
    got = y.float().cpu().numpy()
    for e in range(E):
        mx, mean = rel_errors(got[e, :count[e]], ref[e, :count[e]])
        if dtype == "f32":
            assert mx < TOL_F32_MAX, (e, mx)
        else:
            assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (e, mx, mean)


@pytest.mark.parametrize("act,E,rows,H,I,counts", [(2, 2, 300, 128, 384, [300, 130]), (1, 3, 128, 256, 256, [128, 0, 7])])
def test_expert_ffn_tf32_parity(cp, oracle, act, E, rows, H, I, counts):
    """fp32 tensors through the tf32 tensor-core path (dtype code 1) against the fp32 oracle."""
    torch = _torch()
    x, _, w1, w3, w2 = make_inputs(E * rows, H, I, E, seed=41, swiglu=(act == 2), bf16=False, w_std=0.05)
    xg = x.reshape(E, rows, H)
    count = np.array(counts, np.int32)
    dt = torch.float32
    rng = np.random.default_rng(1)
    b1, b2 = rng.standard_normal((E, I)).astype(np.float32) * 0.2, rng.standard_normal((E, H)).astype(np.float32) * 0.2
    y = cp.expert_ffn(to_dev(xg, dt), torch.from_numpy(count).cuda(), to_dev(w1, dt), to_dev(w3, dt), to_dev(w2, dt),
                      act, b1=to_dev(b1, dt), b2=to_dev(b2, dt), dtype=1)
    ref = oracle.expert_ffn(xg, count, w1, w3, w2, act, b1=b1, b2=b2)
    got = y.cpu().numpy()
    for e in range(E):
        n = counts[e]
        assert (got[e, -(-n // 128) * 128:] == 0).all()
        if n:
            mx, mean = rel_errors(got[e, :n], ref[e, :n])
            assert mx < 5e-3 and mean < 5e-3, (e, mx, mean)


@pytest.mark.parametrize("act", [2, 1])
def test_expert_ffn_tile_shapes_agree(cp, oracle, act):
    """The expert GEMM with single-CTA tiles, CTA pairs + single-CTA tail (the pair kernel computes whole 256-row
    tiles, the single-CTA kernel every group's last < 256 rows) and padded CTA pairs: ragged row counts around the
    128- and 256-row boundaries; every shape must match the oracle and leave rows past the last valid tile alone."""
    torch = _torch()
    import cuplayground_b200.layer as layer
    experts, rows, H, I = 4, 1152, 128, 256
    counts = [0, 1, 255, 256, 257, 384, 1000, 1152]
    groups = len(counts)
    x, _, w1, w3, w2 = make_inputs(groups * rows, H, I, experts, seed=31, swiglu=(act == 2), w_std=0.05)
    xg = x.reshape(groups, rows, H)
    count = np.array(counts, np.int32)
    dt = torch.bfloat16
    dev = [to_dev(a, dt) for a in (xg, w1, w3, w2)]
    cnt = torch.from_numpy(count).cuda()
    rep = lambda w: None if w is None else np.concatenate([w] * (groups // experts))     # expert of group g: g % 4
    ref = oracle.expert_ffn(xg, count, rep(w1), rep(w3), rep(w2), act, round_h=1)
    outs = {}
    try:
        for mode in (1, 2, 3):
            layer.ffn_set_tile_mode(mode)
            y = cp.expert_ffn(dev[0], cnt, dev[1], dev[2], dev[3], act, experts=experts)
            torch.cuda.synchronize()
            outs[mode] = y.float().cpu().numpy()
    finally:
        layer.ffn_set_tile_mode(-1)
    for mode, got in outs.items():
        pad = 256 if mode == 3 else 128
        for g in range(groups):
            n = counts[g]
            assert (got[g, min(rows, -(-n // pad) * pad):] == 0).all(), (mode, g)
            if n:
                mx, mean = rel_errors(got[g, :n], ref[g, :n])
                assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mode, g, mx, mean)
    for g in range(groups):
        n = counts[g]
        assert np.array_equal(outs[1][g, :n], outs[2][g, :n]) and np.array_equal(outs[1][g, :n], outs[3][g, :n]), \
            f"group {g}: the tile shapes must give the same bits"


def test_bounded_flag_wait_gives_up(cp):
    """The wait of the up projection for a source rank's arrival flag, on a flag that nothing raises: it expires after
    its limit, the kernel returns, the status says so and the context still works."""
    import ctypes as C
    torch = _torch()
    lib = cp._lib.load()
    waited = C.c_int(0)
    assert lib.aristos_selftest_bounded_flag_wait(150, C.byref(waited), None) == 8     # ARISTOS_ERR_DEVICE_TIMEOUT
    assert 150 <= waited.value < 1500, waited.value
    assert int(torch.ones(4, device="cuda").sum().item()) == 4


@pytest.mark.parametrize("f16", [False, True])
def test_gate_screen_stress_equals_exact_gate(cp, f16):
    """The screened gate against the all-experts gate on inputs built to strain the screen's error bound: 102400
    tokens at H = 7168, E = 256, k = 8 (the longest accumulation chains in use); heavy-tailed magnitudes with random
    signs, so that sum |x w| is far above |logit| (large cancellation, mixed magnitudes); and the experts in 16
    clusters of 16 whose weight rows differ from each other in a handful of elements by one unit in the last place,
    so that the k-th place (8 < 16) always falls inside a cluster of near-ties. Both gates must select the same
    experts in the same order for every token, and the screen must not report a violated bound."""
    torch = _torch()
    S, H, E, k = 102400, 7168, 256, 8
    dt = torch.float16 if f16 else torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(1234 + int(f16))
    heavy = lambda *shape: torch.randn(*shape, generator=g, device="cuda") * torch.exp(
        1.5 * torch.randn(*shape, generator=g, device="cuda"))
    x = heavy(S, H).clamp_(-6e4, 6e4).to(dt)
    base = (heavy(16, H) * 0.02).to(dt)
    wg = base.repeat_interleave(16, dim=0).contiguous()              # expert 16 c + i = cluster c
    # one unit in the last place on 1 + i elements of member i (bit pattern + 1 moves a positive value up by one ulp)
    bits = wg.view(torch.int16)
    for i in range(1, 16):
        cols = torch.randint(0, H, (16, i), generator=g, device="cuda")
        rows = (torch.arange(16, device="cuda") * 16 + i)[:, None].expand(16, i)
        bits[rows, cols] += 1
    x, wg = x.contiguous(), wg.contiguous()
    idx_s, w_s, status = cp.gate_topk_screened(x, wg, k, gate_fn=1, renorm=1)
    idx_e, w_e = cp.gate_topk(x, wg, k, gate_fn=1, renorm=1)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "the screen reported a violated error bound or a non-finite logit"
    assert torch.equal(idx_s, idx_e), f"{int((idx_s != idx_e).any(dim=1).sum())} tokens routed differently"
    assert torch.allclose(w_s, w_e, rtol=1e-5, atol=1e-7)            # sigmoid weights of the same exact logits
    # the clusters really are near-ties: most tokens take their 8 experts from one or two clusters
    assert (idx_e // 16).to(torch.float32).std(dim=1).median() < 16
