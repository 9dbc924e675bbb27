"""GPU parity of the whole layer (aristos_moe_forward through the C ABI) against the CPU oracle."""
import numpy as np
import pytest

from helpers import TOL_BF16_MAX, TOL_BF16_MEAN, TOL_F32_MAX, make_inputs, rel_errors, to_dev

pytestmark = pytest.mark.gpu


def _mods():
    import torch
    import cuplayground_b200 as cp
    import cuplayground_b200.layer as layer
    return torch, cp, layer


def _check_routing(r, ref):
    np.testing.assert_array_equal(r["topk_idx"].cpu().numpy(), ref["topk_idx"])
    np.testing.assert_array_equal(r["count"].cpu().numpy(), ref["count"])
    np.testing.assert_array_equal(r["slot_of"].cpu().numpy(), ref["slot_of"])
    np.testing.assert_array_equal(r["token_of_slot"].cpu().numpy(), ref["token_of_slot"])
    np.testing.assert_allclose(r["topk_w"].cpu().numpy(), ref["topk_w"], rtol=2e-5, atol=1e-7)


def _run_layer(cfg, seed, oracle, w_std=0.02, only_rows=None):
    torch, cp, layer = _mods()
    bf16, f16 = cfg.torch_dtype == 2, cfg.torch_dtype == 3
    dt = torch.bfloat16 if bf16 else (torch.float16 if f16 else torch.float32)
    swiglu = cfg.hidden_act == 2
    x, wg, w1, w3, w2 = make_inputs(cfg.S, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts, seed,
                                    swiglu=swiglu, bf16=bf16, w_std=w_std, f16=f16)
    L = layer.MoELayer(cfg)
    out = L.forward(*(to_dev(a, dt) for a in (x, wg, w1, w3, w2)))
    L.status()
    r = L.routing()
    bias = oracle.zipf_bias(cfg.num_experts, cfg.gate_bias_zipf_s) if cfg.gate_bias_zipf_s > 0 else None
    ref = oracle.moe_forward(x, wg, w1, w3, w2, k=cfg.expert_top_k, cap=cfg.capacity, gate_fn=cfg.gate_fn,
                             renorm=cfg.renorm_topk, hidden_act=cfg.hidden_act, gate_bias=bias, only_rows=only_rows)
    got = out.float().cpu().numpy()
    L.close()
    return got, r, ref


def test_config1_fp32_reference_case(oracle):
    """S=128, H=256, I=512, E=8, top-1 softmax, cf 1.0 (cap 16), ReLU, fp32, seed 0."""
    torch, cp, layer = _mods()
    cfg = cp.baseline_config(1)
    assert cfg.capacity == 16
    got, r, ref = _run_layer(cfg, 0, oracle)
    _check_routing(r, ref)
    mx, _ = rel_errors(got, ref["out"])
    assert mx < TOL_F32_MAX, mx
    dropped = (ref["slot_of"] < 0).all(axis=1)
    assert dropped.any() and (got[dropped] == 0).all(), "dropped tokens give zero rows"


@pytest.mark.parametrize("S,H,I,E,k,act,cf,renorm,zipf", [
    (512, 256, 512, 8, 2, 1, 1.25, 1, 0.0),       # GELU, renormalised top-2 (shape of the single-GPU case, scaled)
    (640, 512, 1024, 8, 2, 2, 1.25, 0, 0.0),      # SwiGLU (Mixtral-shaped, scaled)
    (1024, 256, 256, 32, 4, 1, 1.0, 0, 1.2),      # skewed routing with drops
    (300, 128, 192, 4, 1, 0, 0.5, 0, 0.0),        # ragged token count, heavy drops, ReLU
])
def test_layer_bf16_small(oracle, S, H, I, E, k, act, cf, renorm, zipf):
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(capacity_factor=cf, drop_tokens=1, expert_top_k=k, hidden_act=act, hidden_size=H,
                           intermediate_size=I, num_experts=E, torch_dtype=2, tokens=S, renorm_topk=renorm,
                           gate_bias_zipf_s=zipf)
    got, r, ref = _run_layer(cfg, 7, oracle, w_std=0.05)
    _check_routing(r, ref)
    mx, mean = rel_errors(got, ref["out"])
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mx, mean)
    dropped = (ref["slot_of"] < 0).all(axis=1)
    assert (got[dropped] == 0).all()


def test_layer_matches_committed_golden_case2():
    """The CUDA layer against the committed fixture tests/golden/case2_oracle.npz (no oracle call): routing bit-exact,
    output within the bf16 tolerance."""
    import os
    torch, cp, layer = _mods()
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "case2_oracle.npz"))
    S, H, I, E, k = 96, 128, 256, 16, 4
    cfg = cp.AristosConfig(capacity_factor=1.0, drop_tokens=1, expert_top_k=k, hidden_act=2, hidden_size=H,
                           intermediate_size=I, num_experts=E, torch_dtype=2, tokens=S, renorm_topk=1,
                           gate_bias_zipf_s=1.2)
    assert cfg.capacity == int(g["cap"])
    x, wg, w1, w3, w2 = make_inputs(S, H, I, E, seed=7, swiglu=True, bf16=True, w_std=0.05)
    L = layer.MoELayer(cfg)
    out = L.forward(*(to_dev(a, torch.bfloat16) for a in (x, wg, w1, w3, w2)))
    L.status()
    _check_routing(L.routing(), g)
    mx, mean = rel_errors(out.float().cpu().numpy(), g["out"])
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mx, mean)
    L.close()


def test_layer_no_drop(oracle):
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(drop_tokens=0, expert_top_k=2, hidden_act=2, hidden_size=128, intermediate_size=256,
                           num_experts=8, torch_dtype=2, tokens=256)
    assert cfg.capacity == 256
    got, r, ref = _run_layer(cfg, 3, oracle, w_std=0.05)
    _check_routing(r, ref)
    assert (ref["slot_of"] >= 0).all()
    mx, mean = rel_errors(got, ref["out"])
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mx, mean)


def _full_size(n, seed, oracle, n_sample):
    """Full-size configuration generated on the device; routing checked on every token, outputs on a sample."""
    torch, cp, layer = _mods()
    cfg = cp.baseline_config(n)
    S, H, I, E = cfg.S, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    dt = torch.bfloat16
    mk = lambda shape, std, sid: layer.fill_normal(torch.empty(shape, dtype=dt, device="cuda"), 0.0, std, seed, sid)
    x, wg = mk((S, H), 1.0, 0), mk((E, H), 0.02, 1)
    w1, w2 = mk((E, I, H), 0.02, 2), mk((E, H, I), 0.02, 4)
    w3 = mk((E, I, H), 0.02, 3) if cfg.hidden_act == 2 else None
    L = layer.MoELayer(cfg)
    out = L.forward(x, wg, w1, w3, w2)
    L.status()
    out2 = L.forward(x, wg, w1, w3, w2)
    L.status()
    assert torch.equal(out, out2), "the forward is deterministic"
    r = L.routing()
    rows = np.random.default_rng(n).choice(S, size=n_sample, replace=False).astype(np.int32)
    host = lambda t: None if t is None else t.float().cpu().numpy()
    bias = oracle.zipf_bias(E, cfg.gate_bias_zipf_s) if cfg.gate_bias_zipf_s > 0 else None
    ref = oracle.moe_forward(host(x), host(wg), host(w1), host(w3), host(w2), k=cfg.expert_top_k, cap=cfg.capacity,
                             gate_fn=cfg.gate_fn, renorm=cfg.renorm_topk, hidden_act=cfg.hidden_act, gate_bias=bias,
                             only_rows=rows)
    _check_routing(r, ref)
    got = out[torch.from_numpy(rows.astype(np.int64)).cuda()].float().cpu().numpy()
    mx, mean = rel_errors(got, ref["out"])
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mx, mean)
    # size-independent properties: kept rows per expert never exceed the capacity; every slot maps back to a token
    # that selected that expert; tokens whose assignments were all dropped give zero rows
    count = r["count"].cpu().numpy()
    assert (count <= cfg.capacity).all() and count.sum() == (ref["slot_of"] >= 0).sum()
    all_dropped = torch.from_numpy((ref["slot_of"] < 0).all(axis=1)).cuda()
    assert not out[all_dropped].any()
    L.close()
    return ref


def test_config2_full_size(oracle):
    """S=8192, H=2048, I=2048, E=64, top-2 renormalised softmax, GELU, cf 1.25, bf16, seed 1."""
    _full_size(2, 1, oracle, n_sample=256)


def test_config5_full_size_skewed(oracle):
    """S=8192, H=2048, I=1024, E=128, top-4, Zipf(1.2) prior, cf 1.0 with drops, GELU, bf16, seed 4."""
    ref = _full_size(5, 4, oracle, n_sample=256)
    assert (ref["slot_of"] < 0).sum() > 0, "the skewed case must overflow some experts"


def test_config3_full_size_mixtral_shaped(oracle):
    """S=16384, H=4096, I=14336, E=8, top-2 softmax, SwiGLU, cf 1.25, bf16, seed 2 (one rank holds all experts)."""
    _full_size(3, 2, oracle, n_sample=64)


@pytest.mark.parametrize("tiles", ["single", "pair"])
def test_config3_with_other_tile_shapes(tiles):
    """Padded CTA pairs (cta_group::2, 256 x 256 tiles) are the default where a row group is large; the full-size
    Mixtral-shaped parity test once more in processes that select single-CTA tiles only, and pairs over the whole
    256-row tiles with a single-CTA launch for every group's remaining rows."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ARISTOS_FFN_TILES=tiles)
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_layer.py"), "-q", "-x",
                        "-k", "test_config3_full_size_mixtral_shaped", "-m", "gpu"], env=env, cwd=root,
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "1 passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_forward_host_matches_device_forward(oracle):
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=2, hidden_act=1, hidden_size=256,
                           intermediate_size=512, num_experts=8, torch_dtype=2, tokens=512)
    x, wg, w1, w3, w2 = make_inputs(512, 256, 512, 8, 5)
    dt = torch.bfloat16
    dev = [to_dev(a, dt) for a in (x, wg, w1, w3, w2)]
    L = layer.MoELayer(cfg)
    out = L.forward(*dev)
    xh = torch.from_numpy(x).to(dt).pin_memory()
    oh = torch.empty_like(xh).pin_memory()
    L.forward_host(xh, dev[1], dev[2], dev[3], dev[4], oh)
    L.status()
    assert torch.equal(oh, out.cpu())
    L.close()


@pytest.mark.parametrize("act,k", [(1, 2), (2, 2), (0, 1)])
def test_layer_fp16(oracle, act, k):
    """torch_dtype 3 (fp16, aristos_config.schema.json:54-58): same kernels with f16 MMA inputs; fp16 keeps 11
    significant bits, so the outputs sit well inside the 16-bit tolerance."""
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=k, hidden_act=act, hidden_size=256,
                           intermediate_size=512, num_experts=8, torch_dtype=3, tokens=512, renorm_topk=1)
    got, r, ref = _run_layer(cfg, 13, oracle, w_std=0.05)
    _check_routing(r, ref)
    mx, mean = rel_errors(got, ref["out"])
    assert mx < TOL_BF16_MAX / 4 and mean < TOL_BF16_MEAN / 4, (mx, mean)


@pytest.mark.parametrize("act", [1, 2])
def test_layer_tf32(oracle, act):
    """torch_dtype 1 (tf32, aristos_config.schema.json:54-58): fp32 storage, exact fp32 gate, tf32 tensor-core expert
    GEMMs (10-bit mantissa inputs): routing stays bit-exact, outputs within 5e-3 of the fp32 oracle."""
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=2, hidden_act=act, hidden_size=256,
                           intermediate_size=512, num_experts=8, torch_dtype=1, tokens=512)
    got, r, ref = _run_layer(cfg, 23, oracle, w_std=0.05)
    _check_routing(r, ref)
    mx, mean = rel_errors(got, ref["out"])
    assert mx < 5e-3 and mean < 5e-3, (mx, mean)
    assert mx > 1e-6, "suspiciously exact: the tf32 path did not run"


def test_unsupported_requests_fail_loudly():
    torch, cp, layer = _mods()
    # fp8 needs H % 512 == 0: a configuration error, not a silent fallback
    cfg = cp.AristosConfig(hidden_size=128, intermediate_size=128, num_experts=4, torch_dtype=4, tokens=128)
    with pytest.raises(cp.AristosError) as e:
        layer.MoELayer(cfg)
    assert e.value.status == 2


def test_bounded_device_wait_times_out_and_context_survives(oracle):
    """Failure detection without a GPU fault: a wait that nothing satisfies gives up after its limit, the kernel
    returns, the host reads the status, and the same context then runs a normal forward."""
    import ctypes as C
    torch, cp, layer = _mods()
    lib = cp._lib.load()
    waited = C.c_int(0)
    st = lib.aristos_selftest_bounded_wait(200, C.byref(waited), None)
    assert st == 8, "ARISTOS_ERR_DEVICE_TIMEOUT expected"
    assert 200 <= waited.value < 1500, waited.value
    got, r, ref = _run_layer(cp.baseline_config(1), 0, oracle)
    _check_routing(r, ref)


def test_submit_host_pipelines_consecutive_calls(oracle):
    """Six host-side calls back to back (four staging slots: the fifth waits for the first, the sixth for the
    second): every call's result equals the device-resident forward of the same input."""
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=2, hidden_act=2, hidden_size=256,
                           intermediate_size=512, num_experts=8, torch_dtype=2, tokens=1024)
    dt = torch.bfloat16
    _, wg, w1, w3, w2 = make_inputs(1024, 256, 512, 8, 5, swiglu=True, w_std=0.05)
    dev_w = [to_dev(a, dt) for a in (wg, w1, w3, w2)]
    n_calls = 6
    xs = [make_inputs(1024, 256, 512, 8, 50 + i, w_std=0.05)[0] for i in range(n_calls)]
    L = layer.MoELayer(cfg)
    expect = [L.forward(to_dev(x, dt), *dev_w).cpu() for x in xs]
    xh = [torch.from_numpy(x).to(dt).pin_memory() for x in xs]
    oh = [torch.empty_like(t).pin_memory() for t in xh]
    for i in range(n_calls):
        L.submit_host(xh[i], *dev_w, oh[i])
    L.wait_host()
    L.status()
    for i in range(n_calls):
        assert torch.equal(oh[i], expect[i]), i
    L.close()


def test_layer_with_expert_biases(oracle):
    """aristos_moe_set_bias: the layer equals gate -> dispatch -> gather -> biased expert FFN -> combine of the
    oracle."""
    torch, cp, layer = _mods()
    S, H, I, E, k = 512, 128, 256, 4, 2
    cfg = cp.AristosConfig(capacity_factor=1.25, drop_tokens=1, expert_top_k=k, hidden_act=2, hidden_size=H,
                           intermediate_size=I, num_experts=E, torch_dtype=2, tokens=S)
    x, wg, w1, w3, w2 = make_inputs(S, H, I, E, 17, swiglu=True, w_std=0.05)
    rng = np.random.default_rng(3)
    b1, b3, b2 = (oracle.round_bf16(rng.standard_normal(s).astype(np.float32) * 0.3) for s in ((E, I), (E, I), (E, H)))
    dt = torch.bfloat16
    L = layer.MoELayer(cfg)
    L.set_bias(to_dev(b1, dt), to_dev(b3, dt), to_dev(b2, dt))
    out = L.forward(*(to_dev(a, dt) for a in (x, wg, w1, w3, w2)))
    L.status()
    idx, w = oracle.gate_topk(oracle.gate_logits(x, wg), k, 0, 0)
    count, slot_of, tos = oracle.dispatch(idx, E, cfg.capacity)
    y = oracle.expert_ffn(oracle.permute(x, tos).reshape(E, cfg.capacity, H), count, w1, w3, w2, 2, b1=b1, b3=b3, b2=b2)
    ref = oracle.combine(y, slot_of, w)
    mx, mean = rel_errors(out.float().cpu().numpy(), ref)
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN, (mx, mean)
    L.close()


def test_training_mode_keeps_routing_and_load_balance_statistics(oracle):
    """is_training = 1 (aristos_config.schema.json:20-23): every forward saves its routing and the load-balance
    statistics outside the working buffers; a caller-owned buffer keeps a micro-batch alive across the next forward.
    Routing bit-exact and statistics within fp32 rounding of the oracle's float64 recomputation."""
    torch, cp, layer = _mods()
    S, H, I, E, k = 1024, 256, 256, 16, 2
    cfg = cp.AristosConfig(capacity_factor=1.0, drop_tokens=1, expert_top_k=k, hidden_act=1, hidden_size=H,
                           intermediate_size=I, num_experts=E, torch_dtype=2, tokens=S, is_training=1,
                           gate_bias_zipf_s=1.0)
    dt = torch.bfloat16
    _, wg, w1, w3, w2 = make_inputs(S, H, I, E, 41, w_std=0.05)
    xa, xb = (make_inputs(S, H, I, E, 42 + i, w_std=0.05)[0] for i in range(2))
    dev_w = [to_dev(a, dt) for a in (wg, w1, w3, w2)]
    bias = oracle.zipf_bias(E, 1.0)
    L = layer.MoELayer(cfg)
    assert L.training_bytes > 0
    keep = torch.empty(L.training_bytes + 256, dtype=torch.uint8, device="cuda")
    off = (-keep.data_ptr()) % 256
    L.set_training_buffer(keep[off:off + L.training_bytes])
    L.forward(to_dev(xa, dt), *dev_w)            # micro-batch A goes to the caller's buffer
    state_a = L.training_state()
    L.set_training_buffer(None)
    L.forward(to_dev(xb, dt), *dev_w)            # micro-batch B goes to the layer's own buffer
    L.status()
    state_b = L.training_state()
    assert state_a["device_ptrs"] != state_b["device_ptrs"]
    for x, st in ((xa, state_a), (xb, state_b)):
        ref = oracle.moe_forward(x, wg, w1, w3, w2, k=k, cap=cfg.capacity, hidden_act=1, gate_bias=bias, want_out=False)
        assert np.array_equal(st["topk_idx"].numpy(), ref["topk_idx"])
        assert np.array_equal(st["slot_of"].numpy(), ref["slot_of"])
        assert np.allclose(st["topk_w"].numpy(), ref["topk_w"], rtol=1e-5, atol=1e-7)
        frac, prob, aux, dropped = oracle.load_balance_stats(ref["topk_idx"], ref["topk_w"], ref["slot_of"], E)
        assert np.allclose(st["frac"].numpy(), frac, rtol=1e-6, atol=1e-7)
        assert np.allclose(st["prob"].numpy(), prob, rtol=1e-5, atol=1e-7)
        assert abs(st["aux"] - aux) < 1e-5 * max(1.0, aux) and abs(st["dropped"] - dropped) < 1e-6
    assert state_a["dropped"] > 0, "the Zipf prior with capacity factor 1 must overflow some experts"
    # A's saved state survived B's forward: the kept buffer still holds A's routing
    kept_idx = keep[off:off + S * k * 4].view(torch.int32).view(S, k).cpu()
    assert torch.equal(kept_idx, state_a["topk_idx"]), "the kept buffer was overwritten by the next forward"
    # a layer without is_training has no training state
    L2 = layer.MoELayer(cp.AristosConfig(expert_top_k=k, hidden_size=H, intermediate_size=I, num_experts=E,
                                         torch_dtype=2, tokens=S))
    with pytest.raises(cp.AristosError):
        L2.training_state()
    L.close(); L2.close()
