"""Error behaviour of the C ABI on a GPU box: bad arguments come back as status codes with a message, never as a
crash, and a failed call leaves the library usable (the reference's CHECK_ERROR_EXIT, util.cuh:24-36, exits)."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


def _mods():
    import torch
    import cuplayground_b200 as cp
    import cuplayground_b200.layer as layer
    return torch, cp, layer


def test_stage_entry_points_reject_bad_arguments():
    torch, cp, layer = _mods()
    lib = cp._lib.load()
    x = torch.zeros((16, 64), dtype=torch.bfloat16, device="cuda")
    wg = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros((16, 2), dtype=torch.int32, device="cuda")
    w = torch.zeros((16, 2), dtype=torch.float32, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    # NULL pointer
    assert lib.aristos_gate_topk(None, p(wg), None, 16, 64, 4, 2, 0, 0, 2, p(idx), p(w), None, None) == 1
    assert b"NULL" in lib.aristos_last_error()
    # k > E, H not a multiple of 8
    assert lib.aristos_gate_topk(p(x), p(wg), None, 16, 64, 4, 5, 0, 0, 2, p(idx), p(w), None, None) == 2
    assert lib.aristos_gate_topk(p(x), p(wg), None, 16, 60, 4, 2, 0, 0, 2, p(idx), p(w), None, None) == 2
    # misaligned pointer
    assert lib.aristos_gate_topk(C.c_void_p(x.data_ptr() + 2), p(wg), None, 15, 64, 4, 2, 0, 0, 2, p(idx), p(w), None,
                                 None) == 1
    # unsupported dtype (fp8 is not implemented)
    assert lib.aristos_gate_topk(p(x), p(wg), None, 16, 64, 4, 2, 0, 0, 4, p(idx), p(w), None, None) == 6
    # dispatch: scratch too small
    cnt = torch.zeros(4, dtype=torch.int32, device="cuda")
    tos = torch.zeros(4 * 8, dtype=torch.int32, device="cuda")
    scratch = torch.zeros(16, dtype=torch.uint8, device="cuda")
    assert lib.aristos_dispatch(p(idx), 16, 2, 4, 8, p(cnt), p(idx), p(tos), p(scratch), 1, None) == 7
    # expert FFN: row window rules
    y = torch.zeros((1, 256, 64), dtype=torch.bfloat16, device="cuda")
    w1 = torch.zeros((1, 64, 64), dtype=torch.bfloat16, device="cuda")
    args = (p(y), p(cnt), 1, 256, 1, p(w1), None, p(w1), p(y), p(y), 64, 64)
    assert lib.aristos_expert_ffn(*args, 0, 2, 64, 256, 0, None, None) == 1      # row_begin not a multiple of 128
    assert lib.aristos_expert_ffn(*args, 0, 2, 0, 200, 0, None, None) == 1       # row_end neither x128 nor the end
    assert lib.aristos_expert_ffn(*args, 2, 2, 0, 256, 0, None, None) == 1       # SwiGLU without w3
    # the library still works afterwards
    i2, w2 = layer.gate_topk(torch.randn(16, 64, device="cuda").to(torch.bfloat16), wg, 2)
    torch.cuda.synchronize()
    assert i2.shape == (16, 2)


def test_layer_rejects_bad_requests():
    torch, cp, layer = _mods()
    cfg = cp.AristosConfig(hidden_size=128, intermediate_size=128, num_experts=4, torch_dtype=2, tokens=128,
                           expert_top_k=2, drop_tokens=1)
    with pytest.raises(cp.AristosError) as e:
        layer.MoELayer(cfg, rank=0, world=2)            # config says ep_world 1
    assert e.value.status == 2
    cfg2 = cp.AristosConfig(**{**cfg.__dict__, "ep_world": 2})
    with pytest.raises(cp.AristosError) as e:
        layer.MoELayer(cfg2, rank=0, world=2)           # no NCCL unique id
    assert e.value.status == 1
    L = layer.MoELayer(cfg)
    with pytest.raises(cp.AristosError):
        L.routing()                                     # no forward has run
    lib = cp._lib.load()
    small = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    assert lib.aristos_moe_set_workspace(L._h, C.c_void_p(small.data_ptr()), 1024) == 7
    x = torch.zeros((128, 128), dtype=torch.bfloat16, device="cuda")
    wgt = torch.zeros((4, 128, 128), dtype=torch.bfloat16, device="cuda")
    assert lib.aristos_moe_forward(L._h, None, None, None, None, None, None, None, None, None) == 1
    out = L.forward(x, torch.zeros((4, 128), dtype=torch.bfloat16, device="cuda"), wgt, None, wgt)
    L.status()
    assert not out.any()
    L.close()
