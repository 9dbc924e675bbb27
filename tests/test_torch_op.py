"""The PyTorch operator over the C ABI (torch.ops.aristos.moe_forward, AristosMoE)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")


def test_op_is_registered_and_traces_without_a_gpu():
    import cuplayground_b200.torch_op  # noqa: F401  (registers the op)
    from torch._subclasses.fake_tensor import FakeTensorMode
    assert hasattr(torch.ops.aristos, "moe_forward")
    with FakeTensorMode():
        x = torch.empty(8, 16, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(4, 16, dtype=torch.bfloat16, device="cuda")
        out = torch.ops.aristos.moe_forward(x, w, w, None, w, None, 1)
        assert out.shape == x.shape and out.dtype == x.dtype


def test_op_has_no_cpu_path():
    import cuplayground_b200.torch_op  # noqa: F401
    z = torch.zeros(8, 16)
    with pytest.raises(NotImplementedError):
        torch.ops.aristos.moe_forward(z, z, z, None, z, None, 1)


@pytest.mark.gpu
def test_module_matches_layer_and_oracle(oracle):
    import cuplayground_b200 as cp
    from cuplayground_b200.torch_op import AristosMoE
    from helpers import TOL_BF16_MAX, TOL_BF16_MEAN, rel_errors
    cfg = cp.AristosConfig(expert_top_k=2, hidden_act=2, hidden_size=256, intermediate_size=512, num_experts=8,
                           torch_dtype=2, tokens=512, capacity_factor=1.25, renorm_topk=1)
    m = AristosMoE(cfg)
    torch.manual_seed(5)
    x = torch.randn(4, 128, 256, device="cuda", dtype=torch.bfloat16)      # (batch, seq, H): 512 tokens
    out = m(x)
    assert out.shape == x.shape
    assert torch.equal(out, m(x))                                          # deterministic
    f = lambda t: t.float().cpu().numpy()
    ref = oracle.moe_forward(f(x).reshape(-1, 256), f(m.w_gate), f(m.w1), f(m.w3), f(m.w2), k=2, cap=cfg.capacity,
                             gate_fn=0, renorm=1, hidden_act=2)
    mx, mean = rel_errors(f(out).reshape(-1, 256), ref["out"])
    assert mx < TOL_BF16_MAX and mean < TOL_BF16_MEAN
    with pytest.raises(RuntimeError):
        m(x[:2])                                                           # the handle was created for 512 tokens
    m.close()
