"""PyTorch operator over the C ABI: `torch.ops.aristos.moe_forward` and the module `AristosMoE`.

The reference links libtorch without ever using it (torching.cuh, CMakeLists.txt:126-133); this is the binding a
PyTorch model would call: forward only, every computation in libaristos_moe.so on the current CUDA stream. The op has
a fake (meta) implementation, so it can be traced (torch.export / torch.compile see an opaque call); there is no CPU
kernel - calling it with CPU tensors raises.

Layer handles live in a registry keyed by an integer, because custom-op arguments must be tensors or plain scalars.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .config import AristosConfig

_LAYERS: Dict[int, object] = {}
_NEXT_HANDLE = [1]


def register_layer(moe_layer) -> int:
    """Keeps a cuplayground_b200.layer.MoELayer alive under an integer handle for `aristos::moe_forward`."""
    h = _NEXT_HANDLE[0]
    _NEXT_HANDLE[0] += 1
    _LAYERS[h] = moe_layer
    return h


def release_layer(handle: int) -> None:
    layer = _LAYERS.pop(handle, None)
    if layer is not None:
        layer.close()


@torch.library.custom_op("aristos::moe_forward", mutates_args=(), device_types="cuda")
def moe_forward(x: torch.Tensor, w_gate: torch.Tensor, w1: torch.Tensor, w3: Optional[torch.Tensor],
                w2: torch.Tensor, scales: Optional[torch.Tensor], handle: int) -> torch.Tensor:
    """out (S, H) = combine(expert FFN(dispatch(gate(x)))) through aristos_moe_forward. x (S, H); w_gate (E, H);
    w1 / w3 (E_local, I, H); w2 (E_local, H, I); scales: the fp8 weights' block scales or None."""
    try:
        layer = _LAYERS[handle]
    except KeyError:
        raise RuntimeError(f"aristos::moe_forward: unknown layer handle {handle}") from None
    if tuple(x.shape) != (layer.S, layer.H):
        raise RuntimeError(f"aristos::moe_forward: x is {tuple(x.shape)}, the layer was created for {(layer.S, layer.H)}")
    return layer.forward(x.contiguous(), w_gate, w1, w3, w2, scales=scales)


@moe_forward.register_fake
def _(x, w_gate, w1, w3, w2, scales, handle):
    return torch.empty_like(x)


class AristosMoE(torch.nn.Module):
    """The layer as a module: owns the gate and (this rank's) expert weights as parameters in the reference layouts
    (weights (out, in) row-major) and a library handle. Forward only (the parameters do not receive gradients)."""

    def __init__(self, cfg: AristosConfig, rank: int = 0, world: int = 1, nccl_uid: Optional[bytes] = None,
                 device: str = "cuda"):
        super().__init__()
        from . import _lib
        from . import layer as _layer
        if cfg.torch_dtype == _lib.DTYPE_FP8_E4M3:
            raise ValueError("AristosMoE holds 16/32-bit parameters; call the op directly with quantised weights for fp8")
        dt = _layer._TORCH_DTYPE[cfg.torch_dtype]
        E, H, I = cfg.num_experts, cfg.hidden_size, cfg.intermediate_size
        El = E // world
        new = lambda *shape: torch.nn.Parameter(torch.empty(shape, dtype=dt, device=device).normal_(0.0, 0.02),
                                                requires_grad=False)
        self.w_gate = new(E, H)
        self.w1 = new(El, I, H)
        self.w3 = new(El, I, H) if cfg.hidden_act == _lib.ACT_SWIGLU else None
        self.w2 = new(El, H, I)
        self.cfg = cfg
        self._handle = register_layer(_layer.MoELayer(cfg, rank, world, nccl_uid))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        out = torch.ops.aristos.moe_forward(x.reshape(-1, shape[-1]), self.w_gate, self.w1, self.w3, self.w2, None,
                                            self._handle)
        return out.reshape(shape)

    def close(self) -> None:
        release_layer(self._handle)
