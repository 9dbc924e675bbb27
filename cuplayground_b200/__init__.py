"""cuplayground_b200: a B200 (sm_100a) fused, expert-parallel MoE forward layer behind a C ABI.

The product is libaristos_moe.so (include/aristos_moe.h); this package is its Python host-side mirror. Compute
entry points need the built library and a CUDA device - there is no CPU or PyTorch fallback path.
"""
from . import _lib
from ._lib import AristosError
from .config import AristosConfig, baseline_config

__all__ = ["AristosConfig", "AristosError", "baseline_config", "_lib"]


def __getattr__(name):
    # torch-dependent pieces are imported on first use so that config parsing works without importing torch
    if name in ("MoELayer", "layer", "gate_topk", "gate_topk_screened", "dispatch", "permute", "expert_ffn", "combine",
                "fill_normal", "nccl_unique_id"):
        import importlib

        _layer = importlib.import_module(".layer", __name__)   # `from . import layer` would re-enter __getattr__
        return _layer if name == "layer" else getattr(_layer, name)
    raise AttributeError(name)
