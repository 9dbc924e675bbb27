"""ctypes loader of libaristos_moe.so and the C-ABI prototypes of include/aristos_moe.h.

There is no fallback: if the shared library is missing or fails to load, importing the compute entry points raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaristos_moe.so")

OK = 0
STATUS_NAMES = {0: "ARISTOS_OK", 1: "ARISTOS_ERR_INVALID_ARG", 2: "ARISTOS_ERR_CONFIG", 3: "ARISTOS_ERR_IO",
                4: "ARISTOS_ERR_CUDA", 5: "ARISTOS_ERR_NCCL", 6: "ARISTOS_ERR_UNSUPPORTED",
                7: "ARISTOS_ERR_WORKSPACE", 8: "ARISTOS_ERR_DEVICE_TIMEOUT", 9: "ARISTOS_ERR_DEVICE_BOUNDS",
                10: "ARISTOS_ERR_NOMEM", 11: "ARISTOS_ERR_GATE_SCREEN", 12: "ARISTOS_ERR_NONFINITE"}

DTYPE_F32, DTYPE_TF32, DTYPE_BF16, DTYPE_F16, DTYPE_FP8_E4M3 = 0, 1, 2, 3, 4
ACT_RELU, ACT_GELU, ACT_SWIGLU, ACT_IDENTITY = 0, 1, 2, 3
GATE_SOFTMAX, GATE_SIGMOID = 0, 1


class AristosConfigStruct(C.Structure):
    """Mirror of aristos_config_t."""
    _fields_ = [("capacity_factor", C.c_double), ("drop_tokens", C.c_int), ("expert_top_k", C.c_int),
                ("is_training", C.c_int), ("hidden_act", C.c_int), ("hidden_size", C.c_int),
                ("intermediate_size", C.c_int), ("micro_batch", C.c_int), ("num_experts", C.c_int),
                ("sequence_len", C.c_int), ("torch_dtype", C.c_int), ("tokens", C.c_int), ("gate_fn", C.c_int),
                ("renorm_topk", C.c_int), ("gate_bias_zipf_s", C.c_double), ("ep_world", C.c_int),
                ("seed", C.c_uint64)]


class AristosRoutingStruct(C.Structure):
    """Mirror of aristos_routing_t."""
    _fields_ = [("topk_idx", C.c_void_p), ("topk_w", C.c_void_p), ("count", C.c_void_p), ("slot_of", C.c_void_p),
                ("token_of_slot", C.c_void_p), ("tokens", C.c_int), ("top_k", C.c_int), ("num_experts", C.c_int),
                ("capacity", C.c_int)]


class AristosTrainingStateStruct(C.Structure):
    """Mirror of aristos_training_state_t."""
    _fields_ = [("topk_idx", C.c_void_p), ("topk_w", C.c_void_p), ("slot_of", C.c_void_p),
                ("load_balance", C.c_void_p), ("tokens", C.c_int), ("top_k", C.c_int), ("num_experts", C.c_int)]


class AristosError(RuntimeError):
    def __init__(self, status: int, detail: str):
        self.status = status
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {detail}")


# name -> (restype, argtypes); every symbol include/aristos_moe.h declares
_vp, _i, _sz, _st = C.c_void_p, C.c_int, C.c_size_t, C.c_int
PROTOTYPES = {
    "aristos_status_str": (C.c_char_p, [_st]),
    "aristos_last_error": (C.c_char_p, []),
    "aristos_version": (_i, []),
    "aristos_config_default": (_st, [C.POINTER(AristosConfigStruct)]),
    "aristos_config_parse": (_st, [C.c_char_p, C.POINTER(AristosConfigStruct)]),
    "aristos_config_load": (_st, [C.c_char_p, C.POINTER(AristosConfigStruct)]),
    "aristos_config_validate": (_st, [C.POINTER(AristosConfigStruct)]),
    "aristos_config_tokens": (_i, [C.POINTER(AristosConfigStruct)]),
    "aristos_config_capacity": (_i, [C.POINTER(AristosConfigStruct)]),
    "aristos_zipf_bias_host": (_st, [C.POINTER(C.c_float), _i, C.c_double]),
    "aristos_moe_create": (_st, [C.POINTER(AristosConfigStruct), _i, _i, _vp, C.POINTER(_vp)]),
    "aristos_nccl_unique_id": (_st, [_vp]),
    "aristos_ep_exchange_plan": (_i, [_i, _i, _i, _sz, _sz, _sz, C.POINTER(C.c_int64), _i]),
    "aristos_ep_row_windows": (_st, [_i, C.POINTER(_i), C.POINTER(_i)]),
    "aristos_moe_workspace_bytes": (_sz, [_vp]),
    "aristos_moe_set_workspace": (_st, [_vp, _vp, _sz]),
    "aristos_moe_set_bias": (_st, [_vp, _vp, _vp, _vp]),
    "aristos_moe_forward": (_st, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "aristos_moe_forward_host": (_st, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "aristos_moe_submit_host": (_st, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "aristos_moe_wait_host": (_st, [_vp]),
    "aristos_moe_routing": (_st, [_vp, C.POINTER(AristosRoutingStruct)]),
    "aristos_moe_routing_to_host": (_st, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "aristos_moe_status": (_st, [_vp]),
    "aristos_moe_set_profiling": (_st, [_vp, _i]),
    "aristos_moe_stage_ms": (_st, [_vp, C.POINTER(C.c_float)]),
    "aristos_moe_exchange_ms": (_st, [_vp, C.POINTER(C.c_float)]),
    "aristos_moe_exchange_profile": (_st, [_vp, C.POINTER(C.c_float)]),
    "aristos_moe_ep_transport": (C.c_char_p, [_vp]),
    "aristos_moe_launch_count": (C.c_int64, [_vp]),
    "aristos_moe_destroy": (_st, [_vp]),
    "aristos_gate_topk": (_st, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "aristos_gate_scratch_bytes": (_sz, [_i, _i]),
    "aristos_gate_topk_screened": (_st, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _sz, _vp, _vp]),
    "aristos_dispatch_scratch_bytes": (_sz, [_i, _i, _i]),
    "aristos_dispatch": (_st, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _sz, _vp]),
    "aristos_dispatch_static": (_st, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "aristos_permute": (_st, [_vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "aristos_expert_ffn": (_st, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "aristos_expert_ffn_bias": (_st, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                      _i, _vp, _vp]),
    "aristos_quantize_fp8": (_st, [_vp, C.c_int64, C.c_int64, _i, _i, _i, _vp, _vp, _vp]),
    "aristos_expert_ffn_fp8": (_st, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i,
                                     _i, _i, _i, _i, _vp, _vp]),
    "aristos_combine": (_st, [_vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "aristos_selftest_bounded_wait": (_st, [_i, C.POINTER(_i), _vp]),
    "aristos_selftest_bounded_flag_wait": (_st, [_i, C.POINTER(_i), _vp]),
    "aristos_ffn_set_tile_mode": (_st, [_i]),
    "aristos_ffn_tile_coord": (_i, [_i, _i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "aristos_ep_transport_agreed": (_i, [C.POINTER(_i), _i]),
    "aristos_ep_flag_words": (_i, []),
    "aristos_ep_flag_word_index": (_i, [_i, _i, _i]),
    "aristos_ep_flags_pending": (C.c_uint32, [_vp, C.c_uint32, _i, _i, _i]),
    "aristos_ep_flags_release": (None, [_vp, C.c_uint32]),
    "aristos_moe_set_timeout_ms": (_st, [_vp, _i]),
    "aristos_moe_training_bytes": (_sz, [_vp]),
    "aristos_moe_set_training_buffer": (_st, [_vp, _vp, _sz]),
    "aristos_moe_training_state": (_st, [_vp, C.POINTER(AristosTrainingStateStruct)]),
    "aristos_moe_training_state_to_host": (_st, [_vp, _vp, _vp, _vp, _vp]),
    "aristos_load_balance_stats_bytes": (_sz, [_i]),
    "aristos_load_balance_stats": (_st, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "aristos_ffn_group_order": (_i, [_i, _i, _i]),
    "aristos_ffn_group_order_from": (_i, [_i, _i, _i, _i]),
    "aristos_ep_dense_plan_host": (_st, [_vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "aristos_fill_normal": (_st, [_vp, C.c_int64, C.c_float, C.c_float, C.c_uint64, C.c_uint32, _i, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once) and attach the prototypes. Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m cuplayground_b200.build` "
                          "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise AristosError(status, load().aristos_last_error().decode("utf-8", "replace"))
