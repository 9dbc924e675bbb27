"""ctypes + numpy binding of the CPU oracle (oracle/moe_oracle.c).

Test infrastructure only: tests/, the smoke check and the benchmark's CPU-baseline leg import this module; the
product package never does. Every function takes and returns host numpy arrays (fp32 / int32).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libmoe_oracle.so")

ACT = {"relu": 0, "gelu": 1, "swiglu": 2, "identity": 3}
GATE = {"softmax": 0, "sigmoid": 1}


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc only)."""
    src = os.path.join(_HERE, "moe_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "clean", "all"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_capacity.restype = C.c_int
        _lib.orc_capacity.argtypes = [C.c_int, C.c_int, C.c_int, C.c_double, C.c_int]
        _lib.orc_num_threads.restype = C.c_int
        _lib.orc_moe_forward.restype = C.c_int
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))


def _cf(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def fill_normal(n: int, mean: float, std: float, seed: int, stream: int) -> np.ndarray:
    out = np.empty(int(n), dtype=np.float32)
    lib().orc_fill_normal(_f(out), C.c_int64(int(n)), C.c_float(mean), C.c_float(std), C.c_uint64(seed),
                          C.c_uint32(stream))
    return out


def round_bf16(a: np.ndarray) -> np.ndarray:
    a = np.array(a, dtype=np.float32, copy=True, order="C")
    lib().orc_round_bf16(_f(a), C.c_int64(a.size))
    return a


def capacity(S: int, E: int, k: int, cf: float, drop_tokens: int = 1) -> int:
    return int(lib().orc_capacity(S, E, k, float(cf), int(drop_tokens)))


def zipf_bias(E: int, s: float) -> np.ndarray:
    b = np.empty(E, dtype=np.float32)
    lib().orc_zipf_bias(_f(b), C.c_int(E), C.c_double(s))
    return b


def gate_logits(x, wg, bias=None) -> np.ndarray:
    x, wg = _cf(x), _cf(wg)
    S, H = x.shape
    E = wg.shape[0]
    assert wg.shape[1] == H and H % 8 == 0
    bias = None if bias is None else _cf(bias)
    out = np.empty((S, E), dtype=np.float32)
    lib().orc_gate_logits(_f(x), _f(wg), _f(bias), S, H, E, _f(out))
    return out


def gate_topk(logits, k: int, gate_fn: int = 0, renorm: int = 0):
    logits = _cf(logits)
    S, E = logits.shape
    idx = np.empty((S, k), dtype=np.int32)
    w = np.empty((S, k), dtype=np.float32)
    lib().orc_gate_topk(_f(logits), S, E, k, gate_fn, renorm, _i(idx), _f(w))
    return idx, w


def dispatch(topk_idx, E: int, cap: int):
    topk_idx = np.ascontiguousarray(topk_idx, dtype=np.int32)
    S, k = topk_idx.shape
    count = np.empty(E, dtype=np.int32)
    slot_of = np.empty((S, k), dtype=np.int32)
    tos = np.empty(E * cap, dtype=np.int32)
    lib().orc_dispatch(_i(topk_idx), S, k, E, cap, _i(count), _i(slot_of), _i(tos))
    return count, slot_of, tos


def gemm_bias_act(A, B, bias=None, act: int = 3) -> np.ndarray:
    A, B = _cf(A), _cf(B)
    M, K = A.shape
    N = B.shape[0]
    bias = None if bias is None else _cf(bias)
    out = np.empty((M, N), dtype=np.float32)
    lib().orc_gemm_bias_act(_f(A), _f(B), _f(bias), _f(out), M, N, K, act)
    return out


def permute(x, token_of_slot) -> np.ndarray:
    x = _cf(x)
    tos = np.ascontiguousarray(token_of_slot, dtype=np.int32)
    H = x.shape[1]
    xg = np.empty((tos.size, H), dtype=np.float32)
    lib().orc_permute(_f(x), _i(tos), C.c_int64(tos.size), H, _f(xg))
    return xg


def expert_ffn(xg, count, w1, w3, w2, hidden_act: int, round_h: int = 0, b1=None, b3=None, b2=None) -> np.ndarray:
    """xg (E,cap,H), w1/w3 (E,I,H), w2 (E,H,I), optional biases b1/b3 (E,I), b2 (E,H) -> y (E,cap,H); rows past
    count[e] stay zero."""
    b1, b3, b2 = (None if b is None else _cf(b) for b in (b1, b3, b2))
    xg, w1, w2 = _cf(xg), _cf(w1), _cf(w2)
    w3 = None if w3 is None else _cf(w3)
    count = np.ascontiguousarray(count, dtype=np.int32)
    E, cap, H = xg.shape
    I = w1.shape[1]
    y = np.zeros((E, cap, H), dtype=np.float32)
    lib().orc_expert_ffn(_f(xg), _i(count), _f(w1), _f(w3), _f(w2), _f(b1), _f(b3), _f(b2), _f(y), E, cap, H, I,
                         hidden_act, round_h)
    return y


def combine(y, slot_of, topk_w) -> np.ndarray:
    y = _cf(y)
    slot_of = np.ascontiguousarray(slot_of, dtype=np.int32)
    topk_w = _cf(topk_w)
    S, k = slot_of.shape
    H = y.shape[-1]
    out = np.empty((S, H), dtype=np.float32)
    lib().orc_combine(_f(y.reshape(-1, H)), _i(slot_of), _f(topk_w), S, k, H, _f(out))
    return out


def moe_forward(x, wg, w1, w3, w2, *, k: int, cap: int, gate_fn: int = 0, renorm: int = 0, hidden_act: int = 0,
                gate_bias=None, round_h: int = 0, only_rows=None, want_out: bool = True, x_ffn=None):
    """Whole layer on one rank. Returns dict(out, topk_idx, topk_w, count, slot_of, token_of_slot)."""
    x, wg, w1, w2 = _cf(x), _cf(wg), _cf(w1), _cf(w2)
    w3 = None if w3 is None else _cf(w3)
    gate_bias = None if gate_bias is None else _cf(gate_bias)
    S, H = x.shape
    E, I = w1.shape[0], w1.shape[1]
    assert wg.shape == (E, H) and w2.shape == (E, H, I)
    x_ffn = None if x_ffn is None else _cf(x_ffn)
    only = None if only_rows is None else np.ascontiguousarray(only_rows, dtype=np.int32)
    n_only = 0 if only is None else int(only.size)
    out = np.empty((n_only if n_only else S, H), dtype=np.float32) if want_out else None
    idx = np.empty((S, k), dtype=np.int32)
    tw = np.empty((S, k), dtype=np.float32)
    count = np.empty(E, dtype=np.int32)
    slot_of = np.empty((S, k), dtype=np.int32)
    tos = np.empty(E * cap, dtype=np.int32)
    rc = lib().orc_moe_forward(_f(x), _f(wg), _f(gate_bias), _f(w1), _f(w3), _f(w2), S, H, I, E, k, cap, gate_fn,
                               renorm, hidden_act, round_h, _f(out), _i(idx), _f(tw), _i(count), _i(slot_of),
                               _i(tos), _i(only), n_only, _f(x_ffn))
    if rc != 0:
        raise MemoryError("oracle allocation failed")
    return dict(out=out, topk_idx=idx, topk_w=tw, count=count, slot_of=slot_of, token_of_slot=tos)


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(int(n)))


def use_all_cores() -> int:
    """Run the later calls on every core this process may use (sched_getaffinity), whatever OMP_NUM_THREADS says:
    launchers such as torch.distributed.run export OMP_NUM_THREADS=1. Returns the thread count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    set_num_threads(n)
    return num_threads()


def gate_logits_f64(x, wg, bias=None) -> np.ndarray:
    """Order-independent recomputation of the gate logits in float64 (products of 16-bit inputs are exact in
    float64 and the sum of H of them is accurate to about 1e-13 relative): the yardstick for the fixed-order fp32
    contract of gate_logits, not a contract itself."""
    l = np.asarray(x, dtype=np.float64) @ np.asarray(wg, dtype=np.float64).T
    if bias is not None:
        l = l + np.asarray(bias, dtype=np.float64)[None, :]
    return l


def load_balance_stats(topk_idx, topk_w, slot_of, E: int):
    """Per-expert routing statistics of one forward, the ingredients of the usual auxiliary load-balance loss:
    frac[e] = share of the S*k assignments routed to expert e (before capacity drops), prob[e] = sum of the gate
    weights assigned to e divided by S, aux = E * sum(frac * prob), dropped = share of assignments dropped."""
    idx = np.asarray(topk_idx).reshape(-1)
    w = np.asarray(topk_w, dtype=np.float64).reshape(-1)
    S = np.asarray(topk_idx).shape[0]
    frac = np.bincount(idx, minlength=E).astype(np.float64) / idx.size
    prob = np.bincount(idx, weights=w, minlength=E) / S
    dropped = float((np.asarray(slot_of) < 0).sum()) / idx.size
    return frac, prob, float(E * (frac * prob).sum()), dropped


# ---- fp8 e4m3 (1 sign, 4 exponent bits with bias 7, 3 mantissa bits; no infinities, 0x7f / 0xff are NaN) -----------
def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for code in range(256):
        s, e, m = code >> 7, (code >> 3) & 15, code & 7
        if e == 15 and m == 7:
            v = np.nan
        elif e == 0:
            v = m / 8.0 * 2.0 ** -6
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[code] = -v if s else v
    return t


E4M3 = _e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return E4M3[np.asarray(codes, dtype=np.uint8)]


def e4m3_encode(v: np.ndarray) -> np.ndarray:
    """Round to nearest (ties to the even code), saturating at +-448."""
    v = np.asarray(v, dtype=np.float32)
    pos = E4M3[:127].astype(np.float64)                      # 0 .. 448, increasing with the code
    a = np.minimum(np.abs(v).astype(np.float64), 448.0)
    hi = np.clip(np.searchsorted(pos, a, side="left"), 0, 126)
    lo = np.clip(hi - 1, 0, 126)
    dlo, dhi = a - pos[lo], pos[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    return (code | (np.signbit(v).astype(np.uint8) << 7)).astype(np.uint8)


def dequantize_fp8(codes: np.ndarray, scales: np.ndarray, block_rows: int) -> np.ndarray:
    """codes (..., rows, cols) with scales per block_rows x 128 block -> fp32."""
    v = e4m3_decode(codes)
    s = np.repeat(np.asarray(scales, dtype=np.float32), 128, axis=-1)[..., :codes.shape[-1]]
    if block_rows > 1:
        s = np.repeat(s, block_rows, axis=-2)[..., :codes.shape[-2], :]
    return (v * s).astype(np.float32)
