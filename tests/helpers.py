"""Shared helpers of the parity tests: seeded inputs (from the oracle's Philox generator) and error metrics."""
from __future__ import annotations

import numpy as np

from oracle import moe_oracle as O

# Philox stream ids of the tensors of one layer
STREAM_X, STREAM_WG, STREAM_W1, STREAM_W3, STREAM_W2 = 0, 1, 2, 3, 4


def round_f16(a):
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def make_inputs(S, H, I, E, seed, *, swiglu=False, bf16=True, w_std=0.02, f16=False):
    """x ~ N(0,1), weights ~ N(0, w_std), in storage layout: x (S,H), wg (E,H), w1/w3 (E,I,H), w2 (E,H,I).
    With bf16=True (f16=True) the fp32 arrays hold bf16- (fp16-) representable values (what the GPU stores)."""
    rnd = round_f16 if f16 else (O.round_bf16 if bf16 else (lambda a: a))
    x = rnd(O.fill_normal(S * H, 0.0, 1.0, seed, STREAM_X)).reshape(S, H)
    wg = rnd(O.fill_normal(E * H, 0.0, w_std, seed, STREAM_WG)).reshape(E, H)
    w1 = rnd(O.fill_normal(E * I * H, 0.0, w_std, seed, STREAM_W1)).reshape(E, I, H)
    w3 = rnd(O.fill_normal(E * I * H, 0.0, w_std, seed, STREAM_W3)).reshape(E, I, H) if swiglu else None
    w2 = rnd(O.fill_normal(E * H * I, 0.0, w_std, seed, STREAM_W2)).reshape(E, H, I)
    return x, wg, w1, w3, w2


def to_dev(a, dtype):
    import torch
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(device="cuda", dtype=dtype)


def rel_errors(got: np.ndarray, ref: np.ndarray):
    """(max|d| / max|ref|, mean|d| / mean|ref|) - the normalisation the layer tolerances are stated in."""
    d = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    return float(d.max() / max(np.abs(ref).max(), 1e-30)), float(d.mean() / max(np.abs(ref).mean(), 1e-30))


# output tolerances: fp32 1e-4 relative; 16-bit and fp8 2e-2 max-relative, 1e-2 mean-relative
TOL_F32_MAX = 1e-4
TOL_BF16_MAX, TOL_BF16_MEAN = 2e-2, 1e-2
