"""Generates tests/golden/config1_oracle.npz and tests/golden/case2_oracle.npz from the CPU oracle (run from the
repository root: `python tests/golden/make_golden.py`).

The reference tree holds no golden vector for the MoE path (it has no gate, dispatch or CPU path at all), so these
vectors come from the oracle itself. They do not pin the oracle to the reference; they guard it against drift:
a change to oracle/moe_oracle.c that alters routing or outputs of the fp32 reference case fails tests/test_oracle.py.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import make_inputs  # noqa: E402
from oracle import moe_oracle as O  # noqa: E402


def main():
    S, H, I, E, k, cap = 128, 256, 512, 8, 1, 16      # config 1: fp32, seed 0, top-1 softmax, cf 1.0, ReLU
    x, wg, w1, w3, w2 = make_inputs(S, H, I, E, seed=0, bf16=False)
    r = O.moe_forward(x, wg, w1, None, w2, k=k, cap=cap, gate_fn=0, renorm=0, hidden_act=0)
    logits = O.gate_logits(x, wg)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "config1_oracle.npz")
    np.savez_compressed(out, philox_head=O.fill_normal(16, 0.0, 1.0, 0, 0), logits_bits=logits.view(np.uint32),
                        topk_idx=r["topk_idx"], topk_w=r["topk_w"], count=r["count"], slot_of=r["slot_of"],
                        token_of_slot=r["token_of_slot"], out=r["out"])
    print("wrote", out, os.path.getsize(out), "bytes")

    # case 2: the other code paths in one small layer - bf16-representable inputs, top-4 of 16 with a Zipf prior
    # (several experts overflow their capacity), renormalised softmax weights, SwiGLU, hidden activations rounded to
    # bf16 as the 16-bit GPU path stores them
    S, H, I, E, k = 96, 128, 256, 16, 4
    cap = O.capacity(S, E, k, 1.0)
    x, wg, w1, w3, w2 = make_inputs(S, H, I, E, seed=7, swiglu=True, bf16=True, w_std=0.05)
    bias = O.zipf_bias(E, 1.2)
    r = O.moe_forward(x, wg, w1, w3, w2, k=k, cap=cap, gate_fn=0, renorm=1, hidden_act=2, gate_bias=bias, round_h=1)
    # e4m3: every code decoded, and the encoder on values around the rounding and saturation edges
    probe = np.array([0.0, -0.0, 2.0 ** -10, 2.0 ** -9, 1.5 * 2.0 ** -9, 0.0175, 0.4375, 0.46875, 0.5, 1.0, 1.0625,
                      1.125, 1.1875, 3.75, 240.0, 416.0, 432.0, 447.9, 448.0, 449.0, 1e6, -1e6, -0.3, -17.0, 17.0,
                      20.0, 22.0, 100.0, 104.0, 108.0, -2.0 ** -9 * 0.5, 2.0 ** -9 * 0.5000001], np.float32)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "case2_oracle.npz")
    np.savez_compressed(out, cap=np.int32(cap), logits_bits=O.gate_logits(x, wg, bias).view(np.uint32),
                        topk_idx=r["topk_idx"], topk_w=r["topk_w"], count=r["count"], slot_of=r["slot_of"],
                        token_of_slot=r["token_of_slot"], out=r["out"],
                        e4m3_table_bits=O.e4m3_decode(np.arange(256, dtype=np.uint8)).view(np.uint32),
                        e4m3_probe=probe, e4m3_codes=O.e4m3_encode(probe))
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
