"""Generates tests/golden/config1_oracle.npz from the CPU oracle (run from the repository root:
`python tests/golden/make_golden.py`).

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


if __name__ == "__main__":
    main()
