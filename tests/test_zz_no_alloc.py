"""aristos_dispatch_static: the dispatch entry point for callers that are not allowed to allocate device memory
(an inference server whose memory pool already owns the whole GPU, or a hot loop where cudaMalloc could stall or
fail). It keeps its scratch in a fixed array inside the library, so it must give exactly what aristos_dispatch gives
with caller scratch - also on a second call that finds the first call's leftovers in that array.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _topk(rng, S, E, k, skew):
    p = 1.0 / np.arange(1, E + 1) ** skew
    p /= p.sum()
    return np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(S)]).astype(np.int32)


def test_dispatch_static_matches_dispatch_on_two_calls_in_a_row():
    import torch
    import cuplayground_b200.layer as layer

    rng = np.random.default_rng(2024)
    # first a large skewed problem that fills many chunk histograms, then a small one that reuses the same array
    for S, E, k, cap, skew in ((8192, 128, 4, 256, 1.2), (100, 8, 2, 20, 0.5)):
        topk = torch.from_numpy(_topk(rng, S, E, k, skew)).cuda()
        ref = layer.dispatch(topk, E, cap)                 # caller-provided scratch
        got = layer.dispatch_static(topk, E, cap)          # built-in scratch, no allocation inside the library
        torch.cuda.synchronize()
        for g, r, name in zip(got, ref, ("count", "slot_of", "token_of_slot")):
            assert torch.equal(g, r), name                 # integer work: bit-exact


def test_dispatch_static_rejects_sizes_beyond_its_scratch():
    import torch
    import cuplayground_b200 as cp
    import cuplayground_b200.layer as layer

    too_many_tokens = torch.zeros((131072 // 2 + 1, 2), dtype=torch.int32, device="cuda")
    with pytest.raises(cp.AristosError) as e:
        layer.dispatch_static(too_many_tokens, 8, 16)
    assert e.value.status == 2 and "limit" in str(e.value)
    with pytest.raises(cp.AristosError) as e:
        layer.dispatch_static(torch.zeros((16, 1), dtype=torch.int32, device="cuda"), 257, 16)
    assert e.value.status == 2
