"""Host-side arithmetic of bench.py (no GPU, nothing timed): the layer roofline terms and the busiest rank's rows."""
import importlib.util
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    sys.path.insert(0, ROOT)
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_busiest_rank_rows(bench):
    rows = [10, 0, 3, 7, 1, 1, 1, 1]
    assert bench.busiest_rank_rows(rows, 1) == 24
    assert bench.busiest_rank_rows(rows, 2) == 20          # slots 0-3 against 4-7
    assert bench.busiest_rank_rows(rows, 4) == 10
    assert bench.busiest_rank_rows(rows, 8) == 10


def test_layer_roofline_terms_of_the_mixtral_shape(bench):
    """Config 3 on one rank: 32768 kept assignments x 2 H I 3 FLOP (plus the gate's 2 S H E) at 2250 TFLOP/s is the slowest term; the
    all-to-all term appears only across ranks and grows with the share of rows that leave the rank."""
    import cuplayground_b200 as cp
    cfg = cp.baseline_config(3, world=1)
    t, terms = bench.layer_roofline(cfg, 1, 32768)
    flops = 32768 * 2 * cfg.hidden_size * cfg.intermediate_size * 3 + 2 * cfg.S * cfg.hidden_size * cfg.num_experts  # + gate
    assert terms["t_tensor_ms"] == pytest.approx(flops / 2250e12 * 1e3, rel=1e-9)
    assert t == pytest.approx(terms["t_tensor_ms"] * 1e-3) and terms["t_a2a_ms"] == 0.0
    cfg8 = cp.baseline_config(3, world=8)
    t8, terms8 = bench.layer_roofline(cfg8, 8, 32768)
    assert terms8["t_a2a_ms"] == pytest.approx(32768 * 7 / 8 * cfg.hidden_size * 4 / 900e9 * 1e3, rel=1e-9)
    assert terms8["t_hbm_ms"] < terms["t_hbm_ms"]            # an eighth of the expert weights per rank
    assert t8 == pytest.approx(terms8["t_tensor_ms"] * 1e-3)
