"""CPU tests of the host side: configuration parsing/validation through the C ABI, and that the shared library loads
and exports every symbol include/aristos_moe.h declares (no compute call is made here)."""
import ctypes as C
import json
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# the reference's shipped aristos_config.json (aristos_config.json:1-13), restated
REFERENCE_JSON = json.dumps({"capacity_factor": 1, "drop_tokens": 0, "expert_top_k": 1, "is_training": 0,
                             "hidden_act": 0, "hidden_size": 1024, "intermediate_size": 4096, "micro_batch": 4,
                             "num_experts": 1, "sequence_len": 2048, "torch_dtype": 0})


@pytest.fixture(scope="module")
def cp():
    from cuplayground_b200 import build
    build.build_library()
    import cuplayground_b200
    return cuplayground_b200


def test_library_exports_every_declared_symbol(cp):
    header = open(os.path.join(ROOT, "include", "aristos_moe.h")).read()
    declared = set(re.findall(r"ARISTOS_API\s+[\w\s\*]+?\b(aristos_\w+)\s*\(", header))
    assert len(declared) >= 30
    lib = C.CDLL(cp._lib.LIB_PATH)
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    assert declared == set(cp._lib.PROTOTYPES), declared ^ set(cp._lib.PROTOTYPES)
    cp._lib.load()
    assert cp._lib.load().aristos_version() >= 100
    assert cp._lib.load().aristos_status_str(8) == b"device-side wait timed out"


def test_reference_config_parses(cp):
    c = cp.AristosConfig.from_json(REFERENCE_JSON)
    assert (c.hidden_size, c.intermediate_size, c.num_experts, c.expert_top_k) == (1024, 4096, 1, 1)
    assert c.S == 4 * 2048                       # tokens = micro_batch * sequence_len
    assert c.capacity == c.S                     # drop_tokens = 0 -> nothing is dropped
    assert c.gate_fn == 0 and c.ep_world == 1    # extension keys default


def test_config_file_and_extensions(cp, tmp_path):
    d = json.loads(REFERENCE_JSON)
    d.update(capacity_factor=1.25, drop_tokens=1, expert_top_k=2, hidden_act=2, num_experts=8, torch_dtype=2,
             tokens=16384, hidden_size=4096, intermediate_size=14336, unknown_key={"nested": [1, 2, "x"]})
    p = tmp_path / "aristos_config.json"
    p.write_text(json.dumps(d))
    c = cp.AristosConfig.load(str(p))
    assert c.S == 16384 and c.capacity == 5120 and c.hidden_act == 2 and c.capacity_factor == 1.25
    with pytest.raises(cp.AristosError) as e:
        cp.AristosConfig.load(str(tmp_path / "missing.json"))
    assert e.value.status == 3


@pytest.mark.parametrize("patch,needle", [
    ({"hidden_size": 100}, "hidden_size"),            # multipleOf 64   (aristos_config.schema.json:29-33)
    ({"intermediate_size": 0}, "intermediate_size"),
    ({"sequence_len": 100}, "sequence_len"),          # multipleOf 128  (:49-53)
    ({"micro_batch": 3}, "micro_batch"),              # multipleOf 2    (:39-43)
    ({"drop_tokens": 2}, "drop_tokens"),              # enum 0/1        (:11-14)
    ({"hidden_act": 7}, "hidden_act"),
    ({"torch_dtype": 9}, "torch_dtype"),
    ({"num_experts": 0}, "num_experts"),
    ({"expert_top_k": 0}, "expert_top_k"),
    ({"expert_top_k": 3, "num_experts": 2}, "expert_top_k"),
    ({"capacity_factor": 0}, "capacity_factor"),
    ({"num_experts": 6, "ep_world": 4}, "ep_world"),
    ({"hidden_size": 64.5}, "integer"),
])
def test_schema_violations_are_rejected(cp, patch, needle):
    d = json.loads(REFERENCE_JSON)
    d.update(patch)
    with pytest.raises(cp.AristosError) as e:
        cp.AristosConfig.from_json(json.dumps(d))
    assert e.value.status == 2 and needle in str(e.value)


def test_missing_required_key_and_bad_json(cp):
    d = json.loads(REFERENCE_JSON)
    del d["torch_dtype"]
    with pytest.raises(cp.AristosError) as e:
        cp.AristosConfig.from_json(json.dumps(d))
    assert "torch_dtype" in str(e.value)
    d2 = json.loads(REFERENCE_JSON)
    del d2["is_training"]                      # not in the schema's "required" list
    cp.AristosConfig.from_json(json.dumps(d2))
    for bad in ("", "{", '{"hidden_size": }', "[1,2]", '{"hidden_size": 64,, }'):
        with pytest.raises(cp.AristosError):
            cp.AristosConfig.from_json(bad)


def test_baseline_configs_validate(cp, oracle):
    caps = {1: 16, 2: 320, 3: 5120, 4: 4096, 5: 256}
    for n, cap in caps.items():
        c = cp.baseline_config(n)
        c.validate()
        assert c.capacity == cap
        assert c.capacity == oracle.capacity(c.S, c.num_experts, c.expert_top_k, c.capacity_factor, c.drop_tokens)


def test_zipf_bias_matches_oracle(cp, oracle):
    import numpy as np
    b = (C.c_float * 128)()
    cp._lib.check(cp._lib.load().aristos_zipf_bias_host(b, 128, 1.2))
    np.testing.assert_array_equal(np.frombuffer(b, dtype=np.float32), oracle.zipf_bias(128, 1.2))


def test_compute_entry_points_fail_loudly_without_a_device(cp):
    """No CPU fallback: on a machine without a CUDA device creating a layer returns a CUDA error."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import cuplayground_b200.layer as layer
    with pytest.raises(RuntimeError):
        layer.MoELayer(cp.baseline_config(1))
    s = cp.baseline_config(1).to_struct()
    h = C.c_void_p()
    st = cp._lib.load().aristos_moe_create(C.byref(s), 0, 1, None, C.byref(h))
    assert st == 4, "aristos_moe_create must report ARISTOS_ERR_CUDA without a device"


def test_gate_scratch_bytes(cp):
    """Scratch of the screened gate: the expert norms plus 16 slices of S x E partial logits, 256-byte granules."""
    lib = cp._lib.load()
    assert lib.aristos_gate_scratch_bytes(0, 128) == 0 and lib.aristos_gate_scratch_bytes(128, 0) == 0
    n = lib.aristos_gate_scratch_bytes(8192, 128)
    assert n % 256 == 0 and n >= 1024 + 16 * 8192 * 128 * 4
    assert lib.aristos_gate_scratch_bytes(4096, 256) >= lib.aristos_gate_scratch_bytes(4096, 128)


def test_status_strings_cover_every_code(cp):
    lib = cp._lib.load()
    names = {lib.aristos_status_str(i).decode() for i in range(13)}
    assert len(names) == 13 and "unknown status" not in names
    assert lib.aristos_status_str(99).decode() == "unknown status"


def test_ffn_group_order_is_a_permutation_that_keeps_experts_adjacent(cp):
    """The expert GEMMs walk the (source, expert) row groups expert-major: every group exactly once, the groups of one
    expert next to each other, identity when a rank has one source or the group count is no multiple of the experts."""
    lib = cp._lib.load()
    for experts in (1, 2, 3, 8, 16, 32):
        for sources in (1, 2, 4, 8, 16):
            groups = experts * sources
            order = [lib.aristos_ffn_group_order(v, groups, experts) for v in range(groups)]
            assert sorted(order) == list(range(groups))
            by_expert = [g % experts for g in order]
            assert by_expert == sorted(by_expert)                       # expert-major
            for e in range(experts):
                srcs = [g // experts for g in order if g % experts == e]
                assert srcs == list(range(sources))                     # sources ascending inside an expert
            if sources == 1:
                assert order == list(range(groups))
    assert [lib.aristos_ffn_group_order(v, 10, 4) for v in range(10)] == list(range(10))
    assert lib.aristos_ffn_group_order(10, 10, 4) == -1 and lib.aristos_ffn_group_order(-1, 8, 4) == -1


@pytest.mark.parametrize("mt,nt,band", [(33, 16, 16), (17, 112, 8), (5, 3, 0), (4, 7, 9), (1, 1, 4), (40, 2, 16)])
def test_ffn_tile_order_is_a_bijection(cp, mt, nt, band):
    """The banded tile order of the expert GEMM visits every (row tile, column tile) of a group exactly once, and
    inside a band walks the row tiles fastest."""
    import ctypes as C
    lib = cp._lib.load()
    seen = []
    for local in range(mt * nt):
        m, n = C.c_int(-1), C.c_int(-1)
        assert lib.aristos_ffn_tile_coord(local, mt, nt, band, C.byref(m), C.byref(n)) == 0
        seen.append((m.value, n.value))
    assert sorted(seen) == [(m, n) for m in range(mt) for n in range(nt)]
    if 0 < band < mt:
        assert seen[:band] == [(m, 0) for m in range(band)]          # row tile fastest inside the first band
        assert seen[band][1] == 1 or nt == 1
        first_of_band1 = seen.index((band, 0))
        assert first_of_band1 == band * nt                            # a band finishes all its column tiles first
    else:
        assert seen[:mt] == [(m, 0) for m in range(mt)]
    m, n = C.c_int(), C.c_int()
    assert lib.aristos_ffn_tile_coord(mt * nt, mt, nt, band, C.byref(m), C.byref(n)) == -1


def test_source_order_starts_with_the_own_rank(cp):
    """The walking order of the row groups on a rank of the expert-parallel layer: expert-major, and inside an expert
    the sources in ring order from the rank itself."""
    lib = cp._lib.load()
    groups, experts = 8, 2
    for first in range(4):
        order = [lib.aristos_ffn_group_order_from(v, groups, experts, first) for v in range(groups)]
        assert sorted(order) == list(range(groups))
        assert order[0] == first * experts and order[4] == first * experts + 1          # own rows first, per expert
        assert [g % experts for g in order] == [0, 0, 0, 0, 1, 1, 1, 1]               # experts stay adjacent
        assert [g // experts for g in order[:4]] == [(first + i) % 4 for i in range(4)]
    assert lib.aristos_ffn_group_order_from(0, 8, 2, 4) == -1


def test_transport_agreement(cp):
    import ctypes as C
    lib = cp._lib.load()
    arr = lambda v: (C.c_int * len(v))(*v)
    assert lib.aristos_ep_transport_agreed(arr([1, 1, 1, 1]), 4) == 1
    assert lib.aristos_ep_transport_agreed(arr([1, 0, 1, 1]), 4) == 0
    assert lib.aristos_ep_transport_agreed(arr([0]), 1) == 0


def test_numa_binding_plan(tmp_path):
    """hostmem: the CPU set a rank binds to comes from the GPU's NUMA node as sysfs reports it (here: a fake tree)."""
    from cuplayground_b200 import hostmem
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("8-15,24-27\n")
    cpus = hostmem.node_cpus(1, sysfs=str(tmp_path))
    assert cpus == set(range(8, 16)) | set(range(24, 28))
    assert hostmem.plan_binding(set(range(0, 32)), 1, cpus) == cpus
    assert hostmem.plan_binding(set(range(8, 16)), 1, cpus) is None          # already local
    assert hostmem.plan_binding(set(range(0, 8)), 1, cpus) is None           # none of the node's CPUs allowed
    assert hostmem.plan_binding(set(range(0, 32)), None, set()) is None      # unknown node
    assert hostmem.node_cpus(7, sysfs=str(tmp_path)) == set()


def test_lazy_package_attributes_resolve_in_a_fresh_interpreter():
    """The torch-dependent names of the package are imported on first use: from a fresh interpreter, where the
    submodule has not been imported yet, both spellings must resolve (and not recurse)."""
    import subprocess
    import sys

    code = ("import cuplayground_b200 as c; assert c.MoELayer.__name__ == 'MoELayer'; "
            "from cuplayground_b200 import layer, gate_topk; assert layer.gate_topk is gate_topk")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]


def test_round_robin_expert_placement_of_a_prior():
    """interleaved_expert_prior: expert e is held in slot (e % world) * (E / world) + e // world, i.e. by rank
    e % world; the hot experts of a Zipf prior end up one per rank and world = 1 changes nothing."""
    import torch
    import cuplayground_b200.layer as layer

    E, world = 128, 8
    prior = layer.zipf_prior(E, 1.2)
    assert prior[0] == 0 and all(prior[i] > prior[i + 1] for i in range(E - 1))
    slots = layer.interleaved_expert_prior(prior, world)
    El = E // world
    for e in range(E):
        assert slots[(e % world) * El + e // world] == prior[e]
    assert sorted(slots.tolist()) == sorted(prior.tolist())
    owners_of_hottest = {int(torch.nonzero(slots == prior[e])[0]) // El for e in range(world)}
    assert owners_of_hottest == set(range(world))
    assert torch.equal(layer.interleaved_expert_prior(prior, 1), prior)
    with pytest.raises(ValueError):
        layer.interleaved_expert_prior(prior[:100], 8)
