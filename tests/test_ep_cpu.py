"""Expert-parallel path on CPU ranks (gloo, world_size 2 and 4): the product's host-side exchange logic
(aristos_ep_exchange_plan / aristos_ep_row_windows, the same functions the NCCL path executes) moves real rows between
processes, the CPU oracle stands in for the kernels, and every rank's output must equal an independent single-rank
oracle run over the global weights (capacity is per source rank)."""
import ctypes as C
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _plan(lib, rank, world, bpp, stride, offset, length):
    n = lib.aristos_ep_exchange_plan(rank, world, bpp, stride, offset, length, None, 0)
    buf = (C.c_int64 * (5 * n))()
    assert lib.aristos_ep_exchange_plan(rank, world, bpp, stride, offset, length, buf, n) == n
    return np.frombuffer(buf, dtype=np.int64).reshape(n, 5)


def _exchange(dist, torch, plan, send: np.ndarray, recv: np.ndarray, rank):
    """Executes a plan on flat byte buffers with gloo point-to-point operations."""
    sb, rb = send.view(np.uint8).reshape(-1), recv.view(np.uint8).reshape(-1)
    reqs, landing = [], []
    for to, so, frm, ro, n in plan:
        if to == rank:
            assert frm == rank
            rb[ro:ro + n] = sb[so:so + n]
            continue
        reqs.append(dist.isend(torch.from_numpy(sb[so:so + n].copy()), dst=int(to)))
        t = torch.empty(int(n), dtype=torch.uint8)
        reqs.append(dist.irecv(t, src=int(frm)))
        landing.append((t, int(ro), int(n)))
    for r in reqs:
        r.wait()
    for t, ro, n in landing:
        rb[ro:ro + n] = t.numpy()


def _worker(rank, world, port, E, S, H, I, k, cf, act, q):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import torch
        import torch.distributed as dist
        from helpers import make_inputs
        from oracle import moe_oracle as O
        import cuplayground_b200 as cp

        os.environ["OMP_NUM_THREADS"] = "2"
        lib = cp._lib.load()
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        El = E // world
        cap = O.capacity(S, E, k, cf)
        _, wg, w1, w3, w2 = make_inputs(S, H, I, E, seed=100, swiglu=(act == 2), w_std=0.1)        # shared weights
        x = make_inputs(S, H, I, E, seed=200 + rank, w_std=0.1)[0]                               # this rank's tokens
        loc = slice(rank * El, (rank + 1) * El)
        w1l, w3l, w2l = w1[loc], (None if w3 is None else w3[loc]), w2[loc]

        # local routing + gather (what gate / dispatch / permute do on the GPU)
        idx, w = O.gate_topk(O.gate_logits(x, wg), k, 0, 1)
        count, slot_of, tos = O.dispatch(idx, E, cap)
        xg = O.permute(x, tos)                                              # (E*cap, H) send layout

        # counts: one block of E_local int32 per peer
        rcount = np.zeros(world * El, np.int32)
        _exchange(dist, torch, _plan(lib, rank, world, 1, El * 4, 0, El * 4), count, rcount, rank)
        all_counts = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(all_counts, torch.from_numpy(count))
        expect = np.concatenate([c.numpy()[loc] for c in all_counts])
        assert (rcount == expect).all(), "count exchange landed in the wrong group"

        # rows travel in the layer's row windows; the FFN runs per window on (source, local expert) groups
        wr, nw = C.c_int(), C.c_int()
        cp._lib.check(lib.aristos_ep_row_windows(cap, C.byref(wr), C.byref(nw)))
        assert wr.value % 128 == 0 and wr.value * nw.value >= cap > wr.value * (nw.value - 1)
        row_bytes, stride = H * 4, cap * H * 4
        xr = np.zeros((world * El * cap, H), np.float32)
        yr = np.zeros((world * El, cap, H), np.float32)
        yg = np.zeros((E * cap, H), np.float32)
        groups_w1 = np.concatenate([w1l] * world)
        groups_w3 = None if w3l is None else np.concatenate([w3l] * world)
        groups_w2 = np.concatenate([w2l] * world)
        for c in range(nw.value):
            r0, r1 = c * wr.value, min(cap, (c + 1) * wr.value)
            _exchange(dist, torch, _plan(lib, rank, world, El, stride, r0 * row_bytes, (r1 - r0) * row_bytes), xg, xr, rank)
            cnt_w = np.clip(rcount - r0, 0, r1 - r0).astype(np.int32)
            y_w = O.expert_ffn(xr.reshape(world * El, cap, H)[:, r0:r1].copy(), cnt_w, groups_w1, groups_w3,
                               groups_w2, act)
            yr[:, r0:r1] = y_w
            _exchange(dist, torch, _plan(lib, rank, world, El, stride, r0 * row_bytes, (r1 - r0) * row_bytes),
                      yr.reshape(-1, H), yg, rank)
        out = O.combine(yg, slot_of, w)

        ref = O.moe_forward(x, wg, w1, w3, w2, k=k, cap=cap, renorm=1, hidden_act=act)
        assert (ref["slot_of"] == slot_of).all()
        np.testing.assert_allclose(out, ref["out"], rtol=1e-5, atol=1e-6)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:      # pragma: no cover - reported to the parent
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))


@pytest.mark.parametrize("world,E,S,k,cf,act", [(2, 4, 96, 2, 1.0, 1), (2, 8, 640, 2, 1.25, 2), (4, 8, 64, 2, 1.5, 0),
                                                  (2, 4, 2200, 2, 1.0, 1)])   # cap 1100: two row windows
def test_expert_parallel_on_cpu_ranks(world, E, S, k, cf, act):
    import torch.multiprocessing as mp
    from cuplayground_b200 import build
    build.build_library()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, E, S, 64, 128, k, cf, act, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    bad = [r for r in results if r[1] != "ok"]
    assert not bad, bad[0][1]


def _toy_worker(rank, world, port, q):
    try:
        sys.path.insert(0, ROOT)
        import torch
        import torch.distributed as dist
        from oracle import moe_oracle as O
        import cuplayground_b200 as cp

        lib = cp._lib.load()
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        M = N = K = 2
        blk = M * K
        # the reference's fill (auditorium/overlap.cuh:197-204): world input blocks rank + i, one weight rank + j + 4
        mk_a = lambda r: (r + np.arange(world * blk, dtype=np.float32)).reshape(world, M, K)
        mk_b = lambda r: (r + 4 + np.arange(N * K, dtype=np.float32)).reshape(N, K)
        a, b = mk_a(rank), mk_b(rank)
        plan = _plan(lib, rank, world, 1, blk * 4, 0, blk * 4)
        # dispatch: block d of every rank goes to rank d (put-with-signal of overlap.cuh:94-101)
        recv = np.zeros_like(a)
        _exchange(dist, torch, plan, a, recv, rank)
        # first stage: GEMM of every received block with the local weight (overlap.cuh:110-115)
        c1 = np.stack([O.gemm_bias_act(recv[s], b, None, 3) for s in range(world)])
        # return (overlap.cuh:124-127), then the fused GEMM + ReLU of the second stage (overlap.cuh:138-146)
        back = np.zeros_like(c1)
        _exchange(dist, torch, plan, c1, back, rank)
        c2 = np.stack([O.gemm_bias_act(back[s], b, None, 0) for s in range(world)])
        # recomputed without any exchange: what rank d did to this rank's block d, then this rank's second stage
        for d in range(world):
            first = mk_a(rank)[d] @ mk_b(d).T
            np.testing.assert_array_equal(back[d], first)
            np.testing.assert_array_equal(c2[d], np.maximum(first @ b.T, 0.0))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception as e:      # pragma: no cover - reported to the parent
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))


def test_reference_overlap_prototype_toy_on_two_ranks():
    """The reference's two-stage exchange/GEMM toy (overlapPrototype: 2x2x2 blocks filled with rank + i and
    rank + j + 4) replayed on CPU ranks through the product's exchange plan; the reference records no expected
    values, so every rank checks against a recomputation that involves no exchange."""
    import torch.multiprocessing as mp
    from cuplayground_b200 import build
    build.build_library()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_toy_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    bad = [r for r in results if r[1] != "ok"]
    assert not bad, bad[0][1]


def test_exchange_plan_is_a_permutation():
    """Every (destination rank, block) is written exactly once and sends pair up with receives."""
    import cuplayground_b200 as cp
    from cuplayground_b200 import build
    build.build_library()
    lib = cp._lib.load()
    world, bpp, stride, off, ln = 8, 3, 1000, 128, 256
    plans = [_plan(lib, r, world, bpp, stride, off, ln) for r in range(world)]
    written = set()
    for r, plan in enumerate(plans):
        assert len(plan) == world * bpp
        assert (plan[:bpp, 0] == r).all() and (plan[:bpp, 2] == r).all(), "own blocks come first"
        for to, so, frm, ro, n in plan:
            assert n == ln and (so - off) % stride == 0 and (so - off) // stride // bpp == to
            assert (ro - off) // stride // bpp == frm
            # the matching send on the peer targets this receive
            peer = plans[frm]
            match = [(t2, s2) for t2, s2, _, _, _ in peer if t2 == r and (s2 - off) // stride % bpp == (ro - off) // stride % bpp]
            assert len(match) == 1
            written.add((r, int(ro)))
    assert len(written) == world * world * bpp
    assert lib.aristos_ep_exchange_plan(3, 2, 1, 8, 0, 8, None, 0) == -1


def test_row_windows():
    import cuplayground_b200 as cp
    lib = cp._lib.load()
    for cap, exp_rows, exp_n in ((5120, 1280, 4), (320, 384, 1), (256, 256, 1), (1100, 640, 2), (16, 128, 1)):
        wr, nw = C.c_int(), C.c_int()
        cp._lib.check(lib.aristos_ep_row_windows(cap, C.byref(wr), C.byref(nw)))
        assert (wr.value, nw.value) == (exp_rows, exp_n), (cap, wr.value, nw.value)


# ---- the arrival-flag protocol and its time limit, among CPU ranks ----------------------------------------------------
def _flag_worker(rank, world, port, q):
    """Two forwards. In the first every rank publishes its flags to every rank; in the second rank 1 never sends.
    Rank 0 must see rank 1 pending until its time limit, release its own page, and end with nothing pending."""
    try:
        sys.path.insert(0, ROOT)
        import time
        import torch.distributed as dist
        import cuplayground_b200 as cp
        lib = cp._lib.load()
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        page = np.zeros(lib.aristos_ep_flag_words(), dtype=np.uint32)
        ptr = page.ctypes.data_as(C.c_void_p)
        KIND_IN, KIND_COUNT = 0, 2
        pending = lambda epoch, kind: lib.aristos_ep_flags_pending(ptr, epoch, world, kind, 0)

        store = dist.distributed_c10d._get_default_store()

        def publish(epoch, kind):          # "store my epoch into my word of every rank's page"
            page[lib.aristos_ep_flag_word_index(kind, 0, rank)] = epoch
            for d in range(world):
                if d != rank:
                    store.set(f"flag/{d}/{kind}/{rank}/{epoch}", "1")

        def poll_arrivals(srcs, epoch, kind, limit_s):
            """Take in the peers' flag stores until nothing is pending or the limit passes; True when complete."""
            t0 = time.time()
            while pending(epoch, kind):
                for s in srcs:
                    if store.check([f"flag/{rank}/{kind}/{s}/{epoch}"]):
                        page[lib.aristos_ep_flag_word_index(kind, 0, s)] = epoch
                if time.time() - t0 > limit_s:
                    return False
                time.sleep(0.005)
            return True

        others = [r for r in range(world) if r != rank]
        # forward 1: everyone takes part (counts, then rows)
        for kind in (KIND_COUNT, KIND_IN):
            publish(1, kind)
            assert poll_arrivals(others, 1, kind, 20.0), f"rank {rank}: forward 1 did not complete"
            assert pending(1, kind) == 0
        assert pending(2, KIND_COUNT) == (1 << world) - 1          # nothing of forward 2 has arrived yet
        result = "ok"
        if rank == 0:
            # forward 2: rank 1 never sends. Rank 0 publishes, waits with a limit, then releases its own page.
            publish(2, KIND_COUNT)
            t0 = time.time()
            done = poll_arrivals(others, 2, KIND_COUNT, 1.0)
            waited = time.time() - t0
            if done or not (0.9 < waited < 10.0):
                result = f"expected a timeout after about 1 s, got done={done} after {waited:.2f} s"
            elif pending(2, KIND_COUNT) != 0b10:
                result = f"pending set {pending(2, KIND_COUNT):b}, expected rank 1 only"
            else:
                lib.aristos_ep_flags_release(ptr, 2)
                if pending(2, KIND_COUNT) or pending(2, KIND_IN) or lib.aristos_ep_flags_pending(ptr, 2, world, 1, 3):
                    result = "flags still pending after the release"
                elif pending(3, KIND_COUNT) != (1 << world) - 1:
                    result = "the release must not satisfy a later epoch"
        # rank 1 simply does not take part in forward 2 (it keeps its process alive until rank 0 is done)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, result))
    except Exception as e:      # pragma: no cover
        import traceback
        q.put((rank, "".join(traceback.format_exception(e))))


def test_missing_peer_and_release_among_cpu_ranks():
    """Host-side failure handling of the exchange, without a GPU: the product's flag-page functions
    (aristos_ep_flags_pending / aristos_ep_flags_release, the same comparison and layout the stream waits and kernels
    use) driven by two gloo ranks, one of which stops sending."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_flag_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    bad = [r for r in results if r[1] != "ok"]
    assert not bad, bad[0][1]


def test_flag_comparison_is_cyclic():
    import cuplayground_b200 as cp
    lib = cp._lib.load()
    page = np.zeros(lib.aristos_ep_flag_words(), dtype=np.uint32)
    ptr = page.ctypes.data_as(C.c_void_p)
    i0, i1 = lib.aristos_ep_flag_word_index(0, 2, 0), lib.aristos_ep_flag_word_index(0, 2, 1)
    assert i0 >= 0 and i1 == i0 + 1 and lib.aristos_ep_flag_word_index(3, 0, 0) == -1
    page[i0], page[i1] = 0xFFFFFFFF, 2                      # epochs wrap around: 2 is AFTER 0xFFFFFFFF
    assert lib.aristos_ep_flags_pending(ptr, 0xFFFFFFFF, 2, 0, 2) == 0
    assert lib.aristos_ep_flags_pending(ptr, 1, 2, 0, 2) == 0b01
    assert lib.aristos_ep_flags_pending(ptr, 3, 2, 0, 2) == 0b11


def test_dense_packing_plan_is_consistent_across_ranks():
    """fp8 expert parallel: from the all-gathered counts every rank computes where its rows start inside each expert's
    dense group at the owner, and every owner where each source's rows start. The senders' start rows must tile the
    owners' groups exactly (no gap, no overlap), whatever the counts."""
    import cuplayground_b200 as cp
    lib = cp._lib.load()
    rng = np.random.default_rng(5)
    for world, E_local in ((2, 3), (4, 2), (8, 4)):
        E = world * E_local
        allcount = rng.integers(0, 300, size=(world, E)).astype(np.int32)
        allcount[rng.integers(0, world), rng.integers(0, E)] = 0
        plans = []
        for rank in range(world):
            send_base = np.full(E, -1, np.int32)
            dense_count = np.full(E_local, -1, np.int32)
            src_off = np.full(E_local * (world + 1), -1, np.int32)
            st = lib.aristos_ep_dense_plan_host(allcount.ctypes.data_as(C.c_void_p), world, E, E_local, rank,
                                                send_base.ctypes.data_as(C.c_void_p),
                                                dense_count.ctypes.data_as(C.c_void_p),
                                                src_off.ctypes.data_as(C.c_void_p))
            assert st == 0
            plans.append((send_base, dense_count, src_off.reshape(E_local, world + 1)))
        for e in range(E):
            owner, el = divmod(e, E_local)
            _, dense_count, src_off = plans[owner]
            assert dense_count[el] == allcount[:, e].sum()
            for s in range(world):
                # sender s starts where the owner expects source s, and the next source starts right behind its rows
                assert plans[s][0][e] == src_off[el, s]
                assert src_off[el, s + 1] == src_off[el, s] + allcount[s, e]
    bad = np.zeros(4, np.int32)
    assert lib.aristos_ep_dense_plan_host(bad.ctypes.data_as(C.c_void_p), 2, 5, 2, 0, bad.ctypes.data_as(C.c_void_p),
                                          bad.ctypes.data_as(C.c_void_p), bad.ctypes.data_as(C.c_void_p)) == 1
