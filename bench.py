#!/usr/bin/env python
"""Benchmark of the fused MoE forward: tokens/s at 1/2/4/8 B200, max over ranks.

    python bench.py --gpus 1 --steps 10 --warmup 3                      # this library (default workload: config 3)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...                                # the CPU restatement on the host cores

One "step" is one forward of the layer over one batch of synthetic tokens (weights stay resident). The timed region
is bracketed by a barrier and a device synchronisation and timed with CUDA events on the launching stream; the
reported time is the maximum over ranks. Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "config2": (2, "single-B200: S=8192 H=2048 I=2048 E=64 top-2 renorm softmax GELU cf=1.25 bf16 seed 1"),
    "config3": (3, "Mixtral-shaped: H=4096 I=14336 SwiGLU E=8 top-2 softmax cf=1.25 bf16, 16384 tokens per rank, "
                   "experts sharded over the ranks, seed 2"),
    # one quarter of config3 (2 of its 8 experts, a quarter of the tokens: the same 5120 rows per expert), small
    # enough for a multi-pass profiler capture
    "config3-profile": (3, "Mixtral-shaped, reduced for profiling: H=4096 I=14336 SwiGLU E=2 top-2 cf=1.25 bf16, "
                           "4096 tokens"),
    "config4": (4, "DeepSeek-V3-shaped (experts sharded over the ranks; one rank holds all of them at --gpus 1): H=7168 I=2048 SwiGLU E=256 top-8 sigmoid gate "
                   "normalised over the selected, no drops, FP8 e4m3 weights with 128x128-block fp32 scales, activations "
                   "quantised per token per 128, bf16 output, 4096 tokens, seed 3"),
    "config4-rank": (4, "DeepSeek-V3-shaped, the share of one of eight ranks: as config4 with the 32 experts a rank "
                        "owns, 4096 tokens"),
    # a quarter of config4-rank (8 of its 32 experts, 1024 tokens that all select the 8: the same ~1024 rows per
    # expert), small enough for a multi-pass profiler capture
    "config4-profile": (4, "DeepSeek-V3-shaped, reduced for profiling: as config4-rank with 8 experts and 1024 tokens "
                           "(top-8 of 8: 1024 rows per expert)"),
    "config1": (1, "the fp32 reference case: S=128 H=256 I=512 E=8 top-1 softmax ReLU cf=1.0 fp32, seed 0 (exact FFMA "
                   "expert GEMM)"),
    "config5": (5, "skewed routing: H=2048 I=1024 GELU E=128 top-4 Zipf(1.2) prior cf=1.0 bf16, 8192 tokens per "
                   "rank, seed 4"),
}


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_burst=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU every 2 ms during the timed region through NVML
    (read-only queries; nothing is set)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        import threading
        self.samples = []
        self.error = None
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:      # NVML missing: report it, do not fail the benchmark
            self.error = repr(e)
            self.thread = None
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def begin_region(self):
        """Drop what was sampled before the timed region."""
        self.samples.clear()

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((sm, pw, rs))
            except Exception as e:
                self.error = repr(e)
                return
            time.sleep(0.002)

    def stop(self) -> dict:
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [f"NVML unavailable: {self.error}"]}
        self._stop.set()
        self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"]}
        bits = 0
        for _, _, rs in self.samples:
            bits |= rs
        return {"sm_mhz": statistics.median(s[0] for s in self.samples), "sm_max_mhz": self.sm_max,
                "sm_min_mhz": min(s[0] for s in self.samples), "power_w_max": max(s[1] for s in self.samples),
                "samples": len(self.samples),
                "reasons": sorted(n for n, b in self.REASONS.items() if bits & b)}


def layer_flops(cfg, kept_assignments: int) -> float:
    m = 3 if cfg.hidden_act == 2 else 2
    return 2.0 * kept_assignments * cfg.hidden_size * cfg.intermediate_size * m + \
        2.0 * cfg.S * cfg.hidden_size * cfg.num_experts


def busiest_rank_rows(rows_per_expert, world):
    """Rows the busiest rank's experts receive: rank r owns the contiguous block of E / world expert slots
    [r E/world, (r + 1) E/world) of rows_per_expert (kept rows per slot, summed over all source ranks)."""
    E = len(rows_per_expert)
    El = E // world
    return max(sum(rows_per_expert[r * El:(r + 1) * El]) for r in range(world))


def layer_roofline(cfg, world, kept):
    """The layer roofline: the slowest of FLOPs at the dense tensor peak (2250 TFLOP/s bf16, 4500 TFLOP/s fp8), minimum
    HBM bytes at 8 TB/s and all-to-all bytes at 900 GB/s per direction (dispatch and return summed). Seconds per rank."""
    m = 3 if cfg.hidden_act == 2 else 2
    H, I, E, S = cfg.hidden_size, cfg.intermediate_size, cfg.num_experts, cfg.S
    fp8 = cfg.torch_dtype == 4
    b_w = 1 if fp8 else 2                      # bytes per weight; activations and outputs are 16-bit either way
    t_tc = layer_flops(cfg, kept) / (4500e12 if fp8 else 2250e12)
    hbm = (E // world) * m * H * I * b_w + S * H * 2 + S * H * 2 + E * H * 2
    t_hbm = hbm / 8e12
    # dispatch moves the rows as the experts read them (fp8: codes + one fp32 scale per 128), the return is 16-bit
    b_out = (1 + 4.0 / 128) if fp8 else 2
    t_a2a = kept * (world - 1) / world * H * (b_out + 2) / 900e9 if world > 1 else 0.0
    return max(t_tc, t_hbm, t_a2a), dict(t_tensor_ms=t_tc * 1e3, t_hbm_ms=t_hbm * 1e3, t_a2a_ms=t_a2a * 1e3)


# ---------------------------------------------------------------------------------------------------------------------
def cpu_sample_forward(oracle, cfg, tensors, n_tokens):
    """One oracle forward over the first n_tokens tokens (capacity scaled to the sample). Returns seconds."""
    x, wg, w1, w3, w2, bias = tensors
    cap = oracle.capacity(n_tokens, cfg.num_experts, cfg.expert_top_k, cfg.capacity_factor, cfg.drop_tokens)
    t0 = time.perf_counter()
    oracle.moe_forward(x[:n_tokens], wg, w1, w3, w2, k=cfg.expert_top_k, cap=cap, gate_fn=cfg.gate_fn,
                       renorm=cfg.renorm_topk, hidden_act=cfg.hidden_act, gate_bias=bias)
    return time.perf_counter() - t0


def cpu_calibrate(oracle, cfg, tensors, target_s):
    """Pick a sample size that takes about target_s seconds on this host."""
    n0 = min(64, tensors[0].shape[0])
    t = cpu_sample_forward(oracle, cfg, tensors, n0)
    rate = n0 / max(t, 1e-6)
    n = int(max(64, min(tensors[0].shape[0], rate * target_s)))
    return max(64, n // 64 * 64)


def host_tensors_from_oracle(oracle, cfg, n_tokens):
    import numpy as np
    H, I, E = cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    seed = cfg.seed
    rb = oracle.round_bf16
    x = rb(oracle.fill_normal(n_tokens * H, 0.0, 1.0, seed, 0)).reshape(n_tokens, H)
    wg = rb(oracle.fill_normal(E * H, 0.0, 0.02, seed, 1)).reshape(E, H)
    w1 = rb(oracle.fill_normal(E * I * H, 0.0, 0.02, seed, 2)).reshape(E, I, H)
    w3 = rb(oracle.fill_normal(E * I * H, 0.0, 0.02, seed, 3)).reshape(E, I, H) if cfg.hidden_act == 2 else None
    w2 = rb(oracle.fill_normal(E * H * I, 0.0, 0.02, seed, 4)).reshape(E, H, I)
    bias = oracle.zipf_bias(E, cfg.gate_bias_zipf_s) if cfg.gate_bias_zipf_s > 0 else None
    return x, wg, w1, w3, w2, bias


def run_reference(args, cfg, workload_desc):
    """The CPU implementation of the path (the oracle: the reference tree has no runnable CPU or GPU MoE forward)
    on all host cores; each step is a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import moe_oracle as oracle
    oracle.build()
    # every core this process may use, whatever the launcher exported (torch.distributed.run sets OMP_NUM_THREADS=1)
    oracle.use_all_cores()
    S = cfg.tokens if cfg.tokens > 0 else cfg.micro_batch * cfg.sequence_len
    n_probe = min(S, 4096)
    tensors = host_tensors_from_oracle(oracle, cfg, n_probe)
    n = min(n_probe, cpu_calibrate(oracle, cfg, tensors, target_s=4.0))
    for _ in range(args.warmup):
        cpu_sample_forward(oracle, cfg, tensors, n)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_sample_forward(oracle, cfg, tensors, n)
    value = n * args.steps / t
    cores = oracle.num_threads()
    sample = f"first {n} tokens of the workload per step (capacity scaled to the sample), fp32, OpenMP"
    line = {"impl": "reference", "metric": "moe_fwd_tokens_per_s", "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_desc, "name": args.workload, "tokens_per_step": n},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------------------
def time_ffn_variants(L, fwd, cfg, kept, local_rank, steps):
    """Both tile shapes of the expert GEMM in this process, back to back: FFN-stage milliseconds (CUDA events inside
    the forward), TFLOP/s and TFLOP/s per GHz of the median SM clock sampled while each ran."""
    import cuplayground_b200._lib as _lib
    lib = _lib.load()
    m = 3 if cfg.hidden_act == 2 else 2
    flops = 2.0 * kept * cfg.hidden_size * cfg.intermediate_size * m
    res = {}
    for name, mode in (("single", 1), ("pair_tail", 2), ("pair_padded", 3), ("single_again", 1), ("pair_tail_again", 2),
                       ("pair_padded_again", 3)):
        _lib.check(lib.aristos_ffn_set_tile_mode(mode))
        for _ in range(2):
            fwd()
        L.status()
        L.set_profiling(True)
        sampler = ClockSampler(local_rank)
        sampler.begin_region()
        for _ in range(steps):
            fwd()
        L.status()
        clocks = sampler.stop()
        ms = L.stage_ms()["ffn"]
        L.set_profiling(False)
        tf = flops / (ms * 1e-3) / 1e12
        res[name] = {"ffn_ms": ms, "tflops": tf, "sm_mhz": clocks.get("sm_mhz"),
                     "tflops_per_ghz": tf / (clocks["sm_mhz"] / 1e3) if clocks.get("sm_mhz") else None,
                     "power_w_max": clocks.get("power_w_max"), "reasons": clocks.get("reasons")}
    _lib.check(lib.aristos_ffn_set_tile_mode(0))
    return res


def copy_only(torch, xh, oh, x_dev, out_dev, steps):
    """The host copies of the end-to-end path alone (the same pinned buffers, no kernels): GB/s host-to-device,
    device-to-host, and both at once on two streams as the pipelined path issues them."""
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    nbytes = xh.numel() * xh.element_size()

    def run(do_in, do_out):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            if do_in:
                with torch.cuda.stream(s_in):
                    x_dev.copy_(xh, non_blocking=True)
            if do_out:
                with torch.cuda.stream(s_out):
                    oh.copy_(out_dev, non_blocking=True)
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    run(True, True)
    t_in, t_out, t_both = run(True, False), run(False, True), run(True, True)
    return {"h2d_gbs": nbytes * steps / t_in / 1e9, "d2h_gbs": nbytes * steps / t_out / 1e9,
            "both_s_per_step": t_both / steps, "pinned": bool(xh.is_pinned() and oh.is_pinned())}


def run_ours(args, cfg, workload_desc):
    import torch
    import torch.distributed as dist
    import cuplayground_b200.layer as layer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    # host threads and the pinned staging buffers go to the NUMA node of this rank's GPU (read from sysfs; nothing is
    # set on the GPU)
    from cuplayground_b200 import hostmem
    numa = hostmem.bind_to_gpu_numa_node(local_rank)
    uid = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        box = [layer.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        uid = box[0]

    S, H, I, E = cfg.S, cfg.hidden_size, cfg.intermediate_size, cfg.num_experts
    El = E // world
    dt = torch.bfloat16
    x, wg, w1, w3, w2, scales = layer.synthetic_tensors(cfg, rank, world)
    L = layer.MoELayer(cfg, rank, world, uid)
    out = torch.empty_like(x)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident throughput ---------------------------------------------------------------------------------
    # Expert placement for a skewed prior: across ranks the experts are held round-robin (expert e by rank e % N), so
    # the prior's hot experts spread over the ranks instead of all belonging to rank 0. The prior, indexed by expert
    # slot, is passed as the forward's gate_bias; one GPU: the layer's own prior, unchanged.
    gate_bias = None
    if world > 1 and cfg.gate_bias_zipf_s > 0 and not args.contiguous_experts:
        gate_bias = layer.interleaved_expert_prior(layer.zipf_prior(cfg.num_experts, cfg.gate_bias_zipf_s), world).cuda()
    for _ in range(args.warmup):
        L.forward(x, wg, w1, w3, w2, gate_bias=gate_bias, out=out, scales=scales)
    L.status()
    count_mine = L.routing()["count"].to(torch.float64)     # kept rows of this rank's tokens, per (global) expert
    kept = int(count_mine.sum())
    L.set_profiling(True)      # stage stopwatch: events inside the timed region, averaged over its steps
    # the sampler thread starts before the barrier: NVML start-up on rank 0 must not delay its first timed step
    # (the other ranks would wait for it inside their timed region)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    if sampler:
        sampler.begin_region()
    launches0 = L.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t_host0 = time.perf_counter()
    for _ in range(args.steps):
        L.forward(x, wg, w1, w3, w2, gate_bias=gate_bias, out=out, scales=scales)
    host_enqueue_ms = (time.perf_counter() - t_host0) * 1e3 / args.steps   # host time to enqueue one forward
    ev1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = L.launch_count - launches0
    L.status()
    ms = ev0.elapsed_time(ev1)
    # stage times averaged over the timed steps (events recorded inside the timed region, at most the last 64)
    stage = L.stage_ms()
    exchange_out_ms = L.exchange_ms() if world > 1 else 0.0
    exchange_split = L.exchange_profile() if world > 1 else None
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    kept_t = torch.tensor([kept], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(kept_t, op=dist.ReduceOp.SUM)
    ms = float(t.item())
    kept_all = float(kept_t.item())
    # rows every rank's experts receive (rank r owns experts [r E/world, (r + 1) E/world)): the forward ends when the
    # busiest rank's GEMMs end, whatever the average is
    busiest_rows = kept_all
    if world > 1:
        per_expert = count_mine.cuda()
        dist.all_reduce(per_expert, op=dist.ReduceOp.SUM)
        busiest_rows = float(busiest_rank_rows(per_expert.cpu().tolist(), world))
    value = S * world * args.steps / (ms * 1e-3)

    # ---- end to end: host activations in, host result out, through the public host API. Every step copies its own
    # pinned input to the device and its result back; consecutive steps are submitted without waiting in between
    # (aristos_moe_submit_host), so the copies of one step overlap the kernels of its neighbours.
    L.set_profiling(False)
    NBUF = 4                        # as many host buffer pairs as the host API keeps calls in flight
    xh = [x.cpu().pin_memory() for _ in range(NBUF)]
    oh = [torch.empty_like(xh[0]).pin_memory() for _ in range(NBUF)]
    L.forward_host(xh[0], wg, w1, w3, w2, oh[0], gate_bias=gate_bias, scales=scales)
    # enough steps that filling and draining the three-stage pipeline (copy in | kernels | copy out) is amortised: a
    # forward of a fraction of a millisecond gets 100 steps, the 8 ms forward of the default workload at most 20
    e2e_steps = max(4, min(args.steps, 20)) if ms / args.steps >= 2.0 else 100
    barrier()
    t_start = time.perf_counter()
    for i in range(e2e_steps):
        L.submit_host(xh[i % NBUF], wg, w1, w3, w2, oh[i % NBUF], gate_bias=gate_bias, scales=scales)
    L.wait_host()
    torch.cuda.synchronize()
    t_e2e = time.perf_counter() - t_start
    barrier()
    te = torch.tensor([t_e2e * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = S * world * e2e_steps / (float(te.item()) * 1e-3)
    # the same through the blocking call (copy in, forward, copy out, return), for reference
    barrier()
    t_start = time.perf_counter()
    for i in range(4):
        L.forward_host(xh[i & 1], wg, w1, w3, w2, oh[i & 1], gate_bias=gate_bias, scales=scales)
    t_blk = time.perf_counter() - t_start
    tb = torch.tensor([t_blk * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tb, op=dist.ReduceOp.MAX)
    e2e_blocking = S * world * 4 / (float(tb.item()) * 1e-3)
    L.status()
    assert all(torch.equal(o, oh[0]) for o in oh[1:]) and torch.equal(oh[0], out.cpu()), \
        "host path result differs from device path"
    # the copies alone, all ranks at once (what the host side of this box allows)
    barrier()
    copies = copy_only(torch, xh[0], oh[0], torch.empty_like(x), out, e2e_steps)
    barrier()
    tc_ = torch.tensor([copies["both_s_per_step"], -copies["h2d_gbs"], -copies["d2h_gbs"]], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(tc_, op=dist.ReduceOp.MAX)
    copies.update(both_s_per_step=float(tc_[0]), h2d_gbs=-float(tc_[1]), d2h_gbs=-float(tc_[2]))

    # ---- parity of this run's last forward against the CPU oracle, on the first and the last rank: routing bit-exact
    # on every token of the rank, sampled output rows within the 16-bit tolerance (checker only, not timed)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    parity = None
    check_ranks = sorted({0, world - 1})
    if not args.no_parity:
        mine = None
        if rank in check_ranks:
            import parity as parity_mod
            from oracle import moe_oracle as oracle
            oracle.build()
            oracle.use_all_cores()
            try:
                mine = parity_mod.check_rank(cfg, L, x, wg, out, n_rows=16 if cfg.torch_dtype == 4 else 64, seed=rank,
                                             gate_bias=None if gate_bias is None else gate_bias.cpu().numpy())
            except AssertionError as e:
                mine = {"ok": False, "routing": f"MISMATCH: {e}", "rows": 0, "max_rel": None, "mean_rel": None}
            mine["rank"] = rank
        if world > 1:
            box = [None] * world
            dist.all_gather_object(box, mine)
            got = [b for b in box if b is not None]
        else:
            got = [mine]
        parity = {"ranks": [g["rank"] for g in got],
                  "routing": "bit-exact" if all(g["routing"] == "bit-exact" for g in got) else
                  "; ".join(str(g["routing"]) for g in got),
                  "rows": sum(g["rows"] for g in got),
                  "max_rel": max((g["max_rel"] for g in got if g["max_rel"] is not None), default=None),
                  "mean_rel": max((g["mean_rel"] for g in got if g["mean_rel"] is not None), default=None),
                  "tolerance": "routing tensors bit-exact on every token of the rank; sampled output rows "
                               "max|d|/max|ref| < 2e-2 and mean|d|/mean|ref| < 1e-2 against the fp32 oracle over the "
                               "global weights",
                  "ok": all(g["ok"] for g in got)}

    # ---- both tile shapes of the expert GEMM, timed in this process (one GPU, 16-bit tensor-core workloads)
    variants = None
    if world == 1 and cfg.torch_dtype in (2, 3) and cfg.capacity >= 1024 and not args.no_variants:
        variants = time_ffn_variants(L, lambda: L.forward(x, wg, w1, w3, w2, gate_bias=gate_bias, out=out, scales=scales), cfg, kept,
                                     local_rank, max(3, min(args.steps, 10)))

    if rank == 0:
        peaks = read_peaks()
        # dominant kernel: the grouped expert GEMM (two launches per forward, up- and down-projection)
        m = 3 if cfg.hidden_act == 2 else 2
        ffn_flops = 2.0 * kept * H * I * m            # this rank's experts' rows (equal across ranks in expectation)
        if world > 1:
            ffn_flops = 2.0 * (kept_all / world) * H * I * m
        # DRAM bytes per GEMM launch: ncu dram__bytes_read+write of the up and down projections on config3-profile
        # (8192 rows: 810 MB + 1282 MB), scaled by the rows of this run; only valid for the config-3 shape
        traffic, traffic_src = None, None
        if args.workload.startswith("config3"):
            rows = kept if world == 1 else kept_all / world
            traffic = (1026e6 + 1196e6) / 8192.0 * rows / 2.0
            traffic_src = ("ncu capture on config3-profile (profiles/ffn_grouped_gemm_config3_profile_ncu_full.md), "
                           "scaled by rows, average of the two launches of a forward")
        ffn_s = stage["ffn"] * 1e-3
        achieved = ffn_flops / ffn_s / 1e12
        fp8 = cfg.torch_dtype == 4
        if fp8:
            # one rank holding many experts with ~128 rows each: the expert GEMMs stream every weight once
            w_bytes = float((E // world) * m * H * I)                       # e4m3: one byte per weight
            a_bytes = float(kept) * (H + 2 * I + I + 2 * H)                 # xq in, h out (bf16), hq in, y out (bf16)
            hbm = (w_bytes + a_bytes) / ffn_s / 1e9
            roofline_fp8 = {"bound": "hbm", "kernel": "ffn_fp8_grouped_gemm_kernel", "achieved": hbm,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm / peaks["hbm_gbs"], "traffic": None,
                            "peak_source": f"{peaks['source']} copy bandwidth", "algorithmic_bytes": w_bytes + a_bytes,
                            "tflops": achieved, "ms_per_step": stage["ffn"]}
        # the timed loop is short (well under a second), so the burst cuBLAS figure is the denominator
        roofline = {"bound": "tensor", "kernel": "ffn_grouped_gemm_pair_kernel",
                    "achieved": achieved,
                    "peak": peaks["bf16_burst"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_burst"],
                    "frac_of_sustained_peak": achieved / peaks["bf16_sustained"],
                    "traffic": traffic, "traffic_source": traffic_src,
                    "peak_source": f"{peaks['source']} bf16 burst (cuBLAS 8192^3, best of 10)",
                    "launches_per_step": 2, "flops_per_step": ffn_flops, "ms_per_step": stage["ffn"]}
        t_roof, terms = layer_roofline(cfg, world, kept_all / world)
        if world > 1:
            # the same with the rows of the busiest rank in the tensor term (routing decides how many rows an expert,
            # and with it a rank, gets: up to the capacity factor above the mean, more with a skewed prior)
            t_busy, _ = layer_roofline(cfg, world, busiest_rows)
            terms["rows_received"] = {"mean_per_rank": kept_all / world, "busiest_rank": busiest_rows,
                                      "busiest_over_mean": busiest_rows / (kept_all / world)}
            terms["frac_busiest_rank"] = t_busy / (ms / args.steps * 1e-3)
        line = {"metric": "moe_fwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": {0: "f32", 1: "tf32", 2: "bf16", 3: "f16", 4: "fp8_e4m3"}[cfg.torch_dtype],
                "data": "synthetic",
                "config": {"workload": workload_desc, "name": args.workload, "tokens_per_rank": S,
                           "parallelism": f"ep{world}", "ep_transport": L.ep_transport,
                           "expert_placement": "round-robin over the ranks (prior indexed by expert slot)" if gate_bias is not None else "contiguous blocks", "l2": "weights (>= 0.4 GB per rank) exceed the 126 MB L2, "
                           "no flush needed between steps", "kept_assignments": kept_all},
                "clocks": clocks,
                "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": xh[0].numel() * xh[0].element_size() * world,
                        "d2h_bytes_per_step": oh[0].numel() * oh[0].element_size() * world, "steps": e2e_steps,
                        "api": "aristos_moe_submit_host per step + aristos_moe_wait_host (pinned host activations "
                               "in, host result out every step; up to four steps in flight)", "timing": "host wall clock, "
                        "device synchronised on both sides, max over ranks",
                        "blocking_call_value": e2e_blocking,
                        "copy_only": {**copies, "tokens_per_s": S * world / copies["both_s_per_step"],
                                      "what": "the same pinned buffers copied in and out per step with no kernels, "
                                              "all ranks at once; GB/s are the slowest rank's"},
                        "numa": numa},
                "gpu_launches": int(launches),
                "roofline": roofline_fp8 if fp8 else roofline,
                "layer_roofline": {"seconds": t_roof, **terms, "frac": t_roof / (ms / args.steps * 1e-3),
                                   "constants": "2250 TFLOP/s dense bf16 (4500 fp8), 8 TB/s HBM, 900 GB/s NVLink per "
                                                "direction"},
                "stage_ms": stage, "host_enqueue_ms_per_step": host_enqueue_ms}
        if world > 1:
            # the outgoing exchange of rank 0: rows that leave the rank x row bytes over the time of its count + gather
            # kernels (part of stage_ms["ffn"]); the rest of that stage is the GEMMs with the return fused in
            sent_bytes = kept_all / world * (world - 1) / world * H * 2
            line["exchange"] = {"gather_ms": exchange_out_ms, "rows_to_peers_bytes": sent_bytes,
                                "gather_gbs": sent_bytes / (exchange_out_ms * 1e-3) / 1e9 if exchange_out_ms > 0 else None,
                                "what": "rank 0: count + gather kernels storing kept rows into the owning ranks over "
                                        "NVLink, CUDA events inside the forward"}
            if exchange_split is not None and exchange_split["gemms"] > 0:
                # the expert-FFN stage of rank 0 split at its cross-rank waits: until every rank's counts have
                # arrived, the GEMMs (arrival waits per source inside, return fused), until every return has arrived
                line["exchange"]["stage_split_ms"] = exchange_split
        if parity is not None:
            line["parity"] = parity
        if variants is not None:
            line["ffn_variants"] = variants
        if world == 1 and not args.no_cpu_baseline:
            from oracle import moe_oracle as oracle
            oracle.build()
            host = lambda a: None if a is None else a.float().cpu().numpy()
            n_probe = min(S, 4096)
            bias = oracle.zipf_bias(E, cfg.gate_bias_zipf_s) if cfg.gate_bias_zipf_s > 0 else None
            tensors = (host(x[:n_probe]), host(wg), host(w1), host(w3), host(w2), bias)
            n = min(n_probe, cpu_calibrate(oracle, cfg, tensors, target_s=12.0))
            tc = cpu_sample_forward(oracle, cfg, tensors, n)
            line["cpu_baseline"] = {"value": n / tc, "unit": "tokens/s", "cores": oracle.num_threads(),
                                    "kind": "port", "sample": f"first {n} tokens of the same workload, one forward "
                                    f"({tc:.1f} s), capacity scaled to the sample, fp32 OpenMP oracle"}
        print(json.dumps(line), flush=True)
    L.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        raise SystemExit("parity check against the CPU oracle failed: " + json.dumps(parity))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="config3")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the last forward")
    ap.add_argument("--no-variants", action="store_true", help="skip the timing of both GEMM tile shapes")
    ap.add_argument("--contiguous-experts", action="store_true",
                    help="N > 1, skewed prior: leave the prior's hot experts on the first rank (no round-robin placement)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3     # timing rule: at least three warm-up steps
    import cuplayground_b200 as cp
    n, desc = WORKLOADS[args.workload]
    cfg = cp.baseline_config(n, world=args.gpus if args.impl == "ours" else 1)
    if args.workload == "config3-profile":
        cfg.num_experts, cfg.tokens = 2, 4096
    if args.workload == "config4-rank":
        cfg.num_experts = 32
    if args.workload == "config4-profile":
        cfg.num_experts, cfg.tokens = 8, 1024
    if args.workload.startswith("config4"):
        if args.workload != "config4" and args.gpus != 1 and args.impl == "ours":
            raise SystemExit(f"{args.workload} is a one-GPU share of config4: run config4 with --gpus N instead")
        args.no_cpu_baseline = True      # the fp32 oracle would need the de-quantised weights of every expert on the host
    if args.impl == "reference":
        run_reference(args, cfg, desc)
    else:
        run_ours(args, cfg, desc)


if __name__ == "__main__":
    main()
