#!/usr/bin/env python
"""Benchmark of the KV-cache data-movement path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--ops LIST]

Headline workload (the line's `metric` / `value`): the Llama-3.1-8B decode-step cache write —
32 layers, 8 KV heads x 128, bf16, block_size 16, 65 536 blocks per GPU (128 GiB cache), batch
256 with context lengths U[128, 4096].  One *step* writes the new token of every sequence into
every layer's paged cache: 256 x 2 KiB x (K, V) read and written per layer = 2 MiB per layer,
64 MiB per step.

Timing protocol of the headline: W untimed warm-up steps; barrier; a few more untimed steps
inside the region (the first launches after an idle GPU and a collective are not
representative); then R rounds of exactly K steps, issued as replays of one CUDA graph that
holds m consecutive rounds (about 2 ms of work), every replay with its own CUDA event pair on
the launching stream, R chosen so that the region lasts at least 120 ms; `ms_per_step` is the
MEDIAN replay divided by m K, max over ranks; best / worst replay, the per-rank medians and the SM clocks sampled inside that region
are reported beside it.  `e2e` times the same step
through the Python API with key / value / slot_mapping packed in pinned host memory: one
host-to-device copy per step on a copy stream, double-buffered against the kernel, and the
library's error record copied back to the host every step.

The other workloads of the path (chunked prefill + copy-on-write, GPU<->host swap, TP-sharded
decode write, prefill->decode transfer, rotary fusion, index preparation, the per-layer call
against flashinfer) are timed in the same run and reported under `ops`.  With N > 1 (torchrun,
one rank per GPU) every rank runs the same per-GPU workload (KV heads are sharded per GPU, no
collective on the data path) and the prefill->decode transfer runs between rank g and rank
g + N/2, where the bytes that arrived are compared with the bytes that were sent.

`--impl reference` times the reference semantics as PyTorch index ops on the host cores, with
the same `config`, rounds and median.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import workloads as W  # noqa: E402  (input generators only; the product package is imported by run_ours)

METRIC = "kv_cache_write_bandwidth"
UNIT = "GB/s"
ROTATE = 8  # disjoint input sets cycled through so sources never sit in L2
NOMINAL = {"hbm_GB/s": 8000.0, "pcie_gen5_x16_GB/s": 64.0, "nvlink5_GB/s_per_direction": 900.0}


def headline_config() -> dict:
    """What is measured, in the same words for both arms (`--impl ours` and `reference`)."""
    w = W.config2()
    s = w.shape
    return {
        "workload": "llama31_8b_decode_write: one step scatters the new K and V row (2 KiB each) of 256 "
                    "sequences into all 32 layers of a 65536-block (128 GiB) paged bf16 cache through "
                    "slot_mapping",
        "bytes_per_step": w.algorithmic_bytes(), "layers": s.num_layers, "tokens_per_step": w.num_tokens,
        "row_bytes": s.row_bytes, "block_size": s.block_size, "cache_blocks_per_gpu": s.num_blocks,
        "context_lengths": "uniform in [128, 4096]", "input_sets_rotated": ROTATE,
        "l2": f"rotating {ROTATE} disjoint input sets ({ROTATE * 64} MiB of sources, distinct destination "
              "blocks) > 126 MB L2",
        "per_gpu": "same workload on every rank (KV heads sharded per GPU, no collective on the path)",
    }


# ----------------------------------------------------------------------------- utilities
def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def profile_traffic(kernel: str, workload: str = "decode_write"):
    """DRAM bytes per launch (`dram__bytes_read.sum + dram__bytes_write.sum`) that the committed
    ncu summary of THIS kernel on this workload states, or None when there is no summary for
    the kernel that ran: the figure follows the kernel, it is not a constant of the bench."""
    f = ROOT / "profiles" / f"{kernel}_{workload}_small.md"
    try:
        m = re.search(r"^traffic_bytes_per_launch:\s*([0-9.eE+]+)", f.read_text(), re.M)
        return (float(m.group(1)), f.name) if m else (None, None)
    except OSError:
        return None, None


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML (read-only) while work is timed."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting",
        0x100: "display_clock_setting", 0x10: "sync_boost",
    }

    def __init__(self, index: int, period: float = 0.02):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period = period
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def sample(self):
        if self._nv is None:
            return
        try:
            self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
            mask = self._nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": sorted(self.reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def timed(comm, stream, fn, steps: int, warmup: int, sampler=None, local_ms=None) -> float:
    """Runs fn(i) warmup + steps times; returns milliseconds for the `steps` timed calls,
    measured with CUDA events on `stream`, max over ranks (this rank's own figure is appended
    to `local_ms` when a list is given)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    comm.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(steps):
        fn(warmup + i)
    e1.record(stream)
    if sampler is not None:
        sampler.sample()
    torch.cuda.synchronize()
    comm.barrier()
    torch.cuda.synchronize()
    if local_ms is not None:
        local_ms.append(e0.elapsed_time(e1))
    return comm.max(e0.elapsed_time(e1))


def rounds_per_graph(steps: int, est_step_us: float, target_ms: float = 2.0, max_nodes: int = 512) -> int:
    """How many rounds of `steps` steps one CUDA graph holds: enough for about `target_ms` of
    device work, at least one, at most `max_nodes` launches per graph.  Between two graph
    launches the programmatic overlap of consecutive kernels is lost once (about 8 us on
    B200); a graph of one 20-step round (0.2 ms) would carry that as 4 % of its time."""
    per_round_ms = max(steps * est_step_us * 1e-3, 1e-6)
    m = max(1, math.ceil(target_ms / per_round_ms))
    return max(1, min(m, max_nodes // max(1, steps)))


def measure_rounds(comm, stream, run_block, steps: int, rounds_per_block: int, device_index: int,
                   min_region_ms: float = 120.0, min_blocks: int = 20, max_blocks: int = 2000):
    """The headline protocol.  `run_block()` enqueues `rounds_per_block` rounds of exactly
    `steps` steps (one graph replay).  After a barrier a few blocks run untimed inside the
    region, then B blocks are timed, each with its own CUDA event pair on the launching stream,
    B chosen so that the region lasts at least `min_region_ms`.  Returns (median ms per round
    as max over ranks, statistics, per-rank medians in us per step, clocks sampled inside the
    region)."""
    m = rounds_per_block
    for _ in range(3):
        run_block()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(3):
        run_block()
    e1.record(stream)
    torch.cuda.synchronize()
    est = max(e0.elapsed_time(e1) / 3, 1e-3)
    blocks = int(min(max_blocks, max(min_blocks, math.ceil(min_region_ms / est))))
    blocks = int(comm.max(float(blocks)))           # the same count on every rank
    warm_blocks = max(2, math.ceil(5 / max(1, steps * m)))
    events = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
    torch.cuda.synchronize()
    comm.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(device_index, period=0.004)
    with sampler:
        for _ in range(warm_blocks):
            run_block()
        events[0].record(stream)
        for b in range(blocks):
            run_block()
            events[b + 1].record(stream)
        torch.cuda.synchronize()
    comm.barrier()
    times = [events[b].elapsed_time(events[b + 1]) / m for b in range(blocks)]   # ms per round
    med = statistics.median(times)
    stats = {"rounds": blocks * m, "steps_per_round": steps, "rounds_per_event_pair": m,
             "event_pairs": blocks, "in_region_warmup_steps": warm_blocks * m * steps,
             "region_ms": round(sum(times) * m, 3),
             "us_per_step_median": round(med / steps * 1e3, 4),
             "us_per_step_best": round(min(times) / steps * 1e3, 4),
             "us_per_step_worst": round(max(times) / steps * 1e3, 4),
             "us_per_step_p10_p90": [round(float(np.percentile(times, q)) / steps * 1e3, 4) for q in (10, 90)]}
    per_rank = [round(x, 4) for x in comm.gather_objects(med / steps * 1e3)]
    return comm.max(med), stats, per_rank, sampler.summary()


def graph_of(stream, fn):
    """Captures fn(raw_stream) on a side stream into a CUDA graph."""
    side = torch.cuda.Stream()
    side.wait_stream(stream)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        fn(torch.cuda.current_stream().cuda_stream)
    stream.wait_stream(side)
    torch.cuda.synchronize()
    return g


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    from lmserve_b200 import _lib, host_topology
    from lmserve_b200.disagg import Comm
    from lmserve_b200.ops import cache_ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the cache ops have no CPU path "
                         "(use --impl reference for the host baseline)")
    rank, world, local = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # as the reference's workers do before they allocate pinned memory: stay on the cores next
    # to this rank's GPU (restored before the CPU baseline, which uses every core)
    try:
        affinity_before = os.sched_getaffinity(0)
    except AttributeError:
        affinity_before = None
    bound_cpus = host_topology.set_cpu_affinity_for_gpu(local)
    link = host_topology.pcie_link(local)
    comm = Comm(world, dev)
    L = _lib.lib()
    stream = torch.cuda.current_stream()
    peak_gbs, peak_kind = load_peaks()
    ops_wanted = set(args.ops.split(","))
    sampler = ClockSampler(local)
    launches0 = L.lms_launch_count()
    failed = []

    # One allocation backs every cache view of the run (sized for the largest: 128 GiB).
    shape2 = W.SHAPES["llama31_8b"]
    if args.small:
        shape2 = shape2.scaled(num_blocks=2048)
    full_blocks = shape2.num_blocks
    pool = None
    while pool is None:
        try:
            pool = torch.empty(shape2.cache_bytes // 2, dtype=torch.bfloat16, device=dev)
        except torch.OutOfMemoryError:
            # a device that cannot hold the 128 GiB cache still gets measured, on the largest
            # power-of-two pool that fits; the per-step inputs stay the same
            if shape2.num_blocks <= 2048:
                raise
            shape2 = shape2.scaled(num_blocks=shape2.num_blocks // 2)
            torch.cuda.empty_cache()
    reduced_pool = shape2.num_blocks != full_blocks

    def cache_view(shape: W.KVShape) -> torch.Tensor:
        n = int(np.prod(shape.cache_shape))
        if n > pool.numel():
            raise RuntimeError(f"{shape.name}: cache view larger than the device pool")
        return pool[:n].view(*shape.cache_shape)

    result = {}
    ops = {}

    with sampler:
        # ------------------------------------------------------------- headline: decode write
        wl = [W.config2(seed=1002 + 17 * i + 1000 * rank) for i in range(ROTATE)]
        if reduced_pool or args.small:
            for i, w in enumerate(wl):
                w.slot_mapping = renumber_blocks(w.slot_mapping, shape2.block_size, shape2.num_blocks, 77 + i)
        T, Lyr = wl[0].num_tokens, shape2.num_layers
        kv = cache_view(shape2)
        keys = [torch.randn(Lyr, T, shape2.num_kv_heads, shape2.head_dim, device=dev,
                            dtype=torch.bfloat16) for _ in range(ROTATE)]
        vals = [torch.randn_like(k) for k in keys]
        slots = [torch.from_numpy(w.slot_mapping).to(dev) for w in wl]
        step_bytes = wl[0].algorithmic_bytes()

        # Arguments are resolved once per input set (WritePlan); a step is then one C call,
        # so the host enqueues faster than the GPU drains and the device time is what is timed.
        sp = stream.cuda_stream
        fused = [cache_ops.WritePlan(keys[j], vals[j], kv, slots[j]) for j in range(ROTATE)]

        def step_fused(i):
            fused[i % ROTATE].run(sp)

        for i in range(args.warmup):
            step_fused(i)
        # A round is exactly K steps.  Rounds are issued as replays of ONE CUDA graph that holds
        # m consecutive rounds (m x K launches, cycling through the input sets), m chosen for
        # about 2 ms of device work per replay, and every replay is timed by its own event pair.
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(50):
            step_fused(i)
        e1.record(stream)
        torch.cuda.synchronize()
        est_us = e0.elapsed_time(e1) / 50 * 1e3
        m_rounds = 1 if args.small else int(comm.max(float(rounds_per_graph(args.steps, est_us))))
        g_steps = m_rounds * args.steps
        fused_graph = graph_of(stream, lambda cs: [fused[j % ROTATE].run(cs) for j in range(g_steps)])
        ms_round, round_stats, per_rank_us, region_clocks = measure_rounds(
            comm, stream, fused_graph.replay, args.steps, m_rounds, local,
            **({"min_region_ms": 1.0, "min_blocks": 3} if args.small else {}))
        ms_per_step = ms_round / args.steps
        value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
        result.update(ms_per_step=ms_per_step, value=value)
        how = (f"replays of one CUDA graph of {m_rounds} round(s) x {args.steps} steps = {g_steps} launches, "
               "one event pair per replay")
        graph_launches = (round_stats["event_pairs"] + 8) * g_steps   # replays bypass the C ABI counter

        # side measurements use at least this many iterations (the profiling case stays short)
        def at_least(n):
            return args.steps if args.small else max(args.steps, n)

        # the same steps as plain eager launches on the stream
        ms_s = timed(comm, stream, step_fused, at_least(200), max(args.warmup, 10), sampler) / at_least(200)
        ops["decode_write_eager_stream"] = {"us_per_step": ms_s * 1e3,
                                            "GB/s": step_bytes / (ms_s * 1e-3) / 1e9}

        # yardstick: a plain contiguous device copy of the same volume (32 MiB in, 32 MiB out),
        # same rotation of sources, torch's copy kernel
        flat_src = [torch.cat((keys[j].view(-1), vals[j].view(-1))) for j in range(2)]
        flat_dst = [torch.empty_like(t) for t in flat_src]
        n_c = at_least(100)
        ms_c = timed(comm, stream, lambda i: flat_dst[i % 2].copy_(flat_src[i % 2]), n_c, 5, sampler) / n_c
        ops["contiguous_copy_same_volume_torch"] = {"us_per_copy": ms_c * 1e3,
                                                    "GB/s": step_bytes / (ms_c * 1e-3) / 1e9}
        del flat_src, flat_dst

        # the same step through the general-purpose wrapper (argument checks on every call)
        ms_w = timed(comm, stream, lambda i: cache_ops.reshape_and_cache_layers(
            keys[i % ROTATE], vals[i % ROTATE], kv, slots[i % ROTATE]), n_c, 5, sampler) / n_c
        ops["decode_write_unplanned_wrapper"] = {"us_per_step": ms_w * 1e3,
                                                 "GB/s": step_bytes / (ms_w * 1e-3) / 1e9}

        # per-layer forms of the same step: 32 launches, eager and replayed from a CUDA graph
        layer_plans = [[cache_ops.WritePlan(keys[j][l], vals[j][l], kv[l], slots[j]) for l in range(Lyr)]
                       for j in range(ROTATE)]

        def step_layers(i):
            for p in layer_plans[i % ROTATE]:
                p.run(sp)

        n_l = at_least(50)
        # host-bound (32 Python calls per step): the best of three runs
        ms_pl = min(timed(comm, stream, step_layers, n_l, 5, sampler) for _ in range(1 if args.small else 3)) / n_l
        ops["decode_write_per_layer_eager"] = {
            "us_per_step": ms_pl * 1e3, "us_per_layer_call": ms_pl * 1e3 / Lyr,
            "GB/s": step_bytes / (ms_pl * 1e-3) / 1e9, "launches_per_step": Lyr}
        graphs = [graph_of(stream, lambda cs, j=j: [p.run(cs) for p in layer_plans[j]]) for j in range(ROTATE)]
        ms_g = timed(comm, stream, lambda i: graphs[i % ROTATE].replay(), n_l, 5, sampler) / n_l
        ops["decode_write_per_layer_graph"] = {
            "us_per_step": ms_g * 1e3, "us_per_layer_call": ms_g * 1e3 / Lyr,
            "GB/s": step_bytes / (ms_g * 1e-3) / 1e9, "launches_per_step": Lyr}
        graph_launches += (n_l + 5) * Lyr
        del graphs

        # ------------------------------------------------------------- e2e: host buffers
        e2e = bench_e2e(comm, stream, kv, keys, vals, wl, step_bytes, world, args, sampler)

        # ------------------------------------------------------------- other workloads
        if args.small:
            ops_wanted = ops_wanted & {"prefill_cow", "swap", "rope", "transfer_local", "index_prep", "tp8"}

        def extra(names, fn):
            """Runs one of the other workloads; a failure there (a pool that does not fit, no
            pinned memory) is recorded and does not lose the headline number."""
            if not (ops_wanted & ({"all"} | set(names))):
                return
            torch.cuda.nvtx.range_push(names[0])   # lets a profiler select one workload's launches
            try:
                ops.update(fn())
            except Exception as e:  # noqa: BLE001 - reported in the output line
                if world > 1:
                    raise  # ranks must not diverge around barriers
                ops[names[0]] = {"skipped": repr(e)[:300]}
                torch.cuda.synchronize()
            finally:
                torch.cuda.nvtx.range_pop()

        if world == 1:
            extra(["prefill_cow"], lambda: bench_prefill_cow(comm, stream, cache_view, dev, peak_gbs,
                                                             sampler, args.small))
            extra(["swap"], lambda: bench_swap(comm, stream, cache_view, dev, args, sampler, link))
            extra(["rope"], lambda: bench_rope_fusion(comm, stream, cache_view, dev, args, sampler))
            extra(["index_prep"], lambda: bench_index_prep(comm, stream, dev, args, sampler))
            if torch.cuda.device_count() >= 2 and "transfer_local" in ops_wanted:
                extra(["transfer_local"], lambda: bench_transfer_local(comm, stream, cache_view, dev,
                                                                       args, sampler))
            if "write_scaling" in ops_wanted:
                extra(["write_scaling"], lambda: bench_write_scaling(comm, stream, cache_view, dev, peak_gbs,
                                                                     args, sampler))
            if not args.small:
                extra(["flashinfer"], lambda: bench_vs_flashinfer(comm, stream, cache_view, dev, args, sampler))
        extra(["tp8"], lambda: bench_tp8_decode(comm, stream, cache_view, dev, rank, world, peak_gbs,
                                                args, sampler, local))
        if world >= 2 and world % 2 == 0:
            extra(["transfer"], lambda: bench_transfer(comm, stream, cache_view, dev, rank, world, sampler))
            if not ops.get("prefill_to_decode_transfer", {}).get("transfer_bit_exact", True):
                failed.append("prefill_to_decode_transfer: bytes that arrived differ from the bytes sent")

    launches = int(L.lms_launch_count() - launches0) + graph_launches
    if affinity_before is not None:
        try:
            os.sched_setaffinity(0, affinity_before)
        except OSError:
            pass
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline(bounded_seconds=10.0)
            cpu["single_thread"] = cpu_single_thread(3.0)
            cpu["other_ops"] = cpu_other_ops(cpu["cores"])
        achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
        kernel = L.lms_write_kernel_name(shape2.row_bytes, step_bytes).decode()
        traffic, traffic_src = profile_traffic(kernel)
        config = headline_config()
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 6),
            "us_per_decode_step_write": round(ms_per_step * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "u8", "data": "synthetic",
            "config": config,
            "run": {"small_profiling_case": bool(args.small), "cache_blocks_allocated": shape2.num_blocks,
                    "steps_issued_as": how, "timing": round_stats, "us_per_step_by_rank": per_rank_us,
                    "cpus_bound_to": (f"{bound_cpus[0]}-{bound_cpus[-1]} ({len(bound_cpus)} cores local to the GPU)"
                                      if bound_cpus else "unchanged (no local_cpulist in sysfs)"),
                    "pcie_link": link},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak_gbs,
                         "unit": "GB/s", "frac": round(achieved / peak_gbs, 4),
                         "peak_kind": peak_kind,
                         "frac_of_nominal_8000": round(achieved / NOMINAL["hbm_GB/s"], 4),
                         "traffic": traffic, "traffic_unit": "bytes per launch, in-kernel, from the ncu summary "
                                                             f"profiles/{traffic_src}" if traffic_src else
                                                             "no ncu summary committed for this kernel",
                         "kernel": kernel, "algorithmic_bytes_per_launch": step_bytes},
            "e2e": {k: (round(v, 3) if isinstance(v, float) else v) for k, v in e2e.items()},
            "gpu_launches": launches,
            "clocks": region_clocks,
            "clocks_whole_run": sampler.summary(),
            "ops": round_floats(ops),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if failed:
            line["failed"] = failed
        print(json.dumps(line), flush=True)
    comm.close()
    if failed:
        raise SystemExit(3)


def bench_e2e(comm, stream, kv, keys, vals, wl, step_bytes, world, args, sampler):
    """The headline step through the Python API from host buffers.  Key, value and the slot
    mapping of a step sit packed in ONE pinned staging buffer; a step is one host-to-device
    copy on a copy stream, the write (WritePlan.run) on the main stream and an asynchronous
    copy of the library's 32-byte error record back to pinned memory.  Two device buffers
    alternate, so the upload of step i+1 overlaps the kernel and the read-back of step i; the
    host looks at the record of step i-2 before it reuses that step's buffers."""
    from lmserve_b200 import _lib
    from lmserve_b200.ops import cache_ops
    L = _lib.lib()
    dev = kv.device
    nkb = keys[0].numel() * 2
    T = wl[0].num_tokens
    stage_bytes = 2 * nkb + T * 8
    host = [torch.empty(stage_bytes, dtype=torch.uint8).pin_memory() for _ in range(2)]
    for j in range(2):
        host[j][:nkb].copy_(keys[j].view(-1).view(torch.uint8))
        host[j][nkb:2 * nkb].copy_(vals[j].view(-1).view(torch.uint8))
        host[j][2 * nkb:].copy_(torch.from_numpy(wl[j].slot_mapping.copy()).view(torch.uint8))
    devb = [torch.empty(stage_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    dk = [b[:nkb].view(torch.bfloat16).view(keys[0].shape) for b in devb]
    dv = [b[nkb:2 * nkb].view(torch.bfloat16).view(keys[0].shape) for b in devb]
    ds = [b[2 * nkb:].view(torch.int64) for b in devb]
    plans = [cache_ops.WritePlan(dk[j], dv[j], kv, ds[j]) for j in range(2)]
    record = torch.zeros(2, 32, dtype=torch.uint8).pin_memory()
    up = torch.cuda.Stream()
    uploaded = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]
    sp = stream.cuda_stream
    state = {"issued": 0, "checked": 0}

    def check(j):
        done[j].synchronize()
        if int(record[j, :4].view(torch.int32)[0]) != 0:
            raise RuntimeError("a cache-write kernel reported an out-of-range slot")
        state["checked"] += 1

    def step_e2e(i):
        j = i % 2
        if state["issued"] >= 2:
            check(j)                       # step i-2 is complete and clean; its buffers are free
        with torch.cuda.stream(up):
            up.wait_stream(stream) if state["issued"] == 0 else None
            devb[j].copy_(host[j], non_blocking=True)
            uploaded[j].record(up)
        stream.wait_event(uploaded[j])
        plans[j].run(sp)
        _lib.check(L.lms_error_record_async(record[j].data_ptr(), sp))
        done[j].record(stream)
        state["issued"] += 1

    n_e2e = 20 if args.small else max(20, min(args.steps, 100))
    times, mine = [], []
    for _ in range(3 if not args.small else 1):
        state["issued"] = 0
        ms = timed(comm, stream, step_e2e, n_e2e, 4, sampler, local_ms=mine) / n_e2e
        for j in range(2):
            check(j)
        times.append(ms)
    ms_e2e = statistics.median(times)
    ms_mine = statistics.median(mine) / n_e2e
    # the host-to-device memcpy rate of this rank in the same run: the very staging buffers of
    # the loop above copied back to back with nothing else going on (20 copies, best of 3), and
    # the same with every rank copying at the same time (after a barrier, max over ranks)
    def copies(i):
        devb[i % 2].copy_(host[i % 2], non_blocking=True)

    best = None
    rank = int(os.environ.get("RANK", "0"))
    for turn in range(world):              # one rank at a time: "alone" must mean alone
        torch.cuda.synchronize()
        comm.barrier()
        if turn != rank:
            continue
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(20):
                copies(i)
            e1.record(stream)
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / 20
            best = t if best is None else min(best, t)
    torch.cuda.synchronize()
    comm.barrier()
    h2d_gbs = stage_bytes / (best * 1e-3) / 1e9
    h2d_concurrent = min(timed(comm, stream, copies, 20, 4, sampler) for _ in range(3)) / 20
    per_rank = comm.gather_objects({"e2e_ms_per_step": round(ms_mine, 4),
                                    "h2d_GB/s_in_e2e": round(stage_bytes / (ms_mine * 1e-3) / 1e9, 2),
                                    "h2d_memcpy_GB/s_alone": round(h2d_gbs, 2)})
    rate = stage_bytes / (ms_e2e * 1e-3) / 1e9
    together = stage_bytes / (h2d_concurrent * 1e-3) / 1e9
    limiter = "the PCIe host-to-device copy of the step's 32 MiB of K/V rows; the kernel is 2 % of the step"
    if world > 1 and together < 0.9 * h2d_gbs:
        limiter += (f"; with {world} ranks uploading at once the host side is the ceiling: plain pinned "
                    f"cudaMemcpy of the same buffers reaches {together:.1f} GB/s on the slowest rank "
                    f"against {h2d_gbs:.1f} GB/s when this rank copies alone")
    return {"value": world * step_bytes / (ms_e2e * 1e-3) / 1e9, "unit": UNIT,
            "h2d_bytes_per_step": stage_bytes, "d2h_bytes_per_step": 32, "ms_per_step": ms_e2e,
            "steps_timed": n_e2e, "rounds": len(times), "h2d_copies_per_step": 1,
            "error_records_read_back": state["checked"], "h2d_GB/s_achieved": rate,
            "h2d_memcpy_GB/s_same_run": h2d_gbs, "frac_of_h2d_memcpy": rate / h2d_gbs,
            "h2d_memcpy_GB/s_all_ranks_at_once": together,
            "limiter": limiter, "by_rank": per_rank}


def round_floats(o):
    if isinstance(o, float):
        return round(o, 3)
    if isinstance(o, dict):
        return {k: round_floats(v) for k, v in o.items()}
    if isinstance(o, list):
        return [round_floats(v) for v in o]
    return o


def renumber_blocks(slots: np.ndarray, block_size: int, num_blocks: int, seed: int) -> np.ndarray:
    """Maps the blocks a slot mapping touches onto random distinct blocks of a smaller pool."""
    blocks, inv = np.unique(slots // block_size, return_inverse=True)
    new = np.random.default_rng(seed).permutation(num_blocks)[:len(blocks)].astype(np.int64)
    return new[inv] * block_size + slots % block_size


def bench_prefill_cow(comm, stream, cache_view, dev, peak_gbs, sampler, small=False):
    """Qwen2.5-7B shape: 64 x 512-token prefill chunks + 4096 copy-on-write pairs (32 -> 128)."""
    from lmserve_b200.ops import cache_ops
    w = W.config3()
    if small:  # 2 of the 28 layers: a 4 GiB cache, same index inputs
        w.shape = w.shape.scaled(num_layers=2)
    s = w.shape
    kv = cache_view(s)
    T = len(w.slot_mapping)
    # sources of two rotating sets: 2 x 28 x 32768 x 1 KiB x 2 = 3.5 GiB each
    sets = 2
    keys = [torch.randn(s.num_layers, T, s.num_kv_heads, s.head_dim, device=dev, dtype=torch.bfloat16)
            for _ in range(sets)]
    vals = [torch.randn_like(k) for k in keys]
    slots = torch.from_numpy(w.slot_mapping).to(dev)
    pairs = torch.from_numpy(w.pairs).to(dev)
    out = {}
    n = 6
    ms = timed(comm, stream, lambda i: cache_ops.reshape_and_cache_layers(
        keys[i % sets], vals[i % sets], kv, slots), n, 3, sampler) / n
    wb = w.write_bytes()
    out["prefill_chunk_write"] = {"ms": ms, "bytes": wb, "GB/s": wb / (ms * 1e-3) / 1e9,
                                  "frac_of_hbm_peak": wb / (ms * 1e-3) / 1e9 / peak_gbs}
    ms = timed(comm, stream, lambda i: cache_ops.copy_blocks(kv, pairs), n, 3, sampler) / n
    cb = w.cow_bytes()
    out["copy_blocks_cow"] = {"ms": ms, "bytes_compulsory": cb, "GB/s": cb / (ms * 1e-3) / 1e9,
                              "frac_of_hbm_peak": cb / (ms * 1e-3) / 1e9 / peak_gbs,
                              "GB/s_counting_every_read": 2 * len(w.pairs) * s.num_layers * s.chunk_bytes / (ms * 1e-3) / 1e9}
    # the reference's call form: a {src: [dst, ...]} dict, flattened and uploaded inside the call
    as_dict = {}
    for src, dst in w.pairs.tolist():
        as_dict.setdefault(src, []).append(dst)
    ms_d = timed(comm, stream, lambda i: cache_ops.copy_blocks(kv, as_dict), n, 3, sampler) / n
    t0 = time.perf_counter()
    for _ in range(20):
        cache_ops.flatten_block_map(as_dict)
    out["copy_blocks_cow"]["ms_with_dict_argument"] = ms_d
    out["copy_blocks_cow"]["host_us_to_flatten_the_dict"] = (time.perf_counter() - t0) / 20 * 1e6
    return out


def bench_rope_fusion(comm, stream, cache_view, dev, args, sampler):
    """One decode layer of Llama-3.1-8B (256 tokens, 32 query / 8 KV heads of 128): rotary
    embedding then cache write as two launches, against the fused launch.  32 layers per CUDA
    graph, rotating input sets."""
    from lmserve_b200.ops import cache_ops, rotary_embedding_ops as R
    s = W.SHAPES["llama31_8b"]
    if args.small:
        s = s.scaled(num_blocks=2048)
    kv = cache_view(s)
    T, NH, NKV, HD = 256, 32, 8, 128
    cs = R.build_cos_sin_cache(8192, HD, torch.bfloat16, device=dev)
    sets = []
    for i in range(ROTATE):
        w = W.config2(seed=3002 + 17 * i)
        slots = w.slot_mapping
        if args.small:
            slots = renumber_blocks(slots, s.block_size, s.num_blocks, 177 + i)
        qkv = torch.randn(s.num_layers, T, (NH + 2 * NKV) * HD, device=dev, dtype=torch.bfloat16)
        pos = torch.from_numpy(w.context_lens.astype(np.int32)).to(dev)
        sets.append((qkv, pos, torch.from_numpy(slots).to(dev)))
    q_out = torch.empty(T, NH * HD, device=dev, dtype=torch.bfloat16)
    k_out = torch.empty(T, NKV * HD, device=dev, dtype=torch.bfloat16)

    def split(qkv_l):
        return qkv_l[:, :NH * HD], qkv_l[:, NH * HD:(NH + NKV) * HD], qkv_l[:, (NH + NKV) * HD:]

    def separate(j):
        qkv, pos, slots = sets[j]
        for l in range(s.num_layers):
            q, k, v = split(qkv[l])
            R._launch(q, k, None, pos, cs, HD, q_out, k_out, None, None)
            cache_ops.reshape_and_cache(k_out.view(T, NKV, HD), v.view(T, NKV, HD), kv[l], slots)

    def fused(j):
        qkv, pos, slots = sets[j]
        for l in range(s.num_layers):
            q, k, v = split(qkv[l])
            R._launch(q, k, v, pos, cs, HD, q_out, None, kv[l], slots)

    out = {}
    for name, fn in (("rope_then_cache_write_2_launches", separate), ("rope_and_cache_fused_1_launch", fused)):
        fn(0)
        torch.cuda.synchronize()
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        for j in range(ROTATE):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn(j)
            graphs.append(g)
        stream.wait_stream(side)
        torch.cuda.synchronize()
        reps = max(8, args.steps // 4)
        ms = timed(comm, stream, lambda i: graphs[i % ROTATE].replay(), reps, 3, sampler) / reps
        out[name] = {"us_per_layer": ms * 1e3 / s.num_layers, "us_per_32_layers": ms * 1e3}
    return out


def reference_way(inputs, dev, flashinfer=None, page_size=16):
    """LMServe's own way to prepare a step's index tensors (model_worker.py:310-433), restated
    as the timed baseline: Python lists, one torch.tensor(...).to('cuda') per array and
    flashinfer's two helpers (a torch restatement of them when flashinfer is absent)."""
    flatten_input_ids, position_ids, seqlens_q = [], [], []
    inputs.sort(key=lambda x: -x.input_len)
    for data in inputs:
        flatten_input_ids += data.input_ids
        position_ids += [i for i in range(data.filled_token_len, data.context_len)]
        seqlens_q.append(data.input_len)
    ids = torch.tensor(flatten_input_ids, dtype=torch.long).to(dev, non_blocking=True)
    pos_ids = torch.tensor(position_ids, dtype=torch.int).to(dev, non_blocking=True)
    cu_q = torch.tensor(np.cumsum([0] + seqlens_q), dtype=torch.int).to(dev, non_blocking=True)
    kv_block_indices, num_blocks_per_seqs, kv_last_block_lens = [], [], []
    for data in inputs:
        kv_block_indices += data.block_ids
        num_blocks_per_seqs.append(len(data.block_ids))
        kv_last_block_lens.append((data.context_len - 1) % page_size + 1)
    indptr = torch.tensor(np.cumsum([0] + num_blocks_per_seqs), dtype=torch.int).to(dev, non_blocking=True)
    indices = torch.tensor(kv_block_indices, dtype=torch.int).to(dev, non_blocking=True)
    last = torch.tensor(kv_last_block_lens, dtype=torch.int).to(dev, non_blocking=True)
    nnz = sum(seqlens_q)
    if flashinfer is not None:
        b, p = flashinfer.get_batch_indices_positions(
            cu_q, flashinfer.get_seq_lens(indptr, last, page_size), nnz)
    else:
        seq = torch.clamp(indptr[1:] - indptr[:-1] - 1, min=0) * page_size + last
        q = cu_q[1:] - cu_q[:-1]
        b = torch.repeat_interleave(torch.arange(len(inputs), device=dev, dtype=torch.int), q.long())
        p = (torch.arange(nnz, device=dev, dtype=torch.int) - cu_q[b.long()] + (seq - q)[b.long()]).int()
    return ids, pos_ids, cu_q, indptr, indices, last, b, p



def bench_index_prep(comm, stream, dev, args, sampler):
    """Per-step index preparation, host wall time per step with a synchronize at the end (the
    forward pass cannot start before its indices exist): LMServe's way — Python lists, one
    torch.tensor(...).to('cuda') per array and flashinfer's two helpers
    (model_worker.py:310-433), restated here as the baseline — against one packed upload and one
    kernel (StepInputBuilder).  Same request objects, seeded; a decode step of 256 requests and
    a chunked-prefill step of 64 x 512 tokens."""
    import copy
    import time
    from lmserve_b200.step_inputs import StepInputBuilder
    try:
        import flashinfer
    except Exception:  # noqa: BLE001
        flashinfer = None

    def reference_way_here(inputs):
        return reference_way(inputs, dev, flashinfer)

    cases = {
        "decode_256_requests": dict(num_decode=256, ctx_lo=128, ctx_hi=4096, num_prefill=0,
                                    chunk_tokens=0, max_offset=0),
        "prefill_64x512_tokens": dict(num_decode=0, ctx_lo=0, ctx_hi=0, num_prefill=64,
                                      chunk_tokens=512, max_offset=8192),
    }
    builder = StepInputBuilder(dev, 16, max_batch=256, max_tokens=32768, max_blocks=131072)
    out = {"flashinfer_helpers": flashinfer is not None}
    for name, kw in cases.items():
        reqs = [W.make_step_requests(65536, 16, seed=6000 + i, **kw) for i in range(4)]
        ref = reference_way_here(copy.copy(reqs[0]))
        ids, s = builder.make_inputs(copy.copy(reqs[0]))
        torch.cuda.synchronize()
        same = (torch.equal(ref[0], ids) and torch.equal(ref[1], s.position_ids)
                and torch.equal(ref[2], s.cu_seqlens_q) and torch.equal(ref[3], s.kv_block_indptrs)
                and torch.equal(ref[4], s.kv_block_indices) and torch.equal(ref[5], s.kv_last_block_lens)
                and torch.equal(ref[6], s.batch_indices) and torch.equal(ref[7], s.positions))
        res = {"results_match": bool(same), "tokens": int(ids.numel()),
               "block_table_entries": int(s.kv_block_indices.numel())}
        for label, fn in (("reference_way_us", reference_way_here), ("one_upload_one_kernel_us", builder.make_inputs)):
            times = []
            for i in range(23):
                r = copy.copy(reqs[i % 4])
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                fn(r)
                torch.cuda.synchronize()
                times.append(time.perf_counter() - t0)
            res[label] = float(np.median(times[3:])) * 1e6
        # the device part alone: the kernel re-run on the uploaded buffer
        T, NB, B = int(ids.numel()), int(s.kv_block_indices.numel()), len(reqs[0])
        builder.make_inputs(copy.copy(reqs[0]))
        ms = timed(comm, stream, lambda i: builder._launch(B, T, NB, 0, 0, 0), 50, 3, sampler) / 50
        res["kernel_us"] = ms * 1e3
        out[name] = res
    return {"index_prep": out}


def host_pool_blocks(chunk_layers_bytes: int, want_blocks: int, cap_gib: float) -> int:
    """Blocks of the pinned host pool: the specified count halved until the pool fits both the
    cap (`--host-pool-gib`) and half of the memory that is available right now.  The
    specification's 131 072 blocks are 256 GiB, more than the GPU box has."""
    avail = None
    try:
        for line in Path("/proc/meminfo").read_text().splitlines():
            if line.startswith("MemAvailable:"):
                avail = int(line.split()[1]) * 1024
    except Exception:
        pass
    for cg in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            v = Path(cg).read_text().strip()
            if v.isdigit():
                avail = min(avail, int(v)) if avail else int(v)
        except Exception:
            pass
    limit = int(cap_gib * (1 << 30))
    if avail:
        limit = min(limit, int(avail * 0.5))
    n = want_blocks
    while n > 1 and n * chunk_layers_bytes > limit:
        n //= 2
    return n


def bench_swap(comm, stream, cache_view, dev, args, sampler, link=None):
    """Llama-3.1-8B swap: 8192 random blocks x 32 layers x 64 KiB each way (16 GiB)."""
    from lmserve_b200 import _lib
    from lmserve_b200.kv_worker import HostPool
    from lmserve_b200.ops import cache_ops
    s = W.SHAPES["llama31_8b_swap"]
    per_block = s.num_layers * s.chunk_bytes
    if args.small:  # profiling case: 2048 GPU blocks (4 GiB), 1 GiB moved each way
        s = s.scaled(num_blocks=2048)
        nhb, n_blocks = 1024, 512
    else:
        nhb = host_pool_blocks(per_block, 131072, args.host_pool_gib)
        n_blocks = min(8192, nhb)
    w = W.make_swap(s, nhb, n_blocks, seed=1004)
    kv = cache_view(s)
    out = {}
    t0 = time.perf_counter()
    pool = HostPool(nhb, s.num_layers, s.chunk_bytes)
    pin_s = time.perf_counter() - t0
    try:
        L = _lib.lib()
        nbytes = w.bytes_per_direction()
        # DMA baseline: one contiguous pinned copy each way (1 GiB), best of 5
        gib = 1 << 30
        dflat = kv.view(-1).view(torch.uint8)
        peaks = {}
        for name, dst, src in (("h2d", dflat.data_ptr(), pool.host_ptr), ("d2h", pool.host_ptr, dflat.data_ptr())):
            best = None
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                _lib.check(L.lms_memcpy_async(dst, src, min(gib, pool.nbytes), stream.cuda_stream))
                e1.record(stream)
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1)
                best = t if best is None else min(best, t)
            peaks[name] = min(gib, pool.nbytes) / (best * 1e-3) / 1e9
        out_pairs = torch.from_numpy(w.out_pairs).to(dev)
        in_pairs = torch.from_numpy(w.in_pairs).to(dev)
        reps = 2

        def rate(fn):
            return nbytes / (timed(comm, stream, fn, reps, 1, sampler) / reps * 1e-3) / 1e9

        gbs_out = rate(lambda i: cache_ops.swap_blocks(kv, pool, out_pairs, "out"))
        gbs_in = rate(lambda i: cache_ops.swap_blocks(kv, pool, in_pairs, "in"))
        # round trip is bit-exact: what came back equals what went out
        back = {int(h): int(g) for g, h in w.out_pairs}
        src_idx = torch.tensor([back[int(h)] for h in w.in_pairs[:, 0]], device=dev)
        dst_idx = torch.from_numpy(w.in_pairs[:, 1].copy()).to(dev)
        flat = kv.view(s.num_layers, s.num_blocks, -1).view(torch.int16)

        def round_trip_ok():
            return all(bool(torch.equal(flat[l].index_select(0, src_idx), flat[l].index_select(0, dst_idx)))
                       for l in range(0, s.num_layers, 8))

        ok = round_trip_ok()

        def entry(gbs, peak):
            return {"ms": nbytes / gbs / 1e6, "bytes": nbytes, "GB/s": gbs,
                    "pcie_peak_GB/s_measured_memcpy": peak, "frac_of_pcie_peak": gbs / peak,
                    "frac_of_nominal_gen5_x16_64": gbs / NOMINAL["pcie_gen5_x16_GB/s"]}

        out["swap_out"] = entry(gbs_out, peaks["d2h"])
        out["swap_in"] = dict(entry(gbs_in, peaks["h2d"]), round_trip_bit_exact=ok)
        # Design B: gather into a device staging ring, one DMA transfer per host block (or per
        # run of adjacent host blocks), scatter on the way back.  Two placements of the host
        # blocks: scattered over the pool (the specified workload) and allocated as one run
        # (what a write-through of freshly reserved blocks looks like).
        staging = torch.empty((64 if args.small else 256) << 20, dtype=torch.uint8, device=dev)
        run_out = np.stack([w.out_pairs[:, 0], np.arange(n_blocks, dtype=np.int64)], axis=1)
        run_in = np.stack([np.arange(n_blocks, dtype=np.int64), w.in_pairs[:, 1]], axis=1)
        flat.view(-1)[: 1 << 26].random_()            # fresh payload so the re-check means something
        staged = {}
        for label, po, pi in (("host_blocks_scattered", w.out_pairs, w.in_pairs),
                              ("host_blocks_in_one_run", run_out, run_in)):
            go = rate(lambda i: cache_ops.swap_blocks(kv, pool, po, "out", engine="staged", staging=staging))
            gi = rate(lambda i: cache_ops.swap_blocks(kv, pool, pi, "in", engine="staged", staging=staging))
            staged[label] = {"out_GB/s": go, "in_GB/s": gi, "out_frac_of_pcie_peak": go / peaks["d2h"],
                             "in_frac_of_pcie_peak": gi / peaks["h2d"]}
        # the scattered case went last-but-one; redo its round trip for the bit-exact check
        cache_ops.swap_blocks(kv, pool, w.out_pairs, "out", engine="staged", staging=staging)
        cache_ops.swap_blocks(kv, pool, w.in_pairs, "in", engine="staged", staging=staging)
        torch.cuda.synchronize()
        staged["round_trip_bit_exact"] = round_trip_ok()
        staged["staging_MiB"] = staging.numel() >> 20
        out["swap_staged_dma"] = staged
        del staging
        best_out = max(gbs_out, staged["host_blocks_scattered"]["out_GB/s"])
        best_in = max(gbs_in, staged["host_blocks_scattered"]["in_GB/s"])
        out["swap_best_engine"] = {
            "scattered_host_blocks": {"out_GB/s": best_out, "in_GB/s": best_in,
                                      "out_frac_of_pcie_peak": best_out / peaks["d2h"],
                                      "in_frac_of_pcie_peak": best_in / peaks["h2d"]},
            "host_blocks_in_one_run": staged["host_blocks_in_one_run"]}
        # layer-pipelined form: one launch per layer, each gated on / signalling a per-layer
        # event, the way the KV worker and the model hand layers to each other
        from lmserve_b200.kv_worker import KVWorker
        worker = KVWorker.__new__(KVWorker)
        worker.gpu_kv_caches, worker.device, worker.host_pool = kv, dev, pool
        worker.num_layers = s.num_layers
        worker.model_queue = worker.kv_queue = None
        post = [torch.cuda.Event() for _ in range(s.num_layers)]
        for e in post:
            e.record(stream)
        pre = [torch.cuda.Event() for _ in range(s.num_layers)]
        per_layer = {"launches": s.num_layers}
        for engine in ("kernel", "dma"):
            worker.swap_engine = engine
            ms_lo = timed(comm, stream, lambda i: worker._swap([w.out_pairs], "out", stream, None, post, 1), 1, 1, sampler)
            ms_li = timed(comm, stream, lambda i: worker._swap([w.in_pairs], "in", stream, pre, None, 1), 1, 1, sampler)
            per_layer[engine] = {"out_GB/s": nbytes / (ms_lo * 1e-3) / 1e9, "in_GB/s": nbytes / (ms_li * 1e-3) / 1e9}
        out["swap_per_layer_launches"] = per_layer
        # the copy-engine form (no kernel, no SM): one strided DMA per block
        ms_do = timed(comm, stream, lambda i: cache_ops.swap_blocks(kv, pool, w.out_pairs, "out", engine="dma"), reps, 1, sampler) / reps
        ms_di = timed(comm, stream, lambda i: cache_ops.swap_blocks(kv, pool, w.in_pairs, "in", engine="dma"), reps, 1, sampler) / reps
        out["swap_copy_engine"] = {"out_GB/s": nbytes / (ms_do * 1e-3) / 1e9, "in_GB/s": nbytes / (ms_di * 1e-3) / 1e9,
                                   "dma_copies_per_swap": n_blocks}
        # what a concurrent swap-out costs a stream of dense GEMMs (the forward pass it overlaps)
        if not args.small:
            a = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
            b = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
            copy_stream = torch.cuda.Stream()

            # the layer handshake end to end: a stand-in forward pass (3 GEMMs per layer) whose
            # layer l waits for pre_events[l], against a swap-in issued layer by layer on the
            # worker's stream (kv_worker.py:249-270 / model_worker.py:232-276 in LMServe)
            quarter = w.in_pairs[: max(1, n_blocks // 4)]
            worker.swap_engine = "kernel"

            def forward(events):
                for l in range(s.num_layers):
                    if events is not None:
                        stream.wait_event(events[l])
                    for _ in range(3):
                        torch.matmul(a, b)

            def pipelined(i):
                copy_stream.wait_stream(stream)
                worker._swap([quarter], "in", copy_stream, pre, None, 1)
                forward(pre)

            def serial(i):
                worker._swap([quarter], "in", stream, pre, None, 1)
                forward(None)

            forward(None)
            ms_f = timed(comm, stream, lambda i: forward(None), 1, 1, sampler)
            ms_s = timed(comm, stream, lambda i: worker._swap([quarter], "in", stream, pre, None, 1), 1, 1, sampler)
            ms_ser = timed(comm, stream, serial, 1, 1, sampler)
            ms_p = timed(comm, stream, pipelined, 1, 1, sampler)
            out["swap_in_pipelined_with_forward"] = {
                "forward_alone_ms": ms_f, "swap_in_alone_ms": ms_s, "one_after_the_other_ms": ms_ser,
                "layer_pipelined_ms": ms_p, "lower_bound_ms": max(ms_f, ms_s),
                "hidden_fraction_of_the_shorter": (ms_f + ms_s - ms_p) / min(ms_f, ms_s),
                "note": f"{len(quarter)} blocks x {s.num_layers} layers x 64 KiB swapped in, one launch and "
                        "one event per layer; forward = 3 bf16 GEMMs of 8192^3 per layer gated on that event"}

            staging2 = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

            def gemms(engine):
                """150 GEMMs on the main thread and stream; the swap is issued at the same
                moment from a second host thread on its own stream (as a KV worker would)."""
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start = threading.Barrier(2)

                def swap():
                    torch.cuda.set_device(dev)
                    start.wait()
                    with torch.cuda.stream(copy_stream):
                        cache_ops.swap_blocks(kv, pool, out_pairs if engine == "kernel" else w.out_pairs,
                                              "out", engine=engine,
                                              staging=staging2 if engine == "staged" else None)

                t = threading.Thread(target=swap if engine else start.wait)
                t.start()
                start.wait()
                e0.record(stream)
                for _ in range(150):
                    torch.matmul(a, b)
                e1.record(stream)
                t.join()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1)

            gemms(None)
            alone = gemms(None)
            out["swap_out_overlapping_gemms"] = {
                "gemm_ms_alone": alone,
                "gemm_slowdown_with_kernel_swap": gemms("kernel") / alone,
                "gemm_slowdown_with_copy_engine_swap": gemms("dma") / alone,
                "gemm_slowdown_with_staged_swap": gemms("staged") / alone,
                "note": "150 bf16 GEMMs of 8192^3 on one stream; a 16 GiB swap-out issued at the "
                        "same time from a second host thread on another stream"}
            del a, b, staging2
        out["swap_pool"] = {"host_blocks": nhb, "host_pool_GiB": pool.nbytes / (1 << 30),
                            "specified_host_blocks": 131072,
                            "rule": "131072 blocks halved until the pool fits --host-pool-gib and half of "
                                    "MemAvailable (the specified 256 GiB exceed the box's RAM)",
                            "moved_blocks": n_blocks, "pin_seconds": pin_s, "pcie_link": link}
    finally:
        pool.close()
    return out


def flashinfer_is_usable(budget_s: float = 240.0):
    """flashinfer compiles its append kernel on first use; do that in a child process with a
    time limit so that a slow or broken JIT toolchain costs the bench a bounded time."""
    code = ("import torch, flashinfer\n"
            "d='cuda'\n"
            "k=torch.zeros(2,2,64,device=d,dtype=torch.bfloat16)\n"
            "c=torch.zeros(4,2,16,2,64,device=d,dtype=torch.bfloat16)\n"
            "i=torch.arange(2,dtype=torch.int32,device=d)\n"
            "flashinfer.append_paged_kv_cache(k,k,i,i,c,i,torch.arange(3,dtype=torch.int32,device=d),"
            "torch.ones(2,dtype=torch.int32,device=d))\n"
            "torch.cuda.synchronize()\n")
    try:
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=budget_s)
        return r.returncode == 0, (r.stderr.strip().splitlines() or [""])[-1][:200]
    except subprocess.TimeoutExpired:
        return False, f"flashinfer's first call did not finish within {budget_s:.0f} s"


def bench_vs_flashinfer(comm, stream, cache_view, dev, args, sampler):
    """The decode step's 32 per-layer cache writes through flashinfer.append_paged_kv_cache (the
    call LMServe makes, models/layers/attention.py:76-85) and through this library, eager and
    replayed from CUDA graphs, on the same rotating inputs."""
    ok, why = flashinfer_is_usable()
    if not ok:
        return {"vs_flashinfer_per_layer_decode_write": {"skipped": why}}
    import flashinfer
    from lmserve_b200.ops import cache_ops
    s = W.SHAPES["llama31_8b"]
    kv = cache_view(s)
    Lyr, T = s.num_layers, 256
    sets = []
    for i in range(ROTATE):
        w = W.config2(seed=4002 + 17 * i)
        indptr, indices = W.paged_metadata(w.tables.tables)
        sets.append(dict(
            key=torch.randn(Lyr, T, s.num_kv_heads, s.head_dim, device=dev, dtype=torch.bfloat16),
            value=torch.randn(Lyr, T, s.num_kv_heads, s.head_dim, device=dev, dtype=torch.bfloat16),
            slots=torch.from_numpy(w.slot_mapping).to(dev),
            batch=torch.arange(T, dtype=torch.int32, device=dev),
            pos=torch.from_numpy(w.context_lens.astype(np.int32)).to(dev),
            indptr=torch.from_numpy(indptr).to(dev), indices=torch.from_numpy(indices).to(dev),
            last=torch.from_numpy(((w.context_lens % 16) + 1).astype(np.int32)).to(dev)))
    plans = [[cache_ops.WritePlan(d["key"][l], d["value"][l], kv[l], d["slots"]) for l in range(Lyr)]
             for d in sets]
    paged_plans = [[cache_ops.PagedWritePlan(d["key"][l], d["value"][l], d["batch"], d["pos"], kv[l],
                                             d["indices"], d["indptr"]) for l in range(Lyr)] for d in sets]

    def fi(j):
        d = sets[j]
        for l in range(Lyr):
            flashinfer.append_paged_kv_cache(d["key"][l], d["value"][l], d["batch"], d["pos"], kv[l],
                                             d["indices"], d["indptr"], d["last"])

    def ours_paged(j):
        d = sets[j]
        for l in range(Lyr):
            cache_ops.append_paged_kv_cache(d["key"][l], d["value"][l], d["batch"], d["pos"], kv[l],
                                            d["indices"], d["indptr"], d["last"])

    def ours_paged_plan(j):
        sp = torch.cuda.current_stream().cuda_stream
        for p in paged_plans[j]:
            p.run(sp)

    def ours_plan(j):
        sp = torch.cuda.current_stream().cuda_stream
        for p in plans[j]:
            p.run(sp)

    fi(0)
    torch.cuda.synchronize()
    d0 = sets[0]
    blk, ent = d0["slots"] // 16, d0["slots"] % 16
    same = bool(torch.equal(kv[:, blk, 0, ent].view(torch.int16), d0["key"].view(torch.int16)))
    kv[:, blk] = 0
    ours_paged(0)
    torch.cuda.synchronize()
    same_ours = bool(torch.equal(kv[:, blk, 0, ent].view(torch.int16), d0["key"].view(torch.int16))
                     and torch.equal(kv[:, blk, 1, ent].view(torch.int16), d0["value"].view(torch.int16)))
    out = {"flashinfer_version": getattr(flashinfer, "__version__", "?"), "flashinfer_result_matches": same,
           "drop_in_result_matches": same_ours}
    for name, fn in (("flashinfer", fi), ("ours_flashinfer_signature", ours_paged),
                     ("ours_paged_write_plan", ours_paged_plan), ("ours_write_plan", ours_plan)):
        fn(0)
        ms_e = min(timed(comm, stream, lambda i: fn(i % ROTATE), 30, 3, sampler) for _ in range(3)) / 30
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        for j in range(ROTATE):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn(j)
            graphs.append(g)
        stream.wait_stream(side)
        torch.cuda.synchronize()
        ms_g = statistics.median(timed(comm, stream, lambda i: graphs[i % ROTATE].replay(), 100, 5, sampler)
                                 for _ in range(5)) / 100
        out[name] = {"eager_us_per_layer": ms_e * 1e3 / Lyr, "graph_us_per_layer": ms_g * 1e3 / Lyr}
    # The cache path of a whole decode step as a model worker runs it, host wall time from the
    # request objects to all 32 layers' rows in the cache (synchronised at the end): LMServe's
    # way (its index preparation + 32 flashinfer appends) against ModelStepCache (one packed
    # upload + one index kernel + 32 cached-plan appends).  K / V are ready on the device.
    import copy
    from lmserve_b200.model_step import ModelStepCache
    step_cache = ModelStepCache(kv, max_batch=256, max_tokens=4096, max_blocks=131072)
    reqs = [W.make_step_requests(s.num_blocks, 16, seed=8100 + i, num_decode=256, ctx_lo=128, ctx_hi=4096,
                                 num_prefill=0, chunk_tokens=0, max_offset=0) for i in range(4)]
    k0, v0 = sets[0]["key"], sets[0]["value"]

    def step_reference(r):
        ref = reference_way(r, dev, flashinfer)
        for l in range(Lyr):
            flashinfer.append_paged_kv_cache(k0[l], v0[l], ref[6], ref[7], kv[l], ref[4], ref[3], ref[5])

    def step_ours(r):
        _, params = step_cache.begin_step(r)
        for l in range(Lyr):
            step_cache.write_layer(l, k0[l], v0[l], params)

    whole = {}
    for label, fn in (("lmserve_way_us", step_reference), ("this_library_us", step_ours)):
        times = []
        for i in range(13):
            r = copy.copy(reqs[i % 4])
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            fn(r)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
        whole[label] = float(np.median(times[3:])) * 1e6
    whole["speedup"] = whole["lmserve_way_us"] / whole["this_library_us"]
    whole["note"] = ("host wall time of one decode step's cache path, 256 requests x 32 layers: index "
                     "preparation from the request objects + the 32 per-layer cache writes, eager")
    out["decode_step_cache_path"] = whole
    f = out["flashinfer"]
    d = out["ours_flashinfer_signature"]
    out["drop_in_vs_flashinfer"] = {"eager_speedup": f["eager_us_per_layer"] / d["eager_us_per_layer"],
                                    "graph_speedup": f["graph_us_per_layer"] / d["graph_us_per_layer"]}
    return {"vs_flashinfer_per_layer_decode_write": out}


def bench_write_scaling(comm, stream, cache_view, dev, peak_gbs, args, sampler):
    """Decode-step write against the size of the step: the all-layer launch for 128 ... 2048
    tokens of the Llama-3.1-70B TP8 shard (256-byte rows, 80 layers) and of Llama-3.1-8B
    (2 KiB rows, 32 layers), steps replayed back to back from CUDA graphs.  Separates the fixed
    cost of a launch from the streaming rate.  Not part of --ops all."""
    from lmserve_b200.ops import cache_ops
    out = {}
    GS = 40
    for name, shape_key, tokens, ctx in (("tp8_256B_rows_80_layers", "llama31_70b_tp8", (128, 256, 512, 1024, 2048), (512, 1024)),
                                         ("8b_2KiB_rows_32_layers", "llama31_8b", (64, 128, 256, 512), (128, 1024))):
        s = W.SHAPES[shape_key]
        kv = cache_view(s)
        rows = []
        for T in tokens:
            wl = [W.make_decode_write(s, T, ctx[0], ctx[1], seed=7005 + 31 * i) for i in range(ROTATE)]
            keys = [torch.randn(s.num_layers, T, s.num_kv_heads, s.head_dim, device=dev, dtype=torch.bfloat16)
                    for _ in range(ROTATE)]
            vals = [torch.randn_like(k) for k in keys]
            slots = [torch.from_numpy(w.slot_mapping).to(dev) for w in wl]
            plans = [cache_ops.WritePlan(keys[j], vals[j], kv, slots[j]) for j in range(ROTATE)]
            g = graph_of(stream, lambda cs: [plans[j % ROTATE].run(cs) for j in range(GS)])
            ms = statistics.median(timed(comm, stream, lambda i: g.replay(), 10, 3, sampler) for _ in range(7)) / (10 * GS)
            b = wl[0].algorithmic_bytes()
            rows.append({"tokens": T, "MiB": b / 2**20, "us_per_step": ms * 1e3,
                         "GB/s": b / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": b / (ms * 1e-3) / 1e9 / peak_gbs})
            del plans, keys, vals, g
        # least-squares line us = fixed + bytes / rate over the sizes measured
        x = np.array([r["MiB"] * 2**20 for r in rows])
        y = np.array([r["us_per_step"] for r in rows])
        slope, fixed = np.polyfit(x, y, 1)
        out[name] = {"steps": rows, "fit_fixed_us_per_launch": float(fixed),
                     "fit_streaming_GB/s": float(1.0 / slope / 1e3)}
    return {"decode_write_vs_step_size": out}


def bench_tp8_decode(comm, stream, cache_view, dev, rank, world, peak_gbs, args, sampler, local=0):
    """Llama-3.1-70B under TP=8: one KV head per GPU (256-byte rows), 80 layers, batch 512."""
    from lmserve_b200.ops import cache_ops
    s = W.SHAPES["llama31_70b_tp8"]
    wl = [W.config5_decode(rank=rank, seed=1005 + 31 * i) for i in range(ROTATE)]
    if args.small:   # profiling case: the same slots renumbered into a 4096-block (2.5 GiB) pool
        s = s.scaled(num_blocks=4096)
        for i, w in enumerate(wl):
            w.slot_mapping = renumber_blocks(w.slot_mapping, s.block_size, s.num_blocks, seed=77 + i)
    kv = cache_view(s)
    T = wl[0].num_tokens
    keys = [torch.randn(s.num_layers, T, 1, s.head_dim, device=dev, dtype=torch.bfloat16) for _ in range(ROTATE)]
    vals = [torch.randn_like(k) for k in keys]
    slots = [torch.from_numpy(w.slot_mapping).to(dev) for w in wl]
    plans = [cache_ops.WritePlan(keys[j], vals[j], kv, slots[j]) for j in range(ROTATE)]
    sp = stream.cuda_stream
    n_e = args.steps if args.small else max(args.steps, 200)
    ms_eager = timed(comm, stream, lambda i: plans[i % ROTATE].run(sp), n_e, 3 if args.small else 10, sampler) / n_e
    GS = 40 if args.small else 240          # about 2 ms of device work per replay
    g = graph_of(stream, lambda cs: [plans[j % ROTATE].run(cs) for j in range(GS)])
    if args.small:
        ms = timed(comm, stream, lambda i: g.replay(), 1, 1, sampler) / GS
        stats, per_rank = None, None
    else:
        ms_round, stats, per_rank, _ = measure_rounds(comm, stream, g.replay, GS, 1, local, min_region_ms=80.0)
        ms = ms_round / GS
    b = wl[0].algorithmic_bytes()
    gbs = b / (ms * 1e-3) / 1e9
    return {"tp8_decode_write": {"us_per_step": ms * 1e3, "us_per_step_eager_stream": ms_eager * 1e3,
                                 "bytes_per_gpu": b, "GB/s_per_gpu": gbs, "GB/s_all_gpus": world * gbs,
                                 "frac_of_hbm_peak": gbs / peak_gbs,
                                 "frac_of_nominal_8000": gbs / NOMINAL["hbm_GB/s"],
                                 "timing": stats, "us_per_step_by_rank": per_rank}}


def bench_transfer_local(comm, stream, cache_view, dev, args, sampler):
    """The prefill->decode push between two GPUs of ONE process (peer access instead of CUDA
    IPC): the case a single-process profiler can capture.  Llama-3.1-70B TP8 shard geometry;
    4096 blocks x 80 layers x 8 KiB (512 blocks in the small profiling case)."""
    from lmserve_b200.ops import cache_ops
    s = W.SHAPES["llama31_70b_tp8"]
    n_seqs = 4 if args.small else 32
    if args.small:
        s = s.scaled(num_blocks=4096)
    src = cache_view(s)
    dshape = s.scaled(num_blocks=8192)
    dst = torch.empty(dshape.cache_shape, dtype=torch.bfloat16, device="cuda:1")
    tr = W.make_transfer(s, n_seqs, 2048, seed=1105, dst_num_blocks=dshape.num_blocks)
    pairs = torch.from_numpy(tr.pairs).to(dev)
    reps = 3
    ms = timed(comm, stream, lambda i: cache_ops.transfer_blocks(src, dst, pairs), reps, 2, sampler) / reps
    torch.cuda.synchronize("cuda:1")
    # the same blocks pulled: the kernel runs on cuda:1 and loads from cuda:0
    with torch.cuda.device(1):
        pairs1 = pairs.to("cuda:1")
        s1 = torch.cuda.current_stream()
        for _ in range(2):
            cache_ops.transfer_blocks(src, dst, pairs1, pull=True)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s1)
        for _ in range(reps):
            cache_ops.transfer_blocks(src, dst, pairs1, pull=True)
        e1.record(s1)
        torch.cuda.synchronize()
        ms_pull = e0.elapsed_time(e1) / reps
    return {"transfer_local": {"ms": ms, "bytes": tr.bytes(), "GB/s": tr.bytes() / (ms * 1e-3) / 1e9,
                               "pull_ms": ms_pull, "pull_GB/s": tr.bytes() / (ms_pull * 1e-3) / 1e9}}


def bench_transfer(comm, stream, cache_view, dev, rank, world, sampler):
    """Prefill GPU g pushes 32 x 2048-token sequences (4096 blocks x 80 layers x 8 KiB = 2.5 GiB)
    into random free blocks of decode GPU g + N/2 over NVLink; then the decode GPU pulls the
    same blocks.  Before anything is timed the bytes are checked: the prefill rank fills its
    source blocks from a seed both ranks know, pushes once, and the decode rank compares every
    destination block of 8 sampled layers bit for bit with the regenerated source, plus a guard
    block that must stay untouched; the same after a pull into zeroed blocks
    (semantics: block i of the local list lands in the i-th reserved remote block, all layers —
    kv_worker.py:386-400 in LMServe)."""
    from lmserve_b200 import _lib
    from lmserve_b200.kv_worker import KVWorker, CacheDescriptor, PeerCache
    from lmserve_b200.ops import cache_ops
    s = W.SHAPES["llama31_70b_tp8"]
    kv = cache_view(s)
    role, peer = W.transfer_peer(rank, world)
    worker = KVWorker(f"kv{rank}", kv)
    descs = comm.gather_objects(worker.get_descriptors([]))
    L = _lib.lib()
    prefill_rank = rank if role == "prefill" else peer
    w = W.config5_transfer(rank=prefill_rank)
    nbytes = w.bytes()
    flat = kv.view(s.num_layers, s.num_blocks, -1).view(torch.int16)
    words = flat.shape[2]
    src_blocks = torch.from_numpy(w.pairs[:, 0].copy()).to(dev)
    dst_blocks = torch.from_numpy(w.pairs[:, 1].copy()).to(dev)
    sampled = sorted(np.random.default_rng(5000 + prefill_rank).choice(s.num_layers, 8, replace=False).tolist())

    def payload(layer):
        g = torch.Generator(device=dev)
        g.manual_seed(900_000 + 4099 * prefill_rank + layer)
        return torch.randint(-32768, 32767, (len(w.pairs), words), dtype=torch.int16, device=dev, generator=g)

    guard = int(np.setdiff1d(np.arange(s.num_blocks), w.pairs[:, 1])[17])
    if role == "prefill":
        for l in range(s.num_layers):
            flat[l, src_blocks] = payload(l)
        pc = PeerCache(CacheDescriptor.deserialize(descs[peer]))
        pairs = torch.from_numpy(w.pairs).to(dev)
        fn = lambda i: cache_ops.transfer_blocks(kv, pc, pairs)
        # DMA baseline: one contiguous 1 GiB peer copy
        gib = 1 << 30
        def dma(i):
            _lib.check(L.lms_memcpy_async(pc.device_ptr, kv.data_ptr(), gib, stream.cuda_stream))
        pull = lambda i: None
    else:
        flat[:, guard] = 0x5A5A
        for l in sampled:
            flat[l, dst_blocks] = 0
        src = PeerCache(CacheDescriptor.deserialize(descs[peer]))
        pairs = torch.from_numpy(w.pairs).to(dev)
        fn = lambda i: None
        dma = lambda i: None
        pull = lambda i: cache_ops.transfer_blocks(src, kv, pairs, pull=True)

    def arrived():
        if role != "decode":
            return True
        ok = all(bool(torch.equal(flat[l, dst_blocks], payload(l))) for l in sampled)
        return ok and bool((flat[:, guard] == 0x5A5A).all())

    torch.cuda.synchronize()
    comm.barrier()
    fn(0)                                   # one push
    torch.cuda.synchronize()
    comm.barrier()
    push_ok = arrived()
    if role == "decode":
        for l in sampled:
            flat[l, dst_blocks] = 0
    torch.cuda.synchronize()
    comm.barrier()
    pull(0)                                 # one pull
    torch.cuda.synchronize()
    comm.barrier()
    pull_ok = arrived()
    flags = comm.gather_objects((role, push_ok, pull_ok))
    bit_exact = all(p and q for _, p, q in flags)

    reps = 3
    ms = timed(comm, stream, fn, reps, 2, sampler) / reps
    # the contiguous peer copy overwrites the head of the decode cache: it runs last
    ms_pull = timed(comm, stream, pull, reps, 2, sampler) / reps
    ms_dma = timed(comm, stream, dma, reps, 2, sampler) / reps
    if role == "prefill":
        pc.close()
    else:
        src.close()
    pairs_n = world // 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    dma_gbs = (1 << 30) / (ms_dma * 1e-3) / 1e9
    pull_gbs = nbytes / (ms_pull * 1e-3) / 1e9
    return {"prefill_to_decode_transfer": {
        "transfer_bit_exact": bit_exact,
        "checked": f"every destination block of layers {sampled} and one guard block on each decode rank, "
                   "after one push and again after one pull into zeroed blocks",
        "pull_ms": ms_pull, "pull_GB/s_per_pair": pull_gbs,
        "ms": ms, "bytes_per_pair": nbytes, "pairs": pairs_n, "GB/s_per_pair": gbs,
        "GB/s_all_pairs": gbs * pairs_n, "nvlink_peer_copy_GB/s_measured_memcpy": dma_gbs,
        "frac_of_measured_peer_copy": gbs / dma_gbs, "frac_of_nominal_900": gbs / 900.0,
        "pull_frac_of_measured_peer_copy": pull_gbs / dma_gbs, "pull_frac_of_nominal_900": pull_gbs / 900.0}}


# ----------------------------------------------------------------------------- host baseline
def compact_decode_cases(n_sets: int):
    """The headline step's `n_sets` rotating input sets with the blocks they touch renumbered
    densely, so that the host cache pool only holds touched blocks (the untouched rest of the
    65 536-block pool plays no part in the step and would only cost host memory)."""
    ws = [W.config2(seed=1002 + 17 * i) for i in range(n_sets)]
    s = ws[0].shape
    all_blocks = np.unique(np.concatenate([w.slot_mapping // s.block_size for w in ws]))
    index = {int(b): i for i, b in enumerate(all_blocks)}
    slots = [np.array([index[int(b)] for b in w.slot_mapping // s.block_size], dtype=np.int64) * s.block_size
             + w.slot_mapping % s.block_size for w in ws]
    return ws[0], s.scaled(num_blocks=len(all_blocks)), slots


def cpu_step_factory(threads: int, n_sets: int = ROTATE):
    from oracle import torch_ref
    torch.set_num_threads(threads)
    w, s, slots = compact_decode_cases(n_sets)
    T = w.num_tokens
    kv = torch.zeros(s.cache_shape, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(11)
    keys = [torch.randn(s.num_layers, T, s.num_kv_heads, s.head_dim, generator=g).to(torch.bfloat16)
            for _ in range(n_sets)]
    vals = [torch.randn(s.num_layers, T, s.num_kv_heads, s.head_dim, generator=g).to(torch.bfloat16)
            for _ in range(n_sets)]
    sl = [torch.from_numpy(x) for x in slots]

    def step(i=0):
        j = i % n_sets
        torch_ref.reshape_and_cache_layers(keys[j], vals[j], kv, sl[j])
    return step, w.algorithmic_bytes(), s


def cpu_sample_text(n_steps: int, s) -> str:
    return (f"{n_steps} full decode steps (32 layers x 256 tokens, 64 MiB each, {ROTATE} rotating input sets) as "
            f"torch index_copy_ on bf16 CPU tensors; host cache pool holds the {s.num_blocks} touched blocks")


def cpu_baseline(bounded_seconds: float):
    threads = os.cpu_count() or 1
    step, nbytes, s = cpu_step_factory(threads)
    for i in range(ROTATE):
        step(i)
    times = []
    t_end = time.perf_counter() + bounded_seconds
    while time.perf_counter() < t_end and len(times) < 2000:
        t0 = time.perf_counter()
        step(len(times))
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return {"value": round(nbytes / med / 1e9, 3), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": cpu_sample_text(len(times), s), "ms_per_step": round(med * 1e3, 4)}


def cpu_single_thread(bounded_seconds: float):
    step, nbytes, s = cpu_step_factory(1, n_sets=2)
    step(0)
    step(1)
    times = []
    t_end = time.perf_counter() + bounded_seconds
    while time.perf_counter() < t_end and len(times) < 200:
        t0 = time.perf_counter()
        step(len(times))
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    torch.set_num_threads(os.cpu_count() or 1)
    return {"value": round(nbytes / med / 1e9, 3), "unit": UNIT, "cores": 1,
            "sample": f"{len(times)} of the same steps with torch.set_num_threads(1)",
            "ms_per_step": round(med * 1e3, 4)}


def cpu_other_ops(threads: int, seconds_each: float = 4.0):
    """Bounded samples of the other cache ops as torch index ops on the host cores: copy-on-write
    (index_select + index_copy_ on the block axis) and the swap as a host-to-host gather between
    a layer-major and a block-major tensor (the PCIe hop has no CPU analogue)."""
    from oracle import torch_ref
    torch.set_num_threads(threads)
    out = {}
    w = W.config3()
    s = w.shape.scaled(num_layers=2)          # 2 of 28 layers, all 4096 pairs: 256 MiB written
    blocks, inv = np.unique(w.pairs.reshape(-1), return_inverse=True)
    pairs = torch.from_numpy(inv.reshape(-1, 2).astype(np.int64))
    kv = torch.zeros(s.num_layers, len(blocks), s.chunk_bytes // 2, dtype=torch.bfloat16)
    nbytes = (len(pairs) + len(np.unique(w.pairs[:, 0]))) * s.num_layers * s.chunk_bytes

    def timed_cpu(fn):
        fn()
        ts, end = [], time.perf_counter() + seconds_each
        while time.perf_counter() < end and len(ts) < 200:
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return statistics.median(ts), len(ts)

    med, n = timed_cpu(lambda: torch_ref.copy_blocks(kv, pairs))
    out["copy_blocks_cow"] = {"GB/s": round(nbytes / med / 1e9, 3), "ms": round(med * 1e3, 3),
                              "sample": f"{n} runs of 4096 pairs x 2 layers x 32 KiB (2 of the 28 layers)"}
    del kv
    s4 = W.SHAPES["llama31_8b_swap"].scaled(num_layers=4, num_blocks=2048)
    sw = W.make_swap(s4, 2048, 1024, seed=1004)   # 1024 blocks x 4 layers x 64 KiB = 256 MiB
    gpu = torch.zeros(s4.num_layers, s4.num_blocks, s4.chunk_bytes // 2, dtype=torch.bfloat16)
    host = torch.zeros(2048, s4.num_layers, s4.chunk_bytes // 2, dtype=torch.bfloat16)
    nb = len(sw.out_pairs) * s4.num_layers * s4.chunk_bytes
    med, n = timed_cpu(lambda: torch_ref.swap_out(gpu, host, sw.out_pairs))
    out["swap_out_host_gather"] = {"GB/s": round(nb / med / 1e9, 3), "ms": round(med * 1e3, 3),
                                   "sample": f"{n} runs of 1024 blocks x 4 layers x 64 KiB, host to host"}
    return out


def run_reference(args):
    """The reference arm: the reference semantics of the same step as torch index ops on all
    host cores (the oracle port; LMServe's own implementation of this path is GPU code).  Same
    protocol as the GPU arm: warm-up, then rounds of exactly K steps, median round; the number
    of rounds is bounded so that the run ends within about twenty seconds of CPU work."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    step, nbytes, s = cpu_step_factory(threads)
    warm = max(args.warmup, 3)
    t0 = time.perf_counter()
    for i in range(warm):
        step(i)
    est_step = (time.perf_counter() - t0) / warm
    steps = args.steps
    rounds = int(max(3, min(50, 20.0 / max(est_step * steps, 1e-6))))
    times = []
    n = 0
    for _ in range(rounds):
        t0 = time.perf_counter()
        for _ in range(steps):
            step(n)
            n += 1
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times) / steps
    value = nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(dt * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": headline_config(),
        "run": {"timing": {"rounds": rounds, "steps_per_round": steps,
                           "ms_per_step_median": round(dt * 1e3, 4),
                           "ms_per_step_best_round": round(min(times) / steps * 1e3, 4),
                           "ms_per_step_worst_round": round(max(times) / steps * 1e3, 4)},
                "note": ("one CPU process on rank 0 (the other ranks exit); its value is the N = 1 CPU "
                         "number and does not scale with --gpus") if args.gpus > 1 else
                        "one CPU process, every host core"},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": cpu_sample_text(rounds * steps, s)},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--ops", default="all",
                    help="comma list of extra workloads: all, none, prefill_cow, swap, rope, index_prep, tp8, "
                         "flashinfer (the per-layer call against flashinfer.append_paged_kv_cache), "
                         "transfer (multi-rank), transfer_local (two GPUs in one process; not in 'all'), "
                         "write_scaling (decode write against step size; not in 'all')")
    ap.add_argument("--host-pool-gib", type=float, default=64.0,
                    help="cap of the pinned host pool of the swap workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: the same kernels and per-step inputs on a 4 GiB cache pool "
                         "(touched blocks renumbered into 2048 blocks) so that a multi-pass ncu "
                         "capture stays small; numbers printed in this mode are not bench values")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
