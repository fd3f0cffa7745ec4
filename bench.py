#!/usr/bin/env python3
"""Benchmark of the Conv2D hot path: forward + dX + dW, images/s.

  python bench.py [--gpus N] [--steps K] [--warmup W]            this library on N B200s
  python bench.py --impl reference [--gpus N] [--steps K] ...    the reference's CPU algorithm on the host cores

Workload (default): the batched low-channel stem, x [256,3,224,224] ~U(-1,1),
w [64,3,3,3] ~N(0, 2/27), stride 1, padding 1; upstream gradient g = 2y (the
VJP seed of loss = sum(y*y)).  One step = conv2d_fwd, conv2d_bwd(dX),
conv2d_bwd(dW) through the C ABI (+ one NCCL all-reduce of dW when N > 1, the
batch being sharded over the ranks).  Inputs are synthetic and seeded
(katsu_b200/workloads.py); y and g are larger than L2, so every step streams
from HBM.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from katsu_b200 import workloads  # noqa: E402

METRIC = "conv2d_fwd_dx_dw_images_per_s"
UNIT = "images/s"


def measured_peaks():
    """(HBM GB/s, dense bf16 TFLOP/s, which) from the driver-written file, else the pool's fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            peaks = json.load(fh)
        return float(peaks["hbm_gbs"]), float(peaks["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def captured_traffic(workload: str, kernel: str, images: int):
    """DRAM bytes per launch of `kernel`, scaled from the committed ncu capture, or None."""
    path = os.path.join(ROOT, "katsu_b200", "dram_traffic_per_image.json")
    try:
        with open(path) as fh:
            table = json.load(fh)
        return int(table[workload][kernel]) * images
    except (OSError, KeyError, ValueError):
        return None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True):
        self.index, self.proc, self.lines, self.enabled = index, None, [], enabled

    def __enter__(self):
        # One sampler per job (rank 0's GPU): every nvidia-smi process polls through the driver, and
        # eight of them stalled the ranks' kernel launches measurably.
        if not self.enabled:
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_first(self, timeout=3.0):
        """Blocks until nvidia-smi has printed its first line: its start-up (device enumeration,
        driver queries) stalls kernel launches for milliseconds and must not fall into a timed region."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                sm_max.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(sm_max), "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def config_dict(spec_full, world, scaling):
    """The `config` object of the JSON line; both arms (this library, the reference's CPU algorithm)
    print the same one for the same command line."""
    if scaling == "strong":
        images, global_batch = -(-spec_full.n // world), spec_full.n
    else:
        images, global_batch = spec_full.n, spec_full.n * world
    return {"workload": spec_full.name, "x": spec_full.x_shape, "w": spec_full.w_shape, "stride": spec_full.stride,
            "padding": spec_full.pad, "global_batch": global_batch, "images_per_gpu": images,
            "parallelism": f"dp{world}", "l2": "y and g exceed L2 (inputs larger than L2, no flush)",
            "upstream_gradient": "g = 2y"}


def bind_near_gpu(local_rank, world):
    """Pins this rank's host thread (and with it the first-touch placement of the page-locked buffers
    it allocates afterwards) to cores of the NUMA node its GPU hangs off, split among the ranks that
    share the node.  Returns a description for the report; any missing piece of /sys leaves the
    affinity alone."""
    try:
        allowed = sorted(os.sched_getaffinity(0))
        out = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout.split()
        nodes = []
        for bus in out[:world]:
            path = f"/sys/bus/pci/devices/{bus.strip()[4:].lower()}/numa_node"
            with open(path) as fh:
                nodes.append(int(fh.read().strip()))
        node = nodes[local_rank]
        if node < 0:
            return {"numa_node": node, "bound": False}
        cpus = []
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.extend(range(int(lo), int(hi or lo) + 1))
        cpus = [c for c in cpus if c in allowed]
        peers = [r for r, nd in enumerate(nodes) if nd == node]
        share = max(1, len(cpus) // len(peers))
        mine = cpus[peers.index(local_rank) * share:(peers.index(local_rank) + 1) * share]
        if not mine:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, mine)
        return {"numa_node": node, "bound": True, "cores": len(mine)}
    except Exception as exc:  # no NUMA information in this container: run unbound
        return {"bound": False, "why": type(exc).__name__}


# ---------------------------------------------------------------------------
# CPU legs (the only place this file touches oracle/)
# ---------------------------------------------------------------------------
def cpu_step(ref, x, w, spec, threaded: bool):
    """One pass of the reference algorithm: forward, g = 2y, backward_buffers."""
    y = ref.conv2d_forward(x, w, spec.x_shape, spec.w_shape, spec.stride, spec.pad, mt=threaded)
    g = y + y
    dx, dw = ref.conv2d_backward(x, w, g, spec.x_shape, spec.w_shape, spec.stride, spec.pad, mt=threaded)
    return dx, dw


def cpu_baseline(spec, sample_images: int):
    """Single-threaded port of the reference on a bounded sample of the workload."""
    from oracle import katsu_ref as ref

    sample = spec.with_batch(sample_images)
    x, w = workloads.conv_inputs(sample)
    ref.lib().ko_set_num_threads(1)
    t0 = time.perf_counter()
    cpu_step(ref, x, w, sample, threaded=False)
    dt = time.perf_counter() - t0
    return {"value": sample_images / dt, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": f"{sample_images} of {spec.n} images of {spec.name}, one pass, {dt:.1f} s",
            "host_cores_total": os.cpu_count()}


def oracle_dw_samples(spec, x_host, g_host, indices):
    """Checker, outside every timed region: the exact (f64) sums of a few dW elements over this rank's
    images, each visited in the reference's order (crates/katsu-core/src/conv2d.rs:269-292)."""
    from oracle import katsu_ref as ref

    ref.lib().ko_set_num_threads(os.cpu_count() or 1)
    _, dw64 = ref.sample_dw(x_host, g_host, indices, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    return dw64


def run_reference(args):
    """The reference's CPU algorithm (oracle port; the Rust original has no toolchain here)
    on all host threads, on a bounded sample of the same workload."""
    rank, _, world = dist_env()
    if rank != 0:
        return 0
    from oracle import katsu_ref as ref

    spec = workloads.CONV[args.workload]
    if args.batch:
        spec = spec.with_batch(args.batch)
    threads = os.cpu_count() or 1
    ref.lib().ko_set_num_threads(threads)
    sample_images = max(1, min(spec.n, threads))
    sample = spec.with_batch(sample_images)
    x, w = workloads.conv_inputs(sample)
    for _ in range(args.warmup):
        cpu_step(ref, x, w, sample, threaded=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(ref, x, w, sample, threaded=True)
    dt = (time.perf_counter() - t0) / args.steps
    value = sample_images / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(spec, max(1, args.gpus), args.scaling),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"{sample_images} of {spec.n} images per step, OpenMP over images/channels"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class Job:
    """What every leg of one bench process shares: ranks, the torch.distributed group (N > 1), one
    compute context and one context whose stream carries the gradient all-reduce."""

    def __init__(self, args):
        from katsu_b200 import cabi, dp

        self.args = args
        self.rank, self.local_rank, self.world = dist_env()
        if self.world != args.gpus and self.world > 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}")
        self.dist = None
        if self.world > 1:
            import torch
            import torch.distributed as dist

            torch.cuda.set_device(self.local_rank)
            dist.init_process_group(backend="nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        self.ctx = cabi.Context(self.local_rank)
        # The dW all-reduce runs on a second context (stream) of the device so that it overlaps the dX
        # kernel, which does not depend on it; events order the two streams, the host never blocks.
        self.comm_ctx = None
        if self.world > 1:
            self.comm_ctx = cabi.Context(self.local_rank)
            dp.init_comm(self.comm_ctx, self.dist, self.rank, self.world)
            self.dw_ready, self.dw_reduced = self.ctx.event(), self.comm_ctx.event()

    def barrier(self):
        self.ctx.sync()
        if self.dist is not None:
            import torch

            self.dist.barrier(device_ids=[self.local_rank])
            torch.cuda.synchronize()

    def reduce_over_ranks(self, values, op="max"):
        """Element-wise max / min / sum of a few host floats over the ranks."""
        if self.dist is None:
            return list(values)
        import torch

        t = torch.tensor(list(values), dtype=torch.float64, device=f"cuda:{self.local_rank}")
        self.dist.all_reduce(t, op={"max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN,
                                    "sum": self.dist.ReduceOp.SUM}[op])
        return [float(v) for v in t]

    def allreduce_behind(self, ptr, count, timing=None):
        """`ptr` is complete on the compute stream: sum it over the ranks on the other stream.  The
        caller makes the compute stream wait for `dw_reduced` where it needs the result."""
        self.ctx.record(self.dw_ready)
        self.comm_ctx.wait_event(self.dw_ready)
        if timing is not None:
            self.comm_ctx.record(timing[0])
        self.comm_ctx.call("katsu_cuda_allreduce_sum", ptr, count)
        if timing is not None:
            self.comm_ctx.record(timing[1])
        self.comm_ctx.record(self.dw_reduced)

    def close(self):
        if self.comm_ctx is not None:
            self.comm_ctx.call("katsu_cuda_comm_destroy")
            self.comm_ctx.close()
        self.ctx.close()
        if self.dist is not None:
            self.dist.destroy_process_group()


def tf32_peaks():
    """TF32 tensor-pipe denominators, TFLOP/s: half the driver-measured dense bf16 rate, and the rate
    this library's own MMA-issue probe reached on this part (N = 256 tiles)."""
    _, bf16_peak, kind = measured_peaks()
    return bf16_peak / 2, 1105.0, kind


def tensor_roofline(useful_tflops, passes):
    half_bf16, direct, kind = tf32_peaks()
    issued = useful_tflops * passes
    return {"bound": "tensor", "achieved": issued, "peak": half_bf16, "unit": "TFLOP/s", "frac": issued / half_bf16,
            "useful_tflops": useful_tflops, "issued_tflops": issued, "useful_frac": useful_tflops / half_bf16,
            "peak_source": f"dense bf16 of {kind} / 2", "traffic": None,
            "vs_direct_tf32_peak": {"peak": direct, "frac": issued / direct, "useful_frac": useful_tflops / direct,
                                    "peak_source": "tcgen05 kind::tf32 issue probe of this library, 128x256x8 MMAs"}}


def conv_leg(job, spec_full, precision_name, steps, warmup):
    """A short fwd + backward_buffers leg of one named shape: batch sharded over the ranks when it has
    at least one image per rank (dW all-reduced), otherwise every rank runs the whole shape."""
    from katsu_b200 import dp

    ctx, world, rank = job.ctx, job.world, job.rank
    sharded = world > 1 and spec_full.n >= world
    first, images = dp.shard(spec_full.n, rank, world) if sharded else (0, spec_full.n)
    spec = spec_full.with_batch(images)
    x_host, w_host = workloads.conv_inputs(spec_full, first, images)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    x_count, w_count, y_count = x_host.size, w_host.size, spec.n * spec.k * spec.oh * spec.ow
    px, pw = ctx.upload(x_host), ctx.upload(w_host)
    py, pg, pdx, pdw = ctx.alloc(y_count), ctx.alloc(y_count), ctx.alloc(x_count), ctx.alloc(w_count)
    ctx.set_precision({"3xtf32": 0, "tf32": 1, "fp32": 2}[precision_name])
    pstaged = 0
    try:
        # The layer holds its input from forward to backward (conv2d.rs:104-107), so it stages x once per
        # step for both (inside the timed forward); shapes whose kernels stage nothing report 0 floats.
        staged_floats = ctx.conv2d_staged_floats(*geom)
        pstaged = ctx.alloc(staged_floats) if staged_floats else 0
        ctx.conv2d_fwd(px, pw, py, *geom)
        ctx.call("katsu_cuda_add", py, py, pg, y_count)
        ctx.sync()
        ev = [[ctx.event() for _ in range(3)] for _ in range(steps)]

        def step(marks=None):
            if marks:
                ctx.record(marks[0])
            if pstaged:
                ctx.conv2d_stage(px, pstaged, spec.n, spec.c, spec.h, spec.w)
            ctx.conv2d_fwd_staged(px, pstaged or None, pw, None, py, *geom, 0)
            if marks:
                ctx.record(marks[1])
            # one call == one backward_buffers
            ctx.conv2d_bwd_staged(px, pstaged or None, pw, pg, None, 1.0, pdx, pdw, *geom, 0)
            if marks:
                ctx.record(marks[2])
            if sharded:
                job.allreduce_behind(pdw, w_count)
                ctx.wait_event(job.dw_reduced)

        for _ in range(max(3, warmup)):
            step()
        job.barrier()
        e0, e1 = ctx.event(), ctx.event()
        ctx.record(e0)
        for i in range(steps):
            step(ev[i])
        ctx.record(e1)
        ctx.sync()
        ms = ctx.elapsed_ms(e0, e1) / steps
        fwd_ms = sum(ctx.elapsed_ms(ev[i][0], ev[i][1]) for i in range(steps)) / steps
        bwd_ms = sum(ctx.elapsed_ms(ev[i][1], ev[i][2]) for i in range(steps)) / steps
        job.barrier()
    finally:
        ctx.set_precision(0)
        for p in (px, pw, py, pg, pdx, pdw, pstaged):
            ctx.free(p)
    ms, fwd_ms, bwd_ms = job.reduce_over_ranks([ms, fwd_ms, bwd_ms], "max")
    batch = spec_full.n  # sharded: the whole batch per step; replicas: each rank did the whole shape
    out = {"workload": spec_full.name, "mode": precision_name, "dtype": "f32", "n_gpus": world,
           "sharded": sharded, "global_batch": batch, "images_per_gpu": images, "steps": steps,
           "ms_per_step": ms, "kernel_ms": {"conv2d_fwd": fwd_ms, "conv2d_bwd_dx_dw": bwd_ms},
           "images_per_s": batch / (ms * 1e-3)}
    useful = 6 * spec_full.macs / (ms * 1e-3) / 1e12 / (1 if sharded else 1)
    out["useful_tflops"] = useful
    hbm_peak, _, kind = measured_peaks()
    if spec_full.c >= 16:
        passes = 3 if precision_name == "3xtf32" else 1
        per_gpu = useful / (world if sharded else 1)
        out["issued_tflops"] = useful * passes
        out["roofline"] = tensor_roofline(per_gpu, passes)
        out["roofline"]["per"] = "GPU, whole step (forward + dX + dW, staging passes included; x staged once per step)"
    else:
        gbs = spec.algorithmic_bytes / (ms * 1e-3) / 1e9
        out["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                           "peak_source": f"of {kind}", "traffic": None,
                           "per": "GPU, whole step, algorithmic bytes 2|y| + 3|x| + 3|w|"}
    return out


def gemm_leg(job, size, precision_name, steps, warmup):
    """Square Tensor::matmul forward, every rank on its own copy (matmul does not shard here)."""
    from katsu_b200 import synth

    ctx = job.ctx
    a = synth.normal(301, size * size, 1.0)
    b = synth.normal(302, size * size, 1.0)
    pa, pb, pc = ctx.upload(a), ctx.upload(b), ctx.alloc(size * size)
    ctx.set_precision({"3xtf32": 0, "tf32": 1}[precision_name])
    try:
        for _ in range(max(3, warmup)):
            ctx.matmul_fwd(pa, pb, pc, size, size, size)
        job.barrier()
        e0, e1 = ctx.event(), ctx.event()
        ctx.record(e0)
        for _ in range(steps):
            ctx.matmul_fwd(pa, pb, pc, size, size, size)
        ctx.record(e1)
        ctx.sync()
        ms = ctx.elapsed_ms(e0, e1) / steps
    finally:
        ctx.set_precision(0)
        for p in (pa, pb, pc):
            ctx.free(p)
    (ms,) = job.reduce_over_ranks([ms], "max")
    useful = 2 * size ** 3 / (ms * 1e-3) / 1e12
    passes = 3 if precision_name == "3xtf32" else 1
    out = {"workload": f"matmul_{size}x{size}x{size}", "mode": precision_name, "dtype": "f32", "n_gpus": job.world,
           "sharded": False, "steps": steps, "ms_per_step": ms, "useful_tflops": useful, "issued_tflops": useful * passes,
           "l2": "operands and result (3 x %d MB) exceed L2" % (4 * size * size // 1000000) if size >= 4096 else "fits L2",
           "roofline": tensor_roofline(useful, passes)}
    out["roofline"]["per"] = "GPU"
    return out


def stem_leg(job, args):
    """The headline leg: BASELINE config 2 (or --workload), device-timed and end to end."""
    from katsu_b200 import cabi, dp

    rank, local_rank, world, dist, ctx, comm_ctx = job.rank, job.local_rank, job.world, job.dist, job.ctx, job.comm_ctx
    spec_full = workloads.CONV[args.workload]
    if args.batch:
        spec_full = spec_full.with_batch(args.batch)
    if args.scaling == "strong":
        first, images = dp.shard(spec_full.n, rank, world)
        global_batch = spec_full.n
    else:
        first, images = 0, spec_full.n
        global_batch = spec_full.n * world
    spec = spec_full.with_batch(images)
    x_host, w_host = workloads.conv_inputs(spec_full, first, images)

    precision = {"3xtf32": 0, "tf32": 1, "fp32": 2}[args.precision]
    ctx.set_precision(precision)

    n, c, h, wd, k, r, s = spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s
    geom = (n, c, h, wd, k, r, s, spec.stride, spec.pad)
    x_count, w_count, y_count = n * c * h * wd, k * c * r * s, n * k * spec.oh * spec.ow
    px, pw = ctx.upload(x_host), ctx.upload(w_host)
    py, pg, pdx, pdw = ctx.alloc(y_count), ctx.alloc(y_count), ctx.alloc(x_count), ctx.alloc(w_count)
    ctx.conv2d_fwd(px, pw, py, *geom)
    ctx.call("katsu_cuda_add", py, py, pg, y_count)  # g = 2y, the seed sum(y*y) sends back
    ctx.sync()

    def step():
        ctx.conv2d_fwd(px, pw, py, *geom)
        ctx.conv2d_bwd(px, pw, pg, 0, pdw, *geom, 0)
        if world > 1:
            job.allreduce_behind(pdw, w_count)
        ctx.conv2d_bwd(px, pw, pg, pdx, 0, *geom, 0)
        if world > 1:
            ctx.wait_event(job.dw_reduced)  # the step ends when dX and the reduced dW are both there

    barrier = job.barrier
    warmup = max(args.warmup, 3)  # never fewer than three untimed steps
    ev = [[ctx.event() for _ in range(4)] for _ in range(args.steps)]
    ar_ev = [[comm_ctx.event(), comm_ctx.event()] for _ in range(args.steps)] if world > 1 else None
    e_start, e_stop = ctx.event(), ctx.event()
    # the clock sampler (nvidia-smi, one line per 100 ms) starts before the warm-up so that it is
    # already running when the timed steps, which may last only milliseconds, go by
    with ClockSampler(local_rank, enabled=rank == 0) as clocks:
        for _ in range(warmup):
            step()
        clocks.wait_first()
        barrier()
        launches0 = ctx.launch_count()
        host_t0 = time.perf_counter()
        ctx.record(e_start)
        for i in range(args.steps):
            ctx.record(ev[i][0])
            ctx.conv2d_fwd(px, pw, py, *geom)
            ctx.record(ev[i][1])
            ctx.conv2d_bwd(px, pw, pg, 0, pdw, *geom, 0)
            ctx.record(ev[i][2])
            if world > 1:
                job.allreduce_behind(pdw, w_count, ar_ev[i])
            ctx.conv2d_bwd(px, pw, pg, pdx, 0, *geom, 0)
            ctx.record(ev[i][3])
            if world > 1:
                ctx.wait_event(job.dw_reduced)
        ctx.record(e_stop)
        host_enqueue_ms = (time.perf_counter() - host_t0) * 1e3 / args.steps
        ctx.sync()
        if world > 1:
            comm_ctx.sync()
        launches = ctx.launch_count() - launches0
        total_ms = ctx.elapsed_ms(e_start, e_stop)
        # a timed region shorter than the sampling period: keep the same load on until two samples exist
        t_probe = time.perf_counter()
        while rank == 0 and len(clocks.lines) < 2 and time.perf_counter() - t_probe < 1.5:
            ctx.conv2d_fwd(px, pw, py, *geom)  # local kernels only: the other ranks have moved on
            ctx.conv2d_bwd(px, pw, pg, pdx, 0, *geom, 0)
            ctx.sync()
    barrier()
    ms_per_step = total_ms / args.steps
    parts = {"conv2d_fwd": [], "conv2d_bwd_dx": [], "conv2d_bwd_dw": []}
    for i in range(args.steps):
        for name, a, b in (("conv2d_fwd", 0, 1), ("conv2d_bwd_dw", 1, 2), ("conv2d_bwd_dx", 2, 3)):
            parts[name].append(ctx.elapsed_ms(ev[i][a], ev[i][b]))
    part_ms = {name: sum(v) / len(v) for name, v in parts.items()}
    allreduce_ms = None
    if world > 1:
        allreduce_ms = sum(comm_ctx.elapsed_ms(a, b) for a, b in ar_ev) / args.steps

    # Checker, outside the timed region: the (all-reduced) dW of the last step against the oracle's
    # exact sums of sampled elements over the GLOBAL batch.  Each rank sums its own images' terms
    # (from its own x and its device's g = 2y); the partial sums are added over the ranks.
    dw_check = None
    if not args.no_dw_check:
        idx = np.random.default_rng(20).choice(w_count, min(48, w_count), replace=False)
        g_host = ctx.download(pg, y_count)
        partial = oracle_dw_samples(spec, x_host, g_host, idx)
        del g_host
        exact = np.asarray(job.reduce_over_ranks(partial, "sum"))
        got = ctx.download(pdw, w_count)[idx].astype(np.float64)
        dw_check = float(np.linalg.norm(got - exact) / max(np.linalg.norm(exact), 1e-300))
        bar = 2e-3 if args.precision == "tf32" else 1e-5
        if not np.isfinite(dw_check) or dw_check > bar:
            raise RuntimeError(f"dW after the all-reduce differs from the oracle: rel-L2 {dw_check:.3e} > {bar}")

    # End to end through the C ABI with HOST buffers: pinned x in, dX and dW out, every step.
    # The batch is cut into chunks that rotate over a few contexts (streams) of the same device:
    # within one stream a chunk's copy in, kernels and copy out are serial, so it takes three or
    # more streams to keep the two copy engines and the SMs busy at once -- what a caller with a
    # data loader does.  The contexts' dW partials are added on the device (events order the
    # other streams before the adds; the host does not
    # block inside a step), all-reduced across ranks and copied to a pinned slot of that step;
    # the host synchronises once after the last step, so consecutive steps pipeline as well.
    for p in (py, pg, pdx):
        ctx.free(p)
    affinity = bind_near_gpu(local_rank, world) if world > 1 else {"bound": False, "why": "one rank"}
    e2e_steps = args.e2e_steps or max(3, min(args.steps, 10))
    x_pin, dx_pin = ctx.pinned(x_count), ctx.pinned(x_count)
    dw_pin = [ctx.pinned(w_count) for _ in range(e2e_steps + 1)]
    x_pin[:] = x_host
    n_lanes = max(1, args.e2e_lanes)
    # Each lane is a context of its own (one stream each); all run the same kernels as the device-timed leg.
    lanes = [cabi.Context(local_rank) for _ in range(n_lanes)]
    for lane_ctx in lanes:
        lane_ctx.set_precision(precision)
    lead = lanes[0]
    # chunks of at least 16 images: with 8 (a rank's 64-image share cut in eight) the leg spent its time on
    # launches and small copies (4 GPUs: 114 700 images/s with eight chunks, 135 600 with four)
    n_chunks = max(1, min(args.e2e_chunks, n // 16))
    bounds = [dp.shard(n, i, n_chunks) for i in range(n_chunks)]
    per_img_x, per_img_y = c * h * wd, k * spec.oh * spec.ow
    chunk_max = max(cnt for _, cnt in bounds)
    lane_buf = []
    for lane_ctx in lanes:
        lane_buf.append({"w": lane_ctx.upload(w_host), "x": lane_ctx.alloc(chunk_max * per_img_x),
                         "y": lane_ctx.alloc(chunk_max * per_img_y), "g": lane_ctx.alloc(chunk_max * per_img_y),
                         "dx": lane_ctx.alloc(chunk_max * per_img_x),
                         # two dW partials per lane, alternating by step, so that a lane can start the
                         # next step while lane 0 is still combining (and all-reducing) this one
                         "dw": [lane_ctx.alloc(w_count), lane_ctx.alloc(w_count)]})
    lane_done = [lane_ctx.event() for lane_ctx in lanes]
    combined = [lead.event(), lead.event()]  # lane 0 has consumed the partials of parity 0 / 1

    # Copy rates alone, every rank at once (all the ranks' copies share the host's memory system
    # and, depending on the box, PCIe switches): the ceiling of the end-to-end leg at N GPUs.
    copy_gbs = {}
    for name, fn in (("h2d", lambda: lead.h2d(lane_buf[0]["x"], x_pin[:chunk_max * per_img_x])),
                     ("d2h", lambda: lead.d2h_async(dx_pin[:chunk_max * per_img_x], lane_buf[0]["dx"]))):
        fn()
        lead.sync()
        barrier()
        t0 = time.perf_counter()
        for _ in range(8):
            fn()
        lead.sync()
        dt = (time.perf_counter() - t0) / 8
        copy_gbs[name] = 4 * chunk_max * per_img_x / dt / 1e9
        barrier()
    copy_min = job.reduce_over_ranks([copy_gbs["h2d"], copy_gbs["d2h"]], "min")

    def e2e_step(slot, fused=True, read_dx=True):
        par = slot & 1
        # a lane must not overwrite a dW partial that lane 0 has not yet added (two steps back)
        for lane_ctx in lanes[1:]:
            lane_ctx.wait_event(combined[par])
        for i, (first_img, cnt) in enumerate(bounds):
            lane_ctx, b = lanes[i % n_lanes], lane_buf[i % n_lanes]
            cg = (cnt, c, h, wd, k, r, s, spec.stride, spec.pad)
            lane_ctx.h2d(b["x"], x_pin[first_img * per_img_x:(first_img + cnt) * per_img_x])
            lane_ctx.conv2d_fwd(b["x"], b["w"], b["y"], *cg)
            if fused:
                # what loss = sum(y * y) sends back is 2 * y: the backward kernels read y and scale their
                # outputs, the gradient of y's size is never written (the graph API does the same)
                lane_ctx.call("katsu_cuda_conv2d_bwd_scaled", b["x"], b["w"], b["y"], 0, 2.0, b["dx"], 0, *cg, 0)
                lane_ctx.call("katsu_cuda_conv2d_bwd_scaled", b["x"], b["w"], b["y"], 0, 2.0, 0, b["dw"][par], *cg,
                              1 if i >= n_lanes else 0)
            else:
                lane_ctx.call("katsu_cuda_add", b["y"], b["y"], b["g"], cnt * per_img_y)
                lane_ctx.conv2d_bwd(b["x"], b["w"], b["g"], b["dx"], 0, *cg, 0)
                lane_ctx.conv2d_bwd(b["x"], b["w"], b["g"], 0, b["dw"][par], *cg, 1 if i >= n_lanes else 0)
            if read_dx:
                lane_ctx.d2h_async(dx_pin[first_img * per_img_x:(first_img + cnt) * per_img_x], b["dx"])
        total = lane_buf[0]["dw"][par]
        for j in range(1, min(n_lanes, n_chunks)):
            lanes[j].record(lane_done[j])
            lead.wait_event(lane_done[j])
            lead.call("katsu_cuda_axpy_acc", total, lane_buf[j]["dw"][par], w_count)
        if world > 1:
            lead.record(job.dw_ready)
            comm_ctx.wait_event(job.dw_ready)
            comm_ctx.call("katsu_cuda_allreduce_sum", total, w_count)
            comm_ctx.record(job.dw_reduced)
            lead.wait_event(job.dw_reduced)
        lead.d2h_async(dw_pin[slot], total)
        lead.record(combined[par])

    lead.record(combined[0]), lead.record(combined[1])

    def e2e_run(fused, read_dx=True):
        e2e_step(e2e_steps, fused, read_dx)
        for lane_ctx in lanes:
            lane_ctx.sync()
        barrier()
        t0 = time.perf_counter()
        for step_index in range(e2e_steps):
            e2e_step(step_index, fused, read_dx)
        for lane_ctx in lanes:
            lane_ctx.sync()
        ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        barrier()
        return ms

    e2e_unfused_ms = e2e_run(False)  # the gradient 2y written out by a separate pass, for comparison
    # dX computed but left on the device (what a training loop that only needs dW and the loss pays: the
    # host classes download a gradient when it is read); a second figure, the headline below reads dX back
    e2e_dw_only_ms = e2e_run(True, read_dx=False)
    e2e_ms = e2e_run(True)
    # Every step's dW reached the host; the inputs are the same every step, so the steps should
    # agree bit for bit.  The largest deviation from step 0 (relative to max |dW|) is reported as
    # e2e.dw_step_spread (0.0 = bit-identical); a gross difference is an error.
    dw_scale = float(np.abs(dw_pin[0]).max()) or 1.0
    dw_spread = max(float(np.abs(dw_pin[0] - dw_pin[i]).max()) for i in range(1, e2e_steps)) / dw_scale
    if not np.isfinite(dw_spread) or dw_spread > 1e-3:
        raise RuntimeError(f"end-to-end leg: dW differs between steps by {dw_spread:.3e} of max |dW|")
    dw_differing = sum(1 for i in range(1, e2e_steps) if not np.array_equal(dw_pin[0], dw_pin[i]))

    step_min, e2e_min = job.reduce_over_ranks([ms_per_step, e2e_ms], "min")
    stats = [ms_per_step, e2e_ms, host_enqueue_ms, allreduce_ms or 0.0, e2e_unfused_ms, e2e_dw_only_ms]
    ms_per_step, e2e_ms, host_enqueue_max, allreduce_max, e2e_unfused_ms, e2e_dw_only_ms = job.reduce_over_ranks(stats, "max")

    line = None
    if rank == 0:
        hbm_peak, bf16_peak, peak_kind = measured_peaks()
        dominant = max(part_ms, key=part_ms.get)
        kernel_bytes = {
            "conv2d_fwd": 4 * (x_count + w_count + y_count),
            "conv2d_bwd_dx": 4 * (y_count + w_count + x_count),
            "conv2d_bwd_dw": 4 * (y_count + x_count + w_count),
        }
        step_gbs = spec.algorithmic_bytes / (ms_per_step * 1e-3) / 1e9
        # Low-channel shapes move ~19 flop per byte: HBM roofline.  Wide-channel shapes are
        # contractions: tensor roofline, against TF32 taken as half the measured dense bf16 rate.
        if spec.c >= 16:
            passes = 3 if args.precision == "3xtf32" else 1
            roof = tensor_roofline(2 * spec.macs / (part_ms[dominant] * 1e-3) / 1e12, passes)
            roof["kernel"] = dominant
        else:
            achieved = kernel_bytes[dominant] / (part_ms[dominant] * 1e-3) / 1e9
            roof = {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                    "frac": achieved / hbm_peak, "traffic": captured_traffic(spec_full.name, dominant, images),
                    "peak_source": f"of {peak_kind}"}
        roof.update({"kernel_ms": part_ms, "step_algorithmic_gbs_per_gpu": step_gbs,
                     "step_frac": step_gbs / hbm_peak})
        line = {
            "metric": METRIC, "value": global_batch / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(spec_full, world, args.scaling),
            "mode": args.precision,
            "tflops": 6 * spec_full.with_batch(global_batch).macs / (ms_per_step * 1e-3) / 1e12,
            "roofline": roof,
            "dw_rel_l2_vs_oracle": dw_check,
            "step_breakdown": {"ms_per_step_min_over_ranks": step_min, "ms_per_step_max_over_ranks": ms_per_step,
                               "host_enqueue_ms_per_step_max": host_enqueue_max,
                               "allreduce_ms_on_comm_stream_max": allreduce_max if world > 1 else None},
            "e2e": {"value": global_batch / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "ms_per_step_min_over_ranks": e2e_min,
                    "h2d_bytes_per_step": 4 * x_count, "d2h_bytes_per_step": 4 * (x_count + w_count),
                    "pipeline": f"{n_chunks} batch chunks over {n_lanes} streams, pinned host buffers, one host sync after the last step",
                    "upstream_gradient": "2y read from y by the backward kernels (scaled outputs)",
                    "ms_per_step_with_gradient_written_out": e2e_unfused_ms,
                    "leaving_dx_on_the_device": {"ms_per_step": e2e_dw_only_ms,
                                                 "images_per_s": global_batch / (e2e_dw_only_ms * 1e-3),
                                                 "d2h_bytes_per_step": 4 * w_count},
                    "copy_only_gbs_min_over_ranks": {"h2d": copy_min[0], "d2h": copy_min[1],
                                                     "note": "one direction at a time, all ranks at once"},
                    "host_affinity": affinity,
                    "dw_step_spread": dw_spread, "dw_steps_differing": dw_differing},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
        }

    for p in (px, pw, pdw):
        ctx.free(p)
    for lane_ctx, b in zip(lanes, lane_buf):
        for p in b.values():
            for q in (p if isinstance(p, list) else [p]):
                lane_ctx.free(q)
    for a in [x_pin, dx_pin] + dw_pin:
        ctx.free_pinned(a)
    for lane_ctx in lanes:
        lane_ctx.close()
    ctx.set_precision(0)
    return line, spec_full


def other_workloads(job, args):
    """Short legs of the other named shapes and of square matmuls, both tensor-core modes, so that one
    default run records every configuration (3-5 steps each)."""
    steps, warmup = args.other_steps, 3
    legs = []

    def run(label, fn):
        t0 = time.perf_counter()
        try:
            entry = fn()
        except Exception as exc:  # one leg failing must not lose the headline line
            entry = {"workload": label, "error": f"{type(exc).__name__}: {exc}"}
        entry["wall_s"] = round(time.perf_counter() - t0, 2)
        legs.append(entry)

    run("rgb_example", lambda: conv_leg(job, workloads.CONV["rgb_example"], "3xtf32", max(steps, 20), warmup))
    for name in ("wide_128x256x56", "down_128x128x112_s2"):
        for mode in ("3xtf32", "tf32"):
            run(f"{name}/{mode}", lambda name=name, mode=mode: conv_leg(job, workloads.CONV[name], mode, steps, warmup))
    run("small_cnn", lambda: small_cnn_leg(job, args, steps=max(steps, 20), warmup=warmup, sample_clocks=False))
    for size in (4096, 8192):
        for mode in ("3xtf32", "tf32"):
            run(f"matmul_{size}/{mode}", lambda size=size, mode=mode: gemm_leg(job, size, mode, steps, warmup))
    return legs


def run_ours(args):
    job = Job(args)
    line, spec_full = stem_leg(job, args)
    others = None
    if args.workload == "stem_256x3x224" and not args.batch and not args.no_others:
        others = other_workloads(job, args)
    if job.rank == 0:
        if others is not None:
            line["other_workloads"] = others
        if job.world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(spec_full, args.cpu_sample)
        print(json.dumps(line), flush=True)
    job.close()
    return 0


def small_cnn_leg(job, args, steps, warmup, sample_clocks=True):
    """BASELINE config 5: conv 3->32 s1 p1, conv 32->64 s2 p1, reshape, matmul [N,65536]@[65536,10], add a
    constant, loss = sum(out*out), loss.backward() -- the whole autograd graph on the device through the
    katsu_b200 surface (the C++ host mirror), batch sharded over the ranks, the three weight gradients
    summed with one all-reduce of a flat bucket."""
    import ctypes

    import katsu_b200 as K
    from katsu_b200 import cabi, dp

    rank, local_rank, world, dist = job.rank, job.local_rank, job.world, job.dist
    K.set_device(local_rank)
    total = args.batch or workloads.CNN["batch"]
    first, batch = dp.shard(total, rank, world)
    c1 = workloads.CONV["cnn_conv1"].with_batch(total)
    c2 = workloads.CONV["cnn_conv2"].with_batch(total)
    x, w1 = workloads.conv_inputs(c1, first, batch)
    _, w2 = workloads.conv_inputs(c2, 0, 1)
    fc_in, fc_out = workloads.CNN["fc_in"], workloads.CNN["fc_out"]
    tx = K.Tensor(x, [batch, c1.c, c1.h, c1.w]).to_device()
    tw1 = K.Tensor(w1, c1.w_shape).to_device()
    tw2 = K.Tensor(w2, c2.w_shape).to_device()
    twfc = K.Tensor(workloads.cnn_fc_weights(), [fc_in, fc_out]).to_device()
    tconst = K.Tensor(workloads.cnn_constant(first, batch), [batch, fc_out]).to_device()
    params = {"w1": tw1, "w2": tw2, "wfc": twfc}
    raw = cabi.load()
    handle = K.context()

    def call(name, *a):
        cabi.check(getattr(raw, name)(handle, *a))

    bucket_ptr, offsets, cursor = None, {}, 0
    for name, t in params.items():
        offsets[name] = cursor
        cursor += -(-t.numel() // 64) * 64
    if world > 1:
        out = ctypes.c_void_p()
        call("katsu_cuda_alloc", cursor, ctypes.byref(out))
        bucket_ptr = out.value
        ident = [None]
        if rank == 0:
            buf = (ctypes.c_uint8 * cabi.COMM_ID_BYTES)()
            cabi.check(raw.katsu_cuda_comm_unique_id(buf))
            ident[0] = bytes(buf)
        dist.broadcast_object_list(ident, src=0)
        call("katsu_cuda_comm_init", (ctypes.c_uint8 * cabi.COMM_ID_BYTES).from_buffer_copy(ident[0]), world, rank)

    def step():
        conv1 = K.Conv2D.from_weights(tw1, 1, 1)
        conv2 = K.Conv2D.from_weights(tw2, 2, 1)
        h2 = conv2.forward(conv1.forward(tx))
        out = h2.reshape([batch, fc_in]).matmul(twfc).add(tconst)
        loss = out.mul(out).sum()
        loss.backward()
        if world > 1:
            for name, t in params.items():
                call("katsu_cuda_d2d", bucket_ptr + 4 * offsets[name], t.device_grad(), t.numel())
            call("katsu_cuda_allreduce_sum", bucket_ptr, cursor)
        for t in (tx, tw1, tw2, twfc, tconst):
            t.zero_grad()
        return loss

    def barrier():
        K.synchronize()
        job.barrier()

    for _ in range(max(warmup, 3)):
        step()
    barrier()
    # three timed groups of K steps, each synchronised at both ends; the median is reported (the
    # timing is on the host, and one group in a few catches a scheduling hiccup of 1 ms per step)
    groups = []
    for _ in range(3):
        t0 = time.perf_counter()
        for _ in range(steps):
            loss = step()
        K.synchronize()
        groups.append((time.perf_counter() - t0) * 1e3 / steps)
        barrier()
    ms = sorted(groups)[1]
    loss_value = float(loss.data()[0])
    (ms,) = job.reduce_over_ranks([ms], "max")
    clock_summary = None
    if sample_clocks:
        # This workload is timed on the host and synchronises inside every step, so an nvidia-smi
        # process polling through the driver slows it (measured: 3.1 instead of 1.7 ms/step on two
        # GPUs).  The clocks are therefore sampled on an untimed replay of the same steps right after:
        # the same number of steps on every rank (they contain a collective), about 0.6 s worth.
        replay = int(min(2000, max(10, 600.0 / ms)))
        with ClockSampler(local_rank, enabled=rank == 0) as clocks:
            for _ in range(replay):
                step()
            K.synchronize()
        barrier()
        clock_summary = clocks.summary()
    flops = 6 * (c1.macs + c2.macs + total * fc_in * fc_out)
    hbm_peak, _, kind = measured_peaks()
    algorithmic = (c1.algorithmic_bytes + c2.algorithmic_bytes + 4 * (3 * total * fc_in + 3 * fc_in * fc_out + 2 * total * fc_out)) / world
    gbs = algorithmic / (ms * 1e-3) / 1e9
    entry = {
        "workload": "small_cnn", "mode": "3xtf32", "dtype": "f32", "n_gpus": world, "sharded": world > 1,
        "global_batch": total, "images_per_gpu": batch, "steps": steps, "ms_per_step": ms,
        "images_per_s": total / (ms * 1e-3), "useful_tflops": flops / (ms * 1e-3) / 1e12,
        "graph": "conv3->32 s1p1, conv32->64 s2p1, reshape, matmul [N,65536]x[65536,10], add, sum(out*out), backward",
        "timing": "host wall clock around whole graph steps, device synchronised at both ends; median of three groups of `steps`",
        "groups_ms_per_step": [round(g, 4) for g in groups], "loss_rank0": loss_value,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                     "peak_source": f"of {kind}", "traffic": None,
                     "per": "GPU, whole graph step; algorithmic bytes of the two convolutions and the matmul only "
                            "(the loss graph's streaming passes come on top)"},
    }
    if clock_summary is not None:
        entry["clocks"] = clock_summary
        entry["clocks_sampled"] = "untimed replay of the same steps right after the timed ones"
    if world > 1:
        call("katsu_cuda_comm_destroy")
        call("katsu_cuda_free", bucket_ptr)
    return entry


def run_small_cnn(args):
    job = Job(args)
    entry = small_cnn_leg(job, args, steps=args.steps, warmup=args.warmup)
    if job.rank == 0:
        line = {"metric": "small_cnn_fwd_bwd_images_per_s", "value": entry["images_per_s"], "unit": UNIT,
                "n_gpus": job.world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": entry["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "small_cnn", "global_batch": entry["global_batch"],
                           "images_per_gpu": entry["images_per_gpu"], "graph": entry["graph"], "timing": entry["timing"],
                           "groups_ms_per_step": entry["groups_ms_per_step"],
                           "clocks_sampled": entry.get("clocks_sampled")},
                "tflops": entry["useful_tflops"], "loss_rank0": entry["loss_rank0"], "roofline": entry["roofline"],
                "clocks": entry.get("clocks")}
        print(json.dumps(line), flush=True)
    job.close()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="stem_256x3x224", choices=sorted(workloads.CONV) + ["small_cnn", "matmul"])
    ap.add_argument("--size", type=int, default=4096, help="--workload matmul: m = k = n")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong")
    ap.add_argument("--cpu-sample", type=int, default=32, help="images in the single-thread CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--precision", choices=["3xtf32", "tf32", "fp32"], default="3xtf32",
                    help="contraction mode of the kernels (the metric is quoted on the default)")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end leg (default: min(steps, 10))")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="batch chunks of the end-to-end leg (at least 16 images each)")
    ap.add_argument("--e2e-lanes", type=int, default=8, help="contexts (streams) the chunks rotate over")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch (small profiling cases)")
    ap.add_argument("--no-others", action="store_true", help="skip the short legs of the other named workloads")
    ap.add_argument("--other-steps", type=int, default=4, help="timed steps of each of those legs")
    ap.add_argument("--no-dw-check", action="store_true", help="skip the oracle check of the all-reduced dW")
    args = ap.parse_args()
    if args.workload == "small_cnn":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm times the conv workloads only"}))
            return 0
        return run_small_cnn(args)
    if args.workload == "matmul":
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm times the conv workloads only"}))
            return 0
        job = Job(args)
        entry = gemm_leg(job, args.size, args.precision, args.steps, args.warmup)
        if job.rank == 0:
            print(json.dumps(entry), flush=True)
        job.close()
        return 0
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
