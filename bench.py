#!/usr/bin/env python
"""Benchmark of the dense-contraction path: LeNet5 inference images/s and GEMM TFLOP/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--quick]

A step is one LeNet5 forward pass over one batch of 1000 synthetic images in f32
(benchmark configuration 0, the one the metric "LeNet5 infer img/s (bs1000)" is
quoted on).  With N > 1 every rank (one process per GPU, launched by torchrun) runs the
same step on its own 1000-image shard: inference shards by batch with no collective, so
scaling is weak and `value` is the images all ranks processed divided by the slowest
rank's device time.

The K-step window is timed REPEATS times (a barrier and a device synchronisation on both
sides of every window, CUDA events on the launching stream, the maximum over ranks per
window) and the median window is reported, so that a 20-step run is not one 0.6 ms sample.

One JSON line is printed by rank 0.  Besides the contract keys it carries
  roofline      the step's kernel against its binding bound (the FP32 pipe; HBM view inside)
  e2e           the same step through Model.infer with pinned host buffers (copies inside the
                timed region); e2e_pipelined: two batches in flight through
                ag_model_infer_enqueue / _wait; e2e_pageable: the same from pageable host memory
  infer_sharded_65536   configs[4a]: 65536 images split evenly over the ranks (strong scaling)
  train_dp      configs[4b]: 100 images per GPU, gradient all-reduce, SGD update
  gemm          the standalone dot sweep (configs[1]) in TFLOP/s, with `gemm_roofline`
                for the 4096^3 bf16 dot against the measured bf16 tensor peak
  cpu_baseline  the CPU oracle (a port of the reference's host path) on this box's cores,
                timed after the GPU work, when rank 0 is the only process left
  extras        bf16 inference, the training step, u8 input pipeline, the wide conv stack

`--impl reference` times the CPU restatement of the reference's host path instead
(the reference is Rust; no Rust toolchain exists on these machines).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "lenet5_infer_img_per_s"
UNIT = "img/s"
BATCH = 1000
FLOPS_PER_IMG = 568720            # 2*(576*25*6 + 64*150*16 + 256*128 + 128*84 + 84*10)
ROTATE = 64                       # distinct input batches: 64 * 3.136 MB = 200 MB > 126 MB L2
REPEATS = 9                       # the K-step window is timed this many times; the median is reported
WORKLOAD = "LeNet5 inference f32, batch 1000 per step per GPU (benchmark configuration 0)"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ------------------------------------------------------------------ clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.marks = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu=timestamp,{self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(gpu_index), "-lms", "50"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self, t0, t1):
        self.marks.append((t0, t1))

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0, samples_in_timed_regions=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = []
        import datetime
        for line in Path(self.file.name).read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(parts[2]), float(parts[3]), float(parts[4]), parts[5:]))
            except ValueError:
                continue
        os.unlink(self.file.name)
        if not rows:
            return out
        timed = [r for r in rows if any(a - 0.05 <= r[0] <= b + 0.05 for a, b in self.marks)]
        busy = timed or [r for r in rows if r[3] > 250.0] or rows
        out["samples"] = len(rows)
        out["samples_in_timed_regions"] = len(timed)
        out["sm_mhz"] = float(np.median([r[1] for r in busy]))
        out["sm_max_mhz"] = max(r[2] for r in rows)
        out["power_w_max"] = max(r[3] for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        seen = set()
        for r in busy:
            flags = r[4]
            for name, val in zip(names, flags[1:5]):
                if val.lower().startswith("active"):
                    seen.add(name)
        out["reasons"] = sorted(seen)
        return out


# ------------------------------------------------------------- CPU baseline
def cpu_forward_windows(steps: int, warm_s: float, sample_s: float, warm_steps: int = 1):
    """The oracle's LeNet5 forward (direct f32 conv restating conv_direct.rs, threaded GEMM) on
    all host cores, batches of 1000: warms up for warm_s seconds, then times windows of `steps`
    passes until there are REPEATS of them and sample_s seconds have passed.  Returns the list of
    window times and the thread count.  Both the reference arm and the GPU arm's cpu_baseline
    are measured by this one routine."""
    import oracle
    from oracle import models
    oracle.use_all_cores()
    # The activations of a pass are fresh 14 MB numpy arrays.  glibc serves blocks of that size
    # with mmap until it has seen such blocks freed, so a fresh process pays a round of page
    # faults per pass (measured: 8.1 ms per pass against 7.0 ms in a process that had allocated
    # and freed large blocks before).  Keep them on the heap in both arms.
    try:
        import ctypes
        libc = ctypes.CDLL("libc.so.6")
        libc.mallopt(-3, 1 << 30)   # M_MMAP_THRESHOLD
        libc.mallopt(-1, 1 << 30)   # M_TRIM_THRESHOLD
    except OSError:
        pass
    P = models.init_params(models.LENET5, 2000)
    x = np.random.default_rng(1000).uniform(0, 1, (BATCH, 1, 28, 28)).astype(np.float32)
    t_warm = time.perf_counter()
    done = 0
    while done < max(warm_steps, 1) or time.perf_counter() - t_warm < warm_s:
        models.forward(models.LENET5, P, x, fast=True)
        done += 1
    windows = []
    t_begin = time.perf_counter()
    while len(windows) < REPEATS or (time.perf_counter() - t_begin < sample_s and len(windows) < 400):
        t0 = time.perf_counter()
        for _ in range(steps):
            models.forward(models.LENET5, P, x, fast=True)
        windows.append(time.perf_counter() - t0)
        if time.perf_counter() - t_begin > 120.0:
            break
    return windows, oracle.num_threads()


def cpu_forward_rate(seconds: float, min_steps: int = 2):
    """Images/s (median window), thread count, passes and seconds of cpu_forward_windows."""
    windows, cores = cpu_forward_windows(20, 1.0, seconds)
    dt = float(np.median(windows))
    return 20 * BATCH / dt, cores, 20 * len(windows), float(sum(windows))


def cpu_train_rate(seconds: float):
    """Steps/s of the oracle's LeNet5 training step at batch 100 (benchmark configuration 2:
    forward, cross-entropy, backward through the reference's host direct-convolution kernels,
    plain SGD) on all host cores."""
    import oracle
    from oracle import models
    oracle.use_all_cores()
    P = models.init_params(models.LENET5, 2000)
    x = np.random.default_rng(4000).uniform(0, 1, (100, 1, 28, 28)).astype(np.float32)
    t = np.random.default_rng(4001).integers(0, 10, 100).astype(np.uint32)
    models.train_step(models.LENET5, P, x, t, 0.01)
    n, t0 = 0, time.perf_counter()
    while n < 3 or time.perf_counter() - t0 < seconds:
        models.train_step(models.LENET5, P, x, t, 0.01)
        n += 1
    dt = time.perf_counter() - t0
    return n / dt, oracle.num_threads(), n, dt


def run_reference(args):
    """The reference arm: the reference's host path, restated in C (oracle/), timed on the
    host cores with all threads; K steps of one 1000-image forward each."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    # Warm up for at least three seconds (thread pool, caches, host clocks), then time windows of
    # K steps until there are REPEATS of them and eight seconds have passed; the median window
    # counts.
    steps = min(args.steps, 2000)
    windows, cores = cpu_forward_windows(steps, 3.0, 8.0, args.warmup)
    dt = float(np.median(windows))
    value = steps * BATCH / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": value / PUBLISHED_IMG_PER_S,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "note": "CPU restatement of the reference's host path (oracle/); the reference "
                           "itself is Rust and cannot be built on this box"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"median of {len(windows)} windows of {steps} forward passes "
                                   "of 1000 images"},
        "repeats_ms_per_step": [w / steps * 1e3 for w in windows[:32]],
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def event_time_ms(torch, fn, iters, stream):
    """Total device time of `iters` calls of fn, CUDA events on the launching stream."""
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for i in range(iters):
        fn(i)
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end)


def run_gpu(args):
    import torch
    import autograph_b200 as ag
    from autograph_b200 import data_parallel as dp

    rank, local_rank, world = dp.env_world()
    if world > 1:
        dist = dp.init_process_group("nccl")
    torch.cuda.set_device(local_rank)
    dev = ag.Device(local_rank)
    stream = dev.stream
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank) if rank == 0 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev.torch_device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    K, W = args.steps, max(args.warmup, 3)
    # Random-init weights of the architecture: the library's seeded default initialiser.
    model = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)

    def timed_windows(fn, steps):
        """REPEATS windows of exactly `steps` calls, each bracketed by a barrier and a device
        synchronisation on both sides and timed with CUDA events on the launching stream; per
        window the maximum over ranks.  Returns the per-window times in ms."""
        out = []
        for _ in range(REPEATS):
            barrier()
            t0 = time.time()
            ms_w = event_time_ms(torch, fn, steps, stream)
            t1 = time.time()
            barrier()
            if sampler:
                sampler.mark(t0, t1)
            out.append(ms_w)
        if world > 1:
            t = torch.tensor(out, dtype=torch.float64, device=dev.torch_device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out = [float(v) for v in t.tolist()]
        return out

    # Device-resident inputs, rotated so that every step reads its images from HBM.
    gen = torch.Generator(device=dev.torch_device).manual_seed(1000 + rank)
    xs = torch.rand((ROTATE, BATCH, 1, 28, 28), generator=gen, device=dev.torch_device)
    out = dev.empty((BATCH, 10), torch.float32)

    def step(i):
        model.forward_device(xs[i % ROTATE], out)

    for i in range(W):
        step(i)
    barrier()
    launches0 = ag.kernel_launch_count()
    windows = timed_windows(step, K)
    launches = (ag.kernel_launch_count() - launches0) // REPEATS
    ms = float(np.median(windows))
    value = world * BATCH * K / (ms * 1e-3)

    # End to end through the public call with host buffers (pinned): H2D of the images and
    # D2H of the logits inside the timed region.
    xh = [torch.rand((BATCH, 1, 28, 28)).pin_memory() for _ in range(4)]
    oh = torch.empty((BATCH, 10), dtype=torch.float32).pin_memory()
    for i in range(W):
        model.infer(xh[i % 4], oh)
    Ke = max(min(K, 2000), 10)
    e2e_windows = timed_windows(lambda i: model.infer(xh[i % 4], oh), Ke)
    ms_e2e = float(np.median(e2e_windows))
    e2e = {"value": world * BATCH * Ke / (ms_e2e * 1e-3), "unit": UNIT,
           "h2d_bytes_per_step": BATCH * 784 * 4, "d2h_bytes_per_step": BATCH * 10 * 4,
           "steps": Ke, "ms_per_step": ms_e2e / Ke, "host_memory": "pinned",
           "repeats_ms_per_step": [w / Ke for w in e2e_windows]}
    # The serving form of the same call: two batches in flight (ag_model_infer_enqueue / _wait),
    # the copy engine moving batch i + 1 while the network runs on batch i.  Every step still
    # has its H2D copy and its D2H logits inside the timed region; what differs from `e2e` is
    # that a step's result is collected one step later.
    try:
        ohs = [torch.empty((BATCH, 10), dtype=torch.float32).pin_memory() for _ in range(2)]
        tickets = []

        def pstep(i):
            if len(tickets) == 2:
                model.infer_wait(tickets.pop(0))
            tickets.append(model.infer_enqueue(xh[i % 4], ohs[i % 2]))

        # the copy engine's first transfers of a process on a freshly started box run at a
        # fraction of the link rate for a while (measured: 113 - 197 us per step in the first
        # process, 70 us in the next one): warm the path up for a second before timing
        t_end = time.perf_counter() + 1.0
        i = 0
        while i < W or time.perf_counter() < t_end:
            pstep(i)
            i += 1
        pipe_windows = timed_windows(pstep, Ke)
        while tickets:
            model.infer_wait(tickets.pop(0))
        ms_pipe = float(np.median(pipe_windows))
        e2e_pipelined = {"value": world * BATCH * Ke / (ms_pipe * 1e-3), "unit": UNIT,
                         "h2d_bytes_per_step": BATCH * 784 * 4, "d2h_bytes_per_step": BATCH * 10 * 4,
                         "steps": Ke, "ms_per_step": ms_pipe / Ke, "in_flight": 2,
                         "host_memory": "pinned",
                         "repeats_ms_per_step": [w / Ke for w in pipe_windows]}
    except Exception as exc:
        e2e_pipelined = {"error": repr(exc)}
    # The same call from pageable host memory (what a caller's Vec hands over): the library
    # stages it through its own pinned buffer.
    try:
        xp = [torch.rand((BATCH, 1, 28, 28)) for _ in range(4)]
        op = torch.empty((BATCH, 10), dtype=torch.float32)
        for i in range(W):
            model.infer(xp[i % 4], op)
        Kp = max(min(K, 500), 10)
        pw = timed_windows(lambda i: model.infer(xp[i % 4], op), Kp)
        msp = float(np.median(pw))
        e2e_pageable = {"value": world * BATCH * Kp / (msp * 1e-3), "unit": UNIT, "steps": Kp,
                        "ms_per_step": msp / Kp, "host_memory": "pageable"}
    except Exception as exc:
        e2e_pageable = {"error": repr(exc)}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
        # the published figure has its transfers inside the timed region: compare like with like
        "vs_baseline": e2e["value"] / PUBLISHED_IMG_PER_S,
        "vs_baseline_device_resident": value / PUBLISHED_IMG_PER_S,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "global_batch": BATCH * world, "parallelism": f"dp{world} (batch shards, no collective)",
                   "l2": f"inputs rotate over {ROTATE} batches (200 MB > 126 MB L2)",
                   "timing": f"median of {REPEATS} windows of K steps, each window the max over ranks",
                   "peaks": peaks["source"]},
        "repeats_ms_per_step": [w / K for w in windows],
        "e2e": e2e, "e2e_pipelined": e2e_pipelined, "e2e_pageable": e2e_pageable,
        "gpu_launches": int(launches),
    }

    # configs[4a]: 65536 images sharded evenly by batch, no collective (strong scaling: the
    # total is fixed, each rank runs 65536 / world images in one launch).
    try:
        n_shard = 65536 // world
        xl = torch.rand((n_shard, 1, 28, 28), generator=gen, device=dev.torch_device)
        ol = dev.empty((n_shard, 10), torch.float32)
        for i in range(3):
            model.forward_device(xl, ol)
        sw = timed_windows(lambda i: model.forward_device(xl, ol), 5)
        ms_shard = float(np.median(sw)) / 5
        line["infer_sharded_65536"] = {
            "img_per_s": 65536 / (ms_shard * 1e-3), "ms_per_pass": ms_shard,
            "images_per_gpu": n_shard, "scaling": "strong",
            "tflops": 65536 * FLOPS_PER_IMG / ms_shard * 1e-9}
        line["infer_sharded_65536_img_per_s"] = line["infer_sharded_65536"]["img_per_s"]
        del xl, ol
    except Exception as exc:
        line["infer_sharded_65536_error"] = repr(exc)

    # configs[4b]: data-parallel training, 100 images per GPU, one sum-all-reduce of the
    # flat gradient bucket per step, 1/world folded into the update.  Runs on every rank.
    try:
        line["train_dp"] = train_data_parallel(torch, ag, dp, dev, rank, world, barrier,
                                               max_over_ranks)
        line["train_dp_ms_per_step"] = line["train_dp"]["ms_per_step"]
        line["train_dp_img_per_s"] = line["train_dp"]["img_per_s"]
    except Exception as exc:
        line["train_dp_error"] = repr(exc)
    if rank == 0:
        line["roofline"], line["stages"] = lenet5_roofline(torch, ag, dev, model, xs, K, peaks)
        if not args.quick:
            for key, fn in (("gemm", lambda: gemm_sweep(torch, ag, dev, peaks, sampler)),
                            ("extras", lambda: extras(torch, ag, dev, peaks, world))):
                try:
                    res = fn()
                    if key == "gemm":
                        line["gemm"], line["gemm_roofline"] = res
                    else:
                        line[key] = res
                except Exception as exc:  # the headline numbers above are still reported
                    line[key + "_error"] = repr(exc)
    barrier()
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        line["clocks"] = sampler.stop()
        # The CPU baseline runs last, on rank 0, once the other ranks have left: they would
        # otherwise compete for the host cores it is timed on.
        if world > 1:
            time.sleep(2.0)
        secs = 3.0 if args.quick else 12.0
        rate, cores, n, dt = cpu_forward_rate(secs)
        line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"median window of {n} forward passes of 1000 images "
                                          f"in {dt:.1f} s (windows of 20)"}
        if not args.quick:
            try:
                sps, cores, n, dt = cpu_train_rate(4.0)
                line["cpu_baseline_train"] = {
                    "value": sps * 100, "unit": "img/s", "ms_per_step": 1e3 / sps, "cores": cores,
                    "kind": "port", "sample": f"{n} training steps of 100 images in {dt:.1f} s "
                                              "(benchmark configuration 2)"}
            except Exception as exc:
                line["cpu_baseline_train_error"] = repr(exc)
        print(json.dumps(line), flush=True)


def train_data_parallel(torch, ag, dp, dev, rank, world, barrier, max_over_ranks):
    """configs[4b]: forward / backward on 100 images per GPU, then the data-parallel tail two
    ways: the fused kernel (one-shot all-reduce over NVLink + 1/world + SGD update) and, for
    comparison, an NCCL all-reduce of the bucket followed by the update kernel."""
    comm = dp.Comm.from_torch_distributed(dev) if world > 1 else dp.Comm.single_process([dev])
    gen = torch.Generator(device=dev.torch_device).manual_seed(7000 + rank)
    x = torch.rand((100, 1, 28, 28), generator=gen, device=dev.torch_device)
    t = torch.randint(0, 10, (100,), generator=gen, device=dev.torch_device, dtype=torch.uint8)
    out = {"global_batch": 100 * world}

    def measure(fused):
        m = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)   # same seed: replicated parameters
        m.set_sgd(None)
        m.set_grad_scale(1.0 / world)
        n_elems = [0]

        def step(i):
            # everything is enqueued back to back on one stream; the host reads the loss once,
            # at the end of the step
            _, ptr, length = m.train_forward_backward(x, t, sync=False)
            n_elems[0] = length
            if fused:
                comm.allreduce_update(m, 0.01)
            else:
                if world > 1:
                    comm.allreduce_bucket(ptr, length, torch.float32)
                m.apply_update(0.01)
            m.last_loss()

        for i in range(5):
            step(i)
        windows = []
        for _ in range(5):
            barrier()
            windows.append(max_over_ranks(event_time_ms(torch, step, 40, dev.stream)) / 40)
        barrier()
        m.close()
        return float(np.median(windows)), n_elems[0]

    try:
        ms_plain, n = measure(False)
        out["nccl_then_update"] = {"ms_per_step": ms_plain, "img_per_s": 100 * world / ms_plain * 1e3}
    except Exception as exc:
        out["nccl_then_update_error"] = repr(exc)
    use_fused = comm.fused_available
    ms, n = measure(use_fused)
    out.update({"ms_per_step": ms, "img_per_s": 100 * world / ms * 1e3, "allreduce_elements": int(n),
                "collective": ("fused one-shot all-reduce over NVLink + update (one kernel)"
                               if use_fused else "nccl all_reduce(sum)") if world > 1 else "none"})
    comm.close()
    return out


def graph_time_us(torch, dev, fns, reps=10):
    """Device time per call of the launches in `fns`, measured by replaying a CUDA graph of
    them (no host launch gaps between the kernels), CUDA events on the launching stream."""
    for fn in fns[:3]:
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=dev.stream):
        for fn in fns:
            fn()
    g.replay()
    torch.cuda.synchronize()
    ms = event_time_ms(torch, lambda i: g.replay(), reps, dev.stream)
    return ms / (reps * len(fns)) * 1e3


# The reference's published figure for this metric: LeNet5 inference, batch 1000, f32, on its
# device path (README.md:133 of the reference: 4.65 ms per batch on a GTX 1060 Max-Q through
# Vulkan; host-to-device transfer and logits read-back inside the timed region).
PUBLISHED_IMG_PER_S = 1000 / 4.65e-3


def lenet5_roofline(torch, ag, dev, model, xs, K, peaks):
    """Times the three kernels of the f32 inference step alone (graph replay, inputs rotating
    through HBM) and reports the dominant one against the measured HBM peak; the FP32-pipe
    view is added because these kernels are FFMA / latency bound, which the hbm / tensor
    choice cannot express."""
    shapes = [(6, 1, 5, 5), (16, 6, 5, 5), (256, 128), (128, 84), (84, 10), (10,)]
    P = [dev.tensor(model.get_parameter(i).reshape(shp)) for i, shp in enumerate(shapes)]
    B = BATCH
    s = 4
    p1 = dev.conv2_relu_max_pool2(xs[0], P[0])
    p1s = [p1 + 0.001 * i for i in range(16)]
    p2 = dev.conv2_relu_max_pool2(p1, P[1])
    fs = [(p2 + 0.001 * i).reshape(B, 256) for i in range(16)]
    stages = {}

    def add(name, fns, flops, bytes_):
        us = graph_time_us(torch, dev, fns)
        stages[name] = {"us": us, "gflops": flops / us * 1e-3, "gbs": bytes_ / us * 1e-3,
                        "alg_bytes": bytes_, "alg_flops": flops}

    add("conv1+relu+pool (conv2_direct_kernel<5,5>, 1->6 ch, 28x28)",
        [lambda i=i: dev.conv2_relu_max_pool2(xs[i], P[0]) for i in range(32)],
        2 * B * 576 * 25 * 6, (B * 784 + 150 + B * 6 * 144) * s)
    add("conv2+relu+pool (conv2_direct_kernel<5,5>, 6->16 ch, 12x12)",
        [lambda i=i: dev.conv2_relu_max_pool2(p1s[i % 16], P[1]) for i in range(32)],
        2 * B * 64 * 150 * 16, (B * 6 * 144 + 2400 + B * 256) * s)
    add("dense chain 256-128-84-10 (dense_chain_kernel)",
        [lambda i=i: dev.dense_chain_forward(fs[i % 16], [P[2], P[3], P[4]], [None, None, P[5]],
                                             [True, True, False]) for i in range(32)],
        2 * B * (256 * 128 + 128 * 84 + 84 * 10), (B * 256 + 46920 - 2550 + B * 10) * s)
    total_flops = sum(v["alg_flops"] for v in stages.values())
    layered_us = sum(v["us"] for v in stages.values())
    convs = [(P[0], None, True, (2, 2)), (P[1], None, True, (2, 2))]
    add("whole network (lenet_chain_kernel: 2 x conv+relu+pool, flatten, dense 256-128-84-10)",
        [lambda i=i: dev.conv_dense_chain_forward(xs[i], convs, [P[2], P[3], P[4]],
                                                  [None, None, P[5]], [True, True, False])
         for i in range(32)],
        total_flops, (B * 784 + 44426 + B * 10) * s)
    # The step runs the whole-network kernel; the three layer kernels above are what it
    # replaces (kept for comparison: their sum is the layer-by-layer step).
    name = next(k for k in stages if k.startswith("whole network"))
    st = stages[name]
    st["layer_by_layer_us"] = layered_us
    fp32_peak = 148 * 128 * 2 * 1.965e-3  # TFLOP/s at the maximum SM clock
    # The binding bound of this kernel is the FP32 (FFMA) pipe: 568,720 flop per image against
    # 3,176 bytes per image puts the HBM bound 15 times further away.  The file of measured
    # peaks holds no FP32 figure, so this peak is computed from the SM count and the maximum
    # SM clock; the HBM view (measured peak) is kept in the `hbm` sub-object.
    roof = {"bound": "fp32_pipe", "kernel": name, "achieved": st["gflops"] * 1e-3,
            "peak": fp32_peak, "unit": "TFLOP/s", "frac": st["gflops"] * 1e-3 / fp32_peak,
            "peak_source": "computed: 148 SMs x 128 lanes x 2 flop x 1.965 GHz (max SM clock)",
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch at batch 1000, from the
            # ncu capture of this kernel
            "traffic": 3405568 if B == 1000 else None,
            "us_per_launch": st["us"], "algorithmic_flops_per_launch": st["alg_flops"],
            "hbm": {"achieved_gbs": st["gbs"], "peak_gbs": peaks["hbm_gbs"],
                    "frac": st["gbs"] / peaks["hbm_gbs"], "peak_source": peaks["source"],
                    "algorithmic_bytes_per_launch": st["alg_bytes"]}}
    return roof, stages


def gemm_sweep(torch, ag, dev, peaks, sampler):
    """configs[1]: square dot products, f32 (SIMT) and bf16 (tcgen05), NN / TN / NT."""
    results = []
    roof = None
    for dtype, name in [(torch.bfloat16, "bf16"), (torch.float32, "f32")]:
        for n in [256, 1024, 4096, 8192]:
            layouts = ["nn", "tn", "nt"] if n == 4096 else ["nn"]
            a = (torch.rand((n, n), device=dev.torch_device) * 2 - 1).to(dtype)
            b = (torch.rand((n, n), device=dev.torch_device) * 2 - 1).to(dtype)
            c = dev.empty((n, n), dtype)
            for layout in layouts:
                av = a.t() if layout[0] == "t" else a
                bv = b.t() if layout[1] == "t" else b
                iters = 20 if n <= 4096 else (10 if name == "bf16" else 4)
                fn = lambda i: dev.gemm(1.0, av, bv, 0.0, c)
                for i in range(3):
                    fn(i)
                t0 = time.time()
                if n <= 1024:
                    # a few microseconds of device work per call: host dispatch (ctypes, two
                    # tensor-map encodes) would be what is timed, so 20 calls are replayed
                    # from a CUDA graph and the device time per call is reported
                    ms = graph_time_us(torch, dev, [lambda: dev.gemm(1.0, av, bv, 0.0, c)] * 20) * 1e-3
                else:
                    ms = event_time_ms(torch, fn, iters, dev.stream) / iters
                if sampler:
                    sampler.mark(t0, time.time())
                tf = 2.0 * n ** 3 / ms * 1e-9
                entry = {"dtype": name, "n": n, "layout": layout, "ms": ms, "tflops": tf,
                         "timing": "graph replay" if n <= 1024 else "stream launches"}
                if name == "bf16":
                    entry["frac_of_measured_bf16_peak"] = tf / peaks["bf16_tflops"]
                else:
                    entry["frac_of_fp32_pipe_peak_at_max_clock"] = tf / (148 * 128 * 2 * 1.965e-3)
                results.append(entry)
                if name == "bf16" and n == 4096 and layout == "nn":
                    roof = {"bound": "tensor", "kernel": "gemm_bf16_tc2_kernel (tcgen05, cta_group::2), 4096^3 nn",
                            "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                            "frac": tf / peaks["bf16_tflops"],
                            # dram bytes of one launch from the ncu capture summarised in
                            # ncu capture of this kernel (A + B + C = 100.7 MB algorithmic)
                            "traffic": 90.0e6,
                            "peak_source": peaks["source"] + " (burst: kernel timed alone)"}
            del a, b, c
    return results, roof


def extras(torch, ag, dev, peaks, world):
    """bf16 inference, the configs[2] training step, u8 input pipeline, the wide conv stack."""
    out = {}
    # bf16 LeNet5 inference, batch 1000
    mb = ag.Model(dev, ag.LENET5_SPEC, torch.bfloat16, seed=2000)
    xb = torch.rand((ROTATE, BATCH, 1, 28, 28), device=dev.torch_device).to(torch.bfloat16)
    ob = dev.empty((BATCH, 10), torch.bfloat16)
    fn = lambda i: mb.forward_device(xb[i % ROTATE], ob)
    for i in range(5):
        fn(i)
    ms = event_time_ms(torch, fn, 200, dev.stream) / 200
    out["lenet5_infer_bf16_bs1000"] = {"img_per_s": BATCH / ms * 1e3, "ms": ms}
    mb.close()
    del xb
    m = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    # configs[2]: training step, batch 100, host buffers, plain SGD lr 0.01
    xt = torch.rand((100, 1, 28, 28)).pin_memory()
    tt = torch.randint(0, 10, (100,), dtype=torch.uint8).pin_memory()
    for i in range(5):
        m.train_step(xt, tt, 0.01)
    ms = event_time_ms(torch, lambda i: m.train_step(xt, tt, 0.01), 100, dev.stream) / 100
    out["lenet5_train_f32_bs100"] = {"ms_per_step": ms, "img_per_s": 100 / ms * 1e3}
    m.close()
    # The reference's own input pipeline (u8 images scaled by 1/255 on the device,
    # examples/neural-network-mnist/src/main.rs:236-243) end to end: pinned u8 images in, logits out.
    mi = ag.Model(dev, ag.LENET5_SPEC, torch.float32, seed=2000)
    x8 = [torch.randint(0, 256, (BATCH, 1, 28, 28), dtype=torch.uint8).pin_memory() for _ in range(4)]
    o8 = [torch.empty((BATCH, 10), dtype=torch.float32).pin_memory() for _ in range(4)]
    for i in range(8):
        mi.infer_u8(x8[i % 4], out_host=o8[i % 4])
    t0 = time.perf_counter()
    n8 = 500
    for i in range(n8):
        mi.infer_u8(x8[i % 4], out_host=o8[i % 4])
    ms = (time.perf_counter() - t0) * 1e3 / n8
    out["lenet5_infer_f32_bs1000_e2e_u8_images"] = {
        "img_per_s": BATCH / ms * 1e3, "ms_per_step": ms, "h2d_bytes_per_step": BATCH * 784,
        "d2h_bytes_per_step": BATCH * 40, "timing": "host wall clock over blocking calls"}
    mi.close()
    if world == 1:
        # configs[3]: the wider conv stack, bf16, batch 256: forward + backward + SGD update.
        # FLOPs of one step: 2 * MACs of (conv1, conv2, dense1, dense2), forward once and
        # backward twice (input and weight gradients; conv1 has no input gradient).
        mw = ag.Model(dev, ag.WIDE_STACK_SPEC, torch.bfloat16, seed=2000)
        xw = torch.randn((256, 3, 64, 64)).to(torch.bfloat16).pin_memory()
        tw = torch.randint(0, 10, (256,), dtype=torch.uint8).pin_memory()
        for i in range(4):
            mw.train_step(xw, tw, 0.01)
        ms = event_time_ms(torch, lambda i: mw.train_step(xw, tw, 0.01), 20, dev.stream) / 20
        macs = 256 * (64 * 62 * 62 * 27 * 2 + 128 * 29 * 29 * 576 * 3 + 25088 * 512 * 3 + 512 * 10 * 3)
        out["wide_stack_train_bf16_bs256"] = {"ms_per_step": ms, "img_per_s": 256 / ms * 1e3,
                                              "tflops": 2.0 * macs / ms * 1e-9}
        mw.close()
        # its second convolution alone (64 -> 128 channels, 3x3, 31x31 images) on tcgen05:
        # forward with bias + ReLU, input gradient, weight gradient
        x = torch.randn((256, 64, 31, 31), device=dev.torch_device).to(torch.bfloat16)
        w = (torch.rand((128, 64, 3, 3), device=dev.torch_device) * 0.1 - 0.05).to(torch.bfloat16)
        bias = torch.zeros((128,), device=dev.torch_device).to(torch.bfloat16)
        dy = torch.randn((256, 128, 29, 29), device=dev.torch_device).to(torch.bfloat16)
        gf = 2.0 * 256 * 128 * 29 * 29 * 64 * 9 * 1e-9
        conv = {}
        for name, fn in [("forward", lambda i: dev.conv2_forward(x, w, bias=bias, relu=True)),
                         ("backward_input", lambda i: dev.conv2_backward_input(w, dy, (31, 31))),
                         ("backward_weight", lambda i: dev.conv2_backward_weight(x, dy, (3, 3)))]:
            for i in range(3):
                fn(i)
            ms = event_time_ms(torch, fn, 20, dev.stream) / 20
            conv[name] = {"ms": ms, "tflops": gf / ms,
                          "frac_of_measured_bf16_peak": gf / ms / peaks["bf16_tflops"]}
        out["conv2_bf16_tcgen05_64to128_3x3_bs256"] = conv
    return out


def run_probe(args):
    """Runs one kernel family alone, for profiler captures:
    gemm:<f32|bf16>:<n>:<nn|tn|nt|tt>, infer:<f32|bf16>:<batch>, train:<f32|bf16>:<batch>,
    wide:<f32|bf16>:<batch> (training step of the wider conv stack), conv:bf16:<batch>
    (its second convolution alone: forward, input gradient and weight gradient),
    op:<f32|bf16>:<relu|relu_backward|scaled_add|sgd_momentum|max_pool2|max_pool2_backward|
    bias_grad>:<elements>."""
    import torch
    import autograph_b200 as ag
    dev = ag.Device(0)
    parts = args.probe.split(":")
    dtype = {"f32": torch.float32, "bf16": torch.bfloat16}[parts[1]]
    K, W = args.steps, args.warmup
    if parts[0] == "op":
        # op:<dtype>:<name>:<elements>  memory-bound kernels on a large array
        name, n = parts[2], int(parts[3])
        es = 4 if dtype == torch.float32 else 2
        a = (torch.rand((n,), device=dev.torch_device) - 0.5).to(dtype)
        b = (torch.rand((n,), device=dev.torch_device) - 0.5).to(dtype)
        c = torch.zeros((n,), device=dev.torch_device, dtype=dtype)
        if name == "relu":
            fn, nbytes = (lambda i: dev.relu(a, inplace=False)), 2 * n * es
        elif name == "relu_backward":
            fn, nbytes = (lambda i: dev.relu_backward(a, b)), 3 * n * es
        elif name == "scaled_add":
            fn, nbytes = (lambda i: dev.scaled_add(c, 0.5, a)), 3 * n * es
        elif name == "sgd_momentum":
            fn, nbytes = (lambda i: dev.sgd_update_momentum(c, a, b, 0.01, 0.01)), 5 * n * es
        elif name == "max_pool2":
            x4 = a[: (n // 4096) * 4096].reshape(-1, 16, 16, 16)
            fn, nbytes = (lambda i: dev.max_pool2(x4)), x4.numel() * es * 5 // 4
        elif name == "max_pool2_backward":
            x4 = a[: (n // 4096) * 4096].reshape(-1, 16, 16, 16)
            dy = b[: x4.numel() // 4].reshape(-1, 16, 8, 8)
            dx = x4.clone()
            fn = lambda i: dev.max_pool2_backward_inplace(dx, dy)
            nbytes = x4.numel() * es * 9 // 4
        elif name == "bias_grad":
            x2 = a[: (n // 512) * 512].reshape(-1, 512)
            fn, nbytes = (lambda i: dev.bias_grad(x2)), x2.numel() * es
        else:
            raise SystemExit(f"unknown op {name}")
        work, unit = nbytes * 1e-9, "GB/s"
    elif parts[0] == "gemm":
        n, layout = int(parts[2]), parts[3]
        a = (torch.rand((n, n), device=dev.torch_device) * 2 - 1).to(dtype)
        b = (torch.rand((n, n), device=dev.torch_device) * 2 - 1).to(dtype)
        c = dev.empty((n, n), dtype)
        av = a.t() if layout[0] == "t" else a
        bv = b.t() if layout[1] == "t" else b
        fn = lambda i: dev.gemm(1.0, av, bv, 0.0, c)
        work, unit = 2.0 * n ** 3 * 1e-12, "TFLOP/s"
    elif parts[0] == "conv":
        bs = int(parts[2])
        x = torch.randn((bs, 64, 31, 31), device=dev.torch_device).to(dtype)
        w = (torch.rand((128, 64, 3, 3), device=dev.torch_device) * 0.1 - 0.05).to(dtype)
        bias = torch.zeros((128,), device=dev.torch_device).to(dtype)
        dy = torch.randn((bs, 128, 29, 29), device=dev.torch_device).to(dtype)
        def fn(i):
            dev.conv2_forward(x, w, bias=bias, relu=True)
            dev.conv2_backward_input(w, dy, (31, 31))
            dev.conv2_backward_weight(x, dy, (3, 3))
        work, unit = 3 * 2.0 * bs * 128 * 29 * 29 * 64 * 9 * 1e-12, "TFLOP/s"
    elif parts[0] == "wide":
        bs = int(parts[2])
        model = ag.Model(dev, ag.WIDE_STACK_SPEC, dtype, seed=2000)
        xh = torch.randn((bs, 3, 64, 64)).to(dtype).pin_memory()
        th = torch.randint(0, 10, (bs,), dtype=torch.uint8).pin_memory()
        fn = lambda i: model.train_step(xh, th, 0.01)
        work, unit = float(bs), "img/s"
    else:
        bs = int(parts[2])
        model = ag.Model(dev, ag.LENET5_SPEC, dtype, seed=2000)
        if parts[0] == "infer":
            x = torch.rand((bs, 1, 28, 28), device=dev.torch_device).to(dtype)
            out = dev.empty((bs, 10), dtype)
            fn = lambda i: model.forward_device(x, out)
        else:
            xh = torch.rand((bs, 1, 28, 28)).to(dtype).pin_memory()
            th = torch.randint(0, 10, (bs,), dtype=torch.uint8).pin_memory()
            fn = lambda i: model.train_step(xh, th, 0.01)
        work, unit = float(bs), "img/s"
    for i in range(W):
        fn(i)
    torch.cuda.synchronize()
    ms = event_time_ms(torch, fn, K, dev.stream) / K
    print(json.dumps({"probe": args.probe, "ms": ms, "rate": work / (ms * 1e-3), "unit": unit}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--quick", action="store_true", help="skip the GEMM sweep and extras")
    ap.add_argument("--probe", default=None,
                    help="run one kernel family alone (for profiler captures), e.g. gemm:bf16:4096:nn")
    args = ap.parse_args()
    if args.probe:
        run_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
