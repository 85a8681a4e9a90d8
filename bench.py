#!/usr/bin/env python
"""Benchmark of the convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload all|c5|c5i8|c1|c2|c3|c3s|c4|dw|...]
                    [--impl reference]

Default (--workload all): ONE JSON line whose headline is c5 -- the VGG-16 convolution stack, fp32
Winograd F(4x4,3x3), global batch 256 -- and whose `per_config` object holds every other benchmark
configuration (c1 FP32 Winograd VGG conv3_2, c2 INT8 1x1, c3 INT8 3x3 stride 2, c4 INT8 Winograd,
c5i8 the stack with INT8 direct kernels, dw INT8 depthwise), each with its own value, ms_per_step,
e2e, roofline and parity.  `--workload X` runs one workload alone (profiling, experiments).

Partitioning: the minibatch is split.  With N GPUs rank r owns images [r*B/N, (r+1)*B/N) of every
configuration's global batch B (c5: 256/N images per GPU in chunks of 64, of 32 from 4 GPUs up), weights are replicated,
nothing is exchanged on the data path, so `scaling` is "strong" (total work fixed).

What the numbers are:
  value / ms_per_step  inputs resident in HBM; the K steps are captured in a CUDA graph and replayed
                       between CUDA events on the launching stream; max over ranks.  Every timed
                       region lasts at least ~0.2 s (short steps are replayed more often; `timing`
                       gives the number of replays and the median / min / max per replay).  A ring of
                       buffer sets larger than L2 is walked (the stack streams > 1 GB per chunk).
  e2e                  the same work through the library call a user makes (elx_conv; for the stack
                       elb_stack_execute) with pinned HOST tensors: host->device and device->host
                       copies inside every step.
  roofline             whole-convolution op count / time against min(P_tensor, AI * HBM bandwidth):
                       AI = op count / algorithmic bytes (input + weights as passed + output
                       [+ residual]); HBM bandwidth = the measured copy bandwidth; P_tensor from this
                       repository's own tcgen05 issue-rate measurement (MAC per clock per SM) at the
                       GPU's maximum SM clock.  `kernels` lists every kernel of a step with its time.
  parity               the output of the last timed step against the reference's own CPU library
                       (oracle/_ref; the C restatement where AVX-512 VNNI is missing): bit-exact for
                       INT8 direct / 1x1 / depthwise, rel-L2 <= 1e-5 for Winograd.
  cpu_baseline         the reference's CPU library timed on this host's cores on a bounded sample
                       (rank 0, N=1 only).
Reference arm (--impl reference): the reference's CPU implementation only, same metric / config.
"""
from __future__ import annotations

import argparse
import dataclasses
import importlib
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from stackutil import (build_stack, oracle_fn, per_layer_parity, stack_layer_outputs,   # noqa: E402
                       stack_reference_chain, vgg_calibrate, vgg_input, vgg_layer_case, vgg_layers)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "sm_max_mhz": 1965.0}
NUM_SMS = 148
# tcgen05 issue rates measured with a one-thread back-to-back MMA loop on fixed operands (M = 128,
# N = 256), multiply-accumulates per clock per SM: the tensor-core ceilings used below.
MAC_PER_CLK_SM = {"i8": 6537.0, "tf32": 1887.0}
MIN_TIMED_S = 0.25
PKG = "deep-learning-math-kernel-research_b200"

WORKLOADS = {
    "c1": dict(metric="effective_conv_tflops_fp32_winograd", unit="TFLOP/s", dtype="tf32x3(fp32)", batch=64,
               desc="FP32 Winograd F(4x4,3x3) VGG-16 conv3_2 N=64 C=K=256 56x56 s1 p1 bias+ReLU nChw16c"),
    "c2": dict(metric="effective_conv_tops_int8", unit="TOP/s", dtype="u8", batch=64,
               desc="INT8 u8s8 1x1 ResNet-50 res4 reduce N=64 C=1024 K=256 14x14 bias+ReLU u8 out nChw16c"),
    "c3": dict(metric="effective_conv_tops_int8", unit="TOP/s", dtype="u8", batch=64,
               desc="INT8 u8s8 3x3 stride 2 pad 1 N=64 C=128 K=256 56x56->28x28 bias+ReLU u8 out nChw16c"),
    "c3s": dict(metric="effective_conv_tops_int8", unit="TOP/s", dtype="u8", batch=64,
                desc="INT8 u8s8 3x3 stride 2 pad 1 N=64 C=128 K=256 56x56->28x28 bias+ReLU+sum (u8 residual in the output "
                     "tensor, sum scale 1.0) u8 out nChw16c; the reference's KxK path ignores the sum flag"),
    "c4": dict(metric="effective_conv_tops_int8_winograd", unit="TOP/s", dtype="u8", batch=128,
               desc="INT8 Winograd F(4x4,3x3) N=128 C=K=512 28x28 s1 p1 f32 out nChw16c"),
    "c1t4": dict(metric="effective_conv_tflops_fp32_winograd_f2x2", unit="TFLOP/s", dtype="tf32x3(fp32)", batch=64,
                 desc="FP32 Winograd F(2x2,3x3) (tile_size 4) VGG-16 conv3_2 N=64 C=K=256 56x56 s1 p1 bias+ReLU nChw16c"),
    "c4t4": dict(metric="effective_conv_tops_int8_winograd_f2x2", unit="TOP/s", dtype="u8", batch=128,
                 desc="INT8 Winograd F(2x2,3x3) (tile_size 4) N=128 C=K=512 28x28 s1 p1 f32 out nChw16c"),
    "v12": dict(metric="effective_conv_tflops_fp32_winograd", unit="TFLOP/s", dtype="tf32x3(fp32)", batch=32,
                desc="FP32 Winograd F(4x4,3x3) VGG-16 conv1_2 N=32 C=K=64 224x224 s1 p1 bias+ReLU nChw16c"),
    "c2f": dict(metric="effective_conv_tflops_fp32_direct_1x1", unit="TFLOP/s", dtype="tf32x3(fp32)", batch=64,
                desc="FP32 direct 1x1 ResNet-50 res4 reduce N=64 C=1024 K=256 14x14 bias+ReLU nChw16c"),
    "c3f": dict(metric="effective_conv_tflops_fp32_direct", unit="TFLOP/s", dtype="tf32x3(fp32)", batch=64,
                desc="FP32 direct 3x3 stride 2 pad 1 N=64 C=128 K=256 56x56->28x28 bias+ReLU nChw16c"),
    "dw": dict(metric="effective_conv_tops_int8_depthwise", unit="TOP/s", dtype="u8", batch=64,
               desc="INT8 depthwise 3x3 MobileNet-v1 Conv2d_3 N=64 C=128 56x56 s1 p1 bias+ReLU u8 out nChw16c T=14"),
    "c5": dict(metric="effective_conv_tflops_fp32_winograd_vgg16_stack", unit="TFLOP/s", dtype="tf32x3(fp32)", batch=256,
               desc="VGG-16 conv stack, 13 layers 3x3 p1, 224x224 input, fp32 Winograd F(4x4,3x3), global batch 256 in "
                    "chunks (see chunk_images), stride-2 subsample between stages, bias+ReLU; the network input is the "
                    "nchw image (3 planes), activations and weights nChw16c / OIhw16i16o"),
    "c5i8": dict(metric="effective_conv_tops_int8_vgg16_stack", unit="TOP/s", dtype="u8", batch=256,
                 desc="VGG-16 conv stack, 13 layers 3x3 p1, 224x224 input, INT8 u8s8 direct, u8 between layers, global "
                      "batch 256 in chunks (see chunk_images), stride-2 subsample between stages, bias+ReLU; the network input is "
                      "the nchw u8 image (3 planes), activations and weights nChw16c / OIhw16i16o"),
}
HEADLINE = "c5"
PER_CONFIG = ["c1", "c2", "c3", "c4", "c5i8", "dw"]
# published number for exactly this metric/config (2 x Xeon 8180, the reference's tuned script comment)
PUBLISHED = {"c1": 11.2}
# Images per chunk of a stack (one chunk = one pass of the chain over that many images): 64 where a
# GPU's share of the global batch is at least two such chunks (end to end, the copy in of one chunk
# hides behind the chain of the previous one), i.e. at 1 and 2 GPUs for 256 images; 32 otherwise.  Measured
# on one B200 (fp32 stack, 256 images): 25.7 ms per step with chunks of 32, 25.0 ms with 64 (the
# 14x14 and 28x28 layers fill their last wave better and there are half the launches); 24.7 ms with
# 128, whose first copy in is too long to hide end to end (25.96 against 25.3 ms).
STACK_CHUNK = 64

# DRAM bytes (read + written) per step from the ncu captures summarised under profiles/ (sum over
# the kernels of a step, full-size workloads; c5: captured at 8 images and scaled to the 256 of a
# step -- the traffic of every kernel of the stack grows in proportion to the images).
NCU_TRAFFIC = {"c1": 2139.6e6, "c2": 13.15e6, "c3": 26.03e6, "c3s": 38.88e6, "c4": 1268.9e6, "dw": 25.72e6, "c2f": 53.5e6,
               "c5": 94.9e9}


# ------------------------------------------------------------------------------------ helpers
def bind_to_gpu_cpus(index: int):
    """Several ranks on one box: keep this process (and therefore the pages of the pinned host buffers
    it is about to allocate, and the threads that feed its copies) on the CPU cores NVML lists as
    local to its GPU.  Process affinity only -- nothing about the GPU changes.  Returns the number of
    cores bound to, or None when NVML or the affinity call is unavailable."""
    try:
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML (read-only) while the GPU is under load."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.active = False

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksEventReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksEventReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksEventReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     nv.nvmlClocksEventReasonSwPowerCap: "sw_power_cap"}
            while not self._stop_evt.is_set():
                if self.active:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                time.sleep(0.005)
        except Exception as e:  # NVML missing: report that instead of failing the bench
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)

    def reset(self):
        self.samples, self.reasons = [], set(r for r in self.reasons if r.startswith("nvml_unavailable"))

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def max_over_ranks(values, dist, device="cuda"):
    """Element-wise maximum of per-rank timings (the slowest rank defines the step time)."""
    if dist is None:
        return [float(v) for v in values]
    import torch
    tt = torch.tensor(list(values), device=device, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    return [float(v) for v in tt]


def split_batch(global_batch: int, world: int, rank: int):
    """Images [first, first + count) of the global minibatch that rank `rank` of `world` owns."""
    first = global_batch * rank // world
    return first, global_batch * (rank + 1) // world - first


def stack_chunk_images(global_batch: int, world: int) -> int:
    """Images per chunk of a stack on one GPU of `world` (see STACK_CHUNK): 64 where the GPU's share
    holds at least two such chunks, else 32 (or the whole share when that is smaller), halved until it
    divides the share."""
    per_gpu = max(1, global_batch // world)
    n = STACK_CHUNK if per_gpu >= 2 * STACK_CHUNK else min(STACK_CHUNK // 2, per_gpu)
    while n > 1 and per_gpu % n:
        n //= 2
    return n


def throughput(ops_global: float, ms_per_step: float) -> float:
    """Whole-job T(FL)OP/s: the op count of the GLOBAL batch over the step time of the slowest rank."""
    return ops_global / (ms_per_step * 1e-3) / 1e12


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d.setdefault("sm_max_mhz", FALLBACK_PEAKS["sm_max_mhz"])
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def tensor_peak(kind: str, peaks) -> float:
    """Dense tensor-core ceiling in T(FL)OP/s: 2 * MAC/clk/SM * SMs * max SM clock; fp32 runs as
    3xTF32 (three tf32 MMAs per product), so its ceiling is a third of the tf32 one."""
    raw = 2.0 * MAC_PER_CLK_SM["i8" if kind == "i8" else "tf32"] * NUM_SMS * peaks["sm_max_mhz"] * 1e6 / 1e12
    return raw / 3.0 if kind == "f32" else raw


def layer_roofline(case, alg_bytes: float, gemm_ops: float | None, ops: float, peaks):
    """Attainable T(FL)OP/s of one convolution in direct-conv op units: min(tensor, AI * HBM).
    gemm_ops = multiply-add work the tensor cores actually do (Winograd: the transform-domain GEMMs;
    direct: ops itself); the tensor ceiling is scaled by ops / gemm_ops."""
    kind = "f32" if case.types == "fp32" else "i8"
    if case.g > 1:
        p_t = float("inf")          # depthwise runs on CUDA cores: ~9 op/B, nowhere near a compute ceiling
    else:
        p_t = tensor_peak(kind, peaks) * (ops / (gemm_ops or ops))
    ai = ops / alg_bytes
    p_m = ai * peaks["hbm_gbs"] * 1e9 / 1e12
    return {"p_tensor": None if math.isinf(p_t) else p_t, "p_hbm": p_m, "attainable": min(p_t, p_m),
            "bound": "tensor" if p_t < p_m else "hbm", "ai": ai}


def algorithmic_bytes(case, t) -> int:
    """input + weights as the user passes them + output (+ residual)."""
    import numpy as np
    out_b = int(np.prod((case.n, (case.oc + 15) // 16 * 16, case.oh, case.ow))) * np.dtype(case.out_dtype).itemsize
    b = t["input"].nbytes + (t["weights"].nbytes - 64 * 4) + out_b
    if case.sum:
        b += out_b
    return b


def gemm_ops_of(case) -> float:
    import refutil as R
    if case.algo == "wino":
        return 2.0 * R.wino_edge(case) ** 2 * R.wino_tiles(case) * R.alignup(case.ic) * R.alignup(case.oc)
    return float(case.cal_ops())


def timed_replays(graph, stream, replays_per_group, est_ms_per_replay, dist, min_s=MIN_TIMED_S):
    """The timed region: G groups of `replays_per_group` replays of `graph`, back to back on `stream`
    between CUDA events, with G chosen so that the region lasts at least min_s (and gives three
    groups for a spread where that is cheap).  Barrier + synchronize on both sides.
    Returns (total_ms, [ms of each group])."""
    import torch
    group_ms = max(replays_per_group * est_ms_per_replay, 1e-4)
    groups = max(1, math.ceil(min_s * 1e3 / group_ms))
    if groups < 3 and 3 * group_ms <= 1500.0:
        groups = 3
    groups = min(groups, 2000)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(groups + 1)]
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        evs[0].record(stream)
        for i in range(groups):
            for _ in range(replays_per_group):
                graph.replay()
            evs[i + 1].record(stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(groups)]
    return evs[0].elapsed_time(evs[groups]), per


def spread(per_group_ms, steps_per_group):
    v = sorted(x / steps_per_group for x in per_group_ms)
    return {"groups": len(v), "steps_per_group": steps_per_group, "ms_per_step_median": statistics.median(v),
            "ms_per_step_min": v[0], "ms_per_step_max": v[-1]}


# ------------------------------------------------------------------------------------ CPU legs
def cpu_reference_run(case, t, steps, warmup, budget_s=6.0):
    """Time the reference's CPU implementation (oracle/_ref, else the C restatement) on this host."""
    import refutil as R
    ops = case.cal_ops()
    cores = os.cpu_count() or 1
    if R.reference_available():
        if steps is None:   # bounded sample: probe, then as many calls as fit the budget
            _, probe = R.run_reference(case, t, iters=2, warmup=1, want_output=False)
            per = max(probe["ms_median"], 1e-3)
            steps = int(min(max(budget_s * 1e3 / per, 4), 512))
            warmup = 2
        _, info = R.run_reference(case, t, iters=steps, warmup=warmup, want_output=False)
        ms = info["ms_total"] / max(info["iters"], 1)
        return dict(kind="reference", cores=cores, ms_per_step=ms, steps=info["iters"],
                    value=ops / (ms * 1e-3) / 1e12,
                    sample=f"{info['iters']} calls on {case.n} images after {warmup} warm-up calls and the "
                           f"weight-transform call; AVX-512 VNNI build of the reference, OpenMP {cores} threads, "
                           f"published tuning knobs {case.knobs}")
    # no AVX-512 VNNI here (or the reference was not built): time the scalar restatement
    small = dataclasses.replace(case, n=max(1, min(case.n, 2)))
    ts = R.make_tensors(small)
    if small.algo == "wino" and small.types != "fp32":
        small = dataclasses.replace(small, tscale=case.tscale, tz=case.tz)
    fn = oracle_fn(case)
    t0 = time.perf_counter()
    fn(small, ts)
    dt = time.perf_counter() - t0
    ms = dt * 1e3 * case.n / small.n
    return dict(kind="port", cores=cores, ms_per_step=ms, steps=1, value=ops / (ms * 1e-3) / 1e12,
                sample=f"C restatement (OpenMP) on n={small.n} images, scaled to n={case.n}")


def reference_output(case, t):
    """Output of the reference's own library for this case (the C restatement where it cannot run)."""
    import refutil as R
    ignored_sum = case.sum and case.types != "fp32" and case.algo != "wino" and case.kh > 1 and case.g == 1
    if R.reference_available() and not ignored_sum:     # (the reference's int8 KxK path ignores with_ip_sum)
        out, _ = R.run_reference(case, t)
        return out, "reference"
    return oracle_fn(case)(case, t), "port"


def parity_of(case, got, want, comparand):
    """bit-exact for INT8 direct / 1x1 / depthwise outputs, rel-L2 <= 1e-5 for Winograd and fp32."""
    import numpy as np
    import refutil as R
    if case.out_dtype != np.float32 and case.algo != "wino":
        bad = int((got != want).sum())
        return {"status": "ok" if bad == 0 else "fail", "rule": "bit-exact", "mismatches": bad, "elements": int(got.size),
                "against": comparand, "images": int(case.n)}
    err = R.rel_l2(got, want)
    return {"status": "ok" if err <= 1e-5 else "fail", "rule": "rel-L2 <= 1e-5", "rel_l2": err, "elements": int(got.size),
            "against": comparand, "images": int(case.n)}


# ------------------------------------------------------------------------------------ one layer
class Ctx:
    def __init__(self, args, rank, world, local_rank, dist, peaks, peak_kind, sampler):
        self.args, self.rank, self.world, self.local_rank, self.dist = args, rank, world, local_rank, dist
        self.peaks, self.peak_kind, self.sampler = peaks, peak_kind, sampler


def slab(t: dict, first: int, count: int) -> dict:
    """Images [first, first+count) of the tensors of the global batch (weights and bias are shared)."""
    u = dict(t)
    for k in ("input", "residual"):
        if k in t:
            u[k] = t[k][first:first + count]
    return u


def run_layer(wid: str, ctx: Ctx, cpu_baseline: bool, steps: int | None = None):
    """One single-layer workload on this rank's share of the global batch.  Returns the entry dict."""
    import numpy as np
    import torch
    import refutil as R
    import gpuutil as G
    E = importlib.import_module(PKG)
    wl = WORKLOADS[wid]
    args = ctx.args
    gbatch = args.batch or wl["batch"]
    if gbatch < ctx.world:
        raise RuntimeError(f"{wid}: global batch {gbatch} < {ctx.world} GPUs")
    case_g = R.baseline_case(wid, gbatch)
    t_g = R.make_tensors(case_g)
    if case_g.algo == "wino" and case_g.types != "fp32":
        case_g = R.calibrate_tinput(case_g, t_g)
    first, count = split_batch(gbatch, ctx.world, ctx.rank)
    case = dataclasses.replace(case_g, n=count)
    t = slab(t_g, first, count)
    ops_g = case_g.cal_ops()
    alg_bytes_g = algorithmic_bytes(case_g, t_g)

    d = G.make_desc(case, device=ctx.local_rank)
    rc = d.setup()
    if rc != 0:
        raise RuntimeError(f"setup failed rc={rc}: {E.last_error()}")
    w_dev = torch.from_numpy(t["weights"]).cuda()
    b_dev = torch.from_numpy(t["bias"]).cuda()
    assert d.prepare(w_dev, b_dev) == 0, E.last_error()

    in_bytes = t["input"].nbytes
    out_elems = int(np.prod(R.out_shape(case)))
    out_dtype = {np.uint8: torch.uint8, np.int8: torch.int8, np.float32: torch.float32}[case.out_dtype]
    out_bytes = out_elems * np.dtype(case.out_dtype).itemsize
    nsets = min(64, max(2, -(-int(1.5 * L2_BYTES) // (in_bytes + out_bytes))))
    x0 = torch.from_numpy(np.ascontiguousarray(t["input"])).cuda()
    xs = [x0] + [x0.clone() for _ in range(nsets - 1)]
    if case.sum:      # in-place sum: the output tensors start as the residual
        r0 = torch.from_numpy(np.ascontiguousarray(t["residual"])).cuda().reshape(-1)
        os_ = [r0.clone() for _ in range(nsets)]
    else:
        os_ = [torch.zeros(out_elems, dtype=out_dtype, device="cuda") for _ in range(nsets)]

    stream = torch.cuda.Stream()

    def launch(i):
        rc = d.enqueue(os_[i % nsets], xs[i % nsets], None, None, stream.cuda_stream)
        if rc != 0:
            raise RuntimeError(f"enqueue failed rc={rc}: {E.last_error()}")

    warm = max(args.warmup, 3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for i in range(warm):
            launch(i)
        ev0.record(stream)
        for i in range(3):
            launch(i)
        ev1.record(stream)
    torch.cuda.synchronize()
    est_ms = ev0.elapsed_time(ev1) / 3
    # K steps per graph (K = --steps for a workload run alone; inside the all-configurations run a
    # multiple of the buffer ring), replayed until the timed region is long enough
    k_steps = steps if steps is not None else max(nsets, 10)
    if case.sum:
        k_steps = min(k_steps, nsets)       # every set's residual is consumed once per replay; see parity below
    l0 = d.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(k_steps):
            launch(i)
    launches_per_replay = d.launch_count() - l0
    with torch.cuda.stream(stream):
        graph.replay()          # untimed: uploads the graph
    torch.cuda.synchronize()
    ctx.sampler.reset()
    ctx.sampler.active = True
    ms_total, per = timed_replays(graph, stream, 1, est_ms * k_steps, ctx.dist)
    ctx.sampler.active = False
    clocks = ctx.sampler.summary()
    if d.device_status() != 0:
        raise RuntimeError(f"device status {d.device_status()}")
    steps_timed = k_steps * len(per)

    # ---- Winograd / fp32 direct: time each of the three kernels of a step live
    stage_ms = None
    if (case.algo == "wino" or d.kernel == "f32_direct_umma") and launches_per_replay == 3 * k_steps:
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for e in evs:
            e.record(stream)          # creates the underlying cudaEvent_t
        torch.cuda.synchronize()
        d.set_stage_events([e.cuda_event for e in evs])
        acc = [0.0, 0.0, 0.0]
        reps = 8
        for i in range(reps):
            launch(i)
            stream.synchronize()
            for k in range(3):
                acc[k] += evs[k].elapsed_time(evs[k + 1])
        d.set_stage_events(None)
        stage_ms = [a / reps for a in acc]

    # ---- parity of what was timed: one more step on set 0 from a fresh residual / zeroed output
    parity = None
    if ctx.rank == 0 and not args.no_parity:
        if case.sum:
            os_[0].copy_(torch.from_numpy(np.ascontiguousarray(t["residual"])).reshape(-1))
        else:
            os_[0].zero_()
        launch(0)
        stream.synchronize()
        got = os_[0].cpu().numpy().reshape(R.out_shape(case))
        try:
            want, comparand = reference_output(case, t)
            parity = parity_of(case, got, want, comparand)
        except Exception as e:          # the comparand could not be produced: say so, do not pass
            parity = {"status": "unchecked", "why": f"{type(e).__name__}: {e}"[:300]}
        if case.sum and case.algo != "wino" and case.types != "fp32" and case.kh > 1:
            parity["note"] = "the reference's KxK path ignores with_ip_sum; comparand = C restatement (parity unpinned)"

    # ---- end to end through the drop-in call with pinned host buffers
    hx = torch.from_numpy(np.ascontiguousarray(t["input"])).pin_memory()
    ho = (torch.from_numpy(np.ascontiguousarray(t["residual"])).reshape(-1).clone() if case.sum
          else torch.zeros(out_elems, dtype=out_dtype)).pin_memory()
    for _ in range(3):
        assert E.elx_conv(d, ho, hx, None, None) == 0, E.last_error()
    t0 = time.perf_counter()
    assert E.elx_conv(d, ho, hx, None, None) == 0, E.last_error()
    one = time.perf_counter() - t0
    e2e_steps = int(min(400, max(5, math.ceil(MIN_TIMED_S / max(one, 1e-5)))))
    torch.cuda.synchronize()
    if ctx.dist is not None:
        ctx.dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        rc = E.elx_conv(d, ho, hx, None, None)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    assert rc == 0, E.last_error()

    ms_step_raw = ms_total / steps_timed
    ms_step, e2e_ms = max_over_ranks([ms_step_raw, e2e_ms], ctx.dist)
    value = throughput(ops_g, ms_step)
    rl = layer_roofline(case_g, alg_bytes_g, gemm_ops_of(case_g), ops_g, ctx.peaks)
    kernels = None
    if stage_ms is not None:
        names = (["f32_gather_kernel", "wino_gemm_kernel", "f32_epilogue_kernel"] if d.kernel == "f32_direct_umma"
                 else ["wino_input_kernel", "wino_gemm_kernel", "wino_output_kernel"])
        kind = "f32" if case.types == "fp32" else "i8"
        gemm_tf = gemm_ops_of(case) / (stage_ms[1] * 1e-3) / 1e12
        kernels = [{"kernel": names[0], "ms": round(stage_ms[0], 5)},
                   {"kernel": names[1], "ms": round(stage_ms[1], 5), "gemm_tops": round(gemm_tf, 1),
                    "frac_of_tensor_peak": round(gemm_tf / tensor_peak(kind, ctx.peaks), 3)},
                   {"kernel": names[2], "ms": round(stage_ms[2], 5)}]
    else:
        kernels = [{"kernel": d.kernel, "ms": round(ms_step_raw, 5)}]
    entry = {
        "metric": wl["metric"], "value": value, "unit": wl["unit"], "ms_per_step": ms_step, "steps": k_steps,
        "dtype": wl["dtype"],
        "config": {"workload": f"{wid}: {wl['desc']}", "global_batch": gbatch, "batch_per_gpu": count,
                   "buffer_sets": nsets, "cache": "ring of buffer sets larger than L2 (126 MB), one set per step"},
        "timing": {**spread(per, k_steps), "timed_s": ms_total * 1e-3},
        "clocks": clocks,
        "e2e": {"value": throughput(ops_g, e2e_ms), "unit": wl["unit"],
                "h2d_bytes_per_step": in_bytes + (out_bytes if case.sum else 0), "d2h_bytes_per_step": out_bytes,
                "steps": e2e_steps, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches_per_replay * len(per)),
        "roofline": {"bound": rl["bound"], "achieved": value, "peak": rl["attainable"], "unit": wl["unit"],
                     "frac": value / ctx.world / rl["attainable"], "traffic": NCU_TRAFFIC.get(wid) if not args.batch else None,
                     "algorithmic_bytes": alg_bytes_g, "ops_per_byte": rl["ai"], "p_tensor": rl["p_tensor"],
                     "p_hbm": rl["p_hbm"], "peak_source": f"{ctx.peak_kind} copy bandwidth {ctx.peaks['hbm_gbs']} GB/s; "
                     f"tensor ceiling from the repository's tcgen05 issue-rate measurement at {ctx.peaks['sm_max_mhz']:.0f} MHz; "
                     "per GPU", "kernels": kernels, "launches_per_step": launches_per_replay / k_steps},
        "cal_ops_per_step": ops_g,
        "vs_baseline": (value / PUBLISHED[wid]) if wid in PUBLISHED and not args.batch else None,
    }
    if parity is not None:
        entry["parity"] = parity
    if cpu_baseline and ctx.rank == 0 and ctx.world == 1:
        try:
            r = cpu_reference_run(case_g, t_g, None, 2)
            entry["cpu_baseline"] = {"value": r["value"], "unit": wl["unit"], "cores": r["cores"], "kind": r["kind"],
                                     "sample": r["sample"], "ms_per_step": r["ms_per_step"]}
        except Exception as e:
            entry["cpu_baseline"] = {"value": None, "unit": wl["unit"], "cores": os.cpu_count(), "kind": "reference",
                                     "sample": f"failed: {e}"[:300]}
    d.close()
    del xs, os_, x0
    torch.cuda.empty_cache()
    return entry


# ------------------------------------------------------------------------------------ VGG-16 stack
def run_stack(wid: str, ctx: Ctx, cpu_baseline: bool, steps: int):
    import numpy as np
    import torch
    E = importlib.import_module(PKG)
    wl = WORKLOADS[wid]
    args = ctx.args
    int8 = wid == "c5i8"
    gbatch = args.batch or wl["batch"]
    n = stack_chunk_images(gbatch, ctx.world)
    chunks_g = gbatch // n
    if chunks_g * n != gbatch or chunks_g % ctx.world:
        raise RuntimeError(f"{wid}: global batch {gbatch} is not {ctx.world} x a whole number of {n}-image chunks")
    chunks = chunks_g // ctx.world                  # per GPU
    c_first = ctx.rank * chunks
    scales = vgg_calibrate(ctx.local_rank) if int8 else None
    # the network input is the caller's nchw image (three planes): the fp32 stack's first kernel reads
    # it directly, the INT8 stack converts it to a blocked tensor on the device (one small kernel,
    # counted in the timed region) -- a fifth of the bytes over PCIe either way
    plain = True
    st, cases = build_stack(n, int8, ctx.local_rank, scales, plain_image=plain)
    ops_chunk = sum(c.cal_ops() for c in cases)
    ops_g = ops_chunk * chunks_g
    x_np = np.concatenate([vgg_input(c_first + c, n, int8, plain) for c in range(chunks)])
    x = torch.from_numpy(x_np).cuda()
    xin = [x[c * n:(c + 1) * n] for c in range(chunks)]
    last = cases[-1]
    odt = torch.uint8 if int8 else torch.float32
    y = torch.zeros((chunks * n, last.oc // 16, last.oh, last.ow, 16), dtype=odt, device="cuda")
    yout = [y[c * n:(c + 1) * n] for c in range(chunks)]
    stream = torch.cuda.Stream()

    def step():
        for c in range(chunks):
            rc = st.enqueue(yout[c], xin[c], stream.cuda_stream)
            if rc != 0:
                raise RuntimeError(f"stack enqueue failed rc={rc}: {E.last_error()}")

    warm = max(args.warmup, 3)
    with torch.cuda.stream(stream):
        for _ in range(warm):
            step()
    torch.cuda.synchronize()
    # per-layer times: one untimed pass of one chunk with events around every convolution
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(cases) + 1)]
    for e in evs:
        e.record(stream)
    torch.cuda.synchronize()
    st.set_layer_events([e.cuda_event for e in evs])
    with torch.cuda.stream(stream):
        st.enqueue(yout[0], xin[0], stream.cuda_stream)
    torch.cuda.synchronize()
    st.set_layer_events(None)
    layer_ms = [evs[k].elapsed_time(evs[k + 1]) for k in range(len(cases))]     # (a pooled layer includes its subsample)
    # ONE step (this GPU's share of the global batch) per graph, replayed K times (and until the
    # timed region is long enough) between events
    l0 = st.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step()
    launches_per_step = st.launch_count() - l0
    with torch.cuda.stream(stream):
        graph.replay()
    torch.cuda.synchronize()
    est = sum(layer_ms) * chunks
    ctx.sampler.reset()
    ctx.sampler.active = True
    ms_total, per = timed_replays(graph, stream, steps, est, ctx.dist)
    t_end = time.perf_counter() + 0.2
    while time.perf_counter() < t_end:        # a little more of the same load for the clock sampler
        graph.replay()
        torch.cuda.synchronize()
    ctx.sampler.active = False
    clocks = ctx.sampler.summary()
    for k in range(len(cases)):
        stv = E.lib.elb_conv_device_status(st.layer_plan(k))
        if stv != 0:
            raise RuntimeError(f"device status {stv} in layer {k}")

    # parity of what was timed: the first two images of this rank's first chunk.  INT8: the u8 result
    # of the whole chain bit-exact against the CPU chain.  fp32: every layer within 1e-5 of the CPU
    # library on the same input (the GPU's own previous activation); the error of the whole chain,
    # which compounds over 13 layers, is reported beside it.
    parity = None
    if ctx.rank == 0 and not args.no_parity:
        try:
            with torch.cuda.stream(stream):
                st.enqueue(yout[0], xin[0], stream.cuda_stream)
            torch.cuda.synchronize()
            got = yout[0][:2].cpu().numpy()
            want, comparand = stack_reference_chain(cases, x_np[:2], int8)
            if int8:
                bad = int((got != want).sum())
                parity = {"status": "ok" if bad == 0 else "fail", "rule": "bit-exact u8 after 13 chained layers",
                          "mismatches": bad, "elements": int(got.size), "against": comparand, "images": 2}
            else:
                import refutil as R
                outs = stack_layer_outputs(st, cases, yout[0], images=2)
                errs, comparand = per_layer_parity(cases, x_np[:2], outs, False)
                worst = max(errs)
                parity = {"status": "ok" if worst <= 1e-5 else "fail",
                          "rule": "every layer rel-L2 <= 1e-5 against the CPU library on the same input",
                          "rel_l2": worst, "per_layer_rel_l2": [float(f"{e:.3e}") for e in errs],
                          "chain_rel_l2_after_13_layers": R.rel_l2(got, want), "elements": int(got.size),
                          "against": comparand, "images": 2}
        except Exception as e:
            parity = {"status": "unchecked", "why": f"{type(e).__name__}: {e}"[:300]}

    # end to end: this GPU's images from pinned host memory through elb_stack_execute, result back to the host
    hx = torch.from_numpy(x_np).pin_memory()
    hy = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    imgs = chunks * n
    assert st.execute(hy, hx, imgs) == 0, E.last_error()
    e2e_steps = max(2, min(steps, int(math.ceil(1.0 / max(est * 1e-3, 1e-4)))))
    torch.cuda.synchronize()
    if ctx.dist is not None:
        ctx.dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        rc = st.execute(hy, hx, imgs)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    assert rc == 0, E.last_error()

    ms_step_raw = ms_total / (len(per) * steps)
    ms_step, e2e_ms = max_over_ranks([ms_step_raw, e2e_ms], ctx.dist)
    value = throughput(ops_g, ms_step)
    # attainable: every layer at the better of its tensor ceiling and its HBM floor (each layer reads
    # its input and writes its output once; the subsample reads a quarter and writes it)
    t_att, alg_bytes = 0.0, 0
    eb = 1 if int8 else 4
    for k, c in enumerate(cases):
        w_b = 9 * c.ic * c.oc * 4
        cin = c.ic if c.ifmt == "nchw" else 16 * ((c.ic + 15) // 16)      # (the plain image has its real channels only)
        b = c.n * (cin * c.ih * c.iw + c.oc * c.oh * c.ow) * eb + w_b
        if vgg_layers()[k][3] == 2:
            b += 2 * c.n * c.oc * (c.oh // 2) * (c.ow // 2) * eb
        alg_bytes += b
        rl = layer_roofline(c, b, c.cal_ops() if int8 else gemm_ops_of(c), c.cal_ops(), ctx.peaks)
        t_att += c.cal_ops() / (rl["attainable"] * 1e12)
    attainable = ops_chunk / t_att / 1e12
    slow = int(np.argmax(layer_ms))
    entry = {
        "metric": wl["metric"], "value": value, "unit": wl["unit"], "ms_per_step": ms_step, "steps": steps,
        "dtype": wl["dtype"],
        "config": {"workload": f"{wid}: {wl['desc']}", "global_batch": gbatch, "batch_per_gpu": chunks * n,
                   "chunk_images": n, "chunks_per_gpu_per_step": chunks,
                   "parallelism": f"minibatch split over {ctx.world} GPU(s), replicated weights, no collective",
                   "cache": "one chunk streams more than 1 GB of activations through the 126 MB L2",
                   "layers": [{"name": c.name, "ms": round(ms, 4), "tops": round(c.cal_ops() / ms / 1e9, 2)}
                              for c, ms in zip(cases, layer_ms)],
                   **({"u8_scales": [round(v, 6) for v in scales]} if int8 else {})},
        "timing": {**spread(per, steps), "timed_s": ms_total * 1e-3},
        "clocks": clocks,
        "e2e": {"value": throughput(ops_g, e2e_ms), "unit": wl["unit"], "h2d_bytes_per_step": x_np.nbytes,
                "d2h_bytes_per_step": hy.numel() * hy.element_size(), "steps": e2e_steps, "ms_per_step": e2e_ms,
                "call": "elb_stack_execute"},
        "gpu_launches": int(launches_per_step * len(per) * steps),
        "roofline": {"bound": "tensor+hbm per layer", "achieved": value, "peak": attainable, "unit": wl["unit"],
                     "frac": value / ctx.world / attainable,
                     "traffic": NCU_TRAFFIC[wid] / ctx.world if wid in NCU_TRAFFIC and not args.batch else None,
                     "algorithmic_bytes": alg_bytes * chunks_g,
                     "peak_source": f"sum over layers of max(ops / tensor ceiling, bytes / {ctx.peak_kind} "
                                    f"{ctx.peaks['hbm_gbs']} GB/s); tensor ceiling from the repository's tcgen05 "
                                    f"issue-rate measurement at {ctx.peaks['sm_max_mhz']:.0f} MHz; per GPU",
                     "kernels": [{"kernel": c.name, "ms": round(ms, 4)} for c, ms in zip(cases, layer_ms)],
                     "slowest_layer": cases[slow].name, "launches_per_step": launches_per_step},
        "cal_ops_per_step": ops_g, "vs_baseline": None,
    }
    if parity is not None:
        entry["parity"] = parity
    if cpu_baseline and ctx.rank == 0 and ctx.world == 1:
        entry["cpu_baseline"] = stack_cpu_baseline(int8, gbatch, wl)
    st.close()
    del x, y, xin, yout
    torch.cuda.empty_cache()
    return entry


def stack_cpu_baseline(int8, gbatch, wl, steps=2):
    """The 13 layers through the reference's CPU library on a bounded sample (8 images per call, enough
    for its thread partitioning over images / tiles to fill the cores), per-layer times summed and
    scaled to the global batch."""
    import refutil as R
    n_s = 8
    total_ms, r = 0.0, None
    for k, (ic, oc, hw, _) in enumerate(vgg_layers()):
        case = vgg_layer_case(k, ic, oc, hw, n_s, int8, 1.0 / 255.0 if k == 0 else 0.02, 0.02)
        t = R.make_tensors(case)
        r = cpu_reference_run(case, t, steps, 1)
        total_ms += r["ms_per_step"] * (gbatch / n_s)
    ops = sum(vgg_layer_case(k, ic, oc, hw, gbatch, int8).cal_ops() for k, (ic, oc, hw, _) in enumerate(vgg_layers()))
    value = ops / (total_ms * 1e-3) / 1e12
    sample = (f"each of the 13 layers on {n_s} images ({steps} timed calls after the weight-transform call), summed "
              f"and scaled to {gbatch} images; {r['sample']}")
    return {"value": value, "unit": wl["unit"], "cores": os.cpu_count() or 1, "kind": r["kind"], "sample": sample,
            "ms_per_step": total_ms}


# ------------------------------------------------------------------------------------ reference arm
def reference_entry(wid, args):
    import refutil as R
    wl = WORKLOADS[wid]
    gbatch = args.batch or wl["batch"]
    if wid in ("c5", "c5i8"):
        cb = stack_cpu_baseline(wid == "c5i8", gbatch, wl, max(2, min(args.steps, 3)))
        return {"metric": wl["metric"], "value": cb["value"], "unit": wl["unit"], "ms_per_step": cb["ms_per_step"],
                "dtype": wl["dtype"], "config": {"workload": f"{wid}: {wl['desc']}", "global_batch": gbatch},
                "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": cb["value"], "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    case = R.baseline_case(wid, gbatch)
    t = R.make_tensors(case)
    if case.algo == "wino" and case.types != "fp32":
        case = R.calibrate_tinput(case, t)
    r = cpu_reference_run(case, t, None, 2, budget_s=8.0)
    return {"metric": wl["metric"], "value": r["value"], "unit": wl["unit"], "ms_per_step": r["ms_per_step"],
            "steps": r["steps"], "dtype": wl["dtype"],
            "config": {"workload": f"{wid}: {wl['desc']}", "global_batch": gbatch},
            "cpu_baseline": {"value": r["value"], "unit": wl["unit"], "cores": r["cores"], "kind": r["kind"],
                             "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="all", choices=["all"] + sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--batch", type=int, default=None,
                    help="global batch instead of the workload's own (small profiler captures only; "
                         "the reported line then names the reduced batch)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    head = HEADLINE if args.workload == "all" else args.workload
    others = PER_CONFIG if args.workload == "all" else []

    # ------------------------------------------------------------------ reference arm
    if args.impl == "reference":
        if rank != 0:
            return 0
        line = reference_entry(head, args)
        line.update({"impl": "reference", "n_gpus": args.gpus, "steps": line.get("steps", args.steps), "warmup": args.warmup,
                     "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic"})
        if others:
            line["per_config"] = {}
            for wid in others:
                try:
                    line["per_config"][wid] = reference_entry(wid, args)
                except Exception as e:
                    line["per_config"][wid] = {"error": f"{type(e).__name__}: {e}"[:300]}
        print(json.dumps(line))
        return 0

    # ------------------------------------------------------------------ own arm
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- this library has no CPU path")
    torch.cuda.set_device(local_rank)
    numa = bind_to_gpu_cpus(local_rank) if world > 1 else None
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import __graft_entry__ as g
    if rank == 0:
        g.build()
    if dist is not None:
        dist.barrier()
    importlib.import_module(PKG)
    peaks, peak_kind = measured_peaks()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ctx = Ctx(args, rank, world, local_rank, dist, peaks, peak_kind, sampler)

    def run(wid, headline):
        cpu = not args.no_cpu_baseline
        if wid in ("c5", "c5i8"):
            return run_stack(wid, ctx, cpu, args.steps)
        return run_layer(wid, ctx, cpu, args.steps if headline and args.workload != "all" else None)

    entry = run(head, True)
    line = {"metric": entry["metric"], "value": entry["value"], "unit": entry["unit"], "n_gpus": world,
            "steps": entry["steps"], "warmup": max(args.warmup, 3), "ms_per_step": entry["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": entry.get("vs_baseline"),
            "dtype": entry["dtype"], "data": "synthetic"}
    for k in ("config", "timing", "clocks", "e2e", "gpu_launches", "roofline", "parity", "cpu_baseline", "cal_ops_per_step"):
        if k in entry:
            line[k] = entry[k]
    if others:
        line["per_config"] = {}
        for wid in others:
            try:
                line["per_config"][wid] = run(wid, False)
            except Exception as e:
                line["per_config"][wid] = {"error": f"{type(e).__name__}: {e}"[:300]}
                if dist is not None:
                    raise           # ranks must stay in step: a failure on one rank ends the run
    sampler.stop()
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
