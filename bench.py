#!/usr/bin/env python
"""Benchmark of the convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|dw] [--impl reference]

One "step" is one convolution call (elx_conv) over one batch of synthetic input of the named
workload.  Workloads are the benchmark configurations: c1 FP32 Winograd F(4x4,3x3) VGG conv3_2,
c2 INT8 1x1 ResNet-50 res4 reduce (default), c3 INT8 3x3 stride 2, c4 INT8 Winograd, dw INT8 depthwise 3x3
(a MobileNet-v1 layer shape; the benchmark configurations name no depthwise case).

Own arm (default): rank r owns one GPU and the whole batch of the workload (weak scaling over the
minibatch: the path shards by image with replicated weights and has no exchange step, so there is
no collective on the data path).  Reported on one JSON line:
  value / ms_per_step : inputs resident in HBM, K back-to-back launches between CUDA events on the
                        launching stream, max over ranks; a ring of input/output buffer sets larger
                        than L2 is walked so no step finds its operands in cache
  e2e                 : the same K steps through the drop-in call with pinned HOST buffers
                        (host->device copy of the input and device->host copy of the output inside
                        every step)
  roofline            : algorithmic bytes (or FLOPs) of one launch / average launch duration
  cpu_baseline        : the reference's own AVX-512 library (oracle/_ref) timed on this host's
                        cores on a bounded sample (rank 0, N=1 only)
Reference arm (--impl reference): the reference's CPU implementation only, same metric/config.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

WORKLOADS = {
    "c1": dict(metric="effective_conv_tflops_fp32_winograd", unit="TFLOP/s", dtype="tf32x3(fp32)",
               desc="FP32 Winograd F(4x4,3x3) VGG-16 conv3_2 N=64 C=K=256 56x56 s1 p1 bias+ReLU nChw16c"),
    "c2": dict(metric="effective_conv_tops_int8", unit="TOP/s", dtype="u8",
               desc="INT8 u8s8 1x1 ResNet-50 res4 reduce N=64 C=1024 K=256 14x14 bias+ReLU u8 out nChw16c"),
    "c3": dict(metric="effective_conv_tops_int8", unit="TOP/s", dtype="u8",
               desc="INT8 u8s8 3x3 stride 2 pad 1 N=64 C=128 K=256 56x56->28x28 bias+ReLU u8 out nChw16c"),
    "c4": dict(metric="effective_conv_tops_int8_winograd", unit="TOP/s", dtype="u8",
               desc="INT8 Winograd F(4x4,3x3) N=128 C=K=512 28x28 s1 p1 f32 out nChw16c"),
    "dw": dict(metric="effective_conv_tops_int8_depthwise", unit="TOP/s", dtype="u8",
               desc="INT8 depthwise 3x3 MobileNet-v1 Conv2d_3 N=64 C=128 56x56 s1 p1 bias+ReLU u8 out nChw16c T=14"),
}
# published number for exactly this metric/config (2 x Xeon 8180, reference's tuned script comment)
PUBLISHED = {"c1": 11.2}


def algorithmic_bytes(case, t) -> int:
    """input + weights as the user passes them + output (+ residual)."""
    import numpy as np
    out_b = int(np.prod((case.n, (case.oc + 15) // 16 * 16, case.oh, case.ow))) * np.dtype(case.out_dtype).itemsize
    b = t["input"].nbytes + (t["weights"].nbytes - 64 * 4) + out_b
    if case.sum:
        b += out_b
    return b


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


def aggregate_throughput(ops, ms_per_step, world):
    """Whole-job T(FL)OP/s: every rank processes the workload's full batch (weak scaling)."""
    return world * ops / (ms_per_step * 1e-3) / 1e12


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def cpu_reference_run(case, t, steps, warmup, budget_s=12.0):
    """Time the reference's CPU implementation (oracle/_ref, else the C restatement) on this host."""
    import refutil as R
    ops = case.cal_ops()
    cores = os.cpu_count() or 1
    if R.reference_available():
        if steps is None:   # bounded sample: probe, then as many calls as fit the budget
            _, probe = R.run_reference(case, t, iters=3, warmup=1, want_output=False)
            per = max(probe["ms_median"], 1e-3)
            steps = int(min(max(budget_s * 1e3 / per, 8), 1024))
            warmup = 2
        _, info = R.run_reference(case, t, iters=steps, warmup=warmup, want_output=False)
        ms = info["ms_total"] / max(info["iters"], 1)
        return dict(kind="reference", cores=cores, ms_per_step=ms, steps=info["iters"],
                    value=ops / (ms * 1e-3) / 1e12,
                    sample=f"{info['iters']} calls of the full workload after {warmup} warm-up calls and the "
                           f"weight-transform call; AVX-512 VNNI build of the reference, OpenMP {cores} threads, "
                           f"published tuning knobs {case.knobs}")
    # no AVX-512 VNNI here (or the reference was not built): time the scalar restatement
    import dataclasses
    small = dataclasses.replace(case, n=max(1, min(case.n, 2)))
    ts = R.make_tensors(small)
    fn = {"fp32": R.oracle_wino_f32}.get(case.types, R.oracle_int8_wino if case.algo == "wino" else
                                         R.oracle_int8_depthwise if case.g > 1 else R.oracle_int8_conv)
    t0 = time.perf_counter()
    fn(small, ts)
    dt = time.perf_counter() - t0
    ms = dt * 1e3 * case.n / small.n
    return dict(kind="port", cores=cores, ms_per_step=ms, steps=1, value=ops / (ms * 1e-3) / 1e12,
                sample=f"C restatement (OpenMP) on n={small.n} images, scaled to n={case.n}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=None,
                    help="images per GPU instead of the workload's own batch (small profiler captures only; "
                         "the reported line then names the reduced batch)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.workload]

    import refutil as R
    case = R.baseline_case(args.workload, args.batch)
    config = {"workload": f"{args.workload}: {wl['desc']}", "batch_per_gpu": case.n,
              "global_batch": case.n * max(world, 1), "parallelism": f"minibatch split, {max(world,1)} x replicated weights",
              "cache": "ring of buffer sets larger than L2 (126 MB), one set per step"}

    # ------------------------------------------------------------------ reference arm
    if args.impl == "reference":
        if rank != 0:
            return 0
        t = R.make_tensors(case)
        if case.algo == "wino" and case.types != "fp32":
            case = R.calibrate_tinput(case, t)
        r = cpu_reference_run(case, t, args.steps, max(args.warmup, 1))
        line = {"impl": "reference", "metric": wl["metric"], "value": r["value"], "unit": wl["unit"],
                "n_gpus": args.gpus, "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"],
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": r["value"], "unit": wl["unit"], "cores": r["cores"], "kind": r["kind"],
                                 "sample": r["sample"]},
                "e2e": {"value": r["value"], "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return 0

    # ------------------------------------------------------------------ own arm
    import numpy as np
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device -- this library has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import __graft_entry__ as g
    if rank == 0:
        g.build()
    if dist is not None:
        dist.barrier()
    E = importlib.import_module("deep-learning-math-kernel-research_b200")
    import gpuutil as G

    t = R.make_tensors(case)
    if case.algo == "wino" and case.types != "fp32":
        case = R.calibrate_tinput(case, t)
    ops = case.cal_ops()
    alg_bytes = algorithmic_bytes(case, t)

    d = G.make_desc(case, device=local_rank)
    rc = d.setup()
    if rc != 0:
        raise SystemExit(f"bench.py: setup failed rc={rc}: {E.last_error()}")
    w_dev = torch.from_numpy(t["weights"]).cuda()
    b_dev = torch.from_numpy(t["bias"]).cuda()
    assert d.prepare(w_dev, b_dev) == 0, E.last_error()

    in_bytes = t["input"].nbytes
    out_elems = int(np.prod(R.out_shape(case)))
    out_dtype = {np.uint8: torch.uint8, np.int8: torch.int8, np.float32: torch.float32}[case.out_dtype]
    out_bytes = out_elems * np.dtype(case.out_dtype).itemsize
    nsets = max(2, -(-int(1.5 * L2_BYTES) // (in_bytes + out_bytes)))
    nsets = min(nsets, 64)
    x0 = torch.from_numpy(t["input"]).cuda()
    xs = [x0] + [x0.clone() for _ in range(nsets - 1)]
    os_ = [torch.zeros(out_elems, dtype=out_dtype, device="cuda") for _ in range(nsets)]
    config["buffer_sets"] = nsets

    stream = torch.cuda.Stream()
    sampler = ClockSampler(local_rank)
    sampler.start()

    def launch(i):
        rc = d.enqueue(os_[i % nsets], xs[i % nsets], None, None, stream.cuda_stream)
        if rc != 0:
            raise SystemExit(f"bench.py: enqueue failed rc={rc}: {E.last_error()}")

    with torch.cuda.stream(stream):
        for i in range(max(args.warmup, 3)):
            launch(i)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    # The K steps are captured once into a CUDA graph (one kernel node per step, each with its own
    # buffer set) and replayed between two events, so the timed region holds the K launches and no
    # Python/driver launch latency.
    l0 = d.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(args.steps):
            launch(i)
    launches_per_replay = d.launch_count() - l0
    with torch.cuda.stream(stream):
        graph.replay()          # untimed: uploads the graph
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.active = True
    l0 = d.launch_count() - launches_per_replay
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        ev0.record(stream)
        graph.replay()
        ev1.record(stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    launches = d.launch_count() - l0
    ms_total = ev0.elapsed_time(ev1)
    if d.device_status() != 0:
        raise SystemExit(f"bench.py: device status {d.device_status()}")

    # keep the GPU under the same load a little longer so that the clock sampler sees it busy
    t_end = time.perf_counter() + 0.4
    with torch.cuda.stream(stream):
        while time.perf_counter() < t_end:
            graph.replay()
            stream.synchronize()
    torch.cuda.synchronize()
    sampler.active = False

    # ---- end to end through the drop-in call with pinned host buffers
    hx = torch.from_numpy(t["input"]).pin_memory()
    ho = torch.zeros(out_elems, dtype=out_dtype).pin_memory()
    e2e_steps = max(3, min(args.steps, 200))
    for _ in range(3):
        assert E.elx_conv(d, ho, hx, None, None) == 0, E.last_error()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        rc = E.elx_conv(d, ho, hx, None, None)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    assert rc == 0, E.last_error()
    sampler.stop()

    ms_total, e2e_ms = max_over_ranks([ms_total, e2e_ms], dist, device="cuda")

    ms_step = ms_total / args.steps
    value = aggregate_throughput(ops, ms_step, world)
    e2e_value = aggregate_throughput(ops, e2e_ms / e2e_steps, world)

    peaks, peak_kind = measured_peaks()
    traffic = None
    tp = ROOT / "profiles" / "traffic.json"
    if tp.exists():
        traffic = json.loads(tp.read_text()).get(args.workload)
    achieved_gbs = alg_bytes / (ms_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved_gbs / peaks["hbm_gbs"], "traffic": traffic, "peak_source": peak_kind,
                "algorithmic_bytes_per_launch": alg_bytes,
                "kernel": d.kernel, "launches_per_step": launches / args.steps}

    line = {"metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / PUBLISHED[args.workload]) if args.workload in PUBLISHED else None,
            "dtype": wl["dtype"], "data": "synthetic", "config": config,
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": wl["unit"], "h2d_bytes_per_step": in_bytes,
                    "d2h_bytes_per_step": out_bytes, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches), "roofline": roofline, "cal_ops_per_step": ops}

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            r = cpu_reference_run(case, t, None, 2)
            line["cpu_baseline"] = {"value": r["value"], "unit": wl["unit"], "cores": r["cores"], "kind": r["kind"],
                                    "sample": r["sample"], "ms_per_step": r["ms_per_step"]}
        except Exception as e:
            line["cpu_baseline"] = {"value": None, "unit": wl["unit"], "cores": os.cpu_count(), "kind": "reference",
                                    "sample": f"failed: {e}"[:300]}
    if rank == 0:
        print(json.dumps(line))
    d.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
