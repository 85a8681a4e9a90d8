#!/usr/bin/env python
"""Benchmark of the convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c3s|c4|c5|c5i8|dw] [--impl reference]

One "step" is one convolution call (elx_conv) over one batch of synthetic input of the named
workload.  Workloads are the benchmark configurations: c1 FP32 Winograd F(4x4,3x3) VGG conv3_2,
c2 INT8 1x1 ResNet-50 res4 reduce (default), c3 INT8 3x3 stride 2, c4 INT8 Winograd, dw INT8 depthwise 3x3
(a MobileNet-v1 layer shape; the benchmark configurations name no depthwise case), c5 / c5i8 the
whole VGG-16 convolution stack (13 layers, 32 images per GPU) with fp32 Winograd / INT8 direct kernels.

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
import dataclasses
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
    "c3s": dict(metric="effective_conv_tops_int8", unit="TOP/s", dtype="u8",
                desc="INT8 u8s8 3x3 stride 2 pad 1 N=64 C=128 K=256 56x56->28x28 bias+ReLU+sum (u8 residual in the output "
                     "tensor, sum scale 1.0) u8 out nChw16c; the reference's KxK path ignores the sum flag"),
    "c4": dict(metric="effective_conv_tops_int8_winograd", unit="TOP/s", dtype="u8",
               desc="INT8 Winograd F(4x4,3x3) N=128 C=K=512 28x28 s1 p1 f32 out nChw16c"),
    "c1t4": dict(metric="effective_conv_tflops_fp32_winograd_f2x2", unit="TFLOP/s", dtype="tf32x3(fp32)",
                 desc="FP32 Winograd F(2x2,3x3) (tile_size 4) VGG-16 conv3_2 N=64 C=K=256 56x56 s1 p1 bias+ReLU nChw16c"),
    "c4t4": dict(metric="effective_conv_tops_int8_winograd_f2x2", unit="TOP/s", dtype="u8",
                 desc="INT8 Winograd F(2x2,3x3) (tile_size 4) N=128 C=K=512 28x28 s1 p1 f32 out nChw16c"),
    "v12": dict(metric="effective_conv_tflops_fp32_winograd", unit="TFLOP/s", dtype="tf32x3(fp32)",
                desc="FP32 Winograd F(4x4,3x3) VGG-16 conv1_2 N=32 C=K=64 224x224 s1 p1 bias+ReLU nChw16c"),
    "c2f": dict(metric="effective_conv_tflops_fp32_direct_1x1", unit="TFLOP/s", dtype="tf32x3(fp32)",
                desc="FP32 direct 1x1 ResNet-50 res4 reduce N=64 C=1024 K=256 14x14 bias+ReLU nChw16c"),
    "c3f": dict(metric="effective_conv_tflops_fp32_direct", unit="TFLOP/s", dtype="tf32x3(fp32)",
                desc="FP32 direct 3x3 stride 2 pad 1 N=64 C=128 K=256 56x56->28x28 bias+ReLU nChw16c"),
    "dw": dict(metric="effective_conv_tops_int8_depthwise", unit="TOP/s", dtype="u8",
               desc="INT8 depthwise 3x3 MobileNet-v1 Conv2d_3 N=64 C=128 56x56 s1 p1 bias+ReLU u8 out nChw16c T=14"),
    "c5": dict(metric="effective_conv_tflops_fp32_winograd_vgg16_stack", unit="TFLOP/s", dtype="tf32x3(fp32)",
               desc="VGG-16 conv stack, 13 layers 3x3 p1, 224x224 input, fp32 Winograd F(4x4,3x3), 32 images per GPU, "
                    "stride-2 subsample between stages, bias+ReLU, nChw16c"),
    "c5i8": dict(metric="effective_conv_tops_int8_vgg16_stack", unit="TOP/s", dtype="u8",
                 desc="VGG-16 conv stack, 13 layers 3x3 p1, 224x224 input, INT8 u8s8 direct, u8 between layers, 32 images "
                      "per GPU, stride-2 subsample between stages, bias+ReLU, nChw16c"),
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


# DRAM bytes (read + written) of ONE launch of each workload's dominant kernel, from the ncu
# captures summarised under profiles/ (launch lists of the full-size workloads).
NCU_TRAFFIC = {
    "c1": {"wino_input_kernel": 205.6e6 + 404.6e6, "wino_gemm_kernel": 481.5e6 + 411.2e6,
           "wino_output_kernel": 462.5e6 + 174.2e6},
    "c2": {"i8_gemm_umma": 13.15e6},
    "c3": {"i8_conv_umma": 26.03e6},
    "c3s": {"i8_conv_umma": 38.88e6},
    "c2f": {"wino_gemm_kernel": 53.5e6},
    "dw": {"i8_depthwise": 25.71e6 + 0.01e6},
    "c4": {"wino_input_kernel": 51.4e6 + 57.0e6, "wino_gemm_kernel": 114.8e6 + 357.9e6,
           "wino_output_kernel": 462.5e6 + 175.3e6},
}


def roofline_of(workload, case, d, alg_bytes, ms_step, stage_ms, peaks, peak_kind, launches_per_step, batch):
    """Roofline entry of the DOMINANT kernel of a step.

    Single-kernel workloads (int8 direct / 1x1 / depthwise): algorithmic bytes of the convolution
    (input + weights as passed + output) over the launch time, against the measured copy bandwidth.
    Winograd workloads launch three kernels; the dominant one is named with its own algorithmic
    figure: for the fp32 GEMM the 2*36*tiles*IC*OC transform-domain flops against one third of the
    measured tf32 rate (tf32 = half the measured bf16 rate; three tf32 MMAs per product keep fp32
    accuracy), for a transform kernel the bytes it must read and write against the copy bandwidth."""
    traffic_tbl = NCU_TRAFFIC.get(workload, {}) if batch is None else {}
    if stage_ms is None:
        traffic = traffic_tbl.get(d.kernel)
        gbs = alg_bytes / (ms_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                "traffic": traffic, "peak_source": peak_kind, "algorithmic_bytes_per_launch": alg_bytes,
                "kernel": d.kernel, "launches_per_step": launches_per_step, "kernel_ms": ms_step}
    import refutil as R
    icp, ocp = R.alignup(case.ic), R.alignup(case.oc)
    tiles = R.wino_tiles(case)
    in_b = case.n * icp * case.ih * case.iw * (4 if case.types == "fp32" else 1)
    out_b = case.n * ocp * case.oh * case.ow * (4 if case.out_dtype.__name__ == "float32" else 1)
    aa = R.wino_edge(case) ** 2
    names = ["wino_input_kernel", "wino_gemm_kernel", "wino_output_kernel"]
    if d.kernel == "f32_direct_umma":
        # implicit GEMM: one row per output pixel, K = taps * input channels, one "position"
        names = ["f32_gather_kernel", "wino_gemm_kernel", "f32_epilogue_kernel"]
        tiles, aa, icp = case.n * case.oh * case.ow, 1, icp * case.kh * case.kw
    v_b = aa * tiles * icp * (4 if case.types == "fp32" else 1)
    m_b = aa * tiles * ocp * 4
    kernels = [{"kernel": names[0], "ms": stage_ms[0], "bytes": in_b + v_b},
               {"kernel": names[1], "ms": stage_ms[1], "bytes": v_b + m_b, "flops": 2 * aa * tiles * icp * ocp},
               {"kernel": names[2], "ms": stage_ms[2], "bytes": m_b + out_b}]
    if launches_per_step == 1:
        # fp32 1x1 stride 1: the GEMM kernel alone reads the input and writes the output
        kernels = [{"kernel": names[1], "ms": ms_step, "bytes": in_b + out_b + ocp * icp * 4,
                    "flops": 2 * aa * tiles * icp * ocp}]
        stage_ms = [ms_step]
    for k in kernels:
        k["gbs"] = k["bytes"] / (k["ms"] * 1e-3) / 1e9
        k["frac_hbm"] = k["gbs"] / peaks["hbm_gbs"]
    dom = max(range(len(kernels)), key=lambda i: stage_ms[i])
    k = kernels[dom]
    if "flops" in k and case.types == "fp32":
        tf = k["flops"] / (k["ms"] * 1e-3) / 1e12
        peak = peaks["bf16_tflops"] / 2 / 3
        rl = {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
              "peak_note": "measured bf16 rate / 2 (tf32) / 3 (3xTF32 split for fp32 accuracy)",
              "algorithmic_flops_per_launch": k["flops"]}
    else:
        rl = {"bound": "hbm", "achieved": k["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": k["frac_hbm"],
              "algorithmic_bytes_per_launch": k["bytes"]}
    rl.update({"traffic": traffic_tbl.get(k["kernel"]), "peak_source": peak_kind,
               "kernel": k["kernel"], "kernel_ms": k["ms"], "launches_per_step": launches_per_step,
               "step_kernels": [{"kernel": q["kernel"], "ms": round(q["ms"], 5), "algorithmic_GBps": round(q["gbs"], 1),
                                 "frac_of_hbm_peak": round(q["frac_hbm"], 3)} for q in kernels]})
    return rl


# ------------------------------------------------------------------------------------ VGG-16 stack
VGG16 = [(3, 64, 224), (64, 64, 224), "pool", (64, 128, 112), (128, 128, 112), "pool", (128, 256, 56),
         (256, 256, 56), (256, 256, 56), "pool", (256, 512, 28), (512, 512, 28), (512, 512, 28), "pool",
         (512, 512, 14), (512, 512, 14), (512, 512, 14)]
VGG_NAMES = ["conv1_1", "conv1_2", "conv2_1", "conv2_2", "conv3_1", "conv3_2", "conv3_3", "conv4_1", "conv4_2",
             "conv4_3", "conv5_1", "conv5_2", "conv5_3"]


def vgg_layer_case(idx, ic, oc, hw, n, int8, iscale=1.0, oscale=1.0):
    import refutil as R
    if int8:
        return R.ConvCase(f"vgg_{VGG_NAMES[idx]}", n, ic, oc, hw, hw, types="u8f32u8f32", algo="direct", relu=True,
                          bias=True, iscale=iscale, oscale=oscale)
    return R.ConvCase(f"vgg_{VGG_NAMES[idx]}", n, ic, oc, hw, hw, types="fp32", algo="wino", tile=6, relu=True, bias=True)


def vgg_weights(idx, ic, oc):
    """He-initialised fp32 weights N(0, sqrt(2/(9*ic))) and bias U[-0.1, 0.1], seeded per layer."""
    import numpy as np
    import refutil as R
    g = np.random.Generator(np.random.Philox(R.seed_for("vgg16", VGG_NAMES[idx])))
    w = (g.standard_normal((oc, ic, 3, 3)) * np.sqrt(2.0 / (9 * ic))).astype(np.float32)
    b = np.zeros(R.alignup(oc), np.float32)
    b[:oc] = g.uniform(-0.1, 0.1, oc).astype(np.float32)
    return R.weights_buffer(R.to_OIhw16i16o(w)), b


class VggStack:
    """The 13 convolutions of VGG-16 as 13 plans of the library, run back to back on device tensors;
    the 2x2 pooling between stages keeps every second row and column (the library's subsample kernel)."""

    def __init__(self, n, int8, device, scales=None):
        import torch
        import gpuutil as G
        E = importlib.import_module("deep-learning-math-kernel-research_b200")
        self.E, self.n, self.int8 = E, n, int8
        self.layers, self.ops, self.names = [], 0, []
        self.pool_launches = 0
        k = 0
        last = None
        for item in VGG16:
            if item == "pool":
                oc, hw = last
                odt = torch.uint8 if int8 else torch.float32
                self.layers.append(("pool", torch.zeros((n, (oc + 15) // 16, hw // 2, hw // 2, 16), dtype=odt, device="cuda"),
                                    (oc, hw)))
                continue
            ic, oc, hw = item
            last = (oc, hw)
            isc, osc = (scales[k], scales[k + 1]) if int8 else (1.0, 1.0)
            case = vgg_layer_case(k, ic, oc, hw, n, int8, isc, osc)
            d = G.make_desc(case, device=device)
            rc = d.setup()
            if rc != 0:
                raise SystemExit(f"bench.py: setup of {case.name} failed rc={rc}: {E.last_error()}")
            w, b = vgg_weights(k, ic, oc)
            wd, bd = torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
            assert d.prepare(wd, bd) == 0, E.last_error()
            odt = torch.uint8 if int8 else torch.float32
            out = torch.zeros((n, (oc + 15) // 16, hw, hw, 16), dtype=odt, device="cuda")
            self.layers.append((d, out, case))
            self.ops += case.cal_ops()
            self.names.append(case.name)
            k += 1

    def run(self, x, stream, events=None):
        """Enqueue the whole stack on `stream` (a torch stream that is current); returns the last output."""
        i = 0
        for layer in self.layers:
            if layer[0] == "pool":
                _, pooled, (oc, hw) = layer
                rc = self.E.subsample(pooled, x, self.n, oc, hw, hw, 2, 2, stream=stream.cuda_stream)
                if rc != 0:
                    raise SystemExit(f"bench.py: subsample failed rc={rc}: {self.E.last_error()}")
                self.pool_launches += 1
                x = pooled
                continue
            d, out, _ = layer
            if events is not None:
                events[i][0].record(stream)
            rc = d.enqueue(out, x, None, None, stream.cuda_stream)
            if rc != 0:
                raise SystemExit(f"bench.py: enqueue failed rc={rc}: {self.E.last_error()}")
            if events is not None:
                events[i][1].record(stream)
            x = out
            i += 1
        return x

    def launches(self):
        return sum(l[0].launch_count() for l in self.layers if l[0] != "pool") + self.pool_launches

    def close(self):
        for l in self.layers:
            if l[0] != "pool":
                l[0].close()


def vgg_input(n, int8):
    """Blocked network input: 3 channels zero-padded to 16 (fp32 U[-1,1] / u8 U[0,255])."""
    import numpy as np
    import refutil as R
    g = np.random.Generator(np.random.Philox(R.seed_for("vgg16", "input")))
    if int8:
        x = g.integers(0, 256, (n, 3, 224, 224), dtype=np.uint8)
    else:
        x = g.uniform(-1.0, 1.0, (n, 3, 224, 224)).astype(np.float32)
    return R.to_nChw16c(x)


def vgg_calibrate(device):
    """Per-tensor u8 scales of the INT8 stack, frozen before anything is timed: the fp32 stack runs
    once on two images of de-quantised input (scale 1/255) and every layer's scale is its largest
    activation / 255 (zero points are 0: activations are post-ReLU)."""
    import torch
    st = VggStack(2, False, device)
    x = torch.from_numpy(vgg_input(2, True)).cuda().to(torch.float32) * (1.0 / 255.0)
    scales = [1.0 / 255.0]
    s = torch.cuda.current_stream()
    for layer in st.layers:
        if layer[0] == "pool":
            x = x[:, :, ::2, ::2, :].contiguous()
            continue
        d, out, _ = layer
        assert d.enqueue(out, x, None, None, s.cuda_stream) == 0
        x = out
        scales.append(float(out.max().item()) / 255.0)
    torch.cuda.synchronize()
    st.close()
    return scales


def run_stack(args, wl, rank, world, local_rank):
    import numpy as np
    import torch
    int8 = args.workload == "c5i8"
    n = args.batch or 32
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
    scales = vgg_calibrate(local_rank) if int8 else None
    st = VggStack(n, int8, local_rank, scales)
    x_np = vgg_input(n, int8)
    x = torch.from_numpy(x_np).cuda()
    stream = torch.cuda.Stream()
    sampler = ClockSampler(local_rank)
    sampler.start()
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            y = st.run(x, stream)
    torch.cuda.synchronize()
    # per-layer times (one untimed pass with events around every convolution)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in st.names]
    with torch.cuda.stream(stream):
        st.run(x, stream, evs)
    torch.cuda.synchronize()
    layer_ms = [a.elapsed_time(b) for a, b in evs]
    # K steps in one CUDA graph, replayed between two events
    l0 = st.launches()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for _ in range(args.steps):
            y = st.run(x, stream)
    launches = st.launches() - l0
    with torch.cuda.stream(stream):
        graph.replay()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.active = True
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        ev0.record(stream)
        graph.replay()
        ev1.record(stream)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    ms_total = ev0.elapsed_time(ev1)
    t_end = time.perf_counter() + 0.3
    with torch.cuda.stream(stream):
        while time.perf_counter() < t_end:
            graph.replay()
            stream.synchronize()
    sampler.active = False
    # end to end: network input from pinned host memory every step, last activation back to the host
    hx = torch.from_numpy(x_np).pin_memory()
    hy = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        with torch.cuda.stream(stream):
            xd = hx.to("cuda", non_blocking=True)
            yd = st.run(xd, stream)
            hy.copy_(yd, non_blocking=True)
        stream.synchronize()
    for _ in range(2):
        e2e_step()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    sampler.stop()
    ms_total, e2e_ms = max_over_ranks([ms_total, e2e_ms], dist)
    ms_step = ms_total / args.steps
    ops = st.ops
    value = aggregate_throughput(ops, ms_step, world)
    peaks, peak_kind = measured_peaks()
    act_bytes = x_np.nbytes + sum(l[1].numel() * l[1].element_size() + (0 if i == 0 else 0)
                                  for i, l in enumerate(st.layers) if l[0] != "pool")
    # every layer reads its input and writes its output once: inputs are the previous outputs
    # (a quarter of them after a pooling stage)
    alg_bytes = 0
    prev = x_np.nbytes
    for l in st.layers:
        if l[0] == "pool":
            prev //= 4
            alg_bytes += 2 * prev       # the subsample kernel reads a quarter of the pixels and writes them
            continue
        ob = l[1].numel() * l[1].element_size()
        alg_bytes += prev + ob
        prev = ob
    slow = int(np.argmax(layer_ms))
    line = {"metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: {wl['desc']}", "batch_per_gpu": n, "global_batch": n * world,
                       "parallelism": f"minibatch split, {world} x replicated weights, {n} images per GPU",
                       "cache": "one step streams more than 1 GB of activations through the 126 MB L2",
                       "layers": [{"name": nm, "ms": round(ms, 4), "tops": round(l[2].cal_ops() / ms / 1e9, 2)}
                                  for nm, ms, l in zip(st.names, layer_ms, [q for q in st.layers if q[0] != "pool"])],
                       **({"u8_scales": [round(v, 6) for v in scales]} if int8 else {})},
            "clocks": sampler.summary(),
            "e2e": {"value": aggregate_throughput(ops, e2e_ms / e2e_steps, world), "unit": wl["unit"],
                    "h2d_bytes_per_step": x_np.nbytes, "d2h_bytes_per_step": hy.numel() * hy.element_size(),
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": alg_bytes / (ms_step * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": alg_bytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": peak_kind, "algorithmic_bytes_per_launch": alg_bytes,
                         "kernel": "whole stack (slowest layer: %s)" % st.names[slow],
                         "launches_per_step": launches / args.steps},
            "cal_ops_per_step": ops}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = stack_cpu_baseline(int8, n, wl)
    if rank == 0:
        print(json.dumps(line))
    st.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


def stack_cpu_baseline(int8, n, wl, steps=2):
    """The 13 layers through the reference's CPU library on a bounded sample (2 images per call),
    per-layer times summed and scaled to the n-image batch."""
    import refutil as R
    n_s = 2
    total_ms, ops, k = 0.0, 0, 0
    for item in VGG16:
        if item == "pool":
            continue
        ic, oc, hw = item
        case = vgg_layer_case(k, ic, oc, hw, n_s, int8, 1.0 / 255.0 if k == 0 else 0.02, 0.02)
        case = dataclasses.replace(case, knobs=dict(blk_i=max(1, R.alignup(ic) // 16), blk_o=1, flt_o=1,
                                                                  flt_t=min(hw, 14)) if int8 else {})
        t = R.make_tensors(case)
        r = cpu_reference_run(case, t, steps, 1)
        total_ms += r["ms_per_step"] * (n / n_s)
        ops += case.cal_ops() * (n // n_s)
        k += 1
    value = ops / (total_ms * 1e-3) / 1e12
    sample = (f"each of the 13 layers on {n_s} images ({steps} timed calls after the weight-transform call), summed "
              f"and scaled to {n} images; {r['sample']}")
    return {"value": value, "unit": wl["unit"], "cores": os.cpu_count() or 1, "kind": r["kind"], "sample": sample,
            "ms_per_step": total_ms}


def run_stack_reference(args, wl, rank):
    """Reference arm of the VGG-16 stack (rank 0 only)."""
    if rank != 0:
        return 0
    n = args.batch or 32
    cb = stack_cpu_baseline(args.workload == "c5i8", n, wl, max(2, min(args.steps, 4)))
    value, total_ms = cb["value"], cb.pop("ms_per_step")
    line = {"impl": "reference", "metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: {wl['desc']}", "batch_per_gpu": n},
            "cpu_baseline": cb,
            "e2e": {"value": value, "unit": wl["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


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
    if args.workload in ("c5", "c5i8"):
        if args.impl == "reference":
            return run_stack_reference(args, wl, rank)
        import torch
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device -- this library has no CPU path")
        return run_stack(args, wl, rank, world, local_rank)
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
    if os.environ.get("ELB_BENCH_SETS"):      # experiments only: e.g. 1 = operands stay in L2 (not a valid bench number)
        nsets = int(os.environ["ELB_BENCH_SETS"])
        config["cache"] = f"EXPERIMENT: {nsets} buffer set(s)"
    x0 = torch.from_numpy(t["input"]).cuda()
    xs = [x0] + [x0.clone() for _ in range(nsets - 1)]
    if case.sum:      # in-place sum: the output tensors start as the residual
        r0 = torch.from_numpy(t["residual"]).cuda().reshape(-1)
        os_ = [r0.clone() for _ in range(nsets)]
    else:
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

    # ---- Winograd: time each of the three kernels of a step live (events on the launching stream
    # between the kernels, over buffer sets the previous steps pushed out of L2)
    stage_ms = None
    if case.algo == "wino" or d.kernel == "f32_direct_umma":
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

    # ---- end to end through the drop-in call with pinned host buffers
    hx = torch.from_numpy(t["input"]).pin_memory()
    ho = (torch.from_numpy(t["residual"]).reshape(-1).clone() if case.sum else torch.zeros(out_elems, dtype=out_dtype)).pin_memory()
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

    # optional exchange step, outside the convolution timing: every rank gathers all output slabs
    # (what a caller would do to hold the full minibatch on one device); device-timed, max over ranks
    gather_ms = 0.0
    if dist is not None:
        full = torch.empty(world * out_elems, dtype=out_dtype, device="cuda")
        for _ in range(2):
            dist.all_gather_into_tensor(full, os_[0])
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            dist.all_gather_into_tensor(full, os_[0])
        g1.record()
        torch.cuda.synchronize()
        gather_ms = g0.elapsed_time(g1) / 5
        del full
    ms_total, e2e_ms, gather_ms = max_over_ranks([ms_total, e2e_ms, gather_ms], dist, device="cuda")
    if dist is not None:
        config["output_all_gather_ms"] = round(gather_ms, 4)

    ms_step = ms_total / args.steps
    value = aggregate_throughput(ops, ms_step, world)
    e2e_value = aggregate_throughput(ops, e2e_ms / e2e_steps, world)

    peaks, peak_kind = measured_peaks()
    roofline = roofline_of(args.workload, case, d, alg_bytes, ms_step, stage_ms, peaks, peak_kind,
                           launches / args.steps, args.batch)

    line = {"metric": wl["metric"], "value": value, "unit": wl["unit"], "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / PUBLISHED[args.workload]) if args.workload in PUBLISHED else None,
            "dtype": wl["dtype"], "data": "synthetic", "config": config,
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": wl["unit"], "h2d_bytes_per_step": in_bytes + (out_bytes if case.sum else 0),
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
