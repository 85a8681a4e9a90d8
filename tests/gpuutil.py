"""Helpers of the GPU parity tests: build a descriptor from a ConvCase and run it through the
C-ABI with device-resident or host tensors."""
from __future__ import annotations

import importlib

import numpy as np

from refutil import ConvCase, out_shape


def package():
    return importlib.import_module("deep-learning-math-kernel-research_b200")


def make_desc(case: ConvCase, device: int = -1):
    E = package()
    d = E.eld_conv_t()
    d.dims.n, d.dims.g, d.dims.ic, d.dims.oc = case.n, case.g, case.ic, case.oc
    d.dims.ih, d.dims.iw, d.dims.oh, d.dims.ow = case.ih, case.iw, case.oh, case.ow
    d.dims.kh, d.dims.kw = case.kh, case.kw
    d.pads.l = d.pads.r = d.pads.t = d.pads.b = case.pad
    d.strides.h = d.strides.w = case.stride
    tin, tout = {"fp32": (E.f32, E.f32), "u8f32u8f32": (E.u8, E.u8), "u8f32s8f32": (E.u8, E.s8),
                 "u8f32f32f32": (E.u8, E.f32)}[case.types]
    d.data_type.input, d.data_type.weights, d.data_type.output, d.data_type.bias = tin, E.f32, tout, E.f32
    d.formats.weights = E.goihw if case.g > 1 else E.OIhw16i16o
    fmts = {"nchw": E.nchw, "nhwc": E.nhwc, "oihw": E.oihw, "hwio": E.hwio, "ghwio": E.ghwio}
    if case.ifmt:
        d.formats.input = fmts[case.ifmt]
    if case.ofmt:
        d.formats.output = fmts[case.ofmt]
    if case.wfmt:
        d.formats.weights = fmts[case.wfmt]
    d.algorithm = {"auto": E.CONV_AUTO, "direct": E.CONV_DIRECT, "1x1": E.CONV_DIRECT_1X1,
                   "wino": E.CONV_WINOGRAD}[case.algo]
    d.tile_size = case.tile
    d.with_relu, d.with_bias, d.with_ip_sum = case.relu, case.bias, case.sum
    if case.types != "fp32":
        d.input_quant.scale, d.input_quant.z = case.iscale, case.iz
        d.output_quant.scale, d.output_quant.z = case.oscale, case.oz
        d.sum_quant.scale, d.sum_quant.z = case.sscale, case.sz
        if case.tscale is not None:
            d.wino_tinput_quant.scale, d.wino_tinput_quant.z = case.tscale, case.tz
        d.sampling_kind = E.CALIBRATED
    d.flatting.t = int(case.knobs.get("flt_t", 0))     # only the int8 depthwise path reads it
    d.device = device
    return d


def run_gpu(case: ConvCase, t: dict, host_buffers: bool = False, want_acc: bool = False, acc_shape=None,
            repeat: int = 1):
    """Run one case through elx_conv.  Returns (output ndarray, desc[, acc ndarray])."""
    import torch
    E = package()
    d = make_desc(case)
    rc = d.setup()
    assert rc == E.ELD_OK, f"setup rc={rc}: {E.last_error()}"
    out_np = np.zeros(out_shape(case), dtype=case.out_dtype)
    if case.sum:
        out_np[...] = t["residual"]
    acc_t = None
    if want_acc:
        acc_t = torch.zeros(acc_shape or out_shape(case), dtype=torch.int32, device="cuda")
        d.set_accumulator_dump(acc_t)
    if host_buffers:
        for _ in range(repeat):
            if case.sum:
                out_np[...] = t["residual"]
            rc = E.elx_conv(d, out_np, t["input"], t["weights"], t["bias"])
            assert rc == E.ELX_OK, f"elx_conv rc={rc}: {E.last_error()}"
        res = out_np
    else:
        x = torch.from_numpy(t["input"]).cuda()
        w = torch.from_numpy(t["weights"]).cuda()
        b = torch.from_numpy(t["bias"]).cuda()
        for _ in range(repeat):
            o = torch.from_numpy(out_np).cuda()
            rc = E.elx_conv(d, o, x, w, b)
            assert rc == E.ELX_OK, f"elx_conv rc={rc}: {E.last_error()}"
        torch.cuda.synchronize()
        res = o.cpu().numpy()
    if want_acc:
        return res, d, acc_t.cpu().numpy()
    return res, d
