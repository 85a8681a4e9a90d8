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


GUARD_BYTES = 4096          # poisoned band on either side of a guarded device tensor
GUARD_BYTE = 0xA5


class Guarded:
    """A device tensor with a poisoned band in front of it and behind it.  compute-sanitizer is not
    available to these tests, so every output (and accumulator dump) the GPU tests hand to the
    library lies between two bands of 0xA5 bytes that must still be intact afterwards: a kernel
    that writes outside the tensor it was given fails the test that ran it."""

    def __init__(self, init: np.ndarray):
        import torch
        self.nbytes = init.nbytes
        pad = (-self.nbytes) % 256
        self.raw = torch.full((GUARD_BYTES + self.nbytes + pad + GUARD_BYTES,), GUARD_BYTE, dtype=torch.uint8, device="cuda")
        self.dtype, self.shape = init.dtype, init.shape
        self.view_u8 = self.raw[GUARD_BYTES:GUARD_BYTES + self.nbytes]
        self.view_u8.copy_(torch.from_numpy(np.ascontiguousarray(init).view(np.uint8).reshape(-1)))

    def data_ptr(self) -> int:
        return self.view_u8.data_ptr()

    def numpy(self) -> np.ndarray:
        return self.view_u8.cpu().numpy().view(self.dtype).reshape(self.shape)

    def check(self, what: str = "output"):
        import torch
        torch.cuda.synchronize()
        front = self.raw[:GUARD_BYTES]
        back = self.raw[GUARD_BYTES + self.nbytes:]
        bad_f = int((front != GUARD_BYTE).sum().item())
        bad_b = int((back != GUARD_BYTE).sum().item())
        assert bad_f == 0 and bad_b == 0, (f"{what}: {bad_f} bytes in front of the tensor and {bad_b} behind it were "
                                           "overwritten (out-of-bounds write)")


def run_gpu(case: ConvCase, t: dict, host_buffers: bool = False, want_acc: bool = False, acc_shape=None,
            repeat: int = 1):
    """Run one case through elx_conv.  Returns (output ndarray, desc[, acc ndarray]).  Device
    outputs and accumulator dumps are guarded (see Guarded)."""
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
        acc_t = Guarded(np.zeros(acc_shape or out_shape(case), dtype=np.int32))
        d.set_accumulator_dump(acc_t.data_ptr())
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
            o = Guarded(out_np)
            rc = E.elx_conv(d, o.data_ptr(), x, w, b)
            assert rc == E.ELX_OK, f"elx_conv rc={rc}: {E.last_error()}"
            o.check(f"{case.name}: output tensor")
        res = o.numpy()
    if want_acc:
        acc_t.check(f"{case.name}: accumulator dump")
        return res, d, acc_t.numpy()
    return res, d
