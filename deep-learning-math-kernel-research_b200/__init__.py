"""euler-b200: B200 (sm_100a) convolution kernels behind the Euler API.

This package is the Python door to the C-ABI library ``lib/libeuler_b200.so`` (sources in
``csrc/``, interface in ``include/euler_b200.h``).  It mirrors the reference's public surface
(``include/euler.hpp``): an ``eld_conv_t`` descriptor with the same field names, ``setup()`` and
``elx_conv(desc, output, input, weights, bias)``.

There is no CPU implementation here.  Importing works without a GPU (the library loads and its
symbols can be inspected), but every compute call needs an sm_100 device and fails loudly
otherwise; a missing or stale shared library raises at import time.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path
from types import SimpleNamespace

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
LIB_PATH = PKG_DIR / "lib" / "libeuler_b200.so"
HOST_LIB_PATH = PKG_DIR / "lib" / "libel.so"

# ----------------------------------------------------------------------------- constants
ELB_OK, ELB_UNIMPLEMENTED, ELB_GENERAL_ERROR = 0, 1, 2
ELD_OK, ELD_UNIMPLEMENTED, ELD_GENERAL_ERROR = 0, 1, 2
ELX_OK, ELX_UNIMPLEMENTED, ELX_GENERAL_ERROR = 0, 1, 2
CONV_AUTO, CONV_DIRECT_1X1, CONV_DIRECT, CONV_DIRECT_VMG, CONV_WINOGRAD, DECONV_DIRECT = range(6)
data_type_undef, f32, f16, u8, s8, s32 = range(6)
(format_undef, nchw, nhwc, nChw16c, nChw8c, oihw, hwio, OIhw16i16o, OIhw8i8o, goihw, ghwio, gOIhw16i16o,
 gOIhw8i8o) = range(13)
forward_training, forward_inference, backward_data, backward_weights = range(4)
FINE, COARSE, CALIBRATED = range(3)
EL_NO_CALI = 3.4028234663852886e38
KERNEL_NAMES = {0: "none", 1: "i8_gemm_umma", 2: "i8_conv_umma", 3: "i8_simt", 4: "wino_f32_umma",
                5: "wino_i8_umma", 6: "i8_depthwise", 7: "f32_direct_umma", 8: "f32_small_ic"}


def build(verbose: bool = False) -> Path:
    """Compile the CUDA library and the C++ host library (see _build.py)."""
    from . import _build
    return _build.build(verbose)


# ----------------------------------------------------------------------------- C structs
class ElbConvDesc(C.Structure):
    _fields_ = [(k, C.c_int32) for k in
                ("n", "g", "ic", "oc", "ih", "iw", "oh", "ow", "kh", "kw", "pad_l", "pad_r", "pad_t", "pad_b",
                 "stride_h", "stride_w", "dilation_h", "dilation_w", "dt_input", "dt_weights", "dt_output",
                 "dt_bias", "fmt_input", "fmt_weights", "fmt_output", "prop_kind", "algorithm", "tile_size",
                 "with_relu", "with_bias", "with_ip_sum", "with_op_sum", "with_argmax", "f16c_opt",
                 "disable_autoparam")] + \
               [("relu_lower", C.c_float), ("relu_upper", C.c_float), ("execution_mode", C.c_int32)] + \
               [(k, C.c_float) for k in ("input_scale", "input_z", "tinput_scale", "tinput_z", "output_scale",
                                         "output_z", "sum_scale", "sum_z")] + \
               [("sampling_kind", C.c_int32), ("flatting_t", C.c_int32), ("device", C.c_int32)]


class ElbConvInfo(C.Structure):
    _fields_ = [("algorithm", C.c_int32), ("tile_size", C.c_int32), ("kernel", C.c_int32), ("device", C.c_int32)] + \
               [(k, C.c_uint64) for k in ("size_input", "size_weights", "size_output", "size_bias", "bytes_input",
                                          "bytes_weights", "bytes_output", "bytes_bias", "workspace_bytes")] + \
               [("launches_per_call", C.c_int32), ("reserved", C.c_int32)]


def _load():
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; g.build()'` "
                          "(there is no CPU fallback)")
    lib = C.CDLL(str(LIB_PATH))
    vp, i32, u64 = C.c_void_p, C.c_int32, C.c_uint64
    sig = {
        "elb_conv_sizes": (i32, [C.POINTER(ElbConvDesc), C.POINTER(ElbConvInfo)]),
        "elb_conv_create": (i32, [C.POINTER(ElbConvDesc), C.POINTER(vp)]),
        "elb_conv_info": (i32, [vp, C.POINTER(ElbConvInfo)]),
        "elb_conv_execute": (i32, [vp, vp, vp, vp, vp]),
        "elb_conv_enqueue": (i32, [vp, vp, vp, vp, vp, vp]),
        "elb_conv_input_step_supported": (i32, [vp]),
        "elb_conv_enqueue_strided": (i32, [vp, vp, vp, i32, i32, i32, vp]),
        "elb_conv_prepare": (i32, [vp, vp, vp]),
        "elb_conv_set_accumulator_dump": (i32, [vp, vp]),
        "elb_conv_device_status": (i32, [vp]),
        "elb_conv_launch_count": (u64, [vp]),
        "elb_conv_set_stage_events": (i32, [vp, C.POINTER(vp)]),
        "elb_conv_destroy": (None, [vp]),
        "elb_last_error": (C.c_char_p, []),
        "elb_device_supported": (i32, [i32]),
        "elb_reorder_nchw_to_nChw16c": (i32, [vp, vp, i32, i32, i32, i32, i32, vp]),
        "elb_reorder_nChw16c_to_nchw": (i32, [vp, vp, i32, i32, i32, i32, i32, vp]),
        "elb_reorder": (i32, [vp, i32, vp, i32, i32, i32, i32, i32, i32, i32, vp]),
        "elb_subsample_nChw16c": (i32, [vp, vp, i32, i32, i32, i32, i32, i32, i32, vp]),
        "elb_selftest_bounded_wait": (i32, [i32, C.c_ulonglong]),
        "elb_conv_set_trace": (i32, [vp, vp]),
        "elb_conv_execute_async": (i32, [vp, vp, vp, vp, vp]),
        "elb_conv_wait": (i32, [vp]),
        "elb_conv_set_name": (i32, [vp, C.c_char_p]),
        "elb_stack_create": (i32, [C.POINTER(ElbConvDesc), C.POINTER(i32), i32, C.POINTER(vp)]),
        "elb_stack_prepare": (i32, [vp, i32, vp, vp]),
        "elb_stack_enqueue": (i32, [vp, vp, vp, vp]),
        "elb_stack_execute": (i32, [vp, vp, vp, C.c_int64]),
        "elb_stack_layer": (i32, [vp, i32, C.POINTER(vp)]),
        "elb_stack_sizes": (i32, [vp, C.POINTER(i32), C.POINTER(u64), C.POINTER(u64)]),
        "elb_stack_launch_count": (u64, [vp]),
        "elb_stack_layer_output": (i32, [vp, i32, C.POINTER(vp), C.POINTER(u64)]),
        "elb_stack_set_layer_events": (i32, [vp, C.POINTER(vp), i32]),
        "elb_stack_destroy": (None, [vp]),
        "elb_conv_multi_create": (i32, [C.POINTER(ElbConvDesc), C.POINTER(i32), i32, C.POINTER(vp)]),
        "elb_conv_multi_execute": (i32, [vp, vp, vp, vp, vp]),
        "elb_conv_multi_parts": (i32, [vp, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)]),
        "elb_conv_multi_destroy": (None, [vp]),
        "elb_wino_f32_conv_noalloc": (i32, [C.POINTER(ElbConvDesc), vp, vp, vp, vp, vp]),
        "elb_wino_f32_noalloc_status": (i32, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)          # AttributeError here = stale library
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()
EXPORTED_SYMBOLS = ["elb_conv_sizes", "elb_conv_create", "elb_conv_info", "elb_conv_execute", "elb_conv_enqueue",
                    "elb_conv_prepare", "elb_conv_set_accumulator_dump", "elb_conv_device_status",
                    "elb_conv_launch_count", "elb_conv_set_stage_events", "elb_conv_destroy", "elb_last_error", "elb_device_supported",
                    "elb_reorder_nchw_to_nChw16c", "elb_reorder_nChw16c_to_nchw", "elb_reorder", "elb_subsample_nChw16c",
                    "elb_conv_execute_async", "elb_conv_wait", "elb_conv_set_name", "elb_conv_set_trace",
                    "elb_selftest_bounded_wait", "elb_stack_create", "elb_stack_prepare", "elb_stack_enqueue",
                    "elb_stack_execute", "elb_stack_layer", "elb_stack_sizes", "elb_stack_launch_count",
                    "elb_stack_layer_output", "elb_stack_set_layer_events", "elb_stack_destroy", "elb_conv_multi_create", "elb_conv_multi_execute", "elb_conv_multi_parts",
                    "elb_conv_multi_destroy", "elb_wino_f32_conv_noalloc", "elb_wino_f32_noalloc_status",
                    "elb_conv_input_step_supported", "elb_conv_enqueue_strided"]


def last_error() -> str:
    return lib.elb_last_error().decode()


def _ptr(x):
    """Address of a torch tensor / numpy array / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if hasattr(x, "ctypes"):
        return x.ctypes.data
    raise TypeError(f"cannot take the address of {type(x)}")


class eld_conv_t:
    """Python mirror of ``euler::eld_conv_t`` (include/euler.hpp:110-187): same field names, same
    defaults (src/eld_conv.cpp:21-50), ``setup()`` returns ELD_* codes and fills ``sizes`` /
    ``byte_sizes``; the plan (``xc``) is released by ``close()`` or garbage collection."""

    def __init__(self):
        self.dims = SimpleNamespace(n=0, g=1, ic=0, oc=0, ih=0, iw=0, oh=0, ow=0, kh=0, kw=0)
        self.pads = SimpleNamespace(l=1, r=1, t=1, b=1)
        self.strides = SimpleNamespace(h=1, w=1)
        self.dilations = SimpleNamespace(h=1, w=1)
        self.data_type = SimpleNamespace(input=f32, weights=f32, output=f32, bias=f32)
        self.formats = SimpleNamespace(input=nChw16c, weights=OIhw16i16o, output=nChw16c)
        self.prop_kind = forward_inference
        self.algorithm = CONV_DIRECT
        self.tile_size = 0
        self.with_relu = self.with_bias = self.with_ip_sum = self.with_op_sum = self.with_argmax = False
        self.f16c_opt = False
        self.is_inference = True
        self.use_scratch_pad = False
        self.disable_autoparam = True
        self.eager_mode = True
        self.stream_sync = False
        self.relu_bound = SimpleNamespace(lower=0.0, upper=EL_NO_CALI)
        self.nthreads = 0
        self.execution_mode = 0
        self.flatting = SimpleNamespace(o=0, t=0)
        self.blocking = SimpleNamespace(i=0, o=0)
        self.partition = SimpleNamespace(i=1, o=1, g=1)
        self.streaming_hint = SimpleNamespace(input=0, output=0)
        self.input_quant = SimpleNamespace(scale=EL_NO_CALI, z=EL_NO_CALI)
        self.wino_tinput_quant = SimpleNamespace(scale=EL_NO_CALI, z=EL_NO_CALI)
        self.output_quant = SimpleNamespace(scale=EL_NO_CALI, z=EL_NO_CALI)
        self.sum_quant = SimpleNamespace(scale=1.0, z=0.0)
        self.sampling_kind = FINE
        self.name = "ioi"
        self.device = -1
        self.sizes = SimpleNamespace(input=0, weights=0, output=0, bias=0)
        self.byte_sizes = SimpleNamespace(input=0, weights=0, output=0, bias=0)
        self.xc = None
        self.info = None

    def _c_desc(self) -> ElbConvDesc:
        d, p = self.dims, self.pads
        return ElbConvDesc(
            d.n, d.g, d.ic, d.oc, d.ih, d.iw, d.oh, d.ow, d.kh, d.kw, p.l, p.r, p.t, p.b, self.strides.h,
            self.strides.w, self.dilations.h, self.dilations.w, self.data_type.input, self.data_type.weights,
            self.data_type.output, self.data_type.bias, self.formats.input, self.formats.weights,
            self.formats.output, self.prop_kind, self.algorithm, self.tile_size, int(self.with_relu),
            int(self.with_bias), int(self.with_ip_sum), int(self.with_op_sum), int(self.with_argmax),
            int(self.f16c_opt), int(self.disable_autoparam), self.relu_bound.lower, self.relu_bound.upper,
            self.execution_mode, self.input_quant.scale, self.input_quant.z, self.wino_tinput_quant.scale,
            self.wino_tinput_quant.z, self.output_quant.scale, self.output_quant.z, self.sum_quant.scale,
            self.sum_quant.z, int(self.sampling_kind), int(self.flatting.t), self.device)

    def setup(self, fully_setup: bool = True) -> int:
        desc = self._c_desc()
        info = ElbConvInfo()
        self.close()
        if fully_setup:
            plan = C.c_void_p()
            rc = lib.elb_conv_create(C.byref(desc), C.byref(plan))
            if rc != ELB_OK:
                return rc
            self.xc = plan
            lib.elb_conv_info(self.xc, C.byref(info))
            lib.elb_conv_set_name(self.xc, str(self.name).encode())
        else:
            rc = lib.elb_conv_sizes(C.byref(desc), C.byref(info))
            if rc != ELB_OK:
                return rc
        self.info = info
        self.algorithm, self.tile_size = info.algorithm, info.tile_size
        self.sizes = SimpleNamespace(input=info.size_input, weights=info.size_weights, output=info.size_output,
                                     bias=info.size_bias)
        self.byte_sizes = SimpleNamespace(input=info.bytes_input, weights=info.bytes_weights,
                                          output=info.bytes_output, bias=info.bytes_bias)
        return ELD_OK

    @property
    def kernel(self) -> str:
        return KERNEL_NAMES.get(self.info.kernel if self.info else 0, "?")

    def prepare(self, weights, bias) -> int:
        return lib.elb_conv_prepare(self.xc, _ptr(weights), _ptr(bias))

    def enqueue(self, output, input, weights=None, bias=None, stream=None) -> int:
        """Device pointers only; returns after the kernels are enqueued on ``stream``."""
        return lib.elb_conv_enqueue(self.xc, _ptr(output), _ptr(input), _ptr(weights), _ptr(bias), stream)

    def input_step_supported(self) -> bool:
        return bool(lib.elb_conv_input_step_supported(self.xc))

    def enqueue_strided(self, output, input, src_h: int, src_w: int, step: int, stream=None) -> int:
        """As enqueue on a prepared plan, but ``input`` holds src_h x src_w pixels per plane of which every
        ``step``-th row and column is read (a subsample folded into the kernel's loads)."""
        return lib.elb_conv_enqueue_strided(self.xc, _ptr(output), _ptr(input), src_h, src_w, step, stream)

    def set_accumulator_dump(self, dev_int32) -> int:
        return lib.elb_conv_set_accumulator_dump(self.xc, _ptr(dev_int32))

    def device_status(self) -> int:
        return lib.elb_conv_device_status(self.xc)

    def launch_count(self) -> int:
        return int(lib.elb_conv_launch_count(self.xc))

    def set_stage_events(self, handles) -> int:
        """Four cudaEvent_t handles (ints) recorded around the three Winograd kernels; None = off."""
        if handles is None:
            return lib.elb_conv_set_stage_events(self.xc, None)
        arr = (C.c_void_p * 4)(*[int(h) for h in handles])
        return lib.elb_conv_set_stage_events(self.xc, arr)

    def wait(self) -> int:
        """Complete the asynchronous calls made with ``eager_mode = False`` (what a later call with
        ``stream_sync = True`` does in the reference, src/elx_conv.cpp:234-235)."""
        return lib.elb_conv_wait(self.xc)

    def close(self):
        if self.xc is not None:
            lib.elb_conv_destroy(self.xc)
            self.xc = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def elx_conv(desc: eld_conv_t, output, input, weights, bias) -> int:
    """``euler::elx_conv`` (include/euler.hpp:190): run the convolution and wait.  Arguments may be
    torch tensors (CUDA or CPU), numpy arrays or raw addresses; output comes first."""
    if desc.xc is None:
        raise RuntimeError("elx_conv: descriptor is not set up")
    if desc.eager_mode:
        return lib.elb_conv_execute(desc.xc, _ptr(output), _ptr(input), _ptr(weights), _ptr(bias))
    # eager_mode = False: enqueue and return; stream_sync = True waits (src/elx_conv.cpp:228-236)
    rc = lib.elb_conv_execute_async(desc.xc, _ptr(output), _ptr(input), _ptr(weights), _ptr(bias))
    if rc == ELB_OK and desc.stream_sync:
        rc = lib.elb_conv_wait(desc.xc)
    return rc


def _elem_bytes(x) -> int:
    if hasattr(x, "element_size"):
        return x.element_size()
    return x.dtype.itemsize


def reorder(dst, dst_format: int, src, src_format: int, *dims, stream=None) -> int:
    """``euler::reorder<T, dst_format, src_format>(dst, src, dims...)`` (include/euler_reorder.hpp:9-64)
    for DEVICE tensors: dims are (n, c, h, w), (o, i, h, w) or (g, o, i, h, w) as in the reference.
    The call is asynchronous on ``stream`` (default stream when None)."""
    if len(dims) == 4:
        g, (a, b, h, w) = 1, dims
    elif len(dims) == 5:
        g, a, b, h, w = dims
    else:
        raise ValueError("reorder takes 4 or 5 extents")
    return lib.elb_reorder(_ptr(dst), dst_format, _ptr(src), src_format, g, a, b, h, w, _elem_bytes(src), _ptr(stream))


def subsample(dst, src, n: int, c: int, h: int, w: int, step_h: int = 2, step_w: int = 2, stream=None) -> int:
    """Keep every step_h-th row and step_w-th column of a device nChw16c tensor (the glue between two
    layers of a stack; the reference's harness chains layers on the host, tests/elt_conv.cpp:399-410)."""
    return lib.elb_subsample_nChw16c(_ptr(dst), _ptr(src), n, c, h, w, step_h, step_w, _elem_bytes(src), _ptr(stream))


class ConvStack:
    """A chain of convolutions that stays on the device (``elb_stack_*``): ``descs`` are set-up-able
    ``eld_conv_t`` descriptors, ``subsample_after[k]`` = 2 keeps every second row and column of layer
    k's output.  The reference's harness chains layers on the host (tests/elt_conv.cpp:399-410)."""

    def __init__(self, descs, subsample_after=None):
        n = len(descs)
        arr = (ElbConvDesc * n)(*[d._c_desc() for d in descs])
        steps = (C.c_int32 * n)(*[int(v) for v in (subsample_after or [1] * n)])
        h = C.c_void_p()
        rc = lib.elb_stack_create(arr, steps, n, C.byref(h))
        if rc != ELB_OK:
            raise RuntimeError(f"elb_stack_create rc={rc}: {last_error()}")
        self.h, self.n_layers = h, n
        nl, bi, bo = C.c_int32(), C.c_uint64(), C.c_uint64()
        lib.elb_stack_sizes(self.h, C.byref(nl), C.byref(bi), C.byref(bo))
        self.bytes_input, self.bytes_output = bi.value, bo.value

    def prepare(self, layer: int, weights, bias) -> int:
        return lib.elb_stack_prepare(self.h, layer, _ptr(weights), _ptr(bias))

    def enqueue(self, output, input, stream=None) -> int:
        return lib.elb_stack_enqueue(self.h, _ptr(output), _ptr(input), stream)

    def execute(self, output, input, images: int) -> int:
        return lib.elb_stack_execute(self.h, _ptr(output), _ptr(input), images)

    def layer_plan(self, layer: int):
        p = C.c_void_p()
        lib.elb_stack_layer(self.h, layer, C.byref(p))
        return p

    def layer_kernel(self, layer: int) -> str:
        info = ElbConvInfo()
        lib.elb_conv_info(self.layer_plan(layer), C.byref(info))
        return KERNEL_NAMES.get(info.kernel, "?")

    def launch_count(self) -> int:
        return int(lib.elb_stack_launch_count(self.h))

    def layer_output(self, layer: int):
        """(device address, bytes) of layer k's output tensor inside the stack; address None for the last layer."""
        p, b = C.c_void_p(), C.c_uint64()
        lib.elb_stack_layer_output(self.h, layer, C.byref(p), C.byref(b))
        return p.value, b.value

    def set_layer_events(self, handles) -> int:
        if handles is None:
            return lib.elb_stack_set_layer_events(self.h, None, 0)
        arr = (C.c_void_p * len(handles))(*[int(h) for h in handles])
        return lib.elb_stack_set_layer_events(self.h, arr, len(handles))

    def close(self):
        if self.h is not None:
            lib.elb_stack_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MultiConv:
    """One convolution whose minibatch is split over the GPUs of this box (``elb_conv_multi_*``):
    GPU r runs images [r*N/G, (r+1)*N/G) of the host tensors; weights are replicated."""

    def __init__(self, desc: eld_conv_t, devices=None, n_devices: int = 0):
        cd = desc._c_desc()
        h = C.c_void_p()
        arr = (C.c_int32 * len(devices))(*devices) if devices else None
        rc = lib.elb_conv_multi_create(C.byref(cd), arr, len(devices) if devices else n_devices, C.byref(h))
        if rc != ELB_OK:
            raise RuntimeError(f"elb_conv_multi_create rc={rc}: {last_error()}")
        self.h = h

    def parts(self):
        n = C.c_int32(64)
        dev, first, cnt = (C.c_int32 * 64)(), (C.c_int32 * 64)(), (C.c_int32 * 64)()
        lib.elb_conv_multi_parts(self.h, C.byref(n), dev, first, cnt)
        return [(dev[i], first[i], cnt[i]) for i in range(n.value)]

    def execute(self, output, input, weights, bias) -> int:
        return lib.elb_conv_multi_execute(self.h, _ptr(output), _ptr(input), _ptr(weights), _ptr(bias))

    def close(self):
        if self.h is not None:
            lib.elb_conv_multi_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
