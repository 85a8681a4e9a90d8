"""Shared helpers for the test-suite, the fixture generator and the CPU legs of bench.py.

TEST INFRASTRUCTURE: this module is the only Python door to ``oracle/`` (the CPU restatement
``oracle/liboracle.so`` and the reference build ``oracle/_ref``).  The product package never imports
it.

Contents
  * blocked-layout helpers (nchw <-> nChw16c, oihw -> OIhw16i16o) in numpy,
  * seeded synthetic tensors with the value distributions of the benchmark configurations,
  * ``ConvCase``: one convolution problem (dims, types, fusion flags, quantisation constants),
  * ctypes bindings of the oracle (``oracle_*`` functions),
  * ``run_reference``: run the unmodified reference library through ``oracle/_ref/ref_driver``.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json
import os
import subprocess
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"
REF_DIR = ORACLE_DIR / "_ref"
V = 16


def alignup(x: int, a: int = V) -> int:
    return (x + a - 1) // a * a


# ----------------------------------------------------------------------------- layouts
def to_nChw16c(x: np.ndarray) -> np.ndarray:
    """nchw -> nChw16c with zero channel padding (reference: src/elx_reorder.cpp:61-66)."""
    n, c, h, w = x.shape
    cp = alignup(c)
    buf = np.zeros((n, cp, h, w), dtype=x.dtype)
    buf[:, :c] = x
    return np.ascontiguousarray(buf.reshape(n, cp // V, V, h, w).transpose(0, 1, 3, 4, 2))


def from_nChw16c(x: np.ndarray, c: int) -> np.ndarray:
    n, c2, h, w, v = x.shape
    return np.ascontiguousarray(x.transpose(0, 1, 4, 2, 3).reshape(n, c2 * v, h, w)[:, :c])


def to_OIhw16i16o(w: np.ndarray) -> np.ndarray:
    """oihw -> OIhw16i16o ([O/16][I/16][kh][kw][16i][16o]) with zero padding
    (reference: src/elx_reorder.cpp:70-94)."""
    o, i, kh, kw = w.shape
    op, ip = alignup(o), alignup(i)
    buf = np.zeros((op, ip, kh, kw), dtype=w.dtype)
    buf[:o, :i] = w
    buf = buf.reshape(op // V, V, ip // V, V, kh, kw).transpose(0, 2, 4, 5, 3, 1)
    return np.ascontiguousarray(buf)


def weights_buffer(w_blocked: np.ndarray) -> np.ndarray:
    """Flat weights buffer with the 4*V elements of slack the reference asks for
    (src/eld_conv.cpp:105)."""
    flat = w_blocked.reshape(-1)
    return np.concatenate([flat, np.zeros(4 * V, dtype=flat.dtype)])


# ----------------------------------------------------------------------------- cases
@dataclasses.dataclass
class ConvCase:
    name: str
    n: int
    ic: int
    oc: int
    ih: int
    iw: int
    kh: int = 3
    kw: int = 3
    pad: int = 1
    stride: int = 1
    types: str = "fp32"            # fp32 | u8f32u8f32 | u8f32s8f32 | u8f32f32f32
    algo: str = "auto"             # auto | direct | 1x1 | wino
    tile: int = 0
    relu: bool = False
    bias: bool = False
    sum: bool = False
    g: int = 1
    iscale: float = 0.05
    iz: float = 0.0
    oscale: float = 0.1
    oz: float = 0.0
    sscale: float = 1.0
    sz: float = 0.0
    tscale: float | None = None
    tz: float | None = None
    knobs: dict = dataclasses.field(default_factory=dict)   # reference tuning knobs (xopt, blk_i ...)
    ifmt: str = ""                 # "" = nChw16c; "nchw" | "nhwc": plain user formats
    ofmt: str = ""
    wfmt: str = ""                 # "" = OIhw16i16o (goihw for depthwise); "oihw" | "hwio" | "ghwio"

    @property
    def oh(self) -> int:
        return (self.ih + 2 * self.pad - self.kh) // self.stride + 1

    @property
    def ow(self) -> int:
        return (self.iw + 2 * self.pad - self.kw) // self.stride + 1

    @property
    def out_dtype(self):
        return {"fp32": np.float32, "u8f32u8f32": np.uint8, "u8f32s8f32": np.int8,
                "u8f32f32f32": np.float32}[self.types]

    @property
    def in_dtype(self):
        return np.float32 if self.types == "fp32" else np.uint8

    def cal_ops(self) -> int:
        """The reference's op count: 2*N*IC*OC*(valid (oh,kh) pairs)*(valid (ow,kw) pairs)
        (tests/elt_conv_utils.cpp:638-659)."""
        def valid(o, k, i, p, s):
            return sum(1 for a in range(o) for b in range(k) if 0 <= a * s - p + b < i)
        return 2 * self.n * self.ic * self.oc // self.g * valid(self.oh, self.kh, self.ih, self.pad, self.stride) \
            * valid(self.ow, self.kw, self.iw, self.pad, self.stride)


# The benchmark configurations (shapes, distributions and knobs as the baseline document states).
def baseline_case(cid: str, n: int | None = None) -> ConvCase:
    """c3s is configuration 3 exactly as named (bias + ReLU + in-place sum of a u8 residual); c3 is
    the same layer without the sum, the variant the reference can pin bit for bit (its KxK int8
    path ignores with_ip_sum, src/elx_int8_conv_direct.cpp:121)."""
    if cid == "c1":
        return ConvCase("c1_fp32_wino_vgg_conv3_2", n or 64, 256, 256, 56, 56, types="fp32", algo="wino",
                        tile=6, relu=True, bias=True,
                        knobs=dict(xopt=0xa061, blk_i=8, blk_o=8, flt_t=28, pat_o=2))
    if cid == "c2":
        return ConvCase("c2_int8_1x1_resnet50_res4", n or 64, 1024, 256, 14, 14, kh=1, kw=1, pad=0,
                        types="u8f32u8f32", algo="1x1", relu=True, bias=True,
                        knobs=dict(xopt=0xa160, blk_i=64, blk_o=4, flt_o=4, flt_t=6))
    if cid == "c3":
        return ConvCase("c3_int8_3x3_s2", n or 64, 128, 256, 56, 56, stride=2, types="u8f32u8f32",
                        algo="direct", relu=True, bias=True,
                        knobs=dict(xopt=0xc160, blk_i=8, blk_o=4, flt_o=2, flt_t=14))
    if cid == "c3s":
        return ConvCase("c3s_int8_3x3_s2_sum", n or 64, 128, 256, 56, 56, stride=2, types="u8f32u8f32",
                        algo="direct", relu=True, bias=True, sum=True, sscale=1.0, sz=0.0,
                        knobs=dict(xopt=0xc160, blk_i=8, blk_o=4, flt_o=2, flt_t=14))
    if cid == "c4":
        return ConvCase("c4_int8_wino", n or 128, 512, 512, 28, 28, types="u8f32f32f32", algo="wino",
                        tile=6, knobs=dict(xopt=0xa161, blk_i=32, blk_o=1, flt_o=2, flt_t=11, pat_o=16))
    if cid == "v12":    # VGG-16 conv1_2, the slowest layer of the fp32 stack (64 -> 64 channels at 224x224)
        return ConvCase("v12_fp32_wino_vgg_conv1_2", n or 32, 64, 64, 224, 224, types="fp32", algo="wino", tile=6,
                        relu=True, bias=True, knobs=dict(xopt=0xa061, blk_i=4, blk_o=4, flt_t=28, pat_o=1))
    if cid == "c2f":    # the c2 layer (ResNet-50 res4 1x1 reduce) in fp32
        return ConvCase("c2f_fp32_1x1_resnet50_res4", n or 64, 1024, 256, 14, 14, kh=1, kw=1, pad=0, types="fp32",
                        algo="1x1", relu=True, bias=True, knobs=dict(blk_i=64, blk_o=1, flt_o=1, flt_t=7))
    if cid == "c3f":    # the c3 layer (3x3 stride 2) in fp32
        return ConvCase("c3f_fp32_3x3_s2", n or 64, 128, 256, 56, 56, stride=2, types="fp32", algo="direct",
                        relu=True, bias=True, knobs=dict(blk_i=8, blk_o=1, flt_o=1, flt_t=7))
    if cid == "c1t4":   # the c1 layer with tile_size 4 = F(2x2,3x3)
        return dataclasses.replace(baseline_case("c1", n), name="c1t4_fp32_wino_f2x2_vgg_conv3_2", tile=4)
    if cid == "c4t4":   # the c4 layer with tile_size 4
        return dataclasses.replace(baseline_case("c4", n), name="c4t4_int8_wino_f2x2", tile=4)
    if cid == "dw":   # MobileNet-v1 Conv2d_3_depthwise shape; chunk T = 14 as in the reference's tuned script
        return ConvCase("dw_int8_mobilenet_conv3", n or 64, 128, 128, 56, 56, g=128, types="u8f32u8f32",
                        algo="direct", relu=True, bias=True, knobs=dict(xopt=0xc160, flt_t=14))
    raise KeyError(cid)


def seed_for(case_name: str, tensor: str) -> int:
    import hashlib
    return int.from_bytes(hashlib.sha256(f"{case_name}/{tensor}".encode()).digest()[:8], "little")


def make_tensors(case: ConvCase) -> dict:
    """Seeded synthetic tensors in BLOCKED layouts.

    fp32: input U[-1,1], weights N(0, sqrt(2/(9*IC))), bias U[-0.1,0.1].
    int8: input u8 U[0,255]; weights are q*scale[oc] with q s8 U[-127,127] (one |q| = 127 per output
    channel so that the library's abs-max quantiser recovers exactly scale[oc] and q), scale[oc]
    U[0.001,0.01]; bias U[-0.1,0.1]; residual (sum) u8 U[0,255].
    """
    def rng(name):
        return np.random.Generator(np.random.Philox(seed_for(case.name, name)))
    icg = case.ic // case.g
    t = {}
    if case.types == "fp32":
        x = rng("input").uniform(-1.0, 1.0, (case.n, case.ic, case.ih, case.iw)).astype(np.float32)
        w = (rng("weights").standard_normal((case.oc, icg, case.kh, case.kw))
             * np.sqrt(2.0 / (case.kh * case.kw * icg))).astype(np.float32)
    else:
        x = rng("input").integers(0, 256, (case.n, case.ic, case.ih, case.iw), dtype=np.uint8)
        q = rng("weights").integers(-127, 128, (case.oc, icg, case.kh, case.kw)).astype(np.int32)
        flat = q.reshape(case.oc, -1)
        pos = rng("peak").integers(0, flat.shape[1], case.oc)
        sign = rng("sign").integers(0, 2, case.oc) * 2 - 1
        flat[np.arange(case.oc), pos] = 127 * sign
        scale = rng("wscale").uniform(0.001, 0.01, case.oc).astype(np.float32)
        w = (flat.reshape(q.shape).astype(np.float32) * scale[:, None, None, None]).astype(np.float32)
        t["q"] = flat.reshape(q.shape).astype(np.int8)
        t["wscale"] = scale
    t["input_plain"] = x
    t["weights_plain"] = w
    t["input"] = to_nChw16c(x)
    if case.g == 1:
        t["weights"] = weights_buffer(to_OIhw16i16o(w))
    else:   # depthwise: goihw with g = channels
        t["weights"] = weights_buffer(w.reshape(case.g, 1, 1, case.kh, case.kw).copy())
    b = rng("bias").uniform(-0.1, 0.1, case.oc).astype(np.float32)
    bb = np.zeros(alignup(case.oc), dtype=np.float32)
    bb[:case.oc] = b
    t["bias"] = bb
    if case.sum:
        ocp = alignup(case.oc)
        if case.out_dtype == np.float32:
            r = rng("residual").uniform(-1, 1, (case.n, ocp // V, case.oh, case.ow, V)).astype(np.float32)
        elif case.out_dtype == np.uint8:
            r = rng("residual").integers(0, 256, (case.n, ocp // V, case.oh, case.ow, V), dtype=np.uint8)
        else:
            r = rng("residual").integers(-128, 128, (case.n, ocp // V, case.oh, case.ow, V)).astype(np.int8)
        t["residual"] = r
    return t


# ----------------------------------------------------------------------------- oracle (ctypes)
class OrcConv(C.Structure):
    _fields_ = [(k, C.c_int32) for k in
                ("n", "ic", "oc", "ih", "iw", "oh", "ow", "kh", "kw", "pad_t", "pad_l", "stride_h",
                 "stride_w", "with_relu", "with_bias", "with_sum", "out_type")] + \
               [(k, C.c_float) for k in
                ("relu_lo", "relu_hi", "in_scale", "in_z", "out_scale", "out_z", "sum_scale", "sum_z",
                 "tin_scale", "tin_z")] + [("fused_epilogue", C.c_int32), ("tile", C.c_int32)]


_ORACLE = None


def oracle_lib():
    global _ORACLE
    if _ORACLE is None:
        so = ORACLE_DIR / "liboracle.so"
        if not so.exists():
            subprocess.check_call(["make", "-C", str(ORACLE_DIR), "liboracle.so"])
        lib = C.CDLL(str(so))
        assert lib.orc_struct_size() == C.sizeof(OrcConv)
        _ORACLE = lib
    return _ORACLE


FLT_MAX = float(np.finfo(np.float32).max)


def orc_params(case: ConvCase, fused: bool = True) -> OrcConv:
    ot = {"fp32": 0, "u8f32f32f32": 0, "u8f32u8f32": 1, "u8f32s8f32": 2}[case.types]
    return OrcConv(case.n, case.ic, case.oc, case.ih, case.iw, case.oh, case.ow, case.kh, case.kw,
                   case.pad, case.pad, case.stride, case.stride, int(case.relu), int(case.bias),
                   int(case.sum), ot, 0.0, FLT_MAX, case.iscale, case.iz, case.oscale, case.oz,
                   case.sscale, case.sz, case.tscale or 1.0, case.tz or 0.0, int(fused), int(case.tile))


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def out_shape(case: ConvCase):
    """Shape of the output tensor as the caller holds it (blocked unless the case names a plain format)."""
    if case.ofmt == "nchw":
        return (case.n, case.oc, case.oh, case.ow)
    if case.ofmt == "nhwc":
        return (case.n, case.oh, case.ow, case.oc)
    return (case.n, alignup(case.oc) // V, case.oh, case.ow, V)


def act_to_user(x_blocked: np.ndarray, c: int, fmt: str) -> np.ndarray:
    """nChw16c -> the plain activation format fmt ("" keeps it blocked)."""
    if not fmt:
        return x_blocked
    x = from_nChw16c(x_blocked, c)
    return np.ascontiguousarray(x if fmt == "nchw" else x.transpose(0, 2, 3, 1))


def act_to_blocked(x_user: np.ndarray, fmt: str) -> np.ndarray:
    if not fmt:
        return x_user
    x = x_user if fmt == "nchw" else x_user.transpose(0, 3, 1, 2)
    return to_nChw16c(np.ascontiguousarray(x))


def user_tensors(case: ConvCase, t: dict) -> dict:
    """The tensors of make_tensors (blocked layouts) in the formats the case names: what a caller with
    plain tensors passes.  Bias has oc elements when the output format is plain (src/eld_conv.cpp:112-114)."""
    u = dict(t)
    u["input"] = act_to_user(t["input"], case.ic, case.ifmt)
    if case.sum:
        u["residual"] = act_to_user(t["residual"], case.oc, case.ofmt)
    if case.ofmt:
        u["bias"] = np.ascontiguousarray(t["bias"][:case.oc])
    if case.wfmt in ("oihw", "hwio"):
        w = t["weights_plain"]                                   # [oc][ic][kh][kw]
        w = w if case.wfmt == "oihw" else w.transpose(2, 3, 1, 0)
        u["weights"] = weights_buffer(np.ascontiguousarray(w))
    return u


def oracle_int8_conv(case: ConvCase, t: dict, fused: bool = True, want_acc: bool = False):
    lib = oracle_lib()
    out = np.zeros(out_shape(case), dtype=case.out_dtype)
    acc = np.zeros(out_shape(case), dtype=np.int32) if want_acc else None
    prev = t.get("residual") if case.sum else None
    p = orc_params(case, fused)
    rc = lib.orc_int8_conv(C.byref(p), _p(t["input"]), _p(t["weights"]), _p(t["bias"]), _p(out), _p(acc),
                           _p(prev))
    assert rc == 0
    return (out, acc) if want_acc else out


def oracle_int8_depthwise(case: ConvCase, t: dict, want_acc: bool = False):
    """Depthwise 3x3 (g = ic = oc).  The chunk length T of the reference (flatting.t) comes from
    ``case.knobs['flt_t']``; it decides which pixels of a u8 output are floored and which are
    rounded to nearest."""
    lib = oracle_lib()
    out = np.zeros(out_shape(case), dtype=case.out_dtype)
    acc = np.zeros(out_shape(case), dtype=np.int32) if want_acc else None
    p = orc_params(case)
    rc = lib.orc_int8_depthwise(C.byref(p), int(case.knobs.get("flt_t", 0)), _p(t["input"]), _p(t["weights"]),
                                _p(t["bias"]), _p(out), _p(acc))
    assert rc == 0, rc
    return (out, acc) if want_acc else out


def oracle_wino_f32(case: ConvCase, t: dict):
    lib = oracle_lib()
    out = np.zeros(out_shape(case), dtype=np.float32)
    prev = t.get("residual") if case.sum else None
    p = orc_params(case)
    rc = lib.orc_wino_f32_conv(C.byref(p), _p(t["input"]), _p(t["weights"]), _p(t["bias"]), _p(out), _p(prev))
    assert rc == 0
    return out


def oracle_direct_f64(case: ConvCase, t: dict):
    lib = oracle_lib()
    out = np.zeros(out_shape(case), dtype=np.float32)
    if case.sum:
        out[...] = t["residual"]      # in-place sum: the output tensor holds the residual on entry
    p = orc_params(case)
    rc = lib.orc_direct_f64_conv(C.byref(p), _p(t["input"]), _p(t["weights"]), _p(t["bias"]), _p(out))
    assert rc == 0
    return out


def wino_edge(case: ConvCase) -> int:
    """Input tile edge A of the case's Winograd tile_size (6 unless the case asks for 4)."""
    return 4 if case.tile == 4 else 6


def wino_tiles(case: ConvCase) -> int:
    o = wino_edge(case) - 2
    return case.n * (-(-case.oh // o)) * (-(-case.ow // o))


def oracle_int8_wino(case: ConvCase, t: dict, dumps: bool = False):
    lib = oracle_lib()
    out = np.zeros(out_shape(case), dtype=case.out_dtype)
    prev = t.get("residual") if case.sum else None
    p = orc_params(case)
    T, IC, OC = wino_tiles(case), alignup(case.ic), alignup(case.oc)
    d = {}
    if dumps:
        aa = wino_edge(case) ** 2
        d = dict(tin=np.zeros((aa, T, IC), np.uint8), tw=np.zeros((aa, OC, IC), np.int8),
                 acc=np.zeros((aa, T, OC), np.int32), tout=np.zeros((aa, T, OC), np.float32))
    rc = lib.orc_int8_wino_conv(C.byref(p), _p(t["input"]), _p(t["weights"]), _p(t["bias"]), _p(out), _p(prev),
                                _p(d.get("tin")), _p(d.get("tw")), _p(d.get("acc")), _p(d.get("tout")))
    assert rc == 0
    return (out, d) if dumps else out


def oracle_tinput_range(case: ConvCase, t: dict):
    lib = oracle_lib()
    mn, mx = C.c_float(), C.c_float()
    p = orc_params(case)
    assert lib.orc_wino_tinput_range(C.byref(p), _p(t["input"]), C.byref(mn), C.byref(mx)) == 0
    return mn.value, mx.value


def calibrate_tinput(case: ConvCase, t: dict) -> ConvCase:
    """wino_tinput_quant as the reference's test derives it: scale = (max-min)/127,
    z = -min*127/(max-min) (tests/elt_conv_utils.cpp:238-255)."""
    mn, mx = oracle_tinput_range(case, t)
    scale = np.float32((np.float32(mx) - np.float32(mn)) / np.float32(127.0))
    z = np.float32(-np.float32(mn) * np.float32(127.0) / (np.float32(mx) - np.float32(mn)))
    return dataclasses.replace(case, tscale=float(scale), tz=float(z))


# ----------------------------------------------------------------------------- reference library
def reference_available() -> bool:
    """The reference build needs AVX-512 VNNI on the host it runs on."""
    if not (REF_DIR / "ref_driver").exists() or not (REF_DIR / "libel.so").exists():
        return False
    try:
        flags = Path("/proc/cpuinfo").read_text()
    except OSError:
        return False
    return all(f in flags for f in ("avx512f", "avx512bw", "avx512dq", "avx512vl", "avx512_vnni"))


def reference_args(case: ConvCase, knobs: bool = True) -> list:
    a = [f"n={case.n}", f"g={case.g}", f"ic={case.ic}", f"oc={case.oc}", f"ih={case.ih}", f"iw={case.iw}",
         f"kh={case.kh}", f"kw={case.kw}", f"pt={case.pad}", f"pl={case.pad}", f"sh={case.stride}",
         f"types={case.types}", f"algo={case.algo}", f"tile={case.tile}", f"relu={int(case.relu)}",
         f"bias={int(case.bias)}", f"sum={int(case.sum)}"]
    if case.types != "fp32":
        a += [f"iscale={case.iscale!r}", f"iz={case.iz!r}", f"oscale={case.oscale!r}", f"oz={case.oz!r}",
              f"sscale={case.sscale!r}", f"sz={case.sz!r}"]
        if case.tscale is not None:
            a += [f"tscale={case.tscale!r}", f"tz={case.tz!r}"]
    if case.g > 1:
        a += [f"wfmt={case.wfmt or 'goihw'}"]
    elif case.wfmt:
        a += [f"wfmt={case.wfmt}"]
    if case.ifmt:
        a += [f"ifmt={case.ifmt}"]
    if case.ofmt:
        a += [f"ofmt={case.ofmt}"]
    if knobs:
        for k, v in case.knobs.items():
            a.append(f"{k}={hex(v) if k == 'xopt' else v}")
    return a


DROPIN_DRIVER = ROOT / "tests" / "bin" / "euler_driver_b200"   # ref_driver.cpp linked against the product's libel.so


def run_reference(case: ConvCase, t: dict, iters: int = 0, warmup: int = 0, threads: int | None = None,
                  knobs: bool = True, want_output: bool = True, driver: Path | None = None):
    """Run the unmodified reference library on the tensors of ``t``.  Returns (output, info).
    ``driver`` selects another build of the same command-line driver (the drop-in test links it
    against this repository's C++ host library instead of the reference's)."""
    if driver is None:
        assert reference_available(), "oracle/_ref is not built or this CPU lacks AVX-512 VNNI"
    with tempfile.TemporaryDirectory(prefix="eulerref_") as td:
        td = Path(td)
        t["input"].tofile(td / "in.bin")
        t["weights"].tofile(td / "w.bin")
        t["bias"].tofile(td / "b.bin")
        args = reference_args(case, knobs) + [f"input_file={td/'in.bin'}", f"weights_file={td/'w.bin'}",
                                              f"bias_file={td/'b.bin'}", f"iters={iters}", f"warmup={warmup}"]
        if want_output:
            args.append(f"output_file={td/'out.bin'}")
        if case.sum:
            t["residual"].tofile(td / "res.bin")
            args.append(f"output_in_file={td/'res.bin'}")
        env = dict(os.environ)
        ncpu = threads or os.cpu_count() or 1
        env.update(OMP_NUM_THREADS=str(ncpu), KMP_AFFINITY="compact,granularity=fine", KMP_BLOCKTIME="infinite"
                   if iters else "0")
        r = subprocess.run([str(driver or REF_DIR / "ref_driver")] + args, capture_output=True, text=True, env=env)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if r.returncode != 0 or not line:
            raise RuntimeError(f"reference failed rc={r.returncode}\nstdout={r.stdout[-2000:]}\nstderr={r.stderr[-2000:]}")
        info = json.loads(line[-1])
        info["threads"] = ncpu
        out = None
        if want_output:
            out = np.fromfile(td / "out.bin", dtype=case.out_dtype).reshape(out_shape(case))
    return out, info


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))
