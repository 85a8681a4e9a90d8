"""CPU-side checks of the C-ABI boundary: the shared library loads without a GPU, exports every
entry point include/euler_b200.h declares, computes sizes / algorithm choice like the reference's
setup(), and refuses to compute without a device (there is no CPU fallback)."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import refutil as R

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "euler_b200.h").read_text()
    return sorted(set(re.findall(r"ELB_API\s+[\w\s\*]+?\b(elb_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for s in ("elb_conv_sizes", "elb_conv_create", "elb_conv_execute", "elb_conv_enqueue", "elb_conv_prepare",
              "elb_conv_destroy", "elb_last_error", "elb_device_supported", "elb_wino_f32_conv_noalloc"):
        assert s in syms


def test_library_exports_every_declared_symbol(pkg):
    lib = C.CDLL(str(pkg.LIB_PATH))
    for s in declared_symbols():
        assert hasattr(lib, s), f"{s} is declared in include/euler_b200.h but not exported"


def test_struct_layout_matches_header(pkg):
    # 35 int32 + 2 float + 1 int32 + 8 float + 3 int32 = 49 four-byte fields
    assert C.sizeof(pkg.ElbConvDesc) == 49 * 4
    assert C.sizeof(pkg.ElbConvInfo) == 4 * 4 + 9 * 8 + 2 * 4


@pytest.mark.parametrize("cid", ["c1", "c2", "c3", "c4"])
def test_sizes_and_algorithm_like_reference_setup(pkg, cid):
    """byte_sizes follow src/eld_conv.cpp:99-126 (weights carry 4*16 elements of slack)."""
    import gpuutil as G
    case = R.baseline_case(cid)
    d = G.make_desc(case)
    assert d.setup(False) == pkg.ELD_OK
    icp, ocp = R.alignup(case.ic), R.alignup(case.oc)
    in_b = 4 if case.types == "fp32" else 1
    out_b = np.dtype(case.out_dtype).itemsize
    assert d.byte_sizes.input == case.n * icp * case.ih * case.iw * in_b
    assert d.byte_sizes.weights == (case.kh * case.kw * icp * ocp + 64) * 4
    assert d.byte_sizes.output == case.n * ocp * case.oh * case.ow * out_b
    assert d.byte_sizes.bias == ocp * 4
    expect = {"c1": pkg.CONV_WINOGRAD, "c2": pkg.CONV_DIRECT_1X1, "c3": pkg.CONV_DIRECT, "c4": pkg.CONV_WINOGRAD}[cid]
    assert d.algorithm == expect


def test_conv_auto_resolution(pkg):
    """CONV_AUTO: 1x1 -> DIRECT_1X1; 3x3 s1 p1 with ic >= 16 -> WINOGRAD; else DIRECT
    (src/eld_conv.cpp:148-159); tile 0 -> 6 when mac_per_read > 25 else 4 (:231-236)."""
    import gpuutil as G
    d = G.make_desc(R.ConvCase("auto1", 1, 64, 64, 8, 8, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="auto"))
    assert d.setup(False) == 0 and d.algorithm == pkg.CONV_DIRECT_1X1
    d = G.make_desc(R.ConvCase("auto2", 64, 256, 256, 56, 56, types="fp32", algo="auto"))
    assert d.setup(False) == 0 and d.algorithm == pkg.CONV_WINOGRAD and d.tile_size == 6
    d = G.make_desc(R.ConvCase("auto3", 1, 16, 16, 4, 4, types="fp32", algo="auto"))
    assert d.setup(False) == 0 and d.algorithm == pkg.CONV_WINOGRAD and d.tile_size == 4
    d = G.make_desc(R.ConvCase("auto4", 1, 64, 64, 8, 8, stride=2, types="u8f32u8f32", algo="auto"))
    assert d.setup(False) == 0 and d.algorithm == pkg.CONV_DIRECT
    d = G.make_desc(R.ConvCase("auto5", 1, 3, 64, 8, 8, types="fp32", algo="auto"))
    assert d.setup(False) == 0 and d.algorithm == pkg.CONV_DIRECT      # ic < 16


def test_invalid_descriptors(pkg):
    import gpuutil as G
    d = G.make_desc(R.ConvCase("bad", 0, 16, 16, 4, 4, types="fp32", algo="wino", tile=6))
    assert d.setup(False) == pkg.ELD_GENERAL_ERROR
    d = G.make_desc(R.ConvCase("bad2", 1, 16, 16, 4, 4, types="fp32", algo="wino", tile=6))
    d.prop_kind = pkg.backward_data
    assert d.setup(False) == pkg.ELD_GENERAL_ERROR and "Propagation" in pkg.last_error()


def test_no_cpu_fallback(pkg):
    """Without a usable sm_100 device plan creation fails loudly; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import gpuutil as G
    d = G.make_desc(R.baseline_case("c2", 1))
    rc = d.setup()
    assert rc != pkg.ELD_OK and d.xc is None
    assert "CUDA" in pkg.last_error() or "device" in pkg.last_error()
    with pytest.raises(RuntimeError):
        pkg.elx_conv(d, None, None, None, None)


def test_cal_ops_matches_reference_formula():
    """Op counts used by the bench: 2*N*IC*OC*valid taps (tests/elt_conv_utils.cpp:638-659)."""
    assert R.baseline_case("c2").cal_ops() == 2 * 64 * 1024 * 256 * 14 * 14
    assert R.baseline_case("c1").cal_ops() == 231_156_482_048 or abs(R.baseline_case("c1").cal_ops() / 231.156e9 - 1) < 1e-3
    assert abs(R.baseline_case("c3").cal_ops() / 28.895e9 - 1) < 1e-3
    assert abs(R.baseline_case("c4").cal_ops() / 451.240e9 - 1) < 1e-3


def test_host_library_exports_the_reference_symbols(pkg):
    """lib/libel.so must define the mangled C++ symbols a program compiled against the reference's
    euler.hpp / euler_reorder.hpp binds (include/euler.hpp:110-190, src/elx_reorder.cpp:209-232)."""
    import subprocess
    lib = pkg.HOST_LIB_PATH
    if not lib.exists():
        pytest.skip("libel.so not built (reference headers missing at build time)")
    out = subprocess.run(["nm", "-D", "--defined-only", str(lib)], capture_output=True, text=True, check=True).stdout
    syms = {ln.split()[-1] for ln in out.splitlines() if ln.strip()}
    need = ["_ZN5euler10eld_conv_tC1Ev", "_ZN5euler10eld_conv_tD1Ev", "_ZN5euler10eld_conv_t5setupEb",
            "_ZN5euler8elx_convERNS_10eld_conv_tEPvS2_S2_S2_"]
    # reorder<T, dst, src>::reorder(T*, T*, int x4|x5): formats are the enum values of euler.hpp
    pairs4 = [(1, 2), (2, 1), (1, 3), (3, 1), (5, 7), (7, 5), (5, 6), (6, 5)]
    pairs5 = [(9, 11), (11, 9), (9, 10), (10, 9)]
    for t in ("f", "h"):
        need += [f"_ZN5euler7reorderI{t}Li{d}ELi{s}EJEEC1EP{t}S2_iiii" for d, s in pairs4]
        need += [f"_ZN5euler7reorderI{t}Li{d}ELi{s}EJEEC1EP{t}S2_iiiii" for d, s in pairs5]
    missing = [n for n in need if n not in syms]
    assert not missing, missing
