"""GPU parity of the fp32 direct convolutions (1x1 and KxK, any stride / padding) against the CPU
restatement (an fp64 direct convolution with the reference's epilogue order), through the C-ABI.
Tolerance: relative L2 error <= 1e-5 (three tf32 products per fp32 product, fp32 accumulation)."""
import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5


def _c(name, n, ic, oc, ih, iw, **kw):
    kw.setdefault("relu", True)
    kw.setdefault("bias", True)
    kw.setdefault("algo", "1x1" if kw.get("kh", 3) == 1 else "direct")
    return R.ConvCase(name, n, ic, oc, ih, iw, types="fp32", **kw)


CASES = [
    _c("f32_1x1", 2, 64, 32, 14, 14, kh=1, kw=1, pad=0),
    _c("f32_1x1_resnet_res4_reduce", 4, 1024, 256, 14, 14, kh=1, kw=1, pad=0),
    _c("f32_1x1_resnet_res2_expand_sum", 2, 64, 256, 56, 56, kh=1, kw=1, pad=0, sum=True),
    _c("f32_1x1_s2", 2, 256, 512, 28, 28, kh=1, kw=1, pad=0, stride=2),
    _c("f32_1x1_plain_pad_lanes", 3, 24, 40, 9, 7, kh=1, kw=1, pad=0, relu=False, bias=False),
    _c("f32_1x1_auto", 1, 32, 32, 8, 8, kh=1, kw=1, pad=0, algo="auto"),
    _c("f32_3x3", 2, 32, 32, 12, 12),
    _c("f32_3x3_s2", 2, 128, 256, 28, 28, stride=2),
    _c("f32_3x3_p0_sum", 1, 48, 16, 9, 11, pad=0, sum=True),
    _c("f32_5x5", 1, 16, 32, 10, 10, kh=5, kw=5, pad=2),
    _c("f32_7x7_s2_rgb", 2, 3, 64, 32, 32, kh=7, kw=7, pad=3, stride=2),      # ResNet conv1 shape family
    _c("f32_oc320", 1, 32, 320, 8, 8, kh=1, kw=1, pad=0),                     # two N tiles of 160
    _c("f32_tiny", 1, 16, 16, 1, 1, kh=1, kw=1, pad=0),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_fp32_direct_matches_oracle(pkg, case):
    import gpuutil as G
    t = R.make_tensors(case)
    want = R.oracle_direct_f64(case, t)
    got, d = G.run_gpu(case, t)
    try:
        assert d.kernel == "f32_direct_umma"
        assert d.device_status() == 0
        err = R.rel_l2(got, want)
        assert err <= F32_TOL, f"rel-L2 {err:.3e}"
        if case.oc % 16 and not case.sum:
            assert np.all(R.from_nChw16c(got, R.alignup(case.oc))[:, case.oc:] == 0)
    finally:
        d.close()


def test_fp32_direct_host_buffers_and_repeat(pkg):
    import gpuutil as G
    case = CASES[7]
    t = R.make_tensors(case)
    want = R.oracle_direct_f64(case, t)
    got, d = G.run_gpu(case, t, host_buffers=True, repeat=2)
    assert R.rel_l2(got, want) <= F32_TOL
    d.close()


def test_relu_bound_is_honoured(pkg):
    """relu_bound clamps on this path (src/kernel/elk_gemm.hxx:230-235), unlike the Winograd output transform."""
    import torch
    import gpuutil as G
    E = G.package()
    case = _c("f32_1x1_relu6", 1, 32, 32, 8, 8, kh=1, kw=1, pad=0)
    t = R.make_tensors(case)
    t["weights"] = t["weights"] * 40.0
    d = G.make_desc(case)
    d.relu_bound.lower, d.relu_bound.upper = 0.0, 6.0
    assert d.setup() == E.ELD_OK, E.last_error()
    out = np.zeros(R.out_shape(case), np.float32)
    assert E.elx_conv(d, out, t["input"], t["weights"], t["bias"]) == E.ELX_OK
    want = np.clip(R.oracle_direct_f64(R.dataclasses.replace(case, relu=False), t), 0.0, 6.0)
    assert out.max() == 6.0 and out.min() == 0.0
    assert R.rel_l2(out, want) <= F32_TOL
    d.close()


def test_1x1_through_the_gather_path(pkg, monkeypatch):
    """The general three-kernel path on a shape the single-kernel 1x1 path would take."""
    import gpuutil as G
    monkeypatch.setenv("ELB_F32_NO_FLAT", "1")
    case = _c("f32_1x1_gathered", 2, 96, 48, 10, 13, kh=1, kw=1, pad=0, sum=True)
    t = R.make_tensors(case)
    want = R.oracle_direct_f64(case, t)
    got, d = G.run_gpu(case, t)
    try:
        assert d.launch_count() == 3
        assert R.rel_l2(got, want) <= F32_TOL
    finally:
        d.close()


def test_1x1_single_kernel_launch_count(pkg):
    import gpuutil as G
    case = CASES[0]
    t = R.make_tensors(case)
    got, d = G.run_gpu(case, t)
    try:
        assert d.launch_count() == 1
        assert R.rel_l2(got, R.oracle_direct_f64(case, t)) <= F32_TOL
    finally:
        d.close()
