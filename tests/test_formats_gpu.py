"""Plain user formats (nchw / nhwc activations, oihw / hwio weights, the formats a caller outside the
reference's blocked world holds; its best INT8 ResNet configurations run nhwc) through the C-ABI:
the library converts on the device around the blocked kernels.  Results must equal the oracle's
(computed on the blocked tensors) on every real channel: bit for bit for integer outputs."""
import dataclasses

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu


def _i8(name, n, ic, oc, hw, **kw):
    kw.setdefault("types", "u8f32u8f32")
    kw.setdefault("relu", True)
    kw.setdefault("bias", True)
    return R.ConvCase(name, n, ic, oc, hw, hw, **kw)


CASES = [
    _i8("fmt_i8_1x1_nhwc", 2, 64, 32, 14, kh=1, kw=1, pad=0, algo="1x1", ifmt="nhwc", ofmt="nhwc", wfmt="hwio"),
    _i8("fmt_i8_1x1_nhwc_sum_ragged", 3, 40, 24, 7, kh=1, kw=1, pad=0, algo="1x1", ifmt="nhwc", ofmt="nhwc", wfmt="hwio",
        sum=True, sscale=0.5, oscale=0.5),
    _i8("fmt_i8_3x3_nhwc_in_blocked_out", 2, 32, 64, 12, algo="direct", ifmt="nhwc", wfmt="oihw"),
    _i8("fmt_i8_3x3s2_nchw_s8", 1, 48, 32, 15, stride=2, algo="direct", types="u8f32s8f32", relu=False, oscale=8.0,
        ifmt="nchw", ofmt="nchw", wfmt="oihw"),
    # u8 planes whose size is a multiple of four pixels: the word-wise nchw -> nChw16c converter
    _i8("fmt_i8_3x3_rgb_nchw", 2, 3, 32, 16, algo="direct", ifmt="nchw"),
    _i8("fmt_i8_3x3_40ch_nchw", 1, 40, 24, 12, algo="direct", ifmt="nchw", wfmt="oihw"),
    _i8("fmt_i8_wino_nhwc_f32", 2, 32, 32, 12, algo="wino", tile=6, types="u8f32f32f32", relu=False, bias=False,
        ifmt="nhwc", ofmt="nhwc", wfmt="hwio"),
    R.ConvCase("fmt_f32_wino_rgb_nchw", 2, 3, 64, 16, 16, types="fp32", algo="wino", tile=6, relu=True, bias=True,
               ifmt="nchw", wfmt="oihw"),
    # the direct kernel for at most four input channels reads an nchw image itself (no conversion)
    R.ConvCase("fmt_f32_wino_rgb_nchw_ragged", 2, 3, 32, 21, 30, types="fp32", algo="wino", tile=6, relu=True, bias=True,
               ifmt="nchw"),
    R.ConvCase("fmt_f32_wino_gray_nchw_both", 1, 1, 16, 9, 13, types="fp32", algo="wino", tile=6, relu=False, bias=True,
               ifmt="nchw", ofmt="nchw", wfmt="oihw"),
    R.ConvCase("fmt_f32_wino_4ch_nchw_sum", 1, 4, 40, 12, 12, types="fp32", algo="wino", tile=6, relu=True, bias=True,
               sum=True, ifmt="nchw"),
    # ... and with exactly 64 output channels the tensor-core first-layer kernel takes it
    R.ConvCase("fmt_f32_rgb64_nchw_ragged", 2, 3, 64, 21, 30, types="fp32", algo="wino", tile=6, relu=True, bias=True,
               ifmt="nchw"),
    R.ConvCase("fmt_f32_gray64_nchw_plain", 1, 1, 64, 9, 13, types="fp32", algo="wino", tile=6, relu=False, bias=True,
               ifmt="nchw", ofmt="nchw", wfmt="oihw"),
    R.ConvCase("fmt_f32_2ch64_nchw", 3, 2, 64, 40, 36, types="fp32", algo="wino", tile=6, relu=True, bias=False,
               ifmt="nchw"),
    R.ConvCase("fmt_f32_4ch64_nchw", 1, 4, 56, 12, 12, types="fp32", algo="wino", tile=6, relu=True, bias=True,
               ifmt="nchw"),
    R.ConvCase("fmt_f32_wino_nhwc", 1, 32, 48, 9, 11, types="fp32", algo="wino", tile=4, relu=True, bias=True,
               ifmt="nhwc", ofmt="nhwc", wfmt="hwio"),
    R.ConvCase("fmt_f32_1x1_nhwc_sum", 2, 64, 40, 8, 8, kh=1, kw=1, pad=0, types="fp32", algo="1x1", relu=True, bias=True,
               sum=True, ifmt="nhwc", ofmt="nhwc", wfmt="hwio"),
    R.ConvCase("fmt_f32_7x7s2_rgb_nchw", 1, 3, 32, 32, 32, kh=7, kw=7, pad=3, stride=2, types="fp32", algo="direct",
               relu=True, bias=True, ifmt="nchw", ofmt="nchw", wfmt="oihw"),
    _i8("fmt_dw_ghwio", 1, 32, 32, 14, g=32, algo="direct", wfmt="ghwio", knobs=dict(flt_t=7)),
]


def oracle(case, t):
    if case.g > 1:
        return R.oracle_int8_depthwise(case, t)
    if case.types == "fp32":
        return R.oracle_wino_f32(case, t) if case.algo == "wino" else R.oracle_direct_f64(case, t)
    return R.oracle_int8_wino(case, t) if case.algo == "wino" else R.oracle_int8_conv(case, t)


@pytest.mark.parametrize("host", [False, True], ids=["device", "host"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_plain_formats_match_oracle(pkg, case, host):
    import gpuutil as G
    blocked = dataclasses.replace(case, ifmt="", ofmt="", wfmt="")
    t = R.make_tensors(blocked)
    if case.algo == "wino" and case.types != "fp32":
        cal = R.calibrate_tinput(blocked, t)
        blocked = cal
        case = dataclasses.replace(case, tscale=cal.tscale, tz=cal.tz)
    want = R.act_to_user(oracle(blocked, t), case.oc, case.ofmt)
    got, d = G.run_gpu(case, R.user_tensors(case, t), host_buffers=host)
    try:
        assert d.device_status() == 0
        assert got.shape == want.shape
        if case.ofmt == "":                      # blocked output: compare the real channel blocks
            got, want = R.from_nChw16c(got, case.oc), R.from_nChw16c(want, case.oc)
        if case.out_dtype != np.float32 and not (case.algo == "wino" and case.tile != 4):
            assert np.array_equal(got, want), f"{int((got != want).sum())} of {got.size} outputs differ"
        elif case.out_dtype != np.float32:
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
        else:
            assert R.rel_l2(got, want) <= 1e-5
    finally:
        d.close()


def test_sizes_follow_the_formats(pkg):
    """sizes / byte_sizes of plain formats count the real channels (src/eld_conv.cpp:99-114)."""
    import gpuutil as G
    case = CASES[1]
    d = G.make_desc(case)
    assert d.setup() == 0
    assert d.sizes.input == case.n * case.ih * case.iw * case.ic
    assert d.sizes.output == case.n * case.oh * case.ow * case.oc
    assert d.sizes.bias == case.oc
    assert d.sizes.weights == case.oc * case.ic + 64
    d.close()
