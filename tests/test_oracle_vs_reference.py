"""Pin of the CPU restatement against the reference library itself (oracle/_ref), run where the
host has AVX-512 VNNI and the reference build exists; skipped elsewhere (tests/golden/ carries the
same pin as fixtures)."""
import dataclasses

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.skipif(not R.reference_available(), reason="reference build or AVX-512 VNNI missing")

BLK = lambda c: dict(blk_i=R.alignup(c.ic) // 16, blk_o=1, flt_o=1, flt_t=min(c.ow, 7))  # noqa: E731


def _with_knobs(c):
    return dataclasses.replace(c, knobs=BLK(c))


@pytest.mark.parametrize("case", [
    R.ConvCase("ovr_1x1", 2, 96, 48, 9, 9, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True),
    R.ConvCase("ovr_1x1_s8", 2, 64, 32, 8, 8, kh=1, kw=1, pad=0, types="u8f32s8f32", algo="1x1", bias=True, oscale=4.0),
    R.ConvCase("ovr_1x1_oz", 1, 64, 32, 8, 8, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", bias=True, oscale=4.0,
               oz=128.0),
    R.ConvCase("ovr_1x1_sum", 1, 64, 32, 8, 8, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True,
               sum=True, sscale=0.25, oscale=0.5),
    R.ConvCase("ovr_3x3", 2, 48, 32, 11, 11, types="u8f32u8f32", algo="direct", relu=True, bias=True),
    R.ConvCase("ovr_3x3_s2", 1, 32, 64, 14, 14, stride=2, types="u8f32u8f32", algo="direct", relu=True, bias=True),
    # non-zero input zero point with padding: the reference's per-position shift tables
    # (src/elx_int8_conv_direct.cpp:227-423) against the restatement's "sum of q over the taps inside the image"
    R.ConvCase("ovr_3x3_iz128", 1, 32, 32, 12, 12, types="u8f32u8f32", algo="direct", relu=True, bias=True, iz=128.0,
               oscale=0.3),
    R.ConvCase("ovr_3x3_s2_iz128", 1, 32, 32, 14, 14, stride=2, types="u8f32u8f32", algo="direct", relu=True, bias=True,
               iz=128.0, oscale=0.3),
    R.ConvCase("ovr_5x5_iz", 1, 32, 32, 14, 14, kh=5, kw=5, pad=2, types="u8f32u8f32", algo="direct", relu=True, bias=True,
               iz=3.0, oscale=0.5),
    R.ConvCase("ovr_7x7_s2_iz_s8", 1, 32, 32, 28, 28, kh=7, kw=7, pad=3, stride=2, types="u8f32s8f32", algo="direct",
               bias=True, iz=17.0, oscale=0.5),
], ids=lambda c: c.name)
def test_int8_direct_bit_exact(case):
    case = _with_knobs(case)
    t = R.make_tensors(case)
    ref, _ = R.run_reference(case, t)
    got = R.oracle_int8_conv(case, t)
    assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))


def test_reference_ignores_sum_on_kxk():
    """with_ip_sum has no effect on the reference's KxK int8 path (src/elx_int8_conv_direct.cpp:121)."""
    base = _with_knobs(R.ConvCase("ovr_sum_kxk", 1, 32, 32, 8, 8, types="u8f32u8f32", algo="direct", relu=True,
                                  bias=True))
    t = R.make_tensors(dataclasses.replace(base, sum=True))
    with_sum, _ = R.run_reference(dataclasses.replace(base, sum=True), t)
    without, _ = R.run_reference(base, t)
    assert np.array_equal(with_sum, without)


def test_epilogue_is_fused_multiply_add():
    """Large sample: the fused form must give zero mismatches against the reference build."""
    case = dataclasses.replace(R.baseline_case("c2", 8), oscale=4.0, relu=False, types="u8f32s8f32")
    t = R.make_tensors(case)
    ref, _ = R.run_reference(case, t)
    assert int((R.oracle_int8_conv(case, t, fused=True) != ref).sum()) == 0


@pytest.mark.parametrize("dims", [(2, 32, 32, 14, 14), (1, 16, 48, 13, 11)])
def test_fp32_winograd_close(dims):
    case = R.ConvCase("ovr_wino", *dims, types="fp32", algo="wino", tile=6, relu=True, bias=True)
    t = R.make_tensors(case)
    ref, _ = R.run_reference(case, t)
    assert R.rel_l2(R.oracle_wino_f32(case, t), ref) < 2e-6


def test_int8_winograd_close():
    case = R.ConvCase("ovr_i8wino", 2, 32, 32, 12, 12, types="u8f32f32f32", algo="wino", tile=6)
    t = R.make_tensors(case)
    case = R.calibrate_tinput(case, t)
    ref, _ = R.run_reference(case, t)
    assert R.rel_l2(R.oracle_int8_wino(case, t), ref) < 2e-6


@pytest.mark.parametrize("dims", [(2, 32, 32, 14, 14), (1, 16, 48, 13, 11), (1, 48, 16, 7, 9)])
def test_fp32_winograd_f2x2_close(dims):
    """tile_size 4 = F(2x2,3x3) (src/kernel/elk_conv_wino_2x2_3x3_*.hxx)."""
    case = R.ConvCase("ovr_wino4", *dims, types="fp32", algo="wino", tile=4, relu=True, bias=True)
    t = R.make_tensors(case)
    ref, _ = R.run_reference(case, t)
    assert R.rel_l2(R.oracle_wino_f32(case, t), ref) < 2e-6


@pytest.mark.parametrize("types,kw", [("u8f32f32f32", {}), ("u8f32u8f32", dict(relu=True, bias=True, oscale=0.05)),
                                      ("u8f32s8f32", dict(bias=True, oscale=0.1))])
def test_int8_winograd_f2x2(types, kw):
    """INT8 F(2x2,3x3); its u8 / s8 stores round toward minus infinity (elk_conv_wino_2x2_3x3_output.hxx:145-153)."""
    case = R.ConvCase("ovr_i8wino4", 2, 32, 32, 12, 12, types=types, algo="wino", tile=4, **kw)
    t = R.make_tensors(case)
    case = R.calibrate_tinput(case, t)
    ref, _ = R.run_reference(case, t)
    got = R.oracle_int8_wino(case, t)
    if types == "u8f32f32f32":
        assert R.rel_l2(got, ref) < 2e-6
    else:
        d = np.abs(got.astype(np.int32) - ref.astype(np.int32))
        assert d.max() == 0, (d.max(), (d != 0).mean())


@pytest.mark.parametrize("name,kw", [
    ("1x1", dict(kh=1, kw=1, pad=0, algo="1x1")), ("1x1_s2", dict(kh=1, kw=1, pad=0, stride=2, algo="1x1")),
    ("3x3", dict(algo="direct")), ("3x3_s2", dict(stride=2, algo="direct")), ("3x3_p0", dict(pad=0, algo="direct")),
    ("5x5", dict(kh=5, kw=5, pad=2, algo="direct")), ("7x7_s2", dict(kh=7, kw=7, pad=3, stride=2, algo="direct")),
    ("1x1_sum", dict(kh=1, kw=1, pad=0, algo="1x1", sum=True)), ("3x3_sum", dict(algo="direct", sum=True)),
    ("1x1_sum_plain", dict(kh=1, kw=1, pad=0, algo="1x1", sum=True, bias=False, relu=False)),
])
def test_fp32_direct_close(name, kw):
    """fp32 1x1 / KxK direct: result, bias, in-place sum (honoured here) and ReLU order."""
    kw = dict(kw)
    kw.setdefault("relu", True)
    kw.setdefault("bias", True)
    case = _with_knobs(R.ConvCase("ovr_f32_" + name, 2, 32, 32, 14, 14, types="fp32", **kw))
    t = R.make_tensors(case)
    ref, _ = R.run_reference(case, t)
    assert R.rel_l2(R.oracle_direct_f64(case, t), ref) < 2e-6


@pytest.mark.parametrize("case", [
    R.ConvCase("ovr_fmt_1x1_nhwc", 2, 64, 32, 8, 8, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True,
               ifmt="nhwc", ofmt="nhwc"),      # (the reference's int8 classes abort on hwio / oihw weights)
    R.ConvCase("ovr_fmt_3x3_nhwc", 1, 32, 32, 10, 10, types="u8f32u8f32", algo="direct", relu=True, bias=True,
               ifmt="nhwc", ofmt="nhwc"),
    R.ConvCase("ovr_fmt_wino_f32_nchw_in", 1, 32, 32, 12, 12, types="fp32", algo="wino", tile=6, relu=True, bias=True,
               ifmt="nchw", wfmt="oihw"),
], ids=lambda c: c.name)
def test_plain_formats_are_the_same_convolution(case):
    """The reference run on nhwc / nchw / hwio / oihw tensors gives the blocked result in another layout."""
    blocked = dataclasses.replace(case, ifmt="", ofmt="", wfmt="")
    t = R.make_tensors(blocked)
    if case.types != "fp32":
        case, blocked = _with_knobs(case), _with_knobs(blocked)
    ref, _ = R.run_reference(case, R.user_tensors(case, t))
    if case.types == "fp32":
        want = R.act_to_user(R.oracle_wino_f32(blocked, t), case.oc, case.ofmt)
        assert R.rel_l2(R.from_nChw16c(ref, case.oc), R.from_nChw16c(want, case.oc)) < 2e-6
    else:
        want = R.act_to_user(R.oracle_int8_conv(blocked, t), case.oc, case.ofmt)
        assert np.array_equal(ref, want)


DW = dict(algo="direct", bias=True)


@pytest.mark.parametrize("case", [
    R.ConvCase("ovr_dw_s1", 2, 32, 32, 16, 16, g=32, types="u8f32u8f32", relu=True, knobs=dict(flt_t=8), **DW),
    R.ConvCase("ovr_dw_s1_t7", 1, 32, 32, 24, 24, g=32, types="u8f32u8f32", relu=True, knobs=dict(flt_t=7), **DW),
    R.ConvCase("ovr_dw_s1_t28", 1, 32, 32, 28, 28, g=32, types="u8f32u8f32", relu=True, knobs=dict(flt_t=28), **DW),
    R.ConvCase("ovr_dw_s2", 2, 64, 64, 16, 16, g=64, stride=2, types="u8f32u8f32", relu=True, knobs=dict(flt_t=8), **DW),
    R.ConvCase("ovr_dw_s2_p0", 1, 48, 48, 15, 15, g=48, stride=2, pad=0, types="u8f32u8f32", relu=True, oscale=0.05,
               knobs=dict(flt_t=7), **DW),
    R.ConvCase("ovr_dw_s8", 1, 32, 32, 28, 28, g=32, types="u8f32s8f32", knobs=dict(flt_t=14), **DW),
    R.ConvCase("ovr_dw_norelu", 1, 32, 32, 28, 28, g=32, types="u8f32u8f32", knobs=dict(flt_t=14), **DW),
    R.ConvCase("ovr_dw_overflow", 1, 32, 32, 20, 12, g=32, types="u8f32u8f32", oscale=0.003, knobs=dict(flt_t=6), **DW),
    R.ConvCase("ovr_dw_iz", 1, 32, 32, 14, 14, g=32, types="u8f32u8f32", relu=True, iz=3.0, knobs=dict(flt_t=5), **DW),
    R.ConvCase("ovr_dw_t1", 1, 32, 32, 9, 9, g=32, types="u8f32u8f32", relu=True, **DW),
], ids=lambda c: c.name)
def test_int8_depthwise_bit_exact(case):
    """Includes the floor / nearest split by chunk position, the 64-bit packing adds (values outside
    [0,255] without ReLU or with a small output scale) and a non-zero input zero point."""
    t = R.make_tensors(case)
    ref, _ = R.run_reference(case, t)
    got = R.oracle_int8_depthwise(case, t)
    cb = case.oc // 16
    assert np.array_equal(got[:, :cb], ref[:, :cb])
