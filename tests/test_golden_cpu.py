"""The CPU restatement against the golden fixtures (outputs of the unmodified reference library
on small seeded problems).  This is the pin that holds on machines where the reference cannot run."""
import numpy as np
import pytest

import goldenutil as GU
import refutil as R


@pytest.mark.parametrize("name", GU.golden_names())
def test_oracle_matches_reference_fixture(name):
    case, t, want = GU.load_golden(name)
    if case.types == "fp32" and case.algo != "wino":
        got = R.oracle_direct_f64(case, t)
    elif case.types == "fp32":
        got = R.oracle_wino_f32(case, t)
    elif case.algo == "wino":
        got = R.oracle_int8_wino(case, t)
    elif case.g > 1:
        got = R.oracle_int8_depthwise(case, t)
    else:
        got = R.oracle_int8_conv(case, t)
    GU.check_against_golden(case, got, want)


def test_fixture_set_covers_every_path():
    names = GU.golden_names()
    assert len(names) >= 12
    for key in ("i8_1x1", "i8_3x3_s1", "i8_3x3_s2", "wino_f32", "wino_i8", "wino4_f32", "wino4_i8", "f32_1x1", "f32_3x3", "c2_shape", "c3_shape", "sum", "dw_s1",
                "dw_s2"):
        assert any(key in n for n in names), key


def test_winograd_restatement_is_a_convolution():
    """Independent of the reference: the restated F(4x4,3x3) pipeline equals an fp64 direct
    convolution to fp32 rounding, including partial border tiles."""
    for dims in ((1, 16, 16, 10, 7), (2, 32, 16, 13, 13), (1, 16, 32, 4, 4)):
        case = R.ConvCase("prop_wino", *dims, types="fp32", algo="wino", tile=6, bias=True, relu=True)
        t = R.make_tensors(case)
        a = R.oracle_wino_f32(case, t)
        b = R.oracle_direct_f64(case, t)
        assert R.rel_l2(a, b) < 2e-6


def test_int8_restatement_linearity():
    """Size-independent property: with unit scales and no bias/ReLU the f32-output int8 convolution
    is the exact integer convolution, hence additive in the weights' integer codes."""
    case = R.ConvCase("prop_lin", 1, 32, 16, 6, 6, types="u8f32f32f32", algo="direct", iscale=1.0, oscale=1.0)
    t = R.make_tensors(case)
    out, acc = R.oracle_int8_conv(case, t, want_acc=True)
    x = R.from_nChw16c(t["input"], case.ic).astype(np.int64)
    q = t["q"].astype(np.int64)
    xp = np.pad(x, ((0, 0), (0, 0), (1, 1), (1, 1)))
    ref = np.zeros((1, case.oc, 6, 6), np.int64)
    for kh in range(3):
        for kw in range(3):
            ref += np.einsum("nchw,oc->nohw", xp[:, :, kh:kh + 6, kw:kw + 6], q[:, :, kh, kw])
    assert np.array_equal(R.from_nChw16c(acc, case.oc), ref)
