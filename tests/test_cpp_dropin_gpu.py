"""Drop-in test of the C++ surface: a program written against the reference's own euler.hpp
(oracle/ref_driver.cpp, the very driver that runs the reference library) is linked against this
repository's libel.so instead and must produce the reference's results on the GPU.

The binary tests/bin/euler_driver_b200 is produced by build() where the reference headers exist; it
fills an euler::eld_conv_t, calls setup() and elx_conv() with HOST tensors read from files."""
import dataclasses

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu


def _run(case, t):
    if not R.DROPIN_DRIVER.exists():
        pytest.skip("tests/bin/euler_driver_b200 was not built (reference headers missing at build time)")
    return R.run_reference(case, t, driver=R.DROPIN_DRIVER, iters=2, warmup=0)


def test_int8_1x1_through_euler_hpp(pkg):
    case = R.baseline_case("c2", 4)
    t = R.make_tensors(case)
    out, info = _run(case, t)
    assert info["rc_setup"] == 0 and info["rc"] == 0 and info["algorithm"] == pkg.CONV_DIRECT_1X1
    assert info["bytes"]["weights"] == (1024 * 256 + 64) * 4
    assert np.array_equal(out, R.oracle_int8_conv(case, t))


def test_int8_3x3_stride2_through_euler_hpp(pkg):
    case = R.baseline_case("c3", 2)
    t = R.make_tensors(case)
    out, info = _run(case, t)
    assert info["rc"] == 0
    assert np.array_equal(out, R.oracle_int8_conv(case, t))


def test_fp32_winograd_sum_through_euler_hpp(pkg):
    """with_ip_sum: the output buffer is read as well as written, also for host tensors."""
    case = R.ConvCase("dropin_wino", 2, 64, 48, 20, 20, types="fp32", algo="wino", tile=6, relu=True, bias=True,
                      sum=True)
    t = R.make_tensors(case)
    out, info = _run(case, t)
    assert info["rc"] == 0 and info["tile_size"] == 6
    assert R.rel_l2(out, R.oracle_wino_f32(case, t)) <= 1e-5      # the tolerance the fp32 path is held to


def test_int8_depthwise_through_euler_hpp(pkg):
    case = R.ConvCase("dropin_dw", 2, 64, 64, 28, 28, g=64, types="u8f32u8f32", algo="direct", relu=True, bias=True,
                      knobs=dict(flt_t=14))
    t = R.make_tensors(case)
    out, info = _run(case, t)
    assert info["rc"] == 0
    assert np.array_equal(out, R.oracle_int8_depthwise(case, t))


def test_fp32_direct_through_euler_hpp(pkg):
    case = R.ConvCase("dropin_f32_3x3s2", 2, 64, 32, 14, 14, stride=2, types="fp32", algo="direct", relu=True, bias=True)
    t = R.make_tensors(case)
    out, info = _run(case, t)
    assert info["rc"] == 0
    assert R.rel_l2(out, R.oracle_direct_f64(case, t)) <= 1e-5


def test_nhwc_tensors_through_euler_hpp(pkg):
    """nhwc activations and hwio weights, the layout the reference's tuned INT8 ResNet scripts run."""
    case = R.ConvCase("dropin_nhwc", 2, 64, 48, 14, 14, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True,
                      bias=True, ifmt="nhwc", ofmt="nhwc", wfmt="hwio")
    blocked = dataclasses.replace(case, ifmt="", ofmt="", wfmt="")
    t = R.make_tensors(blocked)
    out, info = _run(case, R.user_tensors(case, t))
    assert info["rc"] == 0
    assert info["bytes"]["input"] == 2 * 14 * 14 * 64 and info["bytes"]["bias"] == 48 * 4
    assert np.array_equal(out, R.act_to_user(R.oracle_int8_conv(blocked, t), case.oc, "nhwc"))


def test_unsupported_descriptor_returns_code_instead_of_aborting(pkg):
    case = R.ConvCase("dropin_rej", 1, 32, 32, 8, 8, types="fp32", algo="wino", tile=7)    # F(5x5,3x3): not built
    t = R.make_tensors(case)
    if not R.DROPIN_DRIVER.exists():
        pytest.skip("driver not built")
    with pytest.raises(RuntimeError) as e:
        R.run_reference(case, t, driver=R.DROPIN_DRIVER)
    assert '"rc_setup": 1' in str(e.value)
