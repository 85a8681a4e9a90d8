"""The two-CTA (tcgen05 cta_group::2) variants of the tensor-core kernels are opt-in (they are not
faster on B200 today) but must stay correct: same parity bar as the default kernels."""
import os

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu


@pytest.fixture
def pairs_on():
    old = {k: os.environ.get(k) for k in ("ELB_I8_CTA2", "ELB_WINO_CTA2")}
    os.environ["ELB_I8_CTA2"] = "1"
    os.environ["ELB_WINO_CTA2"] = "1"
    yield
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v


@pytest.mark.parametrize("case", [
    R.ConvCase("p2_1x1", 4, 1024, 256, 14, 14, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True),
    R.ConvCase("p2_3x3_s2", 2, 128, 256, 56, 56, stride=2, types="u8f32u8f32", algo="direct", relu=True, bias=True),
    R.ConvCase("p2_3x3_odd_tiles", 3, 32, 48, 13, 19, types="u8f32s8f32", algo="direct", bias=True, oscale=8.0),
    R.ConvCase("p2_3x3_c3", 5, 3, 64, 40, 40, types="u8f32u8f32", algo="direct", relu=True, bias=True),
], ids=lambda c: c.name)
def test_int8_pairs_bit_exact(pkg, pairs_on, case):
    import gpuutil as G
    t = R.make_tensors(case)
    want, want_acc = R.oracle_int8_conv(case, t, want_acc=True)
    got, d, acc = G.run_gpu(case, t, want_acc=True)
    try:
        assert d.device_status() == 0
        assert np.array_equal(acc, want_acc)
        assert np.array_equal(got, want)
    finally:
        d.close()


@pytest.mark.parametrize("case", [
    R.ConvCase("p2_wino_f32", 4, 64, 64, 40, 40, types="fp32", algo="wino", tile=6, relu=True, bias=True),
    R.ConvCase("p2_wino_f32_odd", 3, 32, 96, 28, 28, types="fp32", algo="wino", tile=6, bias=True),    # 147 tiles... odd row blocks
    R.ConvCase("p2_wino_i8", 8, 64, 64, 28, 28, types="u8f32f32f32", algo="wino", tile=6),
], ids=lambda c: c.name)
def test_winograd_pairs(pkg, pairs_on, case):
    import gpuutil as G
    t = R.make_tensors(case)
    if case.types != "fp32":
        case = R.calibrate_tinput(case, t)
        want = R.oracle_int8_wino(case, t)
    else:
        want = R.oracle_wino_f32(case, t)
    got, d = G.run_gpu(case, t)
    try:
        assert d.device_status() == 0
        assert R.rel_l2(got, want) <= 1e-5
    finally:
        d.close()
