"""The drop-in call with HOST tensors cuts the batch into chunks of whole images and overlaps their
copies and kernels; the result must not depend on the number of chunks.  Small problems use one
chunk by themselves, so the chunk count is forced here (ELB_HOST_CHUNKS is read per call)."""
import os

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu


@pytest.fixture
def chunks(request):
    old = os.environ.get("ELB_HOST_CHUNKS")
    os.environ["ELB_HOST_CHUNKS"] = str(request.param)
    yield request.param
    if old is None:
        os.environ.pop("ELB_HOST_CHUNKS", None)
    else:
        os.environ["ELB_HOST_CHUNKS"] = old


CASES = [
    R.ConvCase("hc_1x1", 5, 256, 96, 14, 14, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True),
    R.ConvCase("hc_1x1_sum", 4, 64, 64, 9, 9, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True,
               sum=True, sscale=0.5, oscale=0.5),
    R.ConvCase("hc_3x3_s2", 6, 32, 64, 20, 20, stride=2, types="u8f32u8f32", algo="direct", relu=True, bias=True),
    R.ConvCase("hc_wino_f32_sum", 5, 32, 48, 14, 14, types="fp32", algo="wino", tile=6, relu=True, bias=True, sum=True),
    R.ConvCase("hc_wino_i8", 4, 32, 32, 12, 12, types="u8f32f32f32", algo="wino", tile=6),
    R.ConvCase("hc_dw", 5, 32, 32, 16, 16, g=32, types="u8f32u8f32", algo="direct", relu=True, bias=True,
               knobs=dict(flt_t=8)),
]


@pytest.mark.parametrize("chunks", [1, 3, 64], indirect=True)
@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_host_call_is_independent_of_chunking(pkg, case, chunks):
    import gpuutil as G
    t = R.make_tensors(case)
    if case.algo == "wino" and case.types != "fp32":
        case = R.calibrate_tinput(case, t)
    if case.types == "fp32":
        want = R.oracle_wino_f32(case, t)
    elif case.algo == "wino":
        want = R.oracle_int8_wino(case, t)
    elif case.g > 1:
        want = R.oracle_int8_depthwise(case, t)
    else:
        want = R.oracle_int8_conv(case, t)
    got, d = G.run_gpu(case, t, host_buffers=True, repeat=2)
    try:
        assert d.device_status() == 0
        if want.dtype == np.float32:
            assert R.rel_l2(got, want) <= 1e-5
        else:
            assert np.array_equal(got, want)
    finally:
        d.close()
