"""The CUDA kernels against the golden fixtures (outputs of the unmodified reference library),
through the C-ABI.  Integer outputs must be identical byte for byte."""
import pytest

import goldenutil as GU

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", GU.golden_names())
def test_gpu_matches_reference_fixture(pkg, name):
    import gpuutil as G
    case, t, want = GU.load_golden(name)
    if case.sum and case.algo == "direct" and case.kh > 1 and case.types != "fp32":
        pytest.skip("reference ignores with_ip_sum on this path")
    got, d = G.run_gpu(case, t)
    try:
        assert d.device_status() == 0
        GU.check_against_golden(case, got, want)
    finally:
        d.close()
