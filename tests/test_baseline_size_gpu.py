"""Parity at the benchmark configurations' FULL size, against the reference library itself.

The small-shape tests cannot reach what the full batches exercise: three and more tiles per
persistent CTA (accumulator double-buffer phase flips), the chunking of the Winograd workspace, the
per-layer choice of A-operand placement, four-producer mode.  Each configuration runs once through
elx_conv on device tensors and is compared with oracle/_ref on the same seeded tensors: INT8
direct / 1x1 / depthwise bit-exact, Winograd rel-L2 <= 1e-5 (the tolerance the benchmark names).
Hosts without AVX-512 VNNI cannot run the reference build; the C restatement then stands in for
the INT8 direct paths (seconds at these sizes) and the Winograd cases are skipped there.
"""
import numpy as np
import pytest

import gpuutil as G
import refutil as R

pytestmark = pytest.mark.gpu


def _reference(case, t, allow_port):
    if R.reference_available():
        out, _ = R.run_reference(case, t)
        return out
    if not allow_port:
        pytest.skip("the reference build needs AVX-512 VNNI on this host")
    fn = R.oracle_int8_depthwise if case.g > 1 else R.oracle_int8_conv
    return fn(case, t)


@pytest.mark.parametrize("cid", ["c2", "c3", "dw"])
def test_int8_full_size_bit_exact(pkg, cid):
    case = R.baseline_case(cid)
    t = R.make_tensors(case)
    want = _reference(case, t, allow_port=True)
    got, d = G.run_gpu(case, t)
    d.close()
    bad = int((got != want).sum())
    assert bad == 0, f"{case.name}: {bad} of {got.size} output bytes differ from the reference"


def test_fp32_winograd_c1_full_size(pkg):
    case = R.baseline_case("c1")
    t = R.make_tensors(case)
    want = _reference(case, t, allow_port=False)
    got, d = G.run_gpu(case, t)
    d.close()
    err = R.rel_l2(got, want)
    assert err <= 1e-5, f"{case.name}: rel-L2 {err:.3e} against the reference's fp32 Winograd output"


def test_int8_winograd_c4_full_size(pkg):
    case = R.baseline_case("c4")
    t = R.make_tensors(case)
    case = R.calibrate_tinput(case, t)
    want = _reference(case, t, allow_port=False)
    got, d = G.run_gpu(case, t)
    d.close()
    err = R.rel_l2(got, want)
    assert err <= 1e-5, f"{case.name}: rel-L2 {err:.3e} against the reference's int8 Winograd output"
