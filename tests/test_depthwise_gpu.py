"""GPU parity of the INT8 depthwise 3x3 kernel against the CPU restatement, through the C-ABI.

Bit-exact: u8 / s8 outputs and the raw int32 accumulators.  The cases cover both strides, pads 0
and 1, the reference's split of a u8 output row into floored 4-pixel groups and nearest-rounded
remainders (chunk length T = flatting.t), its wrap-around packing when a floored value leaves
[0, 255], a non-zero input zero point, ragged widths and channel counts beyond one block.
"""
import dataclasses

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu


def _dw(name, n, c, ih, iw, T, **kw):
    kw.setdefault("types", "u8f32u8f32")
    kw.setdefault("relu", True)
    kw.setdefault("bias", True)
    return R.ConvCase(name, n, c, c, ih, iw, g=c, algo="direct", knobs=dict(flt_t=T) if T else {}, **kw)


CASES = [
    _dw("dw_s1_t14", 2, 32, 28, 28, 14),
    _dw("dw_s1_t7_ragged", 2, 48, 23, 19, 7),
    _dw("dw_s1_t28_mobilenet_1", 2, 32, 112, 112, 28),
    _dw("dw_s2_t28_mobilenet_2", 2, 64, 112, 112, 28, stride=2, pad=0),
    _dw("dw_s2_t7", 2, 64, 28, 28, 7, stride=2),
    _dw("dw_s2_p1_odd", 1, 32, 15, 17, 5, stride=2),
    _dw("dw_s1_pad0", 1, 32, 14, 14, 6, pad=0),
    _dw("dw_s1_s8", 2, 32, 28, 28, 14, types="u8f32s8f32", relu=False),
    _dw("dw_s1_u8_norelu", 1, 32, 28, 28, 14, relu=False),
    _dw("dw_s1_overflow", 1, 32, 20, 12, 6, oscale=0.003),
    _dw("dw_s1_overflow_norelu", 1, 32, 20, 12, 6, oscale=0.003, relu=False),
    _dw("dw_s1_iz", 1, 32, 14, 14, 5, iz=3.0),
    _dw("dw_s1_t_default", 1, 32, 9, 9, 0),
    _dw("dw_s1_t3", 1, 32, 9, 10, 3),
    _dw("dw_s1_1024ch_7x7", 2, 1024, 7, 7, 7),
    _dw("dw_s1_tall_strip", 1, 16, 67, 8, 8),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_depthwise_bit_exact(pkg, case):
    import gpuutil as G
    t = R.make_tensors(case)
    want, want_acc = R.oracle_int8_depthwise(case, t, want_acc=True)
    got, d, acc = G.run_gpu(case, t, want_acc=True)
    try:
        assert d.kernel == "i8_depthwise"
        cb = case.oc // 16
        assert np.array_equal(acc[:, :cb], want_acc[:, :cb]), "int32 accumulators differ"
        bad = int((got[:, :cb] != want[:, :cb]).sum())
        assert bad == 0, f"{bad} of {want[:, :cb].size} output bytes differ"
    finally:
        d.close()


def test_depthwise_host_buffers_and_repeat(pkg):
    """The drop-in call with host memory, twice (weights are only read on the first call)."""
    import gpuutil as G
    case = _dw("dw_host", 2, 32, 28, 28, 14)
    t = R.make_tensors(case)
    want = R.oracle_int8_depthwise(case, t)
    got, d = G.run_gpu(case, t, host_buffers=True, repeat=2)
    try:
        assert np.array_equal(got, want)
    finally:
        d.close()


def test_depthwise_is_a_convolution(pkg):
    """Independent of the restatement: accumulators equal a plain integer depthwise convolution
    computed with numpy on the quantised weights the test data was built from."""
    import gpuutil as G
    case = _dw("dw_prop", 2, 32, 20, 20, 4, stride=2)
    t = R.make_tensors(case)
    _, d, acc = G.run_gpu(case, t, want_acc=True)
    d.close()
    x = R.from_nChw16c(t["input"], case.ic).astype(np.int64)
    q = t["q"].astype(np.int64)[:, 0]                       # [c][kh][kw]
    xp = np.pad(x, ((0, 0), (0, 0), (1, 1), (1, 1)))
    ref = np.zeros((case.n, case.oc, case.oh, case.ow), np.int64)
    for kh in range(3):
        for kw in range(3):
            ref += xp[:, :, kh:kh + 2 * case.oh:2, kw:kw + 2 * case.ow:2] * q[None, :, kh, kw, None, None]
    assert np.array_equal(R.from_nChw16c(acc, case.oc), ref)


@pytest.mark.parametrize("case", [
    _dw("dw_rej_s2_t1", 1, 32, 14, 14, 0, stride=2),          # T defaults to 1: reference double-counts
    _dw("dw_rej_s2_tr1", 1, 32, 14, 14, 6, stride=2),         # ow = 7, T = 6 -> remainder chunk of 1
], ids=lambda c: c.name)
def test_depthwise_rejects_undefined_chunkings(pkg, case):
    import gpuutil as G
    d = G.make_desc(case)
    assert d.setup() == pkg.ELD_UNIMPLEMENTED
    assert "one-pixel chunk" in pkg.last_error()
    d.close()
