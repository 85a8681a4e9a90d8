"""GPU parity of the Winograd paths -- F(4x4,3x3) (tile_size 6) and F(2x2,3x3) (tile_size 4), fp32
with the 3xTF32 tensor-core GEMM and int8 -- against the CPU restatement, through the C-ABI.

fp32 tolerance: relative L2 error <= 1e-5 against the restated fp32 Winograd result (the bar the
benchmark definition sets), and additionally against an fp64 direct convolution.
int8: the raw int32 accumulators of the 36 transform-domain GEMMs are compared bit for bit, the
final fp32 output by relative L2 (only the fp32 output transform's summation order differs).
"""
import dataclasses

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5


def _f32(name, n, ic, oc, ih, iw, **kw):
    kw.setdefault("relu", True)
    kw.setdefault("bias", True)
    kw.setdefault("tile", 6)
    return R.ConvCase(name, n, ic, oc, ih, iw, types="fp32", algo="wino", **kw)


F32_CASES = [
    _f32("wino_small", 2, 32, 32, 14, 14),
    _f32("wino_partial_tiles", 1, 16, 48, 13, 11),              # oh, ow not multiples of 4
    _f32("wino_c1_small", 2, 256, 256, 56, 56),                 # the benchmark layer at n=2
    _f32("wino_plain", 3, 64, 32, 8, 8, relu=False, bias=False),
    _f32("wino_sum", 2, 32, 64, 12, 12, sum=True),
    _f32("wino_pad_lanes", 1, 24, 40, 9, 9),                    # channels not multiples of 16
    _f32("wino_oc512", 1, 64, 512, 8, 8),                       # two N tiles of 256
    _f32("wino_oc320", 1, 32, 320, 8, 8),                       # N tiles of 160
    _f32("wino_tiny", 1, 16, 16, 4, 4),
    # at most four input channels: served by the CUDA-core direct kernel (f32_small_ic)
    _f32("small_ic_3", 2, 3, 64, 30, 21),
    _f32("small_ic_4_sum", 1, 4, 40, 9, 10, sum=True),
    _f32("small_ic_1_plain", 2, 1, 16, 5, 3, relu=False, bias=False),
    _f32("small_ic_3_f2x2", 1, 3, 32, 8, 8, tile=4),
    # F(2x2,3x3)
    _f32("wino4_small", 2, 32, 32, 14, 14, tile=4),
    _f32("wino4_partial_tiles", 1, 16, 48, 13, 11, tile=4),     # odd oh, ow: clipped 2x2 tiles
    _f32("wino4_vgg_conv5", 2, 512, 512, 14, 14, tile=4),
    _f32("wino4_sum_pad_lanes", 2, 24, 40, 9, 9, tile=4, sum=True),
    _f32("wino4_plain_oc320", 1, 32, 320, 8, 8, tile=4, relu=False, bias=False),
    _f32("wino4_tiny", 1, 16, 16, 2, 2, tile=4),
]


@pytest.mark.parametrize("case", F32_CASES, ids=lambda c: c.name)
def test_fp32_winograd_matches_oracle(pkg, case):
    import gpuutil as G
    t = R.make_tensors(case)
    want = R.oracle_wino_f32(case, t)
    got, d = G.run_gpu(case, t)
    try:
        assert d.kernel == ("f32_small_ic" if case.ic <= 4 else "wino_f32_umma")
        assert d.device_status() == 0
        err = R.rel_l2(got, want)
        assert err <= F32_TOL, f"rel-L2 vs restated Winograd {err:.3e}"
        if not case.sum:
            exact = R.oracle_direct_f64(case, t)
            oc = case.oc
            g2 = R.from_nChw16c(got, oc)
            e2 = R.from_nChw16c(exact, oc)
            assert R.rel_l2(g2, e2) <= 2e-5
        # padded output channels carry bias-free zeros (relu(0 + 0))
        if case.oc % 16 and not case.sum:
            assert np.all(R.from_nChw16c(got, R.alignup(case.oc))[:, case.oc:] == 0)
    finally:
        d.close()


def test_fp32_winograd_host_buffers_and_repeat(pkg):
    import gpuutil as G
    case = F32_CASES[0]
    t = R.make_tensors(case)
    want = R.oracle_wino_f32(case, t)
    got, d = G.run_gpu(case, t, host_buffers=True, repeat=2)
    assert R.rel_l2(got, want) <= F32_TOL
    d.close()


def _i8(name, n, ic, oc, ih, iw, **kw):
    kw.setdefault("types", "u8f32f32f32")
    kw.setdefault("tile", 6)
    return R.ConvCase(name, n, ic, oc, ih, iw, algo="wino", **kw)


I8_CASES = [
    _i8("i8wino_small", 2, 32, 32, 12, 12),
    _i8("i8wino_c4_small", 2, 512, 512, 28, 28),
    _i8("i8wino_partial", 1, 48, 16, 7, 10, relu=True, bias=True),
    _i8("i8wino_k_tail", 1, 144, 32, 8, 8),                      # 9 channel blocks: partial K stage
    _i8("i8wino_u8out", 2, 64, 64, 8, 8, types="u8f32u8f32", relu=True, bias=True, oscale=2.0),
    # F(2x2,3x3): u8 / s8 stores round toward minus infinity
    _i8("i8wino4_small", 2, 32, 32, 12, 12, tile=4),
    _i8("i8wino4_partial_k_tail", 1, 144, 48, 7, 9, tile=4, relu=True, bias=True),
    _i8("i8wino4_u8out", 2, 64, 64, 8, 8, tile=4, types="u8f32u8f32", relu=True, bias=True, oscale=0.05),
    _i8("i8wino4_u8out_norelu_oz", 1, 32, 32, 10, 10, tile=4, types="u8f32u8f32", bias=True, oscale=0.1, oz=100.0),
    _i8("i8wino4_s8out_sum", 1, 32, 64, 8, 8, tile=4, types="u8f32s8f32", bias=True, oscale=0.1, sum=True),
    _i8("i8wino4_resnet_conv4", 2, 256, 256, 14, 14, tile=4, types="u8f32u8f32", relu=True, bias=True, oscale=0.05),
]


@pytest.mark.parametrize("case", I8_CASES, ids=lambda c: c.name)
def test_int8_winograd_matches_oracle(pkg, case):
    import gpuutil as G
    t = R.make_tensors(case)
    case = R.calibrate_tinput(case, t)
    want, dumps = R.oracle_int8_wino(case, t, dumps=True)
    T, OCP = R.wino_tiles(case), R.alignup(case.oc)
    got, d, acc = G.run_gpu(case, t, want_acc=True, acc_shape=(R.wino_edge(case) ** 2, T, OCP))
    try:
        assert d.kernel == "wino_i8_umma"
        assert d.device_status() == 0
        bad = int((acc != dumps["acc"]).sum())
        assert bad == 0, f"{bad} of {acc.size} transform-domain accumulators differ"
        if case.out_dtype == np.float32:
            assert R.rel_l2(got, want) <= 1e-5
        else:
            # requantised output: the fp32 output transform may differ in the last bit, which can
            # flip a rounding; allow 1 LSB on a tiny fraction
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            if case.tile == 4:      # sums only, in the reference's order: bit-exact
                assert diff.max() == 0, f"{int((diff != 0).sum())} of {diff.size} outputs differ"
            else:
                assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    finally:
        d.close()


@pytest.mark.parametrize("src_hw,step", [((28, 28), 2), ((13, 15), 2), ((24, 24), 3)])
def test_fp32_winograd_reads_its_input_with_a_step(pkg, src_hw, step):
    """elb_conv_enqueue_strided: the convolution of every step-th row and column of a larger plane is
    bit-identical to subsampling first (elb_subsample_nChw16c) and convolving the small tensor."""
    import torch
    import gpuutil as G
    E = G.package()
    sh, sw = src_hw
    ih, iw = (sh + step - 1) // step, (sw + step - 1) // step
    case = _f32(f"wino_step{step}_{sh}x{sw}", 2, 32, 48, ih, iw)
    t = R.make_tensors(case)
    d = G.make_desc(case)
    assert d.setup() == E.ELD_OK, E.last_error()
    try:
        assert d.kernel == "wino_f32_umma" and d.input_step_supported()
        rng = np.random.default_rng(R.seed_for(case.name, "big"))
        big = torch.from_numpy(rng.standard_normal((case.n, 2, sh, sw, 16)).astype(np.float32)).cuda()
        small = torch.empty((case.n, 2, ih, iw, 16), dtype=torch.float32, device="cuda")
        assert E.subsample(small, big, case.n, 32, sh, sw, step, step) == E.ELD_OK
        torch.cuda.synchronize()
        assert torch.equal(small, big[:, :, ::step, ::step, :])
        w = torch.from_numpy(t["weights"]).cuda()
        b = torch.from_numpy(t["bias"]).cuda()
        assert d.prepare(w, b) == E.ELD_OK
        out_a = torch.zeros(int(np.prod(R.out_shape(case))), dtype=torch.float32, device="cuda")
        out_b = torch.zeros_like(out_a)
        s = torch.cuda.current_stream().cuda_stream
        assert d.enqueue(out_a, small, None, None, s) == E.ELD_OK
        assert d.enqueue_strided(out_b, big, sh, sw, step, s) == E.ELD_OK
        torch.cuda.synchronize()
        assert d.device_status() == 0
        assert torch.equal(out_a, out_b)
        # a plane that does not subsample to this plan's input is refused
        assert d.enqueue_strided(out_b, big, sh + step, sw, step, s) != E.ELD_OK
    finally:
        d.close()


def test_strided_input_is_refused_where_the_kernel_cannot_do_it(pkg):
    import gpuutil as G
    E = G.package()
    case = _f32("wino4_step", 1, 32, 32, 8, 8, tile=4)
    d = G.make_desc(case)
    assert d.setup() == E.ELD_OK, E.last_error()
    try:
        assert not d.input_step_supported()
    finally:
        d.close()
