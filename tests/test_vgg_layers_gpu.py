"""Every distinct layer shape of the VGG-16 convolution stack (the multi-layer benchmark
configuration) at one image, against the CPU restatement: fp32 Winograd F(4x4,3x3) within the fp32
tolerance, INT8 direct bit-exact.  conv1_1 has 3 input channels (zero-padded to one block): the
library serves that Winograd request with its direct kernel for layers of at most four input
channels, still within the fp32 tolerance of the reference's Winograd result."""
import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu

SHAPES = [(3, 64, 224), (64, 64, 224), (64, 128, 112), (128, 128, 112), (128, 256, 56), (256, 256, 56),
          (256, 512, 28), (512, 512, 28), (512, 512, 14)]


@pytest.mark.parametrize("ic,oc,hw", SHAPES)
def test_vgg_layer_fp32_winograd(pkg, ic, oc, hw):
    import gpuutil as G
    case = R.ConvCase(f"vggl_f32_{ic}_{oc}_{hw}", 1, ic, oc, hw, hw, types="fp32", algo="wino", tile=6, relu=True,
                      bias=True)
    t = R.make_tensors(case)
    want = R.oracle_wino_f32(case, t)
    got, d = G.run_gpu(case, t)
    try:
        assert d.kernel == ("f32_small_ic" if ic <= 4 else "wino_f32_umma") and d.device_status() == 0
        assert R.rel_l2(got, want) <= 1e-5
    finally:
        d.close()


@pytest.mark.parametrize("ic,oc,hw", SHAPES)
def test_vgg_layer_int8_direct(pkg, ic, oc, hw):
    import gpuutil as G
    case = R.ConvCase(f"vggl_i8_{ic}_{oc}_{hw}", 1, ic, oc, hw, hw, types="u8f32u8f32", algo="direct", relu=True,
                      bias=True, iscale=0.02, oscale=0.5)
    t = R.make_tensors(case)
    want, want_acc = R.oracle_int8_conv(case, t, want_acc=True)
    got, d, acc = G.run_gpu(case, t, want_acc=True)
    try:
        assert d.kernel == "i8_conv_umma" and d.device_status() == 0
        assert np.array_equal(acc, want_acc)
        assert np.array_equal(got, want)
    finally:
        d.close()
