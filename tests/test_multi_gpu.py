"""elb_conv_multi_*: one convolution whose minibatch is split over several GPUs.  GPU r runs images
[r*N/G, (r+1)*N/G) of ONE host tensor; weights are replicated; the result must equal the one-GPU
result byte for byte.  On a box with a single GPU the same device is named twice, which runs the
same code (two plans, two host threads, two slabs) without the second GPU.
"""
import numpy as np
import pytest

import gpuutil as G
import refutil as R

pytestmark = pytest.mark.gpu


def _devices():
    import torch
    return [0, 1] if torch.cuda.device_count() >= 2 else [0, 0]


@pytest.mark.parametrize("case", [
    R.ConvCase("multi_i8_3x3", 5, 32, 48, 12, 12, types="u8f32u8f32", algo="direct", relu=True, bias=True),
    R.ConvCase("multi_i8_1x1_sum", 4, 64, 32, 7, 7, kh=1, kw=1, pad=0, types="u8f32u8f32", algo="1x1", relu=True, bias=True,
               sum=True),
    R.ConvCase("multi_f32_wino", 3, 32, 32, 10, 10, types="fp32", algo="wino", tile=6, relu=True, bias=True),
], ids=lambda c: c.name)
def test_split_equals_single_gpu(pkg, case):
    E = pkg
    t = R.make_tensors(case)
    want, d1 = G.run_gpu(case, t, host_buffers=True)
    d1.close()
    d = G.make_desc(case)
    m = E.MultiConv(d, devices=_devices())
    parts = m.parts()
    assert [p[1] for p in parts] == [0, case.n // 2] and sum(p[2] for p in parts) == case.n
    out = np.zeros(R.out_shape(case), dtype=case.out_dtype)
    for call in range(2):
        if case.sum:
            out[...] = t["residual"]
        assert m.execute(out, t["input"], t["weights"], t["bias"]) == 0, E.last_error()
        assert np.array_equal(out, want), f"call {call}: split result differs from the one-GPU result"
    m.close()
    if case.types != "fp32":
        assert np.array_equal(want, R.oracle_int8_conv(case, t))


def test_multi_rejects_device_tensors_and_too_many_gpus(pkg):
    import torch
    E = pkg
    case = R.ConvCase("multi_bad", 2, 16, 16, 6, 6, types="u8f32u8f32", algo="direct", relu=True, bias=True)
    t = R.make_tensors(case)
    m = E.MultiConv(G.make_desc(case), devices=_devices())
    x = torch.from_numpy(t["input"]).cuda()
    out = np.zeros(R.out_shape(case), dtype=np.uint8)
    assert m.execute(out, x, t["weights"], t["bias"]) != 0
    m.close()
    with pytest.raises(RuntimeError):
        E.MultiConv(G.make_desc(case), n_devices=torch.cuda.device_count() + 1)


def test_more_gpus_than_images_leaves_spares_idle(pkg):
    E = pkg
    case = R.ConvCase("multi_one", 1, 16, 16, 6, 6, types="u8f32u8f32", algo="direct", relu=True, bias=True)
    m = E.MultiConv(G.make_desc(case), devices=_devices())
    assert len(m.parts()) == 1
    m.close()


def test_euler_gpus_through_the_cpp_surface(pkg, monkeypatch):
    """EULER_GPUS=G makes euler::elx_conv itself split the minibatch (the same C++ driver that runs the
    reference library, linked against this repository's libel.so).  Needs two GPUs; with one, the
    request for a second GPU must come back as a setup error code, not as a crash."""
    import torch
    if not R.DROPIN_DRIVER.exists():
        pytest.skip("tests/bin/euler_driver_b200 was not built (reference headers missing at build time)")
    case = R.baseline_case("c3", 6)
    t = R.make_tensors(case)
    monkeypatch.setenv("EULER_GPUS", "2")
    if torch.cuda.device_count() >= 2:
        out, info = R.run_reference(case, t, driver=R.DROPIN_DRIVER, iters=2, warmup=0)
        assert info["rc_setup"] == 0 and info["rc"] == 0
        assert np.array_equal(out, R.oracle_int8_conv(case, t))
    else:
        with pytest.raises(RuntimeError) as e:
            R.run_reference(case, t, driver=R.DROPIN_DRIVER)
        assert '"rc_setup": 2' in str(e.value)
