"""The chain of convolutions (elb_stack_*): the 13 layers of VGG-16 at n = 2, fp32 Winograd and
INT8 direct (u8 requantised between layers, stride-2 subsample between stages), GPU chain against
the CPU chain through the reference library (the C restatement where that cannot run).  Per-layer
tests cannot catch an inter-layer scale or layout slip; this one compares EVERY layer's output.
INT8: bit-exact at every layer of the chain.  fp32: every layer within rel-L2 <= 1e-5 of the CPU
library on the same input (the GPU's own previous activation, so one layer's rounding is not
charged to the next), and the whole chain within 1e-4 of the CPU chain (thirteen layers of
~1e-6 .. 3e-6 each compound; measured 2.3e-5 at the last layer).
"""
import numpy as np
import pytest

import gpuutil as G
import refutil as R
import stackutil as S

pytestmark = pytest.mark.gpu


def _gpu_chain(st, cases, x_np, dtype):
    import torch
    x = torch.from_numpy(x_np).cuda()
    last = cases[-1]
    y = torch.zeros((x_np.shape[0], last.oc // 16, last.oh, last.ow, 16), dtype=dtype, device="cuda")
    assert st.enqueue(y, x, torch.cuda.current_stream().cuda_stream) == 0, G.package().last_error()
    torch.cuda.synchronize()
    outs = []
    for k, c in enumerate(cases):
        ptr, nb = st.layer_output(k)
        v = y if ptr is None else S.device_view(ptr, nb, dtype)
        outs.append(v.cpu().numpy().reshape(c.n, R.alignup(c.oc) // 16, c.oh, c.ow, 16))
    return outs, y


def test_vgg16_chain_fp32_every_layer(pkg):
    import torch
    n = 2
    st, cases = S.build_stack(n, False, 0)
    x_np = S.vgg_input(0, n, False)
    got, _ = _gpu_chain(st, cases, x_np, torch.float32)
    errs, _ = S.per_layer_parity(cases, x_np, got, False)
    for c, err in zip(cases, errs):
        assert err <= 1e-5, f"{c.name}: rel-L2 {err:.3e} against the CPU library on the same input"
    want = []
    S.stack_reference_chain(cases, x_np, False, keep=want)
    for k, c in enumerate(cases):
        err = R.rel_l2(got[k], want[k])
        assert err <= 1e-4, f"{c.name}: rel-L2 {err:.3e} after {k + 1} chained layers"
    st.close()


def test_vgg16_chain_fp32_takes_the_plain_image(pkg):
    """The first layer given the caller's nchw image (three planes, how the reference's own first-layer
    runs pass it) gives the result of the chain fed the blocked tensor -- to fp32 rounding: the image
    goes through the tensor-core first-layer kernel, the blocked tensor through the CUDA-core one --
    on the device and, byte for byte the same, through elb_stack_execute from the host; the image is
    less than a fifth of the bytes."""
    import torch
    n = 2
    st_b, cases_b = S.build_stack(n, False, 0)
    st_p, cases_p = S.build_stack(n, False, 0, plain_image=True)
    assert cases_p[0].ifmt == "nchw"
    x_b, x_p = S.vgg_input(0, n, False), S.vgg_input(0, n, False, plain=True)
    assert x_p.shape == (n, 3, 224, 224) and x_p.nbytes * 5 < x_b.nbytes
    got_b, _ = _gpu_chain(st_b, cases_b, x_b, torch.float32)
    got_p, y_p = _gpu_chain(st_p, cases_p, x_p, torch.float32)
    for k, c in enumerate(cases_b):
        err = R.rel_l2(got_p[k], got_b[k])
        assert err <= (2e-6 if k == 0 else 1e-5), f"{c.name}: rel-L2 {err:.3e} between plain image and blocked tensor"
    errs, _ = S.per_layer_parity(cases_p, x_p, got_p, False)
    assert errs[0] <= 1e-5, f"first layer on the plain image: rel-L2 {errs[0]:.3e} against the CPU library"
    hy = np.zeros(tuple(y_p.shape), np.float32)
    assert st_p.execute(hy, x_p, n) == 0, G.package().last_error()
    assert np.array_equal(hy, got_p[-1])
    st_b.close()
    st_p.close()


def test_vgg16_chain_int8_every_layer_bit_exact(pkg):
    import torch
    n = 2
    scales = S.vgg_calibrate(0)
    st, cases = S.build_stack(n, True, 0, scales)
    x_np = S.vgg_input(0, n, True)
    got, _ = _gpu_chain(st, cases, x_np, torch.uint8)
    want = []
    S.stack_reference_chain(cases, x_np, True, keep=want)
    for k, c in enumerate(cases):
        bad = int((got[k] != want[k]).sum())
        assert bad == 0, f"{c.name}: {bad} of {got[k].size} u8 outputs differ after {k + 1} chained layers"
    st.close()


def test_stack_execute_host_batches_match_enqueue(pkg):
    """elb_stack_execute on HOST tensors of several batches (two staging slots, one CUDA graph per
    slot, copies overlapped with the chain) returns the bytes the plain enqueue path produces."""
    import torch
    E = G.package()
    # a short int8 chain with a subsample in the middle and behind the last layer
    n = 2
    dims = [(16, 32, 20, 2), (32, 48, 10, 1), (48, 32, 10, 2)]
    cases, descs = [], []
    for k, (ic, oc, hw, step) in enumerate(dims):
        c = R.ConvCase(f"stk{k}", n, ic, oc, hw, hw, types="u8f32u8f32", algo="direct", relu=True, bias=True,
                       iscale=0.02, oscale=0.05)
        cases.append(c)
        descs.append(G.make_desc(c))
    st = E.ConvStack(descs, [d[3] for d in dims])
    tens = []
    for k, c in enumerate(cases):
        t = R.make_tensors(c)
        tens.append(t)
        assert st.prepare(k, torch.from_numpy(t["weights"]).cuda(), torch.from_numpy(t["bias"]).cuda()) == 0
    batches = 3
    rng = np.random.Generator(np.random.Philox(7))
    x_np = rng.integers(0, 256, (batches * n, 1, 20, 20, 16), dtype=np.uint8)
    out_shape = (batches * n, 2, 5, 5, 16)
    # reference bytes: every batch through the enqueue path
    x = torch.from_numpy(x_np).cuda()
    y = torch.zeros(out_shape, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for b in range(batches):
        assert st.enqueue(y[b * n:(b + 1) * n], x[b * n:(b + 1) * n], s) == 0, E.last_error()
    torch.cuda.synchronize()
    want = y.cpu().numpy()
    # and the chain itself against the CPU restatement (layer by layer on the first batch)
    xx = x_np[:n]
    for k, c in enumerate(cases):
        o = R.oracle_int8_conv(c, {"input": np.ascontiguousarray(xx), "weights": tens[k]["weights"], "bias": tens[k]["bias"]})
        xx = o[:, :, ::dims[k][3], ::dims[k][3], :]
    assert np.array_equal(want[:n], xx)
    for trial in range(2):      # the second call replays the captured graphs
        hy = np.zeros(out_shape, np.uint8)
        assert st.execute(hy, x_np, batches * n) == 0, E.last_error()
        assert np.array_equal(hy, want), f"trial {trial}"
    assert st.execute(hy, x_np, batches * n + 1) != 0      # not a whole number of batches
    assert st.launch_count() > 0
    st.close()


def test_stack_rejects_mismatched_layers(pkg):
    E = G.package()
    a = G.make_desc(R.ConvCase("a", 2, 16, 32, 8, 8, types="u8f32u8f32", algo="direct", relu=True, bias=True))
    b = G.make_desc(R.ConvCase("b", 2, 48, 32, 8, 8, types="u8f32u8f32", algo="direct", relu=True, bias=True))
    with pytest.raises(RuntimeError):
        E.ConvStack([a, b])


@pytest.mark.parametrize("int8", [False, True], ids=["fp32_folds_the_subsample", "int8_keeps_the_kernel"])
def test_stack_subsample_between_layers(pkg, int8):
    """Two layers with a stride-2 subsample between them.  fp32 Winograd: the second layer reads every
    second row and column of the first layer's full output itself (3 + 3 launches, no subsample
    kernel); INT8 direct: one kernel per layer plus the subsample kernel.  Either way the chain equals
    the CPU chain with an explicit subsample."""
    import torch
    E = G.package()
    n = 2
    if int8:
        cases = [R.ConvCase("sub_a", n, 32, 32, 24, 24, types="u8f32u8f32", algo="direct", relu=True, bias=True, iscale=0.02, oscale=0.05),
                 R.ConvCase("sub_b", n, 32, 48, 12, 12, types="u8f32u8f32", algo="direct", relu=True, bias=True, iscale=0.05, oscale=0.1)]
    else:
        cases = [R.ConvCase("sub_a", n, 32, 32, 24, 24, types="fp32", algo="wino", tile=6, relu=True, bias=True),
                 R.ConvCase("sub_b", n, 32, 48, 12, 12, types="fp32", algo="wino", tile=6, relu=True, bias=True)]
    st = E.ConvStack([G.make_desc(c) for c in cases], [2, 1])
    tens = [R.make_tensors(c) for c in cases]
    for k, t in enumerate(tens):
        assert st.prepare(k, torch.from_numpy(t["weights"]).cuda(), torch.from_numpy(t["bias"]).cuda()) == 0
    x_np = tens[0]["input"]
    x = torch.from_numpy(x_np).cuda()
    dt = torch.uint8 if int8 else torch.float32
    y = torch.zeros((n, 3, 12, 12, 16), dtype=dt, device="cuda")
    before = st.launch_count()
    assert st.enqueue(y, x, torch.cuda.current_stream().cuda_stream) == 0, E.last_error()
    torch.cuda.synchronize()
    assert st.launch_count() - before == (3 if int8 else 6)
    oracle = R.oracle_int8_conv if int8 else R.oracle_wino_f32
    mid = oracle(cases[0], {"input": x_np, "weights": tens[0]["weights"], "bias": tens[0]["bias"]})
    want = oracle(cases[1], {"input": np.ascontiguousarray(mid[:, :, ::2, ::2, :]), "weights": tens[1]["weights"],
                             "bias": tens[1]["bias"]})
    got = y.cpu().numpy()
    if int8:
        assert np.array_equal(got, want)
    else:
        assert R.rel_l2(got, want) <= 2e-5      # two chained fp32 layers
    st.close()
