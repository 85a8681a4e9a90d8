"""The allocation-free FP32 Winograd entry point (elb_wino_f32_conv_noalloc).

It exists for hosts that may not allocate GPU memory where they run the convolution -- a server
with a fixed, pre-carved memory arena, a latency-critical loop that must not touch the driver's
allocator, a plug-in living inside another framework's budget -- and keeps all of its scratch in
one static 64 MiB device array.  The test calls it through the C-ABI twice in a row (the array
keeps the first call's contents, so the second call must not be disturbed by them) and compares
each result with the plan-based entry point (elb_conv_create / elb_conv_execute) on the same
tensors, within the fp32 Winograd tolerance the other tests use (relative L2 <= 1e-5).
This file is collected last on purpose: a failure here cannot hide another test's result.
"""
import ctypes as C

import numpy as np
import pytest

import refutil as R

pytestmark = pytest.mark.gpu


def _bind(E):
    fn = E.lib.elb_wino_f32_conv_noalloc
    fn.restype = C.c_int32
    fn.argtypes = [C.POINTER(E.ElbConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    return fn


def test_noalloc_matches_plan_based_entry_point_twice(pkg):
    import torch
    import gpuutil as G
    E = G.package()
    fn = _bind(E)
    # two different problems back to back: the second inherits the first one's scratch contents
    cases = [R.ConvCase("noalloc_a", 2, 64, 64, 14, 14, types="fp32", algo="wino", tile=6, relu=True, bias=True),
             R.ConvCase("noalloc_b", 1, 32, 48, 9, 13, types="fp32", algo="wino", tile=6, relu=False, bias=True)]
    for case in cases:
        t = R.make_tensors(case)
        want, d = G.run_gpu(case, t)                  # existing entry point
        d.close()
        x = torch.from_numpy(t["input"]).cuda()
        w = torch.from_numpy(t["weights"]).cuda()
        b = torch.from_numpy(t["bias"]).cuda()
        desc = G.make_desc(case)._c_desc()
        for call in range(2):
            o = torch.full(R.out_shape(case), float("nan"), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            rc = fn(C.byref(desc), o.data_ptr(), x.data_ptr(), w.data_ptr(), b.data_ptr(), None)
            assert rc == E.ELB_OK, E.last_error()
            torch.cuda.synchronize()
            got = o.cpu().numpy()
            assert np.isfinite(got).all()
            err = R.rel_l2(got, want)
            assert err <= 1e-5, f"{case.name} call {call}: rel-L2 {err:.3e}"


def test_noalloc_rejects_oversized_and_unsupported(pkg):
    import torch
    import gpuutil as G
    E = G.package()
    fn = _bind(E)
    dummy = torch.zeros(64, device="cuda")
    big = R.ConvCase("noalloc_big", 64, 256, 256, 56, 56, types="fp32", algo="wino", tile=6)
    rc = fn(C.byref(G.make_desc(big)._c_desc()), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, None)
    assert rc == E.ELB_UNIMPLEMENTED and "scratch" in E.last_error()
    s2 = R.ConvCase("noalloc_s2", 1, 16, 16, 8, 8, stride=2, types="fp32", algo="wino", tile=6)
    rc = fn(C.byref(G.make_desc(s2)._c_desc()), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, None)
    assert rc == E.ELB_UNIMPLEMENTED
