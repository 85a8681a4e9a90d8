"""The allocation-free FP32 Winograd entry point (elb_wino_f32_conv_noalloc).

It exists for hosts that may not allocate GPU memory where they run the convolution -- a server
with a fixed, pre-carved memory arena, a latency-critical loop that must not touch the driver's
allocator, a plug-in living inside another framework's budget -- and keeps all of its scratch in
one static 64 MiB device array.  The test calls it through the C-ABI twice in a row (the array
keeps the first call's contents, so the second call must not be disturbed by them) and compares
each result with the plan-based entry point (elb_conv_create / elb_conv_execute) on the same
tensors AND with the CPU restatement, within the fp32 Winograd tolerance the other tests use
(relative L2 <= 1e-5).  The cases also reach the parts of the path small problems skip: more tiles
than SMs (two accumulator buffers), two tiles of output channels with padded weight rows, channel
counts that are not multiples of 16, the in-place sum; and the free device memory is read before
and after a call to see that nothing was allocated.
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


def _free_bytes():
    import torch
    return torch.cuda.mem_get_info()[0]


CASES = [
    # two different problems back to back: the second inherits the first one's scratch contents
    R.ConvCase("noalloc_a", 2, 64, 64, 14, 14, types="fp32", algo="wino", tile=6, relu=True, bias=True),
    R.ConvCase("noalloc_b", 1, 32, 48, 9, 13, types="fp32", algo="wino", tile=6, relu=False, bias=True),
    # 10 * 8 * 8 tiles -> 5 row blocks x 36 positions = 180 GEMM tiles > 148 SMs, 4 K stages: A in shared
    # memory, two accumulator buffers, CTAs that run two tiles
    R.ConvCase("noalloc_many_tiles", 10, 64, 64, 32, 32, types="fp32", algo="wino", tile=6, relu=True, bias=True),
    # 272 output channels = two n tiles of 144 rows, 16 of them padding in the second
    R.ConvCase("noalloc_two_ntiles", 1, 32, 272, 8, 8, types="fp32", algo="wino", tile=6, relu=True, bias=True),
    # channel tails on both sides
    R.ConvCase("noalloc_tails", 2, 24, 40, 11, 7, types="fp32", algo="wino", tile=6, relu=True, bias=True),
    # in-place sum: the output tensor holds the residual on entry
    R.ConvCase("noalloc_sum", 2, 32, 32, 12, 12, types="fp32", algo="wino", tile=6, relu=True, bias=True, sum=True),
]


def test_noalloc_matches_plan_based_entry_point_twice(pkg):
    import torch
    import gpuutil as G
    E = G.package()
    fn = _bind(E)
    for case in CASES:
        t = R.make_tensors(case)
        want, d = G.run_gpu(case, t)                  # existing entry point
        d.close()
        oracle = R.oracle_wino_f32(case, t)           # and the CPU restatement of the reference
        x = torch.from_numpy(t["input"]).cuda()
        w = torch.from_numpy(t["weights"]).cuda()
        b = torch.from_numpy(t["bias"]).cuda()
        desc = G.make_desc(case)._c_desc()
        for call in range(2):
            init = t["residual"] if case.sum else np.full(R.out_shape(case), np.nan, dtype=np.float32)
            o = G.Guarded(init)
            torch.cuda.synchronize()
            free0 = _free_bytes()
            rc = fn(C.byref(desc), o.data_ptr(), x.data_ptr(), w.data_ptr(), b.data_ptr(), None)
            assert rc == E.ELB_OK, E.last_error()
            torch.cuda.synchronize()
            if call == 1:      # (the very first call on a device may load the kernels' code)
                assert _free_bytes() == free0, "the call changed the amount of free device memory"
            assert E.lib.elb_wino_f32_noalloc_status() == 0
            o.check(f"{case.name}: output tensor")
            got = o.numpy()
            assert np.isfinite(got).all()
            err = R.rel_l2(got, want)
            assert err <= 1e-5, f"{case.name} call {call}: rel-L2 {err:.3e} against the plan-based entry point"
            err = R.rel_l2(got, oracle)
            assert err <= 1e-5, f"{case.name} call {call}: rel-L2 {err:.3e} against the CPU restatement"


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
