"""Device layout converters and the stack glue against a numpy restatement of the reference's
reorder<T, dst, src> (src/elx_reorder.cpp:11-207): every exported pair, both element types, extents
that are not multiples of 16, and the zero fill of blocked padding lanes."""
import numpy as np
import pytest

from gpuutil import package

pytestmark = pytest.mark.gpu


def physical(E, logical, fmt):
    """logical[g][a][b][h][w] -> the tensor in format fmt (blocked lanes past the extents = 0)."""
    g, a, b, h, w = logical.shape
    A, B = -(-a // 16) * 16, -(-b // 16) * 16
    if fmt in (E.nchw, E.oihw, E.goihw):
        return logical.copy()
    if fmt == E.nhwc:
        return logical.transpose(0, 1, 3, 4, 2).copy()
    if fmt in (E.hwio, E.ghwio):
        return logical.transpose(0, 3, 4, 2, 1).copy()
    pad = np.zeros((g, A if fmt != E.nChw16c else a, B, h, w), logical.dtype)
    pad[:, :a, :b] = logical
    if fmt == E.nChw16c:
        return pad.reshape(g, a, B // 16, 16, h, w).transpose(0, 1, 2, 4, 5, 3).copy()
    if fmt in (E.OIhw16i16o, E.gOIhw16i16o):
        return pad.reshape(g, A // 16, 16, B // 16, 16, h, w).transpose(0, 1, 3, 5, 6, 4, 2).copy()
    raise ValueError(fmt)


def pairs(E):
    act = [E.nchw, E.nhwc, E.nChw16c]
    wei = [E.oihw, E.hwio, E.OIhw16i16o]
    gwe = [E.goihw, E.ghwio, E.gOIhw16i16o]
    out = []
    for fam in (act, wei, gwe):
        out += [(d, s) for d in fam for s in fam if d != s]
    return out


@pytest.mark.parametrize("dtype", [np.float32, np.uint8])
@pytest.mark.parametrize("dims", [(1, 2, 19, 5, 7), (3, 35, 16, 3, 3), (1, 4, 64, 14, 14), (2, 17, 3, 1, 1),
                                  (1, 3, 3, 8, 6), (1, 2, 37, 4, 10)])
def test_every_reorder_pair(dtype, dims):
    import torch
    E = package()
    rng = np.random.default_rng(hash((dims, dtype.__name__)) & 0xffff)
    for dst_fmt, src_fmt in pairs(E):
        grouped = dst_fmt in (E.goihw, E.ghwio, E.gOIhw16i16o)
        g, a, b, h, w = dims if grouped else (1,) + dims[1:]
        logical = (rng.integers(1, 255, size=(g, a, b, h, w)).astype(dtype) if dtype == np.uint8
                   else rng.standard_normal((g, a, b, h, w)).astype(dtype))
        src = physical(E, logical, src_fmt)
        if src_fmt in (E.nChw16c, E.OIhw16i16o, E.gOIhw16i16o):
            # padding lanes of a blocked SOURCE hold junk: it must never reach the destination
            mask = physical(E, np.ones_like(logical), src_fmt) == 0
            src[mask] = 77
        want = physical(E, logical, dst_fmt)
        d_src = torch.from_numpy(src).cuda()
        d_dst = torch.full(want.shape, 99, dtype=d_src.dtype, device="cuda")
        ext = (g, a, b, h, w) if grouped else (a, b, h, w)
        rc = E.reorder(d_dst, dst_fmt, d_src, src_fmt, *ext)
        assert rc == E.ELD_OK, E.last_error()
        torch.cuda.synchronize()
        np.testing.assert_array_equal(d_dst.cpu().numpy(), want, err_msg=f"dst {dst_fmt} src {src_fmt} dims {ext}")


def test_reorder_rejects_pairs_across_families():
    import torch
    E = package()
    x = torch.zeros(1024, device="cuda")
    assert E.reorder(x, E.nchw, x, E.oihw, 1, 16, 2, 2) == E.ELD_UNIMPLEMENTED
    assert E.reorder(x, E.nchw, x, E.nchw, 1, 16, 2, 2) == E.ELD_UNIMPLEMENTED
    assert E.reorder(x, E.nChw8c, x, E.nchw, 1, 16, 2, 2) == E.ELD_UNIMPLEMENTED


def test_large_activation_round_trip():
    """ResNet-sized activation (larger than one wave of CTAs): nchw -> nhwc -> nChw16c -> nchw."""
    import torch
    E = package()
    n, c, h, w = 8, 200, 56, 56
    x = torch.randn(n, c, h, w, device="cuda")
    C = -(-c // 16) * 16
    nhwc = torch.empty(n, h, w, c, device="cuda")
    blk = torch.empty(n, C // 16, h, w, 16, device="cuda")
    back = torch.empty_like(x)
    assert E.reorder(nhwc, E.nhwc, x, E.nchw, n, c, h, w) == E.ELD_OK
    assert E.reorder(blk, E.nChw16c, nhwc, E.nhwc, n, c, h, w) == E.ELD_OK
    assert E.reorder(back, E.nchw, blk, E.nChw16c, n, c, h, w) == E.ELD_OK
    torch.cuda.synchronize()
    assert torch.equal(nhwc, x.permute(0, 2, 3, 1))
    assert torch.equal(back, x)
    assert float(blk[:, -1, :, :, c % 16:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [np.float32, np.uint8])
@pytest.mark.parametrize("shape,steps", [((2, 40, 14, 14), (2, 2)), ((1, 16, 7, 9), (2, 2)), ((3, 64, 8, 8), (1, 2)),
                                         ((1, 32, 5, 5), (3, 1))])
def test_subsample(dtype, shape, steps):
    import torch
    E = package()
    n, c, h, w = shape
    C2 = -(-c // 16)
    rng = np.random.default_rng(5)
    src = (rng.integers(0, 255, size=(n, C2, h, w, 16)).astype(dtype) if dtype == np.uint8
           else rng.standard_normal((n, C2, h, w, 16)).astype(dtype))
    want = src[:, :, ::steps[0], ::steps[1], :]
    d_src = torch.from_numpy(src).cuda()
    d_dst = torch.full(want.shape, 9, dtype=d_src.dtype, device="cuda")
    assert E.subsample(d_dst, d_src, n, c, h, w, steps[0], steps[1]) == E.ELD_OK
    torch.cuda.synchronize()
    np.testing.assert_array_equal(d_dst.cpu().numpy(), want)
