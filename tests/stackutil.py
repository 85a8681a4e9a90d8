"""The VGG-16 convolution stack as a test / benchmark workload: layer table, seeded weights and
inputs, the stack object of the library, the u8 calibration pass and the CPU chain it is checked
against.  TEST INFRASTRUCTURE (imports refutil, the door to oracle/); bench.py uses it for its
c5 / c5i8 workloads."""
from __future__ import annotations

import dataclasses
import importlib

PKG = "deep-learning-math-kernel-research_b200"


def oracle_fn(case):
    """The C restatement that matches a case."""
    import refutil as R
    if case.types == "fp32":
        return R.oracle_wino_f32 if case.algo == "wino" else R.oracle_direct_f64
    if case.algo == "wino":
        return R.oracle_int8_wino
    return R.oracle_int8_depthwise if case.g > 1 else R.oracle_int8_conv


VGG16 = [(3, 64, 224), (64, 64, 224), "pool", (64, 128, 112), (128, 128, 112), "pool", (128, 256, 56),
         (256, 256, 56), (256, 256, 56), "pool", (256, 512, 28), (512, 512, 28), (512, 512, 28), "pool",
         (512, 512, 14), (512, 512, 14), (512, 512, 14)]
VGG_NAMES = ["conv1_1", "conv1_2", "conv2_1", "conv2_2", "conv3_1", "conv3_2", "conv3_3", "conv4_1", "conv4_2",
             "conv4_3", "conv5_1", "conv5_2", "conv5_3"]


def vgg_layers():
    """[(ic, oc, hw, subsample_after)] of the 13 convolutions."""
    out = []
    for item in VGG16:
        if item == "pool":
            out[-1] = out[-1][:3] + (2,)
        else:
            out.append(item + (1,))
    return out


# Tuning knobs of the reference's CPU library for the fp32 Winograd layers, from its own tuned
# script for this network (scripts/best_configs/vgg-n64-8180-2s-wino-f4_3.sh:9-31; conv1_1, which
# the script does not list, takes conv1_2's with one input-channel block).  They only matter when a
# case is run through the reference (CPU baseline, parity comparand); the GPU library ignores them.
VGG_F32_KNOBS = {
    "conv1_1": dict(xopt=0xa061, blk_i=1, blk_o=4, flt_t=28), "conv1_2": dict(xopt=0xa061, blk_i=4, blk_o=4, flt_t=28),
    "conv2_1": dict(xopt=0xa061, blk_i=4, blk_o=8, flt_t=28), "conv2_2": dict(xopt=0xa061, blk_i=8, blk_o=8, flt_t=28),
    "conv3_1": dict(xopt=0xa061, blk_i=8, blk_o=8, flt_t=28, pat_o=2),
    "conv3_2": dict(xopt=0xa061, blk_i=8, blk_o=8, flt_t=28, pat_o=2),
    "conv3_3": dict(xopt=0xa061, blk_i=8, blk_o=8, flt_t=28, pat_o=2),
    "conv4_1": dict(xopt=0xa000, blk_i=8, blk_o=8, flt_t=31), "conv4_2": dict(xopt=0xa000, blk_i=8, blk_o=4, flt_t=31),
    "conv4_3": dict(xopt=0xa000, blk_i=8, blk_o=4, flt_t=31), "conv5_1": dict(xopt=0xa000, blk_i=8, blk_o=4, flt_t=28),
    "conv5_2": dict(xopt=0xa000, blk_i=8, blk_o=4, flt_t=28), "conv5_3": dict(xopt=0xa000, blk_i=8, blk_o=4, flt_t=28),
}


def vgg_layer_case(idx, ic, oc, hw, n, int8, iscale=1.0, oscale=1.0, plain_image=False):
    """plain_image: the first layer takes the caller's nchw image (three planes) instead of a blocked
    tensor of 16 channels of which three are real, as the reference's own first-layer runs do
    (scripts/regression-fp32.sh: --input-format=nchw)."""
    import refutil as R
    if plain_image and idx == 0:
        return dataclasses.replace(vgg_layer_case(idx, ic, oc, hw, n, int8, iscale, oscale), ifmt="nchw")
    if int8:
        # blocking in the style of the reference's tuned int8 direct scripts (e.g.
        # scripts/best_configs/resnet-n64-8180-1s-direct-int8.sh): 1.5 - 2 x faster on the CPU than one
        # 16-channel block at a time, same bytes out
        ic2, oc2 = R.alignup(ic) // 16, R.alignup(oc) // 16
        return R.ConvCase(f"vgg_{VGG_NAMES[idx]}", n, ic, oc, hw, hw, types="u8f32u8f32", algo="direct", relu=True,
                          bias=True, iscale=iscale, oscale=oscale,
                          knobs=dict(xopt=0xc160, blk_i=min(8, ic2), blk_o=min(4, max(1, oc2 // 2)), flt_o=2, flt_t=14))
    return R.ConvCase(f"vgg_{VGG_NAMES[idx]}", n, ic, oc, hw, hw, types="fp32", algo="wino", tile=6, relu=True, bias=True,
                      knobs=dict(VGG_F32_KNOBS[VGG_NAMES[idx]]))


def vgg_weights(idx, ic, oc):
    """He-initialised fp32 weights N(0, sqrt(2/(9*ic))) and bias U[-0.1, 0.1], seeded per layer."""
    import numpy as np
    import refutil as R
    g = np.random.Generator(np.random.Philox(R.seed_for("vgg16", VGG_NAMES[idx])))
    w = (g.standard_normal((oc, ic, 3, 3)) * np.sqrt(2.0 / (9 * ic))).astype(np.float32)
    b = np.zeros(R.alignup(oc), np.float32)
    b[:oc] = g.uniform(-0.1, 0.1, oc).astype(np.float32)
    return R.weights_buffer(R.to_OIhw16i16o(w)), b


def vgg_input(chunk: int, n: int, int8: bool, plain: bool = False):
    """Network input of chunk `chunk` (n images), fp32 U[-1,1] / u8 U[0,255]: blocked (3 channels
    zero-padded to 16), or the same values as an nchw image when plain."""
    import numpy as np
    import refutil as R
    g = np.random.Generator(np.random.Philox(R.seed_for("vgg16", f"input{chunk}")))
    if int8:
        x = g.integers(0, 256, (n, 3, 224, 224), dtype=np.uint8)
    else:
        x = g.uniform(-1.0, 1.0, (n, 3, 224, 224)).astype(np.float32)
    return x if plain else R.to_nChw16c(x)


def build_stack(n, int8, device, scales=None, plain_image=False):
    """The 13 convolutions as ONE stack object of the library (elb_stack_*), weights prepared."""
    import torch
    import gpuutil as G
    E = importlib.import_module(PKG)
    layers = vgg_layers()
    descs, cases = [], []
    for k, (ic, oc, hw, _) in enumerate(layers):
        isc, osc = (scales[k], scales[k + 1]) if int8 else (1.0, 1.0)
        case = vgg_layer_case(k, ic, oc, hw, n, int8, isc, osc, plain_image)
        descs.append(G.make_desc(case, device=device))
        cases.append(case)
    st = E.ConvStack(descs, [l[3] for l in layers])
    for k, (ic, oc, _, _) in enumerate(layers):
        w, b = vgg_weights(k, ic, oc)
        wd, bd = torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()
        rc = st.prepare(k, wd, bd)
        if rc != 0:
            raise RuntimeError(f"prepare of {cases[k].name} failed rc={rc}: {E.last_error()}")
    torch.cuda.synchronize()
    return st, cases


def device_view(ptr, nbytes, dtype):
    """A torch view of device memory owned by the library."""
    import torch

    class _Mem:
        pass
    m = _Mem()
    m.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
    return torch.as_tensor(m, device="cuda").view(dtype)


def vgg_calibrate(device):
    """Per-tensor u8 scales of the INT8 stack, frozen before anything is timed: the fp32 stack runs
    once on two images of de-quantised input (scale 1/255) and every layer's scale is its largest
    activation / 255 (zero points are 0: activations are post-ReLU)."""
    import torch
    st, cases = build_stack(2, False, device)
    x = torch.from_numpy(vgg_input(0, 2, True)).cuda().to(torch.float32) * (1.0 / 255.0)
    last = cases[-1]
    y = torch.zeros((2, last.oc // 16, last.oh, last.ow, 16), dtype=torch.float32, device="cuda")
    s = torch.cuda.current_stream()
    assert st.enqueue(y, x, s.cuda_stream) == 0
    torch.cuda.synchronize()
    scales = [1.0 / 255.0]
    for k in range(len(cases)):
        ptr, nb = st.layer_output(k)
        v = y if ptr is None else device_view(ptr, nb, torch.float32)
        scales.append(float(v.max().item()) / 255.0)
    st.close()
    return scales


def stack_reference_chain(cases, x_np, int8, keep=None):
    """The chain on the CPU: every layer through the reference's library (the C restatement where
    it cannot run), the harness keeping every second row / column behind the pooled layers.
    keep: optional list that receives every layer's output (before the subsample)."""
    import numpy as np
    import refutil as R
    x = R.to_nChw16c(x_np) if x_np.ndim == 4 else x_np        # (an nchw image: the CPU side takes it blocked)
    layers = vgg_layers()
    kind = "reference" if R.reference_available() else "port"
    for k, case in enumerate(cases):
        c = dataclasses.replace(case, n=x.shape[0], ifmt="")
        w, b = vgg_weights(k, c.ic, c.oc)
        t = {"input": np.ascontiguousarray(x), "weights": w, "bias": b}
        if kind == "reference":
            y, _ = R.run_reference(c, t)
        else:
            y = oracle_fn(c)(c, t)
        if keep is not None:
            keep.append(y)
        if layers[k][3] == 2:
            y = np.ascontiguousarray(y[:, :, ::2, ::2, :])
        x = y
    return x, kind


def stack_layer_outputs(st, cases, y_last, images=None):
    """Every layer's output tensor (before its subsample) as the stack holds it after a run:
    numpy arrays [images][OC/16][oh][ow][16]; y_last is the caller's tensor of the last layer."""
    import numpy as np
    import torch
    import refutil as R
    outs = []
    for k, c in enumerate(cases):
        dt = torch.uint8 if c.out_dtype == np.uint8 else torch.float32
        ptr, nb = st.layer_output(k)
        v = y_last if ptr is None else device_view(ptr, nb, dt)
        v = v.reshape(c.n, R.alignup(c.oc) // 16, c.oh, c.ow, 16)
        outs.append(v[:images].cpu().numpy() if images else v.cpu().numpy())
    return outs


def per_layer_parity(cases, x_np, gpu_outs, int8):
    """Each layer against the CPU library ON THE GPU'S OWN INPUT of that layer (the previous GPU
    output, subsampled on the host where the stack subsamples): isolates one layer's error from
    what the layers before it accumulated, and still catches any slip in how the layers are wired
    (scale, layout, subsample).  Returns (per-layer figures, comparand): fp32 rel-L2, int8 the
    number of differing bytes."""
    import numpy as np
    import refutil as R
    layers = vgg_layers()
    kind = "reference" if R.reference_available() else "port"
    figures = []
    x = R.to_nChw16c(x_np) if x_np.ndim == 4 else x_np
    for k, case in enumerate(cases):
        c = dataclasses.replace(case, n=x.shape[0], ifmt="")
        w, b = vgg_weights(k, c.ic, c.oc)
        t = {"input": np.ascontiguousarray(x), "weights": w, "bias": b}
        want = R.run_reference(c, t)[0] if kind == "reference" else oracle_fn(c)(c, t)
        got = gpu_outs[k]
        figures.append(int((got != want).sum()) if int8 else R.rel_l2(got, want))
        x = got[:, :, ::2, ::2, :] if layers[k][3] == 2 else got
    return figures, kind
