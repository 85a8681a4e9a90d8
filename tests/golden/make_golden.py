"""Generate the golden fixtures of this folder by running the UNMODIFIED reference library.

    python tests/golden/make_golden.py

Needs oracle/_ref (oracle/build_ref.sh, i.e. the reference tree and an AVX-512 VNNI host).  The
reference ships no golden vectors of its own (its only test seeds its inputs from the clock), so
these files are its outputs on small seeded problems: one .npz per case holding the blocked input /
weights / bias (/ residual) tensors, the case parameters and the reference's output tensor.  They
travel with the repository so that the CPU restatement and the CUDA kernels can be checked against
the reference on machines where the reference cannot run.
"""
import dataclasses
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import refutil as R  # noqa: E402


def cases():
    C = R.ConvCase
    i8 = dict(types="u8f32u8f32", relu=True, bias=True)
    out = [
        C("g_i8_1x1", 1, 64, 32, 7, 7, kh=1, kw=1, pad=0, algo="1x1", **i8),
        C("g_i8_1x1_c2_shape", 1, 1024, 256, 14, 14, kh=1, kw=1, pad=0, algo="1x1", **i8),
        C("g_i8_1x1_sum", 1, 32, 32, 6, 6, kh=1, kw=1, pad=0, algo="1x1", sum=True, sscale=0.5, oscale=0.5, **i8),
        C("g_i8_1x1_s8_norelu", 1, 48, 16, 5, 5, kh=1, kw=1, pad=0, algo="1x1", types="u8f32s8f32", bias=True,
          oscale=4.0),
        # (no int8-direct case with fp32 output: the reference's KxK class leaves the user tensor
        #  untouched for that type combination and its 1x1 class has no such instance)
        C("g_i8_3x3_s1", 1, 32, 32, 12, 12, algo="direct", **i8),
        C("g_i8_3x3_s2", 1, 32, 32, 14, 14, stride=2, algo="direct", **i8),
        C("g_i8_3x3_c3_shape", 1, 128, 256, 56, 56, stride=2, algo="direct", **i8),
        # non-zero input zero point WITH padding: border pixels see fewer taps, so their shift differs
        # (the reference's per-position tables, src/elx_int8_conv_direct.cpp:227-423)
        C("g_i8_3x3_s1_iz128", 1, 32, 32, 12, 12, algo="direct", iz=128.0, oscale=0.3, **i8),
        C("g_i8_3x3_s2_iz128", 2, 32, 48, 14, 14, stride=2, algo="direct", iz=128.0, oscale=0.3, **i8),
        C("g_i8_5x5_iz", 1, 32, 32, 14, 14, kh=5, kw=5, pad=2, algo="direct", iz=3.0, oscale=0.5, **i8),
        C("g_i8_7x7_s2_iz_s8", 1, 32, 32, 28, 28, kh=7, kw=7, pad=3, stride=2, algo="direct", types="u8f32s8f32",
          bias=True, iz=17.0, oscale=0.5),
        C("g_wino_f32", 1, 32, 32, 12, 12, types="fp32", algo="wino", tile=6, relu=True, bias=True),
        C("g_wino_f32_partial", 1, 16, 16, 10, 7, types="fp32", algo="wino", tile=6, bias=True),
        C("g_wino_f32_sum", 1, 16, 32, 8, 8, types="fp32", algo="wino", tile=6, bias=True, sum=True),
        C("g_wino_i8_f32", 1, 32, 32, 8, 8, types="u8f32f32f32", algo="wino", tile=6),
        C("g_wino_i8_u8", 1, 32, 16, 8, 8, types="u8f32u8f32", algo="wino", tile=6, relu=True, bias=True, oscale=2.0),
        # F(2x2,3x3) = tile_size 4 (its u8 / s8 stores round toward minus infinity)
        C("g_wino4_f32", 1, 32, 32, 12, 12, types="fp32", algo="wino", tile=4, relu=True, bias=True),
        C("g_wino4_f32_partial_sum", 1, 16, 32, 9, 7, types="fp32", algo="wino", tile=4, bias=True, sum=True),
        C("g_wino4_i8_f32", 1, 32, 32, 8, 8, types="u8f32f32f32", algo="wino", tile=4),
        C("g_wino4_i8_u8", 1, 32, 16, 9, 8, types="u8f32u8f32", algo="wino", tile=4, relu=True, bias=True, oscale=0.05),
        C("g_wino4_i8_s8", 1, 48, 32, 6, 6, types="u8f32s8f32", algo="wino", tile=4, bias=True, oscale=0.1),
        # fp32 direct convolutions (1x1 and KxK); the in-place sum IS honoured on these paths
        C("g_f32_1x1", 1, 64, 32, 7, 7, kh=1, kw=1, pad=0, types="fp32", algo="1x1", relu=True, bias=True),
        C("g_f32_1x1_s2_sum", 1, 32, 32, 8, 8, kh=1, kw=1, pad=0, stride=2, types="fp32", algo="1x1", bias=True, sum=True),
        C("g_f32_3x3_s2", 1, 32, 32, 14, 14, stride=2, types="fp32", algo="direct", relu=True, bias=True),
        C("g_f32_3x3_sum", 1, 32, 16, 9, 9, types="fp32", algo="direct", relu=True, bias=True, sum=True),
        C("g_f32_7x7_s2", 1, 32, 32, 14, 14, kh=7, kw=7, pad=3, stride=2, types="fp32", algo="direct", relu=True, bias=True),
        # int8 depthwise 3x3 (g = channels, goihw weights); flt_t is the reference's row chunk T, which
        # decides which u8 pixels are floored and which are rounded to nearest
        C("g_dw_s1_u8_t14", 1, 32, 32, 28, 28, g=32, algo="direct", knobs=dict(flt_t=14), **i8),
        C("g_dw_s1_u8_t7", 1, 48, 48, 14, 14, g=48, algo="direct", knobs=dict(flt_t=7), **i8),
        C("g_dw_s2_u8_t7", 1, 64, 64, 28, 28, g=64, stride=2, algo="direct", knobs=dict(flt_t=7), **i8),
        C("g_dw_s2_p0_s8", 1, 32, 32, 15, 15, g=32, stride=2, pad=0, algo="direct", types="u8f32s8f32", bias=True,
          knobs=dict(flt_t=7)),
        C("g_dw_s1_u8_norelu_wrap", 1, 32, 32, 12, 20, g=32, algo="direct", types="u8f32u8f32", bias=True, oscale=0.02,
          knobs=dict(flt_t=6)),
        C("g_dw_s1_u8_iz", 1, 32, 32, 10, 10, g=32, algo="direct", iz=3.0, knobs=dict(flt_t=5), **i8),
    ]
    return out


def main():
    assert R.reference_available(), "oracle/_ref is missing or this CPU has no AVX-512 VNNI"
    only = sys.argv[1:]           # optional: name prefixes of the fixtures to (re)generate
    for case in cases():
        if only and not any(case.name.startswith(o) for o in only):
            continue
        t = R.make_tensors(case)
        if case.algo == "wino" and case.types != "fp32":
            case = R.calibrate_tinput(case, t)
        if case.algo != "wino" and case.g == 1:
            # the reference's direct kernels need explicit blocking (its defaults divide by zero):
            # all input-channel blocks in one pass, one 16-channel output block, T <= 7 pixels
            case = dataclasses.replace(case, knobs=dict(blk_i=R.alignup(case.ic) // 16, blk_o=1, flt_o=1,
                                                        flt_t=min(case.ow, 7)))
        ref, info = R.run_reference(case, t)
        assert info["rc"] == 0
        arrays = dict(input=t["input"], weights=t["weights"], bias=t["bias"], output=ref)
        if case.sum:
            arrays["residual"] = t["residual"]
        meta = dataclasses.asdict(case)
        np.savez_compressed(HERE / f"{case.name}.npz", meta=json.dumps(meta), **arrays)
        print(f"{case.name}: output {ref.shape} {ref.dtype}, {(HERE / (case.name + '.npz')).stat().st_size} bytes")


if __name__ == "__main__":
    main()
