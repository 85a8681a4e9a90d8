"""Loading of the golden fixtures (outputs of the unmodified reference, see tests/golden/make_golden.py)."""
import json
from pathlib import Path

import numpy as np

import refutil as R

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def golden_names():
    return sorted(p.stem for p in GOLDEN_DIR.glob("*.npz"))


def load_golden(name):
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    meta = json.loads(str(z["meta"]))
    case = R.ConvCase(**meta)
    t = {k: z[k] for k in ("input", "weights", "bias")}
    if "residual" in z.files:
        t["residual"] = z["residual"]
    return case, t, z["output"]


def check_against_golden(case, got, want):
    if case.g > 1:      # depthwise: the reference leaves garbage in channel lanes beyond g; compare the real ones
        cb = case.oc // 16
        assert case.oc % 16 == 0
        got, want = got[:, :cb], want[:, :cb]
    """Bit-exact for integer outputs; fp32 Winograd within 1e-5 relative L2; int8 direct with f32
    output bit-exact (one fma on exact integers)."""
    if case.out_dtype != np.float32:
        if case.algo == "wino" and case.tile == 4:      # sums only: bit-exact
            assert np.array_equal(got, want), f"{int((got != want).sum())} of {got.size} outputs differ"
        elif case.algo == "wino":
            diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert diff.max() <= 1 and (diff != 0).mean() < 5e-3, f"{int((diff != 0).sum())} outputs differ"
        else:
            assert np.array_equal(got, want), f"{int((got != want).sum())} of {got.size} outputs differ"
    elif case.algo == "wino" or case.types == "fp32":
        err = R.rel_l2(got, want)
        assert err <= 1e-5, f"rel-L2 {err:.3e}"
    else:
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
