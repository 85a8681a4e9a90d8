"""Boundary behaviour of elx_conv beyond the plain synchronous call: the asynchronous mode
(eager_mode = false, stream_sync; src/elx_conv.cpp:228-236) and the EULER_VERBOSE perf line
(src/elx_conv.cpp:190-211)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import gpuutil as G
import refutil as R

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("host", [False, True])
def test_async_calls_complete_in_order(pkg, host):
    import torch
    E = pkg
    case = R.ConvCase("async_i8", 6, 64, 64, 14, 14, types="u8f32u8f32", algo="direct", relu=True, bias=True)
    t = R.make_tensors(case)
    want = R.oracle_int8_conv(case, t)
    d = G.make_desc(case)
    assert d.setup() == 0
    d.eager_mode = False
    d.stream_sync = False
    rng = np.random.Generator(np.random.Philox(3))
    x2 = rng.integers(0, 256, t["input"].shape, dtype=np.uint8)
    want2 = R.oracle_int8_conv(case, dict(t, input=x2))
    if host:
        xs = [torch.from_numpy(t["input"]).pin_memory(), torch.from_numpy(x2).pin_memory()]
        outs = [torch.zeros(R.out_shape(case), dtype=torch.uint8).pin_memory() for _ in range(2)]
    else:
        xs = [torch.from_numpy(t["input"]).cuda(), torch.from_numpy(x2).cuda()]
        outs = [torch.zeros(R.out_shape(case), dtype=torch.uint8, device="cuda") for _ in range(2)]
    # two calls without waiting, then a third with stream_sync that completes all of them
    assert E.elx_conv(d, outs[0], xs[0], t["weights"], t["bias"]) == 0, E.last_error()
    assert E.elx_conv(d, outs[1], xs[1], None, None) == 0, E.last_error()
    assert d.wait() == 0
    assert np.array_equal(outs[0].cpu().numpy(), want)
    assert np.array_equal(outs[1].cpu().numpy(), want2)
    d.stream_sync = True
    outs[0].zero_()
    assert E.elx_conv(d, outs[0], xs[1], None, None) == 0
    assert np.array_equal(outs[0].cpu().numpy(), want2)      # no wait() needed: stream_sync waited
    d.close()


def test_euler_verbose_prints_the_perf_line(pkg):
    code = r'''
import sys
sys.path.insert(0, "tests"); sys.path.insert(0, ".")
import numpy as np
import gpuutil as G, refutil as R
E = G.package()
case = R.ConvCase("v", 2, 32, 48, 9, 9, types="u8f32u8f32", algo="direct", relu=True, bias=True)
t = R.make_tensors(case)
d = G.make_desc(case); d.name = "res2a"; assert d.setup() == 0
out = np.zeros(R.out_shape(case), np.uint8)
assert E.elx_conv(d, out, t["input"], t["weights"], t["bias"]) == 0
assert np.array_equal(out, R.oracle_int8_conv(case, t))
'''
    env = dict(os.environ, EULER_VERBOSE="1")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("euler-perf, ")]
    assert len(lines) == 1, r.stdout
    # name,ih:..;oh:..;ic:..;oc:..,algorithm;mode,src:..;wei:..;dst:..,src:..;wei:..;dst:..;b:.., ms
    assert lines[0].startswith("euler-perf, res2a,ih:9;oh:9;ic:32;oc:48,direct_conv;0,src:nChw16c;wei:OIhw16i16o;dst:nChw16c,"
                               "src:u8;wei:f32;dst:u8;b:f32, ")
    assert float(lines[0].rsplit(",", 1)[1]) > 0.0
    # without the variable nothing is printed on stdout
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env={k: v for k, v in os.environ.items() if k != "EULER_VERBOSE"},
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "euler-perf" not in r.stdout
