"""Multi-rank behaviour on CPU (gloo, world_size 2): the path shards by image with replicated
weights and no exchange, so the only cross-rank logic is (a) the max-over-ranks of the timings and
the aggregate throughput, (b) the reference arm running on rank 0 alone."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys, json
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank = dist.get_rank()
ms, e2e = bench.max_over_ranks([10.0 + rank * 5.0, 100.0 - rank], dist, device="cpu")
val = bench.aggregate_throughput(ops=2_000_000_000, ms_per_step=ms, world=dist.get_world_size())
if rank == 0:
    print(json.dumps({{"ms": ms, "e2e": e2e, "value": val}}))
dist.destroy_process_group()
"""


def _torchrun(args, timeout=300):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29517"] + args
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))


def test_max_over_ranks_and_aggregate(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    r = _torchrun([str(script)])
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1]
    out = json.loads(line)
    assert out["ms"] == 15.0 and out["e2e"] == 100.0           # max over the two ranks
    # two ranks, each the full batch (weak scaling): 2 * ops / time
    assert abs(out["value"] - 2 * 2e9 / 15e-3 / 1e12) < 1e-9


@pytest.mark.skipif(not (ROOT / "oracle" / "_ref" / "ref_driver").exists(), reason="reference build missing")
def test_reference_arm_runs_on_rank0_only():
    r = _torchrun(["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "3", "--warmup", "1"])
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["e2e"]["h2d_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["value"] > 0
