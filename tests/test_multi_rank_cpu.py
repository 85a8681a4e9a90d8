"""Multi-rank behaviour on CPU (gloo, world_size 2): the path shards by image with replicated
weights and no exchange, so the only cross-rank logic is (a) which images of the global minibatch a
rank owns, (b) the max-over-ranks of the timings and the whole-job throughput, (c) the reference
arm running on rank 0 alone."""
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
world = dist.get_world_size()
ms, e2e = bench.max_over_ranks([10.0 + rank * 5.0, 100.0 - rank], dist, device="cpu")
val = bench.throughput(2_000_000_000, ms)
# every rank's share of a global batch of 7 images (odd on purpose) and of the 8 chunks of the stack
first, count = bench.split_batch(7, world, rank)
mine = torch.zeros(7, dtype=torch.int64)
mine[first:first + count] = 1
dist.all_reduce(mine)
c_first, c_count = bench.split_batch(8, world, rank)
if rank == 0:
    print(json.dumps({{"ms": ms, "e2e": e2e, "value": val, "owners": mine.tolist(), "chunks0": [c_first, c_count]}}))
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
    # the global batch's op count over the slowest rank's time (strong scaling: the batch is split)
    assert abs(out["value"] - 2e9 / 15e-3 / 1e12) < 1e-9
    assert out["owners"] == [1] * 7            # every image has exactly one owner
    assert out["chunks0"] == [0, 4]


def test_stack_chunks_per_gpu():
    """The stacks' chunk size: 64 images while a GPU has at least two such chunks of the 256, else 32;
    a whole number of chunks per GPU at every N the harness runs."""
    sys.path.insert(0, str(ROOT))
    import bench
    assert [bench.stack_chunk_images(256, w) for w in (1, 2, 4, 8)] == [64, 64, 32, 32]
    assert bench.stack_chunk_images(8, 1) == 8 and bench.stack_chunk_images(96, 1) == 32
    for w in (1, 2, 4, 8):
        n = bench.stack_chunk_images(256, w)
        assert (256 // w) % n == 0 and (256 // n) % w == 0


@pytest.mark.skipif(not (ROOT / "oracle" / "_ref" / "ref_driver").exists(), reason="reference build missing")
def test_reference_arm_runs_on_rank0_only():
    r = _torchrun(["bench.py", "--impl", "reference", "--workload", "c2", "--gpus", "2", "--steps", "3", "--warmup", "1"])
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 2 and d["e2e"]["h2d_bytes_per_step"] == 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["value"] > 0
