"""The multi-rank host logic of bench.py on CPU: two gloo ranks, no GPU. The data path has no collective (each rank
runs its own batch shard on its own GPU); what ranks exchange is the timing reduction, and only rank 0 reports."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

WORKER = r"""
import os, sys, json
sys.path.insert(0, os.environ["REPO"])
import torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
step_ms, e2e_s = bench.max_over_ranks([10.0 + 5.0 * rank, 0.5 - 0.1 * rank], dist, device="cpu")
dist.barrier()
if rank == 0:
    print(json.dumps({"step_ms": step_ms, "e2e_s": e2e_s, "value": bench.whole_job_rate(256, world, step_ms), "world": world}))
dist.destroy_process_group()
"""


def test_two_gloo_ranks_reduce_to_the_slowest(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, REPO=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29533", str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(line) == 1, r.stdout
    d = json.loads(line[0])
    assert d["world"] == 2 and d["step_ms"] == 15.0 and d["e2e_s"] == 0.5  # the slower rank wins each entry
    assert abs(d["value"] - 2 * 256 / 0.015) < 1e-6


def test_reference_arm_prints_on_rank0_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0 and r.stdout.strip() == ""
