"""The multi-GPU host logic on CPU: the batch partition of the Net group (contiguous slices, offsets, gather into the
caller's buffer), alone and across two gloo ranks, and the timing reduction of bench.py. No GPU. The data path has no
collective (each replica runs its own slice on its own GPU)."""
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


def test_partition_is_contiguous_balanced_and_complete():
    from tensor_b200 import partition
    for n in (0, 1, 2, 7, 8, 9, 255, 256, 2048, 2051):
        for parts in (1, 2, 3, 4, 8):
            slices = [partition(n, parts, i) for i in range(parts)]
            assert slices[0][0] == 0
            for (f0, c0), (f1, _) in zip(slices, slices[1:]):
                assert f1 == f0 + c0  # contiguous, in order
            assert sum(c for _, c in slices) == n
            counts = [c for _, c in slices]
            assert max(counts) - min(counts) <= 1 and counts == sorted(counts, reverse=True)  # earlier slices take the extra images
    assert partition(10, 4, 7) == (0, 0) and partition(10, 0, 0) == (0, 0)  # out of range: empty


SHARD_WORKER = r"""
import os, sys, json
sys.path.insert(0, os.environ["REPO"])
import numpy as np
import torch, torch.distributed as dist
from tensor_b200 import partition
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
n, per_image = 11, 6
first, count = partition(n, world, rank)
# every rank "computes" its own slice of the batch (a function of the global image index) ...
mine = np.array([[100 * (first + i) + j for j in range(per_image)] for i in range(count)], np.float32).reshape(count, per_image)
# ... and the slices are gathered into one buffer at their offsets, as ott_net_group_forward does with host pointers
out = torch.zeros(n, per_image)
big = max(partition(n, world, r)[1] for r in range(world))  # gloo all_gather wants equal shapes: pad the ragged slice
padded = torch.zeros(big, per_image)
padded[:count] = torch.from_numpy(mine)
bufs = [torch.zeros(big, per_image) for _ in range(world)]
dist.all_gather(bufs, padded)
pieces = [b[:partition(n, world, r)[1]] for r, b in enumerate(bufs)]
for r, p in enumerate(pieces):
    f, c = partition(n, world, r)
    out[f:f + c] = p
want = torch.tensor([[100 * i + j for j in range(per_image)] for i in range(n)], dtype=torch.float32)
ok = bool(torch.equal(out, want))
dist.barrier()
if rank == 0:
    print(json.dumps({"ok": ok, "slices": [partition(n, world, r) for r in range(world)]}))
dist.destroy_process_group()
"""


def test_two_gloo_ranks_shard_and_gather_a_batch(tmp_path):
    script = tmp_path / "shard_worker.py"
    script.write_text(SHARD_WORKER)
    env = dict(os.environ, REPO=str(ROOT), MASTER_ADDR="127.0.0.1", MASTER_PORT="29535", OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29535", str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][0])
    assert d["ok"] and d["slices"] == [[0, 6], [6, 5]]


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
