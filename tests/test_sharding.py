"""Host-side logic of the multi-GPU path: sequence packing, head groups, and a world-size-2 gloo run of the
benchmark's rank plumbing (shards disjoint and complete; timing is the max over ranks)."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_is_a_balanced_partition():
    import bench
    ctx = bench.contexts()
    assert len(ctx) == 64 and ctx.min() >= 512 and ctx.max() <= 32768
    for world in (1, 2, 4, 8):
        sh = bench.shard(ctx, world)
        flat = sorted(i for s in sh for i in s)
        assert flat == list(range(64))
        loads = [int(sum(ctx[i] for i in s)) for s in sh]
        assert max(loads) <= 1.04 * (sum(loads) / world) + 1, (world, loads)


WORKER = r'''
import os, sys
sys.path.insert(0, %r)
import numpy as np, torch, torch.distributed as dist
import bench
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
ctx = bench.contexts()
mine = bench.shard(ctx, world)[rank]
# every rank reports its shard; rank 0 checks the union
got = [None] * world
dist.all_gather_object(got, mine)
t = torch.tensor([10.0 + rank], dtype=torch.float64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)
pos = torch.tensor([float(sum(int(ctx[i]) for i in mine))], dtype=torch.float64)
dist.all_reduce(pos, op=dist.ReduceOp.SUM)
if rank == 0:
    flat = sorted(i for s in got for i in s)
    assert flat == list(range(len(ctx))), flat
    assert t.item() == 10.0 + world - 1
    assert pos.item() == float(ctx.sum())
    print("OK")
dist.destroy_process_group()
'''


def test_two_rank_gloo_plumbing(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29533", str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "OK" in out.stdout


def test_reference_arm_idle_ranks_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"], capture_output=True, text=True,
                         env=env, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""
