"""KV-head-group sharding: the partition / gather logic on CPU, and (on a box with two GPUs) a two-rank run whose
gathered rows must equal the single-GPU rows bit for bit."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_head_groups_partition_the_heads():
    from gwenedeg_b200.sharded import gather_permutation, head_group
    for n_kv, n_heads in ((8, 32), (8, 16), (4, 16)):
        for world in (1, 2, 4):
            seen = []
            for r in range(world):
                h0, per = head_group(n_kv, r, world)
                seen.extend(range(h0, h0 + per))
            assert seen == list(range(n_kv))
            assert np.array_equal(gather_permutation(n_heads, n_kv, world), np.arange(n_heads))
    with pytest.raises(ValueError):
        head_group(8, 0, 3)


WORKER = r'''
import os, sys
sys.path.insert(0, %r)
import numpy as np, torch, torch.distributed as dist
import gwenedeg_b200 as g
from gwenedeg_b200 import synth
from gwenedeg_b200.sharded import HeadShardedContext
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
n_heads, n_kv, hd, n, kvt = 32, 8, 128, 1500, g.KV_Q8
k, v = synth.normal(1, (n, n_kv, hd)), synth.normal(2, (n, n_kv, hd))
q = synth.normal(3, (2, n_heads, hd))
sh = HeadShardedContext(rank, rank, world, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
s = sh.ctx.new_seq(n, kvt)
for lo in range(0, n, 512):
    hi = min(n, lo + 512)
    sh.ctx.pass_begin([(s, lo, hi - lo)])
    sh.ctx.kv_store(0, np.ascontiguousarray(sh.local_kv(k[lo:hi])), np.ascontiguousarray(sh.local_kv(v[lo:hi])))
    sh.ctx.pass_end()
t = sh.ctx.new_seq(n, kvt)
t.copy_from(s, n)
# three decode calls through the fused gather (the merge kernel stores into both ranks' row buffers, used in turn), one through
# NCCL's all-gather: each must equal the single-GPU rows
outs = []
sh.ctx.pass_begin([(s, n - 1, 1), (t, 700, 1)])
for i, mode in enumerate(("peer", "peer", "nccl", "peer")):
    o = sh.attn_decode(0, torch.from_numpy(q * np.float32(1 + i)).cuda(), gather=mode)
    torch.cuda.synchronize()
    outs.append(o.cpu().numpy().copy())
sh.ctx.sync()
sh.ctx.pass_end(commit=False)
if rank == 0:
    full = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
    a = full.new_seq(n, kvt)
    for lo in range(0, n, 512):
        hi = min(n, lo + 512)
        full.pass_begin([(a, lo, hi - lo)]); full.kv_store(0, k[lo:hi], v[lo:hi]); full.pass_end()
    b = full.new_seq(n, kvt); b.copy_from(a, n)
    full.pass_begin([(a, n - 1, 1), (b, 700, 1)])
    for i, got in enumerate(outs):
        want = full.attn_decode(0, q * np.float32(1 + i))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (i, np.abs(got - want).max())
    full.pass_end(commit=False)
    print("SHARDED_OK")
dist.barrier()
dist.destroy_process_group()
'''


@pytest.mark.gpu
def test_two_gpu_head_sharded_decode_equals_single_gpu(tmp_path):
    import gwenedeg_b200 as g
    if g.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                          "--master-port", "29541", str(script)], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-3000:]
    assert "SHARDED_OK" in out.stdout
