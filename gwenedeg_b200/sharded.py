"""KV-head-group sharding of the attention over the ranks of a torch.distributed process group.

A batch of independent sequences is sharded by sequence and needs no collective (bench.py does that).  A single
long sequence (or a batch of them too large for one GPU) is instead split by KV head: attention is independent per
KV head, so rank r keeps the cache tiles of heads [r * n_kv / W, (r + 1) * n_kv / W) and computes the query heads
that belong to them; the full rows are rebuilt over NVLink either by the merge kernel itself, which stores its heads of every
row straight into every rank's row buffer (peer stores; gather="peer", the default on more than one rank), or by one NCCL
all-gather of the [rows][heads_local][head_dim] outputs (gather="nccl").  Per-(sequence, head) results are computed whole on
one GPU, so the gathered rows equal the single-GPU rows bit for bit either way.  torch is used for the process group, for
exchanging the buffers' handles and for the tensors handed to NCCL only.
"""
import numpy as np

from .api import Context


def head_group(n_kv_heads, rank, world):
    """(first KV head, KV heads) of `rank`: contiguous equal groups."""
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} KV heads do not split evenly over {world} ranks")
    per = n_kv_heads // world
    return rank * per, per


def gather_permutation(n_heads, n_kv_heads, world):
    """Index array p with full[:, p[j]] = gathered[:, j]: position in the full head order of the j-th head of the
    rank-major concatenation (identity for contiguous groups; kept explicit so other groupings stay testable)."""
    g = n_heads // n_kv_heads
    order = []
    for r in range(world):
        h0, per = head_group(n_kv_heads, r, world)
        order.extend(range(h0 * g, (h0 + per) * g))
    return np.array(order, np.int64)


class HeadShardedContext:
    """This rank's share of a head-sharded model: a Context over its KV-head group, plus the output gather."""

    def __init__(self, device, rank, world, *, n_attn, n_heads, n_kv_heads, head_dim=128, gated=False, max_rows=512, group=None,
                 gather="peer"):
        import torch
        self.torch = torch
        self.rank, self.world, self.group = rank, world, group
        self.n_heads, self.n_kv, self.hd = n_heads, n_kv_heads, head_dim
        self.kv0, self.kv_local = head_group(n_kv_heads, rank, world)
        self.G = n_heads // n_kv_heads
        self.heads_local = self.kv_local * self.G
        self.h0 = self.kv0 * self.G
        self.qh = head_dim * (2 if gated else 1)
        self.ctx = Context(device, n_attn=n_attn, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, gated=gated,
                           kv_head0=self.kv0, kv_heads_local=self.kv_local, max_rows=max_rows)
        self.device = torch.device("cuda", device)
        # the library's kernels, the torch copies around them and NCCL's collectives are ordered on one stream of this
        # object (torch's default stream has the null handle, which the library reads as "my own stream": passing it
        # would leave the two unordered)
        self.stream = torch.cuda.Stream(device=self.device)
        self.ctx.set_stream(self.stream.cuda_stream)
        self.gather = gather if world > 1 else "none"
        self.max_rows = max_rows
        if self.gather == "peer":
            # every rank's row buffer, mapped into every other rank (CUDA IPC handles exchanged through the process group)
            import torch.distributed as dist
            mine = self.ctx.peer_export(max_rows)
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
            self.ctx.peer_import(rank, handles)
            dist.barrier(group=group)

    def _view(self, ptr, shape):
        """A torch view of library-owned device memory."""
        class _Mem:
            pass
        m = _Mem()
        m.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 3, "strides": None}
        return self.torch.as_tensor(m, device=self.device)

    def local_q(self, q_full):
        """The query heads of this rank's KV heads: q_full [rows][n_heads][qh] (torch, on this device)."""
        return q_full[:, self.h0:self.h0 + self.heads_local].contiguous()

    def local_kv(self, k_full):
        """K or V rows of this rank's heads: [rows][n_kv][hd] -> [rows][kv_local][hd] (numpy or torch)."""
        return k_full[:, self.kv0:self.kv0 + self.kv_local]

    def attn_decode(self, layer, q_full, gather=None):
        """Attention of the open pass's rows for all heads: local heads on this GPU, gathered over the ranks (gather: this call's
        way, "peer" or "nccl"; default: the object's)."""
        torch = self.torch
        import torch.distributed as dist
        rows = q_full.shape[0]
        caller = torch.cuda.current_stream(self.device)
        self.stream.wait_stream(caller)  # q_full was produced on the caller's stream
        with torch.cuda.stream(self.stream):
            ql = self.local_q(q_full)
            if (gather or self.gather) == "peer" and self.gather == "peer":
                ptr = self.ctx.attn_decode_gather_dev(layer, ql.data_ptr())
                res = self._view(ptr, (rows, self.n_heads, self.hd))
                for t in (q_full, ql):
                    t.record_stream(self.stream)
                caller.wait_stream(self.stream)
                return res  # (the library's buffer of this step: valid until the call after next)
            out_l = torch.empty((rows, self.heads_local, self.hd), dtype=torch.float32, device=self.device)
            self.ctx.attn_decode_dev(layer, ql.data_ptr(), out_l.data_ptr())
            if self.world == 1:
                res = out_l
            else:
                gathered = torch.empty((self.world, rows, self.heads_local, self.hd), dtype=torch.float32, device=self.device)
                dist.all_gather_into_tensor(gathered, out_l, group=self.group)
                # rank-major -> head order (contiguous groups: a plain transpose)
                res = gathered.permute(1, 0, 2, 3).reshape(rows, self.n_heads, self.hd)
            for t in (q_full, ql, out_l, res):
                t.record_stream(self.stream)
        caller.wait_stream(self.stream)  # the result is used on the caller's stream
        return res

    def close(self):
        self.ctx.close()
