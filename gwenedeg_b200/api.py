"""Thin object layer over the C ABI (include/rq_cuda.h) for Python hosts: tests, the benchmark, notebooks.

It mirrors how gwenedeg's C host drives the path: a context (RqCtx), sequences that own their KV cache and
DeltaNet state (RqSeq), and passes over segments of rows (rq_forward_batch; reference src/forward.c:3762) with one
call per layer.  All arithmetic happens inside librq_cuda.so; numpy arrays are only the host buffers.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import KV_F16, KV_NAMES, KV_Q4, KV_Q4K4, KV_Q8, RqCudaModel, RqCudaSegment  # noqa: F401


class RqCudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"rq_cuda error {code}: {msg}")
        self.code = code


def device_count():
    return _lib.load().rq_cuda_device_count()


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, int):
        return C.c_void_p(a)
    return a.ctypes.data_as(C.c_void_p)


class Context:
    """One device's compute context for a model shape (attention heads and / or DeltaNet heads)."""

    def __init__(self, device=0, *, n_attn=0, n_heads=0, n_kv_heads=0, head_dim=128, gated=False, n_lin=0, dn_nk=0,
                 dn_nv=0, dn_dk=128, dn_dv=128, dn_conv=4, kv_head0=0, kv_heads_local=0, max_rows=512):
        self.L = _lib.load()
        self.model = RqCudaModel(n_attn, n_heads, n_kv_heads, head_dim, int(gated), n_lin, dn_nk, dn_nv, dn_dk, dn_dv,
                                 dn_conv, kv_head0, kv_heads_local)
        h = C.c_void_p()
        rc = self.L.rq_cuda_init(device, C.byref(self.model), max_rows, C.byref(h))
        if rc:
            raise RqCudaError(rc, "rq_cuda_init failed (no B200 visible, or invalid model shape)")
        self.h = h
        self.device = device
        self.hd = head_dim
        self.n_kv = (kv_heads_local or n_kv_heads) if n_attn else 0
        self.G = n_heads // n_kv_heads if n_attn else 0
        self.n_heads = self.n_kv * self.G
        self.qh = head_dim * (2 if gated else 1)
        self.lw = 2 * dn_nk * dn_dk + 2 * dn_nv * dn_dv + 2 * dn_nv
        self.vdim = dn_nv * dn_dv
        self.nrows = 0
        self._seqs = []

    # -- errors
    def check(self, rc):
        if rc:
            raise RqCudaError(rc, self.L.rq_cuda_error(self.h).decode())

    def close(self):
        if self.h:
            for s in list(self._seqs):
                s.free()
            self.L.rq_cuda_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        self.check(self.L.rq_cuda_sync(self.h))

    def reserve(self, rows, positions_total, max_ctx):
        """Size the scratch for passes of up to `rows` rows over `positions_total` cached positions (no allocation later)."""
        self.check(self.L.rq_cuda_reserve(self.h, rows, positions_total, max_ctx))

    def pass_timing(self, on=True):
        self.check(self.L.rq_cuda_pass_timing(self.h, int(on)))

    def pass_time(self):
        """(device seconds, rows, S1, S2) of the last closed pass (pass_timing on)."""
        t = _lib.RqCudaPassTime()
        self.check(self.L.rq_cuda_pass_time(self.h, C.byref(t)))
        return t.seconds, t.rows, t.pos_first, t.pos_more

    def pass_cost_measure(self, seq, L, reps=3):
        """(t_w, att, att_x) of the reference's pass-cost model for the attention path on this device."""
        tw, att, attx = C.c_double(), C.c_double(), C.c_double()
        self.check(self.L.rq_cuda_pass_cost_measure(self.h, seq.h, L, reps, C.byref(tw), C.byref(att), C.byref(attx)))
        return tw.value, att.value, attx.value

    def set_wo_quant(self, gs, xq_dev, xs_dev):
        """Attention calls also write int8 levels + scales of their output rows (None, None: off)."""
        self.check(self.L.rq_cuda_set_wo_quant(self.h, gs, _ptr(xq_dev), _ptr(xs_dev)))

    def set_exact(self, exact=True):
        """Quantised caches: the bit-exact CUDA-core kernels (True) or the tensor-core ones (False, the default)."""
        self.check(self.L.rq_cuda_set_exact(self.h, int(exact)))

    def set_prefill_split(self, positions=0):
        """Key positions per split of the tensor-core prefill kernels (0: chosen per pass)."""
        self.check(self.L.rq_cuda_set_prefill_split(self.h, int(positions)))

    def set_stream(self, stream_ptr):
        self.check(self.L.rq_cuda_set_stream(self.h, C.c_void_p(stream_ptr)))

    def new_seq(self, capacity, kv_type=KV_F16):
        return Sequence(self, capacity, kv_type)

    # -- a pass
    def pass_begin(self, segments):
        """segments: iterable of (Sequence, pos0, n)."""
        segs = list(segments)
        arr = (RqCudaSegment * len(segs))()
        for i, (s, pos0, n) in enumerate(segs):
            arr[i].seq, arr[i].pos0, arr[i].n = s.h, pos0, n
        self.check(self.L.rq_cuda_pass_begin(self.h, arr, len(segs)))
        self.nrows = sum(n for _, _, n in segs)

    def pass_checkpoint(self, seg, row, slot):
        """The open pass copies the DeltaNet state after row `row` of segment `seg` into that sequence's slot `slot`."""
        self.check(self.L.rq_cuda_pass_checkpoint(self.h, seg, row, slot))

    def pass_end(self, commit=True):
        self.check(self.L.rq_cuda_pass_end(self.h, int(commit)))

    def kv_store(self, layer, k, v):
        k = None if k is None else np.ascontiguousarray(k, np.float32)
        v = None if v is None else np.ascontiguousarray(v, np.float32)
        for a in (k, v):
            if a is not None and a.size != self.nrows * self.n_kv * self.hd:
                raise ValueError("K / V rows must be [rows][kv_heads][head_dim]")
        self.check(self.L.rq_cuda_kv_store(self.h, layer, _ptr(k), _ptr(v)))

    def qk_norm_rope_store_dev(self, layer, q_dev, k_dev, v_dev, qw_dev, kw_dev, rope_dim, rope_theta=1e6):
        self.check(self.L.rq_cuda_qk_norm_rope_store_dev(self.h, layer, _ptr(q_dev), _ptr(k_dev), _ptr(v_dev), _ptr(qw_dev), _ptr(kw_dev),
                                                        rope_dim, C.c_float(rope_theta)))

    def _attn(self, fn, layer, q):
        q = np.ascontiguousarray(q, np.float32)
        if q.size != self.nrows * self.n_heads * self.qh:
            raise ValueError("q rows must be [rows][heads][qh]")
        out = np.empty((self.nrows, self.n_heads, self.hd), np.float32)
        self.check(fn(self.h, layer, _ptr(q), _ptr(out)))
        return out

    def attn_decode(self, layer, q):
        return self._attn(self.L.rq_cuda_attn_decode, layer, q)

    def attn_prefill(self, layer, q):
        return self._attn(self.L.rq_cuda_attn_prefill, layer, q)

    def attn_decode_dev(self, layer, q_dev, out_dev):
        self.check(self.L.rq_cuda_attn_decode_dev(self.h, layer, _ptr(q_dev), _ptr(out_dev)))

    def peer_export(self, rows):
        """This rank's row buffer for the fused gather of head-sharded contexts: the 64 bytes of its IPC handle."""
        h = (C.c_ubyte * 64)()
        self.check(self.L.rq_cuda_peer_export(self.h, rows, C.cast(h, C.c_void_p)))
        return bytes(h)

    def peer_import(self, rank, handles):
        """handles: the ranks' 64-byte handles in rank order."""
        buf = b"".join(handles)
        self.check(self.L.rq_cuda_peer_import(self.h, rank, len(handles), C.cast(C.c_char_p(buf), C.c_void_p)))

    def attn_decode_gather_dev(self, layer, q_dev):
        """Decode attention of this rank's heads, stored into every rank's full-width row buffer by the merge kernel; returns the
        device address of this rank's buffer of the step ([rows][n_heads][head_dim], all heads)."""
        out = C.c_void_p()
        self.check(self.L.rq_cuda_attn_decode_gather_dev(self.h, layer, _ptr(q_dev), C.byref(out)))
        return out.value

    def attn_prefill_dev(self, layer, q_dev, out_dev):
        self.check(self.L.rq_cuda_attn_prefill_dev(self.h, layer, _ptr(q_dev), _ptr(out_dev)))

    def dn_rec(self, lin_layer, rows):
        rows = np.ascontiguousarray(rows, np.float32)
        if rows.size != self.nrows * self.lw:
            raise ValueError("DeltaNet rows must be [rows][lw]")
        out = np.empty((self.nrows, self.vdim), np.float32)
        self.check(self.L.rq_cuda_dn_rec(self.h, lin_layer, _ptr(rows), _ptr(out)))
        return out

    def dn_chunk(self, lin_layer, rows):
        """The recurrence in its chunked tensor-core form (prompt chunks): same rows, output and state as dn_rec."""
        rows = np.ascontiguousarray(rows, np.float32)
        if rows.size != self.nrows * self.lw:
            raise ValueError("DeltaNet rows must be [rows][lw]")
        out = np.empty((self.nrows, self.vdim), np.float32)
        self.check(self.L.rq_cuda_dn_chunk(self.h, lin_layer, _ptr(rows), _ptr(out)))
        return out

    def dn_chunk_dev(self, lin_layer, rows_dev, out_dev):
        self.check(self.L.rq_cuda_dn_chunk_dev(self.h, lin_layer, _ptr(rows_dev), _ptr(out_dev)))

    def dn_set_weights(self, lin_layer, conv, a, dt, norm):
        arrs = [np.ascontiguousarray(x, np.float32) for x in (conv, a, dt, norm)]
        self.check(self.L.rq_cuda_dn_set_weights(self.h, lin_layer, *[_ptr(x) for x in arrs]))

    def dn_prep_dev(self, lin_layer, rows_dev):
        self.check(self.L.rq_cuda_dn_prep_dev(self.h, lin_layer, _ptr(rows_dev)))

    def dn_out_dev(self, lin_layer, rows_dev, out_dev):
        self.check(self.L.rq_cuda_dn_out_dev(self.h, lin_layer, _ptr(rows_dev), _ptr(out_dev)))

    def dn_rec_dev(self, lin_layer, rows_dev, out_dev):
        self.check(self.L.rq_cuda_dn_rec_dev(self.h, lin_layer, _ptr(rows_dev), _ptr(out_dev)))

    # -- convenience: one whole pass
    def attention(self, layer, segments, q, k=None, v=None, prefill=False, commit=True):
        """Store k / v rows (when given) and attend, for one layer, as one pass."""
        self.pass_begin(segments)
        try:
            if k is not None or v is not None:
                self.kv_store(layer, k, v)
            return (self.attn_prefill if prefill else self.attn_decode)(layer, q)
        finally:
            self.pass_end(commit)

    # -- device memory and timing
    def malloc(self, nbytes):
        p = C.c_void_p()
        self.check(self.L.rq_cuda_malloc(self.h, nbytes, C.byref(p)))
        return p.value

    def mfree(self, p):
        self.check(self.L.rq_cuda_mfree(self.h, C.c_void_p(p)))

    def pinned(self, shape, dtype=np.float32):
        """A numpy array over page-locked host memory (kept alive by the context)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        self.check(self.L.rq_cuda_malloc_host(self.h, max(n, 1), C.byref(p)))
        buf = (C.c_char * n).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype).reshape(shape)

    def h2d(self, dev, host):
        self.check(self.L.rq_cuda_memcpy_h2d(self.h, C.c_void_p(dev), _ptr(host), host.nbytes))

    def d2h(self, host, dev):
        self.check(self.L.rq_cuda_memcpy_d2h(self.h, _ptr(host), C.c_void_p(dev), host.nbytes))

    def to_device(self, host):
        host = np.ascontiguousarray(host)
        p = self.malloc(host.nbytes)
        self.h2d(p, host)
        self.sync()
        return p

    def mem_info(self):
        f, t = C.c_size_t(), C.c_size_t()
        self.check(self.L.rq_cuda_mem_info(self.h, C.byref(f), C.byref(t)))
        return f.value, t.value

    def timer_start(self):
        self.check(self.L.rq_cuda_timer_start(self.h))

    def timer_stop(self):
        ms = C.c_float()
        self.check(self.L.rq_cuda_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def launch_count(self):
        return self.L.rq_cuda_launch_count(self.h)

    def profile_begin(self, max_launches):
        self.check(self.L.rq_cuda_profile_begin(self.h, max_launches))

    def profile_end(self):
        ms, n = C.c_float(), C.c_int()
        self.check(self.L.rq_cuda_profile_end(self.h, C.byref(ms), C.byref(n)))
        return ms.value, n.value


class Sequence:
    """A sequence's device-resident KV cache and DeltaNet state."""

    def __init__(self, ctx, capacity, kv_type):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(ctx.L.rq_cuda_seq_new(ctx.h, capacity, kv_type, C.byref(h)))
        self.h = h
        self.kv_type = kv_type
        ctx._seqs.append(self)

    def free(self):
        if self.h:
            self.ctx.L.rq_cuda_seq_free(self.h)
            self.h = None
            if self in self.ctx._seqs:
                self.ctx._seqs.remove(self)

    @property
    def len(self):
        return self.ctx.L.rq_cuda_seq_len(self.h)

    @property
    def capacity(self):
        return self.ctx.L.rq_cuda_seq_capacity(self.h)

    def truncate(self, n):
        self.ctx.check(self.ctx.L.rq_cuda_seq_truncate(self.h, n))

    def copy_from(self, src, n):
        self.ctx.check(self.ctx.L.rq_cuda_seq_copy(self.h, src.h, n))

    def fill_synthetic(self, n, seed):
        self.ctx.check(self.ctx.L.rq_cuda_seq_fill_synthetic(self.h, n, seed))

    def layer_bytes(self, is_v):
        return self.ctx.L.rq_cuda_seq_layer_bytes(self.h, int(is_v))

    def read_kv(self, layer, is_v, nbytes=None):
        n = self.layer_bytes(is_v) if nbytes is None else nbytes
        buf = np.empty(n, np.uint8)
        self.ctx.check(self.ctx.L.rq_cuda_seq_read_kv(self.h, layer, int(is_v), _ptr(buf), n))
        return buf

    def write_kv(self, layer, is_v, buf, new_len):
        buf = np.ascontiguousarray(buf, np.uint8)
        self.ctx.check(self.ctx.L.rq_cuda_seq_write_kv(self.h, layer, int(is_v), _ptr(buf), buf.nbytes, new_len))

    def save(self, path, tokens, model_fp=0, rng=0):
        """Write the sequence in the reference's saved-sequence format (tokens: its len token ids)."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        assert tokens.size >= self.len
        self.ctx.check(self.ctx.L.rq_cuda_seq_save(self.h, str(path).encode(), _ptr(tokens), model_fp, rng))

    def load(self, path, n, model_fp=0):
        """Load the first n positions of a saved sequence; returns (tokens kept, rng)."""
        tokens = np.zeros(max(n, 1), np.int32)
        rng = C.c_ulonglong()
        self.ctx.check(self.ctx.L.rq_cuda_seq_load(self.h, str(path).encode(), model_fp, n, _ptr(tokens), C.byref(rng)))
        return tokens[:self.len], rng.value

    def set_checkpoints(self, n):
        self.ctx.check(self.ctx.L.rq_cuda_seq_set_checkpoints(self.h, n))

    def checkpoint_pos(self, slot):
        return self.ctx.L.rq_cuda_seq_checkpoint_pos(self.h, slot)

    def restore(self, slot):
        self.ctx.check(self.ctx.L.rq_cuda_seq_restore(self.h, slot))

    def read_checkpoint(self, slot, lin_layer):
        buf = np.empty(self.state_floats(), np.float32)
        self.ctx.check(self.ctx.L.rq_cuda_seq_read_checkpoint(self.h, slot, lin_layer, _ptr(buf)))
        return buf

    def state_floats(self):
        return self.ctx.L.rq_cuda_seq_state_floats(self.h)

    def read_state(self, lin_layer):
        buf = np.empty(self.state_floats(), np.float32)
        self.ctx.check(self.ctx.L.rq_cuda_seq_read_state(self.h, lin_layer, _ptr(buf)))
        return buf

    def write_state(self, lin_layer, st):
        st = np.ascontiguousarray(st, np.float32)
        assert st.size == self.state_floats()
        self.ctx.check(self.ctx.L.rq_cuda_seq_write_state(self.h, lin_layer, _ptr(st)))
