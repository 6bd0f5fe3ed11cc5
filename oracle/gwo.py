"""ctypes binding of the two CPU checkers (test infrastructure; never imported by the product package).

`load("port")` gives this repository's plain-C restatement (oracle/liboracle.so, built from gw_oracle.c);
`load("ref")` gives the reference's own C code behind the same `gwo_*` ABI: the widest build under oracle/_ref
that the host CPU can run (libgwref.so: the build host's -march=native; libgwref_v4.so: x86-64-v4, the AVX-512
attention kernels on any AVX-512 host; libgwref_generic.so: the portable `-DRUNQ_GENERIC` kernels).
Both are numpy-in / numpy-out.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
F32, F16, Q8, Q4, Q4K4 = 0, 2, 3, 8, 9
KV_NAMES = {"f32": F32, "f16": F16, "q8": Q8, "q4": Q4, "q4k4": Q4K4}
T, P = 16, 256

_vp, _i, _sz, _f, _d = C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_double


def _host_flags():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


# /proc/cpuinfo flags a build at each ISA level may use (the x86-64 psABI levels)
_V3 = {"avx", "avx2", "bmi1", "bmi2", "f16c", "fma", "abm", "movbe", "xsave"}
_V4 = _V3 | {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"}


def ref_variants():
    """The reference builds under oracle/_ref, widest ISA first: (path, the host flags it needs)."""
    d = os.path.join(HERE, "_ref")
    try:
        native = set(open(os.path.join(d, "cpuflags.txt")).read().split())  # everything the build host had
    except OSError:
        native = None
    out = []
    if native is not None:
        out.append((os.path.join(d, "libgwref.so"), native))
    out.append((os.path.join(d, "libgwref_v4.so"), _V4))
    out.append((os.path.join(d, "libgwref_generic.so"), _V3))
    return [(p, f) for p, f in out if os.path.exists(p)]


def build_port():
    subprocess.check_call(["make", "-s", "-C", HERE, "liboracle.so"])


def ref_path():
    """Path of the widest reference build this host can run (native build, then the AVX-512 baseline x86-64-v4, then
    the portable -DRUNQ_GENERIC one), or None."""
    have = _host_flags()
    for path, need in ref_variants():
        if need <= have:
            return path
    return None


class Oracle:
    def __init__(self, path):
        self.path = path
        L = self.L = C.CDLL(path)
        L.gwo_kind.restype = _i
        L.gwo_isa.restype = _i
        L.gwo_threads_init.restype = _i
        L.gwo_threads_init.argtypes = [_i]
        L.gwo_kv_tile_bytes.restype = _sz
        L.gwo_kv_tile_bytes.argtypes = [_i, _i, _i]
        L.gwo_kv_layer_bytes.restype = _sz
        L.gwo_kv_layer_bytes.argtypes = [_i, _i, _i, _i, _i]
        for n in ("gwo_f32_f16", "gwo_f16_f32", "gwo_exp_att", "gwo_sigmoid"):
            getattr(L, n).argtypes = [_vp, _vp, _sz]
            getattr(L, n).restype = None
        L.gwo_qk_norm_rope.argtypes = [_vp, _i, _i, _vp, _i, _i, _i, _f]
        L.gwo_qk_norm_rope.restype = None
        L.gwo_kv_store.argtypes = [_i, _vp, _vp, _i, _i, _i, _vp, _vp]
        L.gwo_kv_store.restype = None
        L.gwo_kv_block_f32.argtypes = [_i, _vp, _vp, _i, _i, _vp, _vp]
        L.gwo_kv_block_f32.restype = None
        L.gwo_kv_block_f32_simd.argtypes = [_i, _vp, _vp, _i, _i, _vp, _vp]
        L.gwo_kv_block_f32_simd.restype = _i
        L.gwo_q_rot.argtypes = [_i, _vp, _i, _i, _i]
        L.gwo_q_rot.restype = None
        L.gwo_o_unrot.argtypes = [_i, _vp, _i, _i, _i]
        L.gwo_o_unrot.restype = None
        L.gwo_attention.argtypes = [_i, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _f, _i, _i]
        L.gwo_attention.restype = _i
        L.gwo_bench_decode.argtypes = [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _f, _i, _vp]
        L.gwo_bench_decode.restype = _d
        L.gwo_bench_prefill.argtypes = [_i, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _f, _i, _vp]
        L.gwo_bench_prefill.restype = _d
        L.gwo_dn_new.argtypes = [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]
        L.gwo_dn_new.restype = _vp
        L.gwo_dn_free.argtypes = [_vp]
        L.gwo_dn_free.restype = None
        L.gwo_dn_state_floats.argtypes = [_vp]
        L.gwo_dn_state_floats.restype = _sz
        L.gwo_dn_conv_floats.argtypes = [_vp]
        L.gwo_dn_conv_floats.restype = _sz
        L.gwo_dn_row_floats.argtypes = [_vp]
        L.gwo_dn_row_floats.restype = _i
        L.gwo_dn_rec.argtypes = [_vp, _vp, _i, _vp, _sz, _vp, _sz, _i]
        L.gwo_dn_rec.restype = None
        L.gwo_dn_prep.argtypes = [_vp, _vp, _i, _vp, _sz, _i]
        L.gwo_dn_prep.restype = None
        L.gwo_dn_out.argtypes = [_vp, _vp, _sz, _vp, _sz, _i]
        L.gwo_dn_out.restype = None
        L.gwo_bench_dn.argtypes = [_vp, _i, _vp, _vp, _sz, _vp, _sz, _i, _i, _vp]
        L.gwo_bench_dn.restype = _d
        L.gwo_quantize.argtypes = [_vp, _i, _i, _vp, _vp]
        L.gwo_quantize.restype = None
        self.kind = "ref" if L.gwo_kind() == 1 else "port"
        isa = L.gwo_isa()
        # which attention kernels the library was compiled with (gwo_isa bit 0: the reference's AVX-512 kernels,
        # RUNQ_ATT512; bit 1: hardware fused multiply-add)
        self.isa = ("avx512 attention kernels (RUNQ_ATT512)" if isa & 1 else "portable C kernels") + (", fma" if isa & 2 else "")
        self.library = os.path.relpath(path, os.path.dirname(HERE))

    # ---- helpers
    @staticmethod
    def _p(a):
        return a.ctypes.data_as(_vp) if a is not None else None

    def threads(self, n=0):
        return self.L.gwo_threads_init(n)

    def tile_bytes(self, kvt, hd, is_v):
        return self.L.gwo_kv_tile_bytes(kvt, hd, is_v)

    def layer_bytes(self, kvt, kv_len, n_kv, hd, is_v):
        return self.L.gwo_kv_layer_bytes(kvt, kv_len, n_kv, hd, is_v)

    def f32_f16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        h = np.empty(x.shape, np.uint16)
        self.L.gwo_f32_f16(self._p(x), self._p(h), x.size)
        return h

    def f16_f32(self, h):
        h = np.ascontiguousarray(h, np.uint16)
        x = np.empty(h.shape, np.float32)
        self.L.gwo_f16_f32(self._p(h), self._p(x), h.size)
        return x

    def exp_att(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.L.gwo_exp_att(self._p(x), self._p(y), x.size)
        return y

    def sigmoid(self, x):
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        self.L.gwo_sigmoid(self._p(x), self._p(y), x.size)
        return y

    def quantize(self, x, gs):
        """The activation quantiser in front of the `wo` matmul: x [..., n] -> (int8 levels, fp32 scales per gs values)."""
        x = np.ascontiguousarray(x, np.float32)
        q = np.empty(x.shape, np.int8)
        s = np.empty(x.size // gs, np.float32)
        self.L.gwo_quantize(self._p(x), x.size, gs, self._p(q), self._p(s))
        return q, s

    def qk_norm_rope(self, rows, norm_w, hd, positions, theta=1e6, rd=None, gated=False):
        """rows [n][heads][hd (or 2 hd when gated)] -> normed + rotated copy (the gate half untouched)."""
        rows = np.array(rows, np.float32, order="C")
        n, nh, st = rows.shape
        w = np.ascontiguousarray(norm_w, np.float32)
        lt = np.float32(np.log(np.float64(theta)))
        for r in range(n):
            self.L.gwo_qk_norm_rope(rows[r].ctypes.data_as(_vp), nh, st, self._p(w), hd, rd or hd, int(positions[r]), lt)
        return rows

    def new_cache(self, kvt, kv_len, n_kv, hd):
        """Zeroed K and V byte buffers of one layer (kv_len a multiple of 256)."""
        assert kv_len % P == 0
        return (np.zeros(self.layer_bytes(kvt, kv_len, n_kv, hd, 0), np.uint8),
                np.zeros(self.layer_bytes(kvt, kv_len, n_kv, hd, 1), np.uint8))

    def kv_store(self, kvt, kl, vl, pos0, k, v, n_kv, hd):
        """Rows k, v: [n][n_kv][hd] f32 stored at positions pos0..pos0+n-1 (either may be None)."""
        k = None if k is None else np.ascontiguousarray(k, np.float32).reshape(-1, n_kv * hd)
        v = None if v is None else np.ascontiguousarray(v, np.float32).reshape(-1, n_kv * hd)
        n = (k if k is not None else v).shape[0]
        for r in range(n):
            self.L.gwo_kv_store(kvt, self._p(kl), self._p(vl), pos0 + r, n_kv, hd,
                                None if k is None else k[r].ctypes.data_as(_vp),
                                None if v is None else v[r].ctypes.data_as(_vp))

    def block_f32(self, kvt, kl, vl, n_kv, hd, g, b, ntl=16, simd=False):
        """The first ntl tiles of (kv head g, block b) as fp32 tiles: K [ntl][hd][16], V [ntl][16][hd]."""
        tk, tv = self.tile_bytes(kvt, hd, 0), self.tile_bytes(kvt, hd, 1)
        t0 = (b * n_kv + g) * 16
        kf = np.empty((ntl, hd, 16), np.float32)
        vf = np.empty((ntl, 16, hd), np.float32)
        kb, vb = kl[t0 * tk:], vl[t0 * tv:]
        if simd:
            rc = self.L.gwo_kv_block_f32_simd(kvt, self._p(kb), self._p(vb), ntl, hd, self._p(kf), self._p(vf))
            if rc:
                return None, None
        else:
            self.L.gwo_kv_block_f32(kvt, self._p(kb), self._p(vb), ntl, hd, self._p(kf), self._p(vf))
        return kf, vf

    def q_rot(self, kvt, q, hd):
        q = np.array(q, np.float32, order="C")
        self.L.gwo_q_rot(kvt, self._p(q), q.size // hd, hd, hd)
        return q

    def o_unrot(self, kvt, o, hd):
        o = np.array(o, np.float32, order="C")
        self.L.gwo_o_unrot(kvt, self._p(o), o.size // hd, hd, hd)
        return o

    def attention(self, kvt, kl, vl, n_kv, n_heads, hd, q, np_rows, scale=None, gated=False, split=0, rows_per_item=0):
        """q: [nrows][n_heads][qh] (qh = 2 hd when gated); np_rows[r] = positions row r attends. -> [nrows][n_heads][hd]"""
        qh = 2 * hd if gated else hd
        q = np.ascontiguousarray(q, np.float32).reshape(-1, n_heads, qh)
        npr = np.ascontiguousarray(np_rows, np.int32)
        assert npr.shape[0] == q.shape[0]
        out = np.zeros((q.shape[0], n_heads, hd), np.float32)
        scale = float(1.0 / np.sqrt(np.float32(hd))) if scale is None else scale
        rc = self.L.gwo_attention(kvt, self._p(kl), self._p(vl), n_kv, n_heads, hd, int(gated), q.shape[0], self._p(q),
                                  self._p(npr), self._p(out), np.float32(scale), split, rows_per_item)
        if rc:
            raise ValueError("gwo_attention refused the arguments")
        return out

    def bench_decode(self, kvt, n_kv, n_heads, hd, caches, ctx, q, scale, reps):
        """caches: list of (kl, vl) per sequence; q [nseq][n_heads][hd] (rotated already for q8 / q4).
        -> (seconds total, best single pass, out)"""
        nseq = len(caches)
        kls = (_vp * nseq)(*[self._p(c[0]) for c in caches])
        vls = (_vp * nseq)(*[self._p(c[1]) for c in caches])
        ctx = np.ascontiguousarray(ctx, np.int32)
        q = np.ascontiguousarray(q, np.float32)
        out = np.zeros((nseq, n_heads, hd), np.float32)
        best = _d(0)
        tot = self.L.gwo_bench_decode(kvt, n_kv, n_heads, hd, nseq, kls, vls, self._p(ctx), self._p(q), self._p(out),
                                      np.float32(scale), reps, C.byref(best))
        return tot, best.value, out

    def bench_prefill(self, kvt, kl, vl, n_kv, n_heads, hd, q, np_rows, scale, reps):
        q = np.ascontiguousarray(q, np.float32)
        npr = np.ascontiguousarray(np_rows, np.int32)
        out = np.zeros((npr.shape[0], n_heads, hd), np.float32)
        best = _d(0)
        tot = self.L.gwo_bench_prefill(kvt, self._p(kl), self._p(vl), n_kv, n_heads, hd, npr.shape[0], self._p(q),
                                       self._p(npr), self._p(out), np.float32(scale), reps, C.byref(best))
        return tot, best.value, out


class DeltaNet:
    """One Gated DeltaNet layer's shapes (and optional weights) on an Oracle."""

    def __init__(self, orc, nk, nv, dk, dv, conv=4, w_conv=None, w_a=None, w_dt=None, w_norm=None):
        self.o, self.nk, self.nv, self.dk, self.dv, self.conv = orc, nk, nv, dk, dv, conv
        self._keep = [None if w is None else np.ascontiguousarray(w, np.float32) for w in (w_conv, w_a, w_dt, w_norm)]
        self.h = orc.L.gwo_dn_new(nk, nv, dk, dv, conv, *[Oracle._p(w) for w in self._keep])
        self.state_floats = orc.L.gwo_dn_state_floats(self.h)
        self.conv_floats = orc.L.gwo_dn_conv_floats(self.h)
        self.lw = orc.L.gwo_dn_row_floats(self.h)
        self.conv_dim = 2 * nk * dk + nv * dv
        self.vdim = nv * dv

    def __del__(self):
        try:
            self.o.L.gwo_dn_free(self.h)
        except Exception:
            pass

    def new_state(self):
        return np.zeros(self.state_floats, np.float32)

    def rec(self, state, rows, first):
        """rows [n][lw] (post-prep) -> out [n][nv*dv]; state updated in place."""
        rows = np.ascontiguousarray(rows, np.float32)
        n = rows.shape[0]
        out = np.zeros((n, self.nv * self.dv), np.float32)
        self.o.L.gwo_dn_rec(self.h, Oracle._p(state), int(first), Oracle._p(rows), rows.shape[1], Oracle._p(out),
                            out.shape[1], n)
        return out

    def prep(self, state, rows, first):
        """rows [n][lw] raw projections -> prepared copy; conv state updated in place."""
        rows = np.array(rows, np.float32, order="C")
        self.o.L.gwo_dn_prep(self.h, Oracle._p(state), int(first), Oracle._p(rows), rows.shape[1], rows.shape[0])
        return rows

    def out(self, rows, o):
        rows = np.ascontiguousarray(rows, np.float32)
        o = np.array(o, np.float32, order="C")
        self.o.L.gwo_dn_out(self.h, Oracle._p(rows), rows.shape[1], Oracle._p(o), o.shape[1], rows.shape[0])
        return o


class RefSeq:
    """A host sequence of the reference (rq_seq_new) for the saved-sequence tests: the reference's own rq_seq_save /
    rq_seq_load behind it.  Only on the reference builds (the restatement has no file code)."""

    def __init__(self, orc, kvt, n_attn, n_kv, hd, cap, fp=0, n_lin=0, nk=0, nv=0, dk=128, dv=128, conv=4):
        L = self.L = orc.L
        if not hasattr(L, "gwo_seq_new"):
            raise RuntimeError("this checker has no sequence-file code")
        L.gwo_seq_new.restype = _vp
        L.gwo_seq_new.argtypes = [_i, _i, _i, _i, _i, C.c_ulonglong, _i, _i, _i, _i, _i, _i]
        L.gwo_seq_free.argtypes = [_vp]
        L.gwo_seq_cache_bytes.restype = _sz
        L.gwo_seq_cache_bytes.argtypes = [_vp, _i]
        L.gwo_seq_state_floats.restype = _sz
        L.gwo_seq_state_floats.argtypes = [_vp]
        L.gwo_seq_set.argtypes = [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp]
        L.gwo_seq_get.argtypes = [_vp, _vp, _vp, _vp, _vp, C.POINTER(_i), _vp]
        L.gwo_seq_rng.restype = C.c_ulonglong
        L.gwo_seq_rng.argtypes = [_vp, _i, C.c_ulonglong]
        L.gwo_seq_save.argtypes = [_vp, C.c_char_p]
        L.gwo_seq_load.argtypes = [_vp, C.c_char_p, _i]
        L.gwo_seq_save_bytes.restype = C.c_longlong
        L.gwo_seq_save_bytes.argtypes = [_vp]
        self.h = L.gwo_seq_new(kvt, n_attn, n_kv, hd, cap, fp, n_lin, nk, nv, dk, dv, conv)
        if not self.h:
            raise RuntimeError("rq_seq_new refused the shape")
        self.cap = cap
        self.kbytes, self.vbytes = L.gwo_seq_cache_bytes(self.h, 0), L.gwo_seq_cache_bytes(self.h, 1)
        self.state_floats = L.gwo_seq_state_floats(self.h)

    def __del__(self):
        try:
            self.L.gwo_seq_free(self.h)
        except Exception:
            pass

    def set(self, tokens, k, v, ssm=None, ck_pos=-1, ck=None, rng=0):
        """tokens [len]; k, v: all layers' cache bytes; ssm: the layered state; (ck_pos, ck): a checkpoint in slot 0."""
        tokens = np.ascontiguousarray(tokens, np.int32)
        k, v = np.ascontiguousarray(k, np.uint8), np.ascontiguousarray(v, np.uint8)
        assert k.size == self.kbytes and v.size == self.vbytes
        ssm = None if ssm is None else np.ascontiguousarray(ssm, np.float32)
        ck = None if ck is None else np.ascontiguousarray(ck, np.float32)
        rc = self.L.gwo_seq_set(self.h, tokens.size, Oracle._p(tokens), Oracle._p(k), Oracle._p(v), Oracle._p(ssm), ck_pos, Oracle._p(ck))
        assert rc == 0
        self.L.gwo_seq_rng(self.h, 1, rng)

    def get(self):
        """-> (tokens, k bytes, v bytes, state, checkpoint length or -1, checkpoint state, rng)"""
        tokens = np.zeros(self.cap, np.int32)
        k, v = np.zeros(self.kbytes, np.uint8), np.zeros(self.vbytes, np.uint8)
        ssm, ck = np.zeros(max(self.state_floats, 1), np.float32), np.zeros(max(self.state_floats, 1), np.float32)
        pos = _i(-1)
        n = self.L.gwo_seq_get(self.h, Oracle._p(tokens), Oracle._p(k), Oracle._p(v), Oracle._p(ssm), C.byref(pos), Oracle._p(ck))
        return tokens[:n], k, v, ssm[:self.state_floats], pos.value, ck[:self.state_floats], self.L.gwo_seq_rng(self.h, 0, 0)

    def save(self, path):
        return self.L.gwo_seq_save(self.h, str(path).encode())

    def load(self, path, n):
        return self.L.gwo_seq_load(self.h, str(path).encode(), n)

    def save_bytes(self):
        return self.L.gwo_seq_save_bytes(self.h)


_cache = {}


def load(which="port"):
    """which: 'port' (the restatement; built on demand), 'ref' (the reference's code, the widest build the host can run;
    None when absent), 'ref-v4' (its AVX-512 baseline build) and 'ref-generic' (its portable build): None when absent or
    not runnable on this host."""
    if which in _cache:
        return _cache[which]
    if which == "port":
        path = os.path.join(HERE, "liboracle.so")
        src = os.path.join(HERE, "gw_oracle.c")
        if not os.path.exists(path) or (os.path.exists(src) and os.path.getmtime(src) > os.path.getmtime(path)):
            build_port()
    elif which == "ref":
        path = ref_path()
    elif which in ("ref-generic", "ref-v4"):
        path = os.path.join(HERE, "_ref", "libgwref_generic.so" if which == "ref-generic" else "libgwref_v4.so")
        need = _V3 if which == "ref-generic" else _V4
        path = path if os.path.exists(path) and need <= _host_flags() else None
    else:
        raise ValueError(which)
    _cache[which] = Oracle(path) if path else None
    return _cache[which]


def best():
    """The strongest checker available: the reference's own code when its build is present, else the restatement."""
    return load("ref") or load("port")
