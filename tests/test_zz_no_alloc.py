"""rq_cuda_attn_decode_noalloc: the decode attention for hosts that cannot allocate device memory during a pass
(a server that handed all its memory out at start-up; code that runs where cudaMalloc would stall the device).

Called straight through the C ABI with caller-owned device buffers, twice in a row, and compared with the regular
entry point rq_cuda_attn_decode_dev: the same kernels on a different scratch buffer must give the same bits.  The
file name sorts last so a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from tests.helpers import assert_close, bit_equal

pytestmark = pytest.mark.gpu


def test_noalloc_entry_matches_regular_entry():
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 8, 2, 128
    ctxs = [700, 33, 1500]
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, max_rows=8)
    L = c.L
    seqs = []
    for i, n in enumerate(ctxs):
        s = c.new_seq(n, g.KV_F16)
        s.fill_synthetic(n, 50 + i)
        seqs.append(s)
    nfl = len(ctxs) * n_heads * hd
    q_dev, out_a, out_b = c.malloc(nfl * 4), c.malloc(nfl * 4), c.malloc(nfl * 4)
    c.pass_begin([(s, n - 1, 1) for s, n in zip(seqs, ctxs)])
    try:
        for call in range(2):
            q = synth.normal(900 + call, (len(ctxs), n_heads, hd))
            c.h2d(q_dev, q)
            c.check(L.rq_cuda_attn_decode_dev(c.h, 0, C.c_void_p(q_dev), C.c_void_p(out_a)))
            free_before = c.mem_info()[0]
            c.check(L.rq_cuda_attn_decode_noalloc(c.h, 0, C.c_void_p(q_dev), C.c_void_p(out_b)))
            if call == 1:
                # the second call (kernels and the array's address are in place after the first) takes no device memory
                c.sync()
                assert c.mem_info()[0] == free_before
            a, b = np.empty((len(ctxs), n_heads, hd), np.float32), np.empty((len(ctxs), n_heads, hd), np.float32)
            c.d2h(a, out_a)
            c.d2h(b, out_b)
            c.sync()
            assert np.isfinite(a).all() and np.abs(a).max() > 0
            assert_close(b, a, f"no-alloc call {call}")
            assert bit_equal(b, a)
    finally:
        c.pass_end(commit=False)
    c.close()


def test_noalloc_entry_refuses_oversized_pass():
    import gwenedeg_b200 as g
    n_heads, n_kv, hd = 32, 8, 128
    limit = g._lib.load().rq_cuda_attn_decode_noalloc_max_bytes()
    per_block = n_heads * (hd + 16) * 4
    n = (limit // per_block + 2) * 256  # one row with more 256-position blocks than the fixed scratch holds
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, max_rows=2)
    s = c.new_seq(n, g.KV_Q4K4)
    s.fill_synthetic(n, 1)
    buf = c.malloc(n_heads * hd * 4)
    c.pass_begin([(s, n - 1, 1)])
    rc = c.L.rq_cuda_attn_decode_noalloc(c.h, 0, C.c_void_p(buf), C.c_void_p(buf))
    msg = c.L.rq_cuda_error(c.h).decode()
    c.pass_end(commit=False)
    assert rc == -1 and "fixed scratch" in msg
    c.close()
