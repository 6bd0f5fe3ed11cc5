"""Decode attention against the CPU checker at the benchmark's context lengths, bit for bit.

The merge kernel (attn_combine_kernel; att_combine, reference src/forward.c:1405-1431) walks a row's block partials in
chunks of 8192 / head_dim = 64 and carries its two fused-multiply-add chains from one chunk to the next.  Contexts
up to 16,384 positions fit one chunk; the headline batch has rows of up to 32,768 positions (128 partials, two chunks)
and the quantised-cache configuration 40,960 (160 partials, three chunks).  These cases put the first context past
one chunk, the largest of the ragged batch, and the quantised configuration's context next to the checker, at the
Qwen3-8B head shape (32 query heads, 8 KV heads, head_dim 128), one layer, device-filled caches read back for the CPU.
"""
import numpy as np
import pytest

from tests.helpers import assert_close, bit_equal

pytestmark = pytest.mark.gpu

F16, Q8, Q4, Q4K4 = 2, 3, 8, 9


@pytest.mark.parametrize("kvt,ctxs", [(F16, [16385, 32768, 16384]), (Q8, [40960]), (Q4, [20481]), (Q4K4, [24577, 999])],
                         ids=["f16-16385-32768", "q8-40960", "q4-20481", "q4k4-24577"])
def test_long_context_rows_equal_cpu(checker, kvt, ctxs):
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 32, 8, 128
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, max_rows=8)
    c.set_exact(True)  # (quantised caches: the kernels that give the CPU code's bits; the tensor-core ones are checked below)
    seqs = []
    for i, n in enumerate(ctxs):
        s = c.new_seq(n, kvt)
        s.fill_synthetic(n, 7000 + 13 * kvt + i)
        seqs.append(s)
    q = synth.normal(300 + kvt, (len(ctxs), n_heads, hd))
    c.pass_begin([(s, n - 1, 1) for s, n in zip(seqs, ctxs)])
    got = c.attn_decode(0, q)
    c.pass_end(commit=False)
    assert np.isfinite(got).all()
    for i, (s, n) in enumerate(zip(seqs, ctxs)):
        want = checker.attention(kvt, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[i:i + 1], np.array([n], np.int32), split=1)
        assert_close(got[i:i + 1], want, f"kvt={kvt} ctx={n}")
        assert bit_equal(got[i:i + 1], want), f"kvt={kvt} ctx={n}: the merge over {(n + 255) // 256} partials differs from the CPU code"
        # the row alone (its own pass) gives the same bits as in the batch
        c.pass_begin([(s, n - 1, 1)])
        alone = c.attn_decode(0, q[i:i + 1])
        c.pass_end(commit=False)
        assert bit_equal(alone, got[i:i + 1])
    if kvt != F16:
        # the tensor-core path over quantised caches: the same rows inside the acceptance bar
        c.set_exact(False)
        c.pass_begin([(s, n - 1, 1) for s, n in zip(seqs, ctxs)])
        fast = c.attn_decode(0, q)
        c.pass_end(commit=False)
        assert_close(fast, got, f"tensor-core decode kvt={kvt} at {ctxs}")
    c.close()
