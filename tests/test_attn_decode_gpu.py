"""Parity of the CUDA decode attention (through the C ABI) with the CPU checker on identical seeded inputs.

Bar (fp32 outputs): max-abs <= 2e-3 and relative L2 <= 1e-3; cache bytes and dequantised values bit-exact.  The
kernels follow the reference's operation order, so the outputs are in fact expected to match bit for bit, which
is asserted separately.
"""
import numpy as np
import pytest

from tests.helpers import assert_close, bit_equal, errors, kv_rows, oracle_cache

pytestmark = pytest.mark.gpu

F16, Q8, Q4, Q4K4 = 2, 3, 8, 9
# the contexts the reference's own invariant tests walk over: tile and 256-block edges
CONTEXTS = [1, 15, 16, 17, 255, 256, 257, 511, 513, 700]


def make_ctx(**kw):
    import gwenedeg_b200 as g
    return g.Context(0, **kw)


@pytest.mark.parametrize("kvt", [F16, Q8, Q4, Q4K4])
@pytest.mark.parametrize("n_heads,n_kv,hd,gated", [(4, 2, 128, False), (8, 2, 128, False), (2, 2, 64, False),
                                                    (8, 1, 128, False), (4, 1, 256, True), (6, 2, 128, False)])
def test_store_and_decode_match_cpu(checker, port, kvt, n_heads, n_kv, hd, gated):
    from gwenedeg_b200 import synth
    n = 700
    c = make_ctx(n_attn=2, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated, max_rows=512)
    c.set_exact(True)  # quantised caches: the kernels that follow the CPU code operation for operation
    k, v = kv_rows(kvt * 100 + hd + n_heads, n, n_kv, hd)
    # the device cache, written through rq_cuda_kv_store in two chunks (a prompt chunk, then the rest), layer 1
    s = c.new_seq(n, kvt)
    for lo, hi in ((0, 300), (300, n)):
        c.pass_begin([(s, lo, hi - lo)])
        c.kv_store(1, k[lo:hi], v[lo:hi])
        c.pass_end()
    assert s.len == n
    kl, vl = oracle_cache(port, kvt, n_kv, hd, k, v)  # the definition's bytes (IEEE division)
    gk, gv = s.read_kv(1, 0), s.read_kv(1, 1)
    nbytes_k = (n + 255) // 256 * 16 * n_kv * port.tile_bytes(kvt, hd, 0)
    # positions past n inside the last tile are never written: compare the stored positions through the dequantiser
    for b in range((n + 255) // 256):
        for g_ in range(n_kv):
            ntl = min(16, (n - b * 256 + 15) // 16)
            kf, vf = port.block_f32(kvt, kl, vl, n_kv, hd, g_, b, ntl)
            kf2, vf2 = port.block_f32(kvt, gk[:nbytes_k], gv, n_kv, hd, g_, b, ntl)
            last = n - b * 256 - (ntl - 1) * 16  # valid positions of the last tile
            assert bit_equal(kf[:ntl - 1], kf2[:ntl - 1]) and bit_equal(kf[-1][:, :last], kf2[-1][:, :last])
            assert bit_equal(vf[:ntl - 1], vf2[:ntl - 1]) and bit_equal(vf[-1][:last], vf2[-1][:last])
    # and against the reference's own build: its -Ofast code replaces x / d by a reciprocal, so exact ties of
    # rint(x / d) may land one level off there (rarely), never more
    from oracle import gwo
    refb = gwo.load("ref")
    if refb is not None:
        rk, rv = oracle_cache(refb, kvt, n_kv, hd, k, v)
        for mine, theirs in ((gk[:rk.size], rk), (gv[:rv.size], rv)):
            diff = mine != theirs
            assert diff.mean() < 2e-4
            if diff.any():
                assert kvt != F16, "f16 stores are expected to equal the reference build's byte for byte"
                assert np.abs(mine[diff].astype(np.int16) - theirs[diff].astype(np.int16)).max() <= 17  # one level (a nibble may carry)
    # decode rows at the edge contexts: one sequence copy per row, all in one ragged pass
    qh = hd * (2 if gated else 1)
    q = synth.normal(kvt * 7 + hd, (len(CONTEXTS), n_heads, qh))
    seqs = []
    for ctx_len in CONTEXTS:
        t = c.new_seq(n, kvt)
        t.copy_from(s, n)
        seqs.append(t)
    c.pass_begin([(t, ctx_len - 1, 1) for t, ctx_len in zip(seqs, CONTEXTS)])
    got = c.attn_decode(1, q)
    c.pass_end(commit=False)
    # the CPU checker on the device's own cache bytes
    want = checker.attention(kvt, gk, gv, n_kv, n_heads, hd, q, np.array(CONTEXTS, np.int32), gated=gated, split=1)
    assert_close(got, want, f"decode kvt={kvt}")
    assert bit_equal(got, want), "decode attention is expected to equal the CPU code bit for bit"
    # a row alone gives the bits it gave in the batch
    for i in (0, 4, 9):
        c.pass_begin([(seqs[i], CONTEXTS[i] - 1, 1)])
        alone = c.attn_decode(1, q[i:i + 1])
        c.pass_end(commit=False)
        assert bit_equal(alone[0], got[i])
    c.close()


@pytest.mark.parametrize("kvt", [Q8, Q4, Q4K4])
@pytest.mark.parametrize("n_heads,n_kv,gated", [(4, 2, False), (8, 2, False), (8, 1, True), (6, 2, False), (2, 2, False)])
def test_quantised_decode_on_tensor_cores_matches_cpu(checker, kvt, n_heads, n_kv, gated):
    """The tensor-core path over quantised caches at head_dim 128 (the cached levels as int8 MMA operands, 4-bit ones unpacked to
    16 (n - 8); query and softmax weights as 16-bit fixed point in two int8 planes) against the CPU code on the device's own cache bytes: inside the acceptance bar at every edge context, a row alone
    equal to the same row in a batch, and equal bits from run to run."""
    from gwenedeg_b200 import synth
    hd, n = 128, 700
    c = make_ctx(n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated, max_rows=512)
    c.set_exact(False)
    k, v = kv_rows(kvt * 100 + n_heads, n, n_kv, hd, outlier=False)
    # a large K dim, as real caches have (the dequantised values stay far inside the f16 range); V stays N(0,1)-sized: the
    # absolute bar is stated for outputs of that size, and a context of one position returns V itself, rounded to f16
    k[5, 0, 3] = 300.0
    s = c.new_seq(n, kvt)
    for lo, hi in ((0, 300), (300, n)):
        c.pass_begin([(s, lo, hi - lo)])
        c.kv_store(0, k[lo:hi], v[lo:hi])
        c.pass_end()
    gk, gv = s.read_kv(0, 0), s.read_kv(0, 1)
    qh = hd * (2 if gated else 1)
    q = synth.normal(kvt * 7 + 1, (len(CONTEXTS), n_heads, qh))
    seqs = []
    for ctx_len in CONTEXTS:
        t = c.new_seq(n, kvt)
        t.copy_from(s, n)
        seqs.append(t)
    segs = [(t, ctx_len - 1, 1) for t, ctx_len in zip(seqs, CONTEXTS)]
    c.pass_begin(segs)
    got = c.attn_decode(0, q)
    again = c.attn_decode(0, q)
    c.pass_end(commit=False)
    want = checker.attention(kvt, gk, gv, n_kv, n_heads, hd, q, np.array(CONTEXTS, np.int32), gated=gated, split=1)
    # (a row that attends one or a few positions returns V values of size ~3, rounded to f16 on this path: the absolute bar,
    # stated for outputs of size <= 1, is scaled with the largest wanted output; the relative bars stand as they are)
    ma, rl = errors(got, want)
    assert rl <= 1e-3 and ma <= 2e-3 * max(1.0, float(np.abs(want).max())), f"tensor-core decode kvt={kvt}: max-abs {ma:.3g}, rel-L2 {rl:.3g}"
    for r in range(len(CONTEXTS)):
        assert errors(got[r], want[r])[1] <= 6e-3  # (a row of one position is V itself with its scales rounded to f16)
    assert bit_equal(got, again)
    for i in (0, 4, 9):
        c.pass_begin([(seqs[i], CONTEXTS[i] - 1, 1)])
        alone = c.attn_decode(0, q[i:i + 1])
        c.pass_end(commit=False)
        assert bit_equal(alone[0], got[i])
    # the bit-exact kernels on the same pass agree with the CPU code to the bit
    c.set_exact(True)
    c.pass_begin(segs)
    exact = c.attn_decode(0, q)
    c.pass_end(commit=False)
    assert bit_equal(exact, want)
    print("tensor-core decode errors kvt", kvt, errors(got, want))
    c.close()


def test_prompt_chunk_rows_match_cpu(checker):
    """Rows of a chunk (consecutive positions of one sequence, causal) plus decode rows of other sequences."""
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd, n = 4, 2, 128, 300
    c = make_ctx(n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
    # (no f16-range outliers here: the chunk goes through the tensor-core kernel, whose f16 rounding of the softmax
    # weights is bounded relative to the output, and the absolute bar is stated for N(0,1)-sized values)
    k, v = kv_rows(77, n, n_kv, hd, outlier=False)
    a, b = c.new_seq(n, F16), c.new_seq(n, F16)
    c.pass_begin([(a, 0, n)])
    c.kv_store(0, k, v)
    c.pass_end()
    b.copy_from(a, 260)
    q = synth.normal(5, (21, n_heads, hd))
    c.pass_begin([(a, 248, 20), (b, 259, 1)])   # a 20-row chunk across the 256 edge + one decode row
    got = c.attn_prefill(0, q)
    c.pass_end(commit=False)
    gk, gv = a.read_kv(0, 0), a.read_kv(0, 1)
    npr = np.array(list(range(249, 269)) + [260], np.int32)
    want = checker.attention(F16, gk, gv, n_kv, n_heads, hd, q, npr)
    assert_close(got, want, "chunk rows")
    c.close()


def test_fill_synthetic_and_large_ragged_batch(checker):
    """Device-filled caches at Qwen3-8B head shapes, ragged contexts; the CPU checker runs on the downloaded bytes."""
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 32, 8, 128
    ctxs = [512, 777, 4096, 2049]
    for kvt in (F16, Q8):
        c = make_ctx(n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
        c.set_exact(True)
        seqs = []
        for i, n in enumerate(ctxs):
            s = c.new_seq(n, kvt)
            s.fill_synthetic(n, 1234 + i)
            seqs.append(s)
        q = synth.normal(9, (len(ctxs), n_heads, hd))
        c.pass_begin([(s, n - 1, 1) for s, n in zip(seqs, ctxs)])
        got = c.attn_decode(0, q)
        c.pass_end(commit=False)
        for i, (s, n) in enumerate(zip(seqs, ctxs)):
            want = checker.attention(kvt, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[i:i + 1], np.array([n], np.int32),
                                     split=1)
            assert_close(got[i:i + 1], want, f"ragged kvt={kvt} ctx={n}")
            assert bit_equal(got[i:i + 1], want)
        c.close()


def test_argument_errors_leave_state_untouched():
    import gwenedeg_b200 as g
    c = make_ctx(n_attn=1, n_heads=4, n_kv_heads=2, head_dim=128, max_rows=8)
    s = c.new_seq(100, F16)
    with pytest.raises(g.RqCudaError) as e:
        c.pass_begin([(s, 99, 2)])           # runs past the capacity
    assert e.value.code == -3
    with pytest.raises(g.RqCudaError) as e:
        c.pass_begin([(s, 0, 9)])            # more rows than the context allows
    assert e.value.code == -1
    with pytest.raises(g.RqCudaError) as e:
        c.pass_begin([(s, 5, 1)])            # a gap after the sequence's length
    assert e.value.code == -1
    with pytest.raises(g.RqCudaError) as e:
        c.pass_begin([(s, 0, 1), (s, 1, 1)])  # a sequence twice
    assert e.value.code == -1
    with pytest.raises(g.RqCudaError) as e:
        c.nrows = 1
        c.attn_decode(0, np.zeros((1, 4, 128), np.float32))  # no pass open
    assert e.value.code == -4
    assert s.len == 0
    with pytest.raises(g.RqCudaError):
        c.new_seq(10, 1)                     # bf16 caches are not implemented on the device
    # device pointers that are not 16-byte aligned are refused before anything is launched
    buf = c.malloc(4 * 128 * 4 + 64)
    c.pass_begin([(s, 0, 1)])
    with pytest.raises(g.RqCudaError) as e:
        c.attn_decode_dev(0, buf + 4, buf)
    assert e.value.code == -1 and "aligned" in str(e.value)
    # a sequence freed while it belongs to the open pass goes away when the pass is closed, not under it
    t = c.new_seq(100, F16)
    c.pass_end(commit=False)
    c.pass_begin([(s, 0, 1), (t, 0, 1)])
    t.free()
    c.pass_end()
    assert s.len == 1
    c.pass_begin([(s, 1, 1)])
    c.pass_end(commit=False)
    c.close()


def test_expired_device_wait_is_reported_and_the_context_stays_usable():
    """A kernel whose bounded wait runs out (here: a one-CTA kernel waiting ~1 ms on a barrier nothing completes; it gives
    up and returns by itself) makes the next synchronisation fail with RQ_CUDA_ERR_STATE naming the wait's code, and the
    pass after it computes what the pass before it did."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    c = make_ctx(n_attn=1, n_heads=8, n_kv_heads=2, head_dim=128, max_rows=4)
    s = c.new_seq(1000, F16)
    s.fill_synthetic(1000, 3)
    q = synth.normal(4, (1, 8, 128))
    c.pass_begin([(s, 999, 1)])
    before = c.attn_decode(0, q)
    c.pass_end(commit=False)
    c.check(c.L.rq_cuda_selftest_wait_expiry(c.h, 1000))
    with pytest.raises(g.RqCudaError) as e:
        c.sync()
    assert e.value.code == -4 and "code 99" in str(e.value)
    c.sync()  # the status word was cleared by the failed call
    c.pass_begin([(s, 999, 1)])
    after = c.attn_decode(0, q)
    c.pass_end(commit=False)
    assert bit_equal(before, after)
    c.close()


def test_peer_wait_runs_out_when_a_rank_never_arrives():
    """The wait of the fused gather (rq_cuda_attn_decode_gather_dev) on one GPU: a two-rank exchange whose other rank does not
    exist.  The one-warp kernel gives up after its limit and returns; the sync reports RQ_CUDA_ERR_STATE with code 97, and the
    context computes the same bits afterwards."""
    from gwenedeg_b200 import synth
    import gwenedeg_b200 as g
    c = make_ctx(n_attn=1, n_heads=4, n_kv_heads=2, head_dim=128)
    s = c.new_seq(300, F16)
    s.fill_synthetic(300, 3)
    q = synth.normal(8, (1, 4, 128))
    c.pass_begin([(s, 299, 1)])
    before = c.attn_decode(0, q)
    c.pass_end(commit=False)
    c.check(c.L.rq_cuda_selftest_peer_wait(c.h, 2000))
    with pytest.raises(g.RqCudaError) as ei:
        c.sync()
    assert ei.value.code == -4 and "code 97" in str(ei.value)
    c.sync()  # the status word was cleared by the failed call
    c.pass_begin([(s, 299, 1)])
    after = c.attn_decode(0, q)
    c.pass_end(commit=False)
    assert bit_equal(before, after)
    c.close()


@pytest.mark.parametrize("kvt", [F16, Q8])
def test_page_locked_result_buffer_is_written_in_place(kvt):
    """rq_cuda_attn_decode / _prefill store straight into a page-locked (mapped) host buffer and copy into an ordinary one:
    the rows are the same bit for bit, and nothing outside them is touched."""
    import ctypes as C
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd, rows = 8, 2, 128, 5
    c = make_ctx(n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, max_rows=512)
    seqs = []
    for i in range(rows):
        s = c.new_seq(1200, kvt)
        s.fill_synthetic(300 + 211 * i, 40 + i)
        seqs.append(s)
    q = synth.normal(91, (rows, n_heads, hd))
    pinned = c.pinned((rows + 1, n_heads, hd))
    for fn, name in ((c.L.rq_cuda_attn_decode, "decode"), (c.L.rq_cuda_attn_prefill, "prefill")):
        c.pass_begin([(s, s.len - 1, 1) for s in seqs])
        plain = c._attn(fn, 0, q)  # an ordinary numpy array: staged on the device, then copied
        pinned[:] = 7.0
        c.check(fn(c.h, 0, q.ctypes.data_as(C.c_void_p), pinned.ctypes.data_as(C.c_void_p)))
        c.pass_end(commit=False)
        assert bit_equal(plain, pinned[:rows]), name
        assert np.all(pinned[rows] == 7.0), name
    c.close()


@pytest.mark.parametrize("kvt,hd,gs", [(F16, 128, 32), (Q8, 128, 64), (F16, 256, 256), (F16, 64, 32), (F16, 128, 128)])
def test_quantised_copy_of_the_outputs_for_the_wo_matmul(checker, kvt, hd, gs):
    """rq_cuda_set_wo_quant: the merge kernels (decode and prefill) leave int8 levels and scales of their output rows, the
    bits the reference's quantize() gives on the same fp32 rows (forward.c:803; its call right after the attention,
    :2716-2719)."""
    from gwenedeg_b200 import synth
    n_heads, n_kv = 8, 2
    gated = hd == 256
    c = make_ctx(n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated, max_rows=512)
    s = c.new_seq(2600, kvt)
    s.fill_synthetic(2600, 17)
    rows = 70
    xq_dev, xs_dev = c.malloc(rows * n_heads * hd), c.malloc(rows * n_heads * hd // gs * 4)
    c.set_wo_quant(gs, xq_dev, xs_dev)
    q = synth.normal(3, (rows, n_heads, hd * (2 if gated else 1)))
    for fn in (c.attn_decode, c.attn_prefill):
        c.pass_begin([(s, 2300, rows)])
        out = fn(0, q)
        xq, xs = np.empty((rows, n_heads * hd), np.int8), np.empty((rows, n_heads * hd // gs), np.float32)
        c.d2h(xq, xq_dev)
        c.d2h(xs, xs_dev)
        c.sync()
        c.pass_end(commit=False)
        wq, ws = checker.quantize(out.reshape(rows, -1), gs)
        assert np.array_equal(xq, wq) and bit_equal(xs.reshape(-1), ws), fn.__name__
    c.set_wo_quant(0, None, None)
    c.close()


def test_pass_timing_feeds_the_cost_model():
    """rq_cuda_pass_timing / _pass_time / _pass_cost_measure: the device time of a pass with the sums S1, S2 that the reference's
    cost model multiplies (seg_cost, engine.c:2631), and a calibration whose terms are positive and ordered as the model says
    (further rows of a segment share the first row's read of the cache: att_x <= att)."""
    c = make_ctx(n_attn=4, n_heads=32, n_kv_heads=8, head_dim=128, max_rows=64)
    a, b = c.new_seq(20000, F16), c.new_seq(20000, F16)
    a.fill_synthetic(9000, 1)
    b.fill_synthetic(500, 2)
    qd, od = c.malloc(21 * 32 * 128 * 4), c.malloc(21 * 32 * 128 * 4)
    c.pass_timing(True)
    c.pass_begin([(a, 9000, 20), (b, 500, 1)])
    for l in range(4):
        c.attn_prefill_dev(l, qd, od)
    c.pass_end(commit=False)
    secs, rows, s1, s2 = c.pass_time()
    assert rows == 21 and s1 == 9500 and s2 == 19 * 9000 + 19 * 20 / 2
    assert 1e-6 < secs < 0.1
    c.pass_timing(False)
    tw, att, attx = c.pass_cost_measure(a, 16384, reps=3)
    assert a.len == 0
    assert 0 < att < 1e-6 and 0 <= attx <= att and 0 <= tw < 1e-2, (tw, att, attx)
    # a decode step at 16,384 positions by the model is the time the step takes (4 layers), to a factor of two
    a.fill_synthetic(16385, 3)
    c.pass_timing(True)
    for _ in range(3):
        c.pass_begin([(a, 16384, 1)])
        for l in range(4):
            c.attn_decode_dev(l, qd, od)
        c.pass_end(commit=False)
    took = c.pass_time()[0]
    assert 0.5 < took / (tw + att * 16384) < 2.0, (took, tw, att)
    c.close()
