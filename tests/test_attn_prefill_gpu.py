"""Parity of the tensor-core prefill attention (through the C ABI) with the CPU checker.

Q and the softmax weights are rounded to f16 for the tensor cores, so the comparison is by the acceptance bar
(max-abs <= 2e-3, rel-L2 <= 1e-3; per row 4e-3), not bit for bit; the split-K decode kernels on the same rows
(bit-exact with the CPU) serve as a second reference.
"""
import numpy as np
import pytest

from tests.helpers import assert_close, bit_equal, errors

pytestmark = pytest.mark.gpu
F16 = 2


def fill_seq(c, n, n_kv, hd, seed):
    from gwenedeg_b200 import synth
    s = c.new_seq(n, F16)
    k, v = synth.normal(seed, (n, n_kv, hd)), synth.normal(seed + 1, (n, n_kv, hd))
    for lo in range(0, n, 512):
        hi = min(n, lo + 512)
        c.pass_begin([(s, lo, hi - lo)])
        c.kv_store(0, k[lo:hi], v[lo:hi])
        c.pass_end()
    return s


@pytest.mark.parametrize("n_heads,n_kv,gated", [(16, 4, True), (4, 2, False), (8, 1, True), (3, 3, False)])
def test_head_dim_256_chunks_match_cpu(checker, n_heads, n_kv, gated):
    """The head_dim 256 tensor-core kernel (K / V staged in 128-dim halves, one O accumulator): a chunk from position 0, a
    chunk over a prefix that crosses the 2,048-position split edge, and a decode row of another sequence in one pass;
    with and without the sigmoid output gate, 1, 2, 4 and 8 query heads per KV head."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    hd = 256
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated)
    a = fill_seq(c, 150, n_kv, hd, 21)
    b = fill_seq(c, 2300, n_kv, hd, 23)
    d = fill_seq(c, 700, n_kv, hd, 25)
    segs = [(a, 0, 150), (b, 1990, 210), (d, 699, 1)]
    qh = hd * (2 if gated else 1)
    q = synth.normal(19, (361, n_heads, qh))
    c.pass_begin(segs)
    got = c.attn_prefill(0, q)
    exact = c.attn_decode(0, q)  # the split-K kernels on the same rows: the CPU code's bits
    c.pass_end(commit=False)
    assert_close(got, exact, "head_dim 256 against the split-K path")
    r = 0
    for s, pos0, n in segs:
        pick = sorted(set(i for i in (0, 1, n // 2, n - 1) if i < n))
        want = checker.attention(F16, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[r:r + n][pick],
                                 np.array([pos0 + 1 + i for i in pick], np.int32), gated=gated)
        assert_close(got[r:r + n][pick], want, f"segment at {pos0}")
        assert bit_equal(exact[r:r + n][pick], want)
        r += n
    print("hd256 prefill errors", errors(got, exact))
    c.close()


def test_hybrid_stack_gated_attention_chunk(checker):
    """The Qwen3.5-style gated attention layer at its benchmark shape: 16 query / 4 KV heads x 256, 512 new rows over a
    7,680-position f16 prefix (four splits of 2,048 keys), sigmoid output gate; every row against the bit-exact split-K path,
    a few against the CPU code."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 16, 4, 256
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=True)
    s = c.new_seq(8192, F16)
    s.fill_synthetic(8192, 31)
    q = synth.normal(33, (512, n_heads, 2 * hd))
    c.pass_begin([(s, 7680, 512)])
    got = c.attn_prefill(0, q)
    exact = c.attn_decode(0, q)
    c.pass_end(commit=False)
    assert_close(got, exact, "gated head_dim 256, all rows")
    rows = [0, 31, 32, 255, 511]
    want = checker.attention(F16, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[rows], np.array([7681 + r for r in rows], np.int32), gated=True)
    assert_close(got[rows], want, "gated head_dim 256 rows against the CPU code")
    assert bit_equal(exact[rows], want)
    print("hybrid-stack gated attention errors", errors(got, exact))
    c.close()


@pytest.mark.parametrize("n_heads,n_kv", [(16, 8), (32, 8), (8, 8), (16, 2)])
def test_chunk_over_prefix_matches_cpu(checker, n_heads, n_kv):
    """A chunk of rows over a cached prefix, crossing tile and 256-block edges (the 2,048-position split edge is crossed in test_short_rows_and_mixed_segments)."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    hd, n = 128, 1300
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
    s = fill_seq(c, n, n_kv, hd, 40 + n_heads)
    pos0, rows = 900, 300   # rows at positions 900..1199: np 901..1200
    q = synth.normal(7, (rows, n_heads, hd))
    c.pass_begin([(s, pos0, rows)])
    got = c.attn_prefill(0, q)
    ref_gpu = c.attn_decode(0, q)
    c.pass_end(commit=False)
    want = checker.attention(F16, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q, np.arange(pos0 + 1, pos0 + rows + 1, dtype=np.int32))
    assert_close(ref_gpu, want, "split-K on the chunk")
    assert_close(got, want, "tensor-core prefill")
    print("prefill errors", errors(got, want))
    c.close()


def test_short_rows_and_mixed_segments(checker):
    """Rows from position 0 (a single key, partial tiles), two chunks and decode rows of other sequences in one pass."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 16, 8, 128
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
    a = fill_seq(c, 200, n_kv, hd, 1)
    b = fill_seq(c, 2500, n_kv, hd, 3)
    d = fill_seq(c, 1025, n_kv, hd, 5)
    segs = [(a, 0, 70), (b, 2040, 100), (d, 1024, 1)]
    q = synth.normal(9, (171, n_heads, hd))
    c.pass_begin(segs)
    got = c.attn_prefill(0, q)
    c.pass_end(commit=False)
    r = 0
    for s, pos0, n in segs:
        want = checker.attention(F16, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[r:r + n], np.arange(pos0 + 1, pos0 + n + 1, dtype=np.int32))
        assert_close(got[r:r + n], want, f"segment at {pos0}")
        r += n
    c.close()


def test_config2_shape_one_layer(checker):
    """Qwen3-0.6B-shaped chunked prefill: 512 rows at positions 3584..4095 over a 4096-position cache (one layer)."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 16, 8, 128
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
    s = c.new_seq(4096, F16)
    s.fill_synthetic(4096, 11)
    q = synth.normal(13, (512, n_heads, hd))
    c.pass_begin([(s, 3584, 512)])
    got = c.attn_prefill(0, q)
    exact = c.attn_decode(0, q)  # the split-K kernels on the same rows: the CPU code's bits
    c.pass_end(commit=False)
    rows = [0, 1, 63, 64, 255, 511]  # the CPU checker on a few rows (the full chunk takes it a while)
    want = checker.attention(F16, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[rows], np.array([3585 + r for r in rows], np.int32))
    assert_close(got[rows], want, "config-2 rows")
    assert bit_equal(exact[rows], want), "the split-K path is expected to equal the CPU code bit for bit"
    # every one of the 512 rows x 16 heads against the bit-exact path
    assert_close(got, exact, "config-2, all rows")
    c.close()


@pytest.mark.parametrize("kvt,name", [(3, "q8"), (8, "q4"), (9, "q4k4")])
@pytest.mark.parametrize("n_heads,n_kv,gated,hd", [(8, 2, False, 128), (4, 4, True, 128), (8, 2, True, 256)])
def test_quantised_cache_prompt_chunks_on_tensor_cores(checker, kvt, name, n_heads, n_kv, gated, hd):
    """Prompt passes over q8 / q4 / q4k4 caches at head_dim 128 and 256: the layer's tiles expanded to f16 once per call, the query rows
    rotated, the tensor-core kernel, the un-rotating merge.  Every row against the row-by-row path through the decode kernels
    (rq_cuda_set_exact: the CPU code's bits), a few rows against the CPU code itself; a chunk from position 0, a chunk over a
    prefix that crosses the 2,048-position split edge and ends inside a block, and a third segment."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    c = g.Context(0, n_attn=2, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated, max_rows=512)
    seqs = []
    for i, n in enumerate((150, 2300, 700)):
        s = c.new_seq(n, kvt)
        k, v = synth.normal(40 + 2 * i, (n, n_kv, hd)), synth.normal(41 + 2 * i, (n, n_kv, hd))
        for lo in range(0, n, 512):
            hi = min(n, lo + 512)
            c.pass_begin([(s, lo, hi - lo)])
            for l in range(2):
                c.kv_store(l, k[lo:hi] * np.float32(1 + l), v[lo:hi])
            c.pass_end()
        seqs.append(s)
    a, b, d = seqs
    segs = [(a, 0, 150), (b, 1990, 210), (d, 680, 20)]
    rows = sum(n for _, _, n in segs)
    q = synth.normal(19, (rows, n_heads, hd * (2 if gated else 1)))
    for layer in (1, 0):
        c.set_exact(False)
        c.pass_begin(segs)
        got = c.attn_prefill(layer, q)
        c.pass_end(commit=False)
        c.set_exact(True)
        c.pass_begin(segs)
        exact = c.attn_prefill(layer, q)
        c.pass_end(commit=False)
        assert not bit_equal(got, exact)  # (the two paths are different kernels)
        assert_close(got, exact, f"{name} layer {layer}: tensor-core prompt pass against the row-by-row path")
        r = 0
        for s, pos0, n in segs:
            pick = sorted(set(i for i in (0, 1, n // 2, n - 1) if i < n))
            want = checker.attention(kvt, s.read_kv(layer, 0), s.read_kv(layer, 1), n_kv, n_heads, hd, q[r:r + n][pick],
                                     np.array([pos0 + 1 + i for i in pick], np.int32), gated=gated)
            assert_close(got[r:r + n][pick], want, f"{name} segment at {pos0}")
            assert bit_equal(exact[r:r + n][pick], want)
            r += n
        print(name, "quantised prompt pass errors", errors(got, exact))
    c.set_exact(False)
    c.close()


@pytest.mark.parametrize("kvt,name", [(3, "q8"), (9, "q4k4")])
def test_quantised_cache_prompt_chunk_at_benchmark_shape(kvt, name):
    """The 0.6B-model prompt chunk of the benchmark on a quantised cache: 512 new rows over a 3,584-position prefix, 16 query / 8
    KV heads x 128; every row of the tensor-core pass (f16 expansion of the tiles) against the row-by-row pass through the
    bit-exact decode kernels."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd = 16, 8, 128
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, max_rows=512)
    s = c.new_seq(4096, kvt)
    s.fill_synthetic(4096, 91)
    q = synth.normal(92, (512, n_heads, hd))
    c.set_exact(False)
    c.pass_begin([(s, 3584, 512)])
    got = c.attn_prefill(0, q)
    c.pass_end(commit=False)
    c.set_exact(True)
    c.pass_begin([(s, 3584, 512)])
    exact = c.attn_prefill(0, q)
    c.pass_end(commit=False)
    assert_close(got, exact, f"{name} prompt chunk, all 512 rows")
    print(name, "benchmark-shape quantised prompt chunk errors", errors(got, exact))
    c.set_exact(False)
    c.close()


@pytest.mark.parametrize("kvt,name", [(3, "q8"), (8, "q4")])
def test_quantised_mixed_pass_routes_by_segment(checker, kvt, name):
    """A pass that mixes prompt chunks with decode rows of other sequences over a quantised cache: the prompt segments go
    through the f16 expansion and the tensor-core prefill kernel, the short segments through the tensor-core decode kernels, run by
    run of adjacent rows; every row against the row-by-row bit-exact pass, and the quantised copy for the `wo` matmul equal to
    quantize() of the rows that came out."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    n_heads, n_kv, hd, gs = 8, 2, 128, 64
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, max_rows=512)
    lens = (150, 700, 2300, 301, 60, 900)
    seqs = []
    for i, n in enumerate(lens):
        s = c.new_seq(n, kvt)
        s.fill_synthetic(n, 50 + i)
        seqs.append(s)
    a, d, b, e, f, h = seqs
    # decode row | prompt chunk | two decode-like segments | prompt chunk | decode row
    segs = [(d, 699, 1), (a, 0, 150), (e, 300, 1), (f, 57, 3), (b, 1990, 210), (h, 899, 1)]
    rows = sum(n for _, _, n in segs)
    q = synth.normal(29, (rows, n_heads, hd))
    xq_dev, xs_dev = c.malloc(rows * n_heads * hd), c.malloc(rows * n_heads * hd // gs * 4)
    c.set_wo_quant(gs, xq_dev, xs_dev)
    c.set_exact(False)
    c.pass_begin(segs)
    got = c.attn_prefill(0, q)
    xq, xs = np.empty((rows, n_heads * hd), np.int8), np.empty((rows, n_heads * hd // gs), np.float32)
    c.d2h(xq, xq_dev)
    c.d2h(xs, xs_dev)
    c.sync()
    c.pass_end(commit=False)
    c.set_wo_quant(0, None, None)
    c.set_exact(True)
    c.pass_begin(segs)
    exact = c.attn_prefill(0, q)
    c.pass_end(commit=False)
    assert_close(got, exact, f"{name} mixed pass against the row-by-row path")
    wq, ws = checker.quantize(got.reshape(rows, -1), gs)
    assert np.array_equal(xq, wq) and bit_equal(xs.reshape(-1), ws)
    # the decode rows took the decode kernels: the same bits as a decode call on those rows alone
    c.set_exact(False)
    c.pass_begin([(d, 699, 1)])
    alone = c.attn_decode(0, q[0:1])
    c.pass_end(commit=False)
    assert bit_equal(alone, got[0:1])
    c.close()


@pytest.mark.parametrize("hd,n_heads,n_kv,gated", [(128, 8, 2, False), (256, 8, 2, True)])
def test_prefill_split_lengths_agree(checker, hd, n_heads, n_kv, gated):
    """The split length of a prompt pass is chosen per pass; every length gives the attention inside the tolerance: a chunk of
    300 rows over a 5,000-position prefix with the length fixed to 1,024, 1,280, 2,048, 4,096 and 8,192 positions and left to
    the library, each against the bit-exact split-K path; a few rows against the CPU code."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    c = g.Context(0, n_attn=1, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, gated=gated, max_rows=512)
    s = c.new_seq(5300, F16)
    s.fill_synthetic(5300, 61)
    q = synth.normal(62, (300, n_heads, hd * (2 if gated else 1)))
    c.pass_begin([(s, 5000, 300)])
    exact = c.attn_decode(0, q)
    c.pass_end(commit=False)
    outs = []
    for L in (1024, 1280, 2048, 4096, 8192, 0):
        c.set_prefill_split(L)
        c.pass_begin([(s, 5000, 300)])
        got = c.attn_prefill(0, q)
        c.pass_end(commit=False)
        assert_close(got, exact, f"head_dim {hd}, split {L}")
        outs.append(got)
    assert not bit_equal(outs[0], outs[4])  # (five splits against one: the lengths really differ)
    rows = [0, 150, 299]
    want = checker.attention(F16, s.read_kv(0, 0), s.read_kv(0, 1), n_kv, n_heads, hd, q[rows], np.array([5001 + r for r in rows], np.int32), gated=gated)
    assert_close(outs[-1][rows], want, "chosen split against the CPU code")
    with pytest.raises(g.RqCudaError):
        c.set_prefill_split(1000)
    c.set_prefill_split(0)
    c.close()
