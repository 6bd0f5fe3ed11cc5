"""Parity of the CUDA Gated DeltaNet kernels with the CPU checker: the token recurrence bit for bit (same operation
order), the chunked tensor-core form within the tolerance (max-abs 2e-3, relative L2 1e-3)."""
import numpy as np
import pytest

from tests.helpers import MAX_ABS, REL_L2, assert_close, bit_equal, errors

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nk,nv", [(2, 2), (2, 4)])
def test_recurrence_matches_cpu(checker, nk, nv):
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    dk = dv = 128
    c = g.Context(0, n_lin=2, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, max_rows=256)
    d = gwo.DeltaNet(checker, nk, nv, dk, dv)
    rows_a = synth.deltanet_rows(1, 150, nk, nv, dk, dv)
    rows_b = synth.deltanet_rows(2, 40, nk, nv, dk, dv)
    # DeltaNet-only contexts have no attention layers: sequences carry the state only
    sa, sb = c.new_seq(512, 2), c.new_seq(512, 2)
    st_a, st_b = d.new_state(), d.new_state()
    # pass 1: a 100-row chunk of a and the 40 rows of b, both from position 0
    c.pass_begin([(sa, 0, 100), (sb, 0, 40)])
    got = c.dn_rec(1, np.concatenate([rows_a[:100], rows_b]))
    c.pass_end()
    want_a, want_b = d.rec(st_a, rows_a[:100], True), d.rec(st_b, rows_b, True)
    assert_close(got[:100], want_a, "dn chunk a")
    assert bit_equal(got[:100], want_a) and bit_equal(got[100:], want_b)
    # pass 2: a continues with 49 rows, then a single decode row
    c.pass_begin([(sa, 100, 49)])
    got2 = c.dn_rec(1, rows_a[100:149])
    c.pass_end()
    c.pass_begin([(sa, 149, 1)])
    got3 = c.dn_rec(1, rows_a[149:150])
    c.pass_end()
    want2 = d.rec(st_a, rows_a[100:149], False)
    want3 = d.rec(st_a, rows_a[149:150], False)
    assert bit_equal(got2, want2) and bit_equal(got3, want3)
    assert bit_equal(sa.read_state(1)[d.conv_floats:], st_a[d.conv_floats:])
    assert not sa.read_state(0).any()  # the other layer's state is untouched
    c.close()


def test_prep_rec_out_pipeline_matches_cpu(checker):
    """dn_prep -> dn_rec -> dn_out on the device over two consecutive passes (the conv state carries over): q, k, v and beta
    equal the CPU code's bits, exp(g) agrees to the last bits (libm expf / log1pf), and from the device's own prepared rows
    the recurrence and the output stage equal the CPU code bit for bit."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    nk, nv, dk, dv, K = 2, 4, 128, 128, 4
    cd = 2 * nk * dk + nv * dv
    w_conv = synth.normal(21, (cd * K,)) * np.float32(0.5)
    w_a = (-np.abs(synth.normal(22, (nv,))) - np.float32(0.1)).astype(np.float32)
    w_dt, w_norm = synth.normal(23, (nv,)), synth.normal(24, (dv,))
    d = gwo.DeltaNet(checker, nk, nv, dk, dv, K, w_conv, w_a, w_dt, w_norm)
    c = g.Context(0, n_lin=1, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, dn_conv=K, max_rows=128)
    c.dn_set_weights(0, w_conv, w_a, w_dt, w_norm)
    s = c.new_seq(256, 2)
    st = d.new_state()
    raw = synth.normal(25, (70, d.lw))
    rows_dev = c.malloc(64 * d.lw * 4)
    out_dev = c.malloc(64 * nv * dv * 4)
    for lo, hi in ((0, 3), (3, 64), (64, 70)):   # a pass shorter than the conv window, a long one, a continuation
        n = hi - lo
        c.h2d(rows_dev, np.ascontiguousarray(raw[lo:hi]))
        c.pass_begin([(s, lo, n)])
        c.dn_prep_dev(0, rows_dev)
        prep_gpu = np.empty((n, d.lw), np.float32)
        c.d2h(prep_gpu, rows_dev)
        c.dn_rec_dev(0, rows_dev, out_dev)
        rec_gpu = np.empty((n, nv * dv), np.float32)
        c.d2h(rec_gpu, out_dev)
        c.dn_out_dev(0, rows_dev, out_dev)
        fin_gpu = np.empty((n, nv * dv), np.float32)
        c.d2h(fin_gpu, out_dev)
        c.sync()
        c.pass_end()
        st_before = st.copy()
        prep_cpu = d.prep(st, raw[lo:hi], lo == 0)
        eg0 = cd + nv * dv
        assert bit_equal(prep_gpu[:, :eg0], prep_cpu[:, :eg0])                    # q, k, v (and z untouched)
        assert bit_equal(prep_gpu[:, eg0 + nv:], prep_cpu[:, eg0 + nv:])          # beta
        assert np.abs(prep_gpu[:, eg0:eg0 + nv] / prep_cpu[:, eg0:eg0 + nv] - 1).max() < 1e-6   # exp(g)
        # from the device's prepared rows on, bits again
        st_rec = st_before.copy()
        st_rec[:d.conv_floats] = st[:d.conv_floats]
        rec_cpu = d.rec(st_rec, prep_gpu, lo == 0)
        assert bit_equal(rec_gpu, rec_cpu)
        assert bit_equal(fin_gpu, d.out(prep_gpu, rec_cpu))
        st[:] = st_rec
        got_state = s.read_state(0)
        assert bit_equal(got_state[:d.conv_floats], st[:d.conv_floats]) and bit_equal(got_state[d.conv_floats:], st[d.conv_floats:])
    c.close()


@pytest.mark.parametrize("nk,nv", [(2, 2), (2, 4)])
def test_chunked_form_matches_cpu(checker, nk, nv):
    """rq_cuda_dn_chunk (64-token chunks on the tensor cores) against the token recurrence of the CPU code: full and
    ragged chunks, two segments in a pass, a continuation pass that starts from the stored state, and the state itself."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    dk = dv = 128
    c = g.Context(0, n_lin=2, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, max_rows=512)
    d = gwo.DeltaNet(checker, nk, nv, dk, dv)
    rows_a = synth.deltanet_rows(11, 330, nk, nv, dk, dv)
    rows_b = synth.deltanet_rows(12, 64, nk, nv, dk, dv)
    sa, sb = c.new_seq(1024, 2), c.new_seq(1024, 2)
    st_a, st_b = d.new_state(), d.new_state()
    c.pass_begin([(sa, 0, 200), (sb, 0, 64)])
    got = c.dn_chunk(1, np.concatenate([rows_a[:200], rows_b]))
    c.pass_end()
    want_a, want_b = d.rec(st_a, rows_a[:200], True), d.rec(st_b, rows_b, True)
    assert_close(got[:200], want_a, "chunked a")
    assert_close(got[200:], want_b, "chunked b")
    assert_close(sa.read_state(1)[d.conv_floats:].reshape(-1, 128), st_a[d.conv_floats:].reshape(-1, 128), "state a")
    assert_close(sb.read_state(1)[d.conv_floats:].reshape(-1, 128), st_b[d.conv_floats:].reshape(-1, 128), "state b")
    # continuation from the stored state: 130 more rows of a (two chunks and two rows)
    c.pass_begin([(sa, 200, 130)])
    got2 = c.dn_chunk(1, rows_a[200:330])
    c.pass_end()
    want2 = d.rec(st_a, rows_a[200:330], False)
    assert_close(got2, want2, "chunked a, continued")
    assert_close(sa.read_state(1)[d.conv_floats:].reshape(-1, 128), st_a[d.conv_floats:].reshape(-1, 128), "state a, continued")
    # the exact recurrence carries on from the chunked form's state (decode after prefill)
    nxt = synth.deltanet_rows(13, 1, nk, nv, dk, dv)
    c.pass_begin([(sa, 330, 1)])
    got3 = c.dn_rec(1, nxt)
    c.pass_end()
    assert_close(got3, d.rec(st_a, nxt, False), "decode row after chunked prefill")
    assert not sa.read_state(0).any()
    c.close()


def test_chunked_form_ragged_segments(checker):
    """Segments of 1, 63, 64, 65 and 129 rows in one pass (chunks that are one token, one short, exact, one over), each
    from position 0, then all of them continued by 7 more rows: outputs and states against the token recurrence."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    nk, nv, dk, dv = 2, 4, 128, 128
    lens = [1, 63, 64, 65, 129]
    c = g.Context(0, n_lin=1, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, max_rows=512)
    d = gwo.DeltaNet(checker, nk, nv, dk, dv)
    seqs = [c.new_seq(512, 2) for _ in lens]
    states = [d.new_state() for _ in lens]
    rows = [synth.deltanet_rows(20 + i, n + 7, nk, nv, dk, dv) for i, n in enumerate(lens)]
    c.pass_begin([(s, 0, n) for s, n in zip(seqs, lens)])
    got = c.dn_chunk(0, np.concatenate([r[:n] for r, n in zip(rows, lens)]))
    c.pass_end()
    at = 0
    for i, n in enumerate(lens):
        want = d.rec(states[i], rows[i][:n], True)
        assert_close(got[at:at + n], want, f"segment of {n} rows")
        at += n
    c.pass_begin([(s, n, 7) for s, n in zip(seqs, lens)])
    got = c.dn_chunk(0, np.concatenate([r[n:] for r, n in zip(rows, lens)]))
    c.pass_end()
    for i, n in enumerate(lens):
        want = d.rec(states[i], rows[i][n:], False)
        assert_close(got[7 * i:7 * i + 7], want, f"segment of {n} rows, continued")
        assert_close(seqs[i].read_state(0)[d.conv_floats:].reshape(-1, 128), states[i][d.conv_floats:].reshape(-1, 128), f"state after {n} + 7 rows")
    c.close()


def test_prep_chunk_out_pipeline_matches_cpu(checker):
    """The prompt-pass pipeline on the device, back to back on one stream with no host synchronisation in between:
    dn_prep -> dn_chunk (tensor cores) -> dn_out over a 200-row pass and a 100-row continuation, against the CPU code's
    prep -> token recurrence -> out (tolerance: the chunked form rounds its operands to f16)."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    nk, nv, dk, dv, K = 2, 4, 128, 128, 4
    cd = 2 * nk * dk + nv * dv
    w_conv = synth.normal(31, (cd * K,)) * np.float32(0.5)
    w_a = (-np.abs(synth.normal(32, (nv,))) - np.float32(0.1)).astype(np.float32)
    w_dt, w_norm = synth.normal(33, (nv,)), synth.normal(34, (dv,))
    d = gwo.DeltaNet(checker, nk, nv, dk, dv, K, w_conv, w_a, w_dt, w_norm)
    c = g.Context(0, n_lin=1, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, dn_conv=K, max_rows=256)
    c.dn_set_weights(0, w_conv, w_a, w_dt, w_norm)
    s = c.new_seq(512, 2)
    st = d.new_state()
    raw = synth.normal(35, (300, d.lw))
    rows_dev = c.malloc(200 * d.lw * 4)
    out_dev = c.malloc(200 * nv * dv * 4)
    for lo, hi in ((0, 200), (200, 300)):
        n = hi - lo
        c.h2d(rows_dev, np.ascontiguousarray(raw[lo:hi]))
        c.pass_begin([(s, lo, n)])
        c.dn_prep_dev(0, rows_dev)
        c.dn_chunk_dev(0, rows_dev, out_dev)
        c.dn_out_dev(0, rows_dev, out_dev)
        fin_gpu = np.empty((n, nv * dv), np.float32)
        c.d2h(fin_gpu, out_dev)
        c.sync()
        c.pass_end()
        prep_cpu = d.prep(st, raw[lo:hi], lo == 0)
        fin_cpu = d.out(prep_cpu, d.rec(st, prep_cpu, lo == 0))
        # dn_out divides each head by its RMS (values of order 1 to 10 from recurrence outputs of order 1e-2), so the
        # absolute bar is scaled with the outputs' magnitude here; the relative one stands as it is
        ma, rl = errors(fin_gpu, fin_cpu)
        assert rl <= REL_L2 and ma <= MAX_ABS * max(1.0, float(np.abs(fin_cpu).max())), f"rows {lo}..{hi}: max-abs {ma:.3g}, rel-L2 {rl:.3g}"
    assert_close(s.read_state(0)[d.conv_floats:].reshape(-1, 128), st[d.conv_floats:].reshape(-1, 128), "state after the pipeline")
    c.close()


def _rows_fast(seed, n, nk, nv, dk, dv):
    """Post-prep rows with the distributions of synth.deltanet_rows from numpy's generator (the hash-based one takes most
    of a minute for 8,192 rows of 16 heads; these inputs only have to be the same for the GPU and the CPU)."""
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((n, nk, dk))
    k = rng.standard_normal((n, nk, dk))
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) / np.sqrt(dk)
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    v, z = rng.standard_normal((n, nv * dv)), rng.standard_normal((n, nv * dv))
    eg = np.exp(-np.log1p(np.exp(rng.standard_normal((n, nv)))))
    beta = 1.0 / (1.0 + np.exp(-rng.standard_normal((n, nv))))
    return np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v, z, eg, beta], axis=1).astype(np.float32)


def test_chunked_form_at_hybrid_stack_size(checker):
    """The chunked form at the size of the Qwen3.5-style configuration: one sequence of 8,192 tokens (128 chunks) in
    prompt passes of 512 rows, 16 key heads and 16 value heads of 128 x 128, against the token recurrence of the CPU code
    (dn_rec_run, reference src/forward.c:2224).  The form rounds its operands and a copy of the state to f16 in every
    chunk: outputs of every pass and the state after the last one have to stay inside the bar after 128 chunks."""
    import gwenedeg_b200 as g
    from oracle import gwo
    nk = nv = 16
    dk = dv = 128
    tokens, chunk = 8192, 512
    checker.threads(0)
    c = g.Context(0, n_lin=1, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, max_rows=chunk)
    d = gwo.DeltaNet(checker, nk, nv, dk, dv)
    rows = _rows_fast(5, tokens, nk, nv, dk, dv)
    s = c.new_seq(tokens, 2)
    st = d.new_state()
    worst = (0.0, 0.0)
    for pos in range(0, tokens, chunk):
        c.pass_begin([(s, pos, chunk)])
        got = c.dn_chunk(0, rows[pos:pos + chunk])
        c.pass_end()
        want = d.rec(st, rows[pos:pos + chunk], pos == 0)
        assert_close(got, want, f"rows {pos}..{pos + chunk - 1}")
        ma, rl = errors(got, want)
        worst = (max(worst[0], ma), max(worst[1], rl))
    gs, ws = s.read_state(0)[d.conv_floats:].reshape(-1, 128), st[d.conv_floats:].reshape(-1, 128)
    assert_close(gs, ws, "state after 8,192 tokens")
    print("chunked DeltaNet, 8192 tokens x 16 heads: outputs max-abs %.3g rel-L2 %.3g (worst pass); state max-abs %.3g rel-L2 %.3g"
          % (worst + errors(gs, ws)))
    c.close()


def test_checkpoints_inside_a_pass(checker):
    """State checkpoints taken by the kernels while a pass runs (CkPass; dn_rec_run, reference src/forward.c:2267-2270):
    a 150-row pass with checkpoints after rows 9 and 99; each slot holds the CPU code's state at that length; a sequence
    rolled back to a checkpoint and continued gives the rows it gave before (as the reference's checkpoints_bitwise /
    truncate_reprefill_bitwise tests, tests/api_test.c:635,689).  Exact form: bit for bit; chunked form (its chunks cut at the
    checkpoint rows): inside the tolerance, and the rolled-back run equal to the straight one bit for bit."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    nk, nv, dk, dv, K = 2, 4, 128, 128, 4
    cd = 2 * nk * dk + nv * dv
    w_conv = synth.normal(41, (cd * K,)) * np.float32(0.5)
    w_a = (-np.abs(synth.normal(42, (nv,))) - np.float32(0.1)).astype(np.float32)
    w_dt, w_norm = synth.normal(43, (nv,)), synth.normal(44, (dv,))
    d = gwo.DeltaNet(checker, nk, nv, dk, dv, K, w_conv, w_a, w_dt, w_norm)
    c = g.Context(0, n_lin=2, dn_nk=nk, dn_nv=nv, dn_dk=dk, dn_dv=dv, dn_conv=K, max_rows=256)
    c.dn_set_weights(1, w_conv, w_a, w_dt, w_norm)
    raw = synth.normal(45, (150, d.lw))
    # the CPU code: prepared rows, outputs, and the state after 10, 100 and 150 rows
    st = d.new_state()
    want_rows, want_out, want_state = [], [], {}
    for lo, hi in ((0, 10), (10, 100), (100, 150)):
        pr = d.prep(st, raw[lo:hi], lo == 0)
        want_rows.append(pr)
        want_out.append(d.rec(st, pr, lo == 0))
        want_state[hi] = st.copy()
    want_rows, want_out = np.concatenate(want_rows), np.concatenate(want_out)
    rows_dev, out_dev = c.malloc(150 * d.lw * 4), c.malloc(150 * nv * dv * 4)

    def run(seq, lo, hi, chunked, cks=()):
        n = hi - lo
        c.h2d(rows_dev, np.ascontiguousarray(raw[lo:hi]))
        c.pass_begin([(seq, lo, n)])
        for row, slot in cks:
            c.pass_checkpoint(0, row, slot)
        c.dn_prep_dev(1, rows_dev)
        (c.dn_chunk_dev if chunked else c.dn_rec_dev)(1, rows_dev, out_dev)
        out = np.empty((n, nv * dv), np.float32)
        c.d2h(out, out_dev)
        c.sync()
        c.pass_end()
        return out

    for chunked in (False, True):
        s = c.new_seq(256, 2)
        s.set_checkpoints(3)
        assert s.checkpoint_pos(0) == -1
        out = run(s, 0, 150, chunked, cks=((9, 0), (99, 1)))
        assert s.checkpoint_pos(0) == 10 and s.checkpoint_pos(1) == 100 and s.checkpoint_pos(2) == -1 and s.len == 150
        cf = d.conv_floats
        for slot, at in ((0, 10), (1, 100)):
            got = s.read_checkpoint(slot, 1)
            assert bit_equal(got[:cf], want_state[at][:cf]), "the conv inputs of a checkpoint"
            if chunked:
                assert_close(got[cf:].reshape(-1, 128), want_state[at][cf:].reshape(-1, 128), f"checkpoint at {at}, chunked form")
            else:
                # (exp(g) comes from the device's expf / log1pf: the last bits of S may differ from the CPU's libm)
                assert_close(got[cf:].reshape(-1, 128), want_state[at][cf:].reshape(-1, 128), f"checkpoint at {at}")
            assert not s.read_checkpoint(slot, 0).any()  # (layer 0 never ran: its state is the zero state at every length)
        assert_close(out, want_out, "outputs of the pass with checkpoints")
        # without checkpoints the same rows give the same bits (the exact form walks token by token either way)
        t = c.new_seq(256, 2)
        plain = run(t, 0, 150, chunked)
        if not chunked:
            assert bit_equal(plain, out)
        # roll back to length 100 and continue: rows 100..149 as before, bit for bit, and the same final state
        final = s.read_state(1)
        s.restore(1)
        assert s.len == 100 and s.checkpoint_pos(1) == 100
        again = run(s, 100, 150, chunked)
        if chunked:
            assert_close(again, out[100:], "continued after the rollback, chunked form")
        else:
            assert bit_equal(again, out[100:]), "continued after the rollback"
            assert bit_equal(s.read_state(1), final)
        # a copy of the first 10 positions takes the state from the checkpoint held at 10
        u = c.new_seq(256, 2)
        u.copy_from(s, 10)
        assert bit_equal(u.read_state(1), s.read_checkpoint(0, 1))
        # argument checks: no such slot, a row twice, after the first DeltaNet call of the pass
        c.pass_begin([(s, 150, 5)])
        with pytest.raises(g.RqCudaError):
            c.pass_checkpoint(0, 1, 3)
        c.pass_checkpoint(0, 1, 2)
        with pytest.raises(g.RqCudaError):
            c.pass_checkpoint(0, 1, 0)
        c.pass_end(commit=False)
        assert s.checkpoint_pos(2) == -1
    c.close()
