"""Saved sequences in the reference's file format (src/seqfile.c): files written from device caches load into the
reference's own host sequences through its rq_seq_load, files written by its rq_seq_save load into device caches, byte for
byte, with the DeltaNet state and a checkpoint; a file of another model or a damaged one is refused."""
import os

import numpy as np
import pytest

from tests.helpers import bit_equal

pytestmark = pytest.mark.gpu


def _fill(c, s, n, n_kv, hd, layers, seed):
    from gwenedeg_b200 import synth
    kv = [(synth.normal(seed + 2 * l, (n, n_kv, hd)), synth.normal(seed + 2 * l + 1, (n, n_kv, hd))) for l in range(layers)]
    for lo in range(0, n, 512):
        hi = min(n, lo + 512)
        c.pass_begin([(s, lo, hi - lo)])
        for l in range(layers):
            c.kv_store(l, kv[l][0][lo:hi], kv[l][1][lo:hi])
        c.pass_end()


@pytest.mark.parametrize("kvt", [2, 3, 8], ids=["f16", "q8", "q4"])
def test_sequence_files_interchange_with_the_reference(ref, tmp_path, kvt):
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    n_attn, n_heads, n_kv, hd, cap, n = 2, 4, 2, 128, 700, 600
    fp = 0x1234ABCD5678
    c = g.Context(0, n_attn=n_attn, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd)
    s = c.new_seq(cap, kvt)
    _fill(c, s, n, n_kv, hd, n_attn, 100 + kvt)
    assert s.len == n
    tokens = synth.integers(7, 0, 150000, (n,)).astype(np.int32)
    path = tmp_path / "ours.rqseq"
    s.save(path, tokens, model_fp=fp, rng=0xFEEDFACE)
    # ---- ours -> the reference's loader
    r = gwo.RefSeq(ref, kvt, n_attn, n_kv, hd, cap, fp=fp)
    assert os.path.getsize(path) == c.L.rq_cuda_seq_save_bytes(s.h)
    assert r.load(path, n) == 0, "the reference's rq_seq_load refused the file"
    rt, rk, rv, _, _, _, rrng = r.get()
    assert np.array_equal(rt, tokens) and rrng == 0xFEEDFACE
    nblk = (n + 255) // 256
    for l in range(n_attn):
        for is_v, theirs in ((0, rk), (1, rv)):
            lb = s.layer_bytes(is_v)
            used = nblk * 16 * n_kv * ref.tile_bytes(kvt, hd, is_v)
            assert np.array_equal(s.read_kv(l, is_v)[:used], theirs[l * lb:l * lb + used]), (l, is_v)
    assert r.save_bytes() == os.path.getsize(path)
    # ---- the reference's writer -> ours: the file it writes from that sequence is the file we wrote, byte for byte
    path2 = tmp_path / "theirs.rqseq"
    assert r.save(path2) == 0
    assert open(path, "rb").read() == open(path2, "rb").read()
    t = c.new_seq(cap, kvt)
    tk, rng = t.load(path2, n, model_fp=fp)
    assert t.len == n and np.array_equal(tk, tokens) and rng == 0xFEEDFACE
    q = synth.normal(9, (1, n_heads, hd))
    outs = []
    for seq in (s, t):
        c.pass_begin([(seq, n - 1, 1)])
        outs.append(c.attn_decode(1, q))
        c.pass_end(commit=False)
    assert bit_equal(outs[0], outs[1])
    # a prefix: the first 300 positions (two blocks) of the file
    u = c.new_seq(cap, kvt)
    tk, _ = u.load(path2, 300, model_fp=fp)
    assert u.len == 300 and np.array_equal(tk, tokens[:300])
    c.pass_begin([(s, 299, 1)])
    a = c.attn_decode(0, q)
    c.pass_end(commit=False)
    c.pass_begin([(u, 299, 1)])
    b = c.attn_decode(0, q)
    c.pass_end(commit=False)
    assert bit_equal(a, b)
    # refusals: another model's fingerprint, another cache type, a damaged header, a truncated file
    with pytest.raises(g.RqCudaError) as e:
        u.load(path2, n, model_fp=fp + 1)
    assert e.value.code == -7
    other = c.new_seq(cap, 2 if kvt != 2 else 3)
    with pytest.raises(g.RqCudaError) as e:
        other.load(path2, n, model_fp=fp)
    assert e.value.code == -7
    raw = bytearray(open(path2, "rb").read())
    raw[4096 + 8] ^= 1  # a token changed: the hash no longer matches
    bad = tmp_path / "bad.rqseq"
    open(bad, "wb").write(raw)
    with pytest.raises(g.RqCudaError) as e:
        u.load(bad, n, model_fp=fp)
    assert e.value.code == -7
    open(bad, "wb").write(bytes(raw[:len(raw) - 4096]))
    with pytest.raises(g.RqCudaError) as e:
        u.load(bad, n, model_fp=fp)
    assert e.value.code == -7
    with pytest.raises(g.RqCudaError) as e:
        u.load(tmp_path / "missing.rqseq", n, model_fp=fp)
    assert e.value.code == -6
    c.close()


def test_sequence_file_with_deltanet_state_and_checkpoint(ref, tmp_path):
    """A hybrid model's file: attention caches, the recurrent state at the saved length and a checkpoint below it, both
    ways; loading fewer positions than saved lands on the checkpoint (rq_seq_file_keep)."""
    import gwenedeg_b200 as g
    from gwenedeg_b200 import synth
    from oracle import gwo
    n_attn, n_heads, n_kv, hd, cap = 1, 4, 2, 128, 512
    nk, nv, n_lin, n = 2, 4, 2, 300
    fp = 77
    c = g.Context(0, n_attn=n_attn, n_heads=n_heads, n_kv_heads=n_kv, head_dim=hd, n_lin=n_lin, dn_nk=nk, dn_nv=nv, max_rows=512)
    s = c.new_seq(cap, 2)
    s.set_checkpoints(2)
    rows = synth.deltanet_rows(5, n, nk, nv, 128, 128)
    k, v = synth.normal(1, (n, n_kv, hd)), synth.normal(2, (n, n_kv, hd))
    c.pass_begin([(s, 0, n)])
    c.pass_checkpoint(0, 199, 1)   # a checkpoint at length 200, in slot 1
    c.kv_store(0, k, v)
    for li in range(n_lin):
        c.dn_rec(li, rows)
    c.pass_end()
    assert s.len == n and s.checkpoint_pos(1) == 200
    tokens = np.arange(n, dtype=np.int32)
    path = tmp_path / "hybrid.rqseq"
    s.save(path, tokens, model_fp=fp, rng=5)
    sf = s.state_floats()
    state = np.concatenate([s.read_state(li) for li in range(n_lin)])
    ck = np.concatenate([s.read_checkpoint(1, li) for li in range(n_lin)])
    # ---- into the reference: whole, then a prefix that lands on the checkpoint
    r = gwo.RefSeq(ref, 2, n_attn, n_kv, hd, cap, fp=fp, n_lin=n_lin, nk=nk, nv=nv)
    assert r.state_floats == sf * n_lin
    assert r.load(path, n) == 0
    rt, rk, rv, rs, rpos, rck, _ = r.get()
    assert len(rt) == n and bit_equal(rs, state)
    assert r.load(path, 250) == 0
    rt, rk, rv, rs, rpos, rck, _ = r.get()
    assert len(rt) == 200 and bit_equal(rs, ck), "250 positions asked: the checkpoint at 200 is where the state exists"
    # ---- the reference's file of the whole sequence equals ours; ours loads it, checkpoint included
    assert r.load(path, n) == 0
    path2 = tmp_path / "hybrid_ref.rqseq"
    assert r.save(path2) == 0
    assert open(path, "rb").read() == open(path2, "rb").read()
    t = c.new_seq(cap, 2)
    t.set_checkpoints(2)
    t.load(path2, n, model_fp=fp)
    assert t.len == n and t.checkpoint_pos(0) == 200
    for li in range(n_lin):
        assert bit_equal(t.read_state(li), s.read_state(li)) and bit_equal(t.read_checkpoint(0, li), s.read_checkpoint(1, li))
    t.load(path2, 250, model_fp=fp)
    assert t.len == 200
    for li in range(n_lin):
        assert bit_equal(t.read_state(li), s.read_checkpoint(1, li))
    # the rolled-back copy continues exactly as the original restored to its checkpoint
    s.restore(1)
    outs = []
    for seq in (s, t):
        c.pass_begin([(seq, 200, 50)])
        outs.append(c.dn_rec(1, rows[200:250]))
        c.pass_end(commit=False)
    assert bit_equal(outs[0], outs[1])
    c.close()
