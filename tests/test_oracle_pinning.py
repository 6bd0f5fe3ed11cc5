"""Pins the plain-C restatement (oracle/gw_oracle.c) against the reference's own code compiled by oracle/Makefile,
on fresh seeded inputs, bit for bit.  Skipped where oracle/_ref is not built."""
import numpy as np
import pytest

from gwenedeg_b200 import synth
from oracle import gwo


def beq(a, b):
    return np.array_equal(np.ascontiguousarray(a, np.float32).view(np.uint32), np.ascontiguousarray(b, np.float32).view(np.uint32))


@pytest.mark.parametrize("which", ["ref", "ref-v4", "ref-generic"])
@pytest.mark.parametrize("kvt,hd,n_kv,n_heads,gated", [(gwo.F16, 128, 2, 4, False), (gwo.Q8, 128, 2, 8, False), (gwo.Q4, 128, 1, 2, True),
                                                        (gwo.Q4K4, 64, 2, 2, False), (gwo.F32, 64, 1, 2, False), (gwo.F16, 256, 1, 4, True),
                                                        (gwo.Q8, 256, 1, 2, False)])
def test_attention_and_codec_pinned(which, kvt, hd, n_kv, n_heads, gated):
    ref, port = gwo.load(which), gwo.load("port")
    if ref is None:
        pytest.skip("oracle/_ref not built")
    n = 700
    k, v = synth.normal(kvt + hd, (n, n_kv, hd)), synth.normal(kvt + hd + 1, (n, n_kv, hd))
    k[5, 0, 3] = 300.0
    kl, vl = port.new_cache(kvt, 768, n_kv, hd)
    port.kv_store(kvt, kl, vl, 0, k, v, n_kv, hd)
    kl2, vl2 = ref.new_cache(kvt, 768, n_kv, hd)
    ref.kv_store(kvt, kl2, vl2, 0, k, v, n_kv, hd)
    # stores: identical except where the reference's -Ofast builds replace x / d by a reciprocal (exact ties of
    # rint(x / d) then land one level off); never more than one level, and rare
    for a, b in ((kl, kl2), (vl, vl2)):
        diff = a != b
        assert diff.mean() < 2e-4
        if diff.any():
            assert np.abs(a[diff].astype(np.int16) - b[diff].astype(np.int16)).max() <= 17  # one level (a nibble may carry)
    for g in range(n_kv):
        for simd in (False, True):
            kf2, vf2 = ref.block_f32(kvt, kl, vl, n_kv, hd, g, 1, 16, simd=simd)
            if kf2 is None:
                continue
            kf, vf = port.block_f32(kvt, kl, vl, n_kv, hd, g, 1, 16)
            assert beq(kf, kf2) and beq(vf, vf2)
    q = synth.normal(9, (9, n_heads, hd * (2 if gated else 1)))
    npr = np.array([1, 15, 16, 17, 255, 256, 257, 513, 700], np.int32)
    want = port.attention(kvt, kl, vl, n_kv, n_heads, hd, q, npr, gated=gated)
    for split in (0, 1):
        for rpi in (0, 1, 3):
            assert beq(ref.attention(kvt, kl, vl, n_kv, n_heads, hd, q, npr, gated=gated, split=split, rows_per_item=rpi), want)
    assert beq(ref.q_rot(kvt, q[0, 0, :hd], hd), port.q_rot(kvt, q[0, 0, :hd], hd))
    assert beq(ref.o_unrot(kvt, q[0, 0, :hd], hd), port.o_unrot(kvt, q[0, 0, :hd], hd))


@pytest.mark.parametrize("which", ["ref", "ref-v4", "ref-generic"])
def test_deltanet_pinned(which):
    ref, port = gwo.load(which), gwo.load("port")
    if ref is None:
        pytest.skip("oracle/_ref not built")
    nk, nv, dk, dv = 2, 4, 128, 128
    cd = 2 * nk * dk + nv * dv
    w = [synth.normal(11, (cd * 4,)) * np.float32(0.5), -np.abs(synth.normal(12, (nv,))) - np.float32(0.1), synth.normal(13, (nv,)),
         synth.normal(14, (dv,))]
    res = []
    for o in (port, ref):
        d = gwo.DeltaNet(o, nk, nv, dk, dv, 4, *w)
        st = d.new_state()
        raw = synth.normal(15, (40, d.lw))
        p1 = d.prep(st, raw, True)
        r1 = d.rec(st, p1, True)
        f1 = d.out(p1, r1)
        p2 = d.prep(st, raw[:7], False)
        r2 = d.rec(st, p2, False)
        res.append((p1, r1, f1, p2, r2, st.copy()))
    for a, b in zip(*res):
        assert beq(a, b)


@pytest.mark.parametrize("which", ["ref", "ref-v4", "ref-generic"])
def test_activation_quantiser_pinned(which):
    ref, port = gwo.load(which), gwo.load("port")
    if ref is None:
        pytest.skip("oracle/_ref not built")
    x = synth.normal(77, (64, 512)) * np.float32(0.03)
    x[3, :64] = 0.0          # an all-zero group
    x[5, 7] = 1e-30          # a tiny maximum
    x[9, 100] = 5.0e4
    for gs in (32, 64, 128, 256):
        q1, s1 = port.quantize(x, gs)
        q2, s2 = ref.quantize(x, gs)
        assert np.array_equal(q1, q2) and beq(s1, s2), gs
