"""The CPU checkers against the committed fixtures (generated from the reference's own build by
tests/golden/make_golden.py): the plain-C restatement always, the reference builds when present.  Bit-exact."""
import glob
import hashlib
import os

import numpy as np
import pytest

from gwenedeg_b200 import synth
from oracle import gwo
from tests.golden.make_golden import ATTN_CASES, CONTEXTS, attn_inputs, scalar_inputs

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def checkers():
    out = [("port", gwo.load("port"))]
    for w in ("ref", "ref-v4", "ref-generic"):
        o = gwo.load(w)
        if o is not None:
            out.append((w, o))
    return out


def beq(a, b):
    return np.array_equal(np.ascontiguousarray(a, np.float32).view(np.uint32), np.ascontiguousarray(b, np.float32).view(np.uint32))


def test_fixture_files_present():
    assert len(glob.glob(os.path.join(G, "attn_*.npz"))) == len(ATTN_CASES)


@pytest.mark.parametrize("case", ATTN_CASES, ids=[c[0] for c in ATTN_CASES])
def test_attention_fixture(case):
    name, kvt, n_heads, n_kv, hd, gated = case
    fx = np.load(os.path.join(G, f"attn_{name}.npz"))
    seed = int(fx["shape"][5])
    k, v, q = attn_inputs(seed, n_heads, n_kv, hd, gated)
    port = gwo.load("port")
    kl, vl = port.new_cache(kvt, 512, n_kv, hd)
    port.kv_store(kvt, kl, vl, 0, k, v, n_kv, hd)
    assert digest(kl) == str(fx["k_digest"]) and digest(vl) == str(fx["v_digest"])
    for who, o in checkers():
        for split in (0, 1):
            out = o.attention(kvt, kl, vl, n_kv, n_heads, hd, q, CONTEXTS, gated=gated, split=split)
            assert beq(out, fx["out"]), (who, split)
        kf, vf = o.block_f32(kvt, kl, vl, n_kv, hd, n_kv - 1, 1, 3)
        assert digest(kf) == str(fx["kf_digest"]) and digest(vf) == str(fx["vf_digest"]), who


def test_scalar_fixture():
    fx = np.load(os.path.join(G, "scalars.npz"))
    x, f = scalar_inputs()
    h = np.arange(65536, dtype=np.uint16)
    for who, o in checkers():
        assert beq(o.exp_att(x), fx["exp_y"]), who
        assert beq(o.sigmoid(x + np.float32(50)), fx["sig_y"]), who
        assert digest(o.f32_f16(f)) == str(fx["half_digest"]), who
        assert digest(o.f16_f32(h)) == str(fx["f16_f32_digest"]), who


def test_half_conversion_edge_cases():
    port = gwo.load("port")
    f = np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, np.inf, 2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -25, 1.0009765625 + 2.0 ** -11],
                 np.float32)
    want = np.array([0x0000, 0x8000, 0x7bff, 0x7bff, 0x7bff, 0x7bff, 0xfbff, 0x7bff, 0x0001, 0x0000, 0x0002, 0x3c02], np.uint16)
    assert np.array_equal(port.f32_f16(f), want)
    assert (port.f32_f16(np.array([np.nan], np.float32))[0] & 0x7e00) == 0x7e00


def test_deltanet_fixture():
    fx = np.load(os.path.join(G, "deltanet_nk1_nv2.npz"))
    for who, o in checkers():
        d = gwo.DeltaNet(o, 1, 2, 128, 128, 4, fx["w_conv"], fx["w_a"], fx["w_dt"], fx["w_norm"])
        st = d.new_state()
        prep = d.prep(st, fx["raw"], True)
        assert digest(prep) == str(fx["prep_digest"]), who
        rec = d.rec(st, prep, True)
        assert beq(rec, fx["rec"]), who
        assert beq(d.out(prep, rec), fx["fin"]), who
        assert beq(d.rec(st, prep[:5], False), fx["rec2"]), who
        assert digest(st) == str(fx["state_digest"]), who
    fx = np.load(os.path.join(G, "deltanet_rec_nk2_nv4.npz"))
    for who, o in checkers():
        d = gwo.DeltaNet(o, 2, 4, 128, 128)
        st = d.new_state()
        assert beq(d.rec(st, fx["rows"], True), fx["out"]), who
        assert digest(st) == str(fx["state_digest"]), who


def test_deltanet_matches_float64_matrix_form():
    """Independent cross-check of the recurrence: S <- eg S + beta k (v - eg S^T k)^T, o = S^T q in float64."""
    port = gwo.load("port")
    nk, nv, dk, dv, n = 2, 4, 128, 128, 30
    rows = synth.deltanet_rows(4, n, nk, nv, dk, dv)
    d = gwo.DeltaNet(port, nk, nv, dk, dv)
    st = d.new_state()
    got = d.rec(st, rows, True)
    S = np.zeros((nv, dk, dv))
    want = np.zeros((n, nv * dv))
    for t in range(n):
        r = rows[t].astype(np.float64)
        for h in range(nv):
            kh = h % nk
            q, k = r[kh * dk:(kh + 1) * dk], r[nk * dk + kh * dk: nk * dk + (kh + 1) * dk]
            v = r[2 * nk * dk + h * dv: 2 * nk * dk + (h + 1) * dv]
            eg, beta = r[2 * nk * dk + 2 * nv * dv + h], r[2 * nk * dk + 2 * nv * dv + nv + h]
            S[h] *= eg
            S[h] += np.outer(k, (v - S[h].T @ k) * beta)
            want[t, h * dv:(h + 1) * dv] = S[h].T @ q
    assert np.abs(got - want).max() < 1e-6 and np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-5


def test_attention_matches_float64_softmax():
    """Independent cross-check of the attention definition against a plain float64 softmax on the dequantised cache."""
    port = gwo.load("port")
    kvt, n_heads, n_kv, hd, n = gwo.Q8, 4, 2, 128, 600
    k, v = synth.normal(1, (n, n_kv, hd)), synth.normal(2, (n, n_kv, hd))
    q = synth.normal(3, (2, n_heads, hd))
    kl, vl = port.new_cache(kvt, 768, n_kv, hd)
    port.kv_store(kvt, kl, vl, 0, k, v, n_kv, hd)
    got = port.attention(kvt, kl, vl, n_kv, n_heads, hd, q, np.array([n, 257], np.int32))
    for r, npos in enumerate((n, 257)):
        for h in range(n_heads):
            g = h // (n_heads // n_kv)
            K = np.zeros((npos, hd))
            V = np.zeros((npos, hd))
            for b in range((npos + 255) // 256):
                kf, vf = port.block_f32(kvt, kl, vl, n_kv, hd, g, b, 16)
                m = min(256, npos - b * 256)
                K[b * 256:b * 256 + m] = kf.transpose(0, 2, 1).reshape(256, hd)[:m]
                V[b * 256:b * 256 + m] = vf.reshape(256, hd)[:m]
            qr = port.q_rot(kvt, q[r, h], hd).astype(np.float64)
            s = K @ qr / np.sqrt(hd)
            p = np.exp(s - s.max())
            o = (p / p.sum()) @ V
            o = port.o_unrot(kvt, o.astype(np.float32), hd)
            assert np.abs(got[r, h] - o).max() < 2e-5
    # and the rotation is orthogonal up to the scaling: attention on the rotated pair equals attention on the originals
    want = gwo.load("port").attention(gwo.F32, *f32_cache(port, k, v, n_kv, hd), n_kv, n_heads, hd, q, np.array([n, 257], np.int32))
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 2e-2  # (8-bit quantisation error only)


def f32_cache(port, k, v, n_kv, hd):
    kl, vl = port.new_cache(gwo.F32, 768, n_kv, hd)
    port.kv_store(gwo.F32, kl, vl, 0, k, v, n_kv, hd)
    return kl, vl
