"""Generates tests/golden/*.npz from the reference's own code (oracle/_ref, built by oracle/Makefile from the
reference's sources).  Run in a container that has the reference:  python tests/golden/make_golden.py

Inputs come from gwenedeg_b200.synth (integer hash + exact float64 sums: the same bits on any machine), so the fixtures
hold only outputs, cache digests and, for the DeltaNet cases, the rows (their gates use exp / log1p, which may differ in
the last bit between libm versions).
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from gwenedeg_b200 import synth  # noqa: E402
from oracle import gwo  # noqa: E402

ATTN_CASES = [
    # name, kvt, n_heads, n_kv, hd, gated
    ("f16_h4_kv2_d128", gwo.F16, 4, 2, 128, False),
    ("q8_h8_kv2_d128", gwo.Q8, 8, 2, 128, False),
    ("q4_h4_kv2_d128", gwo.Q4, 4, 2, 128, False),
    ("q4k4_h2_kv2_d64", gwo.Q4K4, 2, 2, 64, False),
    ("f16_h4_kv1_d256_gated", gwo.F16, 4, 1, 256, True),
    ("f32_h2_kv1_d64", gwo.F32, 2, 1, 64, False),
]
CONTEXTS = np.array([1, 15, 16, 17, 255, 256, 257, 300], np.int32)
N_POS = 300


def attn_inputs(seed, n_heads, n_kv, hd, gated):
    k = synth.normal(seed * 10 + 1, (N_POS, n_kv, hd))
    v = synth.normal(seed * 10 + 2, (N_POS, n_kv, hd))
    k[5, 0, 3] = 300.0
    q = synth.normal(seed * 10 + 3, (len(CONTEXTS), n_heads, hd * (2 if gated else 1)))
    return k, v, q


def scalar_inputs():
    x = np.concatenate([-(np.arange(6400, dtype=np.float32) / np.float32(64)), -(np.arange(1, 2000, dtype=np.float32) * np.float32(2.0 ** -20))])
    f = np.concatenate([synth.normal(77, (3000,)) * np.float32(s) for s in (2.0 ** -27, 2.0 ** -17, 2.0 ** -10, 1.0, 256.0, 65536.0)])
    f = np.concatenate([f, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, np.inf, -np.inf, 6e-8, 5.96e-8, 2.98e-8], np.float32)])
    return x.astype(np.float32), f.astype(np.float32)


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    ref = gwo.load("ref-generic")  # the portable build stores with its scalar code; the native one must agree below
    nat = gwo.load("ref")
    assert ref is not None and nat is not None, "build oracle/_ref first (make -C oracle ref)"
    for seed, (name, kvt, n_heads, n_kv, hd, gated) in enumerate(ATTN_CASES):
        k, v, q = attn_inputs(seed, n_heads, n_kv, hd, gated)
        port = gwo.load("port")
        kl, vl = port.new_cache(kvt, 512, n_kv, hd)
        port.kv_store(kvt, kl, vl, 0, k, v, n_kv, hd)  # the definition's bytes (IEEE division: the reference's -Ofast builds round exact ties differently)
        out = ref.attention(kvt, kl, vl, n_kv, n_heads, hd, q, CONTEXTS, gated=gated, split=0)
        for o in (nat.attention(kvt, kl, vl, n_kv, n_heads, hd, q, CONTEXTS, gated=gated, split=1),
                  ref.attention(kvt, kl, vl, n_kv, n_heads, hd, q, CONTEXTS, gated=gated, split=1)):
            assert np.array_equal(o.view(np.uint32), out.view(np.uint32)), name
        kf, vf = ref.block_f32(kvt, kl, vl, n_kv, hd, n_kv - 1, 1, 3)
        np.savez_compressed(os.path.join(HERE, f"attn_{name}.npz"), out=out, k_digest=digest(kl), v_digest=digest(vl),
                            kf_digest=digest(kf), vf_digest=digest(vf), contexts=CONTEXTS,
                            shape=np.array([kvt, n_heads, n_kv, hd, int(gated), seed], np.int32))
        print(name, float(np.sqrt((out ** 2).mean())))
    # scalar functions on exactly representable grids (no libm in the inputs)
    x, f = scalar_inputs()
    h = np.arange(65536, dtype=np.uint16)
    np.savez_compressed(os.path.join(HERE, "scalars.npz"), exp_y=nat.exp_att(x), sig_y=nat.sigmoid(x + np.float32(50)),
                        half_digest=digest(nat.f32_f16(f)), f16_f32_digest=digest(nat.f16_f32(h)))
    # Gated DeltaNet: prep, recurrence, output, continued across two calls
    nk, nv, dk, dv = 1, 2, 128, 128
    cd = 2 * nk * dk + nv * dv
    w_conv = synth.normal(301, (cd * 4,)) * np.float32(0.5)
    w_a = -np.exp(synth.normal(302, (nv,)).astype(np.float64)).astype(np.float32)
    w_dt = synth.normal(303, (nv,))
    w_norm = synth.normal(304, (dv,))
    d = gwo.DeltaNet(nat, nk, nv, dk, dv, 4, w_conv, w_a, w_dt, w_norm)
    raw = synth.normal(305, (16, d.lw))
    st = d.new_state()
    prep = d.prep(st, raw, True)
    rec = d.rec(st, prep, True)
    fin = d.out(prep, rec)
    rec2 = d.rec(st, prep[:5], False)
    np.savez_compressed(os.path.join(HERE, "deltanet_nk1_nv2.npz"), w_conv=w_conv, w_a=w_a, w_dt=w_dt, w_norm=w_norm, raw=raw,
                        prep_digest=digest(prep), rec=rec, fin=fin, rec2=rec2, state_digest=digest(st))
    # post-prep rows as the benchmark generates them (recurrence only)
    rows = synth.deltanet_rows(9, 12, 2, 4, dk, dv)
    d2 = gwo.DeltaNet(nat, 2, 4, dk, dv)
    st2 = d2.new_state()
    o2 = d2.rec(st2, rows, True)
    np.savez_compressed(os.path.join(HERE, "deltanet_rec_nk2_nv4.npz"), rows=rows, out=o2, state_digest=digest(st2))
    print("deltanet", float(np.sqrt((rec ** 2).mean())), float(np.sqrt((o2 ** 2).mean())))


if __name__ == "__main__":
    main()
