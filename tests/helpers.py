"""Shared pieces of the parity tests: the error metrics of the acceptance bar and cache builders."""
import numpy as np

from gwenedeg_b200 import synth

MAX_ABS = 2e-3   # acceptance bar on fp32 outputs: max |gpu - cpu|
REL_L2 = 1e-3    # and ||gpu - cpu|| / ||cpu||


def errors(got, want):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.abs(got - want).max()), float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def assert_close(got, want, what=""):
    """The stated tolerance, overall and per row (outputs are small, so the relative bar is the binding one)."""
    ma, rl = errors(got, want)
    assert ma <= MAX_ABS and rl <= REL_L2, f"{what}: max-abs {ma:.3g}, rel-L2 {rl:.3g}"
    g2 = np.asarray(got).reshape(got.shape[0], -1)
    w2 = np.asarray(want).reshape(want.shape[0], -1)
    for r in range(g2.shape[0]):
        _, rr = errors(g2[r], w2[r])
        assert rr <= 4 * REL_L2, f"{what}: row {r} rel-L2 {rr:.3g}"


def bit_equal(a, b):
    return np.array_equal(np.ascontiguousarray(a, np.float32).view(np.uint32), np.ascontiguousarray(b, np.float32).view(np.uint32))


def kv_rows(seed, n, n_kv, hd, outlier=True):
    k = synth.normal(seed * 2 + 1, (n, n_kv, hd))
    v = synth.normal(seed * 2 + 2, (n, n_kv, hd))
    if outlier and n > 5:
        k[5, 0, 3] = 300.0   # the reference's K has a few large dims; exercises the f16 range and the q8 scales
        v[3, 0, 1] = 70000.0  # saturates to 65504 in an f16 cache
    return k, v


def oracle_cache(orc, kvt, n_kv, hd, k, v):
    """The layer cache the CPU code builds from rows k, v stored at positions 0..n-1."""
    n = k.shape[0]
    kv_len = (n + 255) // 256 * 256
    kl, vl = orc.new_cache(kvt, kv_len, n_kv, hd)
    orc.kv_store(kvt, kl, vl, 0, k, v, n_kv, hd)
    return kl, vl
