"""Seeded synthetic inputs for the attention path (stand-ins for a real model's rows and caches).

Everything is derived from a counter-based integer hash (splitmix64), so the same (seed, shape) gives the same
bits on every machine and numpy version: the golden fixtures under tests/golden/ depend on that.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix(z):
    z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def bits(seed, n):
    """n 64-bit words of stream `seed`."""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64)
        return _mix(idx * np.uint64(0xD6E8FEB86659FD93) + _mix(np.uint64(seed)))


def uniform(seed, shape):
    """float32 uniform in [0, 1) with 24 random bits."""
    n = int(np.prod(shape))
    return ((bits(seed, n) >> np.uint64(40)).astype(np.float64) * 2.0 ** -24).astype(np.float32).reshape(shape)


def normal(seed, shape):
    """float32 ~N(0, 1) as a centred sum of twelve 21-bit uniforms (Irwin-Hall): only exact float64 additions of
    dyadic fractions, so the bits are the same everywhere (no libm call); tails end at +-6."""
    n = int(np.prod(shape))
    acc = np.zeros(n, np.float64)
    m21 = np.uint64((1 << 21) - 1)
    with np.errstate(over="ignore"):
        for r in range(4):
            b = bits((np.uint64(seed) * np.uint64(4) + np.uint64(r)) & _M64, n)
            for f in range(3):
                acc += ((b >> np.uint64(21 * f)) & m21).astype(np.float64) * 2.0 ** -21
    return (acc - 6.0).astype(np.float32).reshape(shape)


def integers(seed, lo, hi, shape):
    """int64 uniform in [lo, hi]."""
    n = int(np.prod(shape))
    return (lo + (bits(seed, n) >> np.uint64(11)) % np.uint64(hi - lo + 1)).astype(np.int64).reshape(shape)


def ragged_contexts(seed, n, lo=512, hi=32768):
    """Per-sequence context lengths of the continuous-batch decode workload: uniform in [lo, hi]."""
    return integers(seed, lo, hi, (n,)).astype(np.int32)


def deltanet_rows(seed, n, nk, nv, dk, dv):
    """Post-prep Gated DeltaNet rows [n][lw], lw = 2 nk dk + 2 nv dv + 2 nv laid out [q | k | v | z | eg | beta]:
    q, k ~N(0,1) L2-normalised per head (q also times 1/sqrt(dk)), v, z ~N(0,1),
    eg = exp(-softplus(N(0,1))), beta = sigmoid(N(0,1))."""
    q = normal(seed * 8 + 1, (n, nk, dk)).astype(np.float64)
    k = normal(seed * 8 + 2, (n, nk, dk)).astype(np.float64)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) / np.sqrt(dk)
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    v = normal(seed * 8 + 3, (n, nv * dv))
    z = normal(seed * 8 + 4, (n, nv * dv))
    a = normal(seed * 8 + 5, (n, nv)).astype(np.float64)
    b = normal(seed * 8 + 6, (n, nv)).astype(np.float64)
    eg = np.exp(-np.log1p(np.exp(a)))
    beta = 1.0 / (1.0 + np.exp(-b))
    return np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v, z, eg, beta], axis=1).astype(np.float32)
