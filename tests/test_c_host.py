"""The boundary as a C host sees it: include/rq_cuda.h is valid C99, and a C99 program that drives the library the way
the integration notes describe for the reference's workers (tests/c_host/host_pass.c) compiles, links against
librq_cuda.so and, on a GPU, produces the CPU checker's results."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c_host", "host_pass.c")
BIN = os.path.join(ROOT, "tests", "c_host", "build", "host_pass")
LIBDIR = os.path.join(ROOT, "gwenedeg_b200")


def build_host():
    os.makedirs(os.path.dirname(BIN), exist_ok=True)
    subprocess.check_call(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", "-I", os.path.join(ROOT, "include"), SRC,
                           "-L", LIBDIR, "-lrq_cuda", "-Wl,-rpath," + LIBDIR, "-o", BIN])


def test_header_is_valid_c99():
    subprocess.check_call(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c",
                           os.path.join(ROOT, "include", "rq_cuda.h")])


def test_c_host_builds_and_links():
    build_host()
    import gwenedeg_b200 as g
    if g.device_count() > 0:
        pytest.skip("a GPU is present: the run is covered by the gpu test")
    r = subprocess.run([BIN, os.devnull], capture_output=True, text=True, timeout=120)
    assert r.returncode == 3 and "RQ_CUDA_ERR_DEVICE" in r.stdout, (r.returncode, r.stdout, r.stderr)


@pytest.mark.gpu
def test_c_host_results_match_cpu(checker):
    from tests.helpers import assert_close, bit_equal
    build_host()
    with tempfile.TemporaryDirectory() as d:
        out = os.path.join(d, "host_pass.bin")
        r = subprocess.run([BIN, out], capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, (r.stdout, r.stderr)
        raw = np.fromfile(out, np.uint8)
    hdr = raw[:36].view(np.int32)
    n_layers, n_heads, n_kv, hd, nseq = (int(x) for x in hdr[:5])
    ctx = [int(x) for x in hdr[5:8]]
    npre = int(hdr[8])
    fl = raw[36:].view(np.float32)
    at = 0

    def take(n):
        nonlocal at
        a = fl[at:at + n]
        at += n
        return a

    caches = []
    for n in ctx:
        k, v = take(n * n_kv * hd).reshape(n, n_kv, hd), take(n * n_kv * hd).reshape(n, n_kv, hd)
        kl, vl = checker.new_cache(2, (n + 255) // 256 * 256, n_kv, hd)
        checker.kv_store(2, kl, vl, 0, k, v, n_kv, hd)
        caches.append((kl, vl))
    q, got = take(nseq * n_heads * hd).reshape(nseq, n_heads, hd), take(nseq * n_heads * hd).reshape(nseq, n_heads, hd)
    pq, pgot = take(npre * n_heads * hd).reshape(npre, n_heads, hd), take(npre * n_heads * hd).reshape(npre, n_heads, hd)
    assert at == fl.size
    for i, n in enumerate(ctx):
        want = checker.attention(2, caches[i][0], caches[i][1], n_kv, n_heads, hd, q[i:i + 1], np.array([n], np.int32), split=1)
        assert bit_equal(got[i:i + 1], want), f"decode row of sequence {i}"
    # the prompt chunk of sequence 0: rows at positions ctx - npre .. ctx - 1 (tensor-core path: the tolerance)
    want = checker.attention(2, caches[0][0], caches[0][1], n_kv, n_heads, hd, pq, np.arange(ctx[0] - npre + 1, ctx[0] + 1, dtype=np.int32))
    assert_close(pgot, want, "prefill rows of the C host")
