"""The C-ABI library loads on a machine without a GPU, exports every function include/rq_cuda.h declares, the ctypes
table names exactly those, and the entry points refuse to work without a device instead of falling back."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_functions():
    src = open(os.path.join(ROOT, "include", "rq_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(rq_cuda_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_function():
    from gwenedeg_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = header_functions()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in rq_cuda.h but not exported"
    assert sorted(_lib.PROTOTYPES) == names


def test_no_device_means_error_not_fallback():
    import gwenedeg_b200 as g
    if g.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(g.RqCudaError) as e:
        g.Context(0, n_attn=1, n_heads=4, n_kv_heads=2, head_dim=128)
    assert e.value.code == -16


def test_product_does_not_import_the_oracle():
    """The package and the CUDA sources never reference oracle/ (the checker is test infrastructure)."""
    for dirpath, _, files in os.walk(os.path.join(ROOT, "gwenedeg_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                txt = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in txt and "gwo" not in txt, f


def test_argument_checks_come_before_the_device():
    """Shapes the kernels cannot run are refused with RQ_CUDA_ERR_ARG whether or not a GPU is present: DeltaNet rows are
    read with 16-byte loads, so a row of 2 nk dk + 2 nv dv + 2 nv floats must be a multiple of four floats (an odd number
    of value heads is not)."""
    import gwenedeg_b200 as g
    for nk, nv in ((1, 1), (1, 3)):
        with pytest.raises(g.RqCudaError) as e:
            g.Context(0, n_lin=1, dn_nk=nk, dn_nv=nv)
        assert e.value.code == -1


def test_peer_entry_points_refuse_a_missing_context():
    """The fused-gather entry points check their arguments before anything else (no GPU needed to be told so)."""
    import ctypes as C
    import gwenedeg_b200 as g
    L = g._lib.load()
    buf = (C.c_ubyte * 128)()
    out = C.c_void_p()
    assert L.rq_cuda_peer_export(None, 4, C.cast(buf, C.c_void_p)) == -1
    assert L.rq_cuda_peer_import(None, 0, 2, C.cast(buf, C.c_void_p)) == -1
    assert L.rq_cuda_attn_decode_gather_dev(None, 0, C.cast(buf, C.c_void_p), C.byref(out)) == -1
    assert L.rq_cuda_selftest_peer_wait(None, 100) == -1


def test_reference_arm_of_the_benchmark_does_not_load_the_cuda_library():
    """bench.py --impl reference times the CPU code only: nothing on that path may import the package (whose import
    maps librq_cuda.so into the process)."""
    import subprocess
    import sys
    code = ("import sys, bench; ctx = bench.contexts(); cfg = bench.workload_config(ctx); "
            "assert len(ctx) == 64 and cfg['workload'] == 'qwen3-8b-decode-b64-ragged'; "
            "assert not any(m.startswith('gwenedeg_b200') for m in sys.modules), 'the package was imported'; "
            "assert 'librq_cuda' not in open('/proc/self/maps').read(), 'the CUDA library is mapped'")
    subprocess.check_call([sys.executable, "-c", code], cwd=ROOT)


@pytest.mark.gpu
def test_debug_build_with_index_checks_runs_the_small_cases():
    """librq_cuda_debug.so (-DRQ_DEBUG: every attention, merge, prefill and store CTA checks its work item against its row
    and cache and reports through the status word instead of touching memory) runs the small-context parity cases of the
    decode and prefill tests in a process of its own, with no check firing."""
    import subprocess
    import sys
    dbg = os.path.join(ROOT, "gwenedeg_b200", "librq_cuda_debug.so")
    assert os.path.exists(dbg), "make -C gwenedeg_b200/csrc debug"
    env = dict(os.environ, RQ_CUDA_LIB=dbg)
    probe = "import gwenedeg_b200 as g; assert g._lib.load().rq_cuda_debug_build() == 1"
    subprocess.check_call([sys.executable, "-c", probe], cwd=ROOT, env=env)
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider",
                        "tests/test_attn_decode_gpu.py::test_prompt_chunk_rows_match_cpu",
                        "tests/test_attn_decode_gpu.py::test_fill_synthetic_and_large_ragged_batch",
                        "tests/test_attn_decode_gpu.py::test_store_and_decode_match_cpu",
                        "tests/test_attn_decode_gpu.py::test_quantised_decode_on_tensor_cores_matches_cpu",
                        "tests/test_attn_prefill_gpu.py::test_head_dim_256_chunks_match_cpu",
                        "tests/test_attn_prefill_gpu.py::test_short_rows_and_mixed_segments"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
