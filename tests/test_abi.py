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
