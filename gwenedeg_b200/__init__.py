"""gwenedeg's attention hot path on NVIDIA B200: a ctypes host layer over librq_cuda.so (include/rq_cuda.h).

Importing the package loads the CUDA library and raises ImportError when it has not been built; nothing here
computes attention on the CPU.
"""
from . import _lib
from .api import (KV_F16, KV_NAMES, KV_Q4, KV_Q4K4, KV_Q8, Context, RqCudaError, Sequence, device_count)  # noqa: F401

_lib.load()
