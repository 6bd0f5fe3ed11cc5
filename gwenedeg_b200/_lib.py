"""ctypes declarations of librq_cuda.so, one per prototype of include/rq_cuda.h.

The shared library is the product; this module only loads it.  There is no fallback of any kind: a missing
library is an ImportError naming the build command, and a machine without a B200 makes rq_cuda_init fail with
RQ_CUDA_ERR_DEVICE.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# RQ_CUDA_LIB selects another build of the same library (the debug build with index checks: librq_cuda_debug.so)
LIB_PATH = os.environ.get("RQ_CUDA_LIB") or os.path.join(HERE, "librq_cuda.so")

OK, ERR_ARG, ERR_NOMEM, ERR_CONTEXT, ERR_STATE, ERR_IO, ERR_MISMATCH, ERR_DEVICE = 0, -1, -2, -3, -4, -6, -7, -16
KV_F32, KV_F16, KV_Q8, KV_Q4, KV_Q4K4 = 0, 2, 3, 8, 9
KV_NAMES = {"f16": KV_F16, "q8": KV_Q8, "q4": KV_Q4, "q4k4": KV_Q4K4}


class RqCudaModel(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "n_attn", "n_heads", "n_kv_heads", "head_dim", "gated", "n_lin", "dn_nk", "dn_nv", "dn_dk", "dn_dv", "dn_conv",
        "kv_head0", "kv_heads_local")]


class RqCudaPassTime(C.Structure):
    _fields_ = [("seconds", C.c_double), ("rows", C.c_int), ("pos_first", C.c_double), ("pos_more", C.c_double)]


class RqCudaSegment(C.Structure):
    _fields_ = [("seq", C.c_void_p), ("pos0", C.c_int), ("n", C.c_int)]


_vp, _i, _sz, _ull = C.c_void_p, C.c_int, C.c_size_t, C.c_ulonglong
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); kept in the order of the header
PROTOTYPES = {
    "rq_cuda_init": (_i, [_i, C.POINTER(RqCudaModel), _i, _pp]),
    "rq_cuda_free": (None, [_vp]),
    "rq_cuda_error": (C.c_char_p, [_vp]),
    "rq_cuda_device_count": (_i, []),
    "rq_cuda_debug_build": (_i, []),
    "rq_cuda_sync": (_i, [_vp]),
    "rq_cuda_reserve": (_i, [_vp, _i, C.c_longlong, _i]),
    "rq_cuda_selftest_wait_expiry": (_i, [_vp, C.c_uint]),
    "rq_cuda_peer_export": (_i, [_vp, _i, _vp]),
    "rq_cuda_peer_import": (_i, [_vp, _i, _i, _vp]),
    "rq_cuda_attn_decode_gather_dev": (_i, [_vp, _i, _vp, C.POINTER(_vp)]),
    "rq_cuda_selftest_peer_wait": (_i, [_vp, C.c_uint]),
    "rq_cuda_set_wo_quant": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_set_exact": (_i, [_vp, _i]),
    "rq_cuda_set_prefill_split": (_i, [_vp, _i]),
    "rq_cuda_set_stream": (_i, [_vp, _vp]),
    "rq_cuda_seq_new": (_i, [_vp, _i, _i, _pp]),
    "rq_cuda_seq_free": (None, [_vp]),
    "rq_cuda_seq_len": (_i, [_vp]),
    "rq_cuda_seq_capacity": (_i, [_vp]),
    "rq_cuda_seq_truncate": (_i, [_vp, _i]),
    "rq_cuda_seq_copy": (_i, [_vp, _vp, _i]),
    "rq_cuda_seq_layer_bytes": (_sz, [_vp, _i]),
    "rq_cuda_seq_read_kv": (_i, [_vp, _i, _i, _vp, _sz]),
    "rq_cuda_seq_write_kv": (_i, [_vp, _i, _i, _vp, _sz, _i]),
    "rq_cuda_seq_state_floats": (_sz, [_vp]),
    "rq_cuda_seq_read_state": (_i, [_vp, _i, _vp]),
    "rq_cuda_seq_write_state": (_i, [_vp, _i, _vp]),
    "rq_cuda_seq_set_checkpoints": (_i, [_vp, _i]),
    "rq_cuda_seq_checkpoint_pos": (_i, [_vp, _i]),
    "rq_cuda_seq_restore": (_i, [_vp, _i]),
    "rq_cuda_seq_checkpoint_drop": (_i, [_vp, _i]),
    "rq_cuda_seq_read_checkpoint": (_i, [_vp, _i, _i, _vp]),
    "rq_cuda_seq_write_checkpoint": (_i, [_vp, _i, _i, _vp, _i]),
    "rq_cuda_seq_save_bytes": (C.c_longlong, [_vp]),
    "rq_cuda_seq_save": (_i, [_vp, C.c_char_p, _vp, _ull, _ull]),
    "rq_cuda_seq_load": (_i, [_vp, C.c_char_p, _ull, _i, _vp, C.POINTER(_ull)]),
    "rq_cuda_seq_fill_synthetic": (_i, [_vp, _i, _ull]),
    "rq_cuda_pass_begin": (_i, [_vp, C.POINTER(RqCudaSegment), _i]),
    "rq_cuda_pass_checkpoint": (_i, [_vp, _i, _i, _i]),
    "rq_cuda_pass_end": (_i, [_vp, _i]),
    "rq_cuda_pass_timing": (_i, [_vp, _i]),
    "rq_cuda_pass_time": (_i, [_vp, C.POINTER(RqCudaPassTime)]),
    "rq_cuda_pass_cost_measure": (_i, [_vp, _vp, _i, _i, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "rq_cuda_kv_store": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_kv_store_dev": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_qk_norm_rope_store_dev": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _i, C.c_float]),
    "rq_cuda_attn_decode": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_attn_decode_dev": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_attn_decode_noalloc": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_attn_decode_noalloc_max_bytes": (_sz, []),
    "rq_cuda_attn_prefill": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_attn_prefill_dev": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_dn_rec": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_dn_rec_dev": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_dn_chunk": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_dn_chunk_dev": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_dn_set_weights": (_i, [_vp, _i, _vp, _vp, _vp, _vp]),
    "rq_cuda_dn_prep_dev": (_i, [_vp, _i, _vp]),
    "rq_cuda_dn_out_dev": (_i, [_vp, _i, _vp, _vp]),
    "rq_cuda_malloc": (_i, [_vp, _sz, _pp]),
    "rq_cuda_mfree": (_i, [_vp, _vp]),
    "rq_cuda_malloc_host": (_i, [_vp, _sz, _pp]),
    "rq_cuda_mfree_host": (_i, [_vp, _vp]),
    "rq_cuda_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "rq_cuda_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "rq_cuda_mem_info": (_i, [_vp, C.POINTER(_sz), C.POINTER(_sz)]),
    "rq_cuda_timer_start": (_i, [_vp]),
    "rq_cuda_timer_stop": (_i, [_vp, C.POINTER(C.c_float)]),
    "rq_cuda_launch_count": (_ull, [_vp]),
    "rq_cuda_profile_begin": (_i, [_vp, _i]),
    "rq_cuda_profile_end": (_i, [_vp, C.POINTER(C.c_float), C.POINTER(_i)]),
}

_lib = None


def load():
    """The loaded library (ctypes.CDLL) with every prototype declared."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(HERE, 'csrc')}` "
            "(or python -c 'import __graft_entry__ as g; g.build()'); there is no fallback implementation")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
