// The tensor-core decode attention kernels for 8-bit KV caches and their launcher (one translation unit of their own).
#define RQ_ATTN_DECODE_TC_INSTANTIATE
#include "attn_decode_tc.cuh"
