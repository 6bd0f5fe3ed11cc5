// The tensor-core prefill attention kernels (head_dim 128 and 256) and their launchers (one translation unit of their own).
#define RQ_ATTN_PREFILL_INSTANTIATE
#include "attn_prefill256.cuh"
