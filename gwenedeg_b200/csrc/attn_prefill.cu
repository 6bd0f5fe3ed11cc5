// The tensor-core prefill attention kernel and its launcher (one translation unit of its own).
#define RQ_ATTN_PREFILL_INSTANTIATE
#include "attn_prefill.cuh"
