// The tensor-core decode attention kernels for quantised KV caches and their launchers (one translation unit of their own).
#define RQ_ATTN_DECODE_TC_INSTANTIATE
#include "attn_decode_tc.cuh"

namespace rq {
template cudaError_t launch_attn_part_tc<KV_Q8>(const AttnPartTcArgs &, cudaStream_t);
template cudaError_t launch_attn_part_tc<KV_Q4>(const AttnPartTcArgs &, cudaStream_t);
template cudaError_t launch_attn_part_tc<KV_Q4K4>(const AttnPartTcArgs &, cudaStream_t);
}  // namespace rq
