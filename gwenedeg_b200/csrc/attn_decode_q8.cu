// Instantiates the split-K decode attention kernels for the Q8 KV cache type (one translation unit per type so the
// library builds in parallel).
#define RQ_ATTN_DECODE_INSTANTIATE
#include "attn_decode.cuh"

namespace rq {
template cudaError_t launch_attn_part<KV_Q8>(int, const AttnPartArgs &, cudaStream_t);
template size_t attn_part_smem<KV_Q8>(int, int);
}  // namespace rq
