// Instantiates the split-K decode attention kernels for the F16 KV cache type (one translation unit per type so the
// library builds in parallel).
#define RQ_ATTN_DECODE_INSTANTIATE
#include "attn_decode.cuh"

namespace rq {
template cudaError_t launch_attn_part<KV_F16>(int, const AttnPartArgs &, cudaStream_t);
template size_t attn_part_smem<KV_F16>(int, int);
}  // namespace rq
