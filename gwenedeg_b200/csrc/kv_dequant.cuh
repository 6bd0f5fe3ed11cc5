// Prompt passes over quantised KV caches (q8, q4, q4k4) on the tensor-core prefill kernel: the layer's cached tiles of every
// segment of the pass are expanded once per layer call into f16 tiles of the f16 cache's own layout (a scratch that the
// prefill kernel reads through tensor maps exactly as it reads an f16 cache), the query rows are rotated as the reference
// rotates them for these cache types (att_q_rot, src/forward.c:1662), and the merge kernel un-rotates the outputs.
//
// The expansion is the reference's dequantisation (block_f32 of src/forward.c:1770-1804: value = level x bf16 scale, exact in
// fp32) followed by one rounding to f16, which is what puts this path at tolerance parity (~3e-4 relative) instead of bit
// parity; the row-by-row path through the decode kernels stays for hosts that select exact results.
#pragma once
#include "attn_decode.cuh"

namespace rq {

struct DqSeg {
    const uint8_t *k, *v;         // the segment's sequence: K / V cache of layer 0
    unsigned long long lk, lv;    // bytes from one layer to the next
    uint8_t *ko, *vo;             // the f16 tiles of the segment in the scratch: [block][KV head][16 tiles] of 16 positions x head_dim
    int len;                      // positions to expand: 0 .. len - 1 (the rest of the last block is zero-filled)
    int tiles;                    // tiles per KV head: 16 x blocks
};

__device__ __forceinline__ uint32_t f16x2_sat(float a, float b) {
    // (finite results only: an infinity in the f16 tiles would turn a masked key's zero weight into a NaN)
    const __half2 h = __floats2half2_rn(fminf(fmaxf(a, -65504.0f), 65504.0f), fminf(fmaxf(b, -65504.0f), 65504.0f));
    return *reinterpret_cast<const uint32_t *>(&h);
}
// 16 cached levels (one 16-byte word: int8, or the low / high nibbles of 16 bytes) times their scales, as 16 halves
template <int FMT>
__device__ __forceinline__ void levels16_to_f16(uint4 w, int hi_nibble, const float *d, bool one_scale, uint4 *dst) {
    uint32_t x[4] = {w.x, w.y, w.z, w.w}, out[8];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        float f[4];
        if constexpr (FMT == KV_Q8) {
            const uint32_t fl = x[k] ^ 0x80808080u;
#pragma unroll
            for (int b = 0; b < 4; b++) f[b] = s8_to_f32(fl, b);
        } else {
            const uint32_t nb = (x[k] >> (4 * hi_nibble)) & 0x0F0F0F0Fu;
#pragma unroll
            for (int b = 0; b < 4; b++) f[b] = __uint_as_float(__byte_perm(nb, 0x4B000000u, 0x7540 | b)) - 8388616.0f;  // 2^23 + 8
        }
#pragma unroll
        for (int b = 0; b < 4; b++) f[b] = __fmul_rn(f[b], one_scale ? d[0] : d[4 * k + b]);
        out[2 * k] = f16x2_sat(f[0], f[1]);
        out[2 * k + 1] = f16x2_sat(f[2], f[3]);
    }
    dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
    dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
}

// The query vector of one (row, head) rotated as att_q_rot does for the quantised cache types (signs, butterflies h = 1, 2,
// 4, ..., scaling by 1 / head_dim), fp32, by one warp: lane L holds dims 4L .. 4L + 3 of every 128-dim part.
template <int HD>
__device__ __forceinline__ void q_rot_warp(const float *__restrict__ q, int qh, size_t wi, float *__restrict__ qr, int lane) {
    constexpr int NP = HD / 128;
    float4 x[NP];
#pragma unroll
    for (int c = 0; c < NP; c++) {
        x[c] = *reinterpret_cast<const float4 *>(q + wi * qh + 128 * c + 4 * lane);
        const int i = 128 * c + 4 * lane;
        x[c].x = kvq_neg(i) ? -x[c].x : x[c].x, x[c].y = kvq_neg(i + 1) ? -x[c].y : x[c].y;
        x[c].z = kvq_neg(i + 2) ? -x[c].z : x[c].z, x[c].w = kvq_neg(i + 3) ? -x[c].w : x[c].w;
    }
    fwht_warp<NP>(x, lane);
    const float f = 1.0f / (float)HD;
#pragma unroll
    for (int c = 0; c < NP; c++)
        *reinterpret_cast<float4 *>(qr + wi * HD + 128 * c + 4 * lane) = make_float4(x[c].x * f, x[c].y * f, x[c].z * f, x[c].w * f);
}

// One CTA of head_dim threads per (tile of 16 positions, KV head, segment).  K: thread = dim (its 16 positions: one 16-byte word
// of levels in, one 32-byte row of the f16 tile out); V: thread = (position, 16 dims of one scale group).
// The grid's z slices past the segments rotate the pass's query rows (q [rows][n_heads][qh] -> qr [rows][n_heads][head_dim]), a
// warp per (row, head): the two jobs are independent, and one launch saves the second one's turn on the stream.
template <int KVT, int HD>
__global__ void __launch_bounds__(HD) kv_dequant_f16_kernel(const DqSeg *__restrict__ segs, int n_segs, int layer, int n_kv, const float *__restrict__ q,
                                                            int qh, int n_rows_heads, float *__restrict__ qr) {
    constexpr int KF = kv_fmt(KVT, 0), VF = kv_fmt(KVT, 1);
    constexpr int KTB = kv_tile_bytes(KVT, HD, 0), VTB = kv_tile_bytes(KVT, HD, 1);
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.z >= n_segs) {
        const size_t wi = ((((size_t)blockIdx.z - n_segs) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * (HD / 32) + (threadIdx.x >> 5);
        if (wi < (size_t)n_rows_heads) q_rot_warp<HD>(q, qh, wi, qr, threadIdx.x & 31);
        return;
    }
    const DqSeg sg = segs[blockIdx.z];
    const int u = blockIdx.x, g = blockIdx.y, tid = threadIdx.x;  // tile of the segment (of this head), head
    if (u >= sg.tiles) return;
    const size_t tile = ((size_t)(u / ATT_PT) * n_kv + g) * ATT_PT + (u % ATT_PT);  // [block][head][tile of the block]
    const uint8_t *kt = sg.k + (size_t)layer * sg.lk + tile * KTB, *vt = sg.v + (size_t)layer * sg.lv + tile * VTB;
    uint8_t *ko = sg.ko + tile * (size_t)(HD * 32), *vo = sg.vo + tile * (size_t)(HD * 32);
    const int p0 = u * ATT_T;  // first position of the tile
    const int live = min(max(sg.len - p0, 0), 16);  // positions of the tile to expand; the others become zeros
    {  // K: dim tid, positions p0 .. p0 + 15.  q8: [dim][16 positions]; 4-bit: [dim pair][16 positions], low nibble the even dim
        const uint4 w = *reinterpret_cast<const uint4 *>(kt + (size_t)(KF == KV_Q8 ? tid : tid >> 1) * 16);
        const uint4 *sp = reinterpret_cast<const uint4 *>(kt + (KF == KV_Q8 ? 16 : 8) * HD + (tid >> 5) * 32);  // [group][16 positions] bf16
        const uint4 s0 = sp[0], s1 = sp[1];
        const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        float d[16];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            d[2 * j] = 2 * j < live ? __uint_as_float(sw[j] << 16) : 0.0f;
            d[2 * j + 1] = 2 * j + 1 < live ? __uint_as_float(sw[j] & 0xffff0000u) : 0.0f;
        }
        levels16_to_f16<KF>(w, tid & 1, d, false, reinterpret_cast<uint4 *>(ko + (size_t)tid * 32));
    }
    {  // V: position tid / (head_dim / 16), 16 dims.  q8: [position][head_dim]; 4-bit: per position and group 16 bytes, byte l =
       // dims 32 c + l (low nibble) and 32 c + 16 + l (high)
        constexpr int PCS = HD / 16;  // 16-dim pieces of a position
        const int j = tid / PCS, i0 = (tid % PCS) * 16, c = i0 >> 5;
        const uint4 w = *reinterpret_cast<const uint4 *>(VF == KV_Q8 ? vt + (size_t)j * HD + i0 : vt + (size_t)j * (HD / 2) + c * 16);
        float d = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(vt + (VF == KV_Q8 ? 16 : 8) * HD + (j * (HD / 32) + c) * 2));
        if (j >= live) d = 0.0f;
        levels16_to_f16<VF>(w, (i0 >> 4) & 1, &d, true, reinterpret_cast<uint4 *>(vo + ((size_t)j * HD + i0) * 2));
    }
}

}  // namespace rq
