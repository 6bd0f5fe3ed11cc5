// Split-K decode attention over q8 / q4 / q4k4 KV caches on the tensor cores (tcgen05 + TMEM), head_dim 128: the fast form of
// attn_part_kernel for quantised caches.
//
// Same work items and the same partial results as attn_part_kernel (one (o, m, l) record per (row, KV head, block of 256
// positions), merged in block order by attn_combine_kernel, which also un-rotates and gates), so the split still
// depends on a row's own length only and a row of a batch gives the bits it gives alone.  What changes is the arithmetic
// inside a block.  The CUDA-core kernel spends ~8 instructions per cached level (conversion, scale, four multiply-adds);
// here a level costs ~1.3: the raw tiles arrive by bulk async copies (TMA) and all threads turn the levels into f16
// integers in the shared-memory layout of an MMA operand, with one byte permutation per two levels: the f16 pattern
// 0x6400 | b is exactly 1024 + b, where b = level + 128 (8-bit) or level + 8 (4-bit).  Neither the offset nor the scale is
// applied per level:
//   S_c^T [128 keys x 16]  = X_K [128 keys x dims of group c] Q^T     per 32-dim scale group c (four accumulators), then
//   s[t][v] = sum_c d_K[t][c] (S_c[t][v] - bias sum_{i in c} q[v][i])                 in the softmax thread of key t;
//   P_c[t][v] = p[t][v] d_V[t][c]  (f16), the four of them side by side as one N = 64 operand,
//   O^T [128 dims x 64] += X_V^T [128 dims x 128 keys] P^T,   W [128 x 64] += 1 [128 x 128 keys] P^T   (column sums),
//   o[i][v] = O[i][16 c(i) + v] - bias W[.][16 c(i) + v]                              in the epilogue thread of dim i.
// The offsets cancel in fp32 (the operands are exact integers and exact f16 weights; the products are exact in the
// tensor cores' fp32 accumulation), so the only roundings are q and the weights p d_V to f16: results agree with the
// reference's fp32 arithmetic to ~3e-4 relative, inside the acceptance bar but not bit for bit; the bit-exact kernel stays
// selectable (rq_cuda_set_exact).  With the keys on the TMEM lanes the softmax of a block is spread over all threads.
// The rotated query vectors are prepared once per (row, KV head) by tcd_q_prep_kernel (f16, operand layout, group sums)
// and fetched by every block's CTA with one bulk copy.
#pragma once
#include "attn_decode.cuh"
#include "tc05.cuh"

namespace rq {

constexpr int TCD_THREADS = 256;
constexpr int TCD_QT_BYTES = 4096 + 256;  // per (row, KV head): Q^T tile [16 vectors][128 dims] f16 + group sums [16][4] fp32

template <int KVT>
struct TcdCfg {
    static constexpr int HD = 128;
    static constexpr int KF = kv_fmt(KVT, 0), VF = kv_fmt(KVT, 1);
    static constexpr int KTB = kv_tile_bytes(KVT, HD, 0), VTB = kv_tile_bytes(KVT, HD, 1);
    static constexpr int KHALF = 8 * KTB, VHALF = 8 * VTB;  // raw bytes of half a block (8 tiles of 16 positions)
    // shared memory (from a 1024-byte aligned base): f16 operand buffer (32 KB: one half block of K, later of V) | Q^T and
    // the group sums (5 KB) | the all-ones operand (4 KB) | raw K half 0, K half 1, V half 0, V half 1 | P^T (32 KB: on top of
    // the raw K bytes where they are that large) | reductions, barriers, TMEM slot
    static constexpr int OP = 0, QT = 32768, ONES = QT + 5120, RAW = ONES + 4096;
    static constexpr int RAW_K0 = RAW, RAW_K1 = RAW_K0 + KHALF, RAW_V0 = RAW_K1 + KHALF, RAW_V1 = RAW_V0 + VHALF;
    static constexpr int RAW_END = (RAW_V1 + VHALF + 1023) / 1024 * 1024;
    static constexpr bool PT_ON_K = 2 * KHALF >= 32768;
    static constexpr int PT = PT_ON_K ? RAW_K0 : RAW_END;
    static constexpr int MISC = PT_ON_K ? RAW_END : RAW_END + 32768;  // red [2][8 warps][8] floats | bars [6] | TMEM slot
    static constexpr int SMEM = MISC + 512 + 64 + 16 + 1024;
    static_assert(RAW % 1024 == 0 && KHALF % 16 == 0 && VHALF % 16 == 0, "operand alignment; bulk copies are multiples of 16 bytes");
};

struct AttnPartTcArgs {
    const PassRow *rows;
    int nrows, total_blocks, layer, n_kv, G;
    const float *q;
    int qh, n_heads;
    float scale;
    float *part;
    uint8_t *qt;    // scratch: nrows x n_kv records of TCD_QT_BYTES
    int *blk2row;   // scratch: total_blocks ints
    int *err;
};
// launches tcd_q_prep_kernel and attn_part_tc_kernel<KVT> on `stream`; cudaErrorInvalidValue for an unsupported shape
template <int KVT>
cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_DECODE_TC_INSTANTIATE

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// The query vectors of one (row, KV head), once per pass and layer: rotated as att_q_rot does (reference src/forward.c:1662:
// signs, butterflies h = 1, 2, 4, ..., scaling by 1 / head_dim) in fp32, rounded to f16 and laid out as the B operand of
// S^T = X_K Q^T ([16 vectors][128 dims], K-major with the 128-byte swizzle, two k-blocks of 64 dims; rows past the G
// vectors zero), followed by the sums of the rounded values over each 32-dim group ([16][4] fp32): what the offset of the
// integer operands multiplies.  The CTA of KV head 0 also fills the block -> row table of its row.
__global__ void __launch_bounds__(128) tcd_q_prep_kernel(const PassRow *__restrict__ rows, int n_kv, int G, const float *__restrict__ q, int qh,
                                                         int n_heads, uint8_t *__restrict__ qt, int *__restrict__ blk2row) {
    constexpr int HD = 128;
    const int r = blockIdx.x, g = blockIdx.y, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float tmp[8][HD];
    __shared__ __half qh16[8][HD];
    const PassRow row = rows[r];
    if (g == 0) {
        const int nb = (row.np + ATT_P - 1) / ATT_P;
        for (int b = tid; b < nb; b += 128) blk2row[row.blk0 + b] = r;
    }
    const float *qrow = q + ((size_t)r * n_heads + (size_t)g * G) * qh;
    for (int v = 0; v < G; v++) {
        const float x = qrow[(size_t)v * qh + tid];
        tmp[v][tid] = kvq_neg(tid) ? -x : x;
    }
    __syncthreads();
    for (int hs = 1; hs < HD; hs <<= 1) {
        for (int e = tid; e < G * HD / 2; e += 128) {
            const int v = e / (HD / 2), p = e % (HD / 2);
            const int j = (p / hs) * 2 * hs + (p % hs);
            const float a = tmp[v][j], bb = tmp[v][j + hs];
            tmp[v][j] = a + bb;
            tmp[v][j + hs] = a - bb;
        }
        __syncthreads();
    }
    const float f = 1.0f / (float)HD;
    for (int v = 0; v < G; v++) qh16[v][tid] = __float2half_rn(tmp[v][tid] * f);
    __syncthreads();
    uint8_t *out = qt + ((size_t)r * n_kv + g) * TCD_QT_BYTES;
    for (int e = tid; e < 16 * 16; e += 128) {  // one 16-byte chunk (8 dims) of one row per step
        const int v = e >> 4, c16 = e & 15;
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (v < G) o = *reinterpret_cast<const uint4 *>(&qh16[v][c16 * 8]);
        *reinterpret_cast<uint4 *>(out + (c16 >> 3) * 2048 + v * 128 + (((c16 & 7) ^ (v & 7)) << 4)) = o;
    }
    if (tid < 64) {
        const int v = tid >> 2, c = tid & 3;
        float s = 0.0f;
        if (v < G)
            for (int i = 0; i < 32; i++) s += __half2float(qh16[v][32 * c + i]);
        reinterpret_cast<float *>(out + 4096)[tid] = s;
    }
}

// 16 bytes (each a level + offset, < 1024) -> 16 f16 integers 1024 + byte, as two 16-byte chunks
__device__ __forceinline__ void tcd_x16(const uint4 w, uint4 &c0, uint4 &c1) {
    c0 = make_uint4(__byte_perm(w.x, 0x64646464u, 0x4140), __byte_perm(w.x, 0x64646464u, 0x4342), __byte_perm(w.y, 0x64646464u, 0x4140),
                    __byte_perm(w.y, 0x64646464u, 0x4342));
    c1 = make_uint4(__byte_perm(w.z, 0x64646464u, 0x4140), __byte_perm(w.z, 0x64646464u, 0x4342), __byte_perm(w.w, 0x64646464u, 0x4140),
                    __byte_perm(w.w, 0x64646464u, 0x4342));
}
__device__ __forceinline__ uint4 tcd_xor(uint4 w, uint32_t m) { return make_uint4(w.x ^ m, w.y ^ m, w.z ^ m, w.w ^ m); }
__device__ __forceinline__ uint4 tcd_lo4(uint4 w) { return make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu); }
__device__ __forceinline__ uint4 tcd_hi4(uint4 w) {
    return make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

template <int KVT, int NVT>
__global__ void __launch_bounds__(TCD_THREADS) attn_part_tc_kernel(const PassRow *__restrict__ rows, const int *__restrict__ blk2row,
                                                                   const uint8_t *__restrict__ qtg, int layer, int n_kv, int G, int n_heads,
                                                                   float scale, float *__restrict__ part, int *err) {
    using C = TcdCfg<KVT>;
    constexpr int HD = C::HD, KF = C::KF, VF = C::VF;
    // TMEM: S_c^T of half h at 64 h + 16 c; O^T (the four groups' columns side by side) at 128; the column sums W at 192
    constexpr int TM_COLS = 256, S_COL = 0, O_COL = 128, W_COL = 192;
    constexpr float KBIAS = KF == KV_Q8 ? 1152.0f : 1032.0f, VBIAS = VF == KV_Q8 ? 1152.0f : 1032.0f;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *op = sm + C::OP, *pt = sm + C::PT;
    const float *qsum = reinterpret_cast<const float *>(sm + C::QT + 4096);  // [16][4]
    float *red = reinterpret_cast<float *>(sm + C::MISC);                    // [2][8][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + C::MISC + 512);       // raw K0, K1, V0, V1 and Q^T landed; MMAs complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + C::MISC + 512 + 64);
    uint64_t *bar_q = bars + 4, *bar_mma = bars + 5;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();

    const int lo = blk2row[blockIdx.x];
    const PassRow row = rows[lo];
    const int b = blockIdx.x - row.blk0, g = blockIdx.y;
    const int n = min(row.np - b * ATT_P, ATT_P);  // positions of this block
    const int ntl = (n + ATT_T - 1) / ATT_T;       // its tiles
    const int nh = (n + 127) >> 7;                 // its halves of 128 positions
    const size_t tile0 = ((size_t)b * n_kv + g) * ATT_PT;
    const uint8_t *kg = row.k + (size_t)layer * row.lk + tile0 * C::KTB;
    const uint8_t *vg = row.v + (size_t)layer * row.lv + tile0 * C::VTB;
    RQ_CHECK(lo >= 0 && b >= 0 && n >= 1 && g < n_kv && (tile0 + ntl) * C::KTB <= row.lk && (tile0 + ntl) * C::VTB <= row.lv, err, 47);

    if (tid == 0) {
        for (int i = 0; i < 6; i++) mbar_init(bars + i, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // the all-ones operand (f16 1.0): 128 x 16 values, any layout
    *reinterpret_cast<uint4 *>(sm + C::ONES + tid * 16) = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
        // every byte the block needs is requested at once: K halves and Q^T first, they are needed first
        const int nt0 = min(ntl, 8), nt1 = ntl - nt0;
        mbar_expect_tx(bars + 0, (uint32_t)nt0 * C::KTB);
        bulk_g2s(sm + C::RAW_K0, kg, (uint32_t)nt0 * C::KTB, bars + 0);
        mbar_expect_tx(bar_q, TCD_QT_BYTES);
        bulk_g2s(sm + C::QT, qtg + ((size_t)lo * n_kv + g) * TCD_QT_BYTES, TCD_QT_BYTES, bar_q);
        if (nt1 > 0) {
            mbar_expect_tx(bars + 1, (uint32_t)nt1 * C::KTB);
            bulk_g2s(sm + C::RAW_K1, kg + 8 * C::KTB, (uint32_t)nt1 * C::KTB, bars + 1);
        }
        mbar_expect_tx(bars + 2, (uint32_t)nt0 * C::VTB);
        bulk_g2s(sm + C::RAW_V0, vg, (uint32_t)nt0 * C::VTB, bars + 2);
        if (nt1 > 0) {
            mbar_expect_tx(bars + 3, (uint32_t)nt1 * C::VTB);
            bulk_g2s(sm + C::RAW_V1, vg + 8 * C::VTB, (uint32_t)nt1 * C::VTB, bars + 3);
        }
    }
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t sbase = smem_u32(sm);
    constexpr uint32_t idesc16 = umma_idesc(128, 16, 1, 0), idesc64 = umma_idesc(128, 64, 1, 0);  // A MN-major, B K-major
    bool ok = true;
    uint32_t mma_phase = 0;
    bool op_busy = false;  // MMAs reading the operand buffer are in flight
    auto wait_mma = [&]() {
        if (op_busy) {
            ok = mbar_wait_bounded(bar_mma, mma_phase, err, 71) && ok;
            mma_phase ^= 1;
            tc_fence_after();
            op_busy = false;
        }
    };

    // ---- S_c^T (half h) = X_K (half h, dims of group c) Q^T
    for (int h = 0; h < nh; h++) {
        const int nt = min(ntl - 8 * h, 8);
        const uint8_t *raw = sm + (h ? C::RAW_K1 : C::RAW_K0);
        ok = mbar_wait_bounded(bars + h, 0, err, 72) && ok;
        wait_mma();  // (S^T of half 0 has been computed: the operand buffer is free)
        // raw tiles -> f16 K tiles [dim][16 positions] (rows of 32 bytes, the two 16-byte chunks of a row swapped where
        // bit 2 of the row index is set: the 32-byte swizzle), 4 KB per tile; tiles past the block's last one are zero
        if constexpr (KF == KV_Q8) {
            uint4 w[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int idx = tid + TCD_THREADS * k, u = idx >> 7, i = idx & 127;
                w[k] = u < nt ? *reinterpret_cast<const uint4 *>(raw + (size_t)u * C::KTB + i * 16) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int idx = tid + TCD_THREADS * k, u = idx >> 7, i = idx & 127;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0;
                if (u < nt) tcd_x16(tcd_xor(w[k], 0x80808080u), c0, c1);
                uint8_t *dst = op + u * 4096 + i * 32;
                const int sw = ((i >> 2) & 1) << 4;
                *reinterpret_cast<uint4 *>(dst + sw) = c0;
                *reinterpret_cast<uint4 *>(dst + (sw ^ 16)) = c1;
            }
        } else {  // 4-bit K: a byte row holds the dim pair (2 p, 2 p + 1) of 16 positions
            uint4 w[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int idx = tid + TCD_THREADS * k, u = idx >> 6, p = idx & 63;
                w[k] = u < nt ? *reinterpret_cast<const uint4 *>(raw + (size_t)u * C::KTB + p * 16) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int idx = tid + TCD_THREADS * k, u = idx >> 6, p = idx & 63;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0, e0 = c0, e1 = c0;
                if (u < nt) {
                    tcd_x16(tcd_lo4(w[k]), c0, c1);
                    tcd_x16(tcd_hi4(w[k]), e0, e1);
                }
                uint8_t *dst = op + u * 4096 + (2 * p) * 32;  // rows 2 p and 2 p + 1 share bit 2 of the row index
                const int sw = ((p >> 1) & 1) << 4;
                *reinterpret_cast<uint4 *>(dst + sw) = c0;
                *reinterpret_cast<uint4 *>(dst + (sw ^ 16)) = c1;
                *reinterpret_cast<uint4 *>(dst + 32 + sw) = e0;
                *reinterpret_cast<uint4 *>(dst + 32 + (sw ^ 16)) = e1;
            }
        }
        if (h == 0) ok = mbar_wait_bounded(bar_q, 0, err, 74) && ok;  // (Q^T has landed: every thread sees it before the MMAs read it)
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            // A: the K tiles, MN-major, 32-byte swizzle (tile stride 4096, 8 dims = 256 bytes); k-step = 16 dims = 512 bytes;
            // the two k-steps of a 32-dim group accumulate into that group's columns
            const uint64_t da = umma_desc(sbase + C::OP, 4096, 256, 6), db = umma_desc(sbase + C::QT, 16, 1024, 2);
#pragma unroll
            for (int ks = 0; ks < 8; ks++)
                umma_ss(tbase + S_COL + 64 * h + 16 * (ks >> 1), da + (uint64_t)(ks * 32), db + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), idesc16,
                        ks & 1);
            umma_commit(bar_mma);
        }
        op_busy = true;
    }

    // ---- softmax of the block: thread (half h2, key t) holds the scores of its key for the G vectors.  While the last
    // products complete it fetches the key's scales (K: [group][16 positions], V: [position][group]; bf16) and the group sums
    const int h2 = tid >> 7, t = tid & 127, pos = 128 * h2 + t;
    const bool valid = pos < n;
    float dk[4] = {0.0f, 0.0f, 0.0f, 0.0f}, dv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (valid) {
        const uint8_t *kt = sm + (h2 ? C::RAW_K1 : C::RAW_K0) + (size_t)(t >> 4) * C::KTB + (KF == KV_Q4 ? 8 : 16) * HD;
#pragma unroll
        for (int c = 0; c < 4; c++) dk[c] = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(kt + (c * 16 + (t & 15)) * 2));
    }
    ok = mbar_wait_bounded(bars + 2, 0, err, 73) && ok;  // (the V halves have landed: the scales are behind their levels)
    if (nh > 1) ok = mbar_wait_bounded(bars + 3, 0, err, 73) && ok;
    if (valid) {
        const uint8_t *vt = sm + (h2 ? C::RAW_V1 : C::RAW_V0) + (size_t)(t >> 4) * C::VTB + (VF == KV_Q4 ? 8 : 16) * HD;
        const uint2 w = *reinterpret_cast<const uint2 *>(vt + (t & 15) * 8);
        dv[0] = __uint_as_float(w.x << 16), dv[1] = __uint_as_float(w.x & 0xffff0000u);
        dv[2] = __uint_as_float(w.y << 16), dv[3] = __uint_as_float(w.y & 0xffff0000u);
    }
    wait_mma();
    const float c2 = scale * 1.44269504088896341f;
    float s[NVT], e[NVT];
    {
#pragma unroll
        for (int v = 0; v < NVT; v++) s[v] = 0.0f;
        if (h2 < nh) {  // (uniform per warp)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t r[8];
                tmem_ld8(lane_addr + S_COL + 64 * h2 + 16 * c, r);
                tmem_wait_ld();
#pragma unroll
                for (int v = 0; v < NVT; v++) s[v] = fmaf(dk[c], fmaf(-KBIAS, qsum[v * 4 + c], __uint_as_float(r[v])), s[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < NVT; v++) s[v] = valid ? s[v] : -INFINITY;
    }
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float mx = s[v];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[warp * 8 + v] = mx;
    }
    __syncthreads();  // (also: every thread holds its key's scales: the raw K bytes may be overwritten by P^T)
    float m[NVT], l[NVT];
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float mx = red[v];
#pragma unroll
        for (int wv = 1; wv < 8; wv++) mx = fmaxf(mx, red[wv * 8 + v]);
        m[v] = mx;
        e[v] = valid ? ex2((s[v] - mx) * c2) : 0.0f;
        float sum = e[v];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) red[64 + warp * 8 + v] = sum;
    }
    // P^T: the B operand of O^T += X_V^T P^T, per half [64 = 16 vectors x 4 groups][128 keys] f16, K-major with the 128-byte
    // swizzle (two k-blocks of 64 keys): row 16 c + v holds p[.][v] d_V[.][c].  Rows of vectors past G only feed output
    // columns that are never read.
    {
        const int c16 = t >> 3;
        uint8_t *pb = pt + h2 * 16384 + (c16 >> 3) * 8192 + (t & 7) * 2;
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int v = 0; v < NVT; v++) {
                const int rw = 16 * c + v;
                *reinterpret_cast<__half *>(pb + rw * 128 + (((c16 & 7) ^ (rw & 7)) << 4)) = __float2half_rn(valid ? e[v] * dv[c] : 0.0f);
            }
    }
    __syncthreads();
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float sum = red[64 + v];
#pragma unroll
        for (int wv = 1; wv < 8; wv++) sum += red[64 + wv * 8 + v];
        l[v] = sum;
    }

    // ---- O^T += X_V^T (half h) P^T (half h), W += 1 P^T (half h)
    for (int h = 0; h < nh; h++) {
        const int nt = min(ntl - 8 * h, 8);
        const uint8_t *raw = sm + (h ? C::RAW_V1 : C::RAW_V0);
        wait_mma();
        // raw tiles -> f16 V rows [position][128 dims] as two 64-dim halves of 128-byte rows with the 128-byte swizzle;
        // positions past the block's last one are zero (their weights are zero as well)
        if constexpr (VF == KV_Q8) {
            uint4 w[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int idx = tid + TCD_THREADS * k, j = idx >> 3, ch = idx & 7;  // position j of the half, dims 16 ch .. 16 ch + 15
                w[k] = 128 * h + j < n ? *reinterpret_cast<const uint4 *>(raw + (size_t)(j >> 4) * C::VTB + (j & 15) * HD + ch * 16) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int idx = tid + TCD_THREADS * k, j = idx >> 3, ch = idx & 7;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0;
                if (128 * h + j < n) tcd_x16(tcd_xor(w[k], 0x80808080u), c0, c1);
                uint8_t *dst = op + (ch >> 2) * 16384 + j * 128;
                const int c8 = (2 * ch) & 7;
                *reinterpret_cast<uint4 *>(dst + ((c8 ^ (j & 7)) << 4)) = c0;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 1) ^ (j & 7)) << 4)) = c1;
            }
        } else {  // 4-bit V: per position and group 16 bytes, byte l = dims 32 c + l (low nibble), 32 c + 16 + l (high)
            uint4 w[2];
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int idx = tid + TCD_THREADS * k, j = idx >> 2, cg = idx & 3;
                w[k] = 128 * h + j < n ? *reinterpret_cast<const uint4 *>(raw + (size_t)(j >> 4) * C::VTB + (j & 15) * (HD / 2) + cg * 16) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int idx = tid + TCD_THREADS * k, j = idx >> 2, cg = idx & 3;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0, e0 = c0, e1 = c0;
                if (128 * h + j < n) {
                    tcd_x16(tcd_lo4(w[k]), c0, c1);
                    tcd_x16(tcd_hi4(w[k]), e0, e1);
                }
                uint8_t *dst = op + (cg >> 1) * 16384 + j * 128;
                const int c8 = (4 * cg) & 7;  // dims 32 cg .. : chunks c8, c8 + 1 (low nibbles), c8 + 2, c8 + 3 (high)
                *reinterpret_cast<uint4 *>(dst + ((c8 ^ (j & 7)) << 4)) = c0;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 1) ^ (j & 7)) << 4)) = c1;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 2) ^ (j & 7)) << 4)) = e0;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 3) ^ (j & 7)) << 4)) = e1;
            }
        }
        (void)nt;
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            // A: the V rows, MN-major, 128-byte swizzle (64-dim halves 16384 apart, 8 positions = 1024 bytes); the ones: the same
            // form over 4 KB; B: P^T of the half, 64 rows; k-step = 16 keys
            const uint64_t da = umma_desc(sbase + C::OP, 16384, 1024, 2), d1 = umma_desc(sbase + C::ONES, 2048, 1024, 2);
            const uint64_t db = umma_desc(sbase + C::PT + h * 16384, 16, 1024, 2);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                const uint64_t bk = db + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4);
                umma_ss(tbase + O_COL, da + (uint64_t)(ks * 128), bk, idesc64, (h > 0) | (ks > 0));
                umma_ss(tbase + W_COL, d1, bk, idesc64, (h > 0) | (ks > 0));
            }
            umma_commit(bar_mma);
        }
        op_busy = true;
    }
    wait_mma();

    // ---- the partial result of (row, head, block): o[hd] (unnormalised), m (in scaled-score units), l.  Thread = dim i of
    // group c = i / 32 (uniform over the warp): its columns of O and of the column sums
    if (warp < 4) {
        uint32_t r[8], wsum[8];
        tmem_ld8(lane_addr + O_COL + 16 * warp, r);
        tmem_ld8(lane_addr + W_COL + 16 * warp, wsum);
        tmem_wait_ld();
#pragma unroll
        for (int v = 0; v < NVT; v++) {
            if (v < G) {
                float *p = part + ((size_t)(row.blk0 + b) * n_heads + (size_t)g * G + v) * RQ_PSTRIDE(HD);
                p[tid] = ok ? fmaf(-VBIAS, __uint_as_float(wsum[v]), __uint_as_float(r[v])) : 0.0f;  // (tid = TMEM lane = dim)
                if (tid == 0) {
                    p[HD] = m[v] * scale;
                    p[HD + 1] = l[v];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(TM_COLS));
}

template <int KVT, int NVT>
static cudaError_t launch_tc_one(const AttnPartTcArgs &a, cudaStream_t stream) {
    constexpr int smem = TcdCfg<KVT>::SMEM;
    static_assert(smem <= 227 * 1024, "one CTA's shared memory");
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = attn_part_tc_kernel<KVT, NVT>;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaError_t e = launch_pdl(tcd_q_prep_kernel, dim3(a.nrows, a.n_kv), dim3(128), 0, stream, a.rows, a.n_kv, a.G, a.q, a.qh, a.n_heads, a.qt, a.blk2row);
    if (e != cudaSuccess) return e;
    return launch_pdl(kern, dim3(a.total_blocks, a.n_kv), dim3(TCD_THREADS), (size_t)smem, stream, a.rows, (const int *)a.blk2row, (const uint8_t *)a.qt,
                      a.layer, a.n_kv, a.G, a.n_heads, a.scale, a.part, a.err);
}

template <int KVT>
cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream) {
    if (a.G < 1 || a.G > 8) return cudaErrorInvalidValue;
    if (a.G == 1) return launch_tc_one<KVT, 1>(a, stream);
    if (a.G == 2) return launch_tc_one<KVT, 2>(a, stream);
    if (a.G <= 4) return launch_tc_one<KVT, 4>(a, stream);
    return launch_tc_one<KVT, 8>(a, stream);
}
#endif  // RQ_ATTN_DECODE_TC_INSTANTIATE

}  // namespace rq
