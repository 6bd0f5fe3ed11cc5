// Split-K decode attention over q8 / q4 / q4k4 KV caches on the tensor cores (tcgen05 + TMEM), head_dim 128: the fast form of
// attn_part_kernel for quantised caches.
//
// Same work items and the same partial results as attn_part_kernel (one (o, m, l) record per (row, KV head, block of 256
// positions), merged in block order by attn_combine_kernel, which also un-rotates and gates), so the split still
// depends on a row's own length only and a row of a batch gives the bits it gives alone.  What changes is the arithmetic
// inside a block.  The CUDA-core kernel spends ~8 instructions per cached level (conversion, scale, four multiply-adds);
// here a level costs ~2: the raw tiles arrive by bulk async copies (TMA), all 256 threads turn them into f16 values
// (level x scale, the exact product rounded once to f16) in the shared-memory layout of an MMA operand, and the dot
// products run as tcgen05.mma with the keys as the M dimension:
//     S^T [128 keys x 16] = K [128 keys x 128 dims] Q^T          (A = K: positions contiguous = MN-major, as cached)
//     O^T [128 dims x 16] += V^T [128 dims x 128 keys] P^T       (A = V^T: dims contiguous = MN-major, as cached)
// per half block of 128 positions; the query vectors of the KV head (at most 8) are the N dimension, padded to 16.  With
// the keys on the TMEM lanes, the softmax of a block is spread over all threads (thread = key: G exponentials each).
// Results agree with the reference's fp32 arithmetic to ~3e-4 relative (q, the dequantised values and the softmax weights
// are rounded to f16; accumulation in fp32), inside the acceptance bar but not bit for bit: the bit-exact kernel stays
// selectable (rq_cuda_set_exact).  The dequantised values themselves are exact products before that one rounding.
// Limits of this form: head_dim 128; dequantised magnitudes up to the f16 range (65504).
#pragma once
#include "attn_decode.cuh"
#include "tc05.cuh"

namespace rq {

constexpr int TCD_THREADS = 256;

template <int KVT>
struct TcdCfg {
    static constexpr int HD = 128;
    static constexpr int KF = kv_fmt(KVT, 0), VF = kv_fmt(KVT, 1);
    static constexpr int KTB = kv_tile_bytes(KVT, HD, 0), VTB = kv_tile_bytes(KVT, HD, 1);
    static constexpr int KHALF = 8 * KTB, VHALF = 8 * VTB;  // raw bytes of half a block (8 tiles of 16 positions)
    // shared memory (from a 1024-byte aligned base): f16 operand buffer (32 KB: one half block of K, later of V) | Q^T (4 KB) |
    // raw K half 0 (later P^T, 8 KB), raw K half 1, raw V half 0, raw V half 1 | reductions, barriers, TMEM slot
    static constexpr int OP = 0, QT = 32768, RAW = QT + 4096;
    static constexpr int RAW_K0 = RAW, RAW_K1 = RAW_K0 + KHALF, RAW_V0 = RAW_K1 + KHALF, RAW_V1 = RAW_V0 + VHALF;
    static constexpr int PT = RAW_K0;  // P^T (2 halves x 4 KB) reuses the raw K bytes once they are dequantised
    static_assert(2 * KHALF >= 8192 && KHALF % 16 == 0 && VHALF % 16 == 0, "P^T fits the raw K area; bulk copies are multiples of 16 bytes");
    static constexpr int MISC = (RAW_V1 + VHALF + 15) / 16 * 16;  // red [2][8 warps][8] floats | bars [5] | TMEM slot
    static constexpr int SMEM = MISC + 512 + 64 + 16 + 1024;
};

struct AttnPartTcArgs {
    const PassRow *rows;
    int nrows, total_blocks, layer, n_kv, G;
    const float *q;
    int qh, n_heads;
    float scale;
    float *part;
    int *err;
};
// launches attn_part_tc_kernel<KVT> on `stream` (grid: total_blocks x n_kv); cudaErrorInvalidValue for an unsupported shape
template <int KVT>
cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_DECODE_TC_INSTANTIATE

// four bytes b (each a level + bias, 0 <= b < 1024) -> four f16 values (b - bias) as two half2
__device__ __forceinline__ void tcd_bytes_to_h2(uint32_t w, const __half2 bias, __half2 &lo, __half2 &hi) {
    // an f16 with exponent field 0x19 (0x6400) has unit spacing: 0x6400 | b is exactly 1024 + b
    const uint32_t a = __byte_perm(w, 0x64646464u, 0x4140), b = __byte_perm(w, 0x64646464u, 0x4342);
    lo = __hsub2(*reinterpret_cast<const __half2 *>(&a), bias);
    hi = __hsub2(*reinterpret_cast<const __half2 *>(&b), bias);
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// 16 levels (the bytes of w, each level + bias) times 16 scales (8 half2 in s0, s1) -> 16 f16 values as two 16-byte chunks
__device__ __forceinline__ void tcd_row16(const uint4 w, const uint4 s0, const uint4 s1, const __half2 bias, uint4 &c0, uint4 &c1) {
    __half2 lo, hi;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const uint32_t ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t o[8];
#pragma unroll
    for (int x = 0; x < 4; x++) {
        tcd_bytes_to_h2(ww[x], bias, lo, hi);
        o[2 * x] = h2_bits(__hmul2(lo, *reinterpret_cast<const __half2 *>(&ss[2 * x])));
        o[2 * x + 1] = h2_bits(__hmul2(hi, *reinterpret_cast<const __half2 *>(&ss[2 * x + 1])));
    }
    c0 = make_uint4(o[0], o[1], o[2], o[3]);
    c1 = make_uint4(o[4], o[5], o[6], o[7]);
}
// the same with one scale for all 16 levels
__device__ __forceinline__ void tcd_row16_1(const uint4 w, const __half2 d2, const __half2 bias, uint4 &c0, uint4 &c1) {
    const uint32_t d = h2_bits(d2);
    tcd_row16(w, make_uint4(d, d, d, d), make_uint4(d, d, d, d), bias, c0, c1);
}

// bf16 scales of one raw half (nt tiles; `off`: where a tile's scales start; 64 per tile at head_dim 128) -> f16, in place
__device__ __forceinline__ void tcd_scales_to_f16(uint8_t *raw, int tile_bytes, int off, int nt, int tid) {
    for (int e = tid; e < nt * 32; e += TCD_THREADS) {  // one pair of scales per step
        uint32_t *p = reinterpret_cast<uint32_t *>(raw + (size_t)(e >> 5) * tile_bytes + off) + (e & 31);
        const uint32_t w = *p;
        const __half2 h = __floats2half2_rn(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
        *p = h2_bits(h);
    }
}

template <int KVT, int NVT>
__global__ void __launch_bounds__(TCD_THREADS) attn_part_tc_kernel(const PassRow *__restrict__ rows, int nrows, int layer, int n_kv, int G,
                                                                   const float *__restrict__ q, int qh, int n_heads, float scale,
                                                                   float *__restrict__ part, int *err) {
    using C = TcdCfg<KVT>;
    constexpr int HD = C::HD, KF = C::KF, VF = C::VF;
    constexpr int TM_COLS = 64, S_COL = 0, O_COL = 32;  // S^T of half h at 16 h, O^T at 32 (16 columns each)
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *op = sm + C::OP, *qt = sm + C::QT, *pt = sm + C::PT;
    float *red = reinterpret_cast<float *>(sm + C::MISC);                    // [2][8][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + C::MISC + 512);       // raw K0, K1, V0, V1 landed; MMAs complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + C::MISC + 512 + 64);
    uint64_t *bar_mma = bars + 4;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();

    // which (row, block) is this CTA: rows[r].blk0 <= blockIdx.x < rows[r + 1].blk0
    int lo = 0, hi = nrows;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (rows[mid].blk0 <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    const PassRow row = rows[lo];
    const int b = blockIdx.x - row.blk0, g = blockIdx.y;
    const int n = min(row.np - b * ATT_P, ATT_P);  // positions of this block
    const int ntl = (n + ATT_T - 1) / ATT_T;       // its tiles
    const int nh = (n + 127) >> 7;                 // its halves of 128 positions
    const size_t tile0 = ((size_t)b * n_kv + g) * ATT_PT;
    const uint8_t *kg = row.k + (size_t)layer * row.lk + tile0 * C::KTB;
    const uint8_t *vg = row.v + (size_t)layer * row.lv + tile0 * C::VTB;
    RQ_CHECK(lo >= 0 && lo < nrows && b >= 0 && n >= 1 && g < n_kv && (tile0 + ntl) * C::KTB <= row.lk && (tile0 + ntl) * C::VTB <= row.lv, err, 47);

    if (tid == 0) {
        for (int i = 0; i < 5; i++) mbar_init(bars + i, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    __syncthreads();
    if (tid == 0) {
        // every raw byte of the block is requested at once: K halves first, they are needed first
        const int nt0 = min(ntl, 8), nt1 = ntl - nt0;
        mbar_expect_tx(bars + 0, (uint32_t)nt0 * C::KTB);
        bulk_g2s(sm + C::RAW_K0, kg, (uint32_t)nt0 * C::KTB, bars + 0);
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

    // ---- the query vectors: rotated (att_q_rot, reference src/forward.c:1662: signs, butterflies h = 1, 2, 4, ..., scaling
    // by 1 / head_dim) in fp32, then f16 into Q^T: the B operand of S^T = K Q^T, [16 vectors][128 dims] K-major with the
    // 128-byte swizzle (two k-blocks of 64 dims: [kb][row][128 B]); rows past the G vectors are zero
    {
        float *tmp = reinterpret_cast<float *>(op);  // [NVT][HD], the operand buffer is not in use yet
        const float *qrow = q + ((size_t)lo * n_heads + (size_t)g * G) * qh;
        for (int e = tid; e < NVT * HD; e += TCD_THREADS) {
            const int v = e / HD, i = e % HD;
            const float x = v < G ? qrow[(size_t)v * qh + i] : 0.0f;
            tmp[e] = kvq_neg(i) ? -x : x;
        }
        __syncthreads();
        for (int hs = 1; hs < HD; hs <<= 1) {
            for (int e = tid; e < NVT * HD / 2; e += TCD_THREADS) {
                const int v = e / (HD / 2), p = e % (HD / 2);
                const int j = (p / hs) * 2 * hs + (p % hs);
                const float a = tmp[v * HD + j], bb = tmp[v * HD + j + hs];
                tmp[v * HD + j] = a + bb;
                tmp[v * HD + j + hs] = a - bb;
            }
            __syncthreads();
        }
        const float f = 1.0f / (float)HD;
        for (int e = tid; e < 16 * (HD / 8); e += TCD_THREADS) {  // one 16-byte chunk (8 dims) of one row per step
            const int v = e >> 4, c16 = e & 15;
            uint4 o = make_uint4(0u, 0u, 0u, 0u);
            if (v < NVT) {
                const float *s = tmp + v * HD + c16 * 8;
                o.x = h2_bits(__floats2half2_rn(s[0] * f, s[1] * f)), o.y = h2_bits(__floats2half2_rn(s[2] * f, s[3] * f));
                o.z = h2_bits(__floats2half2_rn(s[4] * f, s[5] * f)), o.w = h2_bits(__floats2half2_rn(s[6] * f, s[7] * f));
            }
            *reinterpret_cast<uint4 *>(qt + (c16 >> 3) * 2048 + v * 128 + (((c16 & 7) ^ (v & 7)) << 4)) = o;
        }
    }
    tc_fence_before();
    __syncthreads();  // (Q^T is complete, the rotation scratch is free again, the TMEM address is visible)
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t sbase = smem_u32(sm);
    constexpr uint32_t idesc = umma_idesc(128, 16, 1, 0);  // A MN-major (K, V^T as cached), B K-major (Q^T, P^T)
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
    const __half2 bias8 = __floats2half2_rn(1152.0f, 1152.0f), bias4 = __floats2half2_rn(1032.0f, 1032.0f);

    // ---- S^T (half h) = K (half h) Q^T
    for (int h = 0; h < nh; h++) {
        const int nt = min(ntl - 8 * h, 8);
        uint8_t *raw = sm + (h ? C::RAW_K1 : C::RAW_K0);
        ok = mbar_wait_bounded(bars + h, 0, err, 72) && ok;
        tcd_scales_to_f16(raw, C::KTB, (KF == KV_Q4 ? 8 : 16) * HD, nt, tid);
        wait_mma();  // (S^T of half 0 has been computed: the operand buffer is free)
        __syncthreads();
        // raw tiles -> f16 K tiles [dim][16 positions] (rows of 32 bytes, the two 16-byte chunks of a row swapped where
        // bit 2 of the row index is set: the 32-byte swizzle), 4 KB per tile; tiles past the block's last one are zero
        if constexpr (KF == KV_Q8) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int idx = tid + TCD_THREADS * k, u = idx >> 7, i = idx & 127;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0;
                if (u < nt) {
                    const uint8_t *t = raw + (size_t)u * C::KTB;
                    const uint4 *sp = reinterpret_cast<const uint4 *>(t + 16 * HD + (i >> 5) * 32);
                    uint4 w = *reinterpret_cast<const uint4 *>(t + i * 16);
                    w.x ^= 0x80808080u, w.y ^= 0x80808080u, w.z ^= 0x80808080u, w.w ^= 0x80808080u;
                    tcd_row16(w, sp[0], sp[1], bias8, c0, c1);
                }
                uint8_t *dst = op + u * 4096 + i * 32;
                const int sw = ((i >> 2) & 1) << 4;
                *reinterpret_cast<uint4 *>(dst + sw) = c0;
                *reinterpret_cast<uint4 *>(dst + (sw ^ 16)) = c1;
            }
        } else {  // 4-bit K: a byte row holds the dim pair (2 p, 2 p + 1) of 16 positions
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int idx = tid + TCD_THREADS * k, u = idx >> 6, p = idx & 63;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0, e0 = c0, e1 = c0;
                if (u < nt) {
                    const uint8_t *t = raw + (size_t)u * C::KTB;
                    const uint4 *sp = reinterpret_cast<const uint4 *>(t + 8 * HD + (p >> 4) * 32);
                    const uint4 w = *reinterpret_cast<const uint4 *>(t + p * 16), s0 = sp[0], s1 = sp[1];
                    const uint4 wl = make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu);
                    const uint4 wh = make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
                    tcd_row16(wl, s0, s1, bias4, c0, c1);
                    tcd_row16(wh, s0, s1, bias4, e0, e1);
                }
                uint8_t *dst = op + u * 4096 + (2 * p) * 32;  // rows 2 p and 2 p + 1 share bit 2 of the row index
                const int sw = ((p >> 1) & 1) << 4;
                *reinterpret_cast<uint4 *>(dst + sw) = c0;
                *reinterpret_cast<uint4 *>(dst + (sw ^ 16)) = c1;
                *reinterpret_cast<uint4 *>(dst + 32 + sw) = e0;
                *reinterpret_cast<uint4 *>(dst + 32 + (sw ^ 16)) = e1;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            // A: the K tiles, MN-major, 32-byte swizzle (tile stride 4096, 8 dims = 256 bytes); k-step = 16 dims = 512 bytes
            const uint64_t da = umma_desc(sbase + C::OP, 4096, 256, 6), db = umma_desc(sbase + C::QT, 16, 1024, 2);
#pragma unroll
            for (int ks = 0; ks < 8; ks++)
                umma_ss(tbase + S_COL + 16 * h, da + (uint64_t)(ks * 32), db + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), idesc, ks > 0);
            umma_commit(bar_mma);
        }
        op_busy = true;
    }
    wait_mma();

    // ---- softmax of the block: thread (half h2, key t) holds the scores of its key for the G vectors
    const int h2 = tid >> 7, t = tid & 127, pos = 128 * h2 + t;
    const bool valid = pos < n;
    const float c2 = scale * 1.44269504088896341f;
    float s[8], e[8];
    {
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (h2 < nh) {  // (uniform per warp)
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                         : "r"(lane_addr + S_COL + 16 * h2));
            tmem_wait_ld();
        }
#pragma unroll
        for (int v = 0; v < NVT; v++) s[v] = valid ? __uint_as_float(r[v]) : -INFINITY;
    }
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float mx = s[v];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[warp * 8 + v] = mx;
    }
    __syncthreads();
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
    // P^T: the B operand of O^T += V^T P^T, per half [16 vectors][128 keys] f16, K-major with the 128-byte swizzle (two
    // k-blocks of 64 keys); it takes the place of the raw K bytes.  Rows past the G vectors only feed output columns that
    // are never read.
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        const int c16 = t >> 3;
        *reinterpret_cast<__half *>(pt + h2 * 4096 + (c16 >> 3) * 2048 + v * 128 + (((c16 & 7) ^ (v & 7)) << 4) + (t & 7) * 2) = __float2half_rn(e[v]);
    }
    __syncthreads();
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float sum = red[64 + v];
#pragma unroll
        for (int wv = 1; wv < 8; wv++) sum += red[64 + wv * 8 + v];
        l[v] = sum;
    }

    // ---- O^T += V^T (half h) P^T (half h)
    for (int h = 0; h < nh; h++) {
        const int nt = min(ntl - 8 * h, 8);
        uint8_t *raw = sm + (h ? C::RAW_V1 : C::RAW_V0);
        ok = mbar_wait_bounded(bars + 2 + h, 0, err, 73) && ok;
        tcd_scales_to_f16(raw, C::VTB, (VF == KV_Q4 ? 8 : 16) * HD, nt, tid);
        wait_mma();
        __syncthreads();
        // raw tiles -> f16 V rows [position][128 dims] as two 64-dim halves of 128-byte rows with the 128-byte swizzle;
        // positions past the block's last one are zero (their weights are zero: they must not meet a stale NaN pattern)
        if constexpr (VF == KV_Q8) {
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int idx = tid + TCD_THREADS * k, j = idx >> 3, ch = idx & 7;  // position j of the half, dims 16 ch .. 16 ch + 15
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0;
                if (128 * h + j < n) {
                    const uint8_t *tl = raw + (size_t)(j >> 4) * C::VTB;
                    uint4 w = *reinterpret_cast<const uint4 *>(tl + (j & 15) * HD + ch * 16);
                    const uint32_t d = *reinterpret_cast<const uint16_t *>(tl + 16 * HD + ((j & 15) * 4 + (ch >> 1)) * 2);
                    const uint32_t dd = d | (d << 16);
                    w.x ^= 0x80808080u, w.y ^= 0x80808080u, w.z ^= 0x80808080u, w.w ^= 0x80808080u;
                    tcd_row16_1(w, *reinterpret_cast<const __half2 *>(&dd), bias8, c0, c1);
                }
                uint8_t *dst = op + (ch >> 2) * 16384 + j * 128;
                const int c8 = (2 * ch) & 7;
                *reinterpret_cast<uint4 *>(dst + ((c8 ^ (j & 7)) << 4)) = c0;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 1) ^ (j & 7)) << 4)) = c1;
            }
        } else {  // 4-bit V: per position and group 16 bytes, byte l = dims 32 c + l (low nibble), 32 c + 16 + l (high)
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int idx = tid + TCD_THREADS * k, j = idx >> 2, cg = idx & 3;
                uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0, e0 = c0, e1 = c0;
                if (128 * h + j < n) {
                    const uint8_t *tl = raw + (size_t)(j >> 4) * C::VTB;
                    const uint4 w = *reinterpret_cast<const uint4 *>(tl + (j & 15) * (HD / 2) + cg * 16);
                    const uint32_t d = *reinterpret_cast<const uint16_t *>(tl + 8 * HD + ((j & 15) * 4 + cg) * 2);
                    const uint32_t dd = d | (d << 16);
                    const uint4 wl = make_uint4(w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu);
                    const uint4 wh = make_uint4((w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu);
                    tcd_row16_1(wl, *reinterpret_cast<const __half2 *>(&dd), bias4, c0, c1);
                    tcd_row16_1(wh, *reinterpret_cast<const __half2 *>(&dd), bias4, e0, e1);
                }
                uint8_t *dst = op + (cg >> 1) * 16384 + j * 128;
                const int c8 = (4 * cg) & 7;  // dims 32 cg .. : chunks c8, c8 + 1 (low nibbles), c8 + 2, c8 + 3 (high)
                *reinterpret_cast<uint4 *>(dst + ((c8 ^ (j & 7)) << 4)) = c0;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 1) ^ (j & 7)) << 4)) = c1;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 2) ^ (j & 7)) << 4)) = e0;
                *reinterpret_cast<uint4 *>(dst + (((c8 + 3) ^ (j & 7)) << 4)) = e1;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            // A: the V rows, MN-major, 128-byte swizzle (64-dim halves 16384 apart, 8 positions = 1024 bytes); k-step = 16 keys
            const uint64_t da = umma_desc(sbase + C::OP, 16384, 1024, 2), db = umma_desc(sbase + C::PT + h * 4096, 16, 1024, 2);
#pragma unroll
            for (int ks = 0; ks < 8; ks++)
                umma_ss(tbase + O_COL, da + (uint64_t)(ks * 128), db + (uint64_t)(((ks >> 2) * 2048 + (ks & 3) * 32) >> 4), idesc, (h > 0) | (ks > 0));
            umma_commit(bar_mma);
        }
        op_busy = true;
    }
    wait_mma();

    // ---- the partial result of (row, head, block): o[hd] (unnormalised), m (in scaled-score units), l
    if (warp < 4) {
        uint32_t r[8];
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "r"(lane_addr + O_COL));
        tmem_wait_ld();
#pragma unroll
        for (int v = 0; v < NVT; v++) {
            if (v < G) {
                float *p = part + ((size_t)(row.blk0 + b) * n_heads + (size_t)g * G + v) * RQ_PSTRIDE(HD);
                p[tid] = ok ? __uint_as_float(r[v]) : 0.0f;  // (tid = TMEM lane = dim)
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
    return launch_pdl(kern, dim3(a.total_blocks, a.n_kv), dim3(TCD_THREADS), (size_t)smem, stream, a.rows, a.nrows, a.layer, a.n_kv, a.G, a.q, a.qh,
                      a.n_heads, a.scale, a.part, a.err);
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
