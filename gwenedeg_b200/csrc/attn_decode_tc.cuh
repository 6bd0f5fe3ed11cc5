// Split-K decode attention over q8 KV caches on the integer tensor cores (tcgen05.mma kind::i8 + TMEM), head_dim 128: the
// fast form of attn_part_kernel for 8-bit caches.
//
// Same work items and the same partial results as attn_part_kernel (one (o, m, l) record per (row, KV head, block of 256
// positions), merged in block order by attn_combine_kernel, which also un-rotates and gates), so the split still
// depends on a row's own length only and a row of a batch gives the bits it gives alone.  What changes is the arithmetic
// inside a block.  The CUDA-core kernel spends ~8 instructions per cached level (conversion, scale, four multiply-adds).
// Here the cached int8 levels are never converted at all: the tiles go from HBM to shared memory by TMA and from there
// straight into tcgen05.mma as 8-bit operands, accumulated exactly in int32:
//   V rows [position][128 dims] as cached, fetched through a 3-D tensor map with the 128-byte swizzle = an MN-major A operand:
//   O^T [128 dims x N'] += V^T [128 dims x 32 keys] P^T;
//   K tiles [dim][16 positions] hold 16 keys per dim, and the fast operand form wants a dim's 128 keys in one 128-byte row (the
//   tiles as they are, 8 dims x 16 positions per 128-byte core matrix without swizzle, are a valid operand too, but measured
//   ~700 cycles per MMA): every thread moves 16-byte chunks from global memory to their place in the swizzled rows (8 loads and
//   8 stores per thread and block, no arithmetic), then per 32-dim scale group c one MMA
//   S_c^T [128 keys x N] = K_c [128 keys x 32 dims] Q_c^T.
// The other operands are 16-bit fixed point split into two int8 planes (the query per (vector, group), by tcd_q_prep_kernel;
// the softmax weights times the V scale per (vector, group), scaled by the block's largest V scale of the group), so the
// only roundings are those two quantisations to 16 bits; the scales (exact bf16 -> fp32) are applied in fp32 by the
// softmax thread of a key (s = sum_c d_K[t][c] q_scale[v][c] S_c) and the epilogue thread of a dim.  Results agree with the
// reference's fp32 arithmetic to ~1e-4 relative, inside the acceptance bar but not bit for bit; the bit-exact kernel stays
// selectable (rq_cuda_set_exact).  With the keys on the TMEM lanes the softmax of a block is spread over all threads.
#pragma once
#include <cuda.h>

#include "attn_decode.cuh"
#include "tc05.cuh"

namespace rq {

constexpr int TCD_THREADS = 256;
constexpr int TCD_QT_BYTES = 2048 + 256;  // per (row, KV head): Q^T planes [16 rows][128 dims] int8 + scales [8 vectors][4 groups] fp32 (+ pad)

template <int NVT>
struct TcdCfg {
    static constexpr int HD = 128;
    static constexpr int KTB = kv_tile_bytes(KV_Q8, HD, 0), VTB = kv_tile_bytes(KV_Q8, HD, 1);  // 2176 each
    static constexpr int NS = NVT <= 4 ? 8 : 16;  // N of a score MMA: rows 2 v + plane
    static constexpr int NO = 8 * NVT;            // N of an output MMA: rows ((c NVT + v) 2 + plane)
    // shared memory (from a 1024-byte aligned base): K levels of the two halves (2 x 16 KB: 128 rows = dims of 128 keys; later
    // P^T: 2 x NO rows of 128 bytes) | V levels (2 x 16 KB: 128 rows = positions of 128 dims, swizzled by the TMA) | Q^T planes
    // and scales (2304 B) | the rest
    static constexpr int KLEV = 0, VLEV = 32768, QT = 65536;
    static constexpr int PT = KLEV;
    static constexpr int MISC = QT + 2304;  // red [3][8 warps][8] floats (768 B) | bars [4] | TMEM slot
    static constexpr int SMEM = MISC + 768 + 64 + 16 + 1024;
    static constexpr int TM_COLS = NVT <= 4 ? 128 : 256, S_COL = 0, O_COL = 8 * NS;
    static_assert(QT % 1024 == 0 && 2 * NO * 128 <= 32768, "operand alignment; P^T fits the K levels");
};

struct AttnPartTcArgs {
    const PassRow *rows;
    int nrows, total_blocks, layer, n_kv, G;
    const float *q;
    int qh, n_heads;
    float scale;
    float *part;
    uint8_t *qt;              // scratch: nrows x n_kv records of TCD_QT_BYTES
    int *blk2row;             // scratch: total_blocks ints
    const CUtensorMap *maps;  // per segment: [4 seg + 1] = the 3-D view of its sequence's V cache levels
    int *err;
};
// launches tcd_q_prep_kernel and attn_part_tc_kernel on `stream`; cudaErrorInvalidValue for an unsupported shape
cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_DECODE_TC_INSTANTIATE

// instruction descriptor of tcgen05.mma kind::i8: int8 / uint8 operands, int32 accumulator, M x N; a_mn / b_mn: MN-major (1) or
// K-major (0); a_s / b_s: signed (1) or unsigned (0) 8-bit values
__host__ __device__ constexpr uint32_t umma_idesc_i8(int M, int N, int a_mn, int b_mn, int a_s, int b_s) {
    return (2u << 4) | ((uint32_t)a_s << 7) | ((uint32_t)b_s << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem), "l"(a), "l"(b),
                 "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *m, int x, int y, int z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                     smem_u32(dst)),
                 "l"(m), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

// The query vectors of one (row, KV head), once per pass and layer: rotated as att_q_rot does (reference src/forward.c:1662:
// signs, butterflies h = 1, 2, 4, ..., scaling by 1 / head_dim) in fp32, then per (vector v, 32-dim group c) 16-bit fixed point
// q = qs[v][c] (256 hi + lo), hi and lo in [-128, 127], laid out as the B operand of the score MMAs: rows 2 v (hi) and 2 v + 1
// (lo) of [16 rows][128 dims] int8, K-major with the 128-byte swizzle; rows past the G vectors zero; the scales qs behind
// them.  The CTA of KV head 0 also fills the block -> row table of its row.
__global__ void __launch_bounds__(128) tcd_q_prep_kernel(const PassRow *__restrict__ rows, int n_kv, int G, const float *__restrict__ q, int qh,
                                                         int n_heads, uint8_t *__restrict__ qt, int *__restrict__ blk2row) {
    constexpr int HD = 128;
    const int r = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, c = tid >> 5;  // (a warp = a 32-dim group)
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float tmp[8][HD];
    __shared__ __align__(16) int8_t planes[16][HD];
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
    uint8_t *out = qt + ((size_t)r * n_kv + g) * TCD_QT_BYTES;
    float *qs = reinterpret_cast<float *>(out + 2048);
    const float f = 1.0f / (float)HD;
    for (int v = 0; v < 8; v++) {
        int hi = 0, lo = 0;
        if (v < G) {
            const float x = tmp[v][tid] * f;
            float amax = fabsf(x);
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float sc = amax > 0.0f ? amax / 32639.0f : 0.0f;
            const int q16 = amax > 0.0f ? __float2int_rn(x * (32639.0f / amax)) : 0;
            lo = ((q16 + 128) & 255) - 128;
            hi = (q16 - lo) >> 8;
            if (lane == 0) qs[v * 4 + c] = sc;
        } else if (lane == 0) {
            qs[v * 4 + c] = 0.0f;
        }
        planes[2 * v][tid] = (int8_t)hi;
        planes[2 * v + 1][tid] = (int8_t)lo;
    }
    __syncthreads();
    {  // one 16-byte chunk (16 dims) of one row per thread: 16 rows x 8 chunks
        const int rw = tid >> 3, ch = tid & 7;
        *reinterpret_cast<uint4 *>(out + rw * 128 + ((ch ^ (rw & 7)) << 4)) = *reinterpret_cast<const uint4 *>(&planes[rw][ch * 16]);
    }
}

// maps: per segment [4 seg + 1] the tensor map of its sequence's V cache: {128 bytes of levels, 16 positions, tiles} with
// strides {128, tile bytes}, box 128 x 16 x 8, 128-byte swizzle.
template <int NVT>
__global__ void __launch_bounds__(TCD_THREADS, 3) attn_part_tc_kernel(const PassRow *__restrict__ rows, const int *__restrict__ blk2row,
                                                                   const uint8_t *__restrict__ qtg, const CUtensorMap *__restrict__ maps, int layer,
                                                                   int n_kv, int G, int n_heads, float scale, float *__restrict__ part, int *err) {
    using C = TcdCfg<NVT>;
    constexpr int HD = C::HD, NS = C::NS, NO = C::NO;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *pt = sm + C::PT;
    const float *qsc = reinterpret_cast<const float *>(sm + C::QT + 2048);  // [8][4]
    float *red = reinterpret_cast<float *>(sm + C::MISC);                   // [3][8][8]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + C::MISC + 768);      // V half 0, V half 1, Q^T landed; MMAs complete
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + C::MISC + 768 + 64);
    uint64_t *bar_q = bars + 2, *bar_mma = bars + 3;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();

    const int lo = blk2row[blockIdx.x];
    const PassRow row = rows[lo];
    const int b = blockIdx.x - row.blk0, g = blockIdx.y;
    const int n = min(row.np - b * ATT_P, ATT_P);  // positions of this block
    const int nh = (n + 127) >> 7;                 // its halves of 128 positions
    // (whole halves are fetched: a layer is a whole number of 256-position blocks, so the tiles past the block's last
    // position exist; what they hold is masked below and enters the integer products as finite values times zero weights)
    const size_t tile0 = ((size_t)b * n_kv + g) * ATT_PT;
    const uint8_t *kg = row.k + (size_t)layer * row.lk + tile0 * C::KTB;
    const uint8_t *vg = row.v + (size_t)layer * row.lv + tile0 * C::VTB;
    RQ_CHECK(lo >= 0 && b >= 0 && n >= 1 && g < n_kv && (tile0 + 16) * C::KTB <= row.lk && (tile0 + 16) * C::VTB <= row.lv, err, 47);

    if (tid == 0) {
        for (int i = 0; i < 4; i++) mbar_init(bars + i, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t sbase = smem_u32(sm);
    bool ok = true;
    if (tid == 0) {
        // V and the query planes by TMA, at once
        mbar_expect_tx(bar_q, TCD_QT_BYTES);
        bulk_g2s(sm + C::QT, qtg + ((size_t)lo * n_kv + g) * TCD_QT_BYTES, TCD_QT_BYTES, bar_q);
        const CUtensorMap *mv = maps + 4 * row.seg + 1;
        const int vt0 = (int)((size_t)layer * (row.lv / C::VTB) + tile0);  // first tile of the block in the 3-D view
        for (int h = 0; h < nh; h++) {
            mbar_expect_tx(bars + h, 16384);
            tma_load_3d(sm + C::VLEV + h * 16384, mv, 0, 0, vt0 + 8 * h, bars + h);
        }
    }
    // ---- K: every thread fetches 4 chunks of 16 positions x one dim per half and the scales of its own key, then puts the chunks
    // where the operand wants them: row = dim, chunk = tile ^ (dim % 8) (the 128-byte swizzle)
    const int h2 = tid >> 7, t = tid & 127, pos = 128 * h2 + t;
    const bool valid = pos < n;
    float dk[4] = {0.0f, 0.0f, 0.0f, 0.0f}, dv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    {
        uint4 w[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int idx = tid + TCD_THREADS * (k & 3), u = (idx >> 7) + 8 * (k >> 2), i = idx & 127;  // tile u of the block, dim i
            w[k] = (k >> 2) < nh ? __ldg(reinterpret_cast<const uint4 *>(kg + (size_t)u * C::KTB + i * 16)) : make_uint4(0u, 0u, 0u, 0u);
        }
        if (valid) {  // the key's scales: K [group][16 positions], V [position][group], bf16, behind their tile's levels
            const uint16_t *ks = reinterpret_cast<const uint16_t *>(kg + (size_t)(pos >> 4) * C::KTB + 16 * HD) + (pos & 15);
#pragma unroll
            for (int c = 0; c < 4; c++) dk[c] = bf16_bits_to_f32(__ldg(ks + c * 16));
            const uint2 wv = __ldg(reinterpret_cast<const uint2 *>(vg + (size_t)(pos >> 4) * C::VTB + 16 * HD) + (pos & 15));
            dv[0] = __uint_as_float(wv.x << 16), dv[1] = __uint_as_float(wv.x & 0xffff0000u);
            dv[2] = __uint_as_float(wv.y << 16), dv[3] = __uint_as_float(wv.y & 0xffff0000u);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int idx = tid + TCD_THREADS * (k & 3), u = idx >> 7, i = idx & 127;
            *reinterpret_cast<uint4 *>(sm + C::KLEV + (k >> 2) * 16384 + i * 128 + ((u ^ (i & 7)) << 4)) = w[k];
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
        // ---- S_c^T (half h) = K_c (half h) Q_c^T: one MMA per 32-dim group
        tc_fence_after();
        ok = mbar_wait_bounded(bar_q, 0, err, 74) && ok;
        constexpr uint32_t idesc_s = umma_idesc_i8(128, NS, 1, 0, 1, 1);
        for (int h = 0; h < nh; h++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                // A: rows of 128 bytes (one dim, the half's 128 keys = one swizzle atom along MN), 8 dims = 1024 bytes (SBO); the group's
                // 32 dims are 4096 bytes; B: rows of 128 bytes, 128-byte swizzle, the group's 32 dims at 32 c
                const uint64_t da = umma_desc(sbase + C::KLEV + h * 16384 + c * 4096, 16, 1024, 2);
                const uint64_t db = umma_desc(sbase + C::QT + c * 32, 16, 1024, 2);
                umma_i8(tbase + C::S_COL + (4 * h + c) * NS, da, db, idesc_s, 0);
            }
        }
        umma_commit(bar_mma);
    }

    // ---- softmax of the block: thread (half h2, key t) holds the scores of its key for the G vectors
    // the block's largest V scale per group: what the weight planes are scaled by
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float mx = dv[c];
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[128 + warp * 8 + c] = mx;
    }
    if (lane == 0) {  // (one poller per warp)
        ok = mbar_wait_bounded(bar_q, 0, err, 74) && ok;   // (the query scales)
        ok = mbar_wait_bounded(bar_mma, 0, err, 71) && ok;  // (the score products)
    }
    __syncwarp();
    tc_fence_after();
    const float c2 = scale * 1.44269504088896341f;
    float s[NVT], e[NVT];
#pragma unroll
    for (int v = 0; v < NVT; v++) s[v] = 0.0f;
    __syncwarp();
    if (h2 < nh) {  // (uniform per warp)
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t r[NS];
            tmem_ld8(lane_addr + C::S_COL + (4 * h2 + c) * NS, r);
            if constexpr (NVT == 8) tmem_ld8(lane_addr + C::S_COL + (4 * h2 + c) * NS + 8, r + 8);
            tmem_wait_ld();
#pragma unroll
            for (int v = 0; v < NVT; v++)
                s[v] = fmaf(dk[c] * qsc[v * 4 + c], (float)(((int)r[2 * v] << 8) + (int)r[2 * v + 1]), s[v]);
        }
    }
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float mx = valid ? s[v] : -INFINITY;
        s[v] = mx;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[warp * 8 + v] = mx;
    }
    __syncthreads();  // (also: every thread has seen the score products complete: P^T may take the place of the K levels)
    float m[NVT], l[NVT], ps_inv[4], ps[4];
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float mx = red[128 + c];
#pragma unroll
        for (int wv = 1; wv < 8; wv++) mx = fmaxf(mx, red[128 + wv * 8 + c]);
        ps[c] = mx;
        ps_inv[c] = mx > 0.0f ? 65535.0f / mx : 0.0f;
    }
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
    // P^T: the B operand of O^T += V^T P^T, per half [NO rows][128 keys] uint8, K-major with the 128-byte swizzle: rows
    // ((c NVT + v) 2 + plane) hold the two planes of round(p[.][v] d_V[.][c] 65535 / ps[c]); it takes the place of the K levels
    if (h2 < nh) {
        uint8_t *pb = pt + h2 * (NO * 128) + (t & 15);
        const int ch = t >> 4;
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int v = 0; v < NVT; v++) {
                const uint32_t u16 = (uint32_t)__float2int_rn(fminf(e[v] * dv[c] * ps_inv[c], 65535.0f));
                const int rw = (c * NVT + v) * 2;
                pb[rw * 128 + ((ch ^ (rw & 7)) << 4)] = (uint8_t)(u16 >> 8);
                pb[(rw + 1) * 128 + ((ch ^ ((rw + 1) & 7)) << 4)] = (uint8_t)(u16 & 255u);
            }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float sum = red[64 + v];
#pragma unroll
        for (int wv = 1; wv < 8; wv++) sum += red[64 + wv * 8 + v];
        l[v] = sum;
    }

    // ---- O^T += V^T (half h) P^T (half h): 4 k-steps of 32 keys per half
    if (tid == 0) {
        tc_fence_after();
        constexpr uint32_t idesc_o = umma_idesc_i8(128, NO, 1, 0, 1, 0);
        for (int h = 0; h < nh; h++) {
            ok = mbar_wait_bounded(bars + h, 0, err, 73) && ok;  // (the half's V levels have landed)
#pragma unroll
            for (int ks = 0; ks < 4; ks++) {
                // A: rows of 128 bytes (one position, all 128 dims = one swizzle atom along MN), 8 positions = 1024 bytes (SBO); 32 keys
                // = 4096 bytes per k-step; B: the half's P^T rows, 32 keys = 32 bytes per k-step
                const uint64_t da = umma_desc(sbase + C::VLEV + h * 16384 + ks * 4096, 16, 1024, 2);
                const uint64_t db = umma_desc(sbase + C::PT + h * (NO * 128) + ks * 32, 16, 1024, 2);
                umma_i8(tbase + C::O_COL, da, db, idesc_o, (h > 0) | (ks > 0));
            }
        }
        umma_commit(bar_mma);
    }
    if (lane == 0) ok = mbar_wait_bounded(bar_mma, 1, err, 75) && ok;
    __syncwarp();
    tc_fence_after();

    // ---- the partial result of (row, head, block): o[hd] (unnormalised), m (in scaled-score units), l.  Thread = dim i of
    // group c = i / 32 (uniform over the warp): the columns (c, v, plane) of O
    ok = __all_sync(0xffffffffu, ok);
    if (warp < 4) {
        uint32_t r[2 * NVT < 8 ? 8 : 2 * NVT];
        tmem_ld8(lane_addr + C::O_COL + warp * 2 * NVT, r);
        if constexpr (NVT == 8) tmem_ld8(lane_addr + C::O_COL + warp * 2 * NVT + 8, r + 8);
        tmem_wait_ld();
        const float back = ps[warp] * (1.0f / 65535.0f);
#pragma unroll
        for (int v = 0; v < NVT; v++) {
            if (v < G) {
                float *p = part + ((size_t)(row.blk0 + b) * n_heads + (size_t)g * G + v) * RQ_PSTRIDE(HD);
                const float o = fmaf((float)(int)r[2 * v], 256.0f, (float)(int)r[2 * v + 1]) * back;
                p[tid] = ok ? o : 0.0f;  // (tid = TMEM lane = dim)
                if (tid == 0) {
                    p[HD] = m[v] * scale;
                    p[HD + 1] = l[v];
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(C::TM_COLS));
}

template <int NVT>
static cudaError_t launch_tc_one(const AttnPartTcArgs &a, cudaStream_t stream) {
    constexpr int smem = TcdCfg<NVT>::SMEM;
    static_assert(smem <= 227 * 1024, "one CTA's shared memory");
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = attn_part_tc_kernel<NVT>;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaError_t e = launch_pdl(tcd_q_prep_kernel, dim3(a.nrows, a.n_kv), dim3(128), 0, stream, a.rows, a.n_kv, a.G, a.q, a.qh, a.n_heads, a.qt, a.blk2row);
    if (e != cudaSuccess) return e;
    return launch_pdl(kern, dim3(a.total_blocks, a.n_kv), dim3(TCD_THREADS), (size_t)smem, stream, a.rows, (const int *)a.blk2row, (const uint8_t *)a.qt,
                      a.maps, a.layer, a.n_kv, a.G, a.n_heads, a.scale, a.part, a.err);
}

cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream) {
    if (a.G < 1 || a.G > 8) return cudaErrorInvalidValue;
    if (a.G == 1) return launch_tc_one<1>(a, stream);
    if (a.G == 2) return launch_tc_one<2>(a, stream);
    if (a.G <= 4) return launch_tc_one<4>(a, stream);
    return launch_tc_one<8>(a, stream);
}
#endif  // RQ_ATTN_DECODE_TC_INSTANTIATE

}  // namespace rq
