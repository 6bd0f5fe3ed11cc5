// Gated DeltaNet, chunked (WY / UT) form on the 5th-generation tensor cores (tcgen05 + TMEM): the prefill-sized
// counterpart of dn_rec_kernel.  Same inputs, outputs and state as the token recurrence (dn_rec_run, reference
// src/forward.c:2224; one token: S <- eg S + beta k (v - eg S^T k)^T, o = S^T q), re-associated per chunk of 64 tokens so
// that the work is dense products.  Operands are rounded to f16 (fp32 accumulation, fp32 state), so results agree with
// the CPU code to ~5e-4 relative, not bit for bit; dn_rec_kernel stays the exact form (decode, short segments).
//
// Per chunk, tokens i, j = 0 .. 63, g_i = product of eg up to token i (kept as a log2 sum; only ratios g_i / g_j <= 1
// with j <= i are ever formed), S0 the state at the chunk's start ([dk][dv]):
//     u_i  = beta_i (v_i - g_i S0^T k_i - sum_{j<i} (g_i / g_j)(k_i . k_j) u_j)          (the pseudo-values)
//  => U    = T' R,   R = B V - (B G K) S0,   T' = (I + A)^-1,  A_ij = beta_i (g_i / g_j)(k_i . k_j) for j < i
//     O    = (G Q) S0 + M U,                 M_ij = (g_i / g_j)(q_i . k_j) for j <= i
//     S    = g_63 S0 + Kt^T U,               Kt_j = (g_63 / g_j) k_j
// One CTA per (segment, value head, half of the dv columns): the two halves of a head are independent given K and Q, so
// they run on two SMs (each repeats the small K / Q products).  256 threads; warps w and w + 4 own TMEM lanes
// 32 (w % 4) .. + 31 and split the columns.  Steps of a chunk:
//   0  rows -> f16 operands in shared memory (the scaled copies above), gates -> log2 prefix sums; the next chunk's rows
//      are prefetched into L2; S (TMEM, fp32) -> f16 copy in shared memory, and S *= g_63 in place
//   1  MMA: K K^T and Q K^T (N = 64) | -(B G K) S0 and (G Q) S0, which need nothing of this chunk but the operands
//   2  A (fp32) and M (f16) from the first two products, masked and decayed
//   3  T' by blocks of 16 (forward substitution on the diagonal blocks, block products below them) -> f16;
//      R = B V - (B G K) S0 -> f16
//   4  MMA: U = T' R
//   5  U -> f16 in shared memory
//   6  MMA: O += M U;  S += Kt^T U
//   7  O -> global memory through shared memory (coalesced rows)
// All MMAs are M = 128 (rows 64 .. 127 of the token-indexed products are never read).  Every operand buffer has the
// same physical layout, [64-column half][row][128 bytes] with the 128-byte swizzle, which serves as a K-major operand
// (row = M or N index) and as an MN-major one (row = K index) alike.
#pragma once
#include "tc05.cuh"

namespace rq {

constexpr int DNC_C = 64;  // tokens per chunk
constexpr int DNC_THREADS = 256;

struct DnChunkArgs {
    const DnSeg *segs;
    int nseg, lin_layer, nk, nv;
    size_t conv_floats;
    const float *rows;
    int lw;
    float *out;
    int *err;
};
// launches dn_chunk_kernel (grid: 2 x value heads, segments) on `stream`; dk = dv = 128 only
cudaError_t launch_dn_chunk(const DnChunkArgs &a, cudaStream_t stream);

#ifdef RQ_DN_CHUNK_INSTANTIATE
namespace dnc {
// shared-memory map (bytes from a 1024-byte aligned base)
constexpr int K16 = 0, Q16 = 16384, GQ16 = 32768, NBGK16 = 49152, KT16 = 65536, T16 = 81920, M16 = 90112, BV32 = 98304, R16 = 114688,
              U16 = 122880, S16 = 131072, AF = 147456, AST = 68, XF = AF + 64 * AST * 4, PF = XF + 64 * AST * 4, LG = PF + 16 * AST * 4, BETA = LG + 256, BAR = BETA + 256, SLOT = BAR + 16,
              END = SLOT + 16;
constexpr int SMEM = END + 1024;  // (BAR holds two barriers)
constexpr int HV = 64;  // dv columns per CTA
constexpr int S_COL = 0, Y_COL = 64, Z_COL = 128, X_COL = 256;
}  // namespace dnc

// 4 adjacent values (dims 4 lane .. 4 lane + 3 of row `row`) -> the swizzled f16 operand layout of a 64-row buffer
__device__ __forceinline__ void dnc_store4(uint8_t *buf, int row, int lane, float a, float b, float c, float d) {
    __half2 h0 = __floats2half2_rn(a, b), h1 = __floats2half2_rn(c, d);
    const int ch = lane >> 1;
    *reinterpret_cast<uint2 *>(buf + (ch >> 3) * 8192 + row * 128 + (((ch & 7) ^ (row & 7)) << 4) + (lane & 1) * 8) =
        make_uint2(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1));
}
__device__ __forceinline__ uint32_t dnc_pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
// 32 adjacent fp32 values r (columns 32 cb .. 32 cb + 31 of row `row`) -> f16 in a buffer of 128-byte rows
__device__ __forceinline__ void dnc_store_row32(uint8_t *buf, int row, int cb, const float *r) {
#pragma unroll
    for (int x = 0; x < 4; x++) {
        const int ch = 4 * cb + x;
        uint4 w;
        w.x = dnc_pack(r[8 * x], r[8 * x + 1]), w.y = dnc_pack(r[8 * x + 2], r[8 * x + 3]);
        w.z = dnc_pack(r[8 * x + 4], r[8 * x + 5]), w.w = dnc_pack(r[8 * x + 6], r[8 * x + 7]);
        *reinterpret_cast<uint4 *>(buf + row * 128 + ((ch ^ (row & 7)) << 4)) = w;
    }
}

__global__ void __launch_bounds__(DNC_THREADS, 1) dn_chunk_kernel(const DnSeg *__restrict__ segs, int lin_layer, int nk, int nv, size_t conv_floats,
                                                               const float *__restrict__ rows, int lw, float *__restrict__ out, int *err) {
    using namespace dnc;
    constexpr int DK = 128, DV = 128, C = DNC_C;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *s_a = reinterpret_cast<float *>(sm + AF), *s_lg = reinterpret_cast<float *>(sm + LG), *s_beta = reinterpret_cast<float *>(sm + BETA);
    float *s_bv = reinterpret_cast<float *>(sm + BV32);  // [token][HV] beta v
    uint64_t *bar = reinterpret_cast<uint64_t *>(sm + BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + SLOT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x >> 1, hv = blockIdx.x & 1;  // value head, which half of its dv columns
    const int trow = (warp & 3) * 32 + lane, cb = warp >> 2;  // this thread's TMEM lane and its 32-column block of a 64-column tile
    const DnSeg sg = segs[blockIdx.y];
    const int conv_dim = 2 * nk * DK + nv * DV, vdim = nv * DV;
    const size_t oq = (size_t)(h % nk) * DK, okk = (size_t)nk * DK + oq, ov = (size_t)2 * nk * DK + (size_t)h * DV + (size_t)hv * HV;
    const size_t oe = (size_t)conv_dim + vdim + h, ob = oe + nv;
    // the CTA's part of the state: blocks 2 hv, 2 hv + 1 of [dv / 32][dk][32]
    float *Sg = sg.state + (size_t)lin_layer * sg.lstride + conv_floats + (size_t)h * DK * DV + (size_t)hv * 2 * DK * 32;

    if (tid == 0) {
        mbar_init(bar, 1);      // the chunk's products 1a, 4 and 6, each waited for by every thread before the next is issued
        mbar_init(bar + 1, 1);  // product 1b (issued right behind 1a: a barrier of its own keeps the parity waits unambiguous)
        mbar_fence_init();
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;
    uint32_t phase = 0, phase_b = 0;

    // the state -> TMEM: thread (trow, cb) holds columns 32 cb .. + 31 of row trow of S ([dk][HV])
    {
        uint32_t r[32];
        const float4 *src = reinterpret_cast<const float4 *>(Sg + (size_t)cb * DK * 32 + (size_t)trow * 32);
#pragma unroll
        for (int x = 0; x < 8; x++) {
            float4 v = sg.first ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : src[x];
            r[4 * x] = __float_as_uint(v.x), r[4 * x + 1] = __float_as_uint(v.y), r[4 * x + 2] = __float_as_uint(v.z), r[4 * x + 3] = __float_as_uint(v.w);
        }
        tmem_st32(lane_addr + S_COL + cb * 32, r);
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    const uint32_t sbase = smem_u32(sm);
    constexpr uint32_t id_kk = umma_idesc(128, 64, 0, 0), id_kmn = umma_idesc(128, 64, 0, 1), id_mnmn = umma_idesc(128, 64, 1, 1);
    // K-major operand of a 64-row, 128-column buffer, k-step ks of 16 columns
    auto d_k128 = [&](int buf, int ks) { return umma_desc(sbase + buf + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024, 2); };
    // K-major operand of a 64-column buffer (one 128-byte row per M index)
    auto d_k64 = [&](int buf, int ks) { return umma_desc(sbase + buf + ks * 32, 16, 1024, 2); };
    // MN-major operand, rows = K index (k-step ks = 16 rows), `half` = bytes between the 64-column halves (if it has two)
    auto d_mn = [&](int buf, int ks, int half) { return umma_desc(sbase + buf + ks * 2048, half, 1024, 2); };
    auto wait_mma = [&]() {
        ok = mbar_wait_bounded(bar, phase, err, 31) && ok;
        phase ^= 1;
        tc_fence_after();
    };

    for (int c0 = 0; c0 < sg.n; c0 += C) {
        const int cnt = min(C, sg.n - c0);
        // ---- 0: gates -> inclusive log2 prefix sums; rows -> f16 operands; the state's f16 copy and its decay
        if (warp == 0) {
            const float *r0 = rows + (size_t)(sg.row0 + c0 + lane) * lw, *r1 = r0 + (size_t)32 * lw;
            float a0 = lane < cnt ? fmaxf(log2f(r0[oe]), -1.0e4f) : 0.0f, a1 = lane + 32 < cnt ? fmaxf(log2f(r1[oe]), -1.0e4f) : 0.0f;
            s_beta[lane] = lane < cnt ? r0[ob] : 0.0f;
            s_beta[lane + 32] = lane + 32 < cnt ? r1[ob] : 0.0f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float b0 = __shfl_up_sync(0xffffffffu, a0, o), b1 = __shfl_up_sync(0xffffffffu, a1, o);
                if (lane >= o) a0 += b0, a1 += b1;
            }
            a1 += __shfl_sync(0xffffffffu, a0, 31);
            s_lg[lane] = a0;
            s_lg[lane + 32] = a1;
        }
        float4 qv[8], kv[8], vv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int j = warp * 8 + i;
            qv[i] = kv[i] = vv[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (j < cnt) {
                const float *r = rows + (size_t)(sg.row0 + c0 + j) * lw;
                qv[i] = __ldg(reinterpret_cast<const float4 *>(r + oq) + lane);
                kv[i] = __ldg(reinterpret_cast<const float4 *>(r + okk) + lane);
                if (lane < HV / 4) vv[i] = __ldg(reinterpret_cast<const float4 *>(r + ov) + lane);
            }
            if (j + C < sg.n - c0 && (lane & 7) == 0) {  // the same row of the next chunk -> L2
                const float *rn = rows + (size_t)(sg.row0 + c0 + C + j) * lw;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(rn + oq + 4 * lane));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(rn + okk + 4 * lane));
                if (lane < HV / 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(rn + ov + 4 * lane));
            }
        }
        __syncthreads();  // (the gates; and every thread is past the previous chunk's output staging)
        const float lgc = s_lg[C - 1];
        {
            // S (the previous chunk's result) -> its f16 copy, the B operand of this chunk's S0 products; S *= g_63
            uint32_t r[32];
            tmem_ld32(lane_addr + S_COL + cb * 32, r);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int x = 0; x < 32; x++) f[x] = __uint_as_float(r[x]);
            dnc_store_row32(sm + S16, trow, cb, f);
            const float gc = ex2(lgc);
#pragma unroll
            for (int x = 0; x < 32; x++) r[x] = __float_as_uint(f[x] * gc);
            tmem_st32(lane_addr + S_COL + cb * 32, r);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int j = warp * 8 + i;
            const float gam = ex2(s_lg[j]), bet = s_beta[j], nbg = -bet * gam, kt = ex2(lgc - s_lg[j]);
            dnc_store4(sm + K16, j, lane, kv[i].x, kv[i].y, kv[i].z, kv[i].w);
            dnc_store4(sm + Q16, j, lane, qv[i].x, qv[i].y, qv[i].z, qv[i].w);
            dnc_store4(sm + GQ16, j, lane, qv[i].x * gam, qv[i].y * gam, qv[i].z * gam, qv[i].w * gam);
            dnc_store4(sm + NBGK16, j, lane, kv[i].x * nbg, kv[i].y * nbg, kv[i].z * nbg, kv[i].w * nbg);
            dnc_store4(sm + KT16, j, lane, kv[i].x * kt, kv[i].y * kt, kv[i].z * kt, kv[i].w * kt);
            if (lane < HV / 4)
                *reinterpret_cast<float4 *>(s_bv + j * HV + 4 * lane) = make_float4(vv[i].x * bet, vv[i].y * bet, vv[i].z * bet, vv[i].w * bet);
        }
        tmem_wait_st();
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- 1: K K^T and Q K^T -> X; -(B G K) S0 -> Y and (G Q) S0 -> Z
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + X_COL, d_k128(K16, ks), d_k128(K16, ks), id_kk, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + X_COL + 64, d_k128(Q16, ks), d_k128(K16, ks), id_kk, ks > 0);
            umma_commit(bar);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + Y_COL, d_k128(NBGK16, ks), d_mn(S16, ks, 0), id_kmn, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + Z_COL, d_k128(GQ16, ks), d_mn(S16, ks, 0), id_kmn, ks > 0);
            umma_commit(bar + 1);
        }
        wait_mma();
        // ---- 2: A (fp32, strictly lower) and M (f16, lower with the diagonal): row i, columns 32 cb .. + 31 per thread
        if ((warp & 3) < 2) {
            uint32_t g[32], mq[32];
            tmem_ld32(lane_addr + X_COL + cb * 32, g);
            tmem_ld32(lane_addr + X_COL + 64 + cb * 32, mq);
            tmem_wait_ld();
            const int i = trow;
            const float lgi = s_lg[i], bi = s_beta[i];
            float mv[32];
#pragma unroll
            for (int x = 0; x < 32; x++) {
                const int j = 32 * cb + x;
                const float ratio = j <= i ? ex2(lgi - s_lg[j]) : 0.0f;
                s_a[i * AST + j] = j < i ? bi * ratio * __uint_as_float(g[x]) : 0.0f;
                mv[x] = j <= i ? ratio * __uint_as_float(mq[x]) : 0.0f;
            }
            dnc_store_row32(sm + M16, i, cb, mv);
        }
        tc_fence_before();
        __syncthreads();
        // ---- 3: T' = (I + A)^-1 by blocks of 16: the four diagonal blocks by forward substitution (a column per thread),
        // then block row by block row T'_ij = -T'_ii (sum_{k=j}^{i-1} A_ik T'_kj), 256 threads on a 16 x 16 block each time
        {
            float *s_x = reinterpret_cast<float *>(sm + XF), *s_p = reinterpret_cast<float *>(sm + PF);
            if (tid < 64) {
                const int b = tid >> 4, c = tid & 15;
                float x[16];
#pragma unroll
                for (int r = 0; r < 16; r++) {
                    float acc = r == c ? 1.0f : 0.0f;
#pragma unroll
                    for (int q = 0; q < r; q++) acc = fmaf(-s_a[(16 * b + r) * AST + 16 * b + q], x[q], acc);
                    x[r] = acc;
                    s_x[(16 * b + r) * AST + 16 * b + c] = acc;
                }
            }
            __syncthreads();
            const int r = tid >> 4, c = tid & 15;
#pragma unroll
            for (int i = 1; i < 4; i++) {
                const float *arow = s_a + (16 * i + r) * AST;
#pragma unroll
                for (int j = 0; j < i; j++) {
                    float p = 0.0f;
#pragma unroll
                    for (int k4 = 4 * j; k4 < 4 * i; k4++) {
                        const float4 a4 = *reinterpret_cast<const float4 *>(arow + 4 * k4);
                        p = fmaf(a4.x, s_x[(4 * k4) * AST + 16 * j + c], p);
                        p = fmaf(a4.y, s_x[(4 * k4 + 1) * AST + 16 * j + c], p);
                        p = fmaf(a4.z, s_x[(4 * k4 + 2) * AST + 16 * j + c], p);
                        p = fmaf(a4.w, s_x[(4 * k4 + 3) * AST + 16 * j + c], p);
                    }
                    s_p[r * AST + 16 * j + c] = p;
                }
                __syncthreads();
                const float *drow = s_x + (16 * i + r) * AST + 16 * i;  // row r of T'_ii
#pragma unroll
                for (int j = 0; j < i; j++) {
                    float x = 0.0f;
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        const float4 d4 = *reinterpret_cast<const float4 *>(drow + 4 * q4);
                        x = fmaf(-d4.x, s_p[(4 * q4) * AST + 16 * j + c], x);
                        x = fmaf(-d4.y, s_p[(4 * q4 + 1) * AST + 16 * j + c], x);
                        x = fmaf(-d4.z, s_p[(4 * q4 + 2) * AST + 16 * j + c], x);
                        x = fmaf(-d4.w, s_p[(4 * q4 + 3) * AST + 16 * j + c], x);
                    }
                    s_x[(16 * i + r) * AST + 16 * j + c] = x;
                }
                __syncthreads();
            }
            // -> f16, K-major rows of 64: thread (row, 16-column block), zero above the diagonal blocks
            const int row = tid >> 2, jb = tid & 3;
            float f[16];
#pragma unroll
            for (int q = 0; q < 16; q++) f[q] = jb <= (row >> 4) ? s_x[row * AST + 16 * jb + q] : 0.0f;
#pragma unroll
            for (int q = 0; q < 2; q++) {
                uint4 w;
                w.x = dnc_pack(f[8 * q], f[8 * q + 1]), w.y = dnc_pack(f[8 * q + 2], f[8 * q + 3]);
                w.z = dnc_pack(f[8 * q + 4], f[8 * q + 5]), w.w = dnc_pack(f[8 * q + 6], f[8 * q + 7]);
                *reinterpret_cast<uint4 *>(sm + T16 + row * 128 + (((2 * jb + q) ^ (row & 7)) << 4)) = w;
            }
        }
        ok = mbar_wait_bounded(bar + 1, phase_b, err, 32) && ok;  // (the S0 products)
        phase_b ^= 1;
        tc_fence_after();
        // R = B V - (B G K) S0 -> f16: row j, columns 32 cb .. + 31 per thread
        if ((warp & 3) < 2) {
            uint32_t r[32];
            tmem_ld32(lane_addr + Y_COL + cb * 32, r);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
                const float4 b = *reinterpret_cast<const float4 *>(s_bv + trow * HV + 32 * cb + x);
                f[x] = b.x + __uint_as_float(r[x]), f[x + 1] = b.y + __uint_as_float(r[x + 1]);
                f[x + 2] = b.z + __uint_as_float(r[x + 2]), f[x + 3] = b.w + __uint_as_float(r[x + 3]);
            }
            dnc_store_row32(sm + R16, trow, cb, f);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- 4: U = T' R -> Y
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + Y_COL, d_k64(T16, ks), d_mn(R16, ks, 0), id_kmn, ks > 0);
            umma_commit(bar);
        }
        wait_mma();
        // ---- 5: U -> f16
        if ((warp & 3) < 2) {
            uint32_t r[32];
            tmem_ld32(lane_addr + Y_COL + cb * 32, r);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int x = 0; x < 32; x++) f[x] = __uint_as_float(r[x]);
            dnc_store_row32(sm + U16, trow, cb, f);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- 6: O += M U -> Z;  S += Kt^T U
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + Z_COL, d_k64(M16, ks), d_mn(U16, ks, 0), id_kmn, 1);
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + S_COL, d_mn(KT16, ks, 8192), d_mn(U16, ks, 0), id_mnmn, 1);
            umma_commit(bar);
        }
        wait_mma();
        // ---- 7: O rows -> global memory, staged through shared memory (over K16, which no MMA reads any more)
        {
            constexpr int OST = HV + 4;
            float *so = reinterpret_cast<float *>(sm);
            if ((warp & 3) < 2) {
                uint32_t r[32];
                tmem_ld32(lane_addr + Z_COL + cb * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int y = 0; y < 32; y += 4)
                    *reinterpret_cast<float4 *>(so + (size_t)trow * OST + cb * 32 + y) =
                        make_float4(__uint_as_float(r[y]), __uint_as_float(r[y + 1]), __uint_as_float(r[y + 2]), __uint_as_float(r[y + 3]));
            }
            tc_fence_before();
            __syncthreads();
            // a warp writes two rows of 256 bytes per step
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = warp * 8 + 2 * i + (lane >> 4), l16 = lane & 15;
                if (j < cnt)
                    *reinterpret_cast<float4 *>(out + (size_t)(sg.row0 + c0 + j) * vdim + (size_t)h * DV + (size_t)hv * HV + 4 * l16) =
                        ok ? *reinterpret_cast<const float4 *>(so + (size_t)j * OST + 4 * l16) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    }
    // the state back to global memory
    tc_fence_after();
    {
        uint32_t r[32];
        tmem_ld32(lane_addr + S_COL + cb * 32, r);
        tmem_wait_ld();
        float4 *dst = reinterpret_cast<float4 *>(Sg + (size_t)cb * DK * 32 + (size_t)trow * 32);
#pragma unroll
        for (int x = 0; x < 8; x++)
            dst[x] = make_float4(__uint_as_float(r[4 * x]), __uint_as_float(r[4 * x + 1]), __uint_as_float(r[4 * x + 2]), __uint_as_float(r[4 * x + 3]));
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(512));
}

cudaError_t launch_dn_chunk(const DnChunkArgs &a, cudaStream_t stream) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(dn_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dnc::SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    dn_chunk_kernel<<<dim3(2 * a.nv, a.nseg), DNC_THREADS, dnc::SMEM, stream>>>(a.segs, a.lin_layer, a.nk, a.nv, a.conv_floats, a.rows, a.lw, a.out, a.err);
    return cudaGetLastError();
}
#endif  // RQ_DN_CHUNK_INSTANTIATE

}  // namespace rq
