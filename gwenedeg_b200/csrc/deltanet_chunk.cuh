// Gated DeltaNet, chunked (WY / UT) form on the 5th-generation tensor cores (tcgen05 + TMEM): the prefill-sized
// counterpart of dn_rec_kernel.  Same inputs, outputs and state as the token recurrence (dn_rec_run, reference
// src/forward.c:2224; one token: S <- eg S + beta k (v - eg S^T k)^T, o = S^T q), re-associated per chunk of 64 tokens so
// that the work is dense products.  Operands are rounded to f16 (fp32 accumulation, fp32 state), so results agree with
// the CPU code to ~5e-4 relative, not bit for bit; dn_rec_kernel stays the exact form (decode, short segments).
//
// Per chunk, tokens i, j = 0 .. 63, g_i = product of eg up to token i (kept as a log2 sum; only ratios g_i / g_j <= 1
// with j <= i are ever formed), S0 the state at the chunk's start ([dk][dv]):
//     u_i  = beta_i (v_i - g_i S0^T k_i - sum_{j<i} (g_i / g_j)(k_i . k_j) u_j)          (the pseudo-values)
//  => U    = T' (B V) - (T' (B G K)) S0,   T' = (I + A)^-1,  A_ij = beta_i (g_i / g_j)(k_i . k_j) for j < i
//     O    = (G Q) S0 + M U,               M_ij = (g_i / g_j)(q_i . k_j) for j <= i
//     S    = g_63 S0 + Kt^T U,             Kt_j = (g_63 / g_j) k_j
// One CTA per (segment, value head), 256 threads; thread t < 128 owns TMEM lane t.  Steps of a chunk:
//   0  rows -> f16 operands in shared memory (all the scaled copies above), gates -> log2 prefix sums
//   1  MMA: K K^T and Q K^T (N = 64);  meanwhile S (TMEM, fp32) -> f16 copy in shared memory, and S *= g_63 in place
//   2  A (fp32) and M (f16) from the two products, masked and decayed
//   3  T' by forward substitution, one column per thread, -> f16
//   4  MMA: W = T' (B G K), Uv = T' (B V)
//   5  -W -> f16 pairs in TMEM (the A operand of the next product)
//   6  MMA: U = Uv + (-W) S0
//   7  U -> f16 in shared memory
//   8  MMA: O = (G Q) S0 + M U;  S += Kt^T U
//   9  O -> global memory through shared memory (coalesced rows)
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
// launches dn_chunk_kernel (grid: value heads x segments) on `stream`; dk = dv = 128 only
cudaError_t launch_dn_chunk(const DnChunkArgs &a, cudaStream_t stream);

#ifdef RQ_DN_CHUNK_INSTANTIATE
namespace dnc {
// shared-memory map (bytes from a 1024-byte aligned base)
constexpr int K16 = 0, Q16 = 16384, GQ16 = 32768, T16 = 49152, M16 = 57344, BGK16 = 65536, BV16 = 81920, KT16 = 98304, U16 = 114688,
              S16 = 131072, AF = 163840, AST = 68, LG = AF + 64 * AST * 4, BETA = LG + 256, BAR = BETA + 256, SLOT = BAR + 16,
              END = SLOT + 16;
constexpr int SMEM = END + 1024;
constexpr int S_COL = 0, X_COL = 128, Y_COL = 256, Z_COL = 384;
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

__global__ void __launch_bounds__(DNC_THREADS, 1) dn_chunk_kernel(const DnSeg *__restrict__ segs, int lin_layer, int nk, int nv, size_t conv_floats,
                                                               const float *__restrict__ rows, int lw, float *__restrict__ out, int *err) {
    using namespace dnc;
    constexpr int DK = 128, DV = 128, C = DNC_C;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *s_a = reinterpret_cast<float *>(sm + AF), *s_lg = reinterpret_cast<float *>(sm + LG), *s_beta = reinterpret_cast<float *>(sm + BETA);
    uint64_t *bar = reinterpret_cast<uint64_t *>(sm + BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + SLOT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x;
    const DnSeg sg = segs[blockIdx.y];
    const int conv_dim = 2 * nk * DK + nv * DV, vdim = nv * DV;
    const size_t oq = (size_t)(h % nk) * DK, okk = (size_t)nk * DK + oq, ov = (size_t)2 * nk * DK + (size_t)h * DV;
    const size_t oe = (size_t)conv_dim + vdim + h, ob = oe + nv;
    float *Sg = sg.state + (size_t)lin_layer * sg.lstride + conv_floats + (size_t)h * DK * DV;  // [dv / 32][dk][32]

    if (tid == 0) {
        mbar_init(bar, 1);
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
    uint32_t phase = 0;

    // the state -> TMEM: thread d holds row d of S ([dk][dv])
    if (tid < 128) {
#pragma unroll 1
        for (int jb = 0; jb < DV / 32; jb++) {
            uint32_t r[32];
            const float4 *src = reinterpret_cast<const float4 *>(Sg + (size_t)jb * DK * 32 + (size_t)tid * 32);
#pragma unroll
            for (int x = 0; x < 8; x++) {
                float4 v = sg.first ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : src[x];
                r[4 * x] = __float_as_uint(v.x), r[4 * x + 1] = __float_as_uint(v.y), r[4 * x + 2] = __float_as_uint(v.z), r[4 * x + 3] = __float_as_uint(v.w);
            }
            tmem_st32(lane_addr + S_COL + jb * 32, r);
        }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    const uint32_t sbase = smem_u32(sm);
    constexpr uint32_t id_n64 = umma_idesc(128, 64, 0, 0), id_kmn = umma_idesc(128, 128, 0, 1), id_mnmn = umma_idesc(128, 128, 1, 1);
    // K-major operand of a 64-row, 128-column buffer, k-step ks of 16 columns
    auto d_k128 = [&](int buf, int ks) { return umma_desc(sbase + buf + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024, 2); };
    // K-major operand of a 64-column buffer (one 128-byte row per M index)
    auto d_k64 = [&](int buf, int ks) { return umma_desc(sbase + buf + ks * 32, 16, 1024, 2); };
    // MN-major operand, rows = K index (k-step ks = 16 rows), `half` = bytes between the two 64-column halves
    auto d_mn = [&](int buf, int ks, int half) { return umma_desc(sbase + buf + ks * 2048, half, 1024, 2); };
    auto wait_mma = [&]() {
        ok = mbar_wait_bounded(bar, phase, err, 31) && ok;
        phase ^= 1;
        tc_fence_after();
    };

    for (int c0 = 0; c0 < sg.n; c0 += C) {
        const int cnt = min(C, sg.n - c0);
        // ---- 0: gates -> inclusive log2 prefix sums; rows -> f16 operands
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
                vv[i] = __ldg(reinterpret_cast<const float4 *>(r + ov) + lane);
            }
        }
        __syncthreads();  // (the gates; and every thread is past the previous chunk's output staging)
        const float lgc = s_lg[C - 1];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int j = warp * 8 + i;
            const float gam = ex2(s_lg[j]), bet = s_beta[j], bg = bet * gam, kt = ex2(lgc - s_lg[j]);
            dnc_store4(sm + K16, j, lane, kv[i].x, kv[i].y, kv[i].z, kv[i].w);
            dnc_store4(sm + Q16, j, lane, qv[i].x, qv[i].y, qv[i].z, qv[i].w);
            dnc_store4(sm + GQ16, j, lane, qv[i].x * gam, qv[i].y * gam, qv[i].z * gam, qv[i].w * gam);
            dnc_store4(sm + BGK16, j, lane, kv[i].x * bg, kv[i].y * bg, kv[i].z * bg, kv[i].w * bg);
            dnc_store4(sm + BV16, j, lane, vv[i].x * bet, vv[i].y * bet, vv[i].z * bet, vv[i].w * bet);
            dnc_store4(sm + KT16, j, lane, kv[i].x * kt, kv[i].y * kt, kv[i].z * kt, kv[i].w * kt);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- 1: K K^T and Q K^T; meanwhile the state's f16 copy and its decay
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + X_COL, d_k128(K16, ks), d_k128(K16, ks), id_n64, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + X_COL + 64, d_k128(Q16, ks), d_k128(K16, ks), id_n64, ks > 0);
            umma_commit(bar);
        }
        if (tid < 128) {
            const float gc = ex2(lgc);
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t r[32];
                tmem_ld32(lane_addr + S_COL + cc * 32, r);
                tmem_wait_ld();
                // row tid of the 128-row buffer: 16-byte chunks 4 cc .. 4 cc + 3 (8 values each)
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int ch = 4 * cc + x;
                    uint4 w;
                    w.x = dnc_pack(__uint_as_float(r[8 * x]), __uint_as_float(r[8 * x + 1]));
                    w.y = dnc_pack(__uint_as_float(r[8 * x + 2]), __uint_as_float(r[8 * x + 3]));
                    w.z = dnc_pack(__uint_as_float(r[8 * x + 4]), __uint_as_float(r[8 * x + 5]));
                    w.w = dnc_pack(__uint_as_float(r[8 * x + 6]), __uint_as_float(r[8 * x + 7]));
                    *reinterpret_cast<uint4 *>(sm + S16 + (ch >> 3) * 16384 + tid * 128 + (((ch & 7) ^ (tid & 7)) << 4)) = w;
                }
#pragma unroll
                for (int x = 0; x < 32; x++) r[x] = __float_as_uint(__uint_as_float(r[x]) * gc);
                tmem_st32(lane_addr + S_COL + cc * 32, r);
            }
            tmem_wait_st();
            fence_proxy_async();
        }
        wait_mma();
        // ---- 2: A (fp32, strictly lower) and M (f16, lower with the diagonal), row i per thread
        if (tid < 64) {
            uint32_t g[64], mq[64];
            tmem_ld32(lane_addr + X_COL, g);
            tmem_ld32(lane_addr + X_COL + 32, g + 32);
            tmem_ld32(lane_addr + X_COL + 64, mq);
            tmem_ld32(lane_addr + X_COL + 96, mq + 32);
            tmem_wait_ld();
            const int i = tid;
            const float lgi = s_lg[i], bi = s_beta[i];
#pragma unroll
            for (int j8 = 0; j8 < 8; j8++) {
                float av[8], mv[8];
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int j = 8 * j8 + x;
                    const float ratio = j <= i ? ex2(lgi - s_lg[j]) : 0.0f;
                    av[x] = j < i ? bi * ratio * __uint_as_float(g[j]) : 0.0f;
                    mv[x] = j <= i ? ratio * __uint_as_float(mq[j]) : 0.0f;
                }
                *reinterpret_cast<float4 *>(s_a + i * AST + 8 * j8) = make_float4(av[0], av[1], av[2], av[3]);
                *reinterpret_cast<float4 *>(s_a + i * AST + 8 * j8 + 4) = make_float4(av[4], av[5], av[6], av[7]);
                uint4 w;
                w.x = dnc_pack(mv[0], mv[1]), w.y = dnc_pack(mv[2], mv[3]), w.z = dnc_pack(mv[4], mv[5]), w.w = dnc_pack(mv[6], mv[7]);
                *reinterpret_cast<uint4 *>(sm + M16 + i * 128 + ((j8 ^ (i & 7)) << 4)) = w;
            }
        }
        tc_fence_before();
        __syncthreads();
        // ---- 3: T' = (I + A)^-1, column `tid` per thread: x_i = [i == col] - sum_{j<i} A_ij x_j
        if (tid < 64) {
            float x[64];
#pragma unroll
            for (int i = 0; i < 64; i++) {
                float acc[4] = {i == tid ? 1.0f : 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int j4 = 0; j4 < (i + 3) / 4; j4++) {
                    const float4 a4 = *reinterpret_cast<const float4 *>(s_a + i * AST + 4 * j4);  // (entries j >= i are zero)
                    const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                    for (int y = 0; y < 4; y++)
                        if (4 * j4 + y < i) acc[y] = fmaf(-av[y], x[4 * j4 + y], acc[y]);
                }
                x[i] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                *reinterpret_cast<__half *>(sm + T16 + i * 128 + (((tid >> 3) ^ (i & 7)) << 4) + (tid & 7) * 2) = __float2half_rn(x[i]);
            }
        }
        fence_proxy_async();
        __syncthreads();
        // ---- 4: W = T' (B G K) -> X, Uv = T' (B V) -> Y
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + X_COL, d_k64(T16, ks), d_mn(BGK16, ks, 8192), id_kmn, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + Y_COL, d_k64(T16, ks), d_mn(BV16, ks, 8192), id_kmn, ks > 0);
            umma_commit(bar);
        }
        wait_mma();
        // ---- 5: -W as f16 pairs over the first 64 columns of X
        if (tid < 128) {
#pragma unroll 1
            for (int hf = 0; hf < 2; hf++) {
                uint32_t r[64], p[32];
                tmem_ld32(lane_addr + X_COL + hf * 64, r);
                tmem_ld32(lane_addr + X_COL + hf * 64 + 32, r + 32);
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 32; x++) p[x] = dnc_pack(-__uint_as_float(r[2 * x]), -__uint_as_float(r[2 * x + 1]));
                tmem_st32(lane_addr + X_COL + hf * 32, p);
            }
            tmem_wait_st();
        }
        tc_fence_before();
        __syncthreads();
        // ---- 6: U = Uv + (-W) S0
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ts(tbase + Y_COL, tbase + X_COL + ks * 8, d_mn(S16, ks, 16384), id_kmn, 1);
            umma_commit(bar);
        }
        wait_mma();
        // ---- 7: U -> f16, row j per thread
        if (tid < 64) {
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t r[32];
                tmem_ld32(lane_addr + Y_COL + cc * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int ch = 4 * cc + x;
                    uint4 w;
                    w.x = dnc_pack(__uint_as_float(r[8 * x]), __uint_as_float(r[8 * x + 1]));
                    w.y = dnc_pack(__uint_as_float(r[8 * x + 2]), __uint_as_float(r[8 * x + 3]));
                    w.z = dnc_pack(__uint_as_float(r[8 * x + 4]), __uint_as_float(r[8 * x + 5]));
                    w.w = dnc_pack(__uint_as_float(r[8 * x + 6]), __uint_as_float(r[8 * x + 7]));
                    *reinterpret_cast<uint4 *>(sm + U16 + (ch >> 3) * 8192 + tid * 128 + (((ch & 7) ^ (tid & 7)) << 4)) = w;
                }
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- 8: O = (G Q) S0 + M U -> Z;  S += Kt^T U
        if (tid == 128) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + Z_COL, d_k128(GQ16, ks), d_mn(S16, ks, 16384), id_kmn, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + Z_COL, d_k64(M16, ks), d_mn(U16, ks, 8192), id_kmn, 1);
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + S_COL, d_mn(KT16, ks, 8192), d_mn(U16, ks, 8192), id_mnmn, 1);
            umma_commit(bar);
        }
        wait_mma();
        // ---- 9: O rows -> global memory, staged through shared memory (over K16 .. GQ16, which no MMA reads any more)
        {
            constexpr int OST = DV + 4;
            float *so = reinterpret_cast<float *>(sm);
            if (tid < 64) {
#pragma unroll 1
                for (int cc = 0; cc < 4; cc++) {
                    uint32_t r[32];
                    tmem_ld32(lane_addr + Z_COL + cc * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int y = 0; y < 32; y += 4)
                        *reinterpret_cast<float4 *>(so + (size_t)tid * OST + cc * 32 + y) =
                            make_float4(__uint_as_float(r[y]), __uint_as_float(r[y + 1]), __uint_as_float(r[y + 2]), __uint_as_float(r[y + 3]));
                }
            }
            tc_fence_before();
            __syncthreads();
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int j = warp * 8 + i;
                if (j < cnt)
                    *reinterpret_cast<float4 *>(out + (size_t)(sg.row0 + c0 + j) * vdim + (size_t)h * DV + 4 * lane) =
                        ok ? *reinterpret_cast<const float4 *>(so + (size_t)j * OST + 4 * lane) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    }
    // the state back to global memory
    tc_fence_after();
    if (tid < 128) {
#pragma unroll 1
        for (int jb = 0; jb < DV / 32; jb++) {
            uint32_t r[32];
            tmem_ld32(lane_addr + S_COL + jb * 32, r);
            tmem_wait_ld();
            float4 *dst = reinterpret_cast<float4 *>(Sg + (size_t)jb * DK * 32 + (size_t)tid * 32);
#pragma unroll
            for (int x = 0; x < 8; x++)
                dst[x] = make_float4(__uint_as_float(r[4 * x]), __uint_as_float(r[4 * x + 1]), __uint_as_float(r[4 * x + 2]), __uint_as_float(r[4 * x + 3]));
        }
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
    dn_chunk_kernel<<<dim3(a.nv, a.nseg), DNC_THREADS, dnc::SMEM, stream>>>(a.segs, a.lin_layer, a.nk, a.nv, a.conv_floats, a.rows, a.lw, a.out, a.err);
    return cudaGetLastError();
}
#endif  // RQ_DN_CHUNK_INSTANTIATE

}  // namespace rq
