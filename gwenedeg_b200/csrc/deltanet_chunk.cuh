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
// Two kernels per layer and pass:
//   dn_chunk_prep_kernel   everything of a chunk that does not depend on the state, one CTA per (chunk, value head), all
//                          chunks of the pass in parallel: rows -> K and Q as f16 operands, beta v, the gates' log2 prefix
//                          sums; the products K K^T and Q K^T on the tensor cores; A and M from them (masked, decayed);
//                          T' = (I + A)^-1 by two levels of blocks (forward substitution on the four 16 x 16 diagonal
//                          blocks, two products for each block below them).  Everything goes to a work buffer in the operand layout of the second
//                          kernel.
//   dn_chunk_state_kernel  the walk over a segment's chunks in order, one CTA per (segment, value head, half of the dv
//                          columns: the halves are independent given T' and M).  Per chunk, operands arrive by bulk
//                          copies (TMA), two chunks deep:
//                            S (TMEM, fp32) -> f16 copy in shared memory, and S *= g_63 in place
//                            MMA: K S0 and Q S0;               R_j = beta_j v_j - beta_j g_j (K S0)_j -> f16
//                            MMA: U = T' R;                    U and (g_63 / g_j) U -> f16
//                            MMA: M U;  S += K^T (scaled U);   O_i = g_i (Q S0)_i + (M U)_i -> global memory
//                          (the per-token scalings sit on the output side of each product, so K and Q are the only
//                          row operands and a record is 83 KB)
// All MMAs are M = 128 (rows 64 .. 127 of the token-indexed products are never read).  Every operand buffer has the
// same physical layout, [64-column half][row][128 bytes] with the 128-byte swizzle, which serves as a K-major operand
// (row = M or N index) and as an MN-major one (row = K index) alike.
#pragma once
#include "tc05.cuh"

namespace rq {

constexpr int DNC_C = 64;  // tokens per chunk
constexpr int DNC_THREADS = 256;
// the work buffer's record per (chunk, value head): the state kernel's operands, in its shared-memory layout
// K, Q (f16, operand layout) | T' | M | beta v (fp32 [half of dv][token][64 of 68]: the row padding keeps the state kernel's
// row reads conflict-free) | log2 decay prefix sums [64], beta [64]
constexpr int DNC_K = 0, DNC_Q = 16384, DNC_T = 32768, DNC_M = 40960, DNC_BV = 49152, DNC_BVH = 64 * 68 * 4, DNC_SC = DNC_BV + 2 * DNC_BVH,
              DNC_ITEM = DNC_SC + 512;

struct DnChunkArgs {
    const DnSeg *segs;  // (DnSeg::chunk0: chunks of all earlier segments = the segment's first record in `work`)
    const DnChunk *chunks;  // the chunks of the pass, segment by segment
    const DnCk *cks;        // the checkpoints of the pass
    int nseg, n_chunks, lin_layer, nk, nv;
    size_t conv_floats;
    const float *rows;
    int lw;
    float *out;
    uint8_t *work;  // [chunks of the pass][nv] records of DNC_ITEM bytes
    int *err;
};
// launches the two kernels on `stream`; dk = dv = 128 only
cudaError_t launch_dn_chunk(const DnChunkArgs &a, cudaStream_t stream);

#ifdef RQ_DN_CHUNK_INSTANTIATE
namespace dnc {
constexpr int AST = 68;  // floats per row of the fp32 64 x 64 matrices in shared memory
// ---- prep kernel: shared memory (bytes from a 1024-byte aligned base); TMEM: K K^T | Q K^T (128 columns)
// (the fp32 matrices of the inverse take the place of the f16 operands, which are dead once the two products have completed:
// four CTAs fit an SM, so that all chunks of a 2,048-row pass over 16 heads are resident at once)
constexpr int P_K16 = 0, P_Q16 = 16384, P_SLACK = 32768, P_AF = 0, P_XF = P_AF + 64 * AST * 4, P_PF = P_XF + 64 * AST * 4,
              P_LG = 49152, P_BETA = P_LG + 256, P_BAR = P_BETA + 256, P_SLOT = P_BAR + 16, P_SMEM = P_SLOT + 16 + 1024;
static_assert(P_PF + 32 * AST * 4 <= P_LG, "the inverse's matrices fit the operands' place");
// (P_SLACK: 16 KB that the M = 128 products read past the 64 rows of Q16)
// ---- state kernel: two stages of operands (the record's first 64 KB, then the CTA's half of B V, then the gates)
constexpr int ST_BV = 49152, ST_SC = ST_BV + DNC_BVH, ST_BYTES = 67584;
constexpr int S_S16 = 2 * ST_BYTES, S_R16 = S_S16 + 16384, S_U16 = S_R16 + 8192, S_UK16 = S_U16 + 8192, S_BAR = S_UK16 + 8192,
              S_SLOT = S_BAR + 32, S_SMEM = S_SLOT + 16 + 1024;
constexpr int HV = 64;  // dv columns per CTA of the state kernel
constexpr int S_COL = 0, Y_COL = 64, Z1_COL = 128, Z2_COL = 192;
}  // namespace dnc

// byte offset of 4 adjacent values (dims 4 lane .. 4 lane + 3 of row `row`) in the swizzled f16 layout of a 64-row,
// 128-column buffer
__device__ __forceinline__ int dnc_off4(int row, int lane) {
    const int ch = lane >> 1;
    return (ch >> 3) * 8192 + row * 128 + (((ch & 7) ^ (row & 7)) << 4) + (lane & 1) * 8;
}
__device__ __forceinline__ uint32_t dnc_pack(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint2 dnc_pack4(float a, float b, float c, float d) { return make_uint2(dnc_pack(a, b), dnc_pack(c, d)); }
__device__ __forceinline__ void dnc_tmem_ld8(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
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


// grid: (chunk of the pass, value head)
__global__ void __launch_bounds__(DNC_THREADS, 4) dn_chunk_prep_kernel(const DnSeg *__restrict__ segs, const DnChunk *__restrict__ chunks, int nk, int nv,
                                                                  const float *__restrict__ rows, int lw, uint8_t *__restrict__ work, int *err) {
    using namespace dnc;
    constexpr int DK = 128, DV = 128;
    pdl_wait();
    pdl_launch_dependents();
    const DnChunk ch = chunks[blockIdx.x];
    const DnSeg sg = segs[ch.seg];
    const int c0 = ch.row0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *s_a = reinterpret_cast<float *>(sm + P_AF), *s_x = reinterpret_cast<float *>(sm + P_XF), *s_p = reinterpret_cast<float *>(sm + P_PF);
    float *s_lg = reinterpret_cast<float *>(sm + P_LG), *s_beta = reinterpret_cast<float *>(sm + P_BETA);
    uint64_t *bar = reinterpret_cast<uint64_t *>(sm + P_BAR);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + P_SLOT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, cnt = ch.cnt;
    const int trow = (warp & 3) * 32 + lane, cb = warp >> 2;
    const int conv_dim = 2 * nk * DK + nv * DV, vdim = nv * DV;
    const size_t oq = (size_t)(h % nk) * DK, okk = (size_t)nk * DK + oq, ov = (size_t)2 * nk * DK + (size_t)h * DV;
    const size_t oe = (size_t)conv_dim + vdim + h, ob = oe + nv;
    uint8_t *rec = work + ((size_t)blockIdx.x * nv + h) * DNC_ITEM;

    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(128));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // gates (warp 0): the loads now, the inclusive log2 prefix sums after the warp's share of the rows, so that they wait under it
    // (tokens past the end: eg 1, beta 0)
    float ge0 = 1.0f, ge1 = 1.0f, gb0 = 0.0f, gb1 = 0.0f;
    if (warp == 0) {
        const float *r0 = rows + (size_t)(sg.row0 + c0 + lane) * lw, *r1 = r0 + (size_t)32 * lw;
        if (lane < cnt) ge0 = __ldg(r0 + oe), gb0 = __ldg(r0 + ob);
        if (lane + 32 < cnt) ge1 = __ldg(r1 + oe), gb1 = __ldg(r1 + ob);
    }
    bool ok = true;
    // rows -> f16: K and Q for the two products here and into the record (the state kernel applies the per-token
    // scalings g_j, beta_j g_j, g_63 / g_j on the other side of its products); beta v in fp32.  Two rows of a warp's eight at a
    // time: with four CTAs per SM a thread has 64 registers.  Nothing here waits for the gates or for the TMEM allocation.
#pragma unroll 1
    for (int i2 = 0; i2 < 8; i2 += 2) {
        float4 qv[2], kv[2], vv[2];
        float bt[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int j = warp * 8 + i2 + i;
            qv[i] = kv[i] = vv[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            bt[i] = 0.0f;
            if (j < cnt) {
                const float *r = rows + (size_t)(sg.row0 + c0 + j) * lw;
                qv[i] = __ldg(reinterpret_cast<const float4 *>(r + oq) + lane);
                kv[i] = __ldg(reinterpret_cast<const float4 *>(r + okk) + lane);
                vv[i] = __ldg(reinterpret_cast<const float4 *>(r + ov) + lane);
                bt[i] = __ldg(r + ob);
            }
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int j = warp * 8 + i2 + i, off = dnc_off4(j, lane);
            const float bet = bt[i];
            const uint2 k2 = dnc_pack4(kv[i].x, kv[i].y, kv[i].z, kv[i].w), q2 = dnc_pack4(qv[i].x, qv[i].y, qv[i].z, qv[i].w);
            *reinterpret_cast<uint2 *>(sm + P_K16 + off) = k2;
            *reinterpret_cast<uint2 *>(sm + P_Q16 + off) = q2;
            *reinterpret_cast<uint2 *>(rec + DNC_K + off) = k2;
            *reinterpret_cast<uint2 *>(rec + DNC_Q + off) = q2;
            // beta v, fp32, per half of the dv columns: [half][token][64]
            *reinterpret_cast<float4 *>(rec + DNC_BV + (lane >> 4) * DNC_BVH + (j * AST + 4 * (lane & 15)) * 4) =
                make_float4(vv[i].x * bet, vv[i].y * bet, vv[i].z * bet, vv[i].w * bet);
        }
    }
    if (warp == 0) {
        float a0 = lane < cnt ? fmaxf(log2f(ge0), -1.0e4f) : 0.0f, a1 = lane + 32 < cnt ? fmaxf(log2f(ge1), -1.0e4f) : 0.0f;
        s_beta[lane] = gb0;
        s_beta[lane + 32] = gb1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float b0 = __shfl_up_sync(0xffffffffu, a0, o), b1 = __shfl_up_sync(0xffffffffu, a1, o);
            if (lane >= o) a0 += b0, a1 += b1;
        }
        a1 += __shfl_sync(0xffffffffu, a0, 31);
        s_lg[lane] = a0;
        s_lg[lane + 32] = a1;
        float *sc = reinterpret_cast<float *>(rec + DNC_SC);
        sc[lane] = a0, sc[lane + 32] = a1;
        sc[64 + lane] = gb0, sc[96 + lane] = gb1;
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    // K K^T and Q K^T (M 128, N 64, K 128)
    if (warp == 4 && (tc_fence_after(), elect_one())) {
        const uint32_t sbase = smem_u32(sm);
        constexpr uint32_t id_kk = umma_idesc(128, 64, 0, 0);
        auto d_k128 = [&](int buf, int ks) { return umma_desc(sbase + buf + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024, 2); };
#pragma unroll
        for (int ks = 0; ks < 8; ks++) umma_ss(tbase, d_k128(P_K16, ks), d_k128(P_K16, ks), id_kk, ks > 0);
#pragma unroll
        for (int ks = 0; ks < 8; ks++) umma_ss(tbase + 64, d_k128(P_Q16, ks), d_k128(P_K16, ks), id_kk, ks > 0);
        umma_commit(bar);
    }
    ok = mbar_wait_bounded(bar, 0, err, 31) && ok;
    tc_fence_after();
    // A (fp32, strictly lower) and M (f16, lower with the diagonal): row i, columns 32 cb .. + 31 per thread
    // (every thread has seen the products complete: the fp32 matrices may take the operands' place)
    if ((warp & 3) < 2) {
        const int i = trow;
        const float lgi = s_lg[i], bi = s_beta[i];
#pragma unroll 1
        for (int x8 = 0; x8 < 4; x8++) {  // eight columns at a time
            uint32_t g[8], mq[8];
            dnc_tmem_ld8(lane_addr + cb * 32 + 8 * x8, g);
            dnc_tmem_ld8(lane_addr + 64 + cb * 32 + 8 * x8, mq);
            tmem_wait_ld();
            float mv[8], av[8];
#pragma unroll
            for (int x = 0; x < 8; x++) {
                const int j = 32 * cb + 8 * x8 + x;
                const float ratio = j <= i ? ex2(lgi - s_lg[j]) : 0.0f;
                av[x] = j < i ? bi * ratio * __uint_as_float(g[x]) : 0.0f;
                mv[x] = j <= i ? ratio * __uint_as_float(mq[x]) : 0.0f;
            }
            *reinterpret_cast<float4 *>(s_a + i * AST + 32 * cb + 8 * x8) = make_float4(av[0], av[1], av[2], av[3]);
            *reinterpret_cast<float4 *>(s_a + i * AST + 32 * cb + 8 * x8 + 4) = make_float4(av[4], av[5], av[6], av[7]);
            const int ch = 4 * cb + x8;
            uint4 w;
            w.x = dnc_pack(mv[0], mv[1]), w.y = dnc_pack(mv[2], mv[3]), w.z = dnc_pack(mv[4], mv[5]), w.w = dnc_pack(mv[6], mv[7]);
            *reinterpret_cast<uint4 *>(rec + DNC_M + i * 128 + ((ch ^ (i & 7)) << 4)) = w;
        }
    }
    tc_fence_before();
    __syncthreads();
    // T' = (I + A)^-1 by two levels of the block formula  inv [[L11, 0], [A21, L22]] = [[X11, 0], [-X22 A21 X11, X22]]:
    // the four 16 x 16 diagonal blocks by forward substitution (a column per thread: x_r = [r == c] - sum_{q<r} A_rq x_q),
    // from them the two 32 x 32 diagonal blocks, from those the whole; the products run on all threads
    if (tid < 64) {
        const int b = tid >> 4, cc = tid & 15;
        float x[16];
#pragma unroll
        for (int r = 0; r < 16; r++) {
            float acc[4] = {r == cc ? 1.0f : 0.0f, 0.0f, 0.0f, 0.0f};
            const float *arow = s_a + (16 * b + r) * AST + 16 * b;
#pragma unroll
            for (int q4 = 0; q4 < (r + 3) / 4; q4++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(arow + 4 * q4);  // (entries q >= r are zero)
                const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int y = 0; y < 4; y++)
                    if (4 * q4 + y < r) acc[y] = fmaf(-av[y], x[4 * q4 + y], acc[y]);
            }
            x[r] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            s_x[(16 * b + r) * AST + 16 * b + cc] = x[r];
        }
    }
    __syncthreads();
    {
        // inside 32-block B: the lower left 16 x 16 block, thread = (B, row r, two columns c2, c2 + 1)
        const int B = tid >> 7, r = (tid >> 3) & 15, c2 = (tid & 7) * 2;
        {  // P = A21 X11
            float p0 = 0.0f, p1 = 0.0f;
            const float *arow = s_a + (32 * B + 16 + r) * AST + 32 * B;
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(arow + 4 * q4);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int y = 0; y < 4; y++) {
                    const float2 x2 = *reinterpret_cast<const float2 *>(s_x + (32 * B + 4 * q4 + y) * AST + 32 * B + c2);
                    p0 = fmaf(av[y], x2.x, p0), p1 = fmaf(av[y], x2.y, p1);
                }
            }
            *reinterpret_cast<float2 *>(s_p + (16 * B + r) * AST + c2) = make_float2(p0, p1);
        }
        __syncthreads();
        {  // X21 = -X22 P; the block above the diagonal is zero
            float v0 = 0.0f, v1 = 0.0f;
            const float *xrow = s_x + (32 * B + 16 + r) * AST + 32 * B + 16;
#pragma unroll
            for (int q4 = 0; q4 < 4; q4++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(xrow + 4 * q4);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int y = 0; y < 4; y++) {
                    const float2 p2 = *reinterpret_cast<const float2 *>(s_p + (16 * B + 4 * q4 + y) * AST + c2);
                    v0 = fmaf(-av[y], p2.x, v0), v1 = fmaf(-av[y], p2.y, v1);
                }
            }
            *reinterpret_cast<float2 *>(s_x + (32 * B + 16 + r) * AST + 32 * B + c2) = make_float2(v0, v1);
            *reinterpret_cast<float2 *>(s_x + (32 * B + r) * AST + 32 * B + 16 + c2) = make_float2(0.0f, 0.0f);
        }
    }
    __syncthreads();
    {
        const int r = tid >> 3, c4 = (tid & 7) * 4;
        {  // P = A21 X11
            float4 p = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float *arow = s_a + (32 + r) * AST;
#pragma unroll
            for (int q4 = 0; q4 < 8; q4++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(arow + 4 * q4);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int y = 0; y < 4; y++) {
                    const float4 x4 = *reinterpret_cast<const float4 *>(s_x + (4 * q4 + y) * AST + c4);
                    p.x = fmaf(av[y], x4.x, p.x), p.y = fmaf(av[y], x4.y, p.y), p.z = fmaf(av[y], x4.z, p.z), p.w = fmaf(av[y], x4.w, p.w);
                }
            }
            *reinterpret_cast<float4 *>(s_p + r * AST + c4) = p;
        }
        __syncthreads();
        {  // X21 = -X22 P
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float *xrow = s_x + (32 + r) * AST + 32;
#pragma unroll
            for (int q4 = 0; q4 < 8; q4++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(xrow + 4 * q4);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
                for (int y = 0; y < 4; y++) {
                    const float4 p4 = *reinterpret_cast<const float4 *>(s_p + (4 * q4 + y) * AST + c4);
                    v.x = fmaf(-av[y], p4.x, v.x), v.y = fmaf(-av[y], p4.y, v.y), v.z = fmaf(-av[y], p4.z, v.z), v.w = fmaf(-av[y], p4.w, v.w);
                }
            }
            *reinterpret_cast<float4 *>(s_x + (32 + r) * AST + c4) = v;
        }
        __syncthreads();
        // -> f16, K-major rows of 64: thread (row, 16-column block); the upper right block is zero
        const int row = tid >> 2, jb = tid & 3;
        float f[16];
#pragma unroll
        for (int q = 0; q < 16; q++) f[q] = ((row >= 32 || jb < 2) && ok) ? s_x[row * AST + 16 * jb + q] : 0.0f;
#pragma unroll
        for (int q = 0; q < 2; q++) {
            uint4 w;
            w.x = dnc_pack(f[8 * q], f[8 * q + 1]), w.y = dnc_pack(f[8 * q + 2], f[8 * q + 3]);
            w.z = dnc_pack(f[8 * q + 4], f[8 * q + 5]), w.w = dnc_pack(f[8 * q + 6], f[8 * q + 7]);
            *reinterpret_cast<uint4 *>(rec + DNC_T + row * 128 + (((2 * jb + q) ^ (row & 7)) << 4)) = w;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(128));
}

// grid: (2 x value heads, segments)
__global__ void __launch_bounds__(DNC_THREADS, 1) dn_chunk_state_kernel(const DnSeg *__restrict__ segs, const DnChunk *__restrict__ chunks,
                                                                     const DnCk *__restrict__ cks, int lin_layer, int nv, size_t conv_floats,
                                                                     const uint8_t *__restrict__ work, float *__restrict__ out, int *err) {
    using namespace dnc;
    constexpr int DK = 128, DV = 128, C = DNC_C;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(sm + S_BAR), *bar = bar_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + S_SLOT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.x >> 1, hv = blockIdx.x & 1;  // value head, which half of its dv columns
    const int trow = (warp & 3) * 32 + lane, cb = warp >> 2;  // this thread's TMEM lane and its 32-column block of a 64-column tile
    const DnSeg sg = segs[blockIdx.y];
    const int vdim = nv * DV, nch = sg.nch;
    const DnChunk *chs = chunks + sg.chunk0;
    // the CTA's part of the state: blocks 2 hv, 2 hv + 1 of [dv / 32][dk][32]
    float *Sg = sg.state + (size_t)lin_layer * sg.lstride + conv_floats + (size_t)h * DK * DV + (size_t)hv * 2 * DK * 32;
    const uint8_t *rec0 = work + ((size_t)sg.chunk0 * nv + h) * DNC_ITEM;

    if (tid == 0) {
        mbar_init(bar_full, 1);
        mbar_init(bar_full + 1, 1);
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    bool ok = true;
    uint32_t phase = 0;
    // chunk n's operands -> stage n % 2 (one thread): K, Q, T', M (48 KB), the CTA's half of beta v, the gates
    auto load_chunk = [&](int n) {
        uint8_t *st = sm + (n & 1) * ST_BYTES;
        const uint8_t *rec = rec0 + (size_t)n * nv * DNC_ITEM;
        mbar_expect_tx(bar_full + (n & 1), 49152 + DNC_BVH + 512);
        bulk_g2s(st, rec, 49152, bar_full + (n & 1));
        bulk_g2s(st + ST_BV, rec + DNC_BV + hv * DNC_BVH, DNC_BVH, bar_full + (n & 1));
        bulk_g2s(st + ST_SC, rec + DNC_SC, 512, bar_full + (n & 1));
    };
    if (tid == 0 && nch > 0) load_chunk(0);

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
    constexpr uint32_t id_kmn = umma_idesc(128, 64, 0, 1), id_mnmn = umma_idesc(128, 64, 1, 1);
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

    // a chunk's output row stays in registers and is stored under the next chunk's first products, off the chain of
    // dependent steps
    float ov[32];
    float4 *ov_dst = nullptr;
    auto flush_out = [&]() {
        if (ov_dst) {
#pragma unroll
            for (int y = 0; y < 8; y++) ov_dst[y] = ok ? make_float4(ov[4 * y], ov[4 * y + 1], ov[4 * y + 2], ov[4 * y + 3]) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            ov_dst = nullptr;
        }
    };
    for (int n = 0; n < nch; n++) {
        const DnChunk ch = chs[n];
        const int c0 = ch.row0, cnt = ch.cnt, sb = (n & 1) * ST_BYTES;
        // the next chunk's operands start loading (its stage was last read by chunk n - 1, whose products are complete
        // and whose B V rows and gates every thread read before the barrier at the end of that chunk)
        if (tid == 0 && n + 1 < nch) load_chunk(n + 1);
        ok = mbar_wait_bounded(bar_full + (n & 1), (n >> 1) & 1, err, 33) && ok;
        {
            // S (the previous chunk's result) -> its f16 copy, the B operand of this chunk's S0 products; S *= g_63
            uint32_t r[32];
            tmem_ld32(lane_addr + S_COL + cb * 32, r);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int x = 0; x < 32; x++) f[x] = __uint_as_float(r[x]);
            dnc_store_row32(sm + S_S16, trow, cb, f);
            const float gc = ex2(reinterpret_cast<const float *>(sm + sb + ST_SC)[C - 1]);
#pragma unroll
            for (int x = 0; x < 32; x++) r[x] = __float_as_uint(f[x] * gc);
            tmem_st32(lane_addr + S_COL + cb * 32, r);
            tmem_wait_st();
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- K S0 -> Y and Q S0 -> Z1
        if (warp == 4 && (tc_fence_after(), elect_one())) {
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + Y_COL, d_k128(sb + DNC_K, ks), d_mn(S_S16, ks, 0), id_kmn, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 8; ks++) umma_ss(tbase + Z1_COL, d_k128(sb + DNC_Q, ks), d_mn(S_S16, ks, 0), id_kmn, ks > 0);
            umma_commit(bar);
        }
        flush_out();  // (the previous chunk's rows)
        wait_mma();
        // ---- R = beta v - beta_j g_j (k_j S0) -> f16: row j, columns 32 cb .. + 31 per thread
        const float *s_sc = reinterpret_cast<const float *>(sm + sb + ST_SC);
        const float lgj = s_sc[trow & 63], nbg = -s_sc[64 + (trow & 63)] * ex2(lgj);
        if ((warp & 3) < 2) {
            uint32_t r[32];
            tmem_ld32(lane_addr + Y_COL + cb * 32, r);
            tmem_wait_ld();
            const float *s_bv = reinterpret_cast<const float *>(sm + sb + ST_BV);
            float f[32];
#pragma unroll
            for (int x = 0; x < 32; x += 4) {
                const float4 b = *reinterpret_cast<const float4 *>(s_bv + trow * AST + 32 * cb + x);
                f[x] = fmaf(nbg, __uint_as_float(r[x]), b.x), f[x + 1] = fmaf(nbg, __uint_as_float(r[x + 1]), b.y);
                f[x + 2] = fmaf(nbg, __uint_as_float(r[x + 2]), b.z), f[x + 3] = fmaf(nbg, __uint_as_float(r[x + 3]), b.w);
            }
            dnc_store_row32(sm + S_R16, trow, cb, f);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- U = T' R -> Y
        if (warp == 4 && (tc_fence_after(), elect_one())) {
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + Y_COL, d_k64(sb + DNC_T, ks), d_mn(S_R16, ks, 0), id_kmn, ks > 0);
            umma_commit(bar);
        }
        wait_mma();
        // ---- U -> f16, plain (for M U) and with rows scaled by g_63 / g_j (for the state update)
        if ((warp & 3) < 2) {
            uint32_t r[32];
            tmem_ld32(lane_addr + Y_COL + cb * 32, r);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int x = 0; x < 32; x++) f[x] = __uint_as_float(r[x]);
            dnc_store_row32(sm + S_U16, trow, cb, f);
            const float kt = ex2(s_sc[C - 1] - lgj);
#pragma unroll
            for (int x = 0; x < 32; x++) f[x] *= kt;
            dnc_store_row32(sm + S_UK16, trow, cb, f);
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- M U -> Z2;  S += K^T (scaled U)
        if (warp == 4 && (tc_fence_after(), elect_one())) {
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + Z2_COL, d_k64(sb + DNC_M, ks), d_mn(S_U16, ks, 0), id_kmn, ks > 0);
#pragma unroll
            for (int ks = 0; ks < 4; ks++) umma_ss(tbase + S_COL, d_mn(sb + DNC_K, ks, 8192), d_mn(S_UK16, ks, 0), id_mnmn, 1);
            umma_commit(bar);
        }
        wait_mma();
        // ---- O = g_i (q_i S0) + (M U)_i: thread (row, 32-column block) takes its 32 values; they go to global memory
        // (128 bytes per thread) under the next chunk's first products
        if ((warp & 3) < 2) {
            uint32_t r1[32], r2[32];
            tmem_ld32(lane_addr + Z1_COL + cb * 32, r1);
            tmem_ld32(lane_addr + Z2_COL + cb * 32, r2);
            tmem_wait_ld();
            if (trow < cnt) {
                const float gi = ex2(lgj);
#pragma unroll
                for (int y = 0; y < 32; y++) ov[y] = fmaf(gi, __uint_as_float(r1[y]), __uint_as_float(r2[y]));
                ov_dst = reinterpret_cast<float4 *>(out + (size_t)(sg.row0 + c0 + trow) * vdim + (size_t)h * DV + (size_t)hv * HV + 32 * cb);
            }
        }
        if (ch.ck >= 0) {
            // a checkpoint after this chunk's last row: the CTA's part of S as it stands (fp32, from TMEM) into the checkpoint's
            // buffer, in the layout of the state
            uint32_t r[32];
            tmem_ld32(lane_addr + S_COL + cb * 32, r);
            tmem_wait_ld();
            float4 *dst = reinterpret_cast<float4 *>(cks[ch.ck].dst + (Sg - sg.state) + (size_t)cb * DK * 32 + (size_t)trow * 32);
#pragma unroll
            for (int x = 0; x < 8; x++)
                dst[x] = make_float4(__uint_as_float(r[4 * x]), __uint_as_float(r[4 * x + 1]), __uint_as_float(r[4 * x + 2]), __uint_as_float(r[4 * x + 3]));
        }
        fence_proxy_async();  // (this chunk's stage is overwritten by bulk copies next)
        tc_fence_before();
        __syncthreads();      // (this chunk's stage and the O columns are free again)
    }
    flush_out();  // (the last chunk's rows)
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
    if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(256));
}

cudaError_t launch_dn_chunk(const DnChunkArgs &a, cudaStream_t stream) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(dn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dnc::P_SMEM);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(dn_chunk_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dnc::S_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaError_t e = launch_pdl(dn_chunk_prep_kernel, dim3(a.n_chunks, a.nv), dim3(DNC_THREADS), dnc::P_SMEM, stream, a.segs, a.chunks, a.nk, a.nv, a.rows,
                               a.lw, a.work, a.err);
    if (e != cudaSuccess) return e;
    return launch_pdl(dn_chunk_state_kernel, dim3(2 * a.nv, a.nseg), dim3(DNC_THREADS), dnc::S_SMEM, stream, a.segs, a.chunks, a.cks, a.lin_layer, a.nv,
                      a.conv_floats, a.work, a.out, a.err);
}
#endif  // RQ_DN_CHUNK_INSTANTIATE

}  // namespace rq
