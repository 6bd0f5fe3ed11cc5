// Chunked causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), f16 KV cache, head_dim 128.
//
// Replaces the prefill attention items of the reference (attention_kv over a row block x one KV head, reference
// src/forward.c:3096-3146, :1871): rows of a prompt chunk at consecutive positions, each attending the cached prefix
// plus the chunk's earlier rows.
//
// Work item = (M tile of 128 query vectors = 128 / G consecutive rows x the G query heads of one KV head, KV head, split of
// 1024 key positions).  The split length is a constant of the kernel, so what a row computes depends on its own position
// only; every work item leaves a partial result (o, m, l) in the format of the split-K decode kernel and
// attn_combine_kernel merges a row's partials in split order.  Arithmetic: Q and P are rounded to f16 for the tensor
// cores (fp32 accumulation), so results agree with the CPU code to ~3e-4 relative, not bit for bit.
//
// One CTA = 4 softmax warps (thread t owns TMEM lane t = query vector t) + 1 warp whose lane 0 issues the TMA loads and
// the MMAs.  Per 128-position key block:
//   K block: 8 cache tiles [dim][16 pos] -> shared memory by 2-D TMA with the 32-byte swizzle = the MN-major canonical
//            layout of an MMA B operand (positions contiguous), no transposition needed;
//   S = Q K^T: 8 x tcgen05.mma (M 128, N 128, K 16), Q from shared memory (K-major, 128-byte swizzle), S in TMEM;
//   softmax: two passes of tcgen05.ld over the thread's row (max; then p = 2^((s - m) c), row sum), causal mask by
//            position, the running max only moves when it grows by more than 2^8 (then O and l are rescaled);
//   P (f16) overwrites the first 64 columns of S in TMEM and is the A operand of O += P V (8 x tcgen05.mma, V rows
//            [pos][dim] by TMA with the 128-byte swizzle, MN-major B operand), O accumulates in TMEM.
// TMEM: 256 columns per CTA (S / P 128, O 128); 96 KB of shared memory: two CTAs per SM overlap one's softmax with
// the other's MMAs.
#pragma once
#include <cuda.h>

#include "attn_decode.cuh"

namespace rq {

constexpr int PF_SPLIT = 1024;   // key positions per partial result (a multiple of the 128-position key block)
constexpr int PF_BN = 128;       // key positions per MMA block
constexpr int PF_THREADS = 160;  // 4 softmax warps + 1 TMA / MMA warp

struct PfWork {
    int seg;     // segment index (its tensor maps)
    int row0;    // first row of the tile (index in the pass)
    int nrows;   // rows of the tile (<= 128 / G)
    int split;   // which 1024-position split of the keys
};

struct AttnPrefillArgs {
    const PfWork *work;
    int n_work;
    const PassRow *rows;
    const CUtensorMap *maps;
    int layer, n_kv, G;
    const float *q;
    int qh, n_heads;
    float scale;
    int max_splits;
    float *part;
    int *err;
};
// launches attn_prefill_kernel (grid: work items x KV heads) on `stream`
cudaError_t launch_attn_prefill(const AttnPrefillArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_PREFILL_INSTANTIATE
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *m, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst)),
                 "l"(m), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
// shared-memory matrix descriptor of tcgen05.mma (start address, leading / stride byte offsets, layout type)
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | (uint64_t)((lbo >> 4) & 0x3fff) << 16 | (uint64_t)((sbo >> 4) & 0x3fff) << 32 |
           (uint64_t)1 << 46 | (uint64_t)layout << 61;
}
// instruction descriptor: f16 x f16 -> f32, A K-major, B MN-major, M x N
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N) {
    return (1u << 4) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem), "l"(a),
                 "l"(b), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive TMEM columns of this thread's lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t *r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
        "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

#ifdef RQ_PF_TRACE
__device__ long long pf_trace[64];  // experiments only: event times of CTA (0, 0), in clock cycles from its start
#define PF_T(i) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (i) < 64) pf_trace[i] = clock64() - pf_t0; } while (0)
#else
#define PF_T(i) do { } while (0)
#endif

constexpr int PF_SMEM = 3 * 32768 + 1024 + 128;  // Q | K | V (32 KB each), alignment slack, barriers

// maps: per segment the tensor maps of its sequence's K cache ({16 positions, rows of 32 bytes}, 32-byte swizzle, box 16 x
// 256) and V cache ({128 dims, rows of 256 bytes}, 128-byte swizzle, box 64 x 128).  k_rows_per_layer / v_rows_per_layer:
// rows of those 2-D views per layer of each segment's sequence.
__global__ void __launch_bounds__(PF_THREADS, 2) attn_prefill_kernel(const PfWork *__restrict__ work, const PassRow *__restrict__ rows,
                                                                  const CUtensorMap *__restrict__ maps, int layer, int n_kv, int G,
                                                                  const float *__restrict__ q, int qh, int n_heads, float scale,
                                                                  int max_splits, float *__restrict__ part, int *err) {
    constexpr int HD = 128, S_COL = 0, O_COL = 128, TM_COLS = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = sm, *sK = sm + 32768, *sV = sm + 65536;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 98304);  // 0: K loaded, 1: V loaded, 2: S done, 3: O done, 4: P stored
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + 98304 + 64);
    uint64_t *bar_k = bars, *bar_v = bars + 1, *bar_s = bars + 2, *bar_o = bars + 3, *bar_p = bars + 4;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef RQ_PF_TRACE
    const long long pf_t0 = clock64();
#endif
    const PfWork w = work[blockIdx.x];
    const int g = blockIdx.y;
    const PassRow r0 = rows[w.row0];
    const int np_min = r0.np, np_max = r0.np + w.nrows - 1;  // rows of a tile are at consecutive positions
    const int s0 = w.split * PF_SPLIT;                        // first key position of this split
    const int s1 = min(s0 + PF_SPLIT, np_max);                // one past the last key position any row needs
    const int nblk = (s1 - s0 + PF_BN - 1) / PF_BN;          // >= 1 by construction of the work list
    const CUtensorMap *mk = maps + 2 * w.seg, *mv = mk + 1;
    // rows of the 2-D views: K rows are 32 bytes (one dim of a tile), V rows 256 bytes (one position)
    const long long k_layer_rows = (long long)(r0.lk / 32), v_layer_rows = (long long)(r0.lv / 256);

    // first K / V row of key block j in the 2-D views
    auto k_row = [&](int j) {
        int t0 = s0 + j * PF_BN;
        return (long long)layer * k_layer_rows + ((long long)(t0 / ATT_P) * n_kv + g) * (ATT_PT * HD) + (long long)((t0 % ATT_P) / ATT_T) * HD;
    };
    auto v_row = [&](int j) {
        int t0 = s0 + j * PF_BN;
        return (long long)layer * v_layer_rows + ((long long)(t0 / ATT_P) * n_kv + g) * ATT_P + (t0 % ATT_P);
    };

    if (tid == 0) PF_T(44);  // work item and row fetched
    if (tid == 0) {
        mbar_init(bar_k, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_init(bar_p, 128);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 4) {
        if (lane == 0) {  // the first K / V blocks start loading while the other warps convert Q
            mbar_expect_tx(bar_k, 32768);
            for (int i = 0; i < 4; i++) tma_load_2d(sK + i * 8192, mk, 0, (int)k_row(0) + i * 256, bar_k);
            mbar_expect_tx(bar_v, 32768);
            for (int i = 0; i < 2; i++) tma_load_2d(sV + i * 16384, mv, i * 64, (int)v_row(0), bar_v);
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    // Q tile -> shared memory as f16, K-major with the 128-byte swizzle: vector t = row t / G, head g G + t % G;
    // 16-byte chunk c of 16: k-block c / 8, physical chunk (c % 8) ^ (t % 8)
    if (tid == 0) PF_T(45);  // barriers ready, first loads issued
    if (warp < 4) {
        // a warp converts 32 vectors, one per step: its lanes read the vector's 128 floats as one coalesced 512-byte
        // row (lane L: dims 4L .. 4L + 3) and store 4 halves into chunk L / 2
#pragma unroll
        for (int rr = 0; rr < 32; rr++) {
            const int t = warp * 32 + rr, rl = t / G, x = t % G;
            float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (rl < w.nrows) a = *reinterpret_cast<const float4 *>(q + ((size_t)(w.row0 + rl) * n_heads + (size_t)g * G + x) * qh + 4 * lane);
            __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
            const int c = lane >> 1;
            *reinterpret_cast<uint2 *>(sQ + (c >> 3) * 16384 + t * 128 + (((c & 7) ^ (t & 7)) << 4) + (lane & 1) * 8) =
                make_uint2(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1));
        }
    }
    if (tid == 0) PF_T(46);  // Q converted
    fence_proxy_async();  // Q was written by ordinary stores and will be read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    bool ok = true;
    if (tid == 0) PF_T(0);  // prologue done (Q in shared memory, TMEM allocated)

    if (warp == 4) {
        // ---- TMA loads and MMA issue (one thread)
        if (lane == 0) {
            auto load_k = [&](int j) {
                mbar_expect_tx(bar_k, 32768);
                int y = (int)k_row(j);
                for (int i = 0; i < 4; i++) tma_load_2d(sK + i * 8192, mk, 0, y + i * 256, bar_k);
            };
            auto load_v = [&](int j) {
                mbar_expect_tx(bar_v, 32768);
                int y = (int)v_row(j);
                for (int i = 0; i < 2; i++) tma_load_2d(sV + i * 16384, mv, i * 64, y, bar_v);
            };
            constexpr uint32_t idesc = umma_idesc(128, 128);
            auto mma_qk = [&]() {
#pragma unroll
                for (int ks = 0; ks < 8; ks++)
                    umma_ss(tbase + S_COL, umma_desc(smem_u32(sQ) + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024, 2),
                            umma_desc(smem_u32(sK) + ks * 512, 4096, 256, 6), idesc, ks > 0);
                umma_commit(bar_s);
            };
            auto mma_pv = [&](int j) {
#pragma unroll
                for (int ks = 0; ks < 8; ks++)
                    umma_ts(tbase + O_COL, tbase + S_COL + ks * 8, umma_desc(smem_u32(sV) + ks * 2048, 16384, 1024, 2), idesc, (j > 0) | (ks > 0));
                umma_commit(bar_o);
            };
            ok = mbar_wait_bounded(bar_k, 0, err, 11) && ok;
            tc_fence_after();
            mma_qk();
            for (int j = 0; j < nblk; j++) {
                const uint32_t ph = j & 1;
                ok = mbar_wait_bounded(bar_s, ph, err, 12) && ok;  // S(j) done: the K buffer is free
                if (j + 1 < nblk) load_k(j + 1);
                ok = mbar_wait_bounded(bar_p, ph, err, 13) && ok;  // P(j) is in TMEM
                ok = mbar_wait_bounded(bar_v, ph, err, 14) && ok;
                tc_fence_after();
                PF_T(3 + 4 * j);  // P V (j) issued (P and V ready)
                mma_pv(j);
                if (j + 1 < nblk) {
                    ok = mbar_wait_bounded(bar_k, ph ^ 1, err, 15) && ok;
                    tc_fence_after();
                    mma_qk();  // queued behind P V (j): it may overwrite the S / P columns only after they were read
                    ok = mbar_wait_bounded(bar_o, ph, err, 16) && ok;  // the V buffer is free
                    PF_T(4 + 4 * j);  // P V (j) complete
                    load_v(j + 1);
                }
            }
        }
        __syncwarp();
    } else {
        // ---- softmax: thread t owns query vector t (TMEM lane t)
        const int t = tid, rl = t / G;
        const int np = rl < w.nrows ? np_min + rl : 0;  // positions this vector attends (0: a padding vector)
        const uint32_t lane_addr = tbase + ((uint32_t)(warp * 32) << 16);
        const float c = scale * 1.44269504088896341f;
        float m_used = -INFINITY, l = 0.0f;
        for (int j = 0; j < nblk; j++) {
            const uint32_t ph = j & 1;
            const int t0 = s0 + j * PF_BN;
            ok = mbar_wait_bounded(bar_s, ph, err, 21) && ok;
            tc_fence_after();
            if (tid == 0) PF_T(1 + 4 * j);  // S(j) ready
            // the thread's whole row of S (128 scores) in registers: four loads in flight, one wait
            uint32_t r[4][32];
#pragma unroll
            for (int cc = 0; cc < 4; cc++) tmem_ld32(lane_addr + S_COL + cc * 32, r[cc]);
            tmem_wait_ld();
            const bool need_mask = t0 + PF_BN > np_min;  // (uniform over the CTA: only the blocks on the diagonal)
            if (need_mask) {
#pragma unroll
                for (int cc = 0; cc < 4; cc++)
#pragma unroll
                    for (int x = 0; x < 32; x++)
                        if (t0 + cc * 32 + x >= np) r[cc][x] = 0xff800000u;  // -inf
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int cc = 0; cc < 4; cc++)
#pragma unroll
                for (int x = 0; x < 32; x++) mx4[x & 3] = fmaxf(mx4[x & 3], __uint_as_float(r[cc][x]));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // the running max moves only when it grows by more than 8 in the exponent (p stays below 2^8: exact enough
            // in f16, and O is rescaled rarely); the first block with a valid position sets it
            float alpha = 1.0f;
            const bool move = mx > -INFINITY && (m_used == -INFINITY || (mx - m_used) * c > 8.0f);
            if (move) {
                alpha = m_used == -INFINITY ? 0.0f : ex2((m_used - mx) * c);
                m_used = mx;
            }
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // O and l of this warp's rows are rescaled (P V (j - 1) has completed: S (j) was queued behind it)
                l *= alpha;
#pragma unroll 1
                for (int cc = 0; cc < 4; cc++) {
                    uint32_t o[32];
                    tmem_ld32(lane_addr + O_COL + cc * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
                    tmem_st32(lane_addr + O_COL + cc * 32, o);
                }
                tmem_wait_st();
            }
            // p = 2^((s - m) c) (a masked score is -inf: p = 0), row sum, P as f16 pairs over the first 64 columns of S
            const float mc = m_used == -INFINITY ? 0.0f : m_used * c;
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
#pragma unroll
                for (int x = 0; x < 32; x += 2) {
                    float p0 = ex2(fmaf(__uint_as_float(r[cc][x]), c, -mc)), p1 = ex2(fmaf(__uint_as_float(r[cc][x + 1]), c, -mc));
                    l4[(x >> 1) & 3] += p0 + p1;
                    __half2 h = __floats2half2_rn(p0, p1);
                    r[cc >> 1][(cc & 1) * 16 + (x >> 1)] = *reinterpret_cast<uint32_t *>(&h);  // (slots already consumed)
                }
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tmem_st32(lane_addr + S_COL, r[0]);
            tmem_st32(lane_addr + S_COL + 32, r[1]);
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p);
            if (tid == 0) PF_T(2 + 4 * j);  // softmax(j) done
        }
        // ---- epilogue: the partial result (o unnormalised, m in scaled-score units, l)
        ok = mbar_wait_bounded(bar_o, (nblk - 1) & 1, err, 22) && ok;
        tc_fence_after();
        if (tid == 0) PF_T(40);  // last P V complete
        {
            // every thread's row of O goes through shared memory (Q / K / V are no longer needed: all MMAs are
            // complete) so that the global stores are coalesced: a warp then writes one 512-byte row per step
            constexpr int OST = HD + 4;  // floats per staged row (the padding spreads the rows over the banks)
            float *so = reinterpret_cast<float *>(sm);
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t r[32];
                tmem_ld32(lane_addr + O_COL + cc * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int y = 0; y < 32; y += 4)
                    *reinterpret_cast<float4 *>(so + (size_t)t * OST + cc * 32 + y) =
                        make_float4(__uint_as_float(r[y]), __uint_as_float(r[y + 1]), __uint_as_float(r[y + 2]), __uint_as_float(r[y + 3]));
            }
            so[(size_t)t * OST + HD] = m_used * scale;
            so[(size_t)t * OST + HD + 1] = l;
            if (tid == 0) PF_T(42);  // O staged
            __syncwarp();  // (a warp stages and writes the same 32 rows)
#pragma unroll 8
            for (int rr = 0; rr < 32; rr++) {
                const int tt = warp * 32 + rr, rl2 = tt / G, x = tt % G;
                if (rl2 >= w.nrows) continue;
                float *p = part + (((size_t)(w.row0 + rl2) * max_splits + w.split) * n_heads + (size_t)g * G + x) * RQ_PSTRIDE(HD);
                float4 v4 = *reinterpret_cast<const float4 *>(so + (size_t)tt * OST + 4 * lane);
                *reinterpret_cast<float4 *>(p + 4 * lane) = ok ? v4 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (lane < 2) p[HD + lane] = so[(size_t)tt * OST + HD + lane];
            }
        }
    }
    if (tid == 0) PF_T(41);  // partial written
    tc_fence_before();
    __syncthreads();
    if (warp == 4) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(TM_COLS));
}

cudaError_t launch_attn_prefill(const AttnPrefillArgs &a, cudaStream_t stream) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    attn_prefill_kernel<<<dim3(a.n_work, a.n_kv), PF_THREADS, PF_SMEM, stream>>>(a.work, a.rows, a.maps, a.layer, a.n_kv, a.G, a.q, a.qh,
                                                                               a.n_heads, a.scale, a.max_splits, a.part, a.err);
    return cudaGetLastError();
}
#endif  // RQ_ATTN_PREFILL_INSTANTIATE

}  // namespace rq
