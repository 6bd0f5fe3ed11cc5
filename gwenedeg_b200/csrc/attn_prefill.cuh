// Chunked causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), f16 KV cache, head_dim 128.
//
// Replaces the prefill attention items of the reference (attention_kv over a row block x one KV head, reference
// src/forward.c:3096-3146, :1871): rows of a prompt chunk at consecutive positions, each attending the cached prefix
// plus the chunk's earlier rows.
//
// Work item = (M tile of 128 query vectors = 128 / G consecutive rows x the G query heads of one KV head, KV head, split of
// 2048 key positions).  The split length is a constant of the kernel, so what a row computes depends on its own position
// only; every work item leaves a partial result (o, m, l) in the format of the split-K decode kernel and
// attn_combine_rows_kernel merges a row's partials in split order.  Arithmetic: Q and P are rounded to f16 for the tensor
// cores (fp32 accumulation), so results agree with the CPU code to ~3e-4 relative, not bit for bit.
//
// One CTA (one per SM: all 512 TMEM columns, 193 KB of shared memory) = 8 softmax warps + 3 issue warps.  Per
// 128-position key block j:
//   TMA warp:   K block (8 cache tiles [dim][16 pos]) -> shared memory by 2-D TMA with the 32-byte swizzle = the MN-major
//               canonical layout of an MMA B operand (positions contiguous), no transposition needed; V rows [pos][dim]
//               with the 128-byte swizzle, MN-major B operand as well.  3 K stages, 2 V stages.
//   S warp:     S = Q K^T: 8 x tcgen05.mma (M 128, N 128, K 16), Q from shared memory (K-major, 128-byte swizzle), S in TMEM.
//   softmax:    thread t of stream h (warps 4h .. 4h + 3) owns query vector t and the block's keys 64 h .. 64 h + 63: it
//               loads its 64 scores into registers and at once releases S, so S (j + 1) is computed under the softmax of
//               block j and the softmax threads never wait for the tensor cores.  One sweep does p = 2^((s - m) c), the
//               row sum and the block maximum; the running max moves only when the block's exceeds it by more than 2^8
//               (then O and l are rescaled and the sweep repeated), the causal mask goes by position.  P (f16) goes to
//               the block's P buffer in TMEM (double-buffered).
//   P V warp:   O_h += P_h V_h, 4 x tcgen05.mma per stream with P as the A operand from TMEM; the two streams keep their
//               own (m, l, O) and the epilogue merges them, so no thread ever needs another's row maximum.
// TMEM: S 128 columns, P 2 x 64, O 2 x 128.  The loop is bound by the softmax warps' issue slots (~1,750 cycles per
// block against 1,024 of MMA time), prologue (Q conversion, first TMA) and epilogue (partial write) cost ~13k cycles.
#pragma once
#include <cuda.h>

#include "attn_decode.cuh"
#include "tc05.cuh"

namespace rq {

#ifndef RQ_PF_SPLIT
#define RQ_PF_SPLIT 2048
#endif
constexpr int PF_SPLIT = RQ_PF_SPLIT;  // key positions per partial result where nothing better is known (a multiple of the 128-position key block)
constexpr int PF_SPLIT_MIN = 1024;     // the shortest split the host chooses: bounds the partial records of a pass
constexpr int PF_BN = 128;       // key positions per MMA block
constexpr int PF_THREADS = 352;  // 2 streams x 4 softmax warps + the P V, S and TMA warps

struct PfWork {
    int seg;     // segment index (its tensor maps)
    int row0;    // first row of the tile (index in the pass)
    int nrows;   // rows of the tile (<= 128 / G)
    int split;   // which split of split_len key positions
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
    int split_len;  // key positions per split (a multiple of 128; chosen per pass by the host)
    float *part;
    int *err;
};
// launches attn_prefill_kernel (grid: work items x KV heads) on `stream`
cudaError_t launch_attn_prefill(const AttnPrefillArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_PREFILL_INSTANTIATE

constexpr int PF_SMEM = 6 * 32768 + 1024 + 256 + 2048;  // Q | K x 3 stages | V x 2 stages (32 KB each), slack, barriers, (m, l) exchange

// maps: per segment the tensor maps of its sequence's K cache ({16 positions, rows of 32 bytes}, 32-byte swizzle, box 16 x
// 256) and V cache ({128 dims, rows of 256 bytes}, 128-byte swizzle, box 64 x 128).
__global__ void __launch_bounds__(PF_THREADS, 1) attn_prefill_kernel(const PfWork *__restrict__ work, const PassRow *__restrict__ rows,
                                                                  const CUtensorMap *__restrict__ maps, int layer, int n_kv, int G,
                                                                  const float *__restrict__ q, int qh, int n_heads, float scale,
                                                                  int max_splits, int split_len, float *__restrict__ part, int *err) {
    // TMEM columns: S at 0 (128); P (f16 pairs) of key block j, stream h (the block's keys 64 h .. 64 h + 63) at
    // 128 + 64 (j % 2) + 32 h; O of stream h at 256 + 128 h
    constexpr int HD = 128, TM_COLS = 512, P_COL = 128, O_COL = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = sm, *sK = sm + 32768, *sV = sm + 131072;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + 196608);
    // K stage loaded (3), V stage loaded (2), S written (1), S read by every softmax thread (1), K stage free (3),
    // P V of block j complete (2: j % 2), P (j) of stream h stored (4: 2 h + j % 2).  Every barrier's next phase depends
    // on each of its waiters having seen the current one, so a parity wait is never ambiguous
    uint64_t *bar_k = bars, *bar_v = bars + 3, *bar_s = bars + 5, *bar_sfree = bars + 6, *bar_kfree = bars + 7, *bar_o = bars + 10,
             *bar_p = bars + 12;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + 196608 + 192);
    float *sml = reinterpret_cast<float *>(sm + 196608 + 256);  // [stream][vector][m, l]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();
    const PfWork w = work[blockIdx.x];
    const int g = blockIdx.y;
    const PassRow r0 = rows[w.row0];
    const int np_min = r0.np, np_max = r0.np + w.nrows - 1;  // rows of a tile are at consecutive positions
    const int s0 = w.split * split_len;                        // first key position of this split
    const int s1 = min(s0 + split_len, np_max);                // one past the last key position any row needs
    const int nblk = (s1 - s0 + PF_BN - 1) / PF_BN;          // >= 1 by construction of the work list
    // (debug build) the split starts inside the tile's keys, the tile is one of at most 128 vectors, the KV head exists
    RQ_CHECK(w.nrows >= 1 && w.nrows * G <= 128 && s0 >= 0 && s0 < np_max && nblk >= 1 && nblk <= split_len / PF_BN && g < n_kv && w.split < max_splits, err, 43);
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
    auto load_k = [&](int j) {  // key block j -> stage j % 3
        uint64_t *bar = bar_k + j % 3;
        uint8_t *dst = sK + (j % 3) * 32768;
        mbar_expect_tx(bar, 32768);
        const int y = (int)k_row(j);
        for (int i = 0; i < 4; i++) tma_load_2d(dst + i * 8192, mk, 0, y + i * 256, bar);
    };
    auto load_v = [&](int j) {  // -> stage j % 2
        uint64_t *bar = bar_v + (j & 1);
        uint8_t *dst = sV + (j & 1) * 32768;
        mbar_expect_tx(bar, 32768);
        const int y = (int)v_row(j);
        for (int i = 0; i < 2; i++) tma_load_2d(dst + i * 16384, mv, i * 64, y, bar);
    };

    if (tid == 0) {
        for (int i = 0; i < 12; i++) mbar_init(bars + i, i == 6 ? 256 : 1);
        for (int i = 0; i < 4; i++) mbar_init(bar_p + i, 128);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 10) {
        // The first K block starts loading while the other warps convert Q; the other stages are requested once Q is in
        // (all SMs start at once and together take in ~4.5 TB/s: everything at once would put 160 KB per SM beside the
        // 96 KB that the first MMA waits for)
        if (lane == 0) load_k(0);
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    } else if (warp < 8) {
        // Q tile -> shared memory as f16, K-major with the 128-byte swizzle: vector t = row t / G, head g G + t % G;
        // 16-byte chunk c of 16: k-block c / 8, physical chunk (c % 8) ^ (t % 8).
        // A warp converts 16 vectors, one per step: its lanes read the vector's 128 floats as one coalesced 512-byte
        // row (lane L: dims 4L .. 4L + 3) and store 4 halves into chunk L / 2
        // (all 16 loads are issued before the first conversion, so that their latencies overlap)
        float4 a[16];
        int rl = (warp * 16) / G, x = (warp * 16) % G;
#pragma unroll
        for (int rr = 0; rr < 16; rr++) {
            a[rr] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (rl < w.nrows) a[rr] = __ldg(reinterpret_cast<const float4 *>(q + ((size_t)(w.row0 + rl) * n_heads + (size_t)g * G + x) * qh) + lane);
            if (++x == G) x = 0, rl++;
        }
#pragma unroll
        for (int rr = 0; rr < 16; rr++) {
            const int t = warp * 16 + rr;
            __half2 h0 = __floats2half2_rn(a[rr].x, a[rr].y), h1 = __floats2half2_rn(a[rr].z, a[rr].w);
            const int c = lane >> 1;
            *reinterpret_cast<uint2 *>(sQ + (c >> 3) * 16384 + t * 128 + (((c & 7) ^ (t & 7)) << 4) + (lane & 1) * 8) =
                make_uint2(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1));
        }
    }
    fence_proxy_async();  // Q was written by ordinary stores and will be read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    bool ok = true;

    if (warp >= 8) {
        // ---- three warps: P V issue, S issue, TMA loads.  The softmax threads free S as soon as they hold their scores
        // in registers, so S (j + 1) is computed while they work on block j and they never wait for the tensor cores;
        // P is double-buffered, so P V (j) runs under the softmax of block j + 1.  Each of the three warps runs its loop
        // converged (all lanes wait, descriptors stay warp-uniform) and one elected lane issues
        constexpr uint32_t idesc = umma_idesc(128, 128);
        // (a descriptor's address field counts 16-byte units from bit 0: adding bytes / 16 moves the start)
        if (warp == 8) {
            // O (stream h) += P (j, h) V (j, h): keys 64 h .. 64 h + 63 of block j, 4 k-steps of 16 keys each
            const uint64_t dv = umma_desc(smem_u32(sV), 16384, 1024, 2);
            for (int j = 0; j < nblk; j++) {
                const uint32_t ph = j & 1, ph2 = (j >> 1) & 1;
                const uint64_t b0 = dv + (uint64_t)(ph * (32768 >> 4));
                const uint32_t pa = tbase + P_COL + ph * 64;
                ok = mbar_wait_sleepy(bar_v + ph, ph2, err, 14) && ok;
                ok = mbar_wait_sleepy(bar_p + ph, ph2, err, 13) && ok;  // P(j) of stream 0 is in TMEM
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) umma_ts(tbase + O_COL, pa + ks * 8, b0 + (uint64_t)(ks * 128), idesc, (j > 0) | (ks > 0));
                }
                __syncwarp();
                ok = mbar_wait_sleepy(bar_p + 2 + ph, ph2, err, 13) && ok;
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < 4; ks++)
                        umma_ts(tbase + O_COL + 128, pa + 32 + ks * 8, b0 + (uint64_t)(512 + ks * 128), idesc, (j > 0) | (ks > 0));
                    umma_commit(bar_o + ph);  // both streams' P (j) were read, V (j) too
                }
                __syncwarp();
            }
        } else if (warp == 9) {
            // S (j) = Q K (j)^T, once every softmax thread has read S (j - 1)
            const uint64_t dq = umma_desc(smem_u32(sQ), 16, 1024, 2), dk = umma_desc(smem_u32(sK), 4096, 256, 6);
            for (int j = 0; j < nblk; j++) {
                const uint64_t b0 = dk + (uint64_t)((j % 3) * (32768 >> 4));
                ok = mbar_wait_sleepy(bar_k + j % 3, (j / 3) & 1, err, 11) && ok;
                if (j >= 1) ok = mbar_wait_sleepy(bar_sfree, (j - 1) & 1, err, 12) && ok;
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < 8; ks++)
                        umma_ss(tbase, dq + (uint64_t)(((ks >> 2) * 16384 + (ks & 3) * 32) >> 4), b0 + (uint64_t)(ks * 32), idesc,
                                ks > 0);
                    umma_commit(bar_s);
                    umma_commit(bar_kfree + j % 3);
                }
                __syncwarp();
            }
        } else if (warp == 10) {
            // K (j + 3) into the stage of K (j) once S (j) is complete; V (j + 2) into the stage of V (j) once P V (j) is
            if (lane == 0) {
                if (nblk > 1) load_k(1);
                load_v(0);
                if (nblk > 2) load_k(2);
                if (nblk > 1) load_v(1);
            }
            __syncwarp();
            for (int j = 0; j < nblk; j++) {
                if (j + 3 < nblk) {
                    ok = mbar_wait_sleepy(bar_kfree + j % 3, (j / 3) & 1, err, 15) && ok;
                    if (lane == 0) load_k(j + 3);
                }
                if (j + 2 < nblk) {
                    ok = mbar_wait_sleepy(bar_o + (j & 1), (j >> 1) & 1, err, 16) && ok;
                    if (lane == 0) load_v(j + 2);
                }
                __syncwarp();
            }
        }
    } else {
        // ---- softmax: warps 0-3 are stream 0, warps 4-7 stream 1; thread t of a stream owns query vector t (TMEM lane t)
        // and, of every key block, the 64 keys of its stream, with its own running max, row sum and O accumulator:
        // the two streams are independent until the epilogue merges them
        const int h = warp >> 2, t = tid & 127, rl = t / G;
        const int np = rl < w.nrows ? np_min + rl : 0;  // positions this vector attends (0: a padding vector)
        const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t o_col = O_COL + h * 128;
        const float c = scale * 1.44269504088896341f;
        float m_used = -INFINITY, l = 0.0f;
        // The waits of the loop are polled once well before their result is needed (a poll of a completed barrier
        // still takes ~150 cycles to answer), and only a poll that failed is followed by a real wait
        bool s_seen = false;
        for (int j = 0; j < nblk; j++) {
            const int t0 = s0 + j * PF_BN + h * 64;  // first key of this thread's half of the block
            if (!s_seen) ok = mbar_wait_bounded(bar_s, j & 1, err, 21) && ok;
            tc_fence_after();
            uint32_t r[2][32], pk[32];
            tmem_ld32(lane_addr + h * 64, r[0]);
            tmem_ld32(lane_addr + h * 64 + 32, r[1]);
            // P V (j - 2) was the last reader of the P buffer this block will store to
            const bool o_seen = j < 2 || mbar_try_wait(bar_o + (j & 1), ((j - 2) >> 1) & 1);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar_sfree);  // the scores are in registers: S (j + 1) may be computed
            const bool need_mask = s0 + (j + 1) * PF_BN > np_min;  // (uniform over the CTA: only the blocks on the diagonal)
            if (need_mask) {
#pragma unroll
                for (int cc = 0; cc < 2; cc++)
#pragma unroll
                    for (int x = 0; x < 32; x++)
                        if (t0 + cc * 32 + x >= np) r[cc][x] = 0xff800000u;  // -inf
            }
            // p = 2^((s - m) c) (a masked score is -inf: p = 0) as f16 pairs, the row sum, and the row maximum in the
            // same sweep, so that its comparisons fill the issue slots the exponential unit leaves
            float mx, lsum;
            auto sweep = [&](float mc) {
                // (scalar FMA / add on purpose: measured on this kernel's mix, the packed f32x2 forms and a polynomial
                // 2^x on the FMA pipe are both slower: the sweep is bound by issue slots, not by the exponential unit)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                for (int cc = 0; cc < 2; cc++) {
#pragma unroll
                    for (int x = 0; x < 32; x += 2) {
                        const int i = cc * 16 + (x >> 1);  // pair index
                        const float a0 = __uint_as_float(r[cc][x]), a1 = __uint_as_float(r[cc][x + 1]);
                        const float p0 = ex2(fmaf(a0, c, -mc)), p1 = ex2(fmaf(a1, c, -mc));
                        mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(a0, a1));
                        l4[i & 3] += p0 + p1;
                        __half2 hh = __floats2half2_rn(p0, p1);
                        pk[i] = *reinterpret_cast<uint32_t *>(&hh);
                    }
                }
                mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                lsum = (l4[0] + l4[1]) + (l4[2] + l4[3]);
            };
            // The running max moves only when the block's maximum exceeds it by more than 8 in the exponent (p stays
            // below 2^8: exact enough in f16, and O is rescaled rarely).  So the sweep runs with the running max as it
            // stands; in the rare block where some row's max has to move (the first block with a valid key always),
            // O and l of the warp's rows are rescaled and the sweep is repeated with the new max
            const bool fresh = __any_sync(0xffffffffu, m_used == -INFINITY);  // (the first block; rows without a valid key so far)
            if (fresh) {  // no running max to sweep with yet: the block's maximum first
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int cc = 0; cc < 2; cc++)
#pragma unroll
                    for (int x = 0; x < 32; x++) mx4[x & 3] = fmaxf(mx4[x & 3], __uint_as_float(r[cc][x]));
                mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            } else {
                sweep(m_used * c);
            }
            const bool move = mx > -INFINITY && (m_used == -INFINITY || (mx - m_used) * c > 8.0f);
            const bool any_move = __any_sync(0xffffffffu, move);
            if (fresh || any_move) {
                float alpha = 1.0f;
                if (move) {
                    alpha = m_used == -INFINITY ? 0.0f : ex2((m_used - mx) * c);
                    m_used = mx;
                }
                if (j > 0 && any_move) {
                    // (P V (j - 1) must have completed; P V (j - 3), the barrier's phase before, was seen complete
                    // before P (j - 1) was stored)
                    ok = mbar_wait_bounded(bar_o + ((j - 1) & 1), ((j - 1) >> 1) & 1, err, 23) && ok;
                    tc_fence_after();
                    l *= alpha;
#pragma unroll 1
                    for (int cc = 0; cc < 4; cc++) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + o_col + cc * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
                        tmem_st32(lane_addr + o_col + cc * 32, o);
                    }
                    tmem_wait_st();
                }
                sweep(m_used == -INFINITY ? 0.0f : m_used * c);
            }
            l += lsum;
            if (!o_seen) ok = mbar_wait_bounded(bar_o + (j & 1), ((j - 2) >> 1) & 1, err, 24) && ok;
            tc_fence_after();
            tmem_st32(lane_addr + P_COL + (j & 1) * 64 + h * 32, pk);
            s_seen = j + 1 < nblk && mbar_try_wait(bar_s, (j + 1) & 1);  // (answered while the store completes)
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p + 2 * h + (j & 1));
        }
        // ---- epilogue: the two streams merge into the partial result (o unnormalised, m in scaled-score units, l)
        sml[(h * 128 + t) * 2] = m_used;
        sml[(h * 128 + t) * 2 + 1] = l;
        ok = mbar_wait_bounded(bar_o + ((nblk - 1) & 1), ((nblk - 1) >> 1) & 1, err, 22) && ok;
        tc_fence_after();
        asm volatile("bar.sync 1, 256;" ::: "memory");  // (the softmax warps only) every MMA of the CTA is complete
        const float m_other = sml[((h ^ 1) * 128 + t) * 2], l_other = sml[((h ^ 1) * 128 + t) * 2 + 1];
        const float M = fmaxf(m_used, m_other);
        const float c_own = m_used == -INFINITY ? 0.0f : ex2((m_used - M) * c), c_other = m_other == -INFINITY ? 0.0f : ex2((m_other - M) * c);
        {
            // The merged rows go through shared memory (Q, K and V are no longer needed) so that the global stores are
            // coalesced.  Thread (h, t) merges dims 64 h .. 64 h + 63 of vector t: both streams' O are in its TMEM lane
            constexpr int OST = HD + 4;  // floats per staged row (the padding spreads the rows over the banks)
            float *so = reinterpret_cast<float *>(sm);
            const float c0 = h ? c_other : c_own, c1 = h ? c_own : c_other;  // the factors of stream 0's and stream 1's O
#pragma unroll 1
            for (int cc = 0; cc < 2; cc++) {
                uint32_t r0[32], r1[32];
                tmem_ld32(lane_addr + O_COL + h * 64 + cc * 32, r0);
                tmem_ld32(lane_addr + O_COL + 128 + h * 64 + cc * 32, r1);
                tmem_wait_ld();
#pragma unroll
                for (int y = 0; y < 32; y += 4)
                    *reinterpret_cast<float4 *>(so + (size_t)t * OST + h * 64 + cc * 32 + y) =
                        make_float4(__uint_as_float(r0[y]) * c0 + __uint_as_float(r1[y]) * c1, __uint_as_float(r0[y + 1]) * c0 + __uint_as_float(r1[y + 1]) * c1,
                                    __uint_as_float(r0[y + 2]) * c0 + __uint_as_float(r1[y + 2]) * c1, __uint_as_float(r0[y + 3]) * c0 + __uint_as_float(r1[y + 3]) * c1);
            }
            if (h == 0) {
                so[(size_t)t * OST + HD] = M * scale;
                so[(size_t)t * OST + HD + 1] = c_own * l + c_other * l_other;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            // a warp writes 16 vectors, one 512-byte row (+ m, l) per step; the steps are independent, so their shared-memory
            // loads and global stores overlap
            int rl2 = (warp * 16) / G, x = (warp * 16) % G;
#pragma unroll
            for (int rr = 0; rr < 16; rr++) {
                const int tt = warp * 16 + rr;
                const bool valid = rl2 < w.nrows;
                float *p = part + (((size_t)(w.row0 + rl2) * max_splits + w.split) * n_heads + (size_t)g * G + x) * RQ_PSTRIDE(HD);
                const float4 a = *reinterpret_cast<const float4 *>(so + (size_t)tt * OST + 4 * lane);
                const float ml = so[(size_t)tt * OST + HD + (lane & 1)];
                if (valid) {
                    *reinterpret_cast<float4 *>(p + 4 * lane) = ok ? a : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (lane < 2) p[HD + lane] = ml;
                }
                if (++x == G) x = 0, rl2++;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 10) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(TM_COLS));
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
    return launch_pdl(attn_prefill_kernel, dim3(a.n_work, a.n_kv), dim3(PF_THREADS), PF_SMEM, stream, a.work, a.rows, a.maps, a.layer, a.n_kv, a.G, a.q,
                      a.qh, a.n_heads, a.scale, a.max_splits, a.split_len, a.part, a.err);
}
#endif  // RQ_ATTN_PREFILL_INSTANTIATE

}  // namespace rq
