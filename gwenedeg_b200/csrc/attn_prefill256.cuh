// Chunked causal prefill attention on tcgen05 + TMEM for head_dim 256 (f16 KV cache): the Qwen3.5-style gated attention
// layers (16 query / 4 KV heads x 256).  Same work items, partial-result format and merge as attn_prefill_kernel (head_dim
// 128): (M tile of 128 query vectors = 128 / G consecutive rows x the G query heads of one KV head, KV head, split of
// PF_SPLIT key positions); the reference runs this shape through the same attention_kv as head_dim 128
// (src/kernels_avx512.h:1416: head dims that are multiples of 128 up to 256; call site src/forward.c:3096-3146, output gate
// :2291-2295, applied here by the merge kernel).
//
// What differs from the head_dim 128 kernel is the budget: Q alone is 64 KB of shared memory and O needs 256 TMEM
// columns, so there is one O accumulator and one running maximum per query vector; the softmax of a block is still spread
// over eight warps: threads t and 128 + t own query vector t (TMEM lane t) and 64 keys of the block each, exchange their
// block maxima through shared memory (one barrier of the softmax warps per block) and so scale their halves of P alike.
// K and V are staged in halves of 128 dims (32 KB each: the shared-memory layouts, tensor-map boxes and descriptors of
// the head_dim 128 kernel):
//   TMA warp   K (j) dims 0-127, K (j) dims 128-255 into a ring of 3 half stages, V (j) likewise into a ring of 2,
//              refilled as their consumers' MMAs complete (one lane polls both rings).
//   S warp     S = Q K^T: 2 x 8 tcgen05.mma (M 128, N 128, K 16), the first 8 against the first K half.
//   softmax    scores -> registers (S is freed at once), p = 2^((s - m) c) with the lazily moved running max, row sums per
//              half, P (f16) -> TMEM, double-buffered over key blocks.
//   P V warp   O[:, 0:128] += P V[:, 0:128], then O[:, 128:256] += P V[:, 128:256]: 2 x 8 MMAs with P from TMEM.
// TMEM: S 128 columns, P 2 x 64, O 256.  Per 128-key block the tensor cores have 2,048 cycles of work; with four softmax
// warps (one per scheduler, 128 keys per thread) the softmax took longer than that, with eight it does not.
#pragma once
#include "attn_prefill.cuh"

namespace rq {

constexpr int PF256_THREADS = 352;  // 8 softmax warps + the P V, S and TMA warps
// launches attn_prefill_hd256_kernel (grid: work items x KV heads) on `stream`
cudaError_t launch_attn_prefill_hd256(const AttnPrefillArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_PREFILL_INSTANTIATE

constexpr int PF256_Q = 65536, PF256_HALF = 32768, PF256_BARS = PF256_Q + 5 * PF256_HALF;
constexpr int PF256_XCH = PF256_BARS + 256;  // the softmax threads' exchange: [2 halves][128 vectors] floats
constexpr int PF256_SMEM = PF256_XCH + 1024 + 1024;  // Q | K x 3 half stages | V x 2 half stages | barriers, TMEM slot | exchange | alignment slack
static_assert(PF256_SMEM <= 227 * 1024, "one CTA's shared memory");

// maps: per segment the tensor maps of its sequence's K cache ({16 positions, rows of 32 bytes}, 32-byte swizzle, box 16 x
// 128: the 128-dim half of one tile) and V cache ({256 dims, rows of 512 bytes}, 128-byte swizzle, box 64 x 128).
__global__ void __launch_bounds__(PF256_THREADS, 1) attn_prefill_hd256_kernel(const PfWork *__restrict__ work, const PassRow *__restrict__ rows,
                                                                            const CUtensorMap *__restrict__ maps, int layer, int n_kv, int G,
                                                                            const float *__restrict__ q, int qh, int n_heads, float scale,
                                                                            int max_splits, int split_len, float *__restrict__ part, int *err) {
    constexpr int HD = 256, TM_COLS = 512, P_COL = 128, O_COL = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = sm, *sK = sm + PF256_Q, *sV = sK + 3 * PF256_HALF;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + PF256_BARS);
    // K half stage loaded (3) / free again (3), V half stage loaded (2) / free again (2), S written (1), S read by every
    // softmax thread (1), P V of block j complete (2: j % 2), P (j) stored (2: j % 2)
    uint64_t *bar_k = bars, *bar_kfree = bars + 3, *bar_v = bars + 6, *bar_vfree = bars + 8, *bar_s = bars + 10, *bar_sfree = bars + 11,
             *bar_o = bars + 12, *bar_p = bars + 14;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + PF256_BARS + 192);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_wait();
    pdl_launch_dependents();
    const PfWork w = work[blockIdx.x];
    const int g = blockIdx.y;
    const PassRow r0 = rows[w.row0];
    const int np_min = r0.np, np_max = r0.np + w.nrows - 1;  // rows of a tile are at consecutive positions
    const int s0 = w.split * split_len;
    const int s1 = min(s0 + split_len, np_max);
    const int nblk = (s1 - s0 + PF_BN - 1) / PF_BN;  // >= 1 by construction of the work list
    RQ_CHECK(w.nrows >= 1 && w.nrows * G <= 128 && s0 >= 0 && s0 < np_max && nblk >= 1 && nblk <= split_len / PF_BN && g < n_kv && w.split < max_splits, err, 46);
    const int n_items = 2 * nblk;  // half stages of K (and of V) this CTA consumes
    const CUtensorMap *mk = maps + 2 * w.seg, *mv = mk + 1;
    // rows of the 2-D views: K rows are 32 bytes (one dim of a tile), V rows 512 bytes (one position)
    const long long k_layer_rows = (long long)(r0.lk / 32), v_layer_rows = (long long)(r0.lv / 512);

    auto load_k = [&](int item) {  // dims 128 h .. 128 h + 127 of key block j (item = 2 j + h) -> K slot item % 3
        const int j = item >> 1, h = item & 1, t0 = s0 + j * PF_BN;
        uint64_t *bar = bar_k + item % 3;
        uint8_t *dst = sK + (item % 3) * PF256_HALF;
        mbar_expect_tx(bar, PF256_HALF);
        const long long y = (long long)layer * k_layer_rows + ((long long)(t0 / ATT_P) * n_kv + g) * (ATT_PT * HD) + (long long)((t0 % ATT_P) / ATT_T) * HD + 128 * h;
        for (int u = 0; u < 8; u++) tma_load_2d(dst + u * 4096, mk, 0, (int)(y + (long long)u * HD), bar);
    };
    auto load_v = [&](int item) {  // -> V slot item % 2
        const int j = item >> 1, h = item & 1, t0 = s0 + j * PF_BN;
        uint64_t *bar = bar_v + (item & 1);
        uint8_t *dst = sV + (item & 1) * PF256_HALF;
        mbar_expect_tx(bar, PF256_HALF);
        const long long y = (long long)layer * v_layer_rows + ((long long)(t0 / ATT_P) * n_kv + g) * ATT_P + (t0 % ATT_P);
        for (int i = 0; i < 2; i++) tma_load_2d(dst + i * 16384, mv, 128 * h + 64 * i, (int)y, bar);
    };

    if (tid == 0) {
        for (int i = 0; i < 16; i++) mbar_init(bars + i, (i == 11 || i >= 14) ? 256 : 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 10) {
        if (lane == 0) {  // the first half stages start loading while the other warps convert Q
            load_k(0);
            load_k(1);
            load_v(0);
            if (n_items > 2) load_k(2);
            load_v(1);
        }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    } else {
        // Q tile -> shared memory as f16, K-major with the 128-byte swizzle, four k-blocks of 64 dims: vector t = row t / G,
        // head g G + t % G; 16-byte chunk c of 32: k-block c / 8, physical chunk (c % 8) ^ (t % 8).  Six warps take the
        // vectors round robin, eight at a time (16 row loads per lane in flight: lane L holds dims 4L .. 4L + 3 and
        // 128 + 4L .. 128 + 4L + 3)
        constexpr int QW = 10;  // warps that convert
        for (int tb = warp; tb < 128; tb += 8 * QW) {
            float4 a[8][2];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int t = tb + QW * u, rl = t / G, x = t % G;
                a[u][0] = a[u][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (t < 128 && rl < w.nrows) {
                    const float4 *src = reinterpret_cast<const float4 *>(q + ((size_t)(w.row0 + rl) * n_heads + (size_t)g * G + x) * qh);
                    a[u][0] = __ldg(src + lane);
                    a[u][1] = __ldg(src + 32 + lane);
                }
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int t = tb + QW * u;
                if (t < 128) {
#pragma unroll
                    for (int hh = 0; hh < 2; hh++) {
                        __half2 h0 = __floats2half2_rn(a[u][hh].x, a[u][hh].y), h1 = __floats2half2_rn(a[u][hh].z, a[u][hh].w);
                        const int c = 16 * hh + (lane >> 1);
                        *reinterpret_cast<uint2 *>(sQ + (c >> 3) * 16384 + t * 128 + (((c & 7) ^ (t & 7)) << 4) + (lane & 1) * 8) =
                            make_uint2(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1));
                    }
                }
            }
        }
    }
    fence_proxy_async();  // Q was written by ordinary stores and will be read by the tensor core
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    bool ok = true;

    if (warp >= 8) {
        constexpr uint32_t idesc = umma_idesc(128, 128);
        if (warp == 8) {
            // O[:, 128 h : 128 h + 128] += P (j) V (j)[:, 128 h : 128 h + 128]: 8 k-steps of 16 keys each
            const uint64_t dv = umma_desc(smem_u32(sV), 16384, 1024, 2);
            for (int j = 0; j < nblk; j++) {
                const uint32_t pa = tbase + P_COL + (j & 1) * 64;
                for (int h = 0; h < 2; h++) {
                    const int item = 2 * j + h, slot = item & 1;
                    ok = mbar_wait_sleepy(bar_v + slot, (item >> 1) & 1, err, 54) && ok;
                    if (h == 0) ok = mbar_wait_sleepy(bar_p + (j & 1), (j >> 1) & 1, err, 53) && ok;  // P (j) is in TMEM
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t b0 = dv + (uint64_t)(slot * (PF256_HALF >> 4));
#pragma unroll
                        for (int ks = 0; ks < 8; ks++) umma_ts(tbase + O_COL + 128 * h, pa + ks * 8, b0 + (uint64_t)(ks * 128), idesc, (j > 0) | (ks > 0));
                        umma_commit(bar_vfree + slot);
                        if (h == 1) umma_commit(bar_o + (j & 1));  // P (j) and both V halves were read, O holds block j
                    }
                    __syncwarp();
                }
            }
        } else if (warp == 9) {
            // S (j) = Q K (j)^T over the two K halves, once every softmax thread has read S (j - 1)
            const uint64_t dq = umma_desc(smem_u32(sQ), 16, 1024, 2), dk = umma_desc(smem_u32(sK), 4096, 256, 6);
            for (int j = 0; j < nblk; j++) {
                for (int h = 0; h < 2; h++) {
                    const int item = 2 * j + h, slot = item % 3;
                    ok = mbar_wait_sleepy(bar_k + slot, (item / 3) & 1, err, 51) && ok;
                    if (h == 0 && j >= 1) ok = mbar_wait_sleepy(bar_sfree, (j - 1) & 1, err, 52) && ok;
                    tc_fence_after();
                    if (elect_one()) {
                        const uint64_t b0 = dk + (uint64_t)(slot * (PF256_HALF >> 4));
#pragma unroll
                        for (int ks = 0; ks < 8; ks++) {
                            const int kg = 8 * h + ks;  // k-step of 16 dims over the 256
                            umma_ss(tbase, dq + (uint64_t)(((kg >> 2) * 16384 + (kg & 3) * 32) >> 4), b0 + (uint64_t)(ks * 32), idesc, (h > 0) | (ks > 0));
                        }
                        umma_commit(bar_kfree + slot);
                        if (h == 1) umma_commit(bar_s);
                    }
                    __syncwarp();
                }
            }
        } else {
            // refills: K item i + 3 into the slot of item i once its MMAs are complete, V item i + 2 likewise; one lane
            // polls both rings so that neither waits for the other (a bounded number of polls: on expiry the status word
            // is set and the consumers' own bounded waits end the kernel)
            if (lane == 0) {
                int kn = 3, vn = 2;
                unsigned long long t_start = 0;
                for (unsigned it = 0; (kn < n_items || vn < n_items) && it < (1u << 28); it++) {
                    bool progress = false;
                    if (kn < n_items && mbar_try_wait(bar_kfree + (kn - 3) % 3, ((kn - 3) / 3) & 1)) {
                        load_k(kn++);
                        progress = true;
                    }
                    if (vn < n_items && mbar_try_wait(bar_vfree + (vn & 1), ((vn - 2) >> 1) & 1)) {
                        load_v(vn++);
                        progress = true;
                    }
                    if (progress) {
                        t_start = 0;
                    } else {
                        unsigned long long now;
                        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                        if (t_start == 0) t_start = now;
                        if (now - t_start > 200000000ull || *reinterpret_cast<volatile int *>(err) != 0) {
                            atomicCAS(err, 0, 55);
                            break;
                        }
                        __nanosleep(200);
                    }
                }
            }
            __syncwarp();
        }
    } else {
        // ---- softmax: threads t and 128 + t own query vector t (TMEM lane t); of every key block thread (h, t) takes keys
        // 64 h .. 64 h + 63.  The two share the vector's running maximum (exchanged per block) and its O accumulator
        const int h = warp >> 2, t = tid & 127, rl = t / G;
        const int np = rl < w.nrows ? np_min + rl : 0;  // positions this vector attends (0: a padding vector)
        const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        float *xch = reinterpret_cast<float *>(sm + PF256_XCH);  // [2][128]
        const float c = scale * 1.44269504088896341f;
        float m_used = -INFINITY, l = 0.0f;
        bool s_seen = false;
        for (int j = 0; j < nblk; j++) {
            const int t0 = s0 + j * PF_BN + 64 * h;  // first key of this thread's half of the block
            if (!s_seen) ok = mbar_wait_bounded(bar_s, j & 1, err, 61) && ok;
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
            float mx, lsum;
            auto sweep = [&](float mc) {
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
            // the running max moves only when the block's maximum exceeds it by more than 8 in the exponent (as in the
            // head_dim 128 kernel): the sweep runs with the running max as it stands and is repeated, after O and l were
            // rescaled, in the rare block where some row's max has to move (the first block with a valid key always).
            // The block's maximum of a vector is the larger of its two threads' (same m_used in both, so the same decision)
            const bool fresh = __any_sync(0xffffffffu, m_used == -INFINITY);
            if (fresh) {
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int cc = 0; cc < 2; cc++)
#pragma unroll
                    for (int x = 0; x < 32; x++) mx4[x & 3] = fmaxf(mx4[x & 3], __uint_as_float(r[cc][x]));
                mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            } else {
                sweep(m_used * c);
            }
            xch[h * 128 + t] = mx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            mx = fmaxf(mx, xch[(h ^ 1) * 128 + t]);
            asm volatile("bar.sync 1, 256;" ::: "memory");  // (the exchange buffer may be written again)
            const bool move = mx > -INFINITY && (m_used == -INFINITY || (mx - m_used) * c > 8.0f);
            const bool any_move = __any_sync(0xffffffffu, move);
            if (fresh || any_move) {
                float alpha = 1.0f;
                if (move) {
                    alpha = m_used == -INFINITY ? 0.0f : ex2((m_used - mx) * c);
                    m_used = mx;
                }
                if (j > 0 && any_move) {
                    // (P V (j - 1) must have completed before its accumulator is rescaled; each half rescales its 128 columns,
                    // and P V (j) waits for both halves' P)
                    ok = mbar_wait_bounded(bar_o + ((j - 1) & 1), ((j - 1) >> 1) & 1, err, 63) && ok;
                    tc_fence_after();
                    l *= alpha;
#pragma unroll 1
                    for (int cc = 0; cc < 4; cc++) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + O_COL + h * 128 + cc * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int x = 0; x < 32; x++) o[x] = __float_as_uint(__uint_as_float(o[x]) * alpha);
                        tmem_st32(lane_addr + O_COL + h * 128 + cc * 32, o);
                    }
                    tmem_wait_st();
                }
                sweep(m_used == -INFINITY ? 0.0f : m_used * c);
            }
            l += lsum;
            if (!o_seen) ok = mbar_wait_bounded(bar_o + (j & 1), ((j - 2) >> 1) & 1, err, 64) && ok;
            tc_fence_after();
            tmem_st32(lane_addr + P_COL + (j & 1) * 64 + h * 32, pk);
            s_seen = j + 1 < nblk && mbar_try_wait(bar_s, (j + 1) & 1);  // (answered while the stores complete)
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p + (j & 1));
        }
        // ---- epilogue: the partial result (o unnormalised, m in scaled-score units, l) of every vector of the tile
        ok = mbar_wait_bounded(bar_o + ((nblk - 1) & 1), ((nblk - 1) >> 1) & 1, err, 62) && ok;
        tc_fence_after();
        xch[h * 128 + t] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");  // (the softmax warps only) every MMA of the CTA is complete
        {
            // the rows of O go through shared memory (Q, K and V are no longer needed) so that the global stores are coalesced:
            // thread (h, t) stages columns 128 h .. 128 h + 127 of row t, then a warp writes one vector's 1 KB row per step
            constexpr int OST = HD + 4;  // floats per staged row (the padding spreads the rows over the banks)
            float *so = reinterpret_cast<float *>(sm);
            const float l_all = l + xch[(h ^ 1) * 128 + t];
#pragma unroll 1
            for (int cc = 0; cc < 4; cc++) {
                uint32_t rr[32];
                tmem_ld32(lane_addr + O_COL + h * 128 + cc * 32, rr);
                tmem_wait_ld();
#pragma unroll
                for (int y = 0; y < 32; y += 4)
                    *reinterpret_cast<float4 *>(so + (size_t)t * OST + h * 128 + cc * 32 + y) =
                        make_float4(__uint_as_float(rr[y]), __uint_as_float(rr[y + 1]), __uint_as_float(rr[y + 2]), __uint_as_float(rr[y + 3]));
            }
            if (h == 0) {
                so[(size_t)t * OST + HD] = m_used * scale;
                so[(size_t)t * OST + HD + 1] = l_all;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            int rl2 = (warp * 16) / G, x = (warp * 16) % G - 1;
#pragma unroll 4
            for (int rr = 0; rr < 16; rr++) {
                const int tt = warp * 16 + rr;
                if (++x == G) x = 0, rl2++;
                if (rl2 >= w.nrows) continue;
                float *p = part + (((size_t)(w.row0 + rl2) * max_splits + w.split) * n_heads + (size_t)g * G + x) * RQ_PSTRIDE(HD);
                const float4 a = *reinterpret_cast<const float4 *>(so + (size_t)tt * OST + 4 * lane);
                const float4 b = *reinterpret_cast<const float4 *>(so + (size_t)tt * OST + 128 + 4 * lane);
                const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                *reinterpret_cast<float4 *>(p + 4 * lane) = ok ? a : z;
                *reinterpret_cast<float4 *>(p + 128 + 4 * lane) = ok ? b : z;
                if (lane < 2) p[HD + lane] = so[(size_t)tt * OST + HD + lane];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 10) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(TM_COLS));
}

cudaError_t launch_attn_prefill_hd256(const AttnPrefillArgs &a, cudaStream_t stream) {
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_hd256_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF256_SMEM);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    return launch_pdl(attn_prefill_hd256_kernel, dim3(a.n_work, a.n_kv), dim3(PF256_THREADS), PF256_SMEM, stream, a.work, a.rows, a.maps, a.layer, a.n_kv, a.G,
                      a.q, a.qh, a.n_heads, a.scale, a.max_splits, a.split_len, a.part, a.err);
}
#endif  // RQ_ATTN_PREFILL_INSTANTIATE

}  // namespace rq
