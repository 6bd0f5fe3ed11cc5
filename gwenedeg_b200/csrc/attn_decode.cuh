// Split-K flash-decode attention over the tiled KV cache (f16 / q8 / q4 / q4k4), sm_100a.
//
// Work decomposition = the reference's: one partial result (o, m, l) per (row, KV head, block of 256 positions)
// (attention_part, reference src/forward.c:1806; definition src/kernels_avx512.h:1109-1126), merged per query vector in
// block order (att_combine, src/forward.c:1405).  The split depends on a row's own length only, so a row of a batch
// gives the bits it gives alone, on any grid.  The arithmetic inside a block also follows the definition operation for
// operation (fp32, fused multiply-add chains over 32-dim chunks for the scores and over the positions for the
// outputs, the 16-lane sum of exponentials and its tree), so results agree with the CPU code to the last bit.
//
// attn_part_kernel: one CTA of 128 threads per (block, KV head).  The K tiles of the block (64 KB at head_dim 128,
// f16) arrive in shared memory through bulk async copies (TMA) completing on an mbarrier; every thread scores two
// positions for all the query heads of the KV head; the V tiles then reuse the same shared-memory buffer while the
// softmax of the block is computed; every thread accumulates one (or two) output dims over the block's positions.
// Three CTAs fit on an SM, so the copies of two blocks are in flight while a third computes.
// attn_combine_kernel: one CTA per (row, query head) merges the partials, un-rotates (q8 / q4) and gates the output.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace rq {

// One row of the open pass, as the kernels see it.
struct PassRow {
    const uint8_t *k, *v;        // the row's sequence: K / V cache of layer 0
    unsigned long long lk, lv;   // bytes from one layer to the next
    int np;                      // positions the row attends: 0 .. np - 1
    int blk0;                    // 256-position blocks of all earlier rows (prefix sum: the partials' index)
    int seg;                     // index of the row's segment
    int pos;                     // the row's own position (np - 1)
};

constexpr int DEC_THREADS = 128;

template <int KVT, int HD>
struct DecCfg {
    static constexpr int KF = kv_fmt(KVT, 0), VF = kv_fmt(KVT, 1);
    static constexpr int KTB = kv_tile_bytes(KVT, HD, 0), VTB = kv_tile_bytes(KVT, HD, 1);
    // positions per stage: a 16-bit cache at head_dim 256 is streamed in two halves of 128 positions
    static constexpr int STAGES = (KF == KV_F16 && HD == 256) ? 2 : 1;
    static constexpr int ST_TILES = ATT_PT / STAGES;
    static constexpr int ST_POS = ATT_P / STAGES;
    // bytes the 16 positions of one dim (pair) occupy in a K tile: the padding that spreads the tiles a warp reads
    // at once over different banks
    static constexpr int KPAD = KF == KV_F16 ? 32 : 16;
    static constexpr int KSTRIDE = KTB + KPAD;
    static constexpr int KBUF = ST_TILES * KSTRIDE, VBUF = ST_TILES * VTB;
    static constexpr int BUF = (KBUF > VBUF ? KBUF : VBUF);
    static constexpr int DPT = HD > 128 ? HD / 128 : 1;  // output dims per thread
};

__host__ __device__ inline size_t dec_smem_bytes(int buf, int hd, int nvt) {
    // kv buffer | q [groups][hd][4] | e [256][nvt] | reductions [4][nvt] + m[nvt] + l[nvt] | barrier
    int ngrp = (nvt + 3) / 4;
    return (size_t)buf + (size_t)ngrp * hd * 4 * 4 + (size_t)ATT_P * nvt * 4 + (size_t)6 * nvt * 4 + 16 + 64;
}

// dims i of positions (2 jp, 2 jp + 1) of a K tile
template <int KF, int HD>
__device__ __forceinline__ void load_k2(const uint8_t *kt, int i, int jp, float d0, float d1, float &k0, float &k1) {
    if constexpr (KF == KV_F16) {
        __half2 h = *reinterpret_cast<const __half2 *>(kt + (size_t)i * 32 + jp * 4);
        k0 = __low2float(h);
        k1 = __high2float(h);
    } else if constexpr (KF == KV_Q8) {
        uint32_t w = *reinterpret_cast<const uint16_t *>(kt + (size_t)i * 16 + jp * 2);
        k0 = (float)(int)(int8_t)(w & 0xff) * d0;
        k1 = (float)(int)(int8_t)(w >> 8) * d1;
    } else {  // q4: byte [dim pair][position], low nibble dim 2p, high nibble dim 2p + 1
        uint32_t w = *reinterpret_cast<const uint16_t *>(kt + (size_t)(i >> 1) * 16 + jp * 2);
        int sh = 4 * (i & 1);
        k0 = (float)((int)((w >> sh) & 15) - 8) * d0;
        k1 = (float)((int)((w >> (8 + sh)) & 15) - 8) * d1;
    }
}

// dim i of position j of a K tile (head_dim 256, f16 only)
template <int KF, int HD>
__device__ __forceinline__ float load_k1(const uint8_t *kt, int i, int j) {
    return __half2float(*reinterpret_cast<const __half *>(kt + ((size_t)i * 16 + j) * 2));
}

// bf16 scale of (chunk c, position j) of a quantised K tile
template <int KF, int HD>
__device__ __forceinline__ float k_scale(const uint8_t *kt, int c, int j) {
    constexpr int off = (KF == KV_Q4 ? 8 : 16) * HD;
    return bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(kt + off + (c * 16 + j) * 2));
}

// dim i of position j of a V tile
template <int VF, int HD>
__device__ __forceinline__ float load_v(const uint8_t *vt, int j, int i) {
    if constexpr (VF == KV_F16) {
        return __half2float(*reinterpret_cast<const __half *>(vt + ((size_t)j * HD + i) * 2));
    } else if constexpr (VF == KV_Q8) {
        float d = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(vt + 16 * HD + (j * (HD / 32) + (i >> 5)) * 2));
        return (float)(int)*reinterpret_cast<const int8_t *>(vt + (size_t)j * HD + i) * d;
    } else {  // q4: per position and group 16 bytes, byte l = dims 32c + l (low), 32c + 16 + l (high)
        float d = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(vt + 8 * HD + (j * (HD / 32) + (i >> 5)) * 2));
        uint32_t b = vt[(size_t)j * (HD / 2) + (i >> 5) * 16 + (i & 15)];
        return (float)((int)((b >> (4 * ((i >> 4) & 1))) & 15) - 8) * d;
    }
}

template <int KVT, int HD, int NV>
__global__ void __launch_bounds__(DEC_THREADS) attn_part_kernel(const PassRow *__restrict__ rows, int nrows, int layer, int n_kv,
                                                                int G, const float *__restrict__ q, int qh, int n_heads,
                                                                float scale, float *__restrict__ part, int *err) {
    using C = DecCfg<KVT, HD>;
    constexpr int KF = C::KF, VF = C::VF;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NGRP = (G + NV - 1) / NV, NVT = NGRP * NV;

    uint8_t *buf = smem;
    float *qs = reinterpret_cast<float *>(smem + C::BUF);  // [NGRP][HD][NV]
    float *es = qs + (size_t)NGRP * HD * NV;               // [256][NVT]
    float *red = es + (size_t)ATT_P * NVT;                 // [4][NVT]
    float *ms = red + 4 * NVT, *ls = ms + NVT;             // [NVT] each
    uint64_t *bar = reinterpret_cast<uint64_t *>((reinterpret_cast<uintptr_t>(ls + NVT) + 15) & ~(uintptr_t)15);

    // which (row, block) is this CTA: rows[r].blk0 <= blockIdx.x < rows[r + 1].blk0
    int lo = 0, hi = nrows;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (rows[mid].blk0 <= (int)blockIdx.x) lo = mid; else hi = mid;
    }
    const PassRow row = rows[lo];
    const int b = blockIdx.x - row.blk0, g = blockIdx.y;
    const int n = min(row.np - b * ATT_P, ATT_P);  // positions of this block
    const int ntl = (n + ATT_T - 1) / ATT_T;
    const size_t tile0 = ((size_t)b * n_kv + g) * ATT_PT;
    const uint8_t *kg = row.k + (size_t)layer * row.lk + tile0 * C::KTB;
    const uint8_t *vg = row.v + (size_t)layer * row.lv + tile0 * C::VTB;

    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    uint32_t phase = 0;
    bool ok = true;

    auto issue_k = [&](int stage) {
        int t0 = stage * C::ST_TILES, nt = min(ntl - t0, C::ST_TILES);
        if (nt <= 0) return;
        mbar_expect_tx(bar, (uint32_t)nt * C::KTB);
        for (int u = 0; u < nt; u++) bulk_g2s(buf + (size_t)u * C::KSTRIDE, kg + (size_t)(t0 + u) * C::KTB, C::KTB, bar);
    };
    auto issue_v = [&](int stage) {
        int t0 = stage * C::ST_TILES, nt = min(ntl - t0, C::ST_TILES);
        if (nt <= 0) return;
        mbar_expect_tx(bar, (uint32_t)nt * C::VTB);
        bulk_g2s(buf, vg + (size_t)t0 * C::VTB, (uint32_t)nt * C::VTB, bar);
    };

    if (tid == 0) issue_k(0);

    // ---- the query vectors of this KV head: q[i][v] per group of NV vectors; q8 / q4: rotated first (att_q_rot,
    // reference src/forward.c:1662: signs, butterflies h = 1, 2, 4, ..., then the exact scaling by 1 / head_dim)
    {
        const float *qrow = q + ((size_t)lo * n_heads + (size_t)g * G) * qh;
        if constexpr (kv_quant(KVT)) {
            float *tmp = es;  // [NVT][HD] scratch (the e array is not in use yet; NVT * HD <= 256 * NVT)
            for (int e = tid; e < NVT * HD; e += DEC_THREADS) {
                int v = e / HD, i = e % HD;
                float x = qrow[(size_t)min(v, G - 1) * qh + i];
                tmp[e] = kvq_neg(i) ? -x : x;
            }
            __syncthreads();
            for (int h = 1; h < HD; h <<= 1) {
                for (int e = tid; e < NVT * HD / 2; e += DEC_THREADS) {
                    int v = e / (HD / 2), p = e % (HD / 2);
                    int j = (p / h) * 2 * h + (p % h);
                    float a = tmp[v * HD + j], bb = tmp[v * HD + j + h];
                    tmp[v * HD + j] = a + bb;
                    tmp[v * HD + j + h] = a - bb;
                }
                __syncthreads();
            }
            const float f = 1.0f / (float)HD;
            for (int e = tid; e < NVT * HD; e += DEC_THREADS) {
                int v = e / HD, i = e % HD;
                qs[((size_t)(v / NV) * HD + i) * NV + (v % NV)] = tmp[e] * f;
            }
        } else {
            for (int e = tid; e < NVT * HD; e += DEC_THREADS) {
                int v = e / HD, i = e % HD;
                qs[((size_t)(v / NV) * HD + i) * NV + (v % NV)] = qrow[(size_t)min(v, G - 1) * qh + i];
            }
        }
    }
    __syncthreads();

    // ---- scores: s[t] = (sum over 32-dim chunks, in order, of the fma chain over the chunk's dims) * scale
    for (int stage = 0; stage < C::STAGES; stage++) {
        if (stage * C::ST_POS >= n) break;
        if (stage > 0) {
            __syncthreads();  // everyone is done with the previous stage's tiles
            if (tid == 0) {
                fence_proxy_async();
                issue_k(stage);
            }
        }
        ok = mbar_wait_bounded(bar, phase & 1, err, 1) && ok;
        phase++;
        if constexpr (C::STAGES == 1) {
            const int u = tid >> 3, jp = tid & 7;
            if (u < ntl) {
                const uint8_t *kt = buf + (size_t)u * C::KSTRIDE;
                for (int grp = 0; grp < NGRP; grp++) {
                    const float *qg = qs + (size_t)grp * HD * NV;
                    float a0[NV], a1[NV];
#pragma unroll
                    for (int c = 0; c < HD / ATT_DC; c++) {
                        float c0[NV], c1[NV];
#pragma unroll
                        for (int v = 0; v < NV; v++) c0[v] = c1[v] = 0.0f;
                        float d0 = 0.0f, d1 = 0.0f;
                        if constexpr (KF != KV_F16) {
                            d0 = k_scale<KF, HD>(kt, c, 2 * jp);
                            d1 = k_scale<KF, HD>(kt, c, 2 * jp + 1);
                        }
#pragma unroll 8
                        for (int ii = 0; ii < ATT_DC; ii++) {
                            const int i = c * ATT_DC + ii;
                            float k0, k1;
                            load_k2<KF, HD>(kt, i, jp, d0, d1, k0, k1);
                            float qq[NV];
                            if constexpr (NV == 4) {
                                float4 t4 = *reinterpret_cast<const float4 *>(qg + (size_t)i * 4);
                                qq[0] = t4.x; qq[1] = t4.y; qq[2] = t4.z; qq[3] = t4.w;
                            } else if constexpr (NV == 2) {
                                float2 t2 = *reinterpret_cast<const float2 *>(qg + (size_t)i * 2);
                                qq[0] = t2.x; qq[1] = t2.y;
                            } else {
#pragma unroll
                                for (int v = 0; v < NV; v++) qq[v] = qg[(size_t)i * NV + v];
                            }
#pragma unroll
                            for (int v = 0; v < NV; v++) {
                                c0[v] = fmaf(qq[v], k0, c0[v]);
                                c1[v] = fmaf(qq[v], k1, c1[v]);
                            }
                        }
#pragma unroll
                        for (int v = 0; v < NV; v++) {
                            a0[v] = c ? a0[v] + c0[v] : c0[v];
                            a1[v] = c ? a1[v] + c1[v] : c1[v];
                        }
                    }
                    const int t = u * ATT_T + 2 * jp;
#pragma unroll
                    for (int v = 0; v < NV; v++) {
                        es[(size_t)t * NVT + grp * NV + v] = a0[v] * scale;
                        es[(size_t)(t + 1) * NVT + grp * NV + v] = a1[v] * scale;
                    }
                }
            }
        } else {
            const int u = tid >> 4, j = tid & 15;
            if (stage * C::ST_TILES + u < ntl) {
                const uint8_t *kt = buf + (size_t)u * C::KSTRIDE;
                for (int grp = 0; grp < NGRP; grp++) {
                    const float *qg = qs + (size_t)grp * HD * NV;
                    float a0[NV];
#pragma unroll
                    for (int c = 0; c < HD / ATT_DC; c++) {
                        float c0[NV];
#pragma unroll
                        for (int v = 0; v < NV; v++) c0[v] = 0.0f;
#pragma unroll 8
                        for (int ii = 0; ii < ATT_DC; ii++) {
                            const int i = c * ATT_DC + ii;
                            float k0 = load_k1<KF, HD>(kt, i, j);
#pragma unroll
                            for (int v = 0; v < NV; v++) c0[v] = fmaf(qg[(size_t)i * NV + v], k0, c0[v]);
                        }
#pragma unroll
                        for (int v = 0; v < NV; v++) a0[v] = c ? a0[v] + c0[v] : c0[v];
                    }
                    const int t = stage * C::ST_POS + tid;
#pragma unroll
                    for (int v = 0; v < NV; v++) es[(size_t)t * NVT + grp * NV + v] = a0[v] * scale;
                }
            }
        }
    }
    __syncthreads();  // all scores are in es; the K tiles are free
    if (tid == 0) {
        fence_proxy_async();
        issue_v(0);
    }

    // ---- softmax of the block (while the V tiles arrive): m = max, e = exp_att(s - m), l = 16 lane sums + tree
    for (int v0 = 0; v0 < NVT; v0 += 4) {  // four vectors at a time keep the registers few
        float mx[4];
#pragma unroll
        for (int x = 0; x < 4; x++) mx[x] = -INFINITY;
        for (int t = tid; t < n; t += DEC_THREADS)
#pragma unroll
            for (int x = 0; x < 4; x++)
                if (v0 + x < NVT) mx[x] = fmaxf(mx[x], es[(size_t)t * NVT + v0 + x]);
#pragma unroll
        for (int x = 0; x < 4; x++) {
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) mx[x] = fmaxf(mx[x], __shfl_xor_sync(0xffffffffu, mx[x], o));
            if (lane == 0 && v0 + x < NVT) red[warp * NVT + v0 + x] = mx[x];
        }
    }
    __syncthreads();
    if (tid < NVT) ms[tid] = fmaxf(fmaxf(red[tid], red[NVT + tid]), fmaxf(red[2 * NVT + tid], red[3 * NVT + tid]));
    __syncthreads();
    {
        const int npad = ntl * ATT_T;
        for (int e = tid; e < npad * NVT; e += DEC_THREADS) {
            int t = e / NVT, v = e % NVT;
            es[e] = t < n ? exp_att(es[e] - ms[v]) : 0.0f;
        }
    }
    __syncthreads();
    for (int base = 0; base < NVT * 16; base += DEC_THREADS) {
        // lane j of vector v adds e[t] for t = j, j + 16, ... in order; then the tree (j + 8, + 4, + 2, + 1)
        int idx = base + tid, v = min(idx >> 4, NVT - 1), j = idx & 15;
        float s = 0.0f;
        for (int u = 0; u < ntl; u++) s = s + es[(size_t)(u * ATT_T + j) * NVT + v];
        s = s + __shfl_down_sync(0xffffffffu, s, 8, 16);
        s = s + __shfl_down_sync(0xffffffffu, s, 4, 16);
        s = s + __shfl_down_sync(0xffffffffu, s, 2, 16);
        s = s + __shfl_down_sync(0xffffffffu, s, 1, 16);
        if (j == 0 && idx < NVT * 16) ls[v] = s;
    }

    // ---- outputs: o[i] = fma chain over the block's positions, in order, of e[t] * v[t][i]; then the partial result
    // of (row, head, block): o[hd], m, l
    const int i0 = tid * C::DPT;
    auto pv = [&](auto nvt_c) {
        constexpr int NVTC = decltype(nvt_c)::value;
        float o[C::DPT][NVTC];
#pragma unroll
        for (int d = 0; d < C::DPT; d++)
#pragma unroll
            for (int x = 0; x < NVTC; x++) o[d][x] = 0.0f;
        for (int stage = 0; stage < C::STAGES; stage++) {
            const int p0 = stage * C::ST_POS;
            if (p0 >= n) break;
            if (stage > 0) {
                __syncthreads();
                if (tid == 0) {
                    fence_proxy_async();
                    issue_v(stage);
                }
            }
            ok = mbar_wait_bounded(bar, phase & 1, err, 2) && ok;
            phase++;
            if (stage == 0) __syncthreads();  // (the e values and l of every thread are visible)
            const int cnt = min(n - p0, C::ST_POS);
            if (i0 < HD) {
#pragma unroll 4
                for (int t = 0; t < cnt; t++) {
                    const uint8_t *vt = buf + (size_t)(t >> 4) * C::VTB;
                    float vv[C::DPT];
                    if constexpr (VF == KV_F16 && C::DPT == 2) {
                        __half2 h = *reinterpret_cast<const __half2 *>(vt + ((size_t)(t & 15) * HD + i0) * 2);
                        vv[0] = __low2float(h);
                        vv[1] = __high2float(h);
                    } else {
#pragma unroll
                        for (int d = 0; d < C::DPT; d++) vv[d] = load_v<VF, HD>(vt, t & 15, i0 + d);
                    }
                    const float *et = es + (size_t)(p0 + t) * NVTC;
                    float ee[NVTC];
                    if constexpr (NVTC % 4 == 0) {
#pragma unroll
                        for (int x = 0; x < NVTC / 4; x++) {
                            float4 t4 = *reinterpret_cast<const float4 *>(et + 4 * x);
                            ee[4 * x] = t4.x; ee[4 * x + 1] = t4.y; ee[4 * x + 2] = t4.z; ee[4 * x + 3] = t4.w;
                        }
                    } else {
#pragma unroll
                        for (int x = 0; x < NVTC; x++) ee[x] = et[x];
                    }
#pragma unroll
                    for (int d = 0; d < C::DPT; d++)
#pragma unroll
                        for (int x = 0; x < NVTC; x++) o[d][x] = fmaf(ee[x], vv[d], o[d][x]);
                }
            }
        }
        if (i0 < HD) {
#pragma unroll
            for (int x = 0; x < NVTC; x++) {
                if (x < G) {
                    float *p = part + ((size_t)(row.blk0 + b) * n_heads + (size_t)g * G + x) * RQ_PSTRIDE(HD);
#pragma unroll
                    for (int d = 0; d < C::DPT; d++) p[i0 + d] = ok ? o[d][x] : 0.0f;
                    if (tid == 0) {
                        p[HD] = ms[x];
                        p[HD + 1] = ls[x];
                    }
                }
            }
        }
    };
    switch (NVT) {
        case 1: pv(std::integral_constant<int, 1>{}); break;
        case 2: pv(std::integral_constant<int, 2>{}); break;
        case 3: pv(std::integral_constant<int, 3>{}); break;
        case 4: pv(std::integral_constant<int, 4>{}); break;
        case 8: pv(std::integral_constant<int, 8>{}); break;
        case 12: pv(std::integral_constant<int, 12>{}); break;
        default: pv(std::integral_constant<int, 16>{}); break;
    }
}

// Merge of the block partials of one query vector (att_combine, reference src/forward.c:1405), then the inverse rotation
// for q8 / q4 caches (att_o_unrot :1672: butterflies, signs, exact scaling) and the optional sigmoid gate (attn_gate
// :2291).  One CTA of HD threads per (row, query head).
template <int HD, bool QUANT>
__global__ void __launch_bounds__(HD) attn_combine_kernel(const PassRow *__restrict__ rows, int n_heads, const float *__restrict__ part,
                                                          const float *__restrict__ q, int qh, int gated, float *__restrict__ out) {
    const int r = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
    const PassRow row = rows[r];
    const int nb = (row.np + ATT_P - 1) / ATT_P;
    const size_t pst = RQ_PSTRIDE(HD);
    const float *p0 = part + ((size_t)row.blk0 * n_heads + h) * pst;
    const size_t bstride = (size_t)n_heads * pst;
    float res;
    if (nb == 1) {
        float inv = 1.0f / p0[HD + 1];
        res = p0[i] * inv;
    } else {
        float M = p0[HD];
        for (int b = 1; b < nb; b++) {
            float m = p0[b * bstride + HD];
            if (m > M) M = m;
        }
        float L = 0.0f, acc = 0.0f;
        for (int b = 0; b < nb; b++) {
            const float *p = p0 + b * bstride;
            float c = exp_att(p[HD] - M);
            L = fmaf(c, p[HD + 1], L);
            acc = fmaf(c, p[i], acc);
        }
        float inv = 1.0f / L;
        res = acc * inv;
    }
    if constexpr (QUANT) {
        __shared__ float x[HD];
        x[i] = res;
        __syncthreads();
        for (int hh = 1; hh < HD; hh <<= 1) {
            float a = 0.0f, bb = 0.0f;
            int j = 0;
            if (i < HD / 2) {
                j = (i / hh) * 2 * hh + (i % hh);
                a = x[j];
                bb = x[j + hh];
            }
            __syncthreads();
            if (i < HD / 2) {
                x[j] = a + bb;
                x[j + hh] = a - bb;
            }
            __syncthreads();
        }
        res = kvq_neg(i) ? -x[i] : x[i];
        res = res * (1.0f / (float)HD);
    }
    if (gated) res = res * sigmoid_att(q[((size_t)r * n_heads + h) * qh + HD + i]);
    out[((size_t)r * n_heads + h) * HD + i] = res;
}

}  // namespace rq

namespace rq {

struct AttnPartArgs {
    const PassRow *rows;
    int nrows, total_blocks, layer, n_kv, G;
    const float *q;
    int qh, n_heads;
    float scale;
    float *part;
    int *err;
};

// shared memory one CTA of attn_part_kernel needs, or 0 when the shape is not supported
template <int KVT>
size_t attn_part_smem(int hd, int G);
// launches attn_part_kernel<KVT, hd, ...> on `stream` (grid: total_blocks x n_kv); cudaErrorInvalidValue for an
// unsupported shape
template <int KVT>
cudaError_t launch_attn_part(int hd, const AttnPartArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_DECODE_INSTANTIATE
template <int KVT, int HD, int NV>
static cudaError_t launch_one(const AttnPartArgs &a, cudaStream_t stream) {
    const int ngrp = (a.G + NV - 1) / NV, nvt = ngrp * NV;
    const size_t smem = dec_smem_bytes(DecCfg<KVT, HD>::BUF, HD, nvt);
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = attn_part_kernel<KVT, HD, NV>;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    if (smem > 227 * 1024) return cudaErrorInvalidValue;
    kern<<<dim3(a.total_blocks, a.n_kv), DEC_THREADS, smem, stream>>>(a.rows, a.nrows, a.layer, a.n_kv, a.G, a.q, a.qh, a.n_heads,
                                                                   a.scale, a.part, a.err);
    return cudaGetLastError();
}

template <int KVT, int HD>
static cudaError_t launch_hd(const AttnPartArgs &a, cudaStream_t stream) {
    if (a.G < 1 || a.G > 16) return cudaErrorInvalidValue;
    if (a.G == 1) return launch_one<KVT, HD, 1>(a, stream);
    if (a.G == 2) return launch_one<KVT, HD, 2>(a, stream);
    return launch_one<KVT, HD, 4>(a, stream);
}

template <int KVT>
cudaError_t launch_attn_part(int hd, const AttnPartArgs &a, cudaStream_t stream) {
    if (hd == 64) return launch_hd<KVT, 64>(a, stream);
    if (hd == 128) return launch_hd<KVT, 128>(a, stream);
    if (hd == 256) return launch_hd<KVT, 256>(a, stream);
    return cudaErrorInvalidValue;
}

template <int KVT>
size_t attn_part_smem(int hd, int G) {
    const int nv = G >= 3 ? 4 : G, nvt = (G + nv - 1) / nv * nv;
    const int buf = hd == 64 ? DecCfg<KVT, 64>::BUF : hd == 128 ? DecCfg<KVT, 128>::BUF : hd == 256 ? DecCfg<KVT, 256>::BUF : 0;
    return buf ? dec_smem_bytes(buf, hd, nvt) : 0;
}
#endif

}  // namespace rq
