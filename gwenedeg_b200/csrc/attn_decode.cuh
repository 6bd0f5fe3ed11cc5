// Split-K flash-decode attention over the tiled KV cache (f16 / q8 / q4 / q4k4), sm_100a.
//
// Work decomposition = the reference's: one partial result (o, m, l) per (row, KV head, block of 256 positions)
// (attention_part, reference src/forward.c:1806; definition src/kernels_avx512.h:1109-1126), merged per query vector in
// block order (att_combine, src/forward.c:1405).  The split depends on a row's own length only, so a row of a batch
// gives the bits it gives alone, on any grid.  The arithmetic inside a block also follows the definition operation for
// operation (fp32, fused multiply-add chains over 32-dim chunks for the scores and over the positions for the
// outputs, the 16-lane sum of exponentials and its tree), so results agree with the CPU code to the last bit.
//
// attn_part_kernel: one CTA of 64 threads per (block, KV head).  The K tiles of the block arrive in shared memory
// through bulk async copies (TMA) completing on an mbarrier, half a block (128 positions, 32 KB at head_dim 128, f16)
// at a time; every thread scores two adjacent positions per half for all the query heads of the KV head with packed
// fp32x2 fused multiply-adds (lanes = a pair of query vectors), keeping the scores in registers; the V tiles then
// reuse the same shared-memory buffer while the softmax of the block is computed; every thread accumulates two
// adjacent output dims over the block's positions.  The small buffer lets six CTAs share an SM: the copies of some
// are in flight while the others compute.
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

constexpr int DEC_THREADS = 64;

template <int KVT, int HD>
struct DecCfg {
    static constexpr int KF = kv_fmt(KVT, 0), VF = kv_fmt(KVT, 1);
    static constexpr int KTB = kv_tile_bytes(KVT, HD, 0), VTB = kv_tile_bytes(KVT, HD, 1);
    // positions per stage: 16-bit and all-8-bit caches at head_dim >= 128 are streamed in two halves of 128 positions
    // (smaller buffer, more CTAs per SM); with 4-bit levels the whole block at once measured faster
    static constexpr int STAGES = ((KF == KV_F16 || VF == KV_Q8) && HD >= 128) ? 2 : 1;
    static constexpr int ST_TILES = ATT_PT / STAGES;
    static constexpr int ST_POS = ATT_P / STAGES;
    static constexpr int PPT = ST_POS / DEC_THREADS;  // adjacent positions a thread scores per stage: 4 or 2
    // bytes the 16 positions of one dim (pair) occupy in a K tile: the padding that spreads the tiles a warp reads
    // at once over different shared-memory banks
    static constexpr int KPAD = KF == KV_F16 ? 32 : 16;
    static constexpr int KSTRIDE = KTB + KPAD;
    static constexpr int KBUF = ST_TILES * KSTRIDE, VBUF = ST_TILES * VTB;
    static constexpr int BUF = (KBUF > VBUF ? KBUF : VBUF);
    static constexpr int DPT = HD / DEC_THREADS;  // adjacent output dims per thread: 1, 2 or 4
};

// shared memory of one CTA: kv buffer | q [HD][NVT], later e [256][NVT] | rotation scratch (q8 / q4) | reductions |
// barrier
__host__ __device__ constexpr size_t dec_smem_bytes(int buf, int hd, int nvt, bool quant) {
    return (size_t)buf + (size_t)ATT_P * nvt * 4 + (quant ? (size_t)nvt * hd * 4 : 0) + (size_t)4 * nvt * 4 + 16 + 32;
}

// int8 level in byte `sel` (0..3) of w_flipped (the packed levels with their sign bits flipped: n + 128 per byte) as an
// exact float, without the slow integer-to-float conversion unit: the byte becomes the low mantissa bits of 2^23
__device__ __forceinline__ float s8_to_f32(uint32_t w_flipped, int sel) {
    // bytes of the result: [3] = 0x4B, [2] = [1] = 0x00 (from the constant), [0] = byte `sel` of the levels
    return __uint_as_float(__byte_perm(w_flipped, 0x4B000000u, 0x7540 | sel)) - 8388736.0f;  // 2^23 + 128
}
// 4-bit level (stored + 8) at bit `sh` of w as an exact float: (nibble - 8)
__device__ __forceinline__ float u4_to_f32(uint32_t w, int sh) {
    return __uint_as_float(((w >> sh) & 15u) | 0x4B000000u) - 8388616.0f;  // 2^23 + 8
}

// dim i of PPT adjacent positions (first one: j0) of a K tile; d: the bf16 scales of those positions for dim i's
// 32-dim chunk (quantised formats: value = level x scale, exact in fp32)
template <int KF, int PPT>
__device__ __forceinline__ void load_k(const uint8_t *kt, int i, int j0, const float *d, float *k) {
    if constexpr (KF == KV_F16) {
        if constexpr (PPT == 4) {
            uint2 w = *reinterpret_cast<const uint2 *>(kt + (size_t)i * 32 + j0 * 2);
            float2 f0 = __half22float2(*reinterpret_cast<__half2 *>(&w.x)), f1 = __half22float2(*reinterpret_cast<__half2 *>(&w.y));
            k[0] = f0.x; k[1] = f0.y; k[2] = f1.x; k[3] = f1.y;
        } else {
            float2 f = __half22float2(*reinterpret_cast<const __half2 *>(kt + (size_t)i * 32 + j0 * 2));
            k[0] = f.x; k[1] = f.y;
        }
    } else {
        uint32_t w;
        if constexpr (KF == KV_Q8) {
            if constexpr (PPT == 4) w = *reinterpret_cast<const uint32_t *>(kt + (size_t)i * 16 + j0);
            else w = *reinterpret_cast<const uint16_t *>(kt + (size_t)i * 16 + j0);
            // (packed fp32x2 subtract and multiply: two levels per instruction, each lane rounded as the scalar form)
            w ^= 0x80808080u;
#pragma unroll
            for (int p = 0; p < PPT; p += 2) {
                float2 f = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | p)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | (p + 1))));
                f = __fmul2_rn(__fadd2_rn(f, make_float2(-8388736.0f, -8388736.0f)), make_float2(d[p], d[p + 1]));
                k[p] = f.x, k[p + 1] = f.y;
            }
        } else {  // q4: byte [dim pair][position], low nibble dim 2p, high nibble dim 2p + 1
            if constexpr (PPT == 4) w = *reinterpret_cast<const uint32_t *>(kt + (size_t)(i >> 1) * 16 + j0);
            else w = *reinterpret_cast<const uint16_t *>(kt + (size_t)(i >> 1) * 16 + j0);
            // the dim's nibble of every position moved to the low half of its byte, then as the q8 path: a level + 8
            // becomes the low mantissa bits of 2^23 and the subtract and multiply run two positions per instruction
            w = (w >> (4 * (i & 1))) & 0x0F0F0F0Fu;
#pragma unroll
            for (int p = 0; p < PPT; p += 2) {
                float2 f = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | p)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540 | (p + 1))));
                f = __fmul2_rn(__fadd2_rn(f, make_float2(-8388616.0f, -8388616.0f)), make_float2(d[p], d[p + 1]));  // 2^23 + 8
                k[p] = f.x, k[p + 1] = f.y;
            }
        }
    }
}

// the bf16 scales of chunk c for PPT adjacent positions (first one: j0) of a quantised K tile
template <int KF, int HD, int PPT>
__device__ __forceinline__ void k_scales(const uint8_t *kt, int c, int j0, float *d) {
    constexpr int off = (KF == KV_Q4 ? 8 : 16) * HD;
    const uint8_t *p = kt + off + (c * 16 + j0) * 2;
    if constexpr (PPT == 4) {
        uint2 w = *reinterpret_cast<const uint2 *>(p);
        d[0] = __uint_as_float(w.x << 16); d[1] = __uint_as_float(w.x & 0xffff0000u);
        d[2] = __uint_as_float(w.y << 16); d[3] = __uint_as_float(w.y & 0xffff0000u);
    } else {
        uint32_t w = *reinterpret_cast<const uint32_t *>(p);
        d[0] = __uint_as_float(w << 16); d[1] = __uint_as_float(w & 0xffff0000u);
    }
}

// dims i0 .. i0 + DPT - 1 of position j of a V tile
template <int VF, int HD, int DPT>
__device__ __forceinline__ void load_v(const uint8_t *vt, int j, int i0, float *vv) {
    if constexpr (VF == KV_F16) {
        const uint8_t *p = vt + ((size_t)j * HD + i0) * 2;
        if constexpr (DPT == 1) {
            vv[0] = __half2float(*reinterpret_cast<const __half *>(p));
        } else if constexpr (DPT == 2) {
            float2 f = __half22float2(*reinterpret_cast<const __half2 *>(p));
            vv[0] = f.x; vv[1] = f.y;
        } else {
            uint2 w = *reinterpret_cast<const uint2 *>(p);
            float2 f0 = __half22float2(*reinterpret_cast<__half2 *>(&w.x)), f1 = __half22float2(*reinterpret_cast<__half2 *>(&w.y));
            vv[0] = f0.x; vv[1] = f0.y; vv[2] = f1.x; vv[3] = f1.y;
        }
    } else if constexpr (VF == KV_Q8) {
        const float d = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(vt + 16 * HD + (j * (HD / 32) + (i0 >> 5)) * 2));
        const int8_t *p = reinterpret_cast<const int8_t *>(vt + (size_t)j * HD + i0);
        if constexpr (DPT == 1) {
            vv[0] = s8_to_f32((uint32_t)(uint8_t)p[0] ^ 0x80u, 0) * d;
        } else if constexpr (DPT == 2) {
            uint32_t w = (uint32_t)*reinterpret_cast<const uint16_t *>(p) ^ 0x8080u;
            float2 f = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)));
            f = __fmul2_rn(__fadd2_rn(f, make_float2(-8388736.0f, -8388736.0f)), make_float2(d, d));
            vv[0] = f.x, vv[1] = f.y;
        } else {
            uint32_t w = *reinterpret_cast<const uint32_t *>(p) ^ 0x80808080u;
#pragma unroll
            for (int x = 0; x < 4; x++) vv[x] = s8_to_f32(w, x) * d;
        }
    } else {  // q4: per position and group 16 bytes, byte l = dims 32c + l (low nibble), 32c + 16 + l (high)
        const float d = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(vt + 8 * HD + (j * (HD / 32) + (i0 >> 5)) * 2));
        const uint8_t *p = vt + (size_t)j * (HD / 2) + (i0 >> 5) * 16 + (i0 & 15);
        const int sh = 4 * ((i0 >> 4) & 1);
        if constexpr (DPT == 2) {  // two adjacent bytes at once, packed subtract and multiply (each lane rounds as the scalar form)
            const uint32_t w = ((uint32_t)*reinterpret_cast<const uint16_t *>(p) >> sh) & 0x0F0Fu;
            float2 f = make_float2(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)), __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)));
            f = __fmul2_rn(__fadd2_rn(f, make_float2(-8388616.0f, -8388616.0f)), make_float2(d, d));
            vv[0] = f.x, vv[1] = f.y;
        } else {
#pragma unroll
            for (int x = 0; x < DPT; x++) vv[x] = u4_to_f32(p[x], sh) * d;
        }
    }
}

// NVT: query vectors a CTA handles (the query heads of one KV head, padded to 1, 2, 4 or 8)
template <int KVT, int HD, int NVT>
__global__ void __launch_bounds__(DEC_THREADS) attn_part_kernel(const PassRow *__restrict__ rows, int nrows, int layer, int n_kv,
                                                                int G, const float *__restrict__ q, int qh, int n_heads,
                                                                float scale, float *__restrict__ part, int *err) {
    using C = DecCfg<KVT, HD>;
    constexpr int KF = C::KF, VF = C::VF, PPT = C::PPT, DPT = C::DPT, NPOS = PPT * C::STAGES;
    constexpr int NV = NVT < 4 ? NVT : 4, NGRP = NVT / NV;
    constexpr bool QUANT = kv_quant(KVT);
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_wait();
    pdl_launch_dependents();

    uint8_t *buf = smem;
    float *qs = reinterpret_cast<float *>(smem + C::BUF);  // q [NGRP][HD][NV] while scoring ...
    float *es = qs;                                        // ... then e [256][NVT]
    float *tmp = qs + (size_t)ATT_P * NVT;                 // [NVT][HD] (q8 / q4 only)
    float *red = tmp + (QUANT ? NVT * HD : 0);               // [2][NVT]
    float *ms = red + 2 * NVT, *ls = ms + NVT;               // [NVT] each
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
    // (debug build) the block lies inside the row and its tiles inside one layer of the cache
    RQ_CHECK(lo >= 0 && lo < nrows && b >= 0 && n >= 1 && g < n_kv && (tile0 + ntl) * C::KTB <= row.lk && (tile0 + ntl) * C::VTB <= row.lv, err, 41);

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

    // ---- the query vectors of this KV head as q[group][dim][vector]; q8 / q4: rotated first (att_q_rot,
    // reference src/forward.c:1662: signs, butterflies h = 1, 2, 4, ..., then the exact scaling by 1 / head_dim)
    {
        const float *qrow = q + ((size_t)lo * n_heads + (size_t)g * G) * qh;
        if constexpr (QUANT) {
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

    // ---- scores of this thread's positions, kept in registers:
    // s[t] = (sum over 32-dim chunks, in order, of the fma chain over the chunk's dims) * scale
    float sc[NVT][NPOS];
    // the thread's positions of a stage: tile u, PPT adjacent positions from j0 on
    const int u = PPT == 4 ? tid >> 2 : tid >> 3, j0 = PPT == 4 ? (tid & 3) * 4 : (tid & 7) * 2;
#pragma unroll
    for (int stage = 0; stage < C::STAGES; stage++) {
        if (stage * C::ST_POS < n) {
            if (stage > 0) {
                __syncthreads();  // everyone is done with the previous stage's tiles
                if (tid == 0) {
                    fence_proxy_async();
                    issue_k(stage);
                }
            }
            ok = mbar_wait_bounded(bar, phase & 1, err, 1) && ok;
            phase++;
        }
        const bool have = stage * C::ST_TILES + u < ntl;  // (tiles past the block's last one are not loaded)
        const uint8_t *kt = buf + (size_t)u * C::KSTRIDE;
#pragma unroll
        for (int grp = 0; grp < NGRP; grp++) {
            // packed fp32x2 fused multiply-adds over vector pairs: lanes (q[2vp], q[2vp + 1]) x (k, k) for each of the
            // thread's positions; a single vector (NV == 1) takes the scalar path.  The loads of step i + PF are issued
            // before the arithmetic of step i (software pipeline: few warps are resident, so the shared-memory latency
            // has to be hidden inside the thread).
            constexpr int NVP = NV / 2, PF = KF == KV_F16 ? 3 : 4;
            const float *qg = qs + (size_t)grp * HD * NV;
            float2 a2[NVP > 0 ? NVP : 1][PPT], c2[NVP > 0 ? NVP : 1][PPT];
            float a1[PPT], c1[PPT];
#pragma unroll
            for (int p = 0; p < PPT; p++) {
                a1[p] = c1[p] = 0.0f;
#pragma unroll
                for (int vp = 0; vp < (NVP > 0 ? NVP : 1); vp++) a2[vp][p] = c2[vp][p] = make_float2(0.0f, 0.0f);
            }
            if (have) {
                float kq[PF][PPT], dsc[PPT];
                float4 qq[PF];
                auto fetch = [&](int i, int slot) {
                    if constexpr (KF != KV_F16) {
                        if ((i & (ATT_DC - 1)) == 0) k_scales<KF, HD, PPT>(kt, i / ATT_DC, j0, dsc);
                    }
                    load_k<KF, PPT>(kt, i, j0, dsc, kq[slot]);
                    if constexpr (NV == 4) qq[slot] = *reinterpret_cast<const float4 *>(qg + (size_t)i * 4);
                    else if constexpr (NV == 2) {
                        float2 t2 = *reinterpret_cast<const float2 *>(qg + (size_t)i * 2);
                        qq[slot] = make_float4(t2.x, t2.y, 0.0f, 0.0f);
                    } else qq[slot] = make_float4(qg[i], 0.0f, 0.0f, 0.0f);
                };
#pragma unroll
                for (int i = 0; i < PF; i++) fetch(i, i);
#pragma unroll(KF == KV_F16 ? HD : ATT_DC)  // (quantised formats: one chunk per trip keeps the code in the instruction cache)
                for (int i = 0; i < HD; i++) {
                    const int slot = i % PF;
                    float kk[PPT];
#pragma unroll
                    for (int p = 0; p < PPT; p++) kk[p] = kq[slot][p];
                    const float4 qv = qq[slot];
                    if (i + PF < HD) fetch(i + PF, slot);
                    if constexpr (NVP > 0) {
                        const float2 qp[2] = {make_float2(qv.x, qv.y), make_float2(qv.z, qv.w)};
#pragma unroll
                        for (int p = 0; p < PPT; p++) {
                            const float2 kd = make_float2(kk[p], kk[p]);
#pragma unroll
                            for (int vp = 0; vp < NVP; vp++) c2[vp][p] = __ffma2_rn(qp[vp], kd, c2[vp][p]);  // fma(q, k, c) per lane
                        }
                    } else {
#pragma unroll
                        for (int p = 0; p < PPT; p++) c1[p] = fmaf(qv.x, kk[p], c1[p]);
                    }
                    if ((i & (ATT_DC - 1)) == ATT_DC - 1) {  // end of a 32-dim chunk: chunk 0 is assigned, later ones added
#pragma unroll
                        for (int p = 0; p < PPT; p++) {
                            if constexpr (NVP > 0) {
#pragma unroll
                                for (int vp = 0; vp < NVP; vp++) {
                                    a2[vp][p] = i >= ATT_DC ? __fadd2_rn(a2[vp][p], c2[vp][p]) : c2[vp][p];
                                    c2[vp][p] = make_float2(0.0f, 0.0f);
                                }
                            } else {
                                a1[p] = i >= ATT_DC ? a1[p] + c1[p] : c1[p];
                                c1[p] = 0.0f;
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int p = 0; p < PPT; p++) {
                if constexpr (NVP > 0) {
#pragma unroll
                    for (int vp = 0; vp < NVP; vp++) {
                        sc[grp * NV + 2 * vp][stage * PPT + p] = a2[vp][p].x * scale;
                        sc[grp * NV + 2 * vp + 1][stage * PPT + p] = a2[vp][p].y * scale;
                    }
                } else {
                    sc[grp * NV][stage * PPT + p] = a1[p] * scale;
                }
            }
        }
    }

    // ---- softmax of the block: m = max over the block's positions, e = exp_att(s - m), l = 16 lane sums + tree
    // position of register slot x of this thread
    auto slot_pos = [&](int x) { return (x / PPT) * C::ST_POS + u * ATT_T + j0 + (x % PPT); };
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        float mx = -INFINITY;
#pragma unroll
        for (int x = 0; x < NPOS; x++)
            if (slot_pos(x) < n) mx = fmaxf(mx, sc[v][x]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red[warp * NVT + v] = mx;
    }
    __syncthreads();  // (also: every thread is done with the K tiles and the staged q)
    if (tid == 0) {
        fence_proxy_async();
        issue_v(0);
    }
    if (tid < NVT) ms[tid] = fmaxf(red[tid], red[NVT + tid]);
#pragma unroll
    for (int x = 0; x < NPOS; x++) {
        const int t = slot_pos(x);
        if (t < ntl * ATT_T) {
#pragma unroll
            for (int v = 0; v < NVT; v++) {
                const float m = fmaxf(red[v], red[NVT + v]);
                es[(size_t)t * NVT + v] = t < n ? exp_att(sc[v][x] - m) : 0.0f;
            }
        }
    }
    __syncthreads();
    for (int base = 0; base < NVT * 16; base += DEC_THREADS) {
        // lane j of vector v adds e[t] for t = j, j + 16, ... in order; then the tree (j + 8, + 4, + 2, + 1)
        int idx = base + tid, v = min(idx >> 4, NVT - 1), j = idx & 15;
        float s = 0.0f;
        for (int uu = 0; uu < ntl; uu++) s = s + es[(size_t)(uu * ATT_T + j) * NVT + v];
        s = s + __shfl_down_sync(0xffffffffu, s, 8, 16);
        s = s + __shfl_down_sync(0xffffffffu, s, 4, 16);
        s = s + __shfl_down_sync(0xffffffffu, s, 2, 16);
        s = s + __shfl_down_sync(0xffffffffu, s, 1, 16);
        if (j == 0 && idx < NVT * 16) ls[v] = s;
    }

    // ---- outputs: o[i] = fma chain over the block's positions, in order, of e[t] * v[t][i], for this thread's
    // DPT adjacent dims and all vectors
    const int i0 = tid * DPT;
    constexpr int NVPT = NVT / 2;
    float2 o2[DPT][NVPT > 0 ? NVPT : 1];  // lanes: vectors (2vp, 2vp + 1)
    float o1[DPT];                        // a single vector (NVT == 1)
#pragma unroll
    for (int d = 0; d < DPT; d++) {
        o1[d] = 0.0f;
#pragma unroll
        for (int vp = 0; vp < (NVPT > 0 ? NVPT : 1); vp++) o2[d][vp] = make_float2(0.0f, 0.0f);
    }
    // one position: e[t][.] x (v, v) per dim, accumulated per vector pair
    auto accum = [&](const float *vv, const float2 *ee) {
        if constexpr (NVPT > 0) {
#pragma unroll
            for (int d = 0; d < DPT; d++) {
                const float2 vd = make_float2(vv[d], vv[d]);
#pragma unroll
                for (int vp = 0; vp < NVPT; vp++) o2[d][vp] = __ffma2_rn(ee[vp], vd, o2[d][vp]);  // fma(e, v, o) per lane
            }
        } else {
#pragma unroll
            for (int d = 0; d < DPT; d++) o1[d] = fmaf(ee[0].x, vv[d], o1[d]);
        }
    };
    auto fetch_e = [&](const float *et, float2 *ee) {
        if constexpr (NVT % 4 == 0) {
#pragma unroll
            for (int x = 0; x < NVT / 4; x++) {
                float4 t4 = *reinterpret_cast<const float4 *>(et + 4 * x);
                ee[2 * x] = make_float2(t4.x, t4.y);
                ee[2 * x + 1] = make_float2(t4.z, t4.w);
            }
        } else if constexpr (NVT == 2) {
            ee[0] = *reinterpret_cast<const float2 *>(et);
        } else {
            ee[0] = make_float2(et[0], 0.0f);
        }
    };
#pragma unroll
    for (int stage = 0; stage < C::STAGES; stage++) {
        const int p0 = stage * C::ST_POS;
        if (p0 < n) {
            if (stage > 0) {
                __syncthreads();
                if (tid == 0) {
                    fence_proxy_async();
                    issue_v(stage);
                }
            }
            ok = mbar_wait_bounded(bar, phase & 1, err, 2) && ok;
            phase++;
            const int cnt = min(n - p0, C::ST_POS), full = cnt >> 4;
            const uint8_t *vt = buf;
            const float *et = es + (size_t)p0 * NVT;
            for (int uu = 0; uu < full; uu++, vt += C::VTB, et += ATT_T * NVT) {
                // a whole tile with constant offsets, its loads running PF positions ahead of the arithmetic
                constexpr int PF = 3;
                float vv[PF][DPT];
                float2 ee[PF][NVPT > 0 ? NVPT : 1];
#pragma unroll
                for (int j = 0; j < PF; j++) {
                    load_v<VF, HD, DPT>(vt, j, i0, vv[j]);
                    fetch_e(et + j * NVT, ee[j]);
                }
#pragma unroll
                for (int j = 0; j < ATT_T; j++) {
                    const int slot = j % PF;
                    float vc[DPT];
                    float2 ec[NVPT > 0 ? NVPT : 1];
#pragma unroll
                    for (int d = 0; d < DPT; d++) vc[d] = vv[slot][d];
#pragma unroll
                    for (int vp = 0; vp < (NVPT > 0 ? NVPT : 1); vp++) ec[vp] = ee[slot][vp];
                    if (j + PF < ATT_T) {
                        load_v<VF, HD, DPT>(vt, j + PF, i0, vv[slot]);
                        fetch_e(et + (j + PF) * NVT, ee[slot]);
                    }
                    accum(vc, ec);
                }
            }
            for (int j = 0; j < (cnt & 15); j++) {
                float vc[DPT];
                float2 ec[NVPT > 0 ? NVPT : 1];
                load_v<VF, HD, DPT>(vt, j, i0, vc);
                fetch_e(et + j * NVT, ec);
                accum(vc, ec);
            }
        }
    }

    // ---- the partial result of (row, head, block): o[hd], m, l
    // ls[v] was written by lane 16 (v % 4) of warp v / 2 and is read by thread 0 below: the only barriers since are the
    // conditional ones between V stages (none when the block has a single stage), so one more is needed here
    __syncthreads();
#pragma unroll
    for (int v = 0; v < NVT; v++) {
        if (v < G) {
            float *p = part + ((size_t)(row.blk0 + b) * n_heads + (size_t)g * G + v) * RQ_PSTRIDE(HD);
#pragma unroll
            for (int d = 0; d < DPT; d++) {
                float val;
                if constexpr (NVPT > 0) val = (v & 1) ? o2[d][v >> 1].y : o2[d][v >> 1].x;
                else val = o1[d];
                p[i0 + d] = ok ? val : 0.0f;
            }
            if (tid == 0) {
                p[HD] = ms[v];
                p[HD + 1] = ls[v];
            }
        }
    }
}

// Merge of the block partials of one query vector (att_combine, reference src/forward.c:1405), then the inverse rotation
// for q8 / q4 caches (att_o_unrot :1672: butterflies, signs, exact scaling) and the optional sigmoid gate (attn_gate
// :2291).  One CTA of HD threads per (row, query head).
// split_len / fixed_stride: the partials of a row are one per `split_len` positions, the first one at record index
// row.blk0 (fixed_stride 0: the decode kernel's 256-position blocks) or r * fixed_stride (the prefill kernel's splits).
// The activation quantiser the reference runs on the attention's outputs right before the `wo` matmul (quantize,
// reference src/forward.c:803; call site :2716-2719), operation for operation: per group of gs values scale = wmax * (1 / 127),
// inv = 127 / wmax, level = (int) trunc(x inv + copysign(0.49999997, x inv)); an all-zero group gives zero levels.
__device__ __forceinline__ int8_t wo_quant_level(float x, float wmax) {
    if (!(wmax > 0.0f)) return 0;
    const float v = x * (127.0f / wmax);
    return (int8_t)__float2int_rz(v + copysignf(0.49999997f, v));
}
// where the merge kernels leave the quantised copy of their output rows: levels [rows][n_heads * head_dim] and one scale per
// gs values (gs: 32, 64, 128 or 256, dividing head_dim); xq null: none
struct WoQuant {
    int8_t *xq;
    float *xs;
    int gs;
};

// Head-sharded contexts (one GPU per group of KV heads): where the merge kernel stores its output rows when the gather over the
// ranks is fused into it: the full-width row buffers [rows][n_heads_full][head_dim] of every rank (this rank's own among them;
// the others are peer mappings over NVLink), this rank's heads starting at head0.  world 0: the plain local store.
constexpr int RQ_MAX_PEERS = 8;
struct PeerOut {
    float *out[RQ_MAX_PEERS];
    int world, n_heads_full, head0;
};

constexpr int COMBINE_NG = 4;  // thread groups of the merge kernel: each fetches a quarter of the partials

// One CTA of COMBINE_NG x HD threads per (row, query head).  The partial results are fetched into shared memory by all
// the threads at once (group g takes the partials b = g mod COMBINE_NG: many loads in flight, the kernel is bound by
// their latency), then the first HD threads run the two fma chains over them in partial order.
template <int HD, bool QUANT>
__global__ void __launch_bounds__(COMBINE_NG *HD) attn_combine_kernel(const PassRow *__restrict__ rows, int n_heads,
                                                                      const float *__restrict__ part, const float *__restrict__ q, int qh,
                                                                      int gated, float *__restrict__ out, int split_len, int fixed_stride,
                                                                      const int *err_src, int *err_dst, WoQuant wq, PeerOut po) {
    constexpr int CH = 8192 / HD;  // partials per chunk: 32 KB of shared memory
    const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, i = tid % HD, grp = tid / HD;
    pdl_wait();
    pdl_launch_dependents();
    // err_dst (a mapped host word, or null): the status word of the kernels before this one, complete after the wait
    // above, goes to the host with the results instead of by a copy of its own
    if (err_dst && r == 0 && h == 0 && tid == 0) *err_dst = *err_src;
    const PassRow row = rows[r];
    const int nb = (row.np + split_len - 1) / split_len;
    RQ_CHECK(nb >= 1 && h < n_heads, const_cast<int *>(err_src), 42);
    const size_t pst = RQ_PSTRIDE(HD);
    const size_t bstride = (size_t)n_heads * pst;
    const float *p0 = part + ((size_t)(fixed_stride ? r * fixed_stride : row.blk0) * n_heads + h) * pst;
    __shared__ float tile[CH][HD];
    __shared__ float cs[CH], ls[CH], red[COMBINE_NG * HD / 32];
    __shared__ float x[QUANT ? HD : 1];
    float res = 0.0f;
    if (nb == 1) {
        if (grp == 0) {
            float inv = 1.0f / p0[HD + 1];
            res = p0[i] * inv;
        }
    } else {
        // M = max of the m_b (any order gives the same maximum)
        float M = -INFINITY;
        for (int b = tid; b < nb; b += COMBINE_NG * HD) M = fmaxf(M, p0[b * bstride + HD]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        if ((tid & 31) == 0) red[tid >> 5] = M;
        __syncthreads();
        M = red[0];
#pragma unroll
        for (int wv = 1; wv < COMBINE_NG * HD / 32; wv++) M = fmaxf(M, red[wv]);
        float L = 0.0f, acc = 0.0f;
        for (int b0 = 0; b0 < nb; b0 += CH) {
            const int cnt = min(CH, nb - b0);
            __syncthreads();  // (the previous chunk has been consumed)
            const float *pc = p0 + (size_t)b0 * bstride;
#pragma unroll 8
            for (int b = grp; b < cnt; b += COMBINE_NG) tile[b][i] = pc[(size_t)b * bstride + i];
            if (tid < cnt) {
                cs[tid] = exp_att(pc[(size_t)tid * bstride + HD] - M);  // c_b = exp_att(m_b - M)
                ls[tid] = pc[(size_t)tid * bstride + HD + 1];
            }
            __syncthreads();
            if (grp == 0) {
                // L = fma chain over the l_b, out[i] = fma chain over the o_b[i], both in partial order
#pragma unroll 8
                for (int b = 0; b < cnt; b++) {
                    L = fmaf(cs[b], ls[b], L);
                    acc = fmaf(cs[b], tile[b][i], acc);
                }
            }
        }
        float inv = 1.0f / L;
        res = acc * inv;
    }
    if constexpr (QUANT) {
        if (grp == 0) x[i] = res;
        __syncthreads();
        for (int hs = 1; hs < HD; hs <<= 1) {
            float a = 0.0f, bb = 0.0f;
            int j = 0;
            if (tid < HD / 2) {
                j = (tid / hs) * 2 * hs + (tid % hs);
                a = x[j];
                bb = x[j + hs];
            }
            __syncthreads();
            if (tid < HD / 2) {
                x[j] = a + bb;
                x[j + hs] = a - bb;
            }
            __syncthreads();
        }
        res = kvq_neg(i) ? -x[i] : x[i];
        res = res * (1.0f / (float)HD);
    }
    if (grp == 0) {
        if (gated) res = res * sigmoid_att(q[((size_t)r * n_heads + h) * qh + HD + i]);
        if (po.world > 0) {  // the gather over the ranks, fused: this rank's heads of the row into every rank's full-width buffer
            const size_t at = ((size_t)r * po.n_heads_full + po.head0 + h) * HD + i;
#pragma unroll
            for (int p = 0; p < RQ_MAX_PEERS; p++)
                if (p < po.world) po.out[p][at] = res;
        } else {
            out[((size_t)r * n_heads + h) * HD + i] = res;
        }
    }
    if (wq.xq) {  // (uniform over the CTA) the quantised copy for the `wo` matmul
        __shared__ float wmaxs[HD / 32];
        float a = grp == 0 ? fabsf(res) : 0.0f;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        if (grp == 0 && (tid & 31) == 0) wmaxs[tid >> 5] = a;
        __syncthreads();
        if (grp == 0) {
            const int nw = wq.gs >> 5, w0 = (i / wq.gs) * nw;
            float wmax = wmaxs[w0];
            for (int x2 = 1; x2 < nw; x2++) wmax = fmaxf(wmax, wmaxs[w0 + x2]);
            const size_t at = ((size_t)r * n_heads + h) * HD + i;
            if (i % wq.gs == 0) wq.xs[at / wq.gs] = wmax * (1.0f / 127.0f);
            wq.xq[at] = wo_quant_level(res, wmax);
        }
    }
}

// The same merge for rows with few partials each (the tensor-core prefill path: head_dim 128 or 256, 16-bit cache, one
// partial per split of PF_SPLIT = 2,048 positions): one warp per (row, query head), lane L holds dims 4L .. 4L + 3 of every
// 128-dim part of the row, so a launch is a few hundred CTAs instead of one per output row.  Arithmetic as
// attn_combine_kernel: M = max of the m_b, c_b = exp_att(m_b - M), L and out as fma chains in partial order, out * (1 / L), gate.
// With `unrot` (quantised caches) the merged row is un-rotated before the gate as attn_combine_kernel does it.
constexpr int COMBINE_ROWS_WARPS = 8;
// the 128-point butterflies (h = 1, 2, 4, ..., 64) of att_q_rot / att_o_unrot over a warp: lane L holds dims 4L .. 4L + 3
__device__ __forceinline__ void fwht128_warp(float4 &x, int lane) {
    {  // h = 1, 2: inside the lane
        const float a = x.x + x.y, b = x.x - x.y, c = x.z + x.w, d = x.z - x.w;
        x = make_float4(a + c, b + d, a - c, b - d);
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {  // h = 4 o: lanes L and L ^ o
        const float4 y = make_float4(__shfl_xor_sync(0xffffffffu, x.x, o), __shfl_xor_sync(0xffffffffu, x.y, o), __shfl_xor_sync(0xffffffffu, x.z, o),
                                     __shfl_xor_sync(0xffffffffu, x.w, o));
        x = (lane & o) ? make_float4(y.x - x.x, y.y - x.y, y.z - x.z, y.w - x.w) : make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
}
// ... of 128 NP points (NP = 1 or 2): the 128-point butterflies on each part, then h = 128 between the parts
template <int NP>
__device__ __forceinline__ void fwht_warp(float4 *x, int lane) {
#pragma unroll
    for (int c = 0; c < NP; c++) fwht128_warp(x[c], lane);
    if constexpr (NP == 2) {
        const float4 a = x[0], b = x[1];
        x[0] = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        x[1] = make_float4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w);
    }
}
template <int HD>
__global__ void __launch_bounds__(32 * COMBINE_ROWS_WARPS) attn_combine_rows_kernel(const PassRow *__restrict__ rows, int nrows, int n_heads,
                                                                                 const float *__restrict__ part, const float *__restrict__ q,
                                                                                 int qh, int gated, float *__restrict__ out, int split_len,
                                                                                 int fixed_stride, const int *err_src, int *err_dst, WoQuant wq, int unrot) {
    static_assert(HD % 128 == 0, "a lane holds 4 dims of every 128 of the row");
    constexpr int NP = HD / 128;
    const int wi = blockIdx.x * COMBINE_ROWS_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch_dependents();
    if (err_dst && blockIdx.x == 0 && threadIdx.x == 0) *err_dst = *err_src;  // (as in attn_combine_kernel)
    if (wi >= nrows * n_heads) return;
    const int r = wi / n_heads, h = wi % n_heads;
    const int nb = (rows[r].np + split_len - 1) / split_len;
    const size_t pst = RQ_PSTRIDE(HD), bstride = (size_t)n_heads * pst;
    const float *p0 = part + ((size_t)r * fixed_stride * n_heads + h) * pst;
    float4 res[NP];
    if (nb == 1) {
        const float inv = 1.0f / p0[HD + 1];
#pragma unroll
        for (int c = 0; c < NP; c++) {
            const float4 o = *reinterpret_cast<const float4 *>(p0 + 128 * c + 4 * lane);
            res[c] = make_float4(o.x * inv, o.y * inv, o.z * inv, o.w * inv);
        }
    } else {
        float M = -INFINITY;
        for (int b = 0; b < nb; b++) M = fmaxf(M, p0[b * bstride + HD]);
        float L = 0.0f;
        float4 acc[NP];
#pragma unroll
        for (int c = 0; c < NP; c++) acc[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 4
        for (int b = 0; b < nb; b++) {
            const float *pb = p0 + b * bstride;
            const float cb = exp_att(pb[HD] - M);
            L = fmaf(cb, pb[HD + 1], L);
#pragma unroll
            for (int c = 0; c < NP; c++) {
                const float4 o = *reinterpret_cast<const float4 *>(pb + 128 * c + 4 * lane);
                acc[c].x = fmaf(cb, o.x, acc[c].x), acc[c].y = fmaf(cb, o.y, acc[c].y), acc[c].z = fmaf(cb, o.z, acc[c].z), acc[c].w = fmaf(cb, o.w, acc[c].w);
            }
        }
        const float inv = 1.0f / L;
#pragma unroll
        for (int c = 0; c < NP; c++) res[c] = make_float4(acc[c].x * inv, acc[c].y * inv, acc[c].z * inv, acc[c].w * inv);
    }
    if (unrot) {  // att_o_unrot: butterflies, signs, scaling by 1 / head_dim
        fwht_warp<NP>(res, lane);
        const float f = 1.0f / (float)HD;
#pragma unroll
        for (int c = 0; c < NP; c++) {
            const int i = 128 * c + 4 * lane;
            res[c].x = (kvq_neg(i) ? -res[c].x : res[c].x) * f, res[c].y = (kvq_neg(i + 1) ? -res[c].y : res[c].y) * f;
            res[c].z = (kvq_neg(i + 2) ? -res[c].z : res[c].z) * f, res[c].w = (kvq_neg(i + 3) ? -res[c].w : res[c].w) * f;
        }
    }
#pragma unroll
    for (int c = 0; c < NP; c++) {
        if (gated) {
            const float4 gq = *reinterpret_cast<const float4 *>(q + ((size_t)r * n_heads + h) * qh + HD + 128 * c + 4 * lane);
            res[c].x = res[c].x * sigmoid_att(gq.x), res[c].y = res[c].y * sigmoid_att(gq.y), res[c].z = res[c].z * sigmoid_att(gq.z),
            res[c].w = res[c].w * sigmoid_att(gq.w);
        }
        *reinterpret_cast<float4 *>(out + ((size_t)r * n_heads + h) * HD + 128 * c + 4 * lane) = res[c];
    }
    if (wq.xq) {  // the quantised copy for the `wo` matmul: a group of gs dims is gs / 4 adjacent lanes of one 128-dim part
        float wm[NP];
#pragma unroll
        for (int c = 0; c < NP; c++) {
            float a = fmaxf(fmaxf(fabsf(res[c].x), fabsf(res[c].y)), fmaxf(fabsf(res[c].z), fabsf(res[c].w)));
            const int span = (wq.gs < 128 ? wq.gs : 128) >> 2;
            for (int o = 1; o < span; o <<= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
            wm[c] = a;
        }
        if (wq.gs > 128)  // (head_dim 256 with one group per head)
#pragma unroll
            for (int c = 1; c < NP; c++) wm[0] = wm[c] = fmaxf(wm[0], wm[c]);
#pragma unroll
        for (int c = 0; c < NP; c++) {
            const size_t at = ((size_t)r * n_heads + h) * HD + 128 * c + 4 * lane;
            if ((128 * c + 4 * lane) % wq.gs == 0) wq.xs[at / wq.gs] = wm[c] * (1.0f / 127.0f);
            char4 lv;
            lv.x = wo_quant_level(res[c].x, wm[c]), lv.y = wo_quant_level(res[c].y, wm[c]), lv.z = wo_quant_level(res[c].z, wm[c]), lv.w = wo_quant_level(res[c].w, wm[c]);
            *reinterpret_cast<char4 *>(wq.xq + at) = lv;
        }
    }
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
template <int KVT, int HD, int NVT>
static cudaError_t launch_one(const AttnPartArgs &a, cudaStream_t stream) {
    constexpr size_t smem = dec_smem_bytes(DecCfg<KVT, HD>::BUF, HD, NVT, kv_quant(KVT));
    static_assert(smem <= 227 * 1024, "one CTA's shared memory");
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = attn_part_kernel<KVT, HD, NVT>;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    return launch_pdl(kern, dim3(a.total_blocks, a.n_kv), dim3(DEC_THREADS), smem, stream, a.rows, a.nrows, a.layer, a.n_kv, a.G, a.q, a.qh, a.n_heads,
                      a.scale, a.part, a.err);
}

template <int KVT, int HD>
static cudaError_t launch_hd(const AttnPartArgs &a, cudaStream_t stream) {
    if (a.G < 1 || a.G > 8) return cudaErrorInvalidValue;
    if (a.G == 1) return launch_one<KVT, HD, 1>(a, stream);
    if (a.G == 2) return launch_one<KVT, HD, 2>(a, stream);
    if (a.G <= 4) return launch_one<KVT, HD, 4>(a, stream);
    return launch_one<KVT, HD, 8>(a, stream);
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
    const int nvt = G == 1 ? 1 : G == 2 ? 2 : G <= 4 ? 4 : 8;
    const int buf = hd == 64 ? DecCfg<KVT, 64>::BUF : hd == 128 ? DecCfg<KVT, 128>::BUF : hd == 256 ? DecCfg<KVT, 256>::BUF : 0;
    return buf ? dec_smem_bytes(buf, hd, nvt, kv_quant(KVT)) : 0;
}
#endif

}  // namespace rq
