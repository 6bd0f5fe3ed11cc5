// Gated DeltaNet recurrence, exact token-by-token form (dn_rec_run, reference src/forward.c:2224; passes dn_p1 / dn_p2
// :2177-2203).
//
// Per value head h (key head h % nk) and value column v, tokens in order, S is [dk][dv]:
//     u    = sum over k, in order, of fma(S[k][v] * eg, key[k], .)         (from 0)
//     u    = (val[v] - u) * beta
//     S[k][v] = fma(key[k], u, S[k][v] * eg)
//     o[v] = sum over k, in order, of fma(S[k][v], query[k], .)            (on the updated S, from 0)
// Each column is independent of the others, which is how the work is cut: one warp per (segment, value head, block of
// 32 columns), each lane keeping its column of S (dk floats) in registers for the whole run of rows; the key / query /
// value rows and gates of the next few tokens are prefetched into a shared-memory ring with cp.async and broadcast.  The u-chain of token t + 1 is interleaved with the
// o-chain of token t, as the reference's fused pass does, which doubles the independent work per lane without
// changing a bit.  Results equal the CPU code's bit for bit.
//
// State layout per linear layer (src/forward.c:125, :2090): conv inputs first, then per value head dv / 32 blocks of
// [dk][32] floats.
#pragma once
#include "attn_decode.cuh"

namespace rq {

constexpr int DN_BW = 32;

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int DN_STAGES = 8;  // tokens in flight in a warp's shared-memory ring

template <int DK>
__global__ void __launch_bounds__(32) dn_rec_kernel(const DnSeg *__restrict__ segs, int lin_layer, int nk, int nv, int dv,
                                                    size_t conv_floats, const float *__restrict__ rows, int lw,
                                                    float *__restrict__ out, const DnCk *__restrict__ cks) {
    const int nblk = dv / DN_BW;
    const int jb = blockIdx.x % nblk, h = blockIdx.x / nblk, lane = threadIdx.x;
    const DnSeg sg = segs[blockIdx.y];
    const int conv_dim = 2 * nk * DK + nv * dv, vdim = nv * dv;
    const size_t oq = (size_t)(h % nk) * DK, ok = (size_t)nk * DK + oq;
    const size_t ov = (size_t)2 * nk * DK + (size_t)h * dv + (size_t)jb * DN_BW;
    const size_t oe = (size_t)conv_dim + vdim + h, ob = oe + nv;
    float *Sg = sg.state + (size_t)lin_layer * sg.lstride + conv_floats + (size_t)h * DK * dv + (size_t)jb * DK * DN_BW + lane;

    // ring of DN_STAGES tokens: key [DK] | query [DK] | values of the 32 columns | exp(g), beta — filled by cp.async a few
    // tokens ahead, so the recurrence never waits for global memory
    struct Stage { float key[DK], qry[DK], val[DN_BW], eg, beta, pad[2]; };
    __shared__ __align__(16) Stage ring[DN_STAGES];
    auto fetch = [&](int t) {
        if (t < sg.n) {
            const float *r = rows + (size_t)(sg.row0 + t) * lw;
            Stage &st = ring[t % DN_STAGES];
#pragma unroll
            for (int x = 0; x < DK / 128; x++) {
                cp_async16(&st.key[x * 128 + lane * 4], r + ok + x * 128 + lane * 4);
                cp_async16(&st.qry[x * 128 + lane * 4], r + oq + x * 128 + lane * 4);
            }
            if (lane < DN_BW / 4) cp_async16(&st.val[lane * 4], r + ov + lane * 4);
            if (lane == 8) cp_async4(&st.eg, r + oe);
            if (lane == 9) cp_async4(&st.beta, r + ob);
        }
        cp_async_commit();  // (an empty group past the end keeps the group count uniform)
    };
#pragma unroll
    for (int t = 0; t < DN_STAGES - 1; t++) fetch(t);

    float S[DK];
#pragma unroll
    for (int k = 0; k < DK; k++) S[k] = sg.first ? 0.0f : Sg[(size_t)k * DN_BW];

    cp_async_wait<DN_STAGES - 2>();  // token 0 has landed
    __syncwarp();
    float eg = ring[0].eg;
    float u = 0.0f;
    int ci = 0;  // checkpoints of the segment taken so far
#pragma unroll
    for (int k = 0; k < DK; k++) u = fmaf(S[k] * eg, ring[0].key[k], u);

    for (int t = 0; t < sg.n; t++) {
        fetch(t + DN_STAGES - 1);          // (its slot held token t - 1: every lane is past it)
        cp_async_wait<DN_STAGES - 2>();    // tokens <= t + 1 have landed
        __syncwarp();
        const Stage &cur = ring[t % DN_STAGES], &nxt = ring[(t + 1) % DN_STAGES];
        u = (cur.val[lane] - u) * cur.beta;
        float o = 0.0f, un = 0.0f;
        // (key / query values are read four at a time: one 16-byte broadcast load serves four steps of the chains)
        const float4 *ck4 = reinterpret_cast<const float4 *>(cur.key), *cq4 = reinterpret_cast<const float4 *>(cur.qry);
        const float4 *nk4 = reinterpret_cast<const float4 *>(nxt.key);
        if (t + 1 < sg.n) {
            const float egn = nxt.eg;
#pragma unroll
            for (int k4 = 0; k4 < DK / 4; k4++) {
                const float4 kk = ck4[k4], qq = cq4[k4], kn = nk4[k4];
                const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w}, nv4[4] = {kn.x, kn.y, kn.z, kn.w};
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int k = 4 * k4 + x;
                    float sv = fmaf(kv[x], u, S[k] * eg);
                    S[k] = sv;
                    o = fmaf(sv, qv[x], o);
                    un = fmaf(sv * egn, nv4[x], un);
                }
            }
            eg = egn;
        } else {
#pragma unroll
            for (int k4 = 0; k4 < DK / 4; k4++) {
                const float4 kk = ck4[k4], qq = cq4[k4];
                const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int k = 4 * k4 + x;
                    float sv = fmaf(kv[x], u, S[k] * eg);
                    S[k] = sv;
                    o = fmaf(sv, qv[x], o);
                }
            }
        }
        out[(size_t)(sg.row0 + t) * vdim + (size_t)h * dv + (size_t)jb * DN_BW + lane] = o;
        u = un;
        if (ci < sg.nck && t == cks[sg.ck0 + ci].row) {
            // a checkpoint after this token: the warp's block of S as it stands (dn_rec_run, reference src/forward.c:2267-2270)
            float *d = cks[sg.ck0 + ci].dst + (Sg - sg.state);
#pragma unroll
            for (int k = 0; k < DK; k++) d[(size_t)k * DN_BW] = S[k];
            ci++;
        }
        __syncwarp();  // every lane is done with token t's slot before it is refilled
    }
    cp_async_wait<0>();
#pragma unroll
    for (int k = 0; k < DK; k++) Sg[(size_t)k * DN_BW] = S[k];
}

// ---- the steps around the recurrence (dn_prep_part, reference src/forward.c:2104; dn_out :2280) ----------------------
// sum of x[i] y[i] over n = 16 m values held in shared memory, in the reference's order (dn_dot16 :2018): lane j of 16
// adds i = j, j + 16, ... as an fma chain, then the tree (j + 8, + 4, + 2, + 1).  Called by the whole CTA (>= 32
// threads); the result comes back to every thread through res_smem.
__device__ __forceinline__ float dn_dot16_cta(const float *x, const float *y, int n, float *res_smem) {
    const int tid = threadIdx.x;
    if (tid < 32) {
        const int j = tid & 15;
        float a = 0.0f;
        for (int i = j; i < n; i += 16) a = fmaf(x[i], y[i], a);
        a = a + __shfl_down_sync(0xffffffffu, a, 8, 16);
        a = a + __shfl_down_sync(0xffffffffu, a, 4, 16);
        a = a + __shfl_down_sync(0xffffffffu, a, 2, 16);
        a = a + __shfl_down_sync(0xffffffffu, a, 1, 16);
        if (tid == 0) *res_smem = a;
    }
    __syncthreads();
    return *res_smem;
}

// Step 1 of a linear-attention layer for the rows of the pass, in place (rows: [q | k | v | z | alpha | beta] raw
// projections -> q, k, v = SiLU(causal conv over the last `conv` inputs), q / k L2-normalised, q also x 1/sqrt(dk),
// exp(g) and beta in place of alpha / beta).  One CTA of 128 threads per (segment, channel group: q or k of a key head,
// v of a value head); thread i owns channel i and walks the segment's rows in order with the last conv - 1 raw
// inputs in registers, so the conv state is read once and written once.  dk = dv = 128, conv <= 8.
// Everything except the two libm calls of the gate (expf, log1pf) repeats the reference's operations in order.
__global__ void __launch_bounds__(128) dn_prep_kernel(const DnSeg *__restrict__ segs, int lin_layer, int nk, int nv, int K,
                                                      const float *__restrict__ w_conv, const float *__restrict__ w_a,
                                                      const float *__restrict__ w_dt, float *__restrict__ rows, int lw,
                                                      const DnCk *__restrict__ cks) {
    constexpr int CN = 128;
    const int i = threadIdx.x, grp = blockIdx.x;
    const DnSeg sg = segs[blockIdx.y];
    const int kind = grp < nk ? 0 : grp < 2 * nk ? 1 : 2, h = kind == 0 ? grp : kind == 1 ? grp - nk : grp - 2 * nk;
    const int conv_dim = 2 * nk * CN + nv * CN, vdim = nv * CN;
    const size_t c0 = kind == 0 ? (size_t)h * CN : kind == 1 ? (size_t)nk * CN + (size_t)h * CN : (size_t)2 * nk * CN + (size_t)h * CN;
    float *st = sg.state + (size_t)lin_layer * sg.lstride + (size_t)(K - 1) * c0;  // [K - 1][CN], oldest first
    const float *w = w_conv + (size_t)K * c0;                                      // [K][CN] taps
    __shared__ float buf[CN];
    __shared__ float dot;
    float win[8], wt[8];
    int ci = 0;  // checkpoints of the segment taken so far
#pragma unroll
    for (int j = 0; j < 8; j++) {
        wt[j] = j < K ? w[(size_t)j * CN + i] : 0.0f;
        win[j] = (j < K - 1 && !sg.first) ? st[(size_t)j * CN + i] : 0.0f;
    }
    for (int t = 0; t < sg.n; t++) {
        float *row = rows + (size_t)(sg.row0 + t) * lw;
        const float x = row[c0 + i];
        float o = wt[0] * win[0];
#pragma unroll
        for (int j = 1; j < 7; j++)
            if (j < K - 1) o = fmaf(wt[j], win[j], o);
        float wl = wt[0];
#pragma unroll
        for (int j = 1; j < 8; j++)
            if (j == K - 1) wl = wt[j];
        o = fmaf(wl, x, o);
#pragma unroll
        for (int j = 0; j < 7; j++)  // the window moves on: win[K - 2] = this row's input
            win[j] = j < K - 2 ? win[j + 1] : (j == K - 2 ? x : win[j]);
        o = o * sigmoid_att(o);
        if (kind < 2) {
            __syncthreads();  // (buf and dot of the previous row have been read)
            buf[i] = o;
            __syncthreads();
            const float inv = 1.0f / sqrtf(dn_dot16_cta(buf, buf, CN, &dot) + 1e-6f);
            if (kind == 0) {
                const float sc = 1.0f / sqrtf((float)CN);
                o = o * inv * sc;
            } else {
                o = o * inv;
            }
        } else if (i == 0) {
            float *ab = row + conv_dim + vdim + h;
            const float xg = ab[0] + w_dt[h];
            const float sp = xg > 20.0f ? xg : log1pf(expf(xg));
            ab[0] = expf(w_a[h] * sp);
            ab[nv] = sigmoid_att(ab[nv]);
        }
        row[c0 + i] = o;
        if (ci < sg.nck && t == cks[sg.ck0 + ci].row) {  // a checkpoint after this row: the conv inputs as they stand
            float *d = cks[sg.ck0 + ci].dst + (st - sg.state);
#pragma unroll
            for (int j = 0; j < 7; j++)
                if (j < K - 1) d[(size_t)j * CN + i] = win[j];
            ci++;
        }
    }
#pragma unroll
    for (int j = 0; j < 7; j++)
        if (j < K - 1) st[(size_t)j * CN + i] = win[j];
}

// Step 3: the gated RMSNorm of a head's outputs times SiLU(z), in place on out [rows][nv * 128] (dn_out :2280)
__global__ void __launch_bounds__(128) dn_out_kernel(int nk, int nv, const float *__restrict__ w_norm, const float *__restrict__ rows, int lw,
                                                     float *__restrict__ out) {
    constexpr int DV = 128;
    const int r = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
    __shared__ float buf[DV];
    __shared__ float dot;
    float *o = out + (size_t)r * nv * DV + (size_t)h * DV;
    const float z = rows[(size_t)r * lw + (size_t)2 * nk * DV + (size_t)nv * DV + (size_t)h * DV + j];
    const float x = o[j];
    buf[j] = x;
    __syncthreads();
    const float ss = 1.0f / sqrtf(dn_dot16_cta(buf, buf, DV, &dot) * (1.0f / DV) + 1e-6f);
    o[j] = w_norm[j] * (ss * x) * (z * sigmoid_att(z));
}

}  // namespace rq
