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

struct DnSeg {
    float *state;   // the segment's sequence: state of linear layer 0 (conv part included)
    size_t lstride; // floats from one linear layer's state to the next
    int row0, n;    // rows of the pass: row0 .. row0 + n - 1
    int first;      // the segment starts at position 0: S is cleared first
    int pad;
};

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
                                                    float *__restrict__ out) {
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
        __syncwarp();  // every lane is done with token t's slot before it is refilled
    }
    cp_async_wait<0>();
#pragma unroll
    for (int k = 0; k < DK; k++) Sg[(size_t)k * DN_BW] = S[k];
}

}  // namespace rq
