// Gated DeltaNet recurrence, exact token-by-token form (dn_rec_run, reference src/forward.c:2224; passes dn_p1 / dn_p2
// :2177-2203).
//
// Per value head h (key head h % nk) and value column v, tokens in order, S is [dk][dv]:
//     u    = sum over k, in order, of fma(S[k][v] * eg, key[k], .)         (from 0)
//     u    = (val[v] - u) * beta
//     S[k][v] = fma(key[k], u, S[k][v] * eg)
//     o[v] = sum over k, in order, of fma(S[k][v], query[k], .)            (on the updated S, from 0)
// Each column is independent of the others, which is how the work is cut: one warp per (segment, value head, block of
// 32 columns), each lane keeping its column of S (dk floats) in registers for the whole run of rows; the key / query
// rows of a token are staged in shared memory and broadcast.  The u-chain of token t + 1 is interleaved with the
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

template <int DK>
__global__ void __launch_bounds__(32) dn_rec_kernel(const DnSeg *__restrict__ segs, int lin_layer, int nk, int nv, int dv,
                                                    size_t conv_floats, const float *__restrict__ rows, int lw,
                                                    float *__restrict__ out) {
    const int nblk = dv / DN_BW;
    const int jb = blockIdx.x % nblk, h = blockIdx.x / nblk, lane = threadIdx.x;
    const DnSeg sg = segs[blockIdx.y];
    const int conv_dim = 2 * nk * DK + nv * dv, vdim = nv * dv;
    const size_t oq = (size_t)(h % nk) * DK, ok = (size_t)nk * DK + oq;
    const size_t ov = (size_t)2 * nk * DK + (size_t)h * dv + (size_t)jb * DN_BW + lane;
    const size_t oe = (size_t)conv_dim + vdim + h, ob = oe + nv;
    float *Sg = sg.state + (size_t)lin_layer * sg.lstride + conv_floats + (size_t)h * DK * dv + (size_t)jb * DK * DN_BW + lane;

    __shared__ float kq[2][2][DK];  // [buffer][0: key, 1: query][dk]
    float S[DK];
#pragma unroll
    for (int k = 0; k < DK; k++) S[k] = sg.first ? 0.0f : Sg[(size_t)k * DN_BW];

    const float *r = rows + (size_t)sg.row0 * lw;
    for (int k = lane; k < DK; k += 32) {
        kq[0][0][k] = r[ok + k];
        kq[0][1][k] = r[oq + k];
    }
    __syncwarp();
    float eg = r[oe];
    float u = 0.0f;
#pragma unroll
    for (int k = 0; k < DK; k++) u = fmaf(S[k] * eg, kq[0][0][k], u);

    for (int t = 0; t < sg.n; t++) {
        const int cur = t & 1, nxt = cur ^ 1;
        const float beta = r[ob], val = r[ov];
        u = (val - u) * beta;
        const float *rn = r + lw;
        float o = 0.0f, un = 0.0f;
        if (t + 1 < sg.n) {
            for (int k = lane; k < DK; k += 32) {
                kq[nxt][0][k] = rn[ok + k];
                kq[nxt][1][k] = rn[oq + k];
            }
            __syncwarp();
            const float egn = rn[oe];
#pragma unroll
            for (int k = 0; k < DK; k++) {
                float sv = fmaf(kq[cur][0][k], u, S[k] * eg);
                S[k] = sv;
                o = fmaf(sv, kq[cur][1][k], o);
                un = fmaf(sv * egn, kq[nxt][0][k], un);
            }
            eg = egn;
        } else {
#pragma unroll
            for (int k = 0; k < DK; k++) {
                float sv = fmaf(kq[cur][0][k], u, S[k] * eg);
                S[k] = sv;
                o = fmaf(sv, kq[cur][1][k], o);
            }
        }
        out[(size_t)(sg.row0 + t) * vdim + (size_t)h * dv + (size_t)jb * DN_BW + lane] = o;
        u = un;
        r = rn;
        __syncwarp();
    }
#pragma unroll
    for (int k = 0; k < DK; k++) Sg[(size_t)k * DN_BW] = S[k];
}

}  // namespace rq
