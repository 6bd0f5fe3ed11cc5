// Split-K decode attention over quantised KV caches (q8, q4, q4k4) on the integer tensor cores (tcgen05.mma kind::i8 + TMEM),
// head_dim 128: the fast form of attn_part_kernel for these caches.
//
// Same work items and the same partial results as attn_part_kernel (one (o, m, l) record per (row, KV head, block of 256
// positions), merged in block order by attn_combine_kernel, which also un-rotates and gates), so the split still
// depends on a row's own length only and a row of a batch gives the bits it gives alone.  What changes is the arithmetic
// inside a block.  The CUDA-core kernel spends ~8 instructions per cached level (conversion, scale, four multiply-adds).
// Here the cached levels are never converted to floats at all: they go from HBM to shared memory by the copy engines and from
// there into tcgen05.mma as 8-bit operands, accumulated exactly in int32:
//   8-bit V rows [position][128 dims] as cached, fetched through a 3-D tensor map with the 128-byte swizzle = an MN-major A operand:
//   O^T [128 dims x N'] += V^T [128 dims x 32 keys] P^T;
//   8-bit K tiles [dim][16 positions] hold 16 keys per dim, and the fast operand form wants a dim's 128 keys in one 128-byte row (the
//   tiles as they are, 8 dims x 16 positions per 128-byte core matrix without swizzle, are a valid operand too, but measured
//   ~700 cycles per MMA): the block's 16 tiles arrive as cached by one bulk copy and every thread moves 16-byte chunks shared ->
//   shared to their place in the swizzled rows (8 loads and 8 stores per thread and block, no arithmetic), then per 32-dim scale
//   group c one MMA  S_c^T [128 keys x N] = K_c [128 keys x 32 dims] Q_c^T;
//   4-bit levels n (stored + 8; K of q4k4, V of q4 and q4k4) are unpacked on that same way: the nibble in the high half of a byte
//   with its top bit flipped is the int8 value 16 (n - 8) (shift, mask, xor per 4 levels), and 1 / 16 goes into the scale; 4-bit
//   V tiles land as cached at the end of the V operand's place and are unpacked over it.
// The other operands are 16-bit fixed point split into two int8 planes (the query per (vector, group), by tcd_q_prep_kernel;
// the softmax weights times the V scale per (vector, group), scaled by the block's largest V scale magnitude of the group), so
// the only roundings are those two quantisations to 16 bits; the scales (exact bf16 -> fp32) are applied in fp32 by the
// softmax thread of a key (s = sum_c d_K[t][c] q_scale[v][c] S_c) and the epilogue thread of a dim.  Results agree with the
// reference's fp32 arithmetic to ~1e-4 relative, inside the acceptance bar but not bit for bit; the bit-exact kernels stay
// selectable (rq_cuda_set_exact).  With the keys on the TMEM lanes the softmax of a block is spread over all threads.
#pragma once
#include <cuda.h>

#include "attn_decode.cuh"
#include "tc05.cuh"

namespace rq {

constexpr int TCD_THREADS = 256;
constexpr int TCD_QT_BYTES = 2048 + 256;  // per (row, KV head): Q^T planes [16 rows][128 dims] int8 + scales [8 vectors][4 groups] fp32 (+ pad)

template <int NVT, int KF = KV_Q8, int VF = KV_Q8>  // KF, VF: 8-bit (KV_Q8) or 4-bit (KV_Q4) levels of K and of V
struct TcdCfg {
    static constexpr int HD = 128;
    static constexpr int KTB = HD * (KF == KV_Q8 ? 17 : 9), VTB = HD * (VF == KV_Q8 ? 17 : 9);  // 2176 (8-bit) or 1152 (4-bit)
    static constexpr int KSC = (KF == KV_Q8 ? 16 : 8) * HD, VSC = (VF == KV_Q8 ? 16 : 8) * HD;  // the scales behind a tile's levels
    // 4-bit V: the block's 16 tiles as cached land at the end of the V operand's place and are unpacked over it
    static constexpr int VRAW_OFF = 32768 - 16 * (HD * 9);
    static constexpr int NS = NVT <= 4 ? 8 : 16;  // N of a score MMA: rows 2 v + plane
    static constexpr int NO = 8 * NVT;            // N of an output MMA: rows ((c NVT + v) 2 + plane)
    // shared memory (from a 1024-byte aligned base): the next block's 16 K tiles as cached (one bulk copy) | K levels of the two
    // halves as the operand wants them (2 x 16 KB: 128 rows = dims of 128 keys) | V levels (2 x 16 KB: 128 rows = positions of 128
    // dims, swizzled by the TMA) | P^T (2 x NO rows of 128 bytes) | Q^T planes, two buffers of 2 KB, and their scales, 2 x 256 B | the rest
    static constexpr int KRAW = 0, KLEV = (16 * KTB + 1023) / 1024 * 1024, VLEV = KLEV + 32768, PT = VLEV + 32768, QT = PT + 2 * NO * 128, QS = QT + 4096;
    static constexpr int MISC = QS + 512;  // red (768 B: two buffers of block reductions, 128 B each)  | bars [6] (64 B) | TMEM slot (16 B) | items [4] (128 B)
    static constexpr int SMEM = MISC + 768 + 64 + 16 + 128 + 1024;
    // TMEM columns: the score products of two blocks (2 x 8 NS) | the output products
    static constexpr int S_COL = 0, O_COL = 16 * NS, TM_COLS = NVT <= 4 ? 256 : 512;
    static_assert(KLEV % 1024 == 0 && VLEV % 1024 == 0 && PT % 1024 == 0 && QT % 1024 == 0, "operand alignment");
    static_assert(O_COL + NO <= TM_COLS, "TMEM columns");
    static_assert(NVT > 4 || 2 * (SMEM + 1024) <= 228 * 1024, "two CTAs per SM");
    static_assert(VRAW_OFF % 16 == 0 && VRAW_OFF > 0, "bulk copy alignment");
    static_assert(KTB == kv_tile_bytes(KF == KV_Q8 ? KV_Q8 : KV_Q4K4, HD, 0) && VTB == kv_tile_bytes(VF == KV_Q8 ? KV_Q8 : KV_Q4K4, HD, 1), "tile bytes");
};

// a work item as the describing thread leaves it in shared memory for the others
struct TcdItem {
    int n;                  // positions of the block (1 .. 256)
    int q;                  // query planes: buffer (bit 0), phase parity of its barrier (bit 1)
    int vt, seg;            // first tile of the block in the 3-D view of its sequence's V cache; the row's segment
    int gb, g;              // block of the pass, KV head: where the partial records go
    unsigned long long vs;  // the block's V tiles in global memory (their scales are read from there)
};
static_assert(sizeof(TcdItem) == 32, "four items in 128 bytes");

struct AttnPartTcArgs {
    int kvt;  // KV_Q8, KV_Q4 (8-bit K, 4-bit V) or KV_Q4K4
    const PassRow *rows;
    int nrows, total_blocks, layer, n_kv, G;
    const float *q;
    int qh, n_heads;
    float scale;
    float *part;
    uint8_t *qt;              // scratch: nrows x n_kv records of TCD_QT_BYTES
    int *blk2row;             // scratch: total_blocks ints
    const CUtensorMap *maps;  // per segment: [4 seg + 1] = the 3-D view of its sequence's V cache levels
    int n_sm;                 // SMs of the device: the grid is a fixed number of CTAs per SM
    int *err;
};
// launches tcd_q_prep_kernel and attn_part_tc_kernel on `stream`; cudaErrorInvalidValue for an unsupported shape
cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream);

#ifdef RQ_ATTN_DECODE_TC_INSTANTIATE

// instruction descriptor of tcgen05.mma kind::i8: int8 / uint8 operands, int32 accumulator, M x N; a_mn / b_mn: MN-major (1) or
// K-major (0); a_s / b_s: signed (1) or unsigned (0) 8-bit values
__host__ __device__ constexpr uint32_t umma_idesc_i8(int M, int N, int a_mn, int b_mn, int a_s, int b_s) {
    return (2u << 4) | ((uint32_t)a_s << 7) | ((uint32_t)b_s << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem), "l"(a), "l"(b),
                 "r"(idesc), "r"(acc)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *m, int x, int y, int z, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                     smem_u32(dst)),
                 "l"(m), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}

// The query vectors of one (row, KV head), once per pass and layer: rotated as att_q_rot does (reference src/forward.c:1662:
// signs, butterflies h = 1, 2, 4, ..., scaling by 1 / head_dim) in fp32, then per (vector v, 32-dim group c) 16-bit fixed point
// q = qs[v][c] (256 hi + lo), hi and lo in [-128, 127], laid out as the B operand of the score MMAs: rows 2 v (hi) and 2 v + 1
// (lo) of [16 rows][128 dims] int8, K-major with the 128-byte swizzle; rows past the G vectors zero; the scales qs behind
// them.  The CTA of KV head 0 also fills the block -> row table of its row.
__global__ void __launch_bounds__(128) tcd_q_prep_kernel(const PassRow *__restrict__ rows, int n_kv, int G, const float *__restrict__ q, int qh,
                                                         int n_heads, uint8_t *__restrict__ qt, int *__restrict__ blk2row) {
    constexpr int HD = 128;
    const int r = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, c = tid >> 5;  // (a warp = a 32-dim group)
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float tmp[8][HD];
    __shared__ __align__(16) int8_t planes[16][HD];
    const PassRow row = rows[r];
    if (g == 0) {
        const int nb = (row.np + ATT_P - 1) / ATT_P;
        for (int b = tid; b < nb; b += 128) blk2row[row.blk0 + b] = r;
    }
    const float *qrow = q + ((size_t)r * n_heads + (size_t)g * G) * qh;
    for (int v = 0; v < G; v++) {
        const float x = qrow[(size_t)v * qh + tid];
        tmp[v][tid] = kvq_neg(tid) ? -x : x;
    }
    __syncthreads();
    for (int hs = 1; hs < HD; hs <<= 1) {
        for (int e = tid; e < G * HD / 2; e += 128) {
            const int v = e / (HD / 2), p = e % (HD / 2);
            const int j = (p / hs) * 2 * hs + (p % hs);
            const float a = tmp[v][j], bb = tmp[v][j + hs];
            tmp[v][j] = a + bb;
            tmp[v][j + hs] = a - bb;
        }
        __syncthreads();
    }
    uint8_t *out = qt + ((size_t)r * n_kv + g) * TCD_QT_BYTES;
    float *qs = reinterpret_cast<float *>(out + 2048);
    const float f = 1.0f / (float)HD;
    for (int v = 0; v < 8; v++) {
        int hi = 0, lo = 0;
        if (v < G) {
            const float x = tmp[v][tid] * f;
            float amax = fabsf(x);
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float sc = amax > 0.0f ? amax / 32639.0f : 0.0f;
            const int q16 = amax > 0.0f ? __float2int_rn(x * (32639.0f / amax)) : 0;
            lo = ((q16 + 128) & 255) - 128;
            hi = (q16 - lo) >> 8;
            if (lane == 0) qs[v * 4 + c] = sc;
        } else if (lane == 0) {
            qs[v * 4 + c] = 0.0f;
        }
        planes[2 * v][tid] = (int8_t)hi;
        planes[2 * v + 1][tid] = (int8_t)lo;
    }
    __syncthreads();
    {  // one 16-byte chunk (16 dims) of one row per thread: 16 rows x 8 chunks
        const int rw = tid >> 3, ch = tid & 7;
        *reinterpret_cast<uint4 *>(out + rw * 128 + ((ch ^ (rw & 7)) << 4)) = *reinterpret_cast<const uint4 *>(&planes[rw][ch * 16]);
    }
}

// order-preserving map between floats and signed integers (its own inverse): integer maxima of mapped values are float maxima
__device__ __forceinline__ int f32_ord(float f) {
    const int b = __float_as_int(f);
    return b >= 0 ? b : b ^ 0x7fffffff;
}
__device__ __forceinline__ float ord_f32(int b) { return __int_as_float(b >= 0 ? b : b ^ 0x7fffffff); }

// One CTA's teardown wait for a copy that may still be in flight once a wait has expired: polls for at most ~2 ms whatever
// the status word says, so that the CTA does not leave while a copy still writes its shared memory.
__device__ __forceinline__ void mbar_drain(uint64_t *bar, uint32_t parity) {
    unsigned long long t0 = 0;
    for (int it = 0; it < (1 << 22); it++) {
        if (mbar_try_wait(bar, parity)) return;
        if ((it & 255) == 255) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            if (now - t0 > 2000000ull) return;
        }
    }
}

// Persistent form: the grid is two CTAs per SM (one for 5..8 vectors per KV head), each CTA walks a contiguous range of the work
// items (KV head g, block gb of the pass) in the order j = g total_blocks + gb, so that consecutive items mostly share their row
// and its query planes.  Everything an item needs from global memory is asked for ahead of its use and by copy engines, not by
// the threads' own loads: item i + 2's K tiles (one bulk copy of the 16 tiles as cached) while item i is computed, item i's V
// levels (TMA) as soon as the output products of item i - 1 have released the buffer.  Item i + 1's K chunks are moved to the
// operand's layout (shared -> shared) and its score MMAs issued while item i goes through its softmax, so a block's scores are
// complete when its turn comes (two score buffers in TMEM).  Per item two CTA barriers:
//   S2  block maxima of every warp; next item's K levels in place  -> weights (all), next item's score MMAs (one thread)
//   S3  P^T planes in place                                        -> output MMAs (one thread)
// (4-bit V: one more, S2b, between reading the V tiles as cached and writing the unpacked rows over them)
// The single-thread duties are spread over the first lanes of warps 4 .. 7 (warps 0 .. 3 store the partial results, and thread 0
// asks for the next V levels there, where it has waited for the output products anyway): (m, l), items + K and Q copies, output
// MMAs, score MMAs.  (An MMA of these shapes keeps its issuing thread for ~150 cycles: the two batches of eight go to two warps.)
// maps: per segment [4 seg + 1] the tensor map of its sequence's V cache: {128 bytes of levels, 16 positions, tiles} with
// strides {128, tile bytes}, box 128 x 16 x 8, 128-byte swizzle.
template <int NVT, int KF, int VF>
__global__ void __launch_bounds__(TCD_THREADS, NVT <= 4 ? 2 : 1)
    attn_part_tc_kernel(const PassRow *__restrict__ rows, const int *__restrict__ blk2row, const uint8_t *__restrict__ qtg,
                        const CUtensorMap *__restrict__ maps, int layer, int n_kv, int G, int n_heads, float scale, float *__restrict__ part,
                        int total_blocks, int *err) {
    using C = TcdCfg<NVT, KF, VF>;
    constexpr int HD = C::HD, NS = C::NS, NO = C::NO;
    // 4-bit levels n (stored + 8) enter the MMAs as the int8 values 16 (n - 8): the nibble in the high half of a byte with its top bit
    // flipped; the factor goes into the scales
    constexpr float KMUL = KF == KV_Q8 ? 1.0f : 0.0625f, VMUL = VF == KV_Q8 ? 1.0f : 0.0625f;
    // the weight planes: 8-bit V scales are positive (largest magnitude / 127): unsigned 16-bit weights; 4-bit scales carry a sign
    // (first largest element / -8, src/forward.c:1901 kv_store): signed weights, +-(127 x 256 + 127), both planes signed
    constexpr float PMAX = VF == KV_Q8 ? 65535.0f : 32639.0f;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *sm = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *pt = sm + C::PT;
    float *red = reinterpret_cast<float *>(sm + C::MISC);               // two buffers of block reductions, used in turn
    uint64_t *bars = reinterpret_cast<uint64_t *>(sm + C::MISC + 768);  // K tiles, V levels, Q^T buffer 0 / 1, scores, outputs
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm + C::MISC + 768 + 64);
    TcdItem *items = reinterpret_cast<TcdItem *>(sm + C::MISC + 768 + 64 + 16);  // [4]: item i in items[i % 4]
    uint64_t *bar_k = bars, *bar_v = bars + 1, *bar_q = bars + 2, *bar_s = bars + 4, *bar_o = bars + 5;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long n_items = (long long)total_blocks * n_kv;
    const int j0 = (int)(n_items * blockIdx.x / gridDim.x), cnt = (int)(n_items * (blockIdx.x + 1) / gridDim.x) - j0;

    if (tid == 0) {
        for (int i = 0; i < 6; i++) mbar_init(bars + i, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tmem_slot;
    const uint32_t lane_addr = tbase + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t sbase = smem_u32(sm);
    const int h2 = tid >> 7, t = tid & 127, pos = 128 * h2 + t;  // this thread's key of a block
    const float c2 = scale * 1.44269504088896341f;
    constexpr int T_V = 0, T_ML = 128, T_ITEMS = 160, T_PV = 192, T_MMA = 224;  // the threads with a duty of their own
    bool ok = true;
    pdl_wait();

    // ---- thread T_ITEMS: the row of the item last described (re-read when an item leaves its blocks), the query planes copied so far
    int r_lo = 0, r_blk0 = 0, r_nb = 0, r_np = 0, r_seg = 0, r_vt0 = 0, r_g = -1, nq = 0;
    const uint8_t *r_k = nullptr, *r_v = nullptr;
#ifdef RQ_DEBUG
    unsigned long long r_lk = 0, r_lv = 0;
#endif
    // describes item i of this CTA into items[i % 4] and asks for its K tiles (and its query planes where they are new)
    auto describe = [&](int i) {
        const int j = j0 + i, g = j / total_blocks, gb = j - g * total_blocks;
        bool qnew = g != r_g;
        if (r_g < 0 || gb < r_blk0 || gb >= r_blk0 + r_nb) {
            r_lo = __ldg(blk2row + gb);
            const PassRow row = rows[r_lo];
            r_blk0 = row.blk0, r_np = row.np, r_nb = (row.np + ATT_P - 1) / ATT_P, r_seg = row.seg;
            r_k = row.k + (size_t)layer * row.lk, r_v = row.v + (size_t)layer * row.lv;
            r_vt0 = (int)((size_t)layer * (row.lv / C::VTB));
#ifdef RQ_DEBUG
            r_lk = row.lk, r_lv = row.lv;
#endif
            qnew = true;
        }
        r_g = g;
        const int b = gb - r_blk0, n = min(r_np - b * ATT_P, ATT_P), nh = (n + 127) >> 7;
        // (whole halves are fetched: a layer is a whole number of 256-position blocks, so the tiles past the block's last
        // position exist; what they hold is masked below and enters the integer products as finite values times zero weights)
        const size_t tile0 = ((size_t)b * n_kv + g) * ATT_PT;
        if (qnew) nq++;
        TcdItem d;
        d.n = n, d.q = ((nq - 1) & 1) | ((((nq - 1) >> 1) & 1) << 1), d.vt = r_vt0 + (int)tile0, d.seg = r_seg, d.gb = gb, d.g = g;
        d.vs = (unsigned long long)(uintptr_t)(r_v + tile0 * C::VTB);
        items[i & 3] = d;
#ifdef RQ_DEBUG
        // (debug build: an item that does not fit its row or cache is not fetched: the CTA records it and ends its loop at the next
        // barrier that votes; the waits for its copies give up at once because the status word is set)
        if (!(r_lo >= 0 && b >= 0 && n >= 1 && g < n_kv && (tile0 + 16) * C::KTB <= r_lk && (tile0 + 16) * C::VTB <= r_lv)) {
            atomicExch(err, 47);
            ok = false;
            return;
        }
#endif
        fence_proxy_async();  // (the threads' reads of the tiles before, ordered by the CTA barrier, before the copy's writes)
        mbar_expect_tx(bar_k, 8u * C::KTB * (uint32_t)nh);
        bulk_g2s(sm + C::KRAW, r_k + tile0 * C::KTB, 8u * C::KTB * (uint32_t)nh, bar_k);
        if (qnew) {
            const int qb = (nq - 1) & 1;
            const uint8_t *src = qtg + ((size_t)r_lo * n_kv + g) * TCD_QT_BYTES;
            mbar_expect_tx(bar_q + qb, TCD_QT_BYTES);
            bulk_g2s(sm + C::QT + qb * 2048, src, 2048, bar_q + qb);
            bulk_g2s(sm + C::QS + qb * 256, src + 2048, 256, bar_q + qb);
        }
    };
    // item i's V levels (thread T_V), once the output products of item i - 1 have released the buffer (store_o)
    auto fetch_v = [&](int i) {
        const TcdItem d = items[i & 3];
        const int nh = (d.n + 127) >> 7;
        if constexpr (VF == KV_Q8) {
            const CUtensorMap *mv = maps + 4 * d.seg + 1;
            mbar_expect_tx(bar_v, 16384u * (uint32_t)nh);
            for (int h = 0; h < nh; h++) tma_load_3d(sm + C::VLEV + h * 16384, mv, 0, 0, d.vt + 8 * h, bar_v);
        } else {  // the tiles as cached, unpacked by the threads (unpack_v)
            fence_proxy_async();
            mbar_expect_tx(bar_v, 8u * C::VTB * (uint32_t)nh);
            bulk_g2s(sm + C::VLEV + C::VRAW_OFF, (const uint8_t *)(uintptr_t)d.vs, 8u * C::VTB * (uint32_t)nh, bar_v);
        }
    };
    // item i's K chunks from the tiles as cached to where the operand wants them (row = dim, chunk = tile ^ (dim % 8): the 128-byte
    // swizzle), and the scales of this thread's key: K [group][16 positions] behind the tile's levels in shared memory, V
    // [position][group] from global memory
    uint32_t ks_n[4];
    uint2 vs_n;
    auto stage_k = [&](int i) {
        const TcdItem d = items[i & 3];
        const int nh = (d.n + 127) >> 7;
        if (lane == 0) ok = mbar_wait_bounded_quiet(bar_k, (uint32_t)i & 1u, err, 72) && ok;
        __syncwarp();
        if constexpr (KF == KV_Q8) {
#pragma unroll
            for (int k = 0; k < 8; k++) {  // chunk (tile u, dim i): 16 positions of one dim
                const int idx = tid + TCD_THREADS * (k & 3), u = (idx >> 7) + 8 * (k >> 2), dim = idx & 127;
                if ((k >> 2) < nh)
                    *reinterpret_cast<uint4 *>(sm + C::KLEV + (k >> 2) * 16384 + dim * 128 + (((u & 7) ^ (dim & 7)) << 4)) =
                        *reinterpret_cast<const uint4 *>(sm + C::KRAW + u * C::KTB + dim * 16);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; k++) {  // chunk (tile u, dim pair p): 16 positions, low nibbles dim 2p, high nibbles dim 2p + 1
                const int idx = tid + TCD_THREADS * (k & 1), u = (idx >> 6) + 8 * (k >> 1), p = idx & 63;
                if ((k >> 1) < nh) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(sm + C::KRAW + u * C::KTB + p * 16);
                    uint8_t *dst = sm + C::KLEV + (k >> 1) * 16384 + (2 * p) * 128;
                    *reinterpret_cast<uint4 *>(dst + (((u & 7) ^ ((2 * p) & 7)) << 4)) =
                        make_uint4(((w.x << 4) & 0xF0F0F0F0u) ^ 0x80808080u, ((w.y << 4) & 0xF0F0F0F0u) ^ 0x80808080u,
                                   ((w.z << 4) & 0xF0F0F0F0u) ^ 0x80808080u, ((w.w << 4) & 0xF0F0F0F0u) ^ 0x80808080u);
                    *reinterpret_cast<uint4 *>(dst + 128 + (((u & 7) ^ ((2 * p + 1) & 7)) << 4)) =
                        make_uint4((w.x & 0xF0F0F0F0u) ^ 0x80808080u, (w.y & 0xF0F0F0F0u) ^ 0x80808080u, (w.z & 0xF0F0F0F0u) ^ 0x80808080u,
                                   (w.w & 0xF0F0F0F0u) ^ 0x80808080u);
                }
            }
        }
        if (pos < d.n) {
            const uint16_t *ks = reinterpret_cast<const uint16_t *>(sm + C::KRAW + (pos >> 4) * C::KTB + C::KSC) + (pos & 15);
#pragma unroll
            for (int c = 0; c < 4; c++) ks_n[c] = ks[c * 16];
            vs_n = __ldg(reinterpret_cast<const uint2 *>((const uint8_t *)(uintptr_t)d.vs + (size_t)(pos >> 4) * C::VTB + C::VSC) + (pos & 15));
        } else {
            ks_n[0] = ks_n[1] = ks_n[2] = ks_n[3] = 0u;
            vs_n = make_uint2(0u, 0u);
        }
    };
    // item i's score MMAs (thread T_MMA): S_c^T (half h) = K_c (half h) Q_c^T, one MMA per 32-dim group, into score buffer i % 2
    auto issue_s = [&](int i) {
        const TcdItem d = items[i & 3];
        const int nh = (d.n + 127) >> 7, qb = d.q & 1;
        tc_fence_after();
        ok = mbar_wait_bounded_quiet(bar_q + qb, (uint32_t)(d.q >> 1) & 1u, err, 74) && ok;
        constexpr uint32_t idesc_s = umma_idesc_i8(128, NS, 1, 0, 1, 1);
        for (int h = 0; h < nh; h++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                // A: rows of 128 bytes (one dim, the half's 128 keys = one swizzle atom along MN), 8 dims = 1024 bytes (SBO); the group's
                // 32 dims are 4096 bytes; B: rows of 128 bytes, 128-byte swizzle, the group's 32 dims at 32 c
                const uint64_t da = umma_desc(sbase + C::KLEV + h * 16384 + c * 4096, 16, 1024, 2);
                const uint64_t db = umma_desc(sbase + C::QT + qb * 2048 + c * 32, 16, 1024, 2);
                umma_i8(tbase + C::S_COL + (i & 1) * 8 * NS + (4 * h + c) * NS, da, db, idesc_s, 0);
            }
        }
        umma_commit(bar_s);
    };
    // the partial result of item i: o[hd] (unnormalised; m and l are stored by its softmax).  Thread = dim of group c = dim / 32
    // (uniform over the warp): the columns (c, v, plane) of O.  Warps 0 .. 3.
    auto store_o = [&](int i, float back, long long pidx, bool next_v) {
        if (lane == 0) {
            ok = mbar_wait_bounded_quiet(bar_o, (uint32_t)i & 1u, err, 75) && ok;
            if (tid == T_V && next_v) fetch_v(i + 1);  // (the output products of item i have released the V buffer)
        }
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        uint32_t r[2 * NVT < 8 ? 8 : 2 * NVT];
        tmem_ld8(lane_addr + C::O_COL + warp * 2 * NVT, r);
        if constexpr (NVT == 8) tmem_ld8(lane_addr + C::O_COL + warp * 2 * NVT + 8, r + 8);
        tmem_wait_ld();
        float o[NVT];
        if constexpr (NVT % 2 == 0) {
#pragma unroll
            for (int v = 0; v < NVT; v += 2) {
                const float2 x = __fmul2_rn(__ffma2_rn(make_float2((float)(int)r[2 * v], (float)(int)r[2 * v + 2]), make_float2(256.0f, 256.0f),
                                                       make_float2((float)(int)r[2 * v + 1], (float)(int)r[2 * v + 3])),
                                            make_float2(back, back));
                o[v] = x.x, o[v + 1] = x.y;
            }
        } else {
#pragma unroll
            for (int v = 0; v < NVT; v++) o[v] = fmaf((float)(int)r[2 * v], 256.0f, (float)(int)r[2 * v + 1]) * back;
        }
#pragma unroll
        for (int v = 0; v < NVT; v++)
            if (v < G) part[pidx + (long long)v * RQ_PSTRIDE(HD) + tid] = ok ? o[v] : 0.0f;  // (tid = TMEM lane = dim)
    };

    // ---- prologue: items 0 and 1 described and asked for, item 0's K in place and its score MMAs issued
    if (tid < 64) reinterpret_cast<int *>(red)[tid] = (tid & 31) < 8 ? INT_MIN : 0;  // the two buffers of block reductions
    if (tid == T_ITEMS) describe(0);
    __syncthreads();
    if (tid == T_V) fetch_v(0);
    stage_k(0);
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == T_MMA) issue_s(0);
    if (tid == T_ITEMS && cnt > 1) describe(1);
    __syncthreads();

    float back_prev = 0.0f;   // of the item before: what its output columns are scaled back by (warps 0..3: their group)
    long long pidx_prev = 0;  // ... and its first partial record
    int it = 0;
    bool failed = false;
    for (; it < cnt; it++) {
        const TcdItem d = items[it & 3];
        const int n = d.n, nh = (n + 127) >> 7, qb = d.q & 1;
        const bool valid = pos < n, more = it + 1 < cnt;
        const long long pidx = ((long long)d.gb * n_heads + (long long)d.g * G) * RQ_PSTRIDE(HD);
        const float *qsc = reinterpret_cast<const float *>(sm + C::QS + qb * 256);  // [8][4]
        // ---- the scales of this thread's key
        float dk[4], dv[4];
#pragma unroll
        for (int c = 0; c < 4; c++) dk[c] = bf16_bits_to_f32(ks_n[c]) * KMUL;
        dv[0] = __uint_as_float(vs_n.x << 16) * VMUL, dv[1] = __uint_as_float(vs_n.x & 0xffff0000u) * VMUL;
        dv[2] = __uint_as_float(vs_n.y << 16) * VMUL, dv[3] = __uint_as_float(vs_n.y & 0xffff0000u) * VMUL;
        // ---- softmax of the block: thread (half h2, key t) holds the scores of its key for the G vectors
        // the block's largest V scale per group, what the weight planes are scaled by (the scales are positive: their bits order
        // like unsigned integers): one warp reduction each, then one shared-memory atomic of lane 8 + c
        // this block's reductions: [0..7] largest score per vector (mapped), [8..11] largest V scales, [16..23] sums of weights (fixed point)
        int *rb = reinterpret_cast<int *>(red) + (it & 1) * 32;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const unsigned mx = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(dv[c])));
            if (lane == 8 + c) atomicMax(reinterpret_cast<unsigned *>(rb) + 8 + c, mx);
        }
        // (the score products complete only after their thread has seen the query planes land: no wait of its own for those)
        if (lane == 0) ok = mbar_wait_bounded_quiet(bar_s, (uint32_t)it & 1u, err, 71) && ok;  // (one poller per warp)
        __syncwarp();
        tc_fence_after();
        float s[NVT], e[NVT];
#pragma unroll
        for (int v = 0; v < NVT; v++) s[v] = 0.0f;
        if (h2 < nh) {  // (uniform per warp)
            float qd[NVT][4];  // the query scales of (vector, group)
#pragma unroll
            for (int v = 0; v < NVT; v++) {
                const float4 x = *reinterpret_cast<const float4 *>(qsc + v * 4);
                qd[v][0] = x.x, qd[v][1] = x.y, qd[v][2] = x.z, qd[v][3] = x.w;
            }
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t r[NS];
                tmem_ld8(lane_addr + C::S_COL + (it & 1) * 8 * NS + (4 * h2 + c) * NS, r);
                if constexpr (NVT == 8) tmem_ld8(lane_addr + C::S_COL + (it & 1) * 8 * NS + (4 * h2 + c) * NS + 8, r + 8);
                tmem_wait_ld();
                if constexpr (NVT % 2 == 0) {  // (packed fp32x2 multiply and multiply-add over vector pairs)
#pragma unroll
                    for (int v = 0; v < NVT; v += 2) {
                        const float2 sc = __fmul2_rn(make_float2(dk[c], dk[c]), make_float2(qd[v][c], qd[v + 1][c]));
                        const float2 val = make_float2((float)(((int)r[2 * v] << 8) + (int)r[2 * v + 1]), (float)(((int)r[2 * v + 2] << 8) + (int)r[2 * v + 3]));
                        const float2 acc = __ffma2_rn(sc, val, make_float2(s[v], s[v + 1]));
                        s[v] = acc.x, s[v + 1] = acc.y;
                    }
                } else {
#pragma unroll
                    for (int v = 0; v < NVT; v++)
                        s[v] = fmaf(dk[c] * qd[v][c], (float)(((int)r[2 * v] << 8) + (int)r[2 * v + 1]), s[v]);
                }
            }
        }
#pragma unroll
        for (int v = 0; v < NVT; v++) {
            s[v] = valid ? s[v] : -INFINITY;
            const int mx = __reduce_max_sync(0xffffffffu, f32_ord(s[v]));
            if (lane == v) atomicMax(rb + v, mx);
        }
        if (it > 0 && warp < 4) store_o(it - 1, back_prev, pidx_prev, true);
        // ---- the next item's K levels and this thread's scales of it (the score products of this item are complete: the K levels
        // it used may go)
        if (more) stage_k(it + 1);
        fence_proxy_async();
        tc_fence_before();
        // S2 (also: every thread now knows the output products of the item before complete: P^T may be overwritten); a wait that
        // ran out anywhere ends the CTA's loop here
        if (__syncthreads_or(!ok)) {
            failed = true;
            break;
        }
        if (tid == T_MMA && more) issue_s(it + 1);
        if (tid == T_ITEMS && it + 2 < cnt) describe(it + 2);
        // 4-bit V: this block's tiles as cached, from where they landed into registers (they are unpacked over that place once every
        // thread has read its share: barrier S2b below); share k of a thread: position (tid / 4) + 64 k, scale group tid % 4
        uint4 vraw[VF == KV_Q8 ? 1 : 4];
        if constexpr (VF != KV_Q8) {
            if (lane == 0) ok = mbar_wait_bounded_quiet(bar_v, (uint32_t)it & 1u, err, 73) && ok;
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int vp = (tid >> 2) + 64 * k;
                vraw[k] = (k >> 1) < nh ? *reinterpret_cast<const uint4 *>(sm + C::VLEV + C::VRAW_OFF + (vp >> 4) * C::VTB + (vp & 15) * 64 + (tid & 3) * 16)
                                        : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        if (tid == T_ML) {  // the other buffer of reductions, for the next block
            int4 *nb = reinterpret_cast<int4 *>(reinterpret_cast<int *>(red) + ((it + 1) & 1) * 32);
            nb[0] = nb[1] = make_int4(INT_MIN, INT_MIN, INT_MIN, INT_MIN);
            nb[2] = nb[4] = nb[5] = make_int4(0, 0, 0, 0);
        }
        float m[NVT], dvp[4];
        const float4 psc = *reinterpret_cast<const float4 *>(rb + 8);
        const float ps_mine = (warp & 2) ? ((warp & 1) ? psc.w : psc.z) : ((warp & 1) ? psc.y : psc.x);
        // the key's V scales in units of the block's largest
        dvp[0] = psc.x > 0.0f ? dv[0] * __fdividef(PMAX, psc.x) : 0.0f;
        dvp[1] = psc.y > 0.0f ? dv[1] * __fdividef(PMAX, psc.y) : 0.0f;
        dvp[2] = psc.z > 0.0f ? dv[2] * __fdividef(PMAX, psc.z) : 0.0f;
        dvp[3] = psc.w > 0.0f ? dv[3] * __fdividef(PMAX, psc.w) : 0.0f;
#pragma unroll
        for (int v = 0; v < NVT; v++) m[v] = ord_f32(rb[v]);
        float ea[NVT], ef[NVT];  // the exponentials' arguments; the weights in fixed point
        if constexpr (NVT % 2 == 0) {
#pragma unroll
            for (int v = 0; v < NVT; v += 2) {
                const float2 x = __fmul2_rn(__fadd2_rn(make_float2(s[v], s[v + 1]), make_float2(-m[v], -m[v + 1])), make_float2(c2, c2));
                ea[v] = x.x, ea[v + 1] = x.y;
            }
        } else {
#pragma unroll
            for (int v = 0; v < NVT; v++) ea[v] = (s[v] - m[v]) * c2;
        }
#pragma unroll
        for (int v = 0; v < NVT; v++) e[v] = valid ? ex2(ea[v]) : 0.0f;
        if constexpr (NVT % 2 == 0) {
#pragma unroll
            for (int v = 0; v < NVT; v += 2) {
                const float2 x = __fmul2_rn(make_float2(e[v], e[v + 1]), make_float2(8388608.0f, 8388608.0f));
                ef[v] = x.x, ef[v + 1] = x.y;
            }
        } else {
#pragma unroll
            for (int v = 0; v < NVT; v++) ef[v] = e[v] * 8388608.0f;
        }
#pragma unroll
        for (int v = 0; v < NVT; v++) {
            // l: the weights summed in 23-bit fixed point (integer sums: exact whatever their order, so that a block gives the same
            // bits every time; the block's largest weight is 1, 256 of them stay below 2^32; error below 2^-16 relative)
            const unsigned sum = __reduce_add_sync(0xffffffffu, (unsigned)__float2int_rn(ef[v]));
            if (lane == v) atomicAdd(reinterpret_cast<unsigned *>(rb) + 16 + v, sum);
        }
        // P^T: the B operand of O^T += V^T P^T, per half [NO rows][128 keys] uint8, K-major with the 128-byte swizzle: rows
        // ((c NVT + v) 2 + plane) hold the two planes of round(p[.][v] d_V[.][c] 65535 / ps[c])
        if (h2 < nh) {
            uint8_t *pb = pt + h2 * (NO * 128) + (t & 15);
            const int ch = t >> 4;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float pw[NVT];  // the weights of the vectors times the key's V scale of the group
                if constexpr (NVT % 2 == 0) {
#pragma unroll
                    for (int v = 0; v < NVT; v += 2) {
                        const float2 x = __fmul2_rn(make_float2(e[v], e[v + 1]), make_float2(dvp[c], dvp[c]));
                        pw[v] = x.x, pw[v + 1] = x.y;
                    }
                } else {
#pragma unroll
                    for (int v = 0; v < NVT; v++) pw[v] = e[v] * dvp[c];
                }
#pragma unroll
                for (int v = 0; v < NVT; v++) {
                    const int rw = (c * NVT + v) * 2;
                    if constexpr (VF == KV_Q8) {
                        // (e <= 1 and d_V <= ps: the product stays within a quarter of an ulp-sized step of PMAX, no clamp needed)
                        const uint32_t u16 = (uint32_t)__float2int_rn(pw[v]);
                        pb[rw * 128 + ((ch ^ (rw & 7)) << 4)] = (uint8_t)(u16 >> 8);
                        pb[(rw + 1) * 128 + ((ch ^ ((rw + 1) & 7)) << 4)] = (uint8_t)(u16 & 255u);
                    } else {
                        // p16 = 256 hi + lo with lo = the low byte read as a signed value: hi = (p16 + 128) >> 8
                        const int p16 = __float2int_rn(pw[v]);
                        pb[rw * 128 + ((ch ^ (rw & 7)) << 4)] = (uint8_t)((p16 + 128) >> 8);
                        pb[(rw + 1) * 128 + ((ch ^ ((rw + 1) & 7)) << 4)] = (uint8_t)p16;
                    }
                }
            }
        }
        if constexpr (VF != KV_Q8) {
            __syncthreads();  // S2b: the tiles as cached are in registers
            // per position and group 16 bytes, byte l = dims 32 c + l (low nibble) and 32 c + 16 + l (high): two 16-byte chunks of the
            // position's row of the operand (row = position, chunk = dims / 16 ^ (position % 8): the 128-byte swizzle)
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int vp = (tid >> 2) + 64 * k, c = tid & 3, rw = vp & 127;
                if ((k >> 1) < nh) {
                    const uint4 w = vraw[k];
                    uint8_t *dst = sm + C::VLEV + (vp >> 7) * 16384 + rw * 128;
                    *reinterpret_cast<uint4 *>(dst + (((2 * c) ^ (rw & 7)) << 4)) =
                        make_uint4(((w.x << 4) & 0xF0F0F0F0u) ^ 0x80808080u, ((w.y << 4) & 0xF0F0F0F0u) ^ 0x80808080u,
                                   ((w.z << 4) & 0xF0F0F0F0u) ^ 0x80808080u, ((w.w << 4) & 0xF0F0F0F0u) ^ 0x80808080u);
                    *reinterpret_cast<uint4 *>(dst + (((2 * c + 1) ^ (rw & 7)) << 4)) =
                        make_uint4((w.x & 0xF0F0F0F0u) ^ 0x80808080u, (w.y & 0xF0F0F0F0u) ^ 0x80808080u, (w.z & 0xF0F0F0F0u) ^ 0x80808080u,
                                   (w.w & 0xF0F0F0F0u) ^ 0x80808080u);
                }
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();  // S3
        if (tid == T_PV) {
            // ---- O^T += V^T (half h) P^T (half h): 4 k-steps of 32 keys per half
            tc_fence_after();
            if constexpr (VF == KV_Q8) ok = mbar_wait_bounded_quiet(bar_v, (uint32_t)it & 1u, err, 73) && ok;  // (the item's V levels have landed)
            constexpr uint32_t idesc_o = umma_idesc_i8(128, NO, 1, 0, 1, VF == KV_Q8 ? 0 : 1);
            for (int h = 0; h < nh; h++) {
#pragma unroll
                for (int ks = 0; ks < 4; ks++) {
                    // A: rows of 128 bytes (one position, all 128 dims = one swizzle atom along MN), 8 positions = 1024 bytes (SBO); 32 keys
                    // = 4096 bytes per k-step; B: the half's P^T rows, 32 keys = 32 bytes per k-step
                    const uint64_t da = umma_desc(sbase + C::VLEV + h * 16384 + ks * 4096, 16, 1024, 2);
                    const uint64_t db = umma_desc(sbase + C::PT + h * (NO * 128) + ks * 32, 16, 1024, 2);
                    umma_i8(tbase + C::O_COL, da, db, idesc_o, (h > 0) | (ks > 0));
                }
            }
            umma_commit(bar_o);
        }
        if (tid == T_ML) {  // m (in scaled-score units) and l of the block, for each vector
#pragma unroll
            for (int v = 0; v < NVT; v++)
                if (v < G) {
                    float *p = part + pidx + (long long)v * RQ_PSTRIDE(HD);
                    p[HD] = m[v] * scale;
                    p[HD + 1] = (float)reinterpret_cast<const unsigned *>(rb)[16 + v] * (1.0f / 8388608.0f);
                }
        }
        back_prev = ps_mine * (1.0f / PMAX);
        pidx_prev = pidx;
    }
    pdl_launch_dependents();
    if (!failed && warp < 4) store_o(cnt - 1, back_prev, pidx_prev, false);  // the last item's partial result
    if (failed && tid == T_MMA) {
        // a wait ran out: give what may still be in flight (the V levels of this item, the K tiles of the next, query planes,
        // the MMAs issued last) a bounded time to finish before the CTA's shared memory and TMEM are released
        mbar_drain(bar_v, (uint32_t)it & 1u);
        if (it + 1 < cnt) mbar_drain(bar_k, (uint32_t)(it + 1) & 1u);
        const TcdItem d = items[(it + (it + 1 < cnt ? 1 : 0)) & 3];
        mbar_drain(bar_q + (d.q & 1), (uint32_t)(d.q >> 1) & 1u);
        mbar_drain(bar_s, (uint32_t)it & 1u);
        if (it > 0) mbar_drain(bar_o, (uint32_t)(it - 1) & 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(C::TM_COLS));
}

template <int NVT, int KF, int VF>
static cudaError_t launch_tc_one(const AttnPartTcArgs &a, cudaStream_t stream) {
    constexpr int smem = TcdCfg<NVT, KF, VF>::SMEM;
    static_assert(smem <= 227 * 1024, "one CTA's shared memory");
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    auto kern = attn_part_tc_kernel<NVT, KF, VF>;
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    cudaError_t e = launch_pdl(tcd_q_prep_kernel, dim3(a.nrows, a.n_kv), dim3(128), 0, stream, a.rows, a.n_kv, a.G, a.q, a.qh, a.n_heads, a.qt, a.blk2row);
    if (e != cudaSuccess) return e;
    const long long items = (long long)a.total_blocks * a.n_kv, slots = (long long)a.n_sm * (NVT <= 4 ? 2 : 1);
    const int grid = (int)(items < slots ? items : slots);
    return launch_pdl(kern, dim3(grid), dim3(TCD_THREADS), (size_t)smem, stream, a.rows, (const int *)a.blk2row, (const uint8_t *)a.qt, a.maps, a.layer,
                      a.n_kv, a.G, a.n_heads, a.scale, a.part, a.total_blocks, a.err);
}
template <int KF, int VF>
static cudaError_t launch_tc_fmt(const AttnPartTcArgs &a, cudaStream_t stream) {
    if (a.G == 1) return launch_tc_one<1, KF, VF>(a, stream);
    if (a.G == 2) return launch_tc_one<2, KF, VF>(a, stream);
    if (a.G <= 4) return launch_tc_one<4, KF, VF>(a, stream);
    return launch_tc_one<8, KF, VF>(a, stream);
}

cudaError_t launch_attn_part_tc(const AttnPartTcArgs &a, cudaStream_t stream) {
    if (a.G < 1 || a.G > 8) return cudaErrorInvalidValue;
    switch (a.kvt) {
        case KV_Q8: return launch_tc_fmt<KV_Q8, KV_Q8>(a, stream);
        case KV_Q4: return launch_tc_fmt<KV_Q8, KV_Q4>(a, stream);
        case KV_Q4K4: return launch_tc_fmt<KV_Q4, KV_Q4>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}
#endif  // RQ_ATTN_DECODE_TC_INSTANTIATE

}  // namespace rq
