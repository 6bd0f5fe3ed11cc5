// librq_cuda: host side of the C ABI declared in include/rq_cuda.h — contexts, device-resident sequences, the open
// pass, and the launches of the kernels in this directory.  No PyTorch, no CPU fallback: every compute entry point
// needs a CUDA device and fails with RQ_CUDA_ERR_DEVICE otherwise.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <functional>
#include <atomic>
#include <new>
#include <string>
#include <vector>

#include "../../include/rq_cuda.h"
#include "attn_decode.cuh"
#include "attn_decode_tc.cuh"
#include "attn_prefill256.cuh"
#include "deltanet.cuh"
#include "deltanet_chunk.cuh"
#include "kv_dequant.cuh"
#include "kv_store.cuh"

using namespace rq;

namespace rq {
extern template cudaError_t launch_attn_part<KV_F16>(int, const AttnPartArgs &, cudaStream_t);
extern template cudaError_t launch_attn_part<KV_Q8>(int, const AttnPartArgs &, cudaStream_t);
extern template cudaError_t launch_attn_part<KV_Q4>(int, const AttnPartArgs &, cudaStream_t);
extern template cudaError_t launch_attn_part<KV_Q4K4>(int, const AttnPartArgs &, cudaStream_t);
extern template size_t attn_part_smem<KV_F16>(int, int);
extern template size_t attn_part_smem<KV_Q8>(int, int);
extern template size_t attn_part_smem<KV_Q4>(int, int);
extern template size_t attn_part_smem<KV_Q4K4>(int, int);
}  // namespace rq

struct RqCudaSeq {
    RqCuda *ctx;
    int cap, kv_len, kvt, len;
    uint8_t *k, *v;        // [n_attn] layers of kv_len / 16 * n_kv_local tiles
    size_t lk, lv;         // bytes per layer
    float *ssm;            // [n_lin] layers of ssm_floats
    size_t ssm_floats;
    // DeltaNet state checkpoints (RqSeq.ck, reference src/internal.h:383): slot buffers of the whole layered state, allocated
    // at first use, and the length each holds the state of (-1: none)
    std::vector<float *> ck_st;
    std::vector<int> ck_pos;
    int in_pass;
    unsigned long long stamp;  // number of the last pass_begin that listed this sequence (duplicate check)
    bool dead;                 // rq_cuda_seq_free was called while the sequence belonged to the open pass: freed at pass_end
    // 2-D views of the K and V caches for the tensor-core prefill kernels (f16, head_dim 128 / 256); q8 at head_dim 128: tm_v is
    // the 3-D view of the V levels for the tensor-core decode kernel (has_tm_q8)
    CUtensorMap tm_k, tm_v, tm_ks, tm_vs;  // (tm_ks, tm_vs: the scales behind each tile's levels, q8 only)
    bool has_tm, has_tm_q8;
};

struct RqCuda {
    int device;
    int n_sm = 0;  // SMs of the device
    RqCudaModel m;
    int n_kv, n_heads, G, qh;  // local (this device's) KV heads / query heads, vectors per KV head, floats per q head row
    int max_rows;
    WoQuant wo_quant;  // rq_cuda_set_wo_quant: the merge kernels also leave int8 levels + scales of their output rows
    int exact;  // rq_cuda_set_exact: quantised caches take the bit-exact CUDA-core kernels instead of the tensor-core ones
    cudaStream_t own_stream, stream;
    cudaEvent_t ev0, ev1;
    // rq_cuda_pass_timing: events around every pass, and what the reference's cost model multiplies (seg_cost, engine.c:2631)
    cudaEvent_t ev_p0, ev_p1;
    int pass_timing, pass_timed, pt_rows;
    double pt_first, pt_more;
    char err[256];
    unsigned long long launches;
    // the open pass
    int pass_open, nrows, nseg, total_blocks, pass_kvt, max_np;
    unsigned long long pass_no;  // counts pass_begin calls (RqCudaSeq::stamp)
    std::vector<RqCudaSegment> segs;
    PassRow *h_rows, *d_rows;  // nrows + 1 entries (the last one holds the total block count)
    DnSeg *h_dseg, *d_dseg;
    // the DeltaNet tables of the open pass (segments, chunks, checkpoints) are made by the first DeltaNet call of the pass,
    // after the host has named the pass's checkpoints
    struct PassCk { int seg, row, slot; };
    std::vector<PassCk> pass_ck;
    DnChunk *h_chunk2[2], *d_chunks;
    DnCk *h_ck2[2], *d_ck;
    int dn_ready, dn_used, max_chunks_cap;
    // the pinned tables are double-buffered: a pass fills the half the pass before the previous one used, after that
    // half's upload (an event) is known to be complete, so opening a pass never waits for the device
    PassRow *h_rows2[2];
    DnSeg *h_dseg2[2];
    cudaEvent_t up_ev[2];
    static constexpr int MAX_PASS_CK = 1024;  // checkpoints one pass may take, all segments together
    int up_idx;
    // scratch, grown on demand
    float *d_part;  size_t part_bytes;
    uint8_t *d_tcq; size_t tcq_bytes;    // tensor-core decode over quantised caches: the prepared query tiles ...
    int *d_blk2row; size_t blk2row_bytes;  // ... and the block -> row table of the pass
    float *d_q;     size_t q_bytes;     // staging of host q rows
    float *d_out;   size_t out_bytes;   // staging of outputs
    float *d_k, *d_v; size_t k_bytes, v_bytes;  // staging of host K / V rows
    float *d_dn;    size_t dn_bytes;    // staging of DeltaNet rows
    int *d_err;
    int *h_err;  // pinned
    int *err_fwd = nullptr;  // set around a launch whose merge kernel should store the status word to h_err itself
    // tensor-core prefill: the segments' tensor maps and the work list of the open pass
    CUtensorMap *h_maps, *d_maps;  // [max_rows][2]
    CUtensorMap *h_maps8, *d_maps8;  // [max_rows][4]: the q8 views of the tensor-core decode kernel
    PfWork *d_work; size_t work_bytes;
    std::vector<PfWork> h_work;
    int pf_ready, pf_max_splits;
    int pf_split = PF_SPLIT;  // key positions per split of the open pass's prefill work items
    int pf_split_fixed = 0;   // non-zero: the host fixed the split length (rq_cuda_set_prefill_split)
    // head-sharded contexts: the gather of the output rows fused into the merge kernel (rq_cuda_peer_*): this rank's buffer
    // (1 KB of flags, then two full-width row buffers used in turn) and the peers' mappings of theirs
    uint8_t *peer_own = nullptr;
    uint8_t *peer_base[RQ_MAX_PEERS] = {nullptr};
    size_t peer_rows_bytes = 0;
    int peer_rank = 0, peer_world = 0, peer_max_rows = 0;
    unsigned peer_step = 0;
    bool peer_now = false;  // the launch in progress stores to the peers
    // ... over quantised caches: the layer's tiles expanded to f16 in a scratch (pf_quant: the open pass takes that route)
    bool pf_quant = false;
    uint8_t *d_dq = nullptr; size_t dq_bytes = 0;   // the f16 tiles, K then V per segment
    float *d_qrot = nullptr; size_t qrot_bytes = 0;  // the rotated query rows
    DqSeg *d_dqseg = nullptr; size_t dqseg_bytes = 0;
    std::vector<DqSeg> h_dqseg;
    int dq_max_tiles = 0;
    // a quantised prompt pass is routed by segment: segments of 16 rows or more through the expansion + the tensor-core prefill
    // kernel (runs of their rows: pf_runs_p), the others (decode rows riding in the same pass) through the decode kernels, run by
    // run of adjacent rows, over a copy of their PassRow entries whose block numbers count from the run's first row
    struct RowRun { int row0, nrows, blocks, table0; size_t part0; };
    std::vector<RowRun> pf_runs_p, pf_runs_d;
    PassRow *d_rows_d = nullptr; size_t rows_d_bytes = 0;
    std::vector<PassRow> h_rows_d;
    size_t pf_part_d = 0;  // floats of partial records the decode runs need, behind the prefill kernel's
    // the rows a decode launch covers when it is not the whole pass (span_rows non-null)
    const PassRow *span_rows = nullptr;
    int span_nrows = 0, span_blocks = 0;
    int tc_ready;  // the open pass's tensor maps for the tensor-core decode kernel are on the device (1), or it does not qualify (-1)
    // DeltaNet weights of the steps around the recurrence (rq_cuda_dn_set_weights): per linear layer conv taps, A, dt
    // bias, norm weight
    float *d_dnw; size_t dnw_layer_floats;
    int dn_chunks;                         // chunks (of at most 64 tokens) of the open pass, all segments
    uint8_t *d_dnwork; size_t dnwork_bytes;  // the chunked DeltaNet's work records
    std::vector<char> dnw_set;
    // optional per-launch timing of the dominant kernel (rq_cuda_profile_begin / _end)
    std::vector<cudaEvent_t> prof_ev;
    int prof_on, prof_n;
};

static int fail(RqCuda *c, int code, const char *fmt, ...) {
    if (c) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(c->err, sizeof(c->err), fmt, ap);
        va_end(ap);
    }
    return code;
}
#define CU(c, call)                                                                                          \
    do {                                                                                                     \
        cudaError_t e_ = (call);                                                                             \
        if (e_ != cudaSuccess)                                                                               \
            return fail(c, e_ == cudaErrorMemoryAllocation ? RQ_CUDA_ERR_NOMEM : RQ_CUDA_ERR_DEVICE, "%s: %s", #call, \
                        cudaGetErrorString(e_));                                                             \
    } while (0)

typedef CUresult (*TmEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                               const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TmEncodeFn tm_encode() {
    // the driver's tensor-map encoder, looked up through the runtime (no link-time dependency on libcuda)
    static TmEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        cudaDriverEntryPointQueryResult qr;
        void *p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            fn = (TmEncodeFn)p;
    }
    return fn;
}

static bool seq_make_maps(RqCuda *c, RqCudaSeq *s) {
    // K: rows of 16 positions x one dim (32 bytes), 32-byte swizzle, box 16 x 256 (two tiles of head_dim 128) or 16 x 128 (the
    // 128-dim half of one tile of head_dim 256);
    // V: rows of one position x head_dim dims (256 or 512 bytes), 128-byte swizzle, box 64 x 128
    s->has_tm = s->has_tm_q8 = false;
    const int hd = c->m.head_dim;
    if (s->kvt == KV_Q8 && hd == 128 && c->m.n_attn >= 1) {
        // The V levels of a q8 cache as the tensor-core decode kernel wants them in shared memory: half a block of one head (8 tiles)
        // as 128 rows (positions) of 128 bytes with the 128-byte swizzle, an MN-major MMA operand: {128 dims, 16 positions, tiles}
        // with strides {128, tile bytes}, box 128 x 16 x 8.
        TmEncodeFn enc8 = tm_encode();
        if (!enc8) return false;
        const cuuint64_t tb = kv_tile_bytes(KV_Q8, 128, 0), tiles = (cuuint64_t)(s->lk * c->m.n_attn / tb);
        cuuint32_t es3[3] = {1, 1, 1};
        const auto u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
        const auto il = CU_TENSOR_MAP_INTERLEAVE_NONE;
        const auto l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
        const auto oob = CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE;
        {
            cuuint64_t dims[3] = {128, 16, tiles}, strides[2] = {128, tb};
            cuuint32_t box[3] = {128, 16, 8};
            if (enc8(&s->tm_v, u8, 3, s->v, dims, strides, box, es3, il, CU_TENSOR_MAP_SWIZZLE_128B, l2, oob) != CUDA_SUCCESS) return false;
        }
        s->tm_k = s->tm_ks = s->tm_vs = s->tm_v;  // (only the V view is used: the K tiles and the scales go by plain bulk copies)
        s->has_tm_q8 = true;
        return true;
    }
    if (kv_quant(s->kvt) && hd == 128 && c->m.n_attn >= 1) {
        // (4-bit V levels go to the tensor-core decode kernel by plain bulk copies: no view needed)
        memset(&s->tm_v, 0, sizeof s->tm_v);
        s->tm_k = s->tm_ks = s->tm_vs = s->tm_v;
        s->has_tm_q8 = true;
        return true;
    }
    if (s->kvt != KV_F16 || (hd != 128 && hd != 256) || c->m.n_attn < 1) return true;
    TmEncodeFn enc = tm_encode();
    if (!enc) return false;
    cuuint32_t es[2] = {1, 1};
    {
        cuuint64_t dims[2] = {16, (cuuint64_t)(s->lk * c->m.n_attn / 32)}, strides[1] = {32};
        cuuint32_t box[2] = {16, hd == 128 ? 256u : 128u};
        if (enc(&s->tm_k, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, s->k, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)(s->lv * c->m.n_attn / (2 * hd))}, strides[1] = {(cuuint64_t)(2 * hd)};
        cuuint32_t box[2] = {64, 128};
        if (enc(&s->tm_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, s->v, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    s->has_tm = true;
    return true;
}

static bool kvt_ok(int t, int hd) {
    if (t == KV_F16) return hd == 64 || hd == 128 || hd == 256;
    return kv_quant(t) && (hd == 64 || hd == 128 || hd == 256);
}

static int grow(RqCuda *c, void **p, size_t *have, size_t need) {
    // device scratch of at least `need` bytes (contents not kept)
    if (*have >= need) return RQ_CUDA_OK;
    CU(c, cudaStreamSynchronize(c->stream));
    if (*p) cudaFree(*p);
    *p = nullptr;
    *have = 0;
    size_t sz = need + need / 4;
    CU(c, cudaMalloc(p, sz));
    *have = sz;
    return RQ_CUDA_OK;
}

// A one-CTA kernel whose only work is a bounded wait on an mbarrier that nothing ever arrives at: the wait runs out after
// `limit_ns`, records `code` in the status word and the kernel returns by itself (rq_cuda_selftest_wait_expiry).
__global__ void wait_expiry_kernel(int *err, unsigned long long limit_ns, int code) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    mbar_wait_bounded_ns(&bar, 0, err, code, limit_ns);
}

// After a merge kernel that stored this rank's heads into every rank's row buffer: lane p tells rank p that this rank's part of
// step `step` is in place (a system-scope release store into rank p's flag word of this rank), then waits until rank p has told
// this rank the same, with a time limit: a rank that never arrives makes the wait run out, the kernel records `code` in the
// status word and returns by itself.  One warp; launched as an ordinary kernel, so the merge kernel before it has completed.
struct PeerFlags {
    unsigned *flags[RQ_MAX_PEERS];  // rank p's flag words [RQ_MAX_PEERS]; [rank]: this rank's own
};
__global__ void peer_sync_kernel(PeerFlags pf, int rank, int world, unsigned step, int *err, unsigned long long limit_ns, int code) {
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf.flags[p] + rank), "r"(step) : "memory");
    const unsigned *mine = pf.flags[rank] + p;
    unsigned long long t0 = 0;
    for (long long it = 0;; it++) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int)(v - step) >= 0) return;
        if ((it & 63) == 63) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            if (now - t0 > limit_ns) break;
        }
    }
    atomicExch(err, code);
}

extern "C" {

int rq_cuda_debug_build(void) {
#ifdef RQ_DEBUG
    return 1;
#else
    return 0;
#endif
}

int rq_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}

int rq_cuda_init(int device, const RqCudaModel *model, int max_rows, RqCuda **ctx) {
    if (!ctx) return RQ_CUDA_ERR_ARG;
    *ctx = nullptr;
    if (!model || max_rows < 1 || max_rows > 16384) return RQ_CUDA_ERR_ARG;
    const RqCudaModel &m = *model;
    int nkv_local = m.kv_heads_local > 0 ? m.kv_heads_local : m.n_kv_heads;
    if (m.n_attn < 0 || m.n_lin < 0 || (m.n_attn == 0 && m.n_lin == 0)) return RQ_CUDA_ERR_ARG;
    if (m.n_attn > 0) {
        if (m.n_kv_heads < 1 || m.n_heads < 1 || m.n_heads % m.n_kv_heads) return RQ_CUDA_ERR_ARG;
        if (m.n_heads / m.n_kv_heads > 8) return RQ_CUDA_ERR_ARG;  // query heads per KV head the kernels are built for
        if (m.head_dim != 64 && m.head_dim != 128 && m.head_dim != 256) return RQ_CUDA_ERR_ARG;
        if (m.kv_head0 < 0 || nkv_local < 1 || m.kv_head0 + nkv_local > m.n_kv_heads) return RQ_CUDA_ERR_ARG;
    }
    if (m.n_lin > 0) {
        if (m.dn_nk < 1 || m.dn_nv < 1 || m.dn_nv % m.dn_nk || m.dn_dk != 128 || m.dn_dv < 32 || m.dn_dv % 32 ||
            m.dn_conv < 2)
            return RQ_CUDA_ERR_ARG;
        // the DeltaNet kernels read rows with 16-byte loads: a row of 2 nk dk + 2 nv dv + 2 nv floats has to be a multiple
        // of 4 floats (an even number of value heads)
        if ((2 * m.dn_nk * m.dn_dk + 2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv) % 4) return RQ_CUDA_ERR_ARG;
    }
    int ndev = rq_cuda_device_count();
    if (ndev < 1 || device < 0 || device >= ndev) return RQ_CUDA_ERR_DEVICE;
    if (cudaSetDevice(device) != cudaSuccess) return RQ_CUDA_ERR_DEVICE;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return RQ_CUDA_ERR_DEVICE;
    if (prop.major != 10) return RQ_CUDA_ERR_DEVICE;  // the kernels are sm_100a only
    RqCuda *c = new (std::nothrow) RqCuda();
    if (!c) return RQ_CUDA_ERR_NOMEM;
    c->device = device;
    c->n_sm = prop.multiProcessorCount;
    c->m = m;
    c->n_kv = m.n_attn ? nkv_local : 0;
    c->G = m.n_attn ? m.n_heads / m.n_kv_heads : 0;
    c->n_heads = c->n_kv * c->G;
    c->qh = (m.gated ? 2 : 1) * m.head_dim;
    c->max_rows = max_rows;
    c->exact = 0;
    c->err[0] = 0;
    bool okk = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking) == cudaSuccess &&
               cudaEventCreate(&c->ev0) == cudaSuccess && cudaEventCreate(&c->ev1) == cudaSuccess &&
               cudaEventCreate(&c->ev_p0) == cudaSuccess && cudaEventCreate(&c->ev_p1) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_rows2[0], sizeof(PassRow) * (max_rows + 1)) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_rows2[1], sizeof(PassRow) * (max_rows + 1)) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_dseg2[0], sizeof(DnSeg) * max_rows) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_dseg2[1], sizeof(DnSeg) * max_rows) == cudaSuccess &&
               cudaEventCreateWithFlags(&c->up_ev[0], cudaEventDisableTiming) == cudaSuccess &&
               cudaEventCreateWithFlags(&c->up_ev[1], cudaEventDisableTiming) == cudaSuccess &&
               cudaMalloc((void **)&c->d_rows, sizeof(PassRow) * (max_rows + 1)) == cudaSuccess &&
               cudaMalloc((void **)&c->d_dseg, sizeof(DnSeg) * max_rows) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_chunk2[0], sizeof(DnChunk) * (max_rows + RqCuda::MAX_PASS_CK)) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_chunk2[1], sizeof(DnChunk) * (max_rows + RqCuda::MAX_PASS_CK)) == cudaSuccess &&
               cudaMalloc((void **)&c->d_chunks, sizeof(DnChunk) * (max_rows + RqCuda::MAX_PASS_CK)) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_ck2[0], sizeof(DnCk) * RqCuda::MAX_PASS_CK) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_ck2[1], sizeof(DnCk) * RqCuda::MAX_PASS_CK) == cudaSuccess &&
               cudaMalloc((void **)&c->d_ck, sizeof(DnCk) * RqCuda::MAX_PASS_CK) == cudaSuccess &&
               cudaMalloc((void **)&c->d_err, sizeof(int)) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_err, sizeof(int)) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_maps, sizeof(CUtensorMap) * 2 * max_rows) == cudaSuccess &&
               cudaMalloc((void **)&c->d_maps, sizeof(CUtensorMap) * 2 * max_rows) == cudaSuccess &&
               cudaMallocHost((void **)&c->h_maps8, sizeof(CUtensorMap) * 4 * max_rows) == cudaSuccess &&
               cudaMalloc((void **)&c->d_maps8, sizeof(CUtensorMap) * 4 * max_rows) == cudaSuccess &&
               cudaMemset(c->d_err, 0, sizeof(int)) == cudaSuccess;
    c->stream = c->own_stream;
    if (!okk) {
        rq_cuda_free(c);
        return RQ_CUDA_ERR_DEVICE;
    }
    *ctx = c;
    return RQ_CUDA_OK;
}

void rq_cuda_free(RqCuda *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (int p = 0; p < c->peer_world; p++)
        if (p != c->peer_rank && c->peer_base[p]) cudaIpcCloseMemHandle(c->peer_base[p]);
    if (c->peer_own) cudaFree(c->peer_own);
    if (c->d_dnw) cudaFree(c->d_dnw);
    if (c->h_maps8) cudaFreeHost(c->h_maps8);
    void *dev[] = {c->d_rows_d, c->d_dq, c->d_qrot, c->d_dqseg, c->d_maps8, c->d_tcq, c->d_blk2row, c->d_chunks, c->d_ck, c->d_rows, c->d_dseg, c->d_part, c->d_q, c->d_out, c->d_k, c->d_v, c->d_dn, c->d_err, c->d_maps, c->d_work, c->d_dnwork};
    if (c->h_maps) cudaFreeHost(c->h_maps);
    for (void *p : dev)
        if (p) cudaFree(p);
    for (int i = 0; i < 2; i++) {
        if (c->h_rows2[i]) cudaFreeHost(c->h_rows2[i]);
        if (c->h_dseg2[i]) cudaFreeHost(c->h_dseg2[i]);
        if (c->h_chunk2[i]) cudaFreeHost(c->h_chunk2[i]);
        if (c->h_ck2[i]) cudaFreeHost(c->h_ck2[i]);
        if (c->up_ev[i]) cudaEventDestroy(c->up_ev[i]);
    }
    if (c->h_err) cudaFreeHost(c->h_err);
    for (cudaEvent_t ev : c->prof_ev) cudaEventDestroy(ev);
    if (c->ev_p0) cudaEventDestroy(c->ev_p0);
    if (c->ev_p1) cudaEventDestroy(c->ev_p1);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
}

const char *rq_cuda_error(const RqCuda *c) { return c ? c->err : "no context"; }

int rq_cuda_sync(RqCuda *c) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    if (*c->h_err) {
        int code = *c->h_err;
        cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream);
        return fail(c, RQ_CUDA_ERR_STATE, "a device-side wait expired (code %d): results of the last pass are invalid", code);
    }
    return RQ_CUDA_OK;
}

int rq_cuda_selftest_wait_expiry(RqCuda *c, unsigned int limit_us) {
    if (!c || limit_us < 1 || limit_us > 1000000) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    wait_expiry_kernel<<<1, 32, 0, c->stream>>>(c->d_err, (unsigned long long)limit_us * 1000ull, 99);
    c->launches++;
    CU(c, cudaGetLastError());
    return RQ_CUDA_OK;
}

int rq_cuda_peer_export(RqCuda *c, int rows, void *handle64) {
    if (!c || !handle64 || rows < 1 || rows > c->max_rows) return c ? fail(c, RQ_CUDA_ERR_ARG, "peer_export: %d rows", rows) : RQ_CUDA_ERR_ARG;
    if (c->peer_own) return fail(c, RQ_CUDA_ERR_STATE, "peer_export: already exported");
    if (c->m.n_attn < 1) return fail(c, RQ_CUDA_ERR_ARG, "peer_export: no attention layers");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
    CU(c, cudaSetDevice(c->device));
    c->peer_rows_bytes = ((size_t)rows * c->m.n_heads * c->m.head_dim * 4 + 255) & ~(size_t)255;
    CU(c, cudaMalloc((void **)&c->peer_own, 1024 + 2 * c->peer_rows_bytes));
    CU(c, cudaMemset(c->peer_own, 0, 1024 + 2 * c->peer_rows_bytes));
    CU(c, cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    CU(c, cudaIpcGetMemHandle(&h, c->peer_own));
    memcpy(handle64, &h, 64);
    c->peer_max_rows = rows;
    return RQ_CUDA_OK;
}

int rq_cuda_peer_import(RqCuda *c, int rank, int world, const void *handles) {
    if (!c || !handles || world < 1 || world > RQ_MAX_PEERS || rank < 0 || rank >= world)
        return c ? fail(c, RQ_CUDA_ERR_ARG, "peer_import: rank %d of %d", rank, world) : RQ_CUDA_ERR_ARG;
    if (!c->peer_own || c->peer_world) return fail(c, RQ_CUDA_ERR_STATE, "peer_import: export first, import once");
    CU(c, cudaSetDevice(c->device));
    for (int p = 0; p < world; p++) {
        if (p == rank) {
            c->peer_base[p] = c->peer_own;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + 64 * (size_t)p, 64);
        void *ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int x = 0; x < p; x++)
                if (x != rank && c->peer_base[x]) cudaIpcCloseMemHandle(c->peer_base[x]), c->peer_base[x] = nullptr;
            return fail(c, RQ_CUDA_ERR_DEVICE, "peer_import: rank %d's buffer: %s", p, cudaGetErrorString(e));
        }
        c->peer_base[p] = (uint8_t *)ptr;
    }
    c->peer_rank = rank, c->peer_world = world;
    return RQ_CUDA_OK;
}

int rq_cuda_selftest_peer_wait(RqCuda *c, unsigned int limit_us) {
    // a two-rank exchange whose other rank never arrives: both flag arrays are this context's own, nothing sets word [1]
    if (!c || limit_us < 1 || limit_us > 1000000) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    unsigned *fl = nullptr;
    CU(c, cudaMalloc((void **)&fl, 1024));
    CU(c, cudaMemsetAsync(fl, 0, 1024, c->stream));
    PeerFlags pf;
    memset(&pf, 0, sizeof pf);
    pf.flags[0] = fl, pf.flags[1] = fl + 64;
    peer_sync_kernel<<<1, 32, 0, c->stream>>>(pf, 0, 2, 1u, c->d_err, (unsigned long long)limit_us * 1000ull, 97);
    c->launches++;
    cudaError_t e = cudaGetLastError();
    cudaStreamSynchronize(c->stream);
    cudaFree(fl);
    CU(c, e);
    return RQ_CUDA_OK;
}

int rq_cuda_reserve(RqCuda *c, int rows, long long positions_total, int max_ctx) {
    if (!c || rows < 1 || rows > c->max_rows || positions_total < rows || max_ctx < 1) return c ? fail(c, RQ_CUDA_ERR_ARG, "reserve: %d rows", rows) : RQ_CUDA_ERR_ARG;
    if (c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "reserve: a pass is open");
    CU(c, cudaSetDevice(c->device));
    int rc = RQ_CUDA_OK;
    if (c->m.n_attn > 0) {
        const size_t rec = (size_t)c->n_heads * RQ_PSTRIDE(c->m.head_dim) * 4;
        const size_t blocks = (size_t)(positions_total / ATT_P) + rows;                       // decode: a record per 256-position block
        const size_t splits = (size_t)rows * ((max_ctx + PF_SPLIT_MIN - 1) / PF_SPLIT_MIN);   // prefill: a record per (row, split)
        const size_t need = std::max(blocks, splits) * rec;
        if (need > ((size_t)8 << 30)) return fail(c, RQ_CUDA_ERR_ARG, "reserve: %zu MB of partial results", need >> 20);
        const size_t qb = (size_t)rows * c->n_heads * c->qh * 4, ob = (size_t)rows * c->n_heads * c->m.head_dim * 4;
        const size_t kb = (size_t)rows * c->n_kv * c->m.head_dim * 4;
        if ((rc = grow(c, (void **)&c->d_part, &c->part_bytes, need))) return rc;
        if ((rc = grow(c, (void **)&c->d_q, &c->q_bytes, qb))) return rc;
        if ((rc = grow(c, (void **)&c->d_out, &c->out_bytes, ob))) return rc;
        if ((rc = grow(c, (void **)&c->d_k, &c->k_bytes, kb))) return rc;
        if ((rc = grow(c, (void **)&c->d_v, &c->v_bytes, kb))) return rc;
        if (c->m.head_dim == 128) {
            // quantised caches on the tensor cores: the query planes and the block -> row table of a decode pass; the rotated
            // query rows of a prompt pass (its f16 expansion of the cache tiles is sized by the pass itself: up to 8 KB per
            // 16 cached positions and KV head of the segments)
            if ((rc = grow(c, (void **)&c->d_tcq, &c->tcq_bytes, (size_t)rows * c->n_kv * TCD_QT_BYTES))) return rc;
            if ((rc = grow(c, (void **)&c->d_blk2row, &c->blk2row_bytes, blocks * sizeof(int)))) return rc;
            if ((rc = grow(c, (void **)&c->d_qrot, &c->qrot_bytes, (size_t)rows * c->n_heads * 128 * 4))) return rc;
        }
    }
    if (c->m.n_lin > 0) {
        const RqCudaModel &m = c->m;
        const size_t lw = (size_t)2 * m.dn_nk * m.dn_dk + (size_t)2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv;
        if ((rc = grow(c, (void **)&c->d_dn, &c->dn_bytes, (size_t)rows * (lw + (size_t)m.dn_nv * m.dn_dv) * 4))) return rc;
    }
    return RQ_CUDA_OK;
}

int rq_cuda_set_prefill_split(RqCuda *c, int positions) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (positions != 0 && (positions < PF_SPLIT_MIN || positions % PF_BN || positions > (1 << 20)))
        return fail(c, RQ_CUDA_ERR_ARG, "set_prefill_split: %d positions (0, or a multiple of %d from %d on)", positions, PF_BN, PF_SPLIT_MIN);
    if (c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "set_prefill_split: a pass is open");
    c->pf_split_fixed = positions;
    return RQ_CUDA_OK;
}

int rq_cuda_set_wo_quant(RqCuda *c, int gs, signed char *xq_dev, float *xs_dev) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (!xq_dev && !xs_dev) {
        c->wo_quant = WoQuant{nullptr, nullptr, 0};
        return RQ_CUDA_OK;
    }
    if (!xq_dev || !xs_dev || c->m.n_attn < 1 || (gs != 32 && gs != 64 && gs != 128 && gs != 256) || c->m.head_dim % gs)
        return fail(c, RQ_CUDA_ERR_ARG, "set_wo_quant: groups of %d values (head_dim %d)", gs, c->m.head_dim);
    if (((uintptr_t)xq_dev & 3) || ((uintptr_t)xs_dev & 3)) return fail(c, RQ_CUDA_ERR_ARG, "set_wo_quant: pointers must be 4-byte aligned");
    c->wo_quant = WoQuant{(int8_t *)xq_dev, xs_dev, gs};
    return RQ_CUDA_OK;
}

int rq_cuda_pass_timing(RqCuda *c, int on) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "pass_timing: a pass is open");
    c->pass_timing = on != 0;
    c->pass_timed = 0;
    return RQ_CUDA_OK;
}

int rq_cuda_pass_time(RqCuda *c, RqCudaPassTime *out) {
    if (!c || !out) return RQ_CUDA_ERR_ARG;
    if (!c->pass_timing || !c->pass_timed) return fail(c, RQ_CUDA_ERR_STATE, "pass_time: no timed pass has been closed (rq_cuda_pass_timing)");
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaEventSynchronize(c->ev_p1));
    float ms = 0.0f;
    CU(c, cudaEventElapsedTime(&ms, c->ev_p0, c->ev_p1));
    out->seconds = ms * 1e-3;
    out->rows = c->pt_rows;
    out->pos_first = c->pt_first;
    out->pos_more = c->pt_more;
    return RQ_CUDA_OK;
}

int rq_cuda_pass_cost_measure(RqCuda *c, RqCudaSeq *s, int L, int reps, double *t_w, double *att, double *att_x) {
    if (!c || !s || s->ctx != c || !t_w || !att || !att_x) return RQ_CUDA_ERR_ARG;
    if (c->m.n_attn < 1 || L < 64 || L + 16 > s->cap || reps < 1 || c->max_rows < 16) return fail(c, RQ_CUDA_ERR_ARG, "pass_cost_measure: context %d (capacity %d)", L, s->cap);
    if (c->pass_open || s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "pass_cost_measure: a pass is open");
    int rc;
    if ((rc = rq_cuda_seq_fill_synthetic(s, L + 16, 12345))) return rc;
    const size_t qb = (size_t)16 * c->n_heads * c->qh * 4, ob = (size_t)16 * c->n_heads * c->m.head_dim * 4;
    if ((rc = grow(c, (void **)&c->d_q, &c->q_bytes, qb))) return rc;
    if ((rc = grow(c, (void **)&c->d_out, &c->out_bytes, ob))) return rc;
    CU(c, cudaMemsetAsync(c->d_q, 0, qb, c->stream));
    const int keep = c->pass_timing;
    c->pass_timing = 1;
    // the fastest of `reps` passes over all attention layers: one row at L / 2, one row at L, a segment of 16 rows at L
    auto run = [&](int pos0, int n, double *secs) -> int {
        double best = 1e30;
        for (int r = 0; r < reps + 1; r++) {  // (the first one warms the kernels up)
            RqCudaSegment g = {s, pos0, n};
            int e = rq_cuda_pass_begin(c, &g, 1);
            for (int l = 0; l < c->m.n_attn && !e; l++) e = n == 1 ? rq_cuda_attn_decode_dev(c, l, c->d_q, c->d_out) : rq_cuda_attn_prefill_dev(c, l, c->d_q, c->d_out);
            if (c->pass_open) rq_cuda_pass_end(c, 0);
            RqCudaPassTime t;
            if (!e) e = rq_cuda_pass_time(c, &t);
            if (e) return e;
            if (r > 0 && t.seconds < best) best = t.seconds;
        }
        *secs = best;
        return RQ_CUDA_OK;
    };
    double t_half = 0, t_one = 0, t_16 = 0;
    rc = run(L / 2, 1, &t_half);
    if (!rc) rc = run(L, 1, &t_one);
    if (!rc) rc = run(L, 16, &t_16);
    c->pass_timing = keep;
    rq_cuda_seq_truncate(s, 0);
    if (rc) return rc;
    // t(1 row at p) = t_w + att p;  t(16 rows at L) = t_w + att L + att_x sum of the 15 further positions
    *att = std::max(0.0, (t_one - t_half) / (double)(L - L / 2));
    *t_w = std::max(0.0, t_one - *att * L);
    *att_x = std::max(0.0, (t_16 - t_one) / (15.0 * L + 15.0 * 16.0 / 2.0));
    return RQ_CUDA_OK;
}

int rq_cuda_set_exact(RqCuda *c, int exact) {
    if (!c) return RQ_CUDA_ERR_ARG;
    c->exact = exact != 0;
    return RQ_CUDA_OK;
}

int rq_cuda_set_stream(RqCuda *c, void *s) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaStreamSynchronize(c->stream));
    c->stream = s ? (cudaStream_t)s : c->own_stream;
    return RQ_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------- sequences
int rq_cuda_seq_new(RqCuda *c, int capacity, int kv_type, RqCudaSeq **seq) {
    if (!c || !seq) return RQ_CUDA_ERR_ARG;
    *seq = nullptr;
    if (capacity < 1) return fail(c, RQ_CUDA_ERR_ARG, "capacity %d", capacity);
    if (c->m.n_attn > 0 && !kvt_ok(kv_type, c->m.head_dim))
        return fail(c, RQ_CUDA_ERR_ARG, "KV type %d with head_dim %d is not supported on the device", kv_type, c->m.head_dim);
    CU(c, cudaSetDevice(c->device));
    RqCudaSeq *s = new (std::nothrow) RqCudaSeq();
    if (!s) return fail(c, RQ_CUDA_ERR_NOMEM, "host allocation");
    s->ctx = c;
    s->cap = capacity;
    s->kv_len = (capacity + ATT_P - 1) / ATT_P * ATT_P;
    s->kvt = kv_type;
    if (c->m.n_attn > 0) {
        s->lk = (size_t)(s->kv_len / ATT_T) * c->n_kv * kv_tile_bytes(kv_type, c->m.head_dim, 0);
        s->lv = (size_t)(s->kv_len / ATT_T) * c->n_kv * kv_tile_bytes(kv_type, c->m.head_dim, 1);
        cudaError_t e1 = cudaMalloc((void **)&s->k, s->lk * c->m.n_attn);
        cudaError_t e2 = e1 == cudaSuccess ? cudaMalloc((void **)&s->v, s->lv * c->m.n_attn) : e1;
        if (e1 != cudaSuccess || e2 != cudaSuccess) {
            cudaGetLastError();
            rq_cuda_seq_free(s);
            return fail(c, RQ_CUDA_ERR_NOMEM, "KV cache of %zu bytes: %s", (s->lk + s->lv) * c->m.n_attn,
                        cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
        }
        // zeroed: positions past a row's length are masked, but the tensor-core kernels multiply them by zero weights
        // and must not meet a NaN or infinity bit pattern there
        cudaMemsetAsync(s->k, 0, s->lk * c->m.n_attn, c->stream);
        cudaMemsetAsync(s->v, 0, s->lv * c->m.n_attn, c->stream);
        if (!seq_make_maps(c, s)) {
            rq_cuda_seq_free(s);
            return fail(c, RQ_CUDA_ERR_DEVICE, "tensor maps of the KV cache could not be encoded");
        }
    }
    if (c->m.n_lin > 0) {
        size_t convf = ((size_t)(c->m.dn_conv - 1) * (2 * c->m.dn_nk * c->m.dn_dk + c->m.dn_nv * c->m.dn_dv) + 15) / 16 * 16;
        s->ssm_floats = convf + (size_t)c->m.dn_nv * c->m.dn_dk * c->m.dn_dv;
        cudaError_t e = cudaMalloc((void **)&s->ssm, s->ssm_floats * 4 * c->m.n_lin);
        if (e == cudaSuccess) e = cudaMemsetAsync(s->ssm, 0, s->ssm_floats * 4 * c->m.n_lin, c->stream);
        if (e != cudaSuccess) {
            cudaGetLastError();
            rq_cuda_seq_free(s);
            return fail(c, RQ_CUDA_ERR_NOMEM, "DeltaNet state: %s", cudaGetErrorString(e));
        }
    }
    *seq = s;
    return RQ_CUDA_OK;
}

void rq_cuda_seq_free(RqCudaSeq *s) {
    if (!s) return;
    if (s->in_pass) {
        // the open pass still refers to the sequence (its row table points at the caches, pass_end updates its length):
        // the memory goes when the pass is closed
        s->dead = true;
        return;
    }
    cudaSetDevice(s->ctx->device);
    cudaStreamSynchronize(s->ctx->stream);
    if (s->k) cudaFree(s->k);
    if (s->v) cudaFree(s->v);
    if (s->ssm) cudaFree(s->ssm);
    for (float *p : s->ck_st)
        if (p) cudaFree(p);
    delete s;
}

int rq_cuda_seq_len(const RqCudaSeq *s) { return s ? s->len : RQ_CUDA_ERR_ARG; }
int rq_cuda_seq_capacity(const RqCudaSeq *s) { return s ? s->cap : RQ_CUDA_ERR_ARG; }

int rq_cuda_seq_truncate(RqCudaSeq *s, int n) {
    if (!s || n < 0 || n > s->len) return RQ_CUDA_ERR_ARG;
    if (s->in_pass) return fail(s->ctx, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    s->len = n;
    for (int &p : s->ck_pos)  // checkpoints past a truncation are dropped (runq.h:239)
        if (p > n) p = -1;
    return RQ_CUDA_OK;
}

size_t rq_cuda_seq_layer_bytes(const RqCudaSeq *s, int is_v) { return s ? (is_v ? s->lv : s->lk) : 0; }
size_t rq_cuda_seq_state_floats(const RqCudaSeq *s) { return s ? s->ssm_floats : 0; }

int rq_cuda_seq_copy(RqCudaSeq *dst, const RqCudaSeq *src, int n) {
    if (!dst || !src || dst == src || dst->ctx != src->ctx) return RQ_CUDA_ERR_ARG;
    RqCuda *c = dst->ctx;
    if (n < 0 || n > src->len || n > dst->cap || dst->kvt != src->kvt) return fail(c, RQ_CUDA_ERR_ARG, "copy of %d positions", n);
    if (dst->in_pass || src->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "a sequence is part of the open pass");
    CU(c, cudaSetDevice(c->device));
    // whole 256-position blocks holding the first n positions, layer by layer (a block's heads are contiguous)
    size_t nblk = (size_t)(n + ATT_P - 1) / ATT_P;
    for (int l = 0; l < c->m.n_attn; l++)
        for (int half = 0; half < 2; half++) {
            size_t bytes = nblk * ATT_PT * c->n_kv * kv_tile_bytes(src->kvt, c->m.head_dim, half);
            uint8_t *d = (half ? dst->v : dst->k) + (size_t)l * (half ? dst->lv : dst->lk);
            const uint8_t *sp = (half ? src->v : src->k) + (size_t)l * (half ? src->lv : src->lk);
            if (bytes) CU(c, cudaMemcpyAsync(d, sp, bytes, cudaMemcpyDeviceToDevice, c->stream));
        }
    if (c->m.n_lin > 0) {
        const float *from = n == src->len ? src->ssm : nullptr;
        for (size_t k = 0; k < src->ck_pos.size() && !from; k++)  // (or a checkpoint the source holds at that length)
            if (src->ck_pos[k] == n && n > 0) from = src->ck_st[k];
        if (from)
            CU(c, cudaMemcpyAsync(dst->ssm, from, src->ssm_floats * 4 * c->m.n_lin, cudaMemcpyDeviceToDevice, c->stream));
        else if (n != 0)
            return fail(c, RQ_CUDA_ERR_STATE, "the DeltaNet state exists only at the source's length %d and at its checkpoints", src->len);
        else
            CU(c, cudaMemsetAsync(dst->ssm, 0, dst->ssm_floats * 4 * c->m.n_lin, c->stream));
        for (int &p : dst->ck_pos) p = -1;  // (the destination's own checkpoints belong to its old content)
    }
    dst->len = n;
    return RQ_CUDA_OK;
}

int rq_cuda_seq_read_kv(RqCudaSeq *s, int layer, int is_v, void *host, size_t bytes) {
    if (!s || !host) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    size_t lb = is_v ? s->lv : s->lk;
    if (layer < 0 || layer >= c->m.n_attn || bytes > lb) return fail(c, RQ_CUDA_ERR_ARG, "layer %d / %zu bytes", layer, bytes);
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(host, (is_v ? s->v : s->k) + (size_t)layer * lb, bytes, cudaMemcpyDeviceToHost, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    return RQ_CUDA_OK;
}

int rq_cuda_seq_write_kv(RqCudaSeq *s, int layer, int is_v, const void *host, size_t bytes, int new_len) {
    if (!s || !host) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    size_t lb = is_v ? s->lv : s->lk;
    if (layer < 0 || layer >= c->m.n_attn || bytes > lb || new_len < 0 || new_len > s->cap)
        return fail(c, RQ_CUDA_ERR_ARG, "layer %d / %zu bytes / length %d", layer, bytes, new_len);
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync((is_v ? s->v : s->k) + (size_t)layer * lb, host, bytes, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    s->len = new_len;
    return RQ_CUDA_OK;
}

int rq_cuda_seq_read_state(RqCudaSeq *s, int lin_layer, float *host) {
    if (!s || !host) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (lin_layer < 0 || lin_layer >= c->m.n_lin) return fail(c, RQ_CUDA_ERR_ARG, "linear layer %d", lin_layer);
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(host, s->ssm + (size_t)lin_layer * s->ssm_floats, s->ssm_floats * 4, cudaMemcpyDeviceToHost, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    return RQ_CUDA_OK;
}

int rq_cuda_seq_write_state(RqCudaSeq *s, int lin_layer, const float *host) {
    if (!s || !host) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (lin_layer < 0 || lin_layer >= c->m.n_lin) return fail(c, RQ_CUDA_ERR_ARG, "linear layer %d", lin_layer);
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(s->ssm + (size_t)lin_layer * s->ssm_floats, host, s->ssm_floats * 4, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    return RQ_CUDA_OK;
}

int rq_cuda_seq_fill_synthetic(RqCudaSeq *s, int n, unsigned long long seed) {
    if (!s) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (n < 1 || n > s->cap) return fail(c, RQ_CUDA_ERR_ARG, "fill of %d positions (capacity %d)", n, s->cap);
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    CU(c, cudaSetDevice(c->device));
    size_t ntiles = (size_t)(n + ATT_P - 1) / ATT_P * ATT_PT * c->n_kv;  // whole blocks
    for (int l = 0; l < c->m.n_attn; l++)
        for (int half = 0; half < 2; half++) {
            uint8_t *base = (half ? s->v : s->k) + (size_t)l * (half ? s->lv : s->lk);
            int fmt = kv_fmt(s->kvt, half);
            size_t words = ntiles * kv_tile_bytes(s->kvt, c->m.head_dim, half) / 2;
            int grid = (int)std::min<size_t>((words + 255) / 256, 148 * 16);
            kv_fill_kernel<<<grid, 256, 0, c->stream>>>(base, ntiles, fmt, c->m.head_dim,
                                                        seed * 0x100000001B3ull + (uint64_t)(l * 2 + half) * 0x9E3779B97F4A7C15ull);
            c->launches++;
        }
    CU(c, cudaGetLastError());
    s->len = n;
    return RQ_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------- the pass
int rq_cuda_pass_begin(RqCuda *c, const RqCudaSegment *seg, int nseg) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "a pass is already open");
    if (!seg || nseg < 1 || nseg > c->max_rows) return fail(c, RQ_CUDA_ERR_ARG, "%d segments", nseg);
    long total = 0;
    int kvt = -1;
    const unsigned long long stamp = ++c->pass_no;  // (a refused call leaves its stamp behind: the next call uses a new one)
    for (int i = 0; i < nseg; i++) {
        const RqCudaSegment &g = seg[i];
        if (!g.seq || g.seq->ctx != c) return fail(c, RQ_CUDA_ERR_ARG, "segment %d: not a sequence of this context", i);
        if (g.n < 1 || g.pos0 < 0) return fail(c, RQ_CUDA_ERR_ARG, "segment %d: %d rows at position %d", i, g.n, g.pos0);
        if ((long)g.pos0 + g.n > g.seq->cap)
            return fail(c, RQ_CUDA_ERR_CONTEXT, "segment %d: positions %d..%d exceed the capacity %d", i, g.pos0, g.pos0 + g.n - 1,
                        g.seq->cap);
        if (g.pos0 > g.seq->len)
            return fail(c, RQ_CUDA_ERR_ARG, "segment %d: position %d leaves a gap after the sequence's %d positions", i, g.pos0,
                        g.seq->len);
        if (g.seq->stamp == stamp) return fail(c, RQ_CUDA_ERR_ARG, "segment %d: its sequence appears twice", i);
        g.seq->stamp = stamp;
        if (kvt < 0) kvt = g.seq->kvt;
        else if (kvt != g.seq->kvt) return fail(c, RQ_CUDA_ERR_ARG, "segment %d: all sequences of a pass share one KV type", i);
        total += g.n;
    }
    if (total > c->max_rows) return fail(c, RQ_CUDA_ERR_ARG, "%ld rows exceed the context's %d", total, c->max_rows);
    CU(c, cudaSetDevice(c->device));
    // (the device table may still be read by kernels of the previous pass: the copy below is stream-ordered behind
    // them; the pinned half written now was last uploaded two passes ago)
    c->up_idx ^= 1;
    CU(c, cudaEventSynchronize(c->up_ev[c->up_idx]));
    c->h_rows = c->h_rows2[c->up_idx];
    c->h_dseg = c->h_dseg2[c->up_idx];
    int r = 0, blk = 0, mx = 0;
    for (int i = 0; i < nseg; i++) {
        const RqCudaSegment &g = seg[i];
        for (int j = 0; j < g.n; j++, r++) {
            PassRow &pr = c->h_rows[r];
            pr.k = g.seq->k;
            pr.v = g.seq->v;
            pr.lk = g.seq->lk;
            pr.lv = g.seq->lv;
            pr.pos = g.pos0 + j;
            pr.np = pr.pos + 1;
            pr.blk0 = blk;
            pr.seg = i;
            blk += (pr.np + ATT_P - 1) / ATT_P;
            mx = std::max(mx, pr.np);
        }
    }
    memset(&c->h_rows[r], 0, sizeof(PassRow));
    c->h_rows[r].blk0 = blk;
    c->pf_ready = c->tc_ready = 0;  // (the tensor-core tables are made by the first call of the pass that needs them)
    if (c->pass_timing) {
        double s1 = 0, s2 = 0;
        for (int i = 0; i < nseg; i++) {
            s1 += seg[i].pos0;
            s2 += (double)(seg[i].n - 1) * seg[i].pos0 + (double)(seg[i].n - 1) * seg[i].n / 2.0;
        }
        c->pt_rows = r, c->pt_first = s1, c->pt_more = s2;
        c->pass_timed = 0;
        CU(c, cudaEventRecord(c->ev_p0, c->stream));
    }
    c->dn_ready = c->dn_used = 0;  // (the DeltaNet tables by the first DeltaNet call, once the pass's checkpoints are named)
    c->pass_ck.clear();
    CU(c, cudaMemcpyAsync(c->d_rows, c->h_rows, sizeof(PassRow) * (r + 1), cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaEventRecord(c->up_ev[c->up_idx], c->stream));
    c->segs.assign(seg, seg + nseg);
    for (int i = 0; i < nseg; i++) seg[i].seq->in_pass = 1;
    c->nrows = r;
    c->nseg = nseg;
    c->total_blocks = blk;
    c->max_np = mx;
    c->pass_kvt = kvt;
    c->pass_open = 1;
    return RQ_CUDA_OK;
}

int rq_cuda_pass_end(RqCuda *c, int commit) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (!c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "no pass is open");
    // the checkpoints the pass took hold the state after their rows (a pass that is not committed leaves their slots empty)
    for (auto &k : c->pass_ck) {
        const RqCudaSegment &g = c->segs[k.seg];
        g.seq->ck_pos[k.slot] = (commit && c->dn_used) ? g.pos0 + k.row + 1 : -1;
    }
    c->pass_ck.clear();
    for (auto &g : c->segs) {
        g.seq->in_pass = 0;
        if (commit) g.seq->len = std::max(g.seq->len, g.pos0 + g.n);
        if (g.seq->dead) rq_cuda_seq_free(g.seq);  // freed by the host while the pass was open
    }
    c->segs.clear();
    c->pass_open = 0;
    if (c->pass_timing) {
        CU(c, cudaEventRecord(c->ev_p1, c->stream));
        c->pass_timed = 1;
    }
    return RQ_CUDA_OK;
}

// The kernels read and write the callers' device rows with 16-byte accesses.
static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }
#define NEED_ALIGNED(c, what, ...)                                                                                   \
    do {                                                                                                             \
        const void *ps_[] = {__VA_ARGS__};                                                                           \
        for (const void *p_ : ps_)                                                                                   \
            if (!aligned16(p_)) return fail(c, RQ_CUDA_ERR_ARG, "%s: device pointers must be 16-byte aligned", what); \
    } while (0)

static int need_pass(RqCuda *c, int layer, int nlayers, const char *what) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (!c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "%s: no pass is open", what);
    if (layer < 0 || layer >= nlayers) return fail(c, RQ_CUDA_ERR_ARG, "%s: layer %d of %d", what, layer, nlayers);
    return RQ_CUDA_OK;
}

int rq_cuda_kv_store_dev(RqCuda *c, int layer, const float *k, const float *v) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "kv_store");
    if (rc) return rc;
    if (!k && !v) return fail(c, RQ_CUDA_ERR_ARG, "kv_store: no rows");
    NEED_ALIGNED(c, "kv_store", k, v);
    CU(c, cudaSetDevice(c->device));
    dim3 grid(c->nrows, c->n_kv, 2);
    switch (c->m.head_dim) {
        case 64: kv_store_kernel<64><<<grid, 64, 0, c->stream>>>(c->d_rows, layer, c->n_kv, c->pass_kvt, k, v, c->d_err); break;
        case 128: kv_store_kernel<128><<<grid, 128, 0, c->stream>>>(c->d_rows, layer, c->n_kv, c->pass_kvt, k, v, c->d_err); break;
        default: kv_store_kernel<256><<<grid, 256, 0, c->stream>>>(c->d_rows, layer, c->n_kv, c->pass_kvt, k, v, c->d_err); break;
    }
    c->launches++;
    CU(c, cudaGetLastError());
    return RQ_CUDA_OK;
}

int rq_cuda_kv_store(RqCuda *c, int layer, const float *k, const float *v) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "kv_store");
    if (rc) return rc;
    if (!k && !v) return fail(c, RQ_CUDA_ERR_ARG, "kv_store: no rows");
    CU(c, cudaSetDevice(c->device));
    size_t bytes = (size_t)c->nrows * c->n_kv * c->m.head_dim * 4;
    if ((rc = grow(c, (void **)&c->d_k, &c->k_bytes, bytes))) return rc;
    if ((rc = grow(c, (void **)&c->d_v, &c->v_bytes, bytes))) return rc;
    if (k) CU(c, cudaMemcpyAsync(c->d_k, k, bytes, cudaMemcpyHostToDevice, c->stream));
    if (v) CU(c, cudaMemcpyAsync(c->d_v, v, bytes, cudaMemcpyHostToDevice, c->stream));
    rc = rq_cuda_kv_store_dev(c, layer, k ? c->d_k : nullptr, v ? c->d_v : nullptr);
    if (rc) return rc;
    CU(c, cudaStreamSynchronize(c->stream));  // the host rows may be reused on return
    return RQ_CUDA_OK;
}

int rq_cuda_qk_norm_rope_store_dev(RqCuda *c, int layer, float *q, const float *k, const float *v, const float *q_norm_w,
                                   const float *k_norm_w, int rope_dim, float rope_theta) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "qk_norm_rope_store");
    if (rc) return rc;
    if (!q || !k || !v || !q_norm_w || !k_norm_w) return fail(c, RQ_CUDA_ERR_ARG, "qk_norm_rope_store: null argument");
    NEED_ALIGNED(c, "qk_norm_rope_store", q, k, v, q_norm_w, k_norm_w);
    const int hd = c->m.head_dim;
    if (rope_dim < 2 || rope_dim > hd || (rope_dim & 1) || !(rope_theta > 1.0f))
        return fail(c, RQ_CUDA_ERR_ARG, "qk_norm_rope_store: %d rotated dims, base %g", rope_dim, (double)rope_theta);
    CU(c, cudaSetDevice(c->device));
    const float log_theta = (float)log((double)rope_theta);
    dim3 grid(c->nrows, c->n_heads + 2 * c->n_kv);
#define PRODUCER(HD_)                                                                                                          \
    qk_norm_rope_store_kernel<HD_><<<grid, HD_, 0, c->stream>>>(c->d_rows, layer, c->n_kv, c->n_heads, c->pass_kvt, q, c->qh, k, v, \
                                                                q_norm_w, k_norm_w, rope_dim, log_theta, c->d_err)
    switch (hd) {
        case 64: PRODUCER(64); break;
        case 128: PRODUCER(128); break;
        default: PRODUCER(256); break;
    }
#undef PRODUCER
    c->launches++;
    CU(c, cudaGetLastError());
    return RQ_CUDA_OK;
}

static int launch_decode_with(RqCuda *c, int layer, const float *q, float *out, float *part, bool may_allocate);
static int launch_combine(RqCuda *c, const float *q, float *out, const float *part, int split_len, int fixed_stride);

static int launch_decode(RqCuda *c, int layer, const float *q, float *out) {
    const int hd = c->m.head_dim;
    size_t need = (size_t)c->total_blocks * c->n_heads * RQ_PSTRIDE(hd) * 4;
    int rc = grow(c, (void **)&c->d_part, &c->part_bytes, need);
    if (rc) return rc;
    return launch_decode_with(c, layer, q, out, c->d_part, true);
}

static int launch_decode_with(RqCuda *c, int layer, const float *q, float *out, float *part, bool may_allocate) {
    const int hd = c->m.head_dim;
    AttnPartArgs a;
    a.rows = c->span_rows ? c->span_rows : c->d_rows;
    a.nrows = c->span_rows ? c->span_nrows : c->nrows;
    a.total_blocks = c->span_rows ? c->span_blocks : c->total_blocks;
    a.layer = layer;
    a.n_kv = c->n_kv;
    a.G = c->G;
    a.q = q;
    a.qh = c->qh;
    a.n_heads = c->n_heads;
    a.scale = 1.0f / sqrtf((float)hd);
    a.part = part;
    a.err = c->d_err;
    cudaError_t e;
    const bool prof = c->prof_on && (size_t)(2 * c->prof_n + 2) <= c->prof_ev.size();
    if (prof) cudaEventRecord(c->prof_ev[2 * c->prof_n], c->stream);
    if (kv_quant(c->pass_kvt) && hd == 128 && !c->exact && may_allocate && c->tc_ready == 0) {
        // once per pass: the tensor maps of the segments' sequences
        c->tc_ready = 1;
        for (auto &g : c->segs)
            if (!g.seq->has_tm_q8) c->tc_ready = -1;
        if (c->tc_ready == 1) {
            for (size_t i = 0; i < c->segs.size(); i++) {
                const RqCudaSeq *sq = c->segs[i].seq;
                c->h_maps8[4 * i] = sq->tm_k, c->h_maps8[4 * i + 1] = sq->tm_v, c->h_maps8[4 * i + 2] = sq->tm_ks, c->h_maps8[4 * i + 3] = sq->tm_vs;
            }
            CU(c, cudaMemcpyAsync(c->d_maps8, c->h_maps8, sizeof(CUtensorMap) * 4 * c->segs.size(), cudaMemcpyHostToDevice, c->stream));
            CU(c, cudaStreamSynchronize(c->stream));  // (the pinned table is reused by the next pass)
        }
    }
    if (kv_quant(c->pass_kvt) && hd == 128 && !c->exact && may_allocate && c->tc_ready == 1) {
        // quantised caches at head_dim 128: the cached levels as int8 MMA operands (results inside the tolerance); the same partial
        // records, merged by the same kernel
        int rcg;
        // (sized for the whole pass also when the launch covers a run of its rows: the scratch is not regrown between runs)
        if ((rcg = grow(c, (void **)&c->d_tcq, &c->tcq_bytes, (size_t)c->nrows * c->n_kv * TCD_QT_BYTES))) return rcg;
        if ((rcg = grow(c, (void **)&c->d_blk2row, &c->blk2row_bytes, (size_t)c->total_blocks * sizeof(int)))) return rcg;
        AttnPartTcArgs t;
        t.kvt = c->pass_kvt;
        t.qt = c->d_tcq, t.blk2row = c->d_blk2row, t.maps = c->d_maps8, t.n_sm = c->n_sm;
        t.rows = a.rows, t.nrows = a.nrows, t.total_blocks = a.total_blocks, t.layer = a.layer, t.n_kv = a.n_kv, t.G = a.G;
        t.q = a.q, t.qh = a.qh, t.n_heads = a.n_heads, t.scale = a.scale, t.part = a.part, t.err = a.err;
        e = launch_attn_part_tc(t, c->stream);
    } else
    switch (c->pass_kvt) {
        case KV_F16: e = launch_attn_part<KV_F16>(hd, a, c->stream); break;
        case KV_Q8: e = launch_attn_part<KV_Q8>(hd, a, c->stream); break;
        case KV_Q4: e = launch_attn_part<KV_Q4>(hd, a, c->stream); break;
        case KV_Q4K4: e = launch_attn_part<KV_Q4K4>(hd, a, c->stream); break;
        default: e = cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return fail(c, RQ_CUDA_ERR_DEVICE, "attention launch: %s", cudaGetErrorString(e));
    if (prof) cudaEventRecord(c->prof_ev[2 * c->prof_n++ + 1], c->stream);
    c->launches++;
    return launch_combine(c, q, out, part, ATT_P, 0);
}

static int launch_combine(RqCuda *c, const float *q, float *out, const float *part, int split_len, int fixed_stride) {
    const int hd = c->m.head_dim;
    const PassRow *rows = c->span_rows ? c->span_rows : c->d_rows;
    dim3 grid(c->span_rows ? c->span_nrows : c->nrows, c->n_heads);
    const bool quant = kv_quant(c->pass_kvt);
    cudaError_t ce = cudaSuccess;
    PeerOut po;
    memset(&po, 0, sizeof po);
    if (c->peer_now) {
        po.world = c->peer_world, po.n_heads_full = c->m.n_heads, po.head0 = c->m.kv_head0 * c->G;
        for (int p = 0; p < c->peer_world; p++) po.out[p] = (float *)(c->peer_base[p] + 1024 + (size_t)(c->peer_step & 1) * c->peer_rows_bytes);
    }
#define COMBINE(HD_)                                                                                                          \
    if (quant) ce = launch_pdl(attn_combine_kernel<HD_, true>, grid, dim3(COMBINE_NG * HD_), 0, c->stream, rows, c->n_heads, part, q, c->qh, c->m.gated, out, split_len, fixed_stride, (const int *)c->d_err, c->err_fwd, c->wo_quant, po); \
    else ce = launch_pdl(attn_combine_kernel<HD_, false>, grid, dim3(COMBINE_NG * HD_), 0, c->stream, rows, c->n_heads, part, q, c->qh, c->m.gated, out, split_len, fixed_stride, (const int *)c->d_err, c->err_fwd, c->wo_quant, po);
    switch (hd) {
        case 64: COMBINE(64) break;
        case 128: COMBINE(128) break;
        default: COMBINE(256) break;
    }
#undef COMBINE
    c->launches++;
    CU(c, ce);
    return RQ_CUDA_OK;
}

int rq_cuda_attn_decode_dev(RqCuda *c, int layer, const float *q, float *out) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "attn_decode");
    if (rc) return rc;
    if (!q || !out) return fail(c, RQ_CUDA_ERR_ARG, "attn_decode: null rows");
    NEED_ALIGNED(c, "attn_decode", q, out);
    CU(c, cudaSetDevice(c->device));
    return launch_decode(c, layer, q, out);
}

int rq_cuda_attn_decode_gather_dev(RqCuda *c, int layer, const float *q, float **out_full) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "attn_decode_gather");
    if (rc) return rc;
    if (!q || !out_full) return fail(c, RQ_CUDA_ERR_ARG, "attn_decode_gather: null rows");
    if (!c->peer_world) return fail(c, RQ_CUDA_ERR_STATE, "attn_decode_gather: no peers imported");
    if (c->nrows > c->peer_max_rows) return fail(c, RQ_CUDA_ERR_ARG, "attn_decode_gather: %d rows exceed the exported %d", c->nrows, c->peer_max_rows);
    NEED_ALIGNED(c, "attn_decode_gather", q, q);
    CU(c, cudaSetDevice(c->device));
    c->peer_step++;
    c->peer_now = true;
    rc = launch_decode(c, layer, q, (float *)(c->peer_own + 1024));
    c->peer_now = false;
    if (rc) return rc;
    PeerFlags pf;
    memset(&pf, 0, sizeof pf);
    for (int p = 0; p < c->peer_world; p++) pf.flags[p] = (unsigned *)c->peer_base[p];
    peer_sync_kernel<<<1, 32, 0, c->stream>>>(pf, c->peer_rank, c->peer_world, c->peer_step, c->d_err, 2000000000ull, 97);
    c->launches++;
    CU(c, cudaGetLastError());
    *out_full = (float *)(c->peer_own + 1024 + (size_t)(c->peer_step & 1) * c->peer_rows_bytes);
    return RQ_CUDA_OK;
}


static int stage_q(RqCuda *c, const float *q, size_t qbytes, size_t obytes) {
    int rc;
    if ((rc = grow(c, (void **)&c->d_q, &c->q_bytes, qbytes))) return rc;
    if ((rc = grow(c, (void **)&c->d_out, &c->out_bytes, obytes))) return rc;
    CU(c, cudaMemcpyAsync(c->d_q, q, qbytes, cudaMemcpyHostToDevice, c->stream));
    return RQ_CUDA_OK;
}

// The device-side address of a host buffer the GPU can write directly (page-locked and mapped: rq_cuda_malloc_host,
// cudaMallocHost, cudaHostRegister), or null for ordinary host memory.  The merge kernel then stores its rows straight
// into the caller's buffer and the separate device-to-host copy (and its latency after the last kernel) goes away.
static float *mapped_host(void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return a.type == cudaMemoryTypeHost ? (float *)a.devicePointer : nullptr;
}

// End of a host-buffer call whose merge kernel stored the status word to h_err itself (err_fwd): only the wait is left.
static int sync_forwarded(RqCuda *c) {
    CU(c, cudaStreamSynchronize(c->stream));
    if (*c->h_err) {
        int code = *c->h_err;
        *c->h_err = 0;
        cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream);
        return fail(c, RQ_CUDA_ERR_STATE, "a device-side wait expired (code %d): results of the last pass are invalid", code);
    }
    return RQ_CUDA_OK;
}

int rq_cuda_attn_decode(RqCuda *c, int layer, const float *q, float *out) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "attn_decode");
    if (rc) return rc;
    if (!q || !out) return fail(c, RQ_CUDA_ERR_ARG, "attn_decode: null rows");
    CU(c, cudaSetDevice(c->device));
    size_t qb = (size_t)c->nrows * c->n_heads * c->qh * 4, ob = (size_t)c->nrows * c->n_heads * c->m.head_dim * 4;
    if ((rc = stage_q(c, q, qb, ob))) return rc;
    float *od = mapped_host(out);
    c->err_fwd = (int *)mapped_host(c->h_err);
    rc = launch_decode(c, layer, c->d_q, od ? od : c->d_out);
    const bool fwd = c->err_fwd != nullptr;
    c->err_fwd = nullptr;
    if (rc) return rc;
    if (!od) CU(c, cudaMemcpyAsync(out, c->d_out, ob, cudaMemcpyDeviceToHost, c->stream));
    return fwd ? sync_forwarded(c) : rq_cuda_sync(c);
}

// ---- decode attention without any allocation -------------------------------------------------------------------------
// The per-block partial results of the split-K attention normally live in a buffer the context grows with cudaMalloc
// when a pass needs more of it.  Some hosts cannot have that: a server that sized all device memory at start-up
// and handed the rest to KV caches (an allocation in the middle of a pass can fail or stall there), and code that
// runs where cudaMalloc is off limits because it synchronises the whole device.  For them the partials of this
// entry point sit in the fixed array below, part of the library's image on every GPU that loads it, until exit.
#define RQ_NOALLOC_PART_BYTES ((size_t)32 << 20)
static __device__ __align__(256) unsigned char g_noalloc_part[RQ_NOALLOC_PART_BYTES];
// per device: the array's device address (not the host-side symbol).  Atomic: contexts of one device may be driven by
// different host threads; two of them racing through the first call both store the same address.
static std::atomic<float *> g_noalloc_ptr[64];

size_t rq_cuda_attn_decode_noalloc_max_bytes(void) { return RQ_NOALLOC_PART_BYTES; }

int rq_cuda_attn_decode_noalloc(RqCuda *c, int layer, const float *q, float *out) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "attn_decode_noalloc");
    if (rc) return rc;
    if (!q || !out) return fail(c, RQ_CUDA_ERR_ARG, "attn_decode_noalloc: null rows");
    NEED_ALIGNED(c, "attn_decode_noalloc", q, out);
    size_t need = (size_t)c->total_blocks * c->n_heads * RQ_PSTRIDE(c->m.head_dim) * 4;
    if (need > RQ_NOALLOC_PART_BYTES)
        return fail(c, RQ_CUDA_ERR_ARG,
                    "attn_decode_noalloc: the pass needs %zu bytes of partial results (%d blocks of 256 positions x %d heads), "
                    "the fixed scratch holds %zu; use rq_cuda_attn_decode_dev or split the pass",
                    need, c->total_blocks, c->n_heads, (size_t)RQ_NOALLOC_PART_BYTES);
    if (c->device < 0 || c->device >= 64) return fail(c, RQ_CUDA_ERR_ARG, "attn_decode_noalloc: device %d", c->device);
    CU(c, cudaSetDevice(c->device));
    float *part = g_noalloc_ptr[c->device].load(std::memory_order_acquire);
    if (!part) {
        // once per device, with that device current: the address the kernels can use (the name g_noalloc_part in
        // host code is only a handle for this query)
        void *p = nullptr;
        CU(c, cudaGetSymbolAddress(&p, g_noalloc_part));
        part = (float *)p;
        g_noalloc_ptr[c->device].store(part, std::memory_order_release);
    }
    // nothing in the array has to start at zero: every record the merge reads was written by this call's first kernel
    return launch_decode_with(c, layer, q, out, part, false);  // (never the kernels that need growable scratch)
}

static int prefill_tables(RqCuda *c) {
    // once per pass: the segments' tensor maps and the work list (M tile of 128 / G rows x split of the keys) of the
    // tensor-core prefill kernel; pf_ready 1: made, -1: the pass does not qualify (cache type, head_dim)
    if (c->pf_ready) return RQ_CUDA_OK;
    c->pf_ready = -1;
    const int nseg = (int)c->segs.size();
    c->pf_quant = false;
    if (kv_quant(c->pass_kvt)) {
        // quantised caches at head_dim 128: the tensor-core kernel over f16 copies of the layer's tiles, where the pass is a prompt
        // pass (on average 16 rows or more per segment: below that the copies cost more than they save) and the copies fit 8 GB;
        // not where the host asked for exact results
        constexpr int PROMPT_ROWS = 16;  // a segment of fewer rows is not worth expanding its cache for
        const int hdq = c->m.head_dim;
        if ((hdq != 128 && hdq != 256) || c->exact || !tm_encode()) return RQ_CUDA_OK;
        const size_t tile_f16 = (size_t)hdq * 32;  // bytes of an f16 tile: 16 positions x head_dim
        size_t tiles = 0;
        int n_prompt = 0;
        for (auto &g : c->segs)
            if (g.n >= PROMPT_ROWS) tiles += (size_t)((g.pos0 + g.n + ATT_P - 1) / ATT_P) * ATT_PT * c->n_kv, n_prompt++;
        if (!n_prompt || tiles * 2 * tile_f16 > ((size_t)8 << 30)) return RQ_CUDA_OK;
        int rcq = grow(c, (void **)&c->d_dq, &c->dq_bytes, tiles * 2 * tile_f16);
        if (rcq) return rcq;
        if ((rcq = grow(c, (void **)&c->d_dqseg, &c->dqseg_bytes, sizeof(DqSeg) * nseg))) return rcq;
        if ((rcq = grow(c, (void **)&c->d_qrot, &c->qrot_bytes, (size_t)c->nrows * c->n_heads * hdq * 4))) return rcq;
        c->h_dqseg.resize(nseg);
        c->dq_max_tiles = 0;
        uint8_t *at = c->d_dq;
        TmEncodeFn enc = tm_encode();
        cuuint32_t es[2] = {1, 1};
        // the runs of rows of each kind, and the decode runs' own row table
        c->pf_runs_p.clear(), c->pf_runs_d.clear(), c->h_rows_d.clear();
        c->pf_part_d = 0;
        {
            int row = 0;
            for (int i = 0; i < nseg; i++) {
                const RqCudaSegment &g = c->segs[i];
                const bool prompt = g.n >= PROMPT_ROWS;
                auto &runs = prompt ? c->pf_runs_p : c->pf_runs_d;
                const bool prev_same = i > 0 && (c->segs[i - 1].n >= PROMPT_ROWS) == prompt;
                if (!prev_same) runs.push_back(RqCuda::RowRun{row, 0, 0, (int)c->h_rows_d.size(), 0});
                RqCuda::RowRun &run = runs.back();
                if (!prompt) {
                    for (int j = 0; j < g.n; j++) {
                        PassRow pr = c->h_rows[row + j];
                        pr.blk0 = run.blocks;
                        run.blocks += (pr.np + ATT_P - 1) / ATT_P;
                        c->h_rows_d.push_back(pr);
                    }
                }
                run.nrows += g.n;
                row += g.n;
            }
            for (auto &run : c->pf_runs_d) {
                run.part0 = c->pf_part_d;
                c->pf_part_d += (size_t)run.blocks * c->n_heads * RQ_PSTRIDE(hdq);
            }
            if (!c->h_rows_d.empty()) {
                if ((rcq = grow(c, (void **)&c->d_rows_d, &c->rows_d_bytes, sizeof(PassRow) * c->h_rows_d.size()))) return rcq;
                CU(c, cudaMemcpyAsync(c->d_rows_d, c->h_rows_d.data(), sizeof(PassRow) * c->h_rows_d.size(), cudaMemcpyHostToDevice, c->stream));
            }
        }
        for (int i = 0; i < nseg; i++) {
            const RqCudaSegment &g = c->segs[i];
            DqSeg &d = c->h_dqseg[i];
            memset(&d, 0, sizeof d);
            if (g.n < PROMPT_ROWS) continue;  // (tiles 0: the expansion kernel's CTAs of this segment return at once)
            d.k = g.seq->k, d.v = g.seq->v, d.lk = g.seq->lk, d.lv = g.seq->lv;
            d.len = g.pos0 + g.n;
            d.tiles = (d.len + ATT_P - 1) / ATT_P * ATT_PT;
            const size_t bytes = (size_t)d.tiles * c->n_kv * tile_f16;
            d.ko = at, d.vo = at + bytes;
            at += 2 * bytes;
            c->dq_max_tiles = std::max(c->dq_max_tiles, d.tiles);
            // the same views as an f16 cache of one layer (seq_make_maps)
            cuuint64_t kd[2] = {16, (cuuint64_t)(bytes / 32)}, ks[1] = {32}, vd[2] = {(cuuint64_t)hdq, (cuuint64_t)(bytes / (2 * hdq))},
                       vs[1] = {(cuuint64_t)(2 * hdq)};
            cuuint32_t kb[2] = {16, hdq == 128 ? 256u : 128u}, vb[2] = {64, 128};
            if (enc(&c->h_maps[2 * i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d.ko, kd, ks, kb, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
                enc(&c->h_maps[2 * i + 1], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, d.vo, vd, vs, vb, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
                return RQ_CUDA_OK;  // (the pass takes the row-by-row path)
        }
        CU(c, cudaMemcpyAsync(c->d_dqseg, c->h_dqseg.data(), sizeof(DqSeg) * nseg, cudaMemcpyHostToDevice, c->stream));
        c->pf_quant = true;
    } else {
        if ((c->m.head_dim != 128 && c->m.head_dim != 256) || c->pass_kvt != KV_F16) return RQ_CUDA_OK;
        for (auto &g : c->segs)
            if (!g.seq->has_tm) return RQ_CUDA_OK;
    }
    const int rpt = 128 / c->G;
    {
        // The split length of the pass: the kernel's M tiles (128 / G rows of a segment x one KV head) are cut along the keys into
        // items of `split` positions, one CTA each, so that short passes still fill the SMs; every item pays its own prologue and
        // epilogue (loading and converting Q, storing a partial record per row: worth about six 128-key blocks of the main loop) and
        // its rows one more partial to merge.  Chosen by scheduling the items of each candidate length onto the SMs as the hardware
        // does (each to the SM that is free first) and taking the shortest finish.
        std::vector<int> nblk;  // key blocks of every tile of the pass
        for (int i = 0; i < nseg; i++) {
            const RqCudaSegment &g = c->segs[i];
            if (c->pf_quant && g.n < 16) continue;
            for (int m0 = 0; m0 < g.n; m0 += rpt) nblk.push_back((g.pos0 + m0 + std::min(rpt, g.n - m0) + PF_BN - 1) / PF_BN);
        }
        const int cand[] = {1024, 1280, 1536, 1792, 2048, 2560, 3072, 3584, 4096, 5120, 6144, 7168, 8192, 12288, 16384, 32768, 65536};
        const double overhead = c->m.head_dim == 256 ? 4.0 : 6.0;  // (a block of head_dim 256 takes about twice as long)
        // (the KV heads are the grid's second dimension, the same items n_kv times: one head's items onto its share of the SMs)
        const int sms = std::max(1, c->n_sm / std::max(1, c->n_kv));
        double best = 0.0;
        c->pf_split = PF_SPLIT;
        std::vector<double> sm_free(sms);
        if (c->pf_split_fixed) c->pf_split = c->pf_split_fixed;
        else
        for (int L : cand) {
            const int lb = L / PF_BN;
            size_t items = 0;
            for (int nb : nblk) items += (size_t)((nb + lb - 1) / lb) * c->n_kv;
            if (items > (size_t)1 << 20) continue;
            std::fill(sm_free.begin(), sm_free.end(), 0.0);
            std::make_heap(sm_free.begin(), sm_free.end(), std::greater<double>());
            auto put = [&](double cost) {
                std::pop_heap(sm_free.begin(), sm_free.end(), std::greater<double>());
                sm_free.back() += cost;
                std::push_heap(sm_free.begin(), sm_free.end(), std::greater<double>());
            };
            // (launch order: tile by tile, its splits in order)
            for (int nb : nblk)
                for (int k = 0; k * lb < nb; k++) put(std::min(lb, nb - k * lb) + overhead);
            const double finish = *std::max_element(sm_free.begin(), sm_free.end());
            if (best == 0.0 || finish <= best) best = finish, c->pf_split = L;  // (ties go to the longer split: fewer partials to merge)
            if (L >= c->max_np) break;  // (no longer split changes anything)
        }
    }
    c->h_work.clear();
    int row = 0;
    for (int i = 0; i < nseg; i++) {
        const RqCudaSegment &g = c->segs[i];
        if (!c->pf_quant) {
            c->h_maps[2 * i] = g.seq->tm_k;
            c->h_maps[2 * i + 1] = g.seq->tm_v;
        }
        if (!c->pf_quant || g.n >= 16)  // (a quantised pass: only its prompt segments)
            for (int m0 = 0; m0 < g.n; m0 += rpt) {
                int nr = std::min(rpt, g.n - m0), np_max = g.pos0 + m0 + nr;
                for (int k = 0; k * c->pf_split < np_max; k++) c->h_work.push_back(PfWork{i, row + m0, nr, k});
            }
        row += g.n;
    }
    c->pf_max_splits = (c->max_np + c->pf_split - 1) / c->pf_split;
    size_t wb = c->h_work.size() * sizeof(PfWork);
    int rc = grow(c, (void **)&c->d_work, &c->work_bytes, wb);
    if (rc) return rc;
    CU(c, cudaMemcpyAsync(c->d_maps, c->h_maps, sizeof(CUtensorMap) * 2 * nseg, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaMemcpyAsync(c->d_work, c->h_work.data(), wb, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));  // (the work list is pageable host memory, the maps are reused next pass)
    c->pf_ready = 1;
    return RQ_CUDA_OK;
}

static int launch_prefill(RqCuda *c, int layer, const float *q, float *out) {
    // tensor-core tiles where the pass qualifies (f16 cache, head_dim 128 or 256); other shapes take the split-K kernels,
    // which compute the same attention on the CUDA cores
    int rc0 = prefill_tables(c);
    if (rc0) return rc0;
    if (c->pf_ready != 1) return launch_decode(c, layer, q, out);
    const int hd = c->m.head_dim;
    const size_t need_pf = (size_t)c->nrows * c->pf_max_splits * c->n_heads * RQ_PSTRIDE(hd) * 4;
    const size_t need = need_pf + (c->pf_quant ? c->pf_part_d * 4 : 0);
    if (need > ((size_t)8 << 30))
        return fail(c, RQ_CUDA_ERR_ARG,
                    "attn_prefill: %d rows x %d splits of %d positions x %d heads need %zu MB of partial results; pass fewer rows at once",
                    c->nrows, c->pf_max_splits, c->pf_split, c->n_heads, need >> 20);
    int rc = grow(c, (void **)&c->d_part, &c->part_bytes, need);
    if (rc) return rc;
    AttnPrefillArgs a;
    a.work = c->d_work;
    a.n_work = (int)c->h_work.size();
    a.rows = c->d_rows;
    a.maps = c->d_maps;
    a.layer = layer;
    a.n_kv = c->n_kv;
    a.G = c->G;
    a.q = q;
    a.qh = c->qh;
    a.n_heads = c->n_heads;
    a.scale = 1.0f / sqrtf((float)hd);
    a.max_splits = c->pf_max_splits;
    a.split_len = c->pf_split;
    a.part = c->d_part;
    a.err = c->d_err;
    if (c->pf_quant) {
        // the layer's tiles as f16 (layer 0 of the scratch's views), the query rows rotated; the merge below un-rotates
        // (the same launch rotates the query rows, in z slices of its grid past the segments': a warp per (row, head))
        const int nrh = c->nrows * c->n_heads, nsegs = (int)c->segs.size();
        const size_t per_slice = (size_t)c->dq_max_tiles * c->n_kv * (hd / 32);
        const dim3 dgrid(c->dq_max_tiles, c->n_kv, (unsigned)(nsegs + (nrh + per_slice - 1) / per_slice));
        cudaError_t de;
#define DEQUANT(KVT_)                                                                                                                          \
    de = hd == 128 ? launch_pdl(kv_dequant_f16_kernel<KVT_, 128>, dgrid, dim3(128), 0, c->stream, (const DqSeg *)c->d_dqseg, nsegs, layer, c->n_kv, \
                                q, c->qh, nrh, c->d_qrot)                                                                                      \
                   : launch_pdl(kv_dequant_f16_kernel<KVT_, 256>, dgrid, dim3(256), 0, c->stream, (const DqSeg *)c->d_dqseg, nsegs, layer, c->n_kv, \
                                q, c->qh, nrh, c->d_qrot)
        switch (c->pass_kvt) {
            case KV_Q8: DEQUANT(KV_Q8); break;
            case KV_Q4: DEQUANT(KV_Q4); break;
            default: DEQUANT(KV_Q4K4); break;
        }
#undef DEQUANT
        if (de != cudaSuccess) return fail(c, RQ_CUDA_ERR_DEVICE, "cache expansion launch: %s", cudaGetErrorString(de));
        c->launches++;
        a.layer = 0;
        a.q = c->d_qrot;
        a.qh = hd;
    }
    const bool prof = c->prof_on && (size_t)(2 * c->prof_n + 2) <= c->prof_ev.size();
    if (prof) cudaEventRecord(c->prof_ev[2 * c->prof_n], c->stream);
    cudaError_t e = hd == 128 ? launch_attn_prefill(a, c->stream) : launch_attn_prefill_hd256(a, c->stream);
    if (e != cudaSuccess) return fail(c, RQ_CUDA_ERR_DEVICE, "prefill attention launch: %s", cudaGetErrorString(e));
    if (prof) cudaEventRecord(c->prof_ev[2 * c->prof_n++ + 1], c->stream);
    c->launches++;
    if (c->pf_quant) {
        // the prompt segments' rows: merged (and un-rotated, gated) run by run; the other rows of the pass: the decode kernels over
        // their own row table, run by run.  The status word goes to the host with the last launch only.
        int *fwd = c->err_fwd;
        const WoQuant wq = c->wo_quant;
        const size_t nlast = c->pf_runs_p.size() + c->pf_runs_d.size();
        size_t done = 0;
        const size_t pst = RQ_PSTRIDE(hd);
        auto wq_at = [&](int row0) {
            WoQuant w = wq;
            if (w.xq) w.xq += (size_t)row0 * c->n_heads * hd, w.xs += (size_t)row0 * c->n_heads * hd / w.gs;
            return w;
        };
        for (const auto &run : c->pf_runs_p) {
            const int nout = run.nrows * c->n_heads;
            const dim3 cgrid((nout + COMBINE_ROWS_WARPS - 1) / COMBINE_ROWS_WARPS), cblock(32 * COMBINE_ROWS_WARPS);
#define ROWS_MERGE(HD_)                                                                                                                       \
    CU(c, launch_pdl(attn_combine_rows_kernel<HD_>, cgrid, cblock, 0, c->stream, (const PassRow *)(c->d_rows + run.row0), run.nrows, c->n_heads,       \
                     (const float *)(c->d_part + (size_t)run.row0 * c->pf_max_splits * c->n_heads * pst),                                              \
                     q + (size_t)run.row0 * c->n_heads * c->qh, c->qh, c->m.gated, out + (size_t)run.row0 * c->n_heads * HD_, c->pf_split,             \
                     c->pf_max_splits, (const int *)c->d_err, ++done == nlast ? fwd : (int *)nullptr, wq_at(run.row0), 1))
            if (hd == 128) ROWS_MERGE(128);
            else ROWS_MERGE(256);
#undef ROWS_MERGE
            c->launches++;
        }
        int rcd = RQ_CUDA_OK;
        for (const auto &run : c->pf_runs_d) {
            c->span_rows = c->d_rows_d + run.table0, c->span_nrows = run.nrows, c->span_blocks = run.blocks;
            c->err_fwd = ++done == nlast ? fwd : nullptr;
            c->wo_quant = wq_at(run.row0);
            rcd = launch_decode_with(c, layer, q + (size_t)run.row0 * c->n_heads * c->qh, out + (size_t)run.row0 * c->n_heads * hd,
                                     c->d_part + need_pf / 4 + run.part0, true);
            if (rcd) break;
        }
        c->span_rows = nullptr, c->span_nrows = c->span_blocks = 0;
        c->err_fwd = fwd;
        c->wo_quant = wq;
        return rcd;
    }
    // (a warp per output row merges its few partials, and applies the output gate)
    const int nout = c->nrows * c->n_heads;
    const dim3 cgrid((nout + COMBINE_ROWS_WARPS - 1) / COMBINE_ROWS_WARPS), cblock(32 * COMBINE_ROWS_WARPS);
    if (hd == 128)
        CU(c, launch_pdl(attn_combine_rows_kernel<128>, cgrid, cblock, 0, c->stream, c->d_rows, c->nrows, c->n_heads, (const float *)c->d_part, q, c->qh,
                         c->m.gated, out, c->pf_split, c->pf_max_splits, (const int *)c->d_err, c->err_fwd, c->wo_quant, c->pf_quant ? 1 : 0));
    else
        CU(c, launch_pdl(attn_combine_rows_kernel<256>, cgrid, cblock, 0, c->stream, c->d_rows, c->nrows, c->n_heads, (const float *)c->d_part, q, c->qh,
                         c->m.gated, out, c->pf_split, c->pf_max_splits, (const int *)c->d_err, c->err_fwd, c->wo_quant, 0));
    c->launches++;
    return RQ_CUDA_OK;
}

int rq_cuda_attn_prefill_dev(RqCuda *c, int layer, const float *q, float *out) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "attn_prefill");
    if (rc) return rc;
    if (!q || !out) return fail(c, RQ_CUDA_ERR_ARG, "attn_prefill: null rows");
    NEED_ALIGNED(c, "attn_prefill", q, out);
    CU(c, cudaSetDevice(c->device));
    return launch_prefill(c, layer, q, out);
}

int rq_cuda_attn_prefill(RqCuda *c, int layer, const float *q, float *out) {
    int rc = need_pass(c, layer, c ? c->m.n_attn : 0, "attn_prefill");
    if (rc) return rc;
    if (!q || !out) return fail(c, RQ_CUDA_ERR_ARG, "attn_prefill: null rows");
    CU(c, cudaSetDevice(c->device));
    size_t qb = (size_t)c->nrows * c->n_heads * c->qh * 4, ob = (size_t)c->nrows * c->n_heads * c->m.head_dim * 4;
    if ((rc = stage_q(c, q, qb, ob))) return rc;
    float *od = mapped_host(out);
    c->err_fwd = (int *)mapped_host(c->h_err);
    rc = launch_prefill(c, layer, c->d_q, od ? od : c->d_out);
    const bool fwd = c->err_fwd != nullptr;
    c->err_fwd = nullptr;
    if (rc) return rc;
    if (!od) CU(c, cudaMemcpyAsync(out, c->d_out, ob, cudaMemcpyDeviceToHost, c->stream));
    return fwd ? sync_forwarded(c) : rq_cuda_sync(c);
}

// The DeltaNet tables of the open pass: per segment its state and rows, its chunks (a cut every 64 rows and after every
// checkpoint row) and its checkpoints.  Made and uploaded by the first DeltaNet call of the pass.
static int dn_tables(RqCuda *c) {
    c->dn_used = 1;
    if (c->dn_ready) return RQ_CUDA_OK;
    const int nseg = c->nseg;
    DnSeg *hs = c->h_dseg2[c->up_idx];
    DnChunk *hc = c->h_chunk2[c->up_idx];
    DnCk *hk = c->h_ck2[c->up_idx];
    std::stable_sort(c->pass_ck.begin(), c->pass_ck.end(), [](const RqCuda::PassCk &a, const RqCuda::PassCk &b) { return a.seg != b.seg ? a.seg < b.seg : a.row < b.row; });
    int r = 0, nch = 0, nck = 0;
    size_t ki = 0;
    for (int i = 0; i < nseg; i++) {
        const RqCudaSegment &g = c->segs[i];
        DnSeg &d = hs[i];
        d.state = g.seq->ssm;
        d.lstride = g.seq->ssm_floats;
        d.row0 = r;
        d.n = g.n;
        d.first = g.pos0 == 0;
        d.chunk0 = nch;
        d.ck0 = nck;
        int at = 0;
        while (at < g.n) {
            int end = std::min(g.n, at + 64), ck = -1;
            if (ki < c->pass_ck.size() && c->pass_ck[ki].seg == i && c->pass_ck[ki].row < end) {
                end = c->pass_ck[ki].row + 1;
                hk[nck].dst = g.seq->ck_st[c->pass_ck[ki].slot];
                hk[nck].row = c->pass_ck[ki].row;
                hk[nck].pad = 0;
                ck = nck++;
                ki++;
            }
            hc[nch++] = DnChunk{i, at, end - at, ck};
            at = end;
        }
        d.nch = nch - d.chunk0;
        d.nck = nck - d.ck0;
        r += g.n;
    }
    c->dn_chunks = nch;
    CU(c, cudaMemcpyAsync(c->d_dseg, hs, sizeof(DnSeg) * nseg, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaMemcpyAsync(c->d_chunks, hc, sizeof(DnChunk) * nch, cudaMemcpyHostToDevice, c->stream));
    if (nck) CU(c, cudaMemcpyAsync(c->d_ck, hk, sizeof(DnCk) * nck, cudaMemcpyHostToDevice, c->stream));
    // (the pinned halves are written again two passes from now: the event then covers these uploads too)
    CU(c, cudaEventRecord(c->up_ev[c->up_idx], c->stream));
    c->dn_ready = 1;
    return RQ_CUDA_OK;
}

int rq_cuda_seq_set_checkpoints(RqCudaSeq *s, int n) {
    if (!s || n < 0 || n > 32) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (c->m.n_lin < 1) return n == 0 ? RQ_CUDA_OK : fail(c, RQ_CUDA_ERR_STATE, "the model has no DeltaNet layers: nothing to checkpoint");
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    CU(c, cudaSetDevice(c->device));
    if ((size_t)n < s->ck_st.size()) CU(c, cudaStreamSynchronize(c->stream));
    while (s->ck_st.size() > (size_t)n) {  // fewer slots: the last ones go
        if (s->ck_st.back()) cudaFree(s->ck_st.back());
        s->ck_st.pop_back();
        s->ck_pos.pop_back();
    }
    while (s->ck_st.size() < (size_t)n) {
        float *p = nullptr;
        CU(c, cudaMalloc((void **)&p, s->ssm_floats * 4 * c->m.n_lin));
        s->ck_st.push_back(p);
        s->ck_pos.push_back(-1);
    }
    return RQ_CUDA_OK;
}

int rq_cuda_seq_checkpoint_pos(const RqCudaSeq *s, int slot) {
    if (!s || slot < 0 || (size_t)slot >= s->ck_pos.size()) return RQ_CUDA_ERR_ARG;
    return s->ck_pos[slot];
}

int rq_cuda_seq_checkpoint_drop(RqCudaSeq *s, int slot) {
    if (!s || slot < 0 || (size_t)slot >= s->ck_pos.size()) return RQ_CUDA_ERR_ARG;
    if (s->in_pass) return fail(s->ctx, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    s->ck_pos[slot] = -1;
    return RQ_CUDA_OK;
}

int rq_cuda_pass_checkpoint(RqCuda *c, int seg, int row, int slot) {
    if (!c) return RQ_CUDA_ERR_ARG;
    if (!c->pass_open) return fail(c, RQ_CUDA_ERR_STATE, "pass_checkpoint: no pass is open");
    if (c->dn_used) return fail(c, RQ_CUDA_ERR_STATE, "pass_checkpoint: a DeltaNet layer of this pass has already run");
    if (seg < 0 || seg >= c->nseg) return fail(c, RQ_CUDA_ERR_ARG, "pass_checkpoint: segment %d of %d", seg, c->nseg);
    const RqCudaSegment &g = c->segs[seg];
    if (row < 0 || row >= g.n) return fail(c, RQ_CUDA_ERR_ARG, "pass_checkpoint: row %d of a segment of %d rows", row, g.n);
    if (slot < 0 || (size_t)slot >= g.seq->ck_st.size()) return fail(c, RQ_CUDA_ERR_ARG, "pass_checkpoint: slot %d (the sequence has %zu)", slot, g.seq->ck_st.size());
    if (c->pass_ck.size() >= (size_t)RqCuda::MAX_PASS_CK) return fail(c, RQ_CUDA_ERR_ARG, "pass_checkpoint: more than %d checkpoints in a pass", RqCuda::MAX_PASS_CK);
    for (auto &k : c->pass_ck)
        if (k.seg == seg && (k.row == row || k.slot == slot)) return fail(c, RQ_CUDA_ERR_ARG, "pass_checkpoint: row %d or slot %d is named twice", row, slot);
    c->pass_ck.push_back(RqCuda::PassCk{seg, row, slot});
    g.seq->ck_pos[slot] = -1;  // (being written; valid once the pass is committed)
    c->dn_ready = 0;
    return RQ_CUDA_OK;
}

int rq_cuda_seq_restore(RqCudaSeq *s, int slot) {
    if (!s || slot < 0 || (size_t)slot >= s->ck_pos.size()) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    if (s->ck_pos[slot] < 0) return fail(c, RQ_CUDA_ERR_STATE, "checkpoint slot %d is empty", slot);
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(s->ssm, s->ck_st[slot], s->ssm_floats * 4 * c->m.n_lin, cudaMemcpyDeviceToDevice, c->stream));
    return rq_cuda_seq_truncate(s, s->ck_pos[slot]);
}

int rq_cuda_seq_read_checkpoint(RqCudaSeq *s, int slot, int lin_layer, float *host) {
    if (!s || !host || slot < 0 || (size_t)slot >= s->ck_pos.size()) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (lin_layer < 0 || lin_layer >= c->m.n_lin) return fail(c, RQ_CUDA_ERR_ARG, "linear layer %d", lin_layer);
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(host, s->ck_st[slot] + (size_t)lin_layer * s->ssm_floats, s->ssm_floats * 4, cudaMemcpyDeviceToHost, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    return RQ_CUDA_OK;
}

int rq_cuda_seq_write_checkpoint(RqCudaSeq *s, int slot, int lin_layer, const float *host, int pos) {
    if (!s || !host || slot < 0 || (size_t)slot >= s->ck_pos.size()) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (lin_layer < 0 || lin_layer >= c->m.n_lin || pos < 0 || pos > s->cap) return fail(c, RQ_CUDA_ERR_ARG, "linear layer %d / length %d", lin_layer, pos);
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(s->ck_st[slot] + (size_t)lin_layer * s->ssm_floats, host, s->ssm_floats * 4, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    s->ck_pos[slot] = pos;
    return RQ_CUDA_OK;
}

int rq_cuda_dn_rec_dev(RqCuda *c, int lin_layer, const float *rows, float *out) {
    int rc = need_pass(c, lin_layer, c ? c->m.n_lin : 0, "dn_rec");
    if (rc) return rc;
    if (!rows || !out) return fail(c, RQ_CUDA_ERR_ARG, "dn_rec: null rows");
    NEED_ALIGNED(c, "dn_rec", rows, out);
    CU(c, cudaSetDevice(c->device));
    const RqCudaModel &m = c->m;
    const int lw = 2 * m.dn_nk * m.dn_dk + 2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv;
    size_t convf = ((size_t)(m.dn_conv - 1) * (2 * m.dn_nk * m.dn_dk + m.dn_nv * m.dn_dv) + 15) / 16 * 16;
    if ((rc = dn_tables(c))) return rc;
    dim3 grid(m.dn_nv * (m.dn_dv / DN_BW), c->nseg);
    dn_rec_kernel<128><<<grid, 32, 0, c->stream>>>(c->d_dseg, lin_layer, m.dn_nk, m.dn_nv, m.dn_dv, convf, rows, lw, out, c->d_ck);
    c->launches++;
    CU(c, cudaGetLastError());
    return RQ_CUDA_OK;
}

int rq_cuda_dn_chunk_dev(RqCuda *c, int lin_layer, const float *rows, float *out) {
    int rc = need_pass(c, lin_layer, c ? c->m.n_lin : 0, "dn_chunk");
    if (rc) return rc;
    if (!rows || !out) return fail(c, RQ_CUDA_ERR_ARG, "dn_chunk: null rows");
    NEED_ALIGNED(c, "dn_chunk", rows, out);
    const RqCudaModel &m = c->m;
    if (m.dn_dk != 128 || m.dn_dv != 128) return fail(c, RQ_CUDA_ERR_ARG, "dn_chunk is built for dk = dv = 128");
    CU(c, cudaSetDevice(c->device));
    if ((rc = dn_tables(c))) return rc;
    // one work record per (64-token chunk, value head): a pass of many short segments (decode rows) would ask for a
    // record per row and belongs to rq_cuda_dn_rec
    const size_t work_need = (size_t)c->dn_chunks * m.dn_nv * DNC_ITEM;
    if (work_need > ((size_t)8 << 30))
        return fail(c, RQ_CUDA_ERR_ARG, "dn_chunk: %d chunks x %d heads need %zu MB of work records; use dn_rec for passes of short segments",
                    c->dn_chunks, m.dn_nv, work_need >> 20);
    int rcg = grow(c, (void **)&c->d_dnwork, &c->dnwork_bytes, work_need);
    if (rcg) return rcg;
    DnChunkArgs a;
    a.segs = c->d_dseg;
    a.chunks = c->d_chunks;
    a.cks = c->d_ck;
    a.nseg = c->nseg;
    a.n_chunks = c->dn_chunks;
    a.work = c->d_dnwork;
    a.lin_layer = lin_layer;
    a.nk = m.dn_nk;
    a.nv = m.dn_nv;
    a.conv_floats = ((size_t)(m.dn_conv - 1) * (2 * m.dn_nk * m.dn_dk + m.dn_nv * m.dn_dv) + 15) / 16 * 16;
    a.rows = rows;
    a.lw = 2 * m.dn_nk * m.dn_dk + 2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv;
    a.out = out;
    a.err = c->d_err;
    cudaError_t e = launch_dn_chunk(a, c->stream);
    if (e != cudaSuccess) return fail(c, RQ_CUDA_ERR_DEVICE, "dn_chunk launch: %s", cudaGetErrorString(e));
    c->launches += 2;
    return RQ_CUDA_OK;
}

static int dn_host(RqCuda *c, int lin_layer, const float *rows, float *out, bool chunked) {
    const RqCudaModel &m = c->m;
    const int lw = 2 * m.dn_nk * m.dn_dk + 2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv;
    size_t rb = (size_t)c->nrows * lw * 4, ob = (size_t)c->nrows * m.dn_nv * m.dn_dv * 4;
    int rc;
    if ((rc = grow(c, (void **)&c->d_dn, &c->dn_bytes, rb + ob))) return rc;
    float *d_rows = c->d_dn, *d_out = c->d_dn + (size_t)c->nrows * lw;
    CU(c, cudaMemcpyAsync(d_rows, rows, rb, cudaMemcpyHostToDevice, c->stream));
    if ((rc = chunked ? rq_cuda_dn_chunk_dev(c, lin_layer, d_rows, d_out) : rq_cuda_dn_rec_dev(c, lin_layer, d_rows, d_out))) return rc;
    CU(c, cudaMemcpyAsync(out, d_out, ob, cudaMemcpyDeviceToHost, c->stream));
    return rq_cuda_sync(c);
}

int rq_cuda_dn_chunk(RqCuda *c, int lin_layer, const float *rows, float *out) {
    int rc = need_pass(c, lin_layer, c ? c->m.n_lin : 0, "dn_chunk");
    if (rc) return rc;
    if (!rows || !out) return fail(c, RQ_CUDA_ERR_ARG, "dn_chunk: null rows");
    CU(c, cudaSetDevice(c->device));
    return dn_host(c, lin_layer, rows, out, true);
}

int rq_cuda_dn_rec(RqCuda *c, int lin_layer, const float *rows, float *out) {
    int rc = need_pass(c, lin_layer, c ? c->m.n_lin : 0, "dn_rec");
    if (rc) return rc;
    if (!rows || !out) return fail(c, RQ_CUDA_ERR_ARG, "dn_rec: null rows");
    CU(c, cudaSetDevice(c->device));
    return dn_host(c, lin_layer, rows, out, false);
}

int rq_cuda_dn_set_weights(RqCuda *c, int lin_layer, const float *conv, const float *a, const float *dt, const float *norm) {
    if (!c) return RQ_CUDA_ERR_ARG;
    const RqCudaModel &m = c->m;
    if (lin_layer < 0 || lin_layer >= m.n_lin || !conv || !a || !dt || !norm) return fail(c, RQ_CUDA_ERR_ARG, "dn_set_weights: layer %d", lin_layer);
    if (m.dn_dk != 128 || m.dn_dv != 128 || m.dn_conv > 8)
        return fail(c, RQ_CUDA_ERR_ARG, "dn_prep / dn_out are built for dk = dv = 128 and at most 8 conv taps");
    CU(c, cudaSetDevice(c->device));
    const size_t cd = (size_t)2 * m.dn_nk * m.dn_dk + (size_t)m.dn_nv * m.dn_dv;
    const size_t nconv = cd * m.dn_conv, per = nconv + 2 * m.dn_nv + m.dn_dv;
    if (!c->d_dnw) {
        CU(c, cudaMalloc((void **)&c->d_dnw, per * m.n_lin * 4));
        c->dnw_layer_floats = per;
        c->dnw_set.assign(m.n_lin, 0);
    }
    float *base = c->d_dnw + (size_t)lin_layer * per;
    CU(c, cudaMemcpyAsync(base, conv, nconv * 4, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaMemcpyAsync(base + nconv, a, m.dn_nv * 4, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaMemcpyAsync(base + nconv + m.dn_nv, dt, m.dn_nv * 4, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaMemcpyAsync(base + nconv + 2 * m.dn_nv, norm, m.dn_dv * 4, cudaMemcpyHostToDevice, c->stream));
    CU(c, cudaStreamSynchronize(c->stream));
    c->dnw_set[lin_layer] = 1;
    return RQ_CUDA_OK;
}

static int dn_weights(RqCuda *c, int lin_layer, const char *what, const float **conv, const float **a, const float **dt, const float **norm) {
    if (!c->d_dnw || !c->dnw_set[lin_layer]) return fail(c, RQ_CUDA_ERR_STATE, "%s: rq_cuda_dn_set_weights was not called for layer %d", what, lin_layer);
    const RqCudaModel &m = c->m;
    const size_t nconv = ((size_t)2 * m.dn_nk * m.dn_dk + (size_t)m.dn_nv * m.dn_dv) * m.dn_conv;
    const float *base = c->d_dnw + (size_t)lin_layer * c->dnw_layer_floats;
    *conv = base;
    *a = base + nconv;
    *dt = *a + m.dn_nv;
    *norm = *dt + m.dn_nv;
    return RQ_CUDA_OK;
}

int rq_cuda_dn_prep_dev(RqCuda *c, int lin_layer, float *rows) {
    int rc = need_pass(c, lin_layer, c ? c->m.n_lin : 0, "dn_prep");
    if (rc) return rc;
    if (!rows) return fail(c, RQ_CUDA_ERR_ARG, "dn_prep: null rows");
    NEED_ALIGNED(c, "dn_prep", rows);
    const float *conv, *a, *dt, *norm;
    if ((rc = dn_weights(c, lin_layer, "dn_prep", &conv, &a, &dt, &norm))) return rc;
    CU(c, cudaSetDevice(c->device));
    if ((rc = dn_tables(c))) return rc;
    const RqCudaModel &m = c->m;
    const int lw = 2 * m.dn_nk * m.dn_dk + 2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv;
    dn_prep_kernel<<<dim3(2 * m.dn_nk + m.dn_nv, c->nseg), 128, 0, c->stream>>>(c->d_dseg, lin_layer, m.dn_nk, m.dn_nv, m.dn_conv, conv, a, dt, rows, lw, c->d_ck);
    c->launches++;
    CU(c, cudaGetLastError());
    return RQ_CUDA_OK;
}

int rq_cuda_dn_out_dev(RqCuda *c, int lin_layer, const float *rows, float *out) {
    int rc = need_pass(c, lin_layer, c ? c->m.n_lin : 0, "dn_out");
    if (rc) return rc;
    if (!rows || !out) return fail(c, RQ_CUDA_ERR_ARG, "dn_out: null rows");
    NEED_ALIGNED(c, "dn_out", rows, out);
    const float *conv, *a, *dt, *norm;
    if ((rc = dn_weights(c, lin_layer, "dn_out", &conv, &a, &dt, &norm))) return rc;
    CU(c, cudaSetDevice(c->device));
    const RqCudaModel &m = c->m;
    const int lw = 2 * m.dn_nk * m.dn_dk + 2 * m.dn_nv * m.dn_dv + 2 * m.dn_nv;
    dn_out_kernel<<<dim3(c->nrows, m.dn_nv), 128, 0, c->stream>>>(m.dn_nk, m.dn_nv, norm, rows, lw, out);
    c->launches++;
    CU(c, cudaGetLastError());
    return RQ_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------- saved sequences
// The reference's sequence file (src/seqfile.c): every section at a multiple of 4096 bytes — the header (SeqFileHdr,
// seqfile.c:32-41), the tokens, per attention layer its first nblk K blocks then V blocks of 256 positions as they lie in
// the cache, then (Qwen3.5) the recurrent state and the checkpoints held, ascending by length.  A file written here is
// read by the reference's rq_seq_load and the other way round: the caches have the same bytes on both sides.
namespace {
constexpr uint64_t SF_ALIGN = 4096;
const char sf_magic[8] = {'R', 'Q', 'S', 'E', 'Q', '\r', '\n', 0x1a};
struct SeqFileHdr {  // version 1's layout, 264 bytes
    char magic[8];
    uint32_t version, endian;
    uint64_t model_fp;
    int32_t n_attn, kv_dim, n_kv_heads, head_dim, att_p, att_t, att, kv_esz, n_lin, len, nblk, nck;
    int32_t ck[32];
    uint64_t ssm_bytes, ssm_stride, blk_bytes;
    uint64_t off_kv, off_ssm, file_bytes, rng;
    uint64_t hash;
};
static_assert(sizeof(SeqFileHdr) == 264, "the reference's header layout");
uint64_t sf_round(uint64_t n) { return (n + SF_ALIGN - 1) / SF_ALIGN * SF_ALIGN; }
uint64_t fnv1a64(uint64_t h, const void *p, size_t n) {
    const unsigned char *b = (const unsigned char *)p;
    for (size_t i = 0; i < n; i++) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}
uint64_t sf_hash(const SeqFileHdr &h, const int *tokens) {
    SeqFileHdr c = h;
    c.hash = 0;
    return fnv1a64(fnv1a64(1469598103934665603ull, &c, sizeof(c)), tokens, (size_t)h.len * sizeof(int));
}
// the derived fields of a header whose shape fields (and len, nck, ck) are set
void sf_layout(SeqFileHdr &h) {
    const uint64_t bk = (uint64_t)ATT_PT * h.n_kv_heads * kv_tile_bytes(h.att, h.head_dim, 0);
    const uint64_t bv = (uint64_t)ATT_PT * h.n_kv_heads * kv_tile_bytes(h.att, h.head_dim, 1);
    h.kv_esz = (int32_t)(kv_tile_bytes(h.att, h.head_dim, 1) / (ATT_T * h.head_dim));
    h.nblk = (h.len + ATT_P - 1) / ATT_P;
    h.ssm_stride = sf_round(h.ssm_bytes);
    h.blk_bytes = bk;
    h.off_kv = SF_ALIGN + sf_round((uint64_t)h.len * sizeof(int));
    h.off_ssm = h.off_kv + (uint64_t)h.n_attn * h.nblk * (bk + bv);
    h.file_bytes = h.off_ssm + (h.n_lin > 0 ? (uint64_t)(1 + h.nck) * h.ssm_stride : 0);
}
bool sf_io(int fd, bool wr, void *buf, size_t n, uint64_t off) {
    char *p = (char *)buf;
    while (n) {
        ssize_t r = wr ? pwrite(fd, p, n, (off_t)off) : pread(fd, p, n, (off_t)off);
        if (r <= 0) return false;
        p += r, off += (uint64_t)r, n -= (size_t)r;
    }
    return true;
}
void sf_header_of(const RqCudaSeq *s, uint64_t model_fp, uint64_t rng, SeqFileHdr &h, int *slots) {
    const RqCuda *c = s->ctx;
    memset(&h, 0, sizeof(h));
    memcpy(h.magic, sf_magic, 8);
    h.version = 1;
    h.endian = 0x01020304;
    h.model_fp = model_fp;
    h.n_attn = c->m.n_attn;
    h.kv_dim = c->m.n_kv_heads * c->m.head_dim;
    h.n_kv_heads = c->m.n_kv_heads;
    h.head_dim = c->m.head_dim;
    h.att_p = ATT_P;
    h.att_t = ATT_T;
    h.att = s->kvt;
    h.n_lin = c->m.n_lin;
    h.len = s->len;
    // the checkpoints held, ascending by length
    std::vector<std::pair<int, int>> ck;
    for (size_t k = 0; k < s->ck_pos.size(); k++)
        if (s->ck_pos[k] >= 0 && s->ck_pos[k] <= s->len) ck.push_back({s->ck_pos[k], (int)k});
    std::sort(ck.begin(), ck.end());
    h.nck = (int32_t)ck.size();
    for (size_t i = 0; i < ck.size(); i++) h.ck[i] = ck[i].first, slots[i] = ck[i].second;
    h.ssm_bytes = (uint64_t)c->m.n_lin * s->ssm_floats * 4;
    h.rng = rng;
    sf_layout(h);
}
}  // namespace

long long rq_cuda_seq_save_bytes(const RqCudaSeq *s) {
    if (!s || s->len < 1) return 0;
    SeqFileHdr h;
    int slots[32];
    sf_header_of(s, 0, 0, h, slots);
    return (long long)h.file_bytes;
}

int rq_cuda_seq_save(RqCudaSeq *s, const char *path, const int *tokens, unsigned long long model_fp, unsigned long long rng) {
    if (!s || !path || !tokens) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (s->len < 1) return fail(c, RQ_CUDA_ERR_ARG, "seq_save: an empty sequence");
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    if (c->m.n_attn > 0 && c->n_kv != c->m.n_kv_heads) return fail(c, RQ_CUDA_ERR_STATE, "seq_save: this context holds a group of the KV heads only");
    CU(c, cudaSetDevice(c->device));
    SeqFileHdr h;
    int slots[32];
    sf_header_of(s, model_fp, rng, h, slots);
    h.hash = sf_hash(h, tokens);
    const std::string tmp = std::string(path) + ".tmp";
    int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC, 0644);
    if (fd < 0) return fail(c, RQ_CUDA_ERR_IO, "seq_save: cannot create %s", tmp.c_str());
    bool good = ftruncate(fd, (off_t)h.file_bytes) == 0;
    std::vector<char> head(h.off_kv, 0);
    memcpy(head.data(), &h, sizeof(h));
    memcpy(head.data() + SF_ALIGN, tokens, (size_t)h.len * sizeof(int));
    good = good && sf_io(fd, true, head.data(), head.size(), 0);
    // the first nblk blocks of every layer's K, then V (a layer's blocks are contiguous from its start)
    const uint64_t bk = h.blk_bytes, bv = (uint64_t)ATT_PT * h.n_kv_heads * kv_tile_bytes(h.att, h.head_dim, 1);
    std::vector<char> buf((size_t)h.nblk * std::max(bk, bv));
    cudaError_t ce = cudaSuccess;
    for (int l = 0; l < h.n_attn && good && ce == cudaSuccess; l++)
        for (int kv = 0; kv < 2 && good && ce == cudaSuccess; kv++) {
            const size_t n = (size_t)h.nblk * (kv ? bv : bk);
            ce = cudaMemcpyAsync(buf.data(), (kv ? s->v : s->k) + (size_t)l * (kv ? s->lv : s->lk), n, cudaMemcpyDeviceToHost, c->stream);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(c->stream);
            good = sf_io(fd, true, buf.data(), n, h.off_kv + (uint64_t)h.nblk * ((uint64_t)l * (bk + bv) + (kv ? bk : 0)));
        }
    if (h.n_lin > 0 && good && ce == cudaSuccess) {
        std::vector<char> st(h.ssm_stride, 0);
        for (int i = 0; i <= h.nck && good && ce == cudaSuccess; i++) {
            const float *src = i == 0 ? s->ssm : s->ck_st[slots[i - 1]];
            ce = cudaMemcpyAsync(st.data(), src, h.ssm_bytes, cudaMemcpyDeviceToHost, c->stream);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(c->stream);
            good = sf_io(fd, true, st.data(), st.size(), h.off_ssm + (uint64_t)i * h.ssm_stride);
        }
    }
    good = good && fdatasync(fd) == 0;
    good = (close(fd) == 0) && good;
    if (ce != cudaSuccess || !good || rename(tmp.c_str(), path) != 0) {
        unlink(tmp.c_str());
        return ce != cudaSuccess ? fail(c, RQ_CUDA_ERR_DEVICE, "seq_save: %s", cudaGetErrorString(ce)) : fail(c, RQ_CUDA_ERR_IO, "seq_save: writing %s failed", path);
    }
    return RQ_CUDA_OK;
}

int rq_cuda_seq_load(RqCudaSeq *s, const char *path, unsigned long long model_fp, int n, int *tokens, unsigned long long *rng) {
    if (!s || !path) return RQ_CUDA_ERR_ARG;
    RqCuda *c = s->ctx;
    if (n < 0 || n > s->cap) return fail(c, RQ_CUDA_ERR_ARG, "seq_load: %d positions (capacity %d)", n, s->cap);
    if (s->in_pass) return fail(c, RQ_CUDA_ERR_STATE, "the sequence is part of the open pass");
    if (c->m.n_attn > 0 && c->n_kv != c->m.n_kv_heads) return fail(c, RQ_CUDA_ERR_STATE, "seq_load: this context holds a group of the KV heads only");
    CU(c, cudaSetDevice(c->device));
    int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return fail(c, RQ_CUDA_ERR_IO, "seq_load: cannot open %s", path);
    struct stat stt;
    SeqFileHdr h, w;
    std::vector<char> page(SF_ALIGN);
    int rc = RQ_CUDA_OK;
    std::vector<char> head;
    if (fstat(fd, &stt) || (uint64_t)stt.st_size < SF_ALIGN || !sf_io(fd, false, page.data(), SF_ALIGN, 0)) rc = RQ_CUDA_ERR_IO;
    if (rc == RQ_CUDA_OK) {
        // the header against this context's shape, the sequence's cache type, and itself (sf_check, seqfile.c:183-217)
        memcpy(&h, page.data(), sizeof(h));
        w = h;
        if (memcmp(h.magic, sf_magic, 8) || h.version != 1 || h.endian != 0x01020304 || h.model_fp != model_fp || h.n_attn != c->m.n_attn ||
            h.kv_dim != c->m.n_kv_heads * c->m.head_dim || h.n_kv_heads != c->m.n_kv_heads || h.head_dim != c->m.head_dim || h.att_p != ATT_P ||
            h.att_t != ATT_T || h.att != s->kvt || h.n_lin != c->m.n_lin || h.len < 1 || h.nck < 0 || h.nck > 32 || (h.n_lin == 0 && h.nck) ||
            h.ssm_bytes != (uint64_t)c->m.n_lin * s->ssm_floats * 4)
            rc = RQ_CUDA_ERR_MISMATCH;
        for (int i = 0; rc == RQ_CUDA_OK && i < h.nck; i++)
            if (h.ck[i] < 0 || h.ck[i] > h.len || (i && h.ck[i] <= h.ck[i - 1])) rc = RQ_CUDA_ERR_MISMATCH;
        if (rc == RQ_CUDA_OK) {
            sf_layout(w);
            if (w.kv_esz != h.kv_esz || w.nblk != h.nblk || w.ssm_stride != h.ssm_stride || w.blk_bytes != h.blk_bytes || w.off_kv != h.off_kv ||
                w.off_ssm != h.off_ssm || w.file_bytes != h.file_bytes || (uint64_t)stt.st_size != h.file_bytes)
                rc = RQ_CUDA_ERR_MISMATCH;
        }
    }
    if (rc == RQ_CUDA_OK) {
        head.resize(h.off_kv);
        if (!sf_io(fd, false, head.data(), head.size(), 0)) rc = RQ_CUDA_ERR_IO;
        else if (sf_hash(h, (const int *)(head.data() + SF_ALIGN)) != h.hash) rc = RQ_CUDA_ERR_MISMATCH;
    }
    if (rc == RQ_CUDA_OK && n > h.len) rc = RQ_CUDA_ERR_ARG;
    if (rc != RQ_CUDA_OK) {
        close(fd);
        return fail(c, rc, "seq_load: %s %s", path, rc == RQ_CUDA_ERR_IO ? "could not be read" : rc == RQ_CUDA_ERR_ARG ? "holds fewer positions" : "is not a saved sequence of this model shape and cache type");
    }
    // the length kept (rq_seq_file_keep, seqfile.c:409): n itself without DeltaNet layers, else the saved length or the longest
    // checkpoint at or below n
    int L = n;
    if (h.n_lin > 0 && n != h.len) {
        L = 0;
        for (int i = 0; i < h.nck; i++)
            if (h.ck[i] <= n) L = h.ck[i];
    }
    const uint64_t bk = h.blk_bytes, bv = (uint64_t)ATT_PT * h.n_kv_heads * kv_tile_bytes(h.att, h.head_dim, 1);
    const int nblk = (L + ATT_P - 1) / ATT_P;
    std::vector<char> buf((size_t)std::max(nblk, 1) * std::max(bk, bv));
    bool good = true;
    cudaError_t ce = cudaSuccess;
    for (int l = 0; l < h.n_attn && good && ce == cudaSuccess && L > 0; l++)
        for (int kv = 0; kv < 2 && good && ce == cudaSuccess; kv++) {
            const size_t nb = (size_t)nblk * (kv ? bv : bk);
            good = sf_io(fd, false, buf.data(), nb, h.off_kv + (uint64_t)h.nblk * ((uint64_t)l * (bk + bv) + (kv ? bk : 0)));
            if (good) ce = cudaMemcpyAsync((kv ? s->v : s->k) + (size_t)l * (kv ? s->lv : s->lk), buf.data(), nb, cudaMemcpyHostToDevice, c->stream);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(c->stream);
        }
    for (int &p : s->ck_pos) p = -1;
    if (h.n_lin > 0 && L > 0 && good && ce == cudaSuccess) {
        // the state at L: the saved one, or the checkpoint there; the saved checkpoints at or below L into the slots (the
        // highest ones if the sequence has fewer slots)
        int top = 0;
        while (top < h.nck && h.ck[top] <= L) top++;
        std::vector<char> st(h.ssm_stride);
        auto fetch = [&](uint64_t off, float *dst) {
            good = good && sf_io(fd, false, st.data(), st.size(), off);
            if (good && ce == cudaSuccess) ce = cudaMemcpyAsync(dst, st.data(), h.ssm_bytes, cudaMemcpyHostToDevice, c->stream);
            if (ce == cudaSuccess) ce = cudaStreamSynchronize(c->stream);
        };
        fetch(h.off_ssm + (L == h.len ? 0 : (uint64_t)top * h.ssm_stride), s->ssm);
        const int nslot = (int)s->ck_st.size();
        for (int i = std::max(0, top - nslot), k = 0; i < top && good && ce == cudaSuccess; i++, k++) {
            fetch(h.off_ssm + (uint64_t)(1 + i) * h.ssm_stride, s->ck_st[k]);
            s->ck_pos[k] = h.ck[i];
        }
    } else if (h.n_lin > 0 && L == 0) {
        ce = cudaMemsetAsync(s->ssm, 0, s->ssm_floats * 4 * c->m.n_lin, c->stream);
    }
    close(fd);
    if (!good || ce != cudaSuccess) {
        s->len = 0;  // (RQ_ERR_IO: the destination is then empty, runq.h:313)
        for (int &p : s->ck_pos) p = -1;
        return ce != cudaSuccess ? fail(c, RQ_CUDA_ERR_DEVICE, "seq_load: %s", cudaGetErrorString(ce)) : fail(c, RQ_CUDA_ERR_IO, "seq_load: reading %s failed", path);
    }
    if (tokens) memcpy(tokens, head.data() + SF_ALIGN, (size_t)L * sizeof(int));
    if (rng) *rng = h.rng;
    s->len = L;
    return RQ_CUDA_OK;
}

// ---------------------------------------------------------------------------------------------------- helpers
int rq_cuda_malloc(RqCuda *c, size_t bytes, void **dev) {
    if (!c || !dev) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMalloc(dev, bytes));
    return RQ_CUDA_OK;
}
int rq_cuda_mfree(RqCuda *c, void *dev) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaStreamSynchronize(c->stream));
    CU(c, cudaFree(dev));
    return RQ_CUDA_OK;
}
int rq_cuda_malloc_host(RqCuda *c, size_t bytes, void **host) {
    if (!c || !host) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMallocHost(host, bytes));
    return RQ_CUDA_OK;
}
int rq_cuda_mfree_host(RqCuda *c, void *host) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaFreeHost(host));
    return RQ_CUDA_OK;
}
int rq_cuda_memcpy_h2d(RqCuda *c, void *dev, const void *host, size_t bytes) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, c->stream));
    return RQ_CUDA_OK;
}
int rq_cuda_memcpy_d2h(RqCuda *c, void *host, const void *dev, size_t bytes) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    return RQ_CUDA_OK;
}
int rq_cuda_mem_info(RqCuda *c, size_t *free_bytes, size_t *total_bytes) {
    if (!c || !free_bytes || !total_bytes) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaMemGetInfo(free_bytes, total_bytes));
    return RQ_CUDA_OK;
}
int rq_cuda_timer_start(RqCuda *c) {
    if (!c) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaEventRecord(c->ev0, c->stream));
    return RQ_CUDA_OK;
}
int rq_cuda_timer_stop(RqCuda *c, float *ms) {
    if (!c || !ms) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaEventRecord(c->ev1, c->stream));
    CU(c, cudaEventSynchronize(c->ev1));
    CU(c, cudaEventElapsedTime(ms, c->ev0, c->ev1));
    return RQ_CUDA_OK;
}
unsigned long long rq_cuda_launch_count(const RqCuda *c) { return c ? c->launches : 0; }

int rq_cuda_profile_begin(RqCuda *c, int max_launches) {
    if (!c || max_launches < 1 || max_launches > (1 << 16)) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    while (c->prof_ev.size() < (size_t)2 * max_launches) {
        cudaEvent_t ev;
        CU(c, cudaEventCreate(&ev));
        c->prof_ev.push_back(ev);
    }
    c->prof_n = 0;
    c->prof_on = 1;
    return RQ_CUDA_OK;
}

int rq_cuda_profile_end(RqCuda *c, float *total_ms, int *launches) {
    if (!c || !total_ms || !launches) return RQ_CUDA_ERR_ARG;
    CU(c, cudaSetDevice(c->device));
    CU(c, cudaStreamSynchronize(c->stream));
    c->prof_on = 0;
    float tot = 0.0f;
    for (int i = 0; i < c->prof_n; i++) {
        float ms = 0.0f;
        CU(c, cudaEventElapsedTime(&ms, c->prof_ev[2 * i], c->prof_ev[2 * i + 1]));
        tot += ms;
    }
    *total_ms = tot;
    *launches = c->prof_n;
    return RQ_CUDA_OK;
}

}  // extern "C"
