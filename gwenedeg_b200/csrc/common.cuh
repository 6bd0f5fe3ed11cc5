// Shared device helpers of librq_cuda: the reference's scalar arithmetic (softmax exponential, sigmoid, half
// conversions), KV tile geometry, and thin wrappers over the sm_100a async-copy (TMA bulk) and mbarrier PTX.
//
// The whole library is compiled with -fmad=false: a * b + c written in source stays two rounded operations, and every
// fused multiply-add is an explicit fmaf(), exactly where the reference's definition has one.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rq {

constexpr int ATT_T = 16;    // positions per cache tile           (reference src/kernels_avx512.h:34)
constexpr int ATT_P = 256;   // positions per attention block      (:36)
constexpr int ATT_PT = 16;   // tiles per block
constexpr int ATT_DC = 32;   // dims per fused-multiply-add chain of a score (:40)
#define RQ_PSTRIDE(hd) ((hd) + 16)  // floats per block partial: o[hd], m, l, padding (:39)

enum { KV_F32 = 0, KV_F16 = 2, KV_Q8 = 3, KV_Q4 = 8, KV_Q4K4 = 9 };

__host__ __device__ constexpr bool kv_quant(int t) { return t == KV_Q8 || t == KV_Q4 || t == KV_Q4K4; }
// element format of the K (half 0) / V (half 1) cache of a type: q4 keeps its K in 8 bits (src/kvtype.h:26)
__host__ __device__ constexpr int kv_fmt(int t, int half) { return t == KV_Q4K4 ? KV_Q4 : (t == KV_Q4 && half == 0) ? KV_Q8 : t; }
// bytes of one 16-position tile of one head (src/kvtype.h:34)
__host__ __device__ constexpr int kv_tile_bytes(int t, int hd, int half) {
    return hd * (kv_fmt(t, half) == KV_F32 ? 64 : kv_fmt(t, half) == KV_Q8 ? 17 : kv_fmt(t, half) == KV_Q4 ? 9 : 32);
}
// index, in tiles, of the tile holding position t of (local) head h in a layer with n_kv heads (src/forward.c:1894)
__host__ __device__ inline size_t kv_tile_index(int t, int h, int n_kv) {
    return ((size_t)(t / ATT_P) * n_kv + h) * ATT_PT + (size_t)(t % ATT_P) / ATT_T;
}

// ---- scalar arithmetic ------------------------------------------------------------------------------------------
// e^x for x <= 0, operation for operation the reference's exp_att (src/forward.c:1301; constants
// src/kernels_avx512.h:41-50): clamp at -86, n = rint(x log2 e), two-step reduction, degree-5 Horner, 2^n via the
// exponent field.
__device__ __forceinline__ float exp_att(float x) {
    x = x > -86.0f ? x : -86.0f;
    float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float z = r * r;
    float y = 1.9875691500e-4f;
    y = fmaf(y, r, 1.3981999507e-3f);
    y = fmaf(y, r, 8.3334519073e-3f);
    y = fmaf(y, r, 4.1665795894e-2f);
    y = fmaf(y, r, 1.6666665459e-1f);
    y = fmaf(y, r, 5.0000001201e-1f);
    y = fmaf(y, z, r);
    y = y + 1.0f;
    return __uint_as_float(__float_as_uint(y) + ((uint32_t)(int32_t)n << 23));
}

// 1 / (1 + e^-x) through e = exp(-|x|) (src/forward.c:2011)
__device__ __forceinline__ float sigmoid_att(float x) {
    float e = exp_att(-fabsf(x));
    float r = 1.0f / (1.0f + e);
    return x >= 0.0f ? r : e * r;
}

// fp32 -> IEEE half bits: round to nearest even, |x| >= 65520 saturates to 65504, NaN stays quiet (src/forward.c:1325)
__device__ __forceinline__ uint16_t f32_to_f16_sat(float f) {
    uint32_t u = __float_as_uint(f), sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu, h;
    if (a > 0x7f800000u) h = 0x7e00u | ((a >> 13) & 0x3ffu);
    else if (a >= 0x477ff000u) h = 0x7bffu;
    else h = __half_as_ushort(__float2half_rn(__uint_as_float(a)));  // RNE, exact subnormals
    return (uint16_t)(sign | h);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// the fixed sign vector D of the KV rotation: -1 where 1 (src/forward.c:1636)
__device__ __forceinline__ int kvq_neg(int i) { return (int)(((uint32_t)i * 0x9E3779B9u) >> 31); }

// ---- mbarrier + bulk async copy (TMA) ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// the same poll, but the thread may be suspended by the hardware for up to `hint_ns` while the phase is incomplete (it is
// woken when the phase completes): a waiting warp then issues a poll every `hint_ns` instead of every few cycles
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t *bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Wait for a phase of the barrier with a time limit (0.2 s, far beyond any healthy copy or MMA): on expiry the kernel
// records `code` in *err and the caller carries on to its exit (results are then invalid and the host reports
// RQ_CUDA_ERR_STATE).  Once any thread has recorded an expiry the other waits give up quickly as well.
__device__ __forceinline__ bool mbar_wait_bounded_ns(uint64_t *bar, uint32_t parity, int *err, int code, unsigned long long limit_ns) {
    unsigned long long t0 = 0;
    for (int it = 0; it < (1 << 26); it++) {
        if (mbar_try_wait(bar, parity)) return true;
        // (the clock and the status word are looked at every 1024 polls only: the status word is a global-memory load of several
        // hundred cycles, which a thread that is about to be released should not be sitting in)
        if ((it & 1023) == 1023) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            if (*reinterpret_cast<volatile int *>(err) != 0) return false;
            if (now - t0 > limit_ns) break;
        }
    }
    atomicExch(err, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int *err, int code) {
    return mbar_wait_bounded_ns(bar, parity, err, code, 200000000ull);
}
// mbar_wait_bounded for waits that normally last a microsecond or more (a copy, a batch of MMAs): polls through
// mbar_try_wait_hint, so that the waiting warp leaves the issue slots to the others; the same 0.2 s limit, counted in polls of at
// most 2 us each, and the same behaviour on expiry
__device__ __forceinline__ bool mbar_wait_bounded_quiet(uint64_t *bar, uint32_t parity, int *err, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    for (int it = 0; it < 100000; it++) {
        if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
        if ((it & 63) == 63 && *reinterpret_cast<volatile int *>(err) != 0) return false;
    }
    atomicExch(err, code);
    return false;
}
// order earlier generic-proxy accesses of shared memory before later async-proxy (bulk copy) writes to it
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// global -> shared bulk copy of `bytes` (a multiple of 16; both addresses 16-byte aligned), completion counted on bar
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// ---- index checks of the debug build (make debug: -DRQ_DEBUG, librq_cuda_debug.so).  The conditions are uniform over
// the CTA and sit before its first barrier: a CTA whose work item does not fit its row or cache records `code` in the
// status word and returns (no trap, nothing is read or written out of range); the host then reports RQ_CUDA_ERR_STATE.
// The release build compiles them away.
#ifdef RQ_DEBUG
#define RQ_CHECK(cond, err, code)                    \
    do {                                             \
        if (!(cond)) {                               \
            if (threadIdx.x == 0) atomicExch(err, code); \
            return;                                  \
        }                                            \
    } while (0)
#else
#define RQ_CHECK(cond, err, code) \
    do {                          \
    } while (0)
#endif

// ---- programmatic dependent launch: a kernel launched with launch_pdl may be scheduled while the kernel before it in
// the stream still runs; it must call pdl_wait() before it touches global memory (the wait returns once the earlier
// kernel has completed and its writes are visible; in a normal launch it returns at once).  pdl_launch_dependents() lets
// the next such kernel be scheduled as soon as every CTA of this one has started.  What is saved is the launch latency
// between the kernels of one layer, a few microseconds each.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// A state checkpoint the open pass takes (CkPass, reference src/internal.h:347-351; dn_rec_run src/forward.c:2267-2270): after
// row `row` of its segment (0-based in the segment), every linear layer's state goes to the buffer `dst` (layer 0 first,
// the sequence's layer stride apart).
struct DnCk {
    float *dst;
    int row;
    int pad;
};
// One chunk of at most 64 tokens of the chunked DeltaNet: rows row0 .. row0 + cnt - 1 of segment seg (0-based in the
// segment).  A segment is cut every 64 rows and after every checkpoint row; ck: index of the checkpoint taken after the
// chunk's last row, or -1.
struct DnChunk {
    int seg, row0, cnt, ck;
};
// One segment of the open pass as the DeltaNet kernels see it.
struct DnSeg {
    float *state;   // the segment's sequence: state of linear layer 0 (conv part included)
    size_t lstride; // floats from one linear layer's state to the next
    int row0, n;    // rows of the pass: row0 .. row0 + n - 1
    int first;      // the segment starts at position 0: S is cleared first
    int chunk0;     // chunks of all earlier segments of the pass (the chunked DeltaNet's work records and chunk table)
    int nch;        // chunks of this segment
    int ck0, nck;   // its checkpoints in the pass's table, ascending by row
};

}  // namespace rq
