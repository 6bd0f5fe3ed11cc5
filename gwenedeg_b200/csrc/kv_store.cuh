// K / V rows -> cache tiles, and the synthetic cache fill.
//
// kv_store_kernel replaces the reference's kv_store (src/forward.c:1901): one CTA of head_dim threads per (row, KV head,
// K or V).  16-bit caches: fp32 -> f16, round to nearest even, saturating (f32_f16 :1325), K transposed inside its
// 16-position tile ([dim][pos]), V row-major ([pos][dim]).  q8 / q4: the row is rotated (x' = H D x: kvq_rot :1638),
// then each group of 32 rotated dims gets a bf16 scale with its magnitude rounded up (kvq_scale :1682) and integer
// levels n = rint(x' / d) (kvq_group :1690), written in the tile layouts of :1629-1634.  Divisions are IEEE
// divisions, as the definition states.
#pragma once
#include "attn_decode.cuh"

namespace rq {

// Element i of one row (x = the row's value for dim i; all HD threads of the CTA call this together) into position j
// of its tile, in the format fmt of that half; xs: HD floats of shared memory (rotation scratch of q8 / q4).
template <int HD>
__device__ __forceinline__ void kv_store_elem(uint8_t *tile, int fmt, int half, int j, int i, float x, float *xs) {
    if (fmt == KV_F16) {
        reinterpret_cast<uint16_t *>(tile)[half ? (size_t)j * HD + i : (size_t)i * ATT_T + j] = f32_to_f16_sat(x);
        return;
    }
    // rotation: signs, then butterflies h = 1, 2, 4, ... (each output one rounded add / subtract)
    __syncthreads();
    xs[i] = kvq_neg(i) ? -x : x;
    __syncthreads();
    for (int hh = 1; hh < HD; hh <<= 1) {
        float a = 0.0f, b = 0.0f;
        int jj = 0;
        if (i < HD / 2) {
            jj = (i / hh) * 2 * hh + (i % hh);
            a = xs[jj];
            b = xs[jj + hh];
        }
        __syncthreads();
        if (i < HD / 2) {
            xs[jj] = a + b;
            xs[jj + hh] = a - b;
        }
        __syncthreads();
    }
    x = xs[i];
    // one warp = one group of 32 dims: largest magnitude, and the first element that has it
    const int lane = i & 31, c = i >> 5, ng = HD / 32;
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    unsigned who = __ballot_sync(0xffffffffu, fabsf(x) == amax);
    float first = __shfl_sync(0xffffffffu, x, __ffs(who) - 1);
    const bool four = fmt == KV_Q4;
    float dq = four ? first / -8.0f : amax / 127.0f;
    if (amax == 0.0f) dq = 0.0f;  // (an all-zero group: the reference's m stays 0)
    uint32_t u = __float_as_uint(dq), sb = (u >> 16) + ((u & 0xffffu) != 0);
    if (!(sb & 0x7f80u)) sb = 0;
    const float d = bf16_bits_to_f32(sb & 0xffffu);
    float t = sb ? rintf(x / d) : 0.0f;
    const int lo = four ? -8 : -127, hi = four ? 7 : 127;
    int n = t < (float)lo ? lo : t > (float)hi ? hi : (int)t;
    uint16_t *scales = reinterpret_cast<uint16_t *>(tile + (size_t)(four ? 8 : 16) * HD);
    if (lane == 0) scales[half ? j * ng + c : c * ATT_T + j] = (uint16_t)sb;
    if (!four) {
        tile[half ? (size_t)j * HD + i : (size_t)i * ATT_T + j] = (uint8_t)(int8_t)n;
    } else if (!half) {  // K: byte of dim pair (2l, 2l + 1)
        int n0 = __shfl_sync(0xffffffffu, n, (2 * lane) & 31), n1 = __shfl_sync(0xffffffffu, n, (2 * lane + 1) & 31);
        if (lane < 16) tile[(size_t)(16 * c + lane) * ATT_T + j] = (uint8_t)((n0 + 8) | (n1 + 8) << 4);
    } else {  // V: byte l = dims 32c + l (low nibble), 32c + 16 + l (high)
        int n1 = __shfl_sync(0xffffffffu, n, (lane + 16) & 31);
        if (lane < 16) tile[(size_t)j * (HD / 2) + 16 * c + lane] = (uint8_t)((n + 8) | (n1 + 8) << 4);
    }
}

template <int HD>
__global__ void __launch_bounds__(HD) kv_store_kernel(const PassRow *__restrict__ rows, int layer, int n_kv, int kvt,
                                                      const float *__restrict__ k, const float *__restrict__ v, int *err) {
    const int r = blockIdx.x, h = blockIdx.y, half = blockIdx.z, i = threadIdx.x;
    const float *src = half ? v : k;
    if (!src) return;
    const PassRow row = rows[r];
    const int pos = row.pos;
    // (debug build) the position's tile lies inside one layer of the cache
    RQ_CHECK(pos >= 0 && (kv_tile_index(pos, h, n_kv) + 1) * (size_t)kv_tile_bytes(kvt, HD, half) <= (half ? row.lv : row.lk), err, 44);
    uint8_t *tile = const_cast<uint8_t *>(half ? row.v : row.k) + (size_t)layer * (half ? row.lv : row.lk) +
                    kv_tile_index(pos, h, n_kv) * (size_t)kv_tile_bytes(kvt, HD, half);
    __shared__ float xs[HD];
    kv_store_elem<HD>(tile, kv_fmt(kvt, half), half, pos % ATT_T, i, src[((size_t)r * n_kv + h) * HD + i], xs);
}

// Fused producer of the attention's inputs, the step right before the path in the reference's workers: per row and head
// the QK-norm (RMSNorm over the head, weight * (x / rms)) and the NeoX-style RoPE of the first `rd` dims for the row's
// position (qk_norm_rope, reference src/forward.c:1266; rope_row :1248; rmsnorm :886), then K and V go straight into
// the cache tiles (kv_store :1901) and q is left in place for the attention call.  The reference compiles this step
// with -Ofast and its vectorised libm, so agreement with it is to rounding (~1e-6), not to the bit.
// grid: (rows, n_heads + 2 n_kv): y < n_heads: a query head; next n_kv: a key head; last n_kv: a value head.
template <int HD>
__global__ void __launch_bounds__(HD) qk_norm_rope_store_kernel(const PassRow *__restrict__ rows, int layer, int n_kv, int n_heads, int kvt,
                                                                float *__restrict__ q, int qh, const float *__restrict__ k,
                                                                const float *__restrict__ v, const float *__restrict__ q_norm_w,
                                                                const float *__restrict__ k_norm_w, int rd, float log_theta, int *err) {
    const int r = blockIdx.x, y = blockIdx.y, i = threadIdx.x;
    const PassRow row = rows[r];
    const int pos = row.pos;
    RQ_CHECK(pos >= 0 && (kv_tile_index(pos, 0, n_kv) + 1) * (size_t)kv_tile_bytes(kvt, HD, 0) <= row.lk, err, 45);
    __shared__ float xs[HD];
    __shared__ float red[HD / 32];
    const int kind = y < n_heads ? 0 : y < n_heads + n_kv ? 1 : 2;  // q, k, v
    const int h = kind == 0 ? y : kind == 1 ? y - n_heads : y - n_heads - n_kv;
    float x;
    if (kind == 0) x = q[((size_t)r * n_heads + h) * qh + i];
    else x = (kind == 1 ? k : v)[((size_t)r * n_kv + h) * HD + i];
    if (kind < 2) {
        float ss = x * x;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((i & 31) == 0) red[i >> 5] = ss;
        __syncthreads();
        ss = 0.0f;
#pragma unroll
        for (int wv = 0; wv < HD / 32; wv++) ss += red[wv];
        ss = 1.0f / sqrtf(ss * (1.0f / HD) + 1e-6f);
        x = (kind == 0 ? q_norm_w : k_norm_w)[i] * (ss * x);
        xs[i] = x;
        __syncthreads();
        if (i < rd) {
            const int j = i < rd / 2 ? i : i - rd / 2;
            const float freq = expf(log_theta * (-(float)j / (float)(rd / 2)));
            float sn, cs;
            sincosf((float)pos * freq, &sn, &cs);
            const float a = xs[j], b = xs[j + rd / 2];
            x = i < rd / 2 ? a * cs - b * sn : a * sn + b * cs;
        }
    }
    if (kind == 0) {
        q[((size_t)r * n_heads + h) * qh + i] = x;
        return;
    }
    const int half = kind - 1;
    uint8_t *tile = const_cast<uint8_t *>(half ? row.v : row.k) + (size_t)layer * (half ? row.lv : row.lk) +
                    kv_tile_index(pos, h, n_kv) * (size_t)kv_tile_bytes(kvt, HD, half);
    kv_store_elem<HD>(tile, kv_fmt(kvt, half), half, pos % ATT_T, i, x, xs);
}

// ---- synthetic fill -----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__device__ __forceinline__ float normal_from(uint64_t r) {
    // Box-Muller from two 24-bit uniforms in (0, 1]
    float u1 = ((float)((r >> 40) & 0xffffff) + 1.0f) * (1.0f / 16777216.0f);
    float u2 = (float)((r >> 8) & 0xffffff) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * __logf(u1)) * __cosf(6.283185307f * u2);
}

// Fills `ntiles` whole tiles (from tile index 0 of one layer's K or V half) with seeded pseudo-random content:
// f16: N(0,1) values; q8 / q4: uniform levels, bf16 scales |N(0, 0.02)| with a non-zero exponent field.
// One thread per 2 bytes of cache.
__global__ void kv_fill_kernel(uint8_t *base, size_t ntiles, int fmt, int hd, uint64_t seed) {
    const size_t tb = (size_t)hd * (fmt == KV_Q8 ? 17 : fmt == KV_Q4 ? 9 : 32), words = ntiles * tb / 2;
    for (size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (size_t)gridDim.x * blockDim.x) {
        uint64_t r = mix64(seed ^ (w * 0xD6E8FEB86659FD93ull));
        uint16_t val;
        if (fmt == KV_F16) {
            val = f32_to_f16_sat(normal_from(r));
        } else {
            size_t off = (w * 2) % tb, qbytes = (size_t)hd * (fmt == KV_Q4 ? 8 : 16);
            if (off < qbytes) {
                if (fmt == KV_Q8) {
                    int a = (int)(r % 255) - 127, b = (int)((r >> 32) % 255) - 127;
                    val = (uint16_t)((uint8_t)(int8_t)a | ((uint16_t)(uint8_t)(int8_t)b << 8));
                } else
                    val = (uint16_t)(r & 0xffff);
            } else {
                float s = fabsf(normal_from(r)) * 0.02f;
                uint32_t sb = __float_as_uint(s) >> 16;
                if (!(sb & 0x7f80u)) sb = 0x3c00u;  // keep the exponent field non-zero
                val = (uint16_t)sb;
            }
        }
        reinterpret_cast<uint16_t *>(base)[w] = val;
    }
}

}  // namespace rq
