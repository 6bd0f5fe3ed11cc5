/* Test infrastructure, not product code: only tests/, the smoke check and the benchmark's CPU-baseline leg may
 * load this.  The CUDA library never links or calls it.
 *
 * A plain-C restatement of gwenedeg's attention hot path, written from the reference's arithmetic definitions
 * (every fp32 operation rounded, fused multiply-add where the reference uses one, nothing reassociated).  It is
 * built with -ffp-contract=off so the compiler neither fuses nor splits anything written here.  It exports the same
 * `gwo_*` C ABI as ref_harness.c (the reference's own code); tests pin this file against that library and against the
 * committed fixtures under tests/golden/ bit for bit.
 *
 * What each part follows in the reference (path inside its project : line):
 *   half conversion            src/forward.c:1325 (f32_f16), src/kquants.h:143 (fp16_to_f32)
 *   softmax exponential        src/forward.c:1301 (exp_att), constants src/kernels_avx512.h:41-50
 *   one vector x one block     src/forward.c:1346 (attention_vec), definition src/kernels_avx512.h:1109-1123
 *   merge of block partials    src/forward.c:1405 (att_combine)
 *   tile addressing            src/forward.c:1894 (kv_tile), src/kvtype.h:34 (kv_tile_bytes)
 *   row -> tile store          src/forward.c:1901 (kv_store), :1710 (kvq_store), :1690 (kvq_group), :1682 (kvq_scale)
 *   rotation                   src/forward.c:1638 (kvq_rot), :1662 (att_q_rot), :1672 (att_o_unrot)
 *   tile -> fp32               src/forward.c:1740 (kvq_block_f32), :1433 (kv_block_f32)
 *   sigmoid gate               src/forward.c:2011 (dn_sigmoid), :2291 (attn_gate)
 *   Gated DeltaNet             src/forward.c:2104 (dn_prep_part), :2044 (dn_conv), :2018 (dn_dot16), :2035 (dn_gates),
 *                              :2177-2272 (dn_p1 / dn_p2 / dn_rec_run), :2280 (dn_out), state layout :2090 (dn_sblock)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#define GWO_API __attribute__((visibility("default")))

enum { T = 16, P = 256, CHUNK = 32 };                 /* tile positions, block positions, dims per score chain */
enum { F32 = 0, F16 = 2, Q8 = 3, Q4 = 8, Q4K4 = 9 }; /* cache types handled here (runq.h RQ_KV_*) */

GWO_API int gwo_kind(void) { return 0; } /* 0: the restatement */
GWO_API int gwo_isa(void) { return 2; }
GWO_API int gwo_threads_init(int n) { (void)n; return 1; }

/* ------------------------------------------------------------------------------------------- element formats */
static int is_quant(int kvt) { return kvt == Q8 || kvt == Q4 || kvt == Q4K4; }
/* format of the K (half 0) or V (half 1) cache of a type: q4 keeps K in 8 bits */
static int half_fmt(int kvt, int half) { return kvt == Q4K4 ? Q4 : (kvt == Q4 && half == 0) ? Q8 : kvt; }
static int type_ok(int kvt, int hd) {
    if (kvt == F32) return hd % 16 == 0;
    if (kvt == F16) return hd % 32 == 0;
    return is_quant(kvt) && hd >= 32 && (hd & (hd - 1)) == 0;
}
static size_t tile_bytes(int kvt, int hd, int half) {
    int f = half_fmt(kvt, half);
    return (size_t)hd * (f == F32 ? 64 : f == Q8 ? 17 : f == Q4 ? 9 : 32);
}
GWO_API size_t gwo_kv_tile_bytes(int kvt, int hd, int is_v) { return tile_bytes(kvt, hd, is_v); }
GWO_API size_t gwo_kv_layer_bytes(int kvt, int kv_len, int n_kv, int hd, int is_v) {
    return (size_t)(kv_len / T) * n_kv * tile_bytes(kvt, hd, is_v);
}
/* index (in tiles) of the tile of position t, head h: blocks of 256 positions, heads inside a block, 16 tiles each */
static size_t tile_index(int t, int h, int n_kv) { return ((size_t)(t / P) * n_kv + h) * (P / T) + (size_t)(t % P) / T; }

static float bits_f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static uint16_t half_from_float(float f) {
    /* round to nearest even; >= 65520 saturates to 65504; subnormals exact; NaN stays quiet */
    uint32_t u = f_bits(f), sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu, h;
    if (a > 0x7f800000u) h = 0x7e00u | ((a >> 13) & 0x3ffu);
    else if (a >= 0x477ff000u) h = 0x7bffu;
    else if (a < 0x38800000u) h = (uint32_t)rintf(bits_f(a) * 0x1p24f);
    else {
        uint32_t n = a - 0x38000000u;
        h = (n + 0xfffu + ((n >> 13) & 1)) >> 13;
    }
    return (uint16_t)(sign | h);
}
static float float_from_half(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31, m = h & 0x3ffu;
    if (e == 0) return bits_f(sign | f_bits((float)m * 0x1p-24f));
    if (e == 31) return bits_f(sign | 0x7f800000u | (m << 13));
    return bits_f(sign | ((e + 112) << 23) | (m << 13));
}
static float float_from_bf16(uint16_t h) { return bits_f((uint32_t)h << 16); }

GWO_API void gwo_f32_f16(const float *x, uint16_t *h, size_t n) { for (size_t i = 0; i < n; i++) h[i] = half_from_float(x[i]); }
GWO_API void gwo_f16_f32(const uint16_t *h, float *x, size_t n) { for (size_t i = 0; i < n; i++) x[i] = float_from_half(h[i]); }

/* ------------------------------------------------------------------------------------------- exp and sigmoid */
static float exp_neg(float x) {
    /* e^x for x <= 0: clamp, n = rint(x log2 e), two-step Cody-Waite reduction, degree-5 polynomial, 2^n by the
     * exponent bits */
    if (!(x > -86.0f)) x = -86.0f;
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
    return bits_f(f_bits(y) + ((uint32_t)(int32_t)n << 23));
}
static float sigmoid_f(float x) {
    float e = exp_neg(-fabsf(x));
    float r = 1.0f / (1.0f + e);
    return x >= 0.0f ? r : e * r;
}
GWO_API void gwo_exp_att(const float *x, float *y, size_t n) { for (size_t i = 0; i < n; i++) y[i] = exp_neg(x[i]); }
GWO_API void gwo_sigmoid(const float *x, float *y, size_t n) { for (size_t i = 0; i < n; i++) y[i] = sigmoid_f(x[i]); }

/* sum of x[i] y[i] (n % 16 == 0) in 16 lanes, then the tree 8, 4, 2, 1 */
static float dot_lanes16(const float *x, const float *y, int n) {
    float a[16] = { 0 };
    for (int i = 0; i < n; i += 16)
        for (int j = 0; j < 16; j++) a[j] = fmaf(x[i + j], y[i + j], a[j]);
    for (int w = 8; w >= 1; w >>= 1)
        for (int j = 0; j < w; j++) a[j] = a[j] + a[j + w];
    return a[0];
}

/* ------------------------------------------------------------------------------------------- rotation + codec */
static int sign_flip(int i) { return (int)(((uint32_t)i * 0x9E3779B9u) >> 31); }

static void hadamard(float *x, int n, int inverse) {
    /* forward: signs then butterflies (H D x); inverse: butterflies then signs (D H x); unnormalised */
    if (!inverse)
        for (int i = 0; i < n; i++) if (sign_flip(i)) x[i] = -x[i];
    for (int h = 1; h < n; h <<= 1)
        for (int base = 0; base < n; base += 2 * h)
            for (int j = base; j < base + h; j++) {
                float a = x[j], b = x[j + h];
                x[j] = a + b;
                x[j + h] = a - b;
            }
    if (inverse)
        for (int i = 0; i < n; i++) if (sign_flip(i)) x[i] = -x[i];
}
static void scale_pow2(float *x, int n) {
    float f = 1.0f / (float)n;
    for (int i = 0; i < n; i++) x[i] = x[i] * f;
}
GWO_API void gwo_q_rot(int kvt, float *q, int nh, int stride, int hd) {
    if (!is_quant(kvt)) return;
    for (int h = 0; h < nh; h++) { hadamard(q + (size_t)h * stride, hd, 0); scale_pow2(q + (size_t)h * stride, hd); }
}
GWO_API void gwo_o_unrot(int kvt, float *o, int nv, int stride, int hd) {
    if (!is_quant(kvt)) return;
    for (int r = 0; r < nv; r++) { hadamard(o + (size_t)r * stride, hd, 1); scale_pow2(o + (size_t)r * stride, hd); }
}

static uint16_t scale_bits(float d) {
    /* bf16 with the magnitude rounded up; zero when the result has a zero exponent field */
    uint32_t u = f_bits(d), r = (u >> 16) + ((u & 0xffffu) != 0);
    return (r & 0x7f80u) ? (uint16_t)r : 0;
}
static void quant_group(int four_bit, const float *x, int8_t *lev, uint16_t *sc) {
    float amax = 0.0f, first = 0.0f;
    for (int i = 0; i < 32; i++) {
        float b = fabsf(x[i]);
        if (b > amax) { amax = b; first = x[i]; }
    }
    uint16_t s = scale_bits(four_bit ? first / -8.0f : amax / 127.0f);
    float d = float_from_bf16(s);
    int lo = four_bit ? -8 : -127, hi = four_bit ? 7 : 127;
    for (int i = 0; i < 32; i++) {
        float t = s ? rintf(x[i] / d) : 0.0f;
        lev[i] = (int8_t)(t < (float)lo ? lo : t > (float)hi ? hi : (int)t);
    }
    *sc = s;
}
static void store_quant_row(int fmt, uint8_t *tile, int j, int hd, const float *row, int is_v) {
    float x[512];
    memcpy(x, row, (size_t)hd * 4);
    hadamard(x, hd, 0);
    int four = fmt == Q4, ng = hd / 32;
    uint16_t *scales = (uint16_t *)(tile + (size_t)(four ? 8 : 16) * hd);
    for (int c = 0; c < ng; c++) {
        int8_t lev[32];
        uint16_t sc;
        quant_group(four, x + 32 * c, lev, &sc);
        if (!is_v) {
            scales[c * T + j] = sc;
            if (!four) for (int l = 0; l < 32; l++) tile[(size_t)(32 * c + l) * T + j] = (uint8_t)lev[l];
            else for (int l = 0; l < 16; l++)
                tile[(size_t)(16 * c + l) * T + j] = (uint8_t)((lev[2 * l] + 8) | (lev[2 * l + 1] + 8) << 4);
        } else {
            scales[j * ng + c] = sc;
            if (!four) memcpy(tile + (size_t)j * hd + 32 * c, lev, 32);
            else for (int l = 0; l < 16; l++)
                tile[(size_t)j * (hd / 2) + 16 * c + l] = (uint8_t)((lev[l] + 8) | (lev[l + 16] + 8) << 4);
        }
    }
}

GWO_API void gwo_qk_norm_rope(float *v, int n_heads, int stride, const float *norm_w, int hd, int rd, int pos, float log_theta) {
    /* per head: x <- w (x / rms(x)) with rms over hd dims (eps 1e-6 inside the root), then the pairs (j, j + rd/2) of
     * the first rd dims rotated by pos * theta^(-j / (rd/2)).  The reference compiles this part with -Ofast (its
     * vectorised libm): agreement is to rounding, not to the bit */
    for (int h = 0; h < n_heads; h++) {
        float *q = v + (size_t)h * stride, ss = 0.0f;
        for (int j = 0; j < hd; j++) ss += q[j] * q[j];
        ss = 1.0f / sqrtf(ss * (1.0f / hd) + 1e-6f);
        for (int j = 0; j < hd; j++) q[j] = norm_w[j] * (ss * q[j]);
        for (int j = 0; j < rd / 2; j++) {
            float freq = expf(log_theta * (-(float)j / (rd / 2)));
            float c = cosf(pos * freq), sn = sinf(pos * freq), x = q[j], y = q[j + rd / 2];
            q[j] = x * c - y * sn;
            q[j + rd / 2] = x * sn + y * c;
        }
    }
}

GWO_API void gwo_kv_store(int kvt, void *kl, void *vl, int pos, int n_kv, int hd, const float *k, const float *v) {
    int j = pos % T;
    for (int h = 0; h < n_kv; h++) {
        size_t ti = tile_index(pos, h, n_kv);
        for (int half = 0; half < 2; half++) {
            const float *row = half ? v : k;
            if (!row) continue;
            row += (size_t)h * hd;
            uint8_t *tile = (uint8_t *)(half ? vl : kl) + ti * tile_bytes(kvt, hd, half);
            int fmt = half_fmt(kvt, half);
            if (fmt == Q8 || fmt == Q4) { store_quant_row(fmt, tile, j, hd, row, half); continue; }
            for (int i = 0; i < hd; i++) {
                size_t e = half ? (size_t)j * hd + i : (size_t)i * T + j; /* V row-major, K dim-major */
                if (fmt == F16) ((uint16_t *)tile)[e] = half_from_float(row[i]);
                else ((float *)tile)[e] = row[i];
            }
        }
    }
}

/* element (position j of the tile, dim i) of a K or V tile as fp32 */
static float tile_elem(int fmt, const uint8_t *tile, int hd, int half, int j, int i) {
    int ng = hd / 32;
    if (fmt == F32) return ((const float *)tile)[half ? (size_t)j * hd + i : (size_t)i * T + j];
    if (fmt == F16) return float_from_half(((const uint16_t *)tile)[half ? (size_t)j * hd + i : (size_t)i * T + j]);
    const uint16_t *sc = (const uint16_t *)(tile + (size_t)(fmt == Q4 ? 8 : 16) * hd);
    float d = float_from_bf16(half ? sc[j * ng + i / 32] : sc[(i / 32) * T + j]);
    int n;
    if (fmt == Q8) n = (int8_t)tile[half ? (size_t)j * hd + i : (size_t)i * T + j];
    else if (!half) n = ((tile[(size_t)(i / 2) * T + j] >> (4 * (i & 1))) & 15) - 8;
    else n = ((tile[(size_t)j * (hd / 2) + (i / 32) * 16 + (i % 16)] >> (4 * ((i / 16) & 1))) & 15) - 8;
    return (float)n * d;
}

GWO_API void gwo_kv_block_f32(int kvt, const void *kb, const void *vb, int ntl, int hd, float *kf, float *vf) {
    /* fp32 tiles in the cache's own tile order: K [dim][16], V [16][dim] */
    for (int half = 0; half < 2; half++) {
        int fmt = half_fmt(kvt, half);
        size_t tb = tile_bytes(kvt, hd, half);
        float *dst = half ? vf : kf;
        const uint8_t *src = half ? vb : kb;
        for (int u = 0; u < ntl; u++)
            for (int j = 0; j < T; j++)
                for (int i = 0; i < hd; i++)
                    dst[(size_t)u * T * hd + (half ? (size_t)j * hd + i : (size_t)i * T + j)] =
                        tile_elem(fmt, src + u * tb, hd, half, j, i);
    }
}
GWO_API int gwo_kv_block_f32_simd(int kvt, const void *kb, const void *vb, int ntl, int hd, float *kf, float *vf) {
    (void)kvt; (void)kb; (void)vb; (void)ntl; (void)hd; (void)kf; (void)vf;
    return -1;
}

/* ------------------------------------------------------------------------------------------------ attention */
/* One (kv head, block) expanded to fp32: kd[dim][256] (dim-major) and vp[pos][hd] */
typedef struct { float *kd, *vp, *s; } BlockBuf;

static void load_block(BlockBuf *bb, int kvt, const uint8_t *kl, const uint8_t *vl, int n_kv, int hd, int g, int b, int n) {
    int ntl = (n + T - 1) / T;
    size_t ti0 = ((size_t)b * n_kv + g) * (P / T);
    for (int u = 0; u < ntl; u++) {
        const uint8_t *kt = kl + (ti0 + u) * tile_bytes(kvt, hd, 0), *vt = vl + (ti0 + u) * tile_bytes(kvt, hd, 1);
        int kf = half_fmt(kvt, 0), vf = half_fmt(kvt, 1);
        for (int j = 0; j < T; j++)
            for (int i = 0; i < hd; i++) {
                bb->kd[(size_t)i * P + u * T + j] = tile_elem(kf, kt, hd, 0, j, i);
                bb->vp[(size_t)(u * T + j) * hd + i] = tile_elem(vf, vt, hd, 1, j, i);
            }
    }
}

/* partial result of one query vector over the first n positions of a block: o[hd] unnormalised, *m, *l */
static void block_partial(const BlockBuf *bb, const float *q, int n, int hd, float scale, float *o, float *m_out, float *l_out) {
    float *s = bb->s;
    int np = (n + T - 1) / T * T;
    for (int c0 = 0; c0 < hd; c0 += CHUNK) {
        float acc[P];
        for (int t = 0; t < np; t++) acc[t] = 0.0f;
        for (int i = c0; i < c0 + CHUNK; i++) {
            const float *kr = bb->kd + (size_t)i * P;
            float qi = q[i];
            for (int t = 0; t < np; t++) acc[t] = fmaf(qi, kr[t], acc[t]);
        }
        for (int t = 0; t < np; t++) s[t] = c0 ? s[t] + acc[t] : acc[t];
    }
    for (int t = 0; t < np; t++) s[t] = s[t] * scale;
    float m = s[0];
    for (int t = 1; t < n; t++) if (s[t] > m) m = s[t];
    float lane[T] = { 0 };
    for (int t = 0; t < np; t++) {
        float e = t < n ? exp_neg(s[t] - m) : 0.0f;
        s[t] = e;
        lane[t % T] = lane[t % T] + e;
    }
    for (int w = T / 2; w >= 1; w >>= 1)
        for (int j = 0; j < w; j++) lane[j] = lane[j] + lane[j + w];
    for (int i = 0; i < hd; i++) o[i] = 0.0f;
    for (int t = 0; t < n; t++) {
        const float *vr = bb->vp + (size_t)t * hd;
        float e = s[t];
        for (int i = 0; i < hd; i++) o[i] = fmaf(e, vr[i], o[i]);
    }
    *m_out = m;
    *l_out = lane[0];
}

static void merge_partials(float *out, int nb, const float *part, size_t stride, int hd) {
    if (nb == 1) {
        float inv = 1.0f / part[hd + 1];
        for (int i = 0; i < hd; i++) out[i] = part[i] * inv;
        return;
    }
    float M = part[hd];
    for (int b = 1; b < nb; b++) if (part[b * stride + hd] > M) M = part[b * stride + hd];
    float L = 0.0f;
    for (int i = 0; i < hd; i++) out[i] = 0.0f;
    for (int b = 0; b < nb; b++) {
        const float *p = part + b * stride;
        float c = exp_neg(p[hd] - M);
        L = fmaf(c, p[hd + 1], L);
        for (int i = 0; i < hd; i++) out[i] = fmaf(c, p[i], out[i]);
    }
    float inv = 1.0f / L;
    for (int i = 0; i < hd; i++) out[i] = out[i] * inv;
}

GWO_API int gwo_attention(int kvt, const void *kl, const void *vl, int n_kv, int n_heads, int hd, int gated, int nrows,
                          const float *q, const int *np, float *out, float scale, int split, int rows_per_item) {
    /* same contract as ref_harness.c's gwo_attention; split / rows_per_item change nothing here: every vector is
     * its own per-block partials merged in block order, which is what both of the reference's schedules compute */
    (void)split; (void)rows_per_item;
    if (!type_ok(kvt, hd) || hd > 512 || n_kv < 1 || n_heads % n_kv || nrows < 1) return -1;
    int kv_mul = n_heads / n_kv, qh = gated ? 2 * hd : hd, nmax = 0;
    for (int r = 0; r < nrows; r++) nmax = np[r] > nmax ? np[r] : nmax;
    int nbmax = (nmax + P - 1) / P;
    size_t pst = (size_t)hd + 16;
    BlockBuf bb = { malloc((size_t)hd * P * 4), malloc((size_t)P * hd * 4), malloc(P * 4) };
    float *part = malloc((size_t)nrows * kv_mul * nbmax * pst * 4), *qr = malloc((size_t)hd * 4);
    for (int g = 0; g < n_kv; g++) {
        for (int b = 0; b < nbmax; b++) {
            int need = 0;
            for (int r = 0; r < nrows; r++) {
                int n = np[r] - b * P;
                n = n > P ? P : n;
                need = n > need ? n : need;
            }
            if (need <= 0) break;
            load_block(&bb, kvt, kl, vl, n_kv, hd, g, b, need);
            for (int r = 0; r < nrows; r++) {
                int n = np[r] - b * P;
                n = n > P ? P : n;
                if (n <= 0) continue;
                for (int x = 0; x < kv_mul; x++) {
                    int h = g * kv_mul + x;
                    memcpy(qr, q + ((size_t)r * n_heads + h) * qh, (size_t)hd * 4);
                    gwo_q_rot(kvt, qr, 1, hd, hd);
                    float *p = part + (((size_t)r * kv_mul + x) * nbmax + b) * pst;
                    block_partial(&bb, qr, n, hd, scale, p, p + hd, p + hd + 1);
                }
            }
        }
        for (int r = 0; r < nrows; r++)
            for (int x = 0; x < kv_mul; x++) {
                int h = g * kv_mul + x;
                float *o = out + ((size_t)r * n_heads + h) * hd;
                merge_partials(o, (np[r] + P - 1) / P, part + ((size_t)r * kv_mul + x) * nbmax * pst, pst, hd);
                gwo_o_unrot(kvt, o, 1, hd, hd);
                if (gated) {
                    const float *gate = q + ((size_t)r * n_heads + h) * qh + hd;
                    for (int i = 0; i < hd; i++) o[i] = o[i] * sigmoid_f(gate[i]);
                }
            }
    }
    free(bb.kd); free(bb.vp); free(bb.s); free(part); free(qr);
    return 0;
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

GWO_API double gwo_bench_decode(int kvt, int n_kv, int n_heads, int hd, int nseq, const void *const *kl,
                                const void *const *vl, const int *ctx, const float *q, float *out, float scale, int reps,
                                double *best) {
    /* q arrives rotated already (as the reference's call site has it); outputs are un-rotated here */
    double total = 0, bst = 1e30;
    for (int r = 0; r < reps; r++) {
        double t0 = now_s();
        for (int s = 0; s < nseq; s++) {
            int kv_mul = n_heads / n_kv, nb = (ctx[s] + P - 1) / P;
            size_t pst = (size_t)hd + 16;
            BlockBuf bb = { malloc((size_t)hd * P * 4), malloc((size_t)P * hd * 4), malloc(P * 4) };
            float *part = malloc((size_t)kv_mul * nb * pst * 4);
            for (int g = 0; g < n_kv; g++) {
                for (int b = 0; b < nb; b++) {
                    int n = ctx[s] - b * P > P ? P : ctx[s] - b * P;
                    load_block(&bb, kvt, kl[s], vl[s], n_kv, hd, g, b, n);
                    for (int x = 0; x < kv_mul; x++) {
                        float *p = part + ((size_t)x * nb + b) * pst;
                        block_partial(&bb, q + ((size_t)s * n_heads + g * kv_mul + x) * hd, n, hd, scale, p, p + hd, p + hd + 1);
                    }
                }
                for (int x = 0; x < kv_mul; x++) {
                    float *o = out + ((size_t)s * n_heads + g * kv_mul + x) * hd;
                    merge_partials(o, nb, part + (size_t)x * nb * pst, pst, hd);
                    gwo_o_unrot(kvt, o, 1, hd, hd);
                }
            }
            free(bb.kd); free(bb.vp); free(bb.s); free(part);
        }
        double dt = now_s() - t0;
        total += dt;
        bst = dt < bst ? dt : bst;
    }
    if (best) *best = bst;
    return total;
}

GWO_API double gwo_bench_prefill(int kvt, const void *kl, const void *vl, int n_kv, int n_heads, int hd, int nrows,
                                 const float *q, const int *np, float *out, float scale, int reps, double *best) {
    double total = 0, bst = 1e30;
    for (int r = 0; r < reps; r++) {
        double t0 = now_s();
        if (gwo_attention(kvt, kl, vl, n_kv, n_heads, hd, 0, nrows, q, np, out, scale, 0, 0)) return -1;
        double dt = now_s() - t0;
        total += dt;
        bst = dt < bst ? dt : bst;
    }
    if (best) *best = bst;
    return total;
}

/* ------------------------------------------------------------------------------------------ Gated DeltaNet */
typedef struct {
    int nk, nv, dk, dv, conv, conv_dim, vdim, lw;
    size_t conv_floats, state_floats;
    const float *w_conv, *w_a, *w_dt, *w_norm;
} Dn;

GWO_API void *gwo_dn_new(int nk, int nv, int dk, int dv, int conv, const float *ssm_conv, const float *ssm_a,
                         const float *ssm_dt, const float *ssm_norm) {
    Dn *d = calloc(1, sizeof(Dn));
    d->nk = nk; d->nv = nv; d->dk = dk; d->dv = dv; d->conv = conv;
    d->conv_dim = 2 * nk * dk + nv * dv;
    d->vdim = nv * dv;
    d->lw = d->conv_dim + d->vdim + 2 * nv; /* [q | k | v | z | eg | beta] */
    d->conv_floats = ((size_t)(conv - 1) * d->conv_dim + 15) / 16 * 16;
    d->state_floats = d->conv_floats + (size_t)nv * dk * dv;
    d->w_conv = ssm_conv; d->w_a = ssm_a; d->w_dt = ssm_dt; d->w_norm = ssm_norm;
    return d;
}
GWO_API void gwo_dn_free(void *p) { free(p); }
GWO_API size_t gwo_dn_state_floats(void *p) { return ((Dn *)p)->state_floats; }
GWO_API size_t gwo_dn_conv_floats(void *p) { return ((Dn *)p)->conv_floats; }
GWO_API int gwo_dn_row_floats(void *p) { return ((Dn *)p)->lw; }

GWO_API void gwo_dn_rec(void *p, float *state, int first, const float *rows, size_t rs, float *out, size_t os, int n) {
    /* per value head h and value column v, tokens in order (S is stored in blocks of 32 columns, [dk][32] each):
     *   u = sum_k (S[k][v] eg) key[k];  u = (val[v] - u) beta;  S[k][v] = fma(key[k], u, S[k][v] eg);
     *   o[v] = sum_k S[k][v] query[k]   (sums over k in order, fused multiply-adds from zero) */
    const Dn *d = p;
    int dk = d->dk, dv = d->dv;
    for (int h = 0; h < d->nv; h++) {
        size_t oq = (size_t)(h % d->nk) * dk, ok = (size_t)d->nk * dk + oq, ov = (size_t)2 * d->nk * dk + (size_t)h * dv;
        size_t oe = (size_t)d->conv_dim + d->vdim + h, ob = oe + d->nv;
        float *Sh = state + d->conv_floats + (size_t)h * dk * dv;
        if (first) memset(Sh, 0, (size_t)dk * dv * 4);
        for (int t = 0; t < n; t++) {
            const float *r = rows + (size_t)t * rs;
            float eg = r[oe], beta = r[ob];
            for (int v = 0; v < dv; v++) {
                float *S = Sh + (size_t)(v / 32) * dk * 32 + (v % 32); /* element k at S[k * 32] */
                float u = 0.0f;
                for (int k = 0; k < dk; k++) u = fmaf(S[(size_t)k * 32] * eg, r[ok + k], u);
                u = (r[ov + v] - u) * beta;
                float o = 0.0f;
                for (int k = 0; k < dk; k++) {
                    float sv = fmaf(r[ok + k], u, S[(size_t)k * 32] * eg);
                    S[(size_t)k * 32] = sv;
                    o = fmaf(sv, r[oq + k], o);
                }
                out[(size_t)t * os + (size_t)h * dv + v] = o;
            }
        }
    }
}

static void conv_silu(float *out, const float *x, float *st, const float *w, int n, int K) {
    for (int i = 0; i < n; i++) out[i] = w[i] * st[i];
    for (int j = 1; j < K - 1; j++)
        for (int i = 0; i < n; i++) out[i] = fmaf(w[(size_t)j * n + i], st[(size_t)j * n + i], out[i]);
    for (int i = 0; i < n; i++) out[i] = fmaf(w[(size_t)(K - 1) * n + i], x[i], out[i]);
    memmove(st, st + n, (size_t)(K - 2) * n * 4);
    memcpy(st + (size_t)(K - 2) * n, x, (size_t)n * 4);
    for (int i = 0; i < n; i++) out[i] = out[i] * sigmoid_f(out[i]);
}

GWO_API void gwo_dn_prep(void *p, float *state, int first, float *rows, size_t rs, int n) {
    /* per token: channel groups (q and k of each key head, v of each value head): causal conv over the last `conv`
     * inputs + SiLU; q, k L2-normalised (eps inside the root), q also times 1/sqrt(dk); eg = exp(A softplus(a + dt)),
     * beta = sigmoid(b) */
    const Dn *d = p;
    int K = d->conv;
    float buf[512];
    for (int t = 0; t < n; t++) {
        float *row = rows + (size_t)t * rs;
        for (int grp = 0; grp < 2 * d->nk + d->nv; grp++) {
            int kind = grp < d->nk ? 0 : grp < 2 * d->nk ? 1 : 2, h = kind == 0 ? grp : kind == 1 ? grp - d->nk : grp - 2 * d->nk;
            size_t c0 = kind == 0 ? (size_t)h * d->dk : kind == 1 ? (size_t)d->nk * d->dk + (size_t)h * d->dk
                                                                   : (size_t)2 * d->nk * d->dk + (size_t)h * d->dv;
            int cn = kind < 2 ? d->dk : d->dv;
            float *sg = state + (size_t)(K - 1) * c0;
            if (first && t == 0) memset(sg, 0, (size_t)(K - 1) * cn * 4);
            conv_silu(buf, row + c0, sg, d->w_conv + (size_t)K * c0, cn, K);
            if (kind < 2) {
                float inv = 1.0f / sqrtf(dot_lanes16(buf, buf, d->dk) + 1e-6f);
                if (kind == 0) {
                    float sc = 1.0f / sqrtf((float)d->dk);
                    for (int i = 0; i < cn; i++) buf[i] = buf[i] * inv * sc;
                } else
                    for (int i = 0; i < cn; i++) buf[i] = buf[i] * inv;
            } else {
                float *ab = row + d->conv_dim + d->vdim + h;
                float x = ab[0] + d->w_dt[h];
                float sp = x > 20.0f ? x : log1pf(expf(x));
                ab[0] = expf(d->w_a[h] * sp);
                ab[d->nv] = sigmoid_f(ab[d->nv]);
            }
            memcpy(row + c0, buf, (size_t)cn * 4);
        }
    }
}

GWO_API void gwo_dn_out(void *p, const float *rows, size_t rs, float *out, size_t os, int n) {
    const Dn *d = p;
    int dv = d->dv;
    for (int t = 0; t < n; t++)
        for (int h = 0; h < d->nv; h++) {
            float *o = out + (size_t)t * os + (size_t)h * dv;
            const float *z = rows + (size_t)t * rs + d->conv_dim + (size_t)h * dv;
            float ss = 1.0f / sqrtf(dot_lanes16(o, o, dv) * (1.0f / dv) + 1e-6f);
            for (int j = 0; j < dv; j++) o[j] = d->w_norm[j] * (ss * o[j]) * (z[j] * sigmoid_f(z[j]));
        }
}

GWO_API double gwo_bench_dn(void *p, int nseq, float *const *state, const float *const *rows, size_t rs, float *const *out,
                            size_t os, int n, int reps, double *best) {
    double total = 0, bst = 1e30;
    for (int r = 0; r < reps; r++) {
        double t0 = now_s();
        for (int s = 0; s < nseq; s++) gwo_dn_rec(p, state[s], 1, rows[s], rs, out[s], os, n);
        double dt = now_s() - t0;
        total += dt;
        bst = dt < bst ? dt : bst;
    }
    if (best) *best = bst;
    return total;
}

/* ------------------------------------------------------------------------------------------ activation quantiser */
/* The quantiser the reference runs on the attention's output rows before the `wo` matmul (quantize, reference
 * src/forward.c:803-836): per group of gs values scale = wmax * (1 / 127) with wmax the largest magnitude, inv = 127 / wmax,
 * level = (int) trunc(x inv + copysign(0.49999997, x inv)); an all-zero group gives zero levels. */
GWO_API void gwo_quantize(const float *x, int n, int gs, int8_t *q, float *s) {
    for (int g = 0; g < n / gs; g++) {
        const float *xg = x + (size_t)g * gs;
        float wmax = 0.0f;
        for (int i = 0; i < gs; i++) {
            float v = fabsf(xg[i]);
            if (v > wmax) wmax = v;
        }
        s[g] = wmax * (1.0f / 127.0f);
        if (!(wmax > 0.0f)) {
            memset(q + (size_t)g * gs, 0, (size_t)gs);
            continue;
        }
        float inv = 127.0f / wmax;
        for (int i = 0; i < gs; i++) {
            float v = xg[i] * inv;
            q[(size_t)g * gs + i] = (int8_t)(int32_t)(v + copysignf(0.49999997f, v));
        }
    }
}
