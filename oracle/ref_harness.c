/* Test infrastructure, not product code.
 *
 * Wrappers around gwenedeg's own attention / KV-codec / Gated DeltaNet functions, which are `static` in the
 * reference's src/forward.c.  This translation unit textually includes that file (path given by -DGW_REF_FORWARD_C
 * at build time; see oracle/Makefile) so every static function is reachable, and exports a small C ABI (`gwo_*`)
 * that the test-suite and the CPU-baseline leg of the benchmark call through ctypes.  Nothing of the reference is
 * copied here: only calls into it.  The same `gwo_*` names are exported by the independent restatement in
 * gw_oracle.c, so a test can run either one and compare them bit for bit.
 *
 * Functions reached (reference src/forward.c): kv_store :1901, kvq_block_f32 :1740, kv_block_f32 :1433,
 * att_q_rot :1662, att_o_unrot :1672, attention_part :1806, attention_kv :1871, att_combine :1405,
 * attn_gate :2291, exp_att :1301, f32_f16 :1325, dn_prep_part :2104, dn_rec_run :2224, dn_out :2280;
 * thread pool rq_threads_init / rq_parallel (src/threads.c:180, src/threads.h:329).
 */
#ifndef GW_REF_FORWARD_C
#error "build with -DGW_REF_FORWARD_C='\"<reference>/src/forward.c\"' (oracle/Makefile does)"
#endif
#include GW_REF_FORWARD_C

#include <stdatomic.h>
#include <time.h>

#define GWO_API __attribute__((visibility("default")))

GWO_API int gwo_kind(void) { return 1; } /* 1: the reference's own code */

GWO_API int gwo_isa(void) {
    /* bit 0: the AVX-512 attention kernels are compiled in, bit 1: fast fmaf */
    int r = 0;
#ifdef RUNQ_ATT512
    r |= 1;
#endif
#ifdef FP_FAST_FMAF
    r |= 2;
#endif
    return r;
}

GWO_API size_t gwo_kv_tile_bytes(int kvt, int hd, int is_v) { return kv_tile_bytes(kvt, hd, is_v); }

GWO_API size_t gwo_kv_layer_bytes(int kvt, int kv_len, int n_kv, int hd, int is_v) {
    return (size_t)(kv_len / ATT_T) * n_kv * kv_tile_bytes(kvt, hd, is_v);
}

GWO_API void gwo_f32_f16(const float *x, uint16_t *h, size_t n) {
    for (size_t i = 0; i < n; i++) h[i] = f32_f16(x[i]);
}

GWO_API void gwo_f16_f32(const uint16_t *h, float *x, size_t n) {
    for (size_t i = 0; i < n; i++) x[i] = fp16_to_f32(h[i]);
}

ATT_EXACT GWO_API void gwo_exp_att(const float *x, float *y, size_t n) { RQ_FP_EXACT
    for (size_t i = 0; i < n; i++) y[i] = exp_att(x[i]);
}

/* (DN_EXACT as every reference function that inlines dn_sigmoid: the division must stay a division) */
DN_EXACT GWO_API void gwo_sigmoid(const float *x, float *y, size_t n) { RQ_FP_EXACT
    for (size_t i = 0; i < n; i++) y[i] = dn_sigmoid(x[i]);
}

/* QK-norm (RMSNorm per head) + NeoX RoPE of one row's heads, in place (rope_row :1248, qk_norm_rope :1266): v holds
 * n_heads heads `stride` floats apart; the first rd dims of each head are rotated for position pos */
GWO_API void gwo_qk_norm_rope(float *v, int n_heads, int stride, const float *norm_w, int hd, int rd, int pos, float log_theta) {
    float cs[512];
    rope_row(cs, rd, pos, log_theta);
    qk_norm_rope(v, n_heads, stride, norm_w, hd, cs, rd);
}

/* K and / or V rows of all kv heads of one position (k, v: [n_kv][hd] floats, either may be NULL) */
GWO_API void gwo_kv_store(int kvt, void *kl, void *vl, int pos, int n_kv, int hd, const float *k, const float *v) {
    for (int h = 0; h < n_kv; h++)
        kv_store(kvt, kl, vl, pos, h, n_kv, hd, k ? k + (size_t)h * hd : NULL, v ? v + (size_t)h * hd : NULL);
}

/* the first ntl tiles of one (kv head, block) as fp32 tiles (K [dim][16], V [16][dim] per tile) */
GWO_API void gwo_kv_block_f32(int kvt, const void *kb, const void *vb, int ntl, int hd, float *kf, float *vf) {
    if (kv_quant(kvt))
        kvq_block_f32(kvt, kf, vf, kb, vb, ntl, hd);
    else if (kvt == KV_F32) {
        memcpy(kf, kb, (size_t)ntl * ATT_T * hd * 4);
        memcpy(vf, vb, (size_t)ntl * ATT_T * hd * 4);
    } else
        kv_block_f32(kvt, kf, vf, kb, vb, ntl, hd);
}

#ifdef RUNQ_ATT512
/* the AVX-512 twin of the q8 / q4 conversion (kernels_avx512.h:1529) */
GWO_API int gwo_kv_block_f32_simd(int kvt, const void *kb, const void *vb, int ntl, int hd, float *kf, float *vf) {
    if (!kv_quant(kvt) || !att512_ok(hd)) return -1;
    att512_q_f32(kvt, kf, vf, kb, vb, ntl, hd);
    return 0;
}
#else
GWO_API int gwo_kv_block_f32_simd(int kvt, const void *kb, const void *vb, int ntl, int hd, float *kf, float *vf) {
    (void)kvt; (void)kb; (void)vb; (void)ntl; (void)hd; (void)kf; (void)vf;
    return -1;
}
#endif

GWO_API void gwo_q_rot(int kvt, float *q, int nh, int stride, int hd) { att_q_rot(kvt, q, nh, stride, hd); }

GWO_API void gwo_o_unrot(int kvt, float *o, int nv, int stride, int hd) {
    for (int r = 0; r < nv; r++) {
        float *p = o + (size_t)r * stride;
        att_o_unrot(kvt, &p, 1, hd);
    }
}

/* Attention of nrows query rows of ONE sequence over one layer's cache (kl / vl: the layer's K and V).
 * q: [nrows][n_heads][qh] with qh = hd, or 2 hd when gated ([q | gate] per head); np[r]: positions row r attends
 * (0..np[r]-1); out: [nrows][n_heads][hd].  split 0: attention_kv per (row block, kv head) as prefill_worker
 * (forward.c:3096-3146); split 1: one attention_part per (kv head, 256-position block) and att_combine, as
 * decode_worker (forward.c:2691-2711).  q8 / q4: q rotated first, outputs un-rotated, then the gate, as the call
 * sites do.  rows_per_item <= 0: the reference's att_rows = min(64 / kv_mul, 6). */
typedef struct {
    int kvt, n_kv, n_heads, hd, qh, nrows, split, rows_per_item;
    const void *kl, *vl;
    const float *q;
    float *qr; /* rotated copy of q (quantised types), else NULL */
    const int *np;
    float *out;
    float scale;
    int gated;
    /* items */
    int n_items;
    atomic_int next;
    int *item_rb, *item_g; /* row block, kv head (sorted longest first) */
    int nbmax;
    /* per-thread scratch */
    float **S, **part, **conv;
} AttJob;

static void att_item(AttJob *j, int rb, int g, int tid) {
    int kv_mul = j->n_heads / j->n_kv, hd = j->hd, qh = j->qh;
    int rpi = j->rows_per_item, r0 = rb * rpi, r1 = r0 + rpi < j->nrows ? r0 + rpi : j->nrows;
    const float *qsrc = j->qr ? j->qr : j->q;
    const float *qv[ATT_NV_MAX];
    float *ov[ATT_NV_MAX], *pv[ATT_NV_MAX];
    int npv[ATT_NV_MAX], nv = 0, nmax = 0;
    size_t pst = ATT_PSTRIDE(hd);
    for (int r = r0; r < r1; r++)
        for (int x = 0; x < kv_mul; x++) {
            int h = g * kv_mul + x;
            qv[nv] = qsrc + ((size_t)r * j->n_heads + h) * qh;
            ov[nv] = j->out + ((size_t)r * j->n_heads + h) * hd;
            npv[nv] = j->np[r];
            nmax = j->np[r] > nmax ? j->np[r] : nmax;
            nv++;
        }
    size_t ts = (size_t)ATT_T * hd, o = kv_tile(0, g, j->n_kv, hd), bs = (size_t)j->n_kv * ATT_P * hd;
    const char *kt = (const char *)j->kl + o / ts * kv_tile_bytes(j->kvt, hd, 0);
    const char *vt = (const char *)j->vl + o / ts * kv_tile_bytes(j->kvt, hd, 1);
    int nb = (nmax + ATT_P - 1) / ATT_P;
    if (!j->split || nb == 1) {
        attention_kv(j->kvt, nv, qv, ov, npv, kt, vt, bs, hd, j->scale, j->S[tid], j->part[tid], j->conv[tid]);
    } else {
        for (int r = 0; r < nv; r++) pv[r] = j->part[tid] + (size_t)r * nb * pst;
        for (int b = 0; b < nb; b++)
            attention_part(j->kvt, nv, qv, ov, pv, npv, b, b + 1, kt, vt, bs, hd, j->scale, j->S[tid], j->conv[tid]);
        for (int r = 0; r < nv; r++) att_combine(ov[r], (npv[r] + ATT_P - 1) / ATT_P, pv[r], pst, hd);
    }
    att_o_unrot(j->kvt, ov, nv, hd);
    if (j->gated)
        for (int r = 0; r < nv; r++) attn_gate(ov[r], qv[r] + hd, hd);
}

static void att_worker(void *arg, int tid, int nt) {
    (void)nt;
    AttJob *j = arg;
    for (;;) {
        int it = atomic_fetch_add(&j->next, 1);
        if (it >= j->n_items) break;
        att_item(j, j->item_rb[it], j->item_g[it], tid);
    }
}

static int g_threads = 0;

GWO_API int gwo_threads_init(int n) {
    /* the reference's pool; its size is fixed by the first call in a process */
    if (!g_threads) {
        rq_threads_init(n);
        g_threads = rq_threads_fix();
    }
    return g_threads;
}

static int att_job_run(AttJob *j) {
    int nt = gwo_threads_init(0);
    int kv_mul = j->n_heads / j->n_kv;
    if (j->rows_per_item <= 0) j->rows_per_item = ATT_NV_MAX / kv_mul < ATT_ROWS ? ATT_NV_MAX / kv_mul : ATT_ROWS;
    if (j->rows_per_item * kv_mul > ATT_NV_MAX) return -1;
    int nrb = (j->nrows + j->rows_per_item - 1) / j->rows_per_item;
    j->n_items = nrb * j->n_kv;
    j->item_rb = malloc(sizeof(int) * j->n_items);
    j->item_g = malloc(sizeof(int) * j->n_items);
    /* row blocks longest first (prefill_plan, forward.c:3273): the rows come in ascending position order from the
     * callers here, so walk them backwards */
    int *len = malloc(sizeof(int) * nrb), *ord = malloc(sizeof(int) * nrb);
    j->nbmax = 1;
    for (int rb = 0; rb < nrb; rb++) {
        int m = 0;
        for (int r = rb * j->rows_per_item; r < (rb + 1) * j->rows_per_item && r < j->nrows; r++)
            m = j->np[r] > m ? j->np[r] : m;
        len[rb] = m;
        ord[rb] = rb;
        int nb = (m + ATT_P - 1) / ATT_P;
        j->nbmax = nb > j->nbmax ? nb : j->nbmax;
    }
    for (int a = 1; a < nrb; a++) { /* insertion sort, descending, stable */
        int x = ord[a], b = a;
        while (b > 0 && len[ord[b - 1]] < len[x]) { ord[b] = ord[b - 1]; b--; }
        ord[b] = x;
    }
    int it = 0;
    for (int a = 0; a < nrb; a++)
        for (int g = 0; g < j->n_kv; g++) { j->item_rb[it] = ord[a]; j->item_g[it] = g; it++; }
    free(len); free(ord);
    j->S = malloc(sizeof(float *) * nt);
    j->part = malloc(sizeof(float *) * nt);
    j->conv = malloc(sizeof(float *) * nt);
    size_t ns = att_scores_floats(ATT_NV_MAX, j->nbmax);
    if (ns < (size_t)ATT_P) ns = ATT_P;
    for (int t = 0; t < nt; t++) {
        j->S[t] = aligned_alloc(64, ns * 4);
        j->part[t] = aligned_alloc(64, (size_t)ATT_NV_MAX * j->nbmax * ATT_PSTRIDE(j->hd) * 4);
        j->conv[t] = aligned_alloc(64, (size_t)2 * ATT_P * j->hd * 4);
    }
    return 0;
}

static void att_job_free(AttJob *j) {
    int nt = g_threads;
    for (int t = 0; t < nt; t++) { free(j->S[t]); free(j->part[t]); free(j->conv[t]); }
    free(j->S); free(j->part); free(j->conv); free(j->item_rb); free(j->item_g); free(j->qr);
}

GWO_API int gwo_attention(int kvt, const void *kl, const void *vl, int n_kv, int n_heads, int hd, int gated, int nrows,
                          const float *q, const int *np, float *out, float scale, int split, int rows_per_item) {
    if (!kv_type_fits(kvt, hd) || (kvt & KV_DOT) || n_kv < 1 || n_heads % n_kv || nrows < 1) return -1;
    AttJob j = { .kvt = kvt, .n_kv = n_kv, .n_heads = n_heads, .hd = hd, .qh = gated ? 2 * hd : hd, .nrows = nrows,
                 .split = split, .rows_per_item = rows_per_item, .kl = kl, .vl = vl, .q = q, .np = np, .out = out,
                 .scale = scale, .gated = gated };
    if (kv_quant(kvt)) {
        size_t n = (size_t)nrows * n_heads * j.qh;
        j.qr = malloc(n * 4);
        memcpy(j.qr, q, n * 4);
        att_q_rot(kvt, j.qr, nrows * n_heads, j.qh, hd);
    }
    if (att_job_run(&j)) { free(j.qr); return -1; }
    atomic_store(&j.next, 0);
    rq_parallel(att_worker, &j);
    att_job_free(&j);
    return 0;
}

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

/* ---- CPU-baseline timing of batched decode: nseq sequences, one query row each, with the reference's work items
 * (kv head, 256-position block) -> attention_part, then att_combine per vector (forward.c:2691-2711 / :3600-3616),
 * on the reference's thread pool.  kl[s] / vl[s]: that sequence's layer cache; ctx[s] its length.  Returns seconds
 * for `reps` passes (best single pass in *best). */
typedef struct {
    int kvt, n_kv, n_heads, hd, nseq;
    const void *const *kl, *const *vl;
    const int *ctx;
    const float *q; /* [nseq][n_heads][hd], already rotated for q8 / q4 */
    float *out;     /* [nseq][n_heads][hd] */
    float scale;
    int n_items;
    int *it_s, *it_g, *it_b;
    size_t *part_off; /* per sequence: offset into part */
    float *part;
    atomic_int next;
    atomic_int *left; /* per (seq, kv head): blocks still running */
    float **S, **conv;
} DecJob;

static void dec_worker(void *arg, int tid, int nt) {
    (void)nt;
    DecJob *j = arg;
    int kv_mul = j->n_heads / j->n_kv, hd = j->hd;
    size_t pst = ATT_PSTRIDE(hd), ts = (size_t)ATT_T * hd, bs = (size_t)j->n_kv * ATT_P * hd;
    for (;;) {
        int it = atomic_fetch_add(&j->next, 1);
        if (it >= j->n_items) break;
        int s = j->it_s[it], g = j->it_g[it], b = j->it_b[it];
        int n = j->ctx[s], nb = (n + ATT_P - 1) / ATT_P;
        const float *qv[ATT_NV_MAX];
        float *ov[ATT_NV_MAX], *pv[ATT_NV_MAX];
        int npv[ATT_NV_MAX];
        for (int r = 0; r < kv_mul; r++) {
            int h = g * kv_mul + r;
            qv[r] = j->q + ((size_t)s * j->n_heads + h) * hd;
            ov[r] = j->out + ((size_t)s * j->n_heads + h) * hd;
            pv[r] = j->part + j->part_off[s] + ((size_t)h * nb) * pst;
            npv[r] = n;
        }
        size_t o = kv_tile(0, g, j->n_kv, hd);
        const char *kt = (const char *)j->kl[s] + o / ts * kv_tile_bytes(j->kvt, hd, 0);
        const char *vt = (const char *)j->vl[s] + o / ts * kv_tile_bytes(j->kvt, hd, 1);
        attention_part(j->kvt, kv_mul, qv, ov, nb == 1 ? NULL : pv, npv, b, b + 1, kt, vt, bs, hd, j->scale, j->S[tid],
                       j->conv[tid]);
        if (nb > 1) {
            if (atomic_fetch_sub(&j->left[s * j->n_kv + g], 1) != 1) continue;
            for (int r = 0; r < kv_mul; r++) att_combine(ov[r], nb, pv[r], pst, hd);
        }
        att_o_unrot(j->kvt, ov, kv_mul, hd);
    }
}

GWO_API double gwo_bench_decode(int kvt, int n_kv, int n_heads, int hd, int nseq, const void *const *kl,
                                const void *const *vl, const int *ctx, const float *q, float *out, float scale, int reps,
                                double *best) {
    int nt = gwo_threads_init(0);
    DecJob j = { .kvt = kvt, .n_kv = n_kv, .n_heads = n_heads, .hd = hd, .nseq = nseq, .kl = kl, .vl = vl, .ctx = ctx,
                 .q = q, .out = out, .scale = scale };
    size_t pst = ATT_PSTRIDE(hd), tot = 0;
    j.part_off = malloc(sizeof(size_t) * nseq);
    int ni = 0;
    for (int s = 0; s < nseq; s++) {
        int nb = (ctx[s] + ATT_P - 1) / ATT_P;
        j.part_off[s] = tot;
        tot += (size_t)n_heads * nb * pst;
        ni += nb * n_kv;
    }
    j.n_items = ni;
    j.it_s = malloc(sizeof(int) * ni); j.it_g = malloc(sizeof(int) * ni); j.it_b = malloc(sizeof(int) * ni);
    ni = 0;
    for (int s = 0; s < nseq; s++)
        for (int g = 0; g < n_kv; g++)
            for (int b = 0; b < (ctx[s] + ATT_P - 1) / ATT_P; b++) { j.it_s[ni] = s; j.it_g[ni] = g; j.it_b[ni] = b; ni++; }
    j.part = aligned_alloc(64, (tot * 4 + 63) / 64 * 64);
    j.left = malloc(sizeof(atomic_int) * nseq * n_kv);
    j.S = malloc(sizeof(float *) * nt); j.conv = malloc(sizeof(float *) * nt);
    size_t ns = att_scores_floats(ATT_NV_MAX, 1);
    if (ns < (size_t)ATT_NV_MAX * ATT_P) ns = (size_t)ATT_NV_MAX * ATT_P;
    for (int t = 0; t < nt; t++) {
        j.S[t] = aligned_alloc(64, ns * 4);
        j.conv[t] = aligned_alloc(64, (size_t)2 * ATT_P * hd * 4);
    }
    double total = 0, bst = 1e30;
    for (int r = 0; r < reps; r++) {
        for (int s = 0; s < nseq; s++)
            for (int g = 0; g < n_kv; g++) atomic_store(&j.left[s * n_kv + g], (ctx[s] + ATT_P - 1) / ATT_P);
        atomic_store(&j.next, 0);
        double t0 = now_s();
        rq_parallel(dec_worker, &j);
        double dt = now_s() - t0;
        total += dt;
        bst = dt < bst ? dt : bst;
    }
    if (best) *best = bst;
    for (int t = 0; t < nt; t++) { free(j.S[t]); free(j.conv[t]); }
    free(j.S); free(j.conv); free(j.left); free(j.part); free(j.it_s); free(j.it_g); free(j.it_b); free(j.part_off);
    return total;
}

/* timed prefill attention of one sequence: the items of gwo_attention (split 0); seconds for reps passes */
GWO_API double gwo_bench_prefill(int kvt, const void *kl, const void *vl, int n_kv, int n_heads, int hd, int nrows,
                                 const float *q, const int *np, float *out, float scale, int reps, double *best) {
    AttJob j = { .kvt = kvt, .n_kv = n_kv, .n_heads = n_heads, .hd = hd, .qh = hd, .nrows = nrows, .kl = kl, .vl = vl,
                 .q = q, .np = np, .out = out, .scale = scale };
    if (att_job_run(&j)) return -1;
    double total = 0, bst = 1e30;
    for (int r = 0; r < reps; r++) {
        atomic_store(&j.next, 0);
        double t0 = now_s();
        rq_parallel(att_worker, &j);
        double dt = now_s() - t0;
        total += dt;
        bst = dt < bst ? dt : bst;
    }
    if (best) *best = bst;
    att_job_free(&j);
    return total;
}

/* ------------------------------------------------------------------------------------------ Gated DeltaNet */
typedef struct {
    RqModel m;
    int lw;
} DnModel;

GWO_API void *gwo_dn_new(int nk, int nv, int dk, int dv, int conv, const float *ssm_conv, const float *ssm_a,
                         const float *ssm_dt, const float *ssm_norm) {
    /* a model holding only the shapes of one linear-attention layer (and optionally its weights:
     * ssm_conv [conv_dim * conv] in the reference's per-channel-group order, ssm_a / ssm_dt [nv], ssm_norm [dv]) */
    DnModel *d = calloc(1, sizeof(DnModel));
    Hybrid *hy = &d->m.hy;
    hy->on = 1; hy->interval = 4; hy->conv = conv; hy->dk = dk; hy->nk = nk; hy->dv = dv; hy->nv = nv;
    hy->conv_dim = 2 * nk * dk + nv * dv;
    hy->vdim = nv * dv;
    hy->n_lin = 1;
    d->m.ssm_layer = ssm_conv_floats(hy) + (size_t)nv * dk * dv;
    d->m.weights.ssm_conv = (float *)ssm_conv;
    d->m.weights.ssm_a = (float *)ssm_a;
    d->m.weights.ssm_dt = (float *)ssm_dt;
    d->m.weights.ssm_norm = (float *)ssm_norm;
    d->lw = lin_width(hy);
    return d;
}

GWO_API void gwo_dn_free(void *p) { free(p); }
GWO_API size_t gwo_dn_state_floats(void *p) { return ((DnModel *)p)->m.ssm_layer; }
GWO_API size_t gwo_dn_conv_floats(void *p) { return ssm_conv_floats(&((DnModel *)p)->m.hy); }
GWO_API int gwo_dn_row_floats(void *p) { return ((DnModel *)p)->lw; }

/* the recurrence over n consecutive rows of one sequence (rows as dn_prep leaves them, stride rs floats), all value
 * heads and column blocks; out [n][nv * dv] (stride os); state: the layer's state (conv part untouched) */
GWO_API void gwo_dn_rec(void *p, float *state, int first, const float *rows, size_t rs, float *out, size_t os, int n) {
    DnModel *d = p;
    const Hybrid *hy = &d->m.hy;
    CkPass ck = { 0 };
    for (int h = 0; h < hy->nv; h++)
        for (int jb = 0; jb < dn_nblk(hy); jb++)
            dn_rec_run(&d->m, h, jb, state, first, rows, rs, out + (size_t)h * hy->dv, os, n, &ck, 0);
}

/* dn_prep_part over n rows in order, all channel groups (rows updated in place), needs the weights */
GWO_API void gwo_dn_prep(void *p, float *state, int first, float *rows, size_t rs, int n) {
    DnModel *d = p;
    const Hybrid *hy = &d->m.hy;
    for (int i = 0; i < dn_prep_items(hy); i++) {
        int h, t;
        dn_prep_item(hy, i, &h, &t);
        for (int r = 0; r < n; r++)
            dn_prep_part(&d->m, 0, h, t, state, first && r == 0, NULL, rows + (size_t)r * rs, NULL);
    }
}

/* dn_out per row and head, in place on out [n][nv * dv]; rows give z */
GWO_API void gwo_dn_out(void *p, const float *rows, size_t rs, float *out, size_t os, int n) {
    DnModel *d = p;
    const Hybrid *hy = &d->m.hy;
    for (int r = 0; r < n; r++)
        for (int h = 0; h < hy->nv; h++)
            dn_out(&d->m, 0, h, rows + (size_t)r * rs, out + (size_t)r * os + (size_t)h * hy->dv);
}

typedef struct {
    DnModel *d;
    int nseq, n;
    float *const *state;
    const float *const *rows;
    float *const *out;
    size_t rs, os;
    atomic_int next;
} DnJob;

static void dn_worker(void *arg, int tid, int nt) {
    (void)tid; (void)nt;
    DnJob *j = arg;
    const Hybrid *hy = &j->d->m.hy;
    int nb = dn_nblk(hy), per = hy->nv * nb;
    CkPass ck = { 0 };
    for (;;) {
        int it = atomic_fetch_add(&j->next, 1);
        if (it >= j->nseq * per) break;
        int s = it / per, h = it % per / nb, jb = it % nb;
        dn_rec_run(&j->d->m, h, jb, j->state[s], 1, j->rows[s], j->rs, j->out[s] + (size_t)h * hy->dv, j->os, j->n, &ck, 0);
    }
}

/* timed recurrence: items (sequence, value head, 32-column block) on the pool (forward.c:3018-3027) */
GWO_API double gwo_bench_dn(void *p, int nseq, float *const *state, const float *const *rows, size_t rs, float *const *out,
                            size_t os, int n, int reps, double *best) {
    gwo_threads_init(0);
    DnJob j = { .d = p, .nseq = nseq, .n = n, .state = state, .rows = rows, .out = out, .rs = rs, .os = os };
    double total = 0, bst = 1e30;
    for (int r = 0; r < reps; r++) {
        atomic_store(&j.next, 0);
        double t0 = now_s();
        rq_parallel(dn_worker, &j);
        double dt = now_s() - t0;
        total += dt;
        bst = dt < bst ? dt : bst;
    }
    if (best) *best = bst;
    return total;
}

/* ------------------------------------------------------------------------------------------ saved sequences */
/* A host sequence of the reference (rq_seq_new, forward.c:148) over a model that holds only the shapes its sequence files
 * depend on, so that the reference's own rq_seq_save / rq_seq_load (seqfile.c) can write and read files next to this
 * repository's writer and reader. */
typedef struct {
    RqModel m;
    RqSeq *s;
} SfSeq;

GWO_API void *gwo_seq_new(int kvt, int n_attn, int n_kv, int hd, int cap, unsigned long long fp, int n_lin, int nk, int nv, int dk,
                          int dv, int conv) {
    SfSeq *q = calloc(1, sizeof(SfSeq));
    int err = 0;
    q->m.config.n_kv_heads = n_kv;
    q->m.config.head_dim = hd;
    q->m.config.seq_len = cap;
    q->m.ctx_max = cap;
    q->m.n_attn = n_attn;
    q->m.kv_dim = n_kv * hd;
    q->m.fp = fp;
    q->m.has_weights = 1;
    if (n_lin > 0) {
        Hybrid *hy = &q->m.hy;
        hy->on = 1; hy->interval = 4; hy->conv = conv; hy->dk = dk; hy->nk = nk; hy->dv = dv; hy->nv = nv;
        hy->conv_dim = 2 * nk * dk + nv * dv;
        hy->vdim = nv * dv;
        hy->n_lin = n_lin;
        q->m.ssm_layer = ssm_conv_floats(hy) + (size_t)nv * dk * dv;
    }
    gwo_threads_init(0);
    q->s = rq_seq_new(&q->m, cap, kvt, &err);
    if (!q->s) {
        free(q);
        return NULL;
    }
    return q;
}
GWO_API void gwo_seq_free(void *p) {
    if (p) rq_seq_free(((SfSeq *)p)->s);
    free(p);
}
/* bytes of all layers of the K (kv 0) / V (kv 1) cache, and floats of the layered DeltaNet state */
GWO_API size_t gwo_seq_cache_bytes(void *p, int kv) { RqSeq *s = ((SfSeq *)p)->s; return seq_kvb(s, s->kv_size, kv); }
GWO_API size_t gwo_seq_state_floats(void *p) { return ((SfSeq *)p)->s->ssm_bytes / sizeof(float); }
/* the sequence's content from the caller's buffers (whole caches, len tokens, the layered state; ck_pos >= 0: a checkpoint
 * at that length with the given state in slot 0) */
GWO_API int gwo_seq_set(void *p, int len, const int *tokens, const void *k, const void *v, const float *ssm, int ck_pos, const float *ck) {
    RqSeq *s = ((SfSeq *)p)->s;
    if (len < 0 || len > s->cap) return -1;
    memcpy(s->key_cache, k, seq_kvb(s, s->kv_size, 0));
    memcpy(s->value_cache, v, seq_kvb(s, s->kv_size, 1));
    memcpy(s->tokens, tokens, (size_t)len * sizeof(int));
    if (s->ssm_bytes && ssm) memcpy(s->ssm, ssm, s->ssm_bytes);
    if (s->ssm_bytes && ck_pos >= 0) {
        if (!s->ck[0].st && !(s->ck[0].st = alloc_big(s->ssm_bytes))) return -2;
        memcpy(s->ck[0].st, ck, s->ssm_bytes);
        s->ck[0].pos = ck_pos;
        s->ck[0].rows = s->ck[0].wr = 0;
    }
    seq_grow(s, len);
    return 0;
}
/* the other way round: returns the length; ck_pos: the length of the checkpoint in slot 0 or -1 */
GWO_API int gwo_seq_get(void *p, int *tokens, void *k, void *v, float *ssm, int *ck_pos, float *ck) {
    RqSeq *s = ((SfSeq *)p)->s;
    memcpy(k, s->key_cache, seq_kvb(s, s->kv_size, 0));
    memcpy(v, s->value_cache, seq_kvb(s, s->kv_size, 1));
    memcpy(tokens, s->tokens, (size_t)s->len * sizeof(int));
    if (s->ssm_bytes && ssm) memcpy(ssm, s->ssm, s->ssm_bytes);
    if (ck_pos) {
        *ck_pos = s->ssm_bytes ? s->ck[0].pos : -1;
        if (*ck_pos >= 0 && ck) memcpy(ck, s->ck[0].st, s->ssm_bytes);
    }
    return s->len;
}
GWO_API unsigned long long gwo_seq_rng(void *p, int set, unsigned long long v) {
    RqSeq *s = ((SfSeq *)p)->s;
    if (set) s->rng = v;
    return s->rng;
}
GWO_API int gwo_seq_save(void *p, const char *path) { return rq_seq_save(((SfSeq *)p)->s, path); }
GWO_API int gwo_seq_load(void *p, const char *path, int n) { return rq_seq_load(((SfSeq *)p)->s, path, n); }
GWO_API long long gwo_seq_save_bytes(void *p) { return rq_seq_save_bytes(((SfSeq *)p)->s); }

/* the activation quantiser (quantize, forward.c:803) on n values in groups of gs */
GWO_API void gwo_quantize(const float *x, int n, int gs, int8_t *q, float *s) {
    QuantizedTensor t = { 0 };
    int keep = GS;
    t.q = q;
    t.s = s;
    GS = gs;
    quantize(&t, (float *)x, n);
    GS = keep;
}
