/* A miniature of gwenedeg's C host around the attention path, in plain C99, linked against librq_cuda.so.
 *
 * It drives the library the way the integration notes describe for the reference's workers (rq_forward_batch,
 * src/forward.c:3762; decode_worker :2691-2715; batch_decode_worker :3582-3616): a context next to rq_ctx_new, one
 * device sequence per host sequence, per pass rq_cuda_pass_begin -> per layer rq_cuda_kv_store + rq_cuda_attn_decode
 * (or rq_cuda_attn_prefill for prompt chunks) -> rq_cuda_pass_end, with page-locked q / out row buffers.
 *
 *   host_pass <out-file>     prompt passes of up to 64 rows for three sequences, then one batched decode step, then the
 *                            same decode rows one sequence at a time; writes the inputs and results to <out-file> for
 *                            the Python test to check against the CPU checker.
 * Exit code: 0 ok, 3 no usable CUDA device (rq_cuda_init returned RQ_CUDA_ERR_DEVICE), 1 any other failure.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "rq_cuda.h"

enum { N_LAYERS = 2, N_HEADS = 8, N_KV = 2, HD = 128, NSEQ = 3, CHUNK = 64 };
static const int CTX[NSEQ] = {300, 17, 1025};

/* xorshift64* -> roughly normal values (sum of four uniforms), the same on every machine */
static unsigned long long rng_state = 0x9E3779B97F4A7C15ull;
static float rnd(void) {
    float s = 0.0f;
    for (int i = 0; i < 4; i++) {
        rng_state ^= rng_state >> 12;
        rng_state ^= rng_state << 25;
        rng_state ^= rng_state >> 27;
        s += (float)((rng_state * 0x2545F4914F6CDD1Dull) >> 40) * (1.0f / 16777216.0f);
    }
    return (s - 2.0f) * 1.7320508f;
}

static int check(RqCuda *cu, int rc, const char *what) {
    if (rc != RQ_CUDA_OK) fprintf(stderr, "%s failed: %d (%s)\n", what, rc, rq_cuda_error(cu));
    return rc;
}
#define TRY(call)                                  \
    do {                                           \
        if (check(cu, (call), #call)) goto fail;   \
    } while (0)

int main(int argc, char **argv) {
    RqCudaModel shape;
    RqCuda *cu = NULL;
    RqCudaSeq *seq[NSEQ] = {NULL, NULL, NULL};
    float *k_rows[NSEQ] = {NULL, NULL, NULL}, *v_rows[NSEQ] = {NULL, NULL, NULL};
    float *q_b = NULL, *xb_b = NULL, *alone = NULL, *pre_q = NULL, *pre_out = NULL;
    FILE *f = NULL;
    int rc, status = 1;

    memset(&shape, 0, sizeof shape);
    shape.n_attn = N_LAYERS;
    shape.n_heads = N_HEADS;
    shape.n_kv_heads = N_KV;
    shape.head_dim = HD;
    rc = rq_cuda_init(0, &shape, CHUNK, &cu);
    if (rc == RQ_CUDA_ERR_DEVICE) {
        printf("no usable CUDA device: rq_cuda_init returned RQ_CUDA_ERR_DEVICE (there is no CPU fallback)\n");
        return 3;
    }
    if (rc != RQ_CUDA_OK) {
        fprintf(stderr, "rq_cuda_init: %d\n", rc);
        return 1;
    }
    if (argc < 2) {
        fprintf(stderr, "usage: host_pass <out-file>\n");
        goto fail;
    }
    /* the host's q and output row buffers, page-locked so that the last kernel stores into them directly */
    TRY(rq_cuda_malloc_host(cu, sizeof(float) * CHUNK * N_HEADS * HD, (void **)&q_b));
    TRY(rq_cuda_malloc_host(cu, sizeof(float) * CHUNK * N_HEADS * HD, (void **)&xb_b));
    alone = (float *)malloc(sizeof(float) * NSEQ * N_HEADS * HD);
    pre_q = (float *)malloc(sizeof(float) * CHUNK * N_HEADS * HD);
    pre_out = (float *)malloc(sizeof(float) * CHUNK * N_HEADS * HD);
    if (!alone || !pre_q || !pre_out) goto fail;
    TRY(rq_cuda_reserve(cu, CHUNK, 4096, 2048));

    /* ---- prompt passes: every sequence's K / V rows (the same rows for both layers), CHUNK rows at a time; the last
     * chunk of sequence 0 also runs the prefill attention of layer 1 over the rows just stored */
    for (int s = 0; s < NSEQ; s++) {
        const size_t nf = (size_t)CTX[s] * N_KV * HD;
        TRY(rq_cuda_seq_new(cu, CTX[s], RQ_CUDA_KV_F16, &seq[s]));
        k_rows[s] = (float *)malloc(sizeof(float) * nf);
        v_rows[s] = (float *)malloc(sizeof(float) * nf);
        if (!k_rows[s] || !v_rows[s]) goto fail;
        for (size_t i = 0; i < nf; i++) k_rows[s][i] = rnd(), v_rows[s][i] = rnd();
        for (int pos = 0; pos < CTX[s]; pos += CHUNK) {
            const int n = CTX[s] - pos < CHUNK ? CTX[s] - pos : CHUNK;
            RqCudaSegment sg;
            sg.seq = seq[s];
            sg.pos0 = rq_cuda_seq_len(seq[s]); /* the host's seq->len */
            sg.n = n;
            if (sg.pos0 != pos) goto fail;
            TRY(rq_cuda_pass_begin(cu, &sg, 1));
            for (int al = 0; al < N_LAYERS; al++)
                TRY(rq_cuda_kv_store(cu, al, k_rows[s] + (size_t)pos * N_KV * HD, v_rows[s] + (size_t)pos * N_KV * HD));
            if (s == 0 && pos + n == CTX[s]) {
                for (int i = 0; i < n * N_HEADS * HD; i++) pre_q[i] = q_b[i] = rnd();
                TRY(rq_cuda_attn_prefill(cu, 1, q_b, xb_b));
                memcpy(pre_out, xb_b, sizeof(float) * n * N_HEADS * HD);
            }
            TRY(rq_cuda_pass_end(cu, 1)); /* where seq_grow() runs in the reference */
        }
        if (rq_cuda_seq_len(seq[s]) != CTX[s]) goto fail;
    }

    /* ---- one batched decode step over the three sequences (each row attends its whole context), layer 1 */
    {
        RqCudaSegment cs[NSEQ];
        for (int s = 0; s < NSEQ; s++) {
            cs[s].seq = seq[s];
            cs[s].pos0 = CTX[s] - 1; /* re-attend the last stored position: nothing is stored in this pass */
            cs[s].n = 1;
        }
        for (int i = 0; i < NSEQ * N_HEADS * HD; i++) q_b[i] = rnd();
        TRY(rq_cuda_pass_begin(cu, cs, NSEQ));
        TRY(rq_cuda_attn_decode(cu, 1, q_b, xb_b));
        TRY(rq_cuda_pass_end(cu, 0));
        /* ---- the same rows, one sequence per pass: a row's result must not depend on the batch (runq.h:22) */
        for (int s = 0; s < NSEQ; s++) {
            TRY(rq_cuda_pass_begin(cu, &cs[s], 1));
            TRY(rq_cuda_attn_decode(cu, 1, q_b + (size_t)s * N_HEADS * HD, alone + (size_t)s * N_HEADS * HD));
            TRY(rq_cuda_pass_end(cu, 0));
        }
        if (memcmp(alone, xb_b, sizeof(float) * NSEQ * N_HEADS * HD) != 0) {
            fprintf(stderr, "a decode row alone differs from the same row in the batch\n");
            goto fail;
        }
    }

    /* ---- everything the checker needs: K / V rows per sequence, the decode q and out rows, the prefill q and out rows */
    f = fopen(argv[1], "wb");
    if (!f) goto fail;
    {
        const int hdr[8] = {N_LAYERS, N_HEADS, N_KV, HD, NSEQ, CTX[0], CTX[1], CTX[2]};
        const int npre = CTX[0] % CHUNK ? CTX[0] % CHUNK : CHUNK;
        fwrite(hdr, sizeof hdr, 1, f);
        fwrite(&npre, sizeof npre, 1, f);
        for (int s = 0; s < NSEQ; s++) {
            fwrite(k_rows[s], sizeof(float), (size_t)CTX[s] * N_KV * HD, f);
            fwrite(v_rows[s], sizeof(float), (size_t)CTX[s] * N_KV * HD, f);
        }
        fwrite(q_b, sizeof(float), NSEQ * N_HEADS * HD, f);
        fwrite(xb_b, sizeof(float), NSEQ * N_HEADS * HD, f);
        fwrite(pre_q, sizeof(float), (size_t)npre * N_HEADS * HD, f);
        fwrite(pre_out, sizeof(float), (size_t)npre * N_HEADS * HD, f);
    }
    if (fclose(f) != 0) goto fail;
    printf("ok: %llu kernels launched\n", rq_cuda_launch_count(cu));
    status = 0;
fail:
    for (int s = 0; s < NSEQ; s++) {
        rq_cuda_seq_free(seq[s]);
        free(k_rows[s]);
        free(v_rows[s]);
    }
    free(alone);
    free(pre_q);
    free(pre_out);
    if (q_b) rq_cuda_mfree_host(cu, q_b);
    if (xb_b) rq_cuda_mfree_host(cu, xb_b);
    rq_cuda_free(cu);
    return status;
}
