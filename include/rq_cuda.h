/* rq_cuda.h — C ABI of librq_cuda.so: gwenedeg's attention hot path on an NVIDIA B200 (sm_100a).
 *
 * gwenedeg (a CPU inference engine in C, API prefix rq_) computes attention inside three worker functions of its
 * src/forward.c, per work item, with static functions.  This library replaces exactly those items: the host keeps
 * its forward pass (embedding, matmuls, norms, RoPE, sampling, scheduling) and, once per layer, hands the rows of
 * the pass to the GPU for (1) the K / V cache store, (2) the attention over the cached positions, or (3) the Gated
 * DeltaNet recurrence.  The KV cache and the DeltaNet state live in device memory, in the reference's own tile
 * layout, owned by RqCudaSeq objects that shadow the host's RqSeq.
 *
 * Conventions follow src/runq.h of the reference: every function returns RQ_OK (0) or a negative RQ_ERR_* code,
 * nothing prints or exits, all arguments are checked before any work is started (a refused call leaves caches and
 * state untouched), details of the last error of a context are in rq_cuda_error().  A context is used by one host
 * thread at a time (runq.h:14-17).  Results of a row never depend on the other rows of the pass, on how the pass
 * was chunked, or on the device the sequence lives on (runq.h:22).
 *
 * There is no CPU fallback: without a CUDA device every entry point that needs one fails with RQ_ERR_DEVICE.
 */
#ifndef RQ_CUDA_H
#define RQ_CUDA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* error codes: the values of src/runq.h:35-44, plus one of this library's own */
enum {
    RQ_CUDA_OK = 0,
    RQ_CUDA_ERR_ARG = -1,     /* invalid argument */
    RQ_CUDA_ERR_NOMEM = -2,   /* host or device allocation failed */
    RQ_CUDA_ERR_CONTEXT = -3, /* positions do not fit in the sequence's capacity */
    RQ_CUDA_ERR_STATE = -4,   /* not possible on this object / in this state (e.g. no pass open, device wait expired) */
    RQ_CUDA_ERR_IO = -6,      /* a saved sequence could not be written or read */
    RQ_CUDA_ERR_MISMATCH = -7, /* not a saved sequence of this model shape and KV type (another file, model, layout; corrupt) */
    RQ_CUDA_ERR_DEVICE = -16  /* no usable CUDA device, or a CUDA call failed (text in rq_cuda_error) */
};

/* KV cache element types: the values of RQ_KV_* (src/runq.h:214-215; src/kvtype.h:12-29).  The device holds f16, q8, q4 and
 * q4k4 caches (attention arithmetic in fp32, as the reference's); RQ_CUDA_KV_F32 is listed for the numbering only:
 * rq_cuda_seq_new refuses it with RQ_CUDA_ERR_ARG. */
enum { RQ_CUDA_KV_F32 = 0, RQ_CUDA_KV_F16 = 2, RQ_CUDA_KV_Q8 = 3, RQ_CUDA_KV_Q4 = 8, RQ_CUDA_KV_Q4K4 = 9 };

typedef struct RqCuda RqCuda;       /* a compute context on one device: stream, scratch, the open pass (RqCtx, forward.c:32) */
typedef struct RqCudaSeq RqCudaSeq; /* a sequence's device-resident KV cache and DeltaNet state (RqSeq, internal.h:353) */

/* Shapes of the model's attention path (Config / Hybrid of src/internal.h:75-104, the derived values of
 * forward_model_init, forward.c:129).  kv_head0 / kv_heads_local select the contiguous group of KV heads this
 * device holds (0 / n_kv_heads: all of them); q and out rows then carry only that group's query heads. */
typedef struct {
    int n_attn;         /* attention layers = layers of the KV cache (RqModel.n_attn) */
    int n_heads;        /* query heads */
    int n_kv_heads;     /* KV heads; n_heads % n_kv_heads == 0 */
    int head_dim;       /* 64, 128 or 256 */
    int gated;          /* Qwen3.5 gated attention: query rows are [q | gate] per head (qh = 2 head_dim, forward.c:134) */
    int n_lin;          /* Gated DeltaNet layers (Hybrid.n_lin), 0 for Qwen3 */
    int dn_nk, dn_nv;   /* DeltaNet key heads / value heads (nv % nk == 0) */
    int dn_dk, dn_dv;   /* DeltaNet key / value head dims (128) */
    int dn_conv;        /* causal conv taps (4) */
    int kv_head0;       /* first KV head held by this context's sequences */
    int kv_heads_local; /* KV heads held (0: all) */
} RqCudaModel;

/* One segment of a pass: n consecutive rows of one sequence at positions pos0 .. pos0 + n - 1 (RqSegment,
 * runq.h:364-374; pos0 is the sequence's length in the reference, passed explicitly here because the host owns it).
 * Row r of the segment attends positions 0 .. pos0 + r. */
typedef struct {
    RqCudaSeq *seq;
    int pos0;
    int n;
} RqCudaSegment;

/* ---- context (rq_ctx_new / rq_ctx_free / rq_ctx_error, runq.h:317-335) ------------------------------------ */
/* max_rows: the most rows (and segments) a pass may hold, 1 .. 16384 (the reference's RQ_BATCH_MAX is 512) */
int rq_cuda_init(int device, const RqCudaModel *model, int max_rows, RqCuda **ctx);
void rq_cuda_free(RqCuda *ctx);
const char *rq_cuda_error(const RqCuda *ctx);
int rq_cuda_device_count(void);
/* 1 when the library was built with the kernels' index checks compiled in (make debug: librq_cuda_debug.so; a work item
 * that does not fit its row or cache sets the status word instead of touching memory), 0 for the release build */
int rq_cuda_debug_build(void);
/* block until everything this context launched is complete; reports a device-side wait that expired as RQ_CUDA_ERR_STATE */
int rq_cuda_sync(RqCuda *ctx);
/* Sizes the context's scratch ahead of time, so that no pass up to the given size allocates or synchronises on its first
 * use (the reference's scratch is sized for max_ctx when the context is made and grown on demand, ctx_check_seq
 * forward.c:628-634; this is the same with the demand stated up front): passes of at most `rows` rows attending at most
 * `positions_total` cached positions in all, no row beyond `max_ctx` positions.  Not inside an open pass. */
int rq_cuda_reserve(RqCuda *ctx, int rows, long long positions_total, int max_ctx);
/* Error-path self test (no counterpart in the reference; the reference checks everything before it starts work,
 * forward.c:3773-3801, and has no device to wait for): launches one small kernel that waits, with a limit of `limit_us`
 * microseconds, on a barrier nothing completes.  The kernel gives up by itself, records code 99 in the context's status
 * word and returns; the next rq_cuda_sync then reports RQ_CUDA_ERR_STATE exactly as it would after an expired wait inside
 * an attention kernel, and the context stays usable. */
int rq_cuda_selftest_wait_expiry(RqCuda *ctx, unsigned int limit_us);
/* Head-sharded contexts on several GPUs of one node (kv_head0 / kv_heads_local: each rank holds a group of KV heads of every
 * sequence; the reference's workers share one address space, forward.c:2691-2715: this is what replaces it across GPUs): the
 * gather of the output rows is fused into the merge kernel.  Every rank exports a row buffer (rq_cuda_peer_export: 64 bytes of
 * cudaIpcMemHandle_t out, for passes of at most `rows` rows), the host exchanges the handles by whatever means it has, and every
 * rank imports all of them in rank order (rq_cuda_peer_import: `handles` = world x 64 bytes; its own entry is ignored).
 * rq_cuda_attn_decode_gather_dev is then rq_cuda_attn_decode_dev whose merge kernel stores this rank's heads of every row straight
 * into every rank's buffer over NVLink (plain peer stores, no library collective), followed by a one-warp kernel that
 * tells every rank "my part of this step is in place" and waits for theirs with a limit of two seconds (a rank that never arrives
 * ends the wait with RQ_CUDA_ERR_STATE at the next rq_cuda_sync; the context stays usable).  *out_full: this rank's buffer of the
 * step, device memory [rows][n_heads][head_dim] with all heads, valid until the call after next; all ranks must make the same
 * sequence of calls.  rq_cuda_selftest_peer_wait runs the wait of a two-rank exchange whose other rank never arrives, with a
 * limit of `limit_us` microseconds, on one GPU (code 97 in the status word). */
int rq_cuda_peer_export(RqCuda *ctx, int rows, void *handle64);
int rq_cuda_peer_import(RqCuda *ctx, int rank, int world, const void *handles);
int rq_cuda_attn_decode_gather_dev(RqCuda *ctx, int layer, const float *q_dev, float **out_full);
int rq_cuda_selftest_peer_wait(RqCuda *ctx, unsigned int limit_us);
/* The quantised copy of the attention's outputs that the reference makes right before the `wo` matmul (quantize,
 * forward.c:803, at :2716-2719 / :3616), fused into the merge kernels: with xq_dev / xs_dev set, every attention call of the
 * context (decode and prefill) also writes int8 levels xq [rows][heads_local * head_dim] and one fp32 scale per `gs`
 * values xs [rows][heads_local * head_dim / gs] (gs = the model's activation group size GS: 32, 64, 128 or 256, dividing
 * head_dim), the reference's operations in its order (scale = max|x| (1 / 127), level = trunc(x (127 / max|x|) + copysign(
 * 0.49999997, .))): the bits quantize() gives on the same fp32 rows.  Both NULL: off.  Device pointers the host owns, sized
 * for the largest pass. */
int rq_cuda_set_wo_quant(RqCuda *ctx, int gs, signed char *xq_dev, float *xs_dev);
/* Which kernels attend over quantised caches at head_dim 128 (prompt passes: 128 and 256).  0 (the default): tensor cores within the reference's acceptance
 * bar (2e-3 absolute / 1e-3 relative), not bit for bit:
 *  - rq_cuda_attn_decode over q8 / q4 / q4k4 caches: the cached levels go into tcgen05.mma (kind::i8) with exact int32
 *    accumulation: int8 levels as they are, 4-bit levels n as the int8 values 16 (n - 8) (one shift / mask / xor per word on their way
 *    to the operand's place); the query and the softmax weights are 16-bit fixed point split into two int8 planes, the bf16
 *    scales are applied in fp32 (~1e-4 relative to the reference's fp32 arithmetic);
 *  - rq_cuda_attn_prefill over q8 / q4 / q4k4 caches, segment by segment: for a segment of 16 rows or more (a prompt chunk) the
 *    layer's tiles are expanded once per call to f16 (the reference's dequantised values, block_f32 of forward.c:1770-1804, rounded once)
 *    and the f16 tensor-core kernel runs over them with rotated query rows (~3e-4 relative); the shorter segments of the same
 *    pass (decode rows that ride along) take the decode kernels above.
 * Non-zero: the CUDA-core kernels that follow attention_part_q (forward.c:1770-1804) operation for operation and give the
 * reference's bits (decode at 0.55-0.75 of the speed, prompt passes row by row).  f16 caches, other head dims and
 * rq_cuda_attn_decode_noalloc always take the bit-exact kernels.  Either way a row's result is independent of the other
 * rows of the pass. */
int rq_cuda_set_exact(RqCuda *ctx, int exact);
/* Prompt passes on the tensor-core prefill kernels cut each tile's keys into splits of equal length, one CTA each, and merge the
 * splits' partial results (the reference splits lone long rows per 256-position block, prefill_plan forward.c:3273-3311; here the cut
 * serves to fill the SMs).  By default the length is chosen per pass (by scheduling the items of each candidate length onto the
 * device's SMs); a non-zero `positions` (a multiple of 128, at least 1024) fixes it, for tests and measurements.  Results are inside
 * the kernel's tolerance for every length, not identical across lengths (the merge order changes). */
int rq_cuda_set_prefill_split(RqCuda *ctx, int positions);
/* run this context's work on a caller-owned stream (a cudaStream_t; NULL: back to the context's own, a non-blocking stream:
 * it is not ordered with the legacy default stream, whose handle is NULL as well).  The attention and DeltaNet kernels are
 * launched with programmatic stream serialization: each waits for the kernel before it in the stream before it touches
 * global memory, so ordinary stream order is all a caller needs. */
int rq_cuda_set_stream(RqCuda *ctx, void *cuda_stream);

/* ---- sequences (rq_seq_new :148, rq_seq_free :192, rq_seq_truncate :409, rq_seq_copy :553 of forward.c) ---- */
/* capacity positions (rounded up to whole 256-position blocks inside), cache type kv_type; DeltaNet state zeroed */
int rq_cuda_seq_new(RqCuda *ctx, int capacity, int kv_type, RqCudaSeq **seq);
void rq_cuda_seq_free(RqCudaSeq *seq);
int rq_cuda_seq_len(const RqCudaSeq *seq);      /* positions stored so far (passes grow it, as seq_grow does) */
int rq_cuda_seq_capacity(const RqCudaSeq *seq);
int rq_cuda_seq_truncate(RqCudaSeq *seq, int n); /* keep the first n positions (attention layers only, as the reference) */
/* the first n positions of src (same context, type and capacity class) into dst; the DeltaNet state is copied
 * when n == rq_cuda_seq_len(src) */
int rq_cuda_seq_copy(RqCudaSeq *dst, const RqCudaSeq *src, int n);
/* bytes of one layer's K (is_v 0) or V (is_v 1) cache; raw transfer of one layer in the reference's byte layout
 * (blocks of 256 positions x KV heads x 16-position tiles; forward.c:1894, kernels_avx512.h:1090-1107), the format
 * of the reference's saved sequences (seqfile.c) */
size_t rq_cuda_seq_layer_bytes(const RqCudaSeq *seq, int is_v);
int rq_cuda_seq_read_kv(RqCudaSeq *seq, int layer, int is_v, void *host, size_t bytes);
int rq_cuda_seq_write_kv(RqCudaSeq *seq, int layer, int is_v, const void *host, size_t bytes, int new_len);
/* DeltaNet state of one linear layer (floats: conv inputs, then S per value head in [dv/32][dk][32] blocks;
 * forward.c:125, :2090) */
size_t rq_cuda_seq_state_floats(const RqCudaSeq *seq);
int rq_cuda_seq_read_state(RqCudaSeq *seq, int lin_layer, float *host);
int rq_cuda_seq_write_state(RqCudaSeq *seq, int lin_layer, const float *host);
/* DeltaNet state checkpoints (rq_seq_set_checkpoints / rq_seq_checkpoint_at / _rows / _drop, runq.h:239-265; RqSeq.ck and
 * CkPass, internal.h:347-351, :383).  The recurrent state cannot be rewound, so a sequence keeps copies of it at chosen
 * lengths in `n` slots (0 .. 32; each the whole layered state, in device memory).  Which lengths to keep is the host's
 * policy, as in the reference; the device side takes the copies while a pass runs (rq_cuda_pass_checkpoint below) and
 * goes back to one:
 *   _checkpoint_pos   the length whose state slot `slot` holds, -1 when it is empty
 *   _restore          state <- slot, length <- that length (rq_seq_truncate onto a checkpoint); later checkpoints are dropped
 *   _checkpoint_drop  forget the slot's content
 *   _read / _write_checkpoint   one linear layer of a slot from / to host memory (saved sequences); write sets the slot's length
 * rq_cuda_seq_truncate drops the checkpoints past the new length; rq_cuda_seq_copy to a length below the source's takes the
 * state from the source's checkpoint at that length. */
int rq_cuda_seq_set_checkpoints(RqCudaSeq *seq, int n);
int rq_cuda_seq_checkpoint_pos(const RqCudaSeq *seq, int slot);
int rq_cuda_seq_restore(RqCudaSeq *seq, int slot);
int rq_cuda_seq_checkpoint_drop(RqCudaSeq *seq, int slot);
int rq_cuda_seq_read_checkpoint(RqCudaSeq *seq, int slot, int lin_layer, float *host);
int rq_cuda_seq_write_checkpoint(RqCudaSeq *seq, int slot, int lin_layer, const float *host, int pos);
/* Saved sequences in the reference's file format (rq_seq_save / rq_seq_load / rq_seq_save_bytes, runq.h:283-314; header and
 * section layout seqfile.c:10-41): the header page, the tokens, per attention layer the first ceil(len / 256) K blocks then V
 * blocks exactly as cached, then the DeltaNet state and the checkpoints held, ascending.  Files written here load into the
 * reference's host sequences and files it wrote load here.  tokens: the host's token ids of positions 0 .. len - 1 (the
 * host owns them; they are stored and hashed with the header); model_fp: the model's fingerprint (RqModel.fp), checked on
 * load; rng: the sequence's sampling state, stored and returned.  rq_cuda_seq_load keeps the first n positions (n <= the
 * saved length and the capacity; with DeltaNet layers: the saved length, else the longest saved checkpoint at or below n,
 * rq_seq_file_keep) and tells the kept length through rq_cuda_seq_len; tokens (room for n ints) and rng may be NULL.
 * RQ_CUDA_ERR_IO / RQ_CUDA_ERR_MISMATCH as the reference (after an I/O error the sequence is empty).  Contexts that hold
 * only a group of the KV heads cannot save or load (RQ_CUDA_ERR_STATE). */
long long rq_cuda_seq_save_bytes(const RqCudaSeq *seq);
int rq_cuda_seq_save(RqCudaSeq *seq, const char *path, const int *tokens, unsigned long long model_fp, unsigned long long rng);
int rq_cuda_seq_load(RqCudaSeq *seq, const char *path, unsigned long long model_fp, int n, int *tokens, unsigned long long *rng);
/* test / benchmark hook (rq_seq_fill_synthetic, forward.c:2418): n positions of seeded pseudo-random K / V written by
 * a device kernel — f32 / f16: ~N(0,1) values; q8 / q4: uniform levels and bf16 scales ~|N(0, 0.02)| in the tile
 * format — and the length set to n */
int rq_cuda_seq_fill_synthetic(RqCudaSeq *seq, int n, unsigned long long seed);

/* ---- a pass (rq_forward_batch, forward.c:3762; rq_decode :2815 is a pass of one row) ---------------------- */
/* Opens a pass over the rows of nseg segments (a sequence at most once; 1 <= total rows <= max_rows; every row
 * inside its sequence's capacity).  Row order = segment order, rows of a segment in position order.  Uploads the
 * row table once; the per-layer calls below refer to "the rows of the pass". */
int rq_cuda_pass_begin(RqCuda *ctx, const RqCudaSegment *seg, int nseg);
/* A checkpoint the open pass takes (ck_plan / CkPass; dn_rec_run forward.c:2267-2270): after row `row` (0-based in the
 * segment) of segment `seg`, the state of every DeltaNet layer of that segment's sequence goes to its slot `slot`, by the
 * kernels themselves (rq_cuda_dn_prep_dev: the conv inputs; rq_cuda_dn_rec / _dn_chunk: S; the chunked form cuts its
 * 64-token chunks at the checkpoint rows, so a pass is never split for them).  Call after rq_cuda_pass_begin and before
 * the pass's first DeltaNet call; at most 1024 per pass.  The slot holds length pos0 + row + 1 once the pass is committed. */
int rq_cuda_pass_checkpoint(RqCuda *ctx, int seg, int row, int slot);
/* closes the pass; commit != 0 grows each sequence's length to pos0 + n (seq_grow) */
int rq_cuda_pass_end(RqCuda *ctx, int commit);

/* What the reference's server feeds its pass-cost model with (RqPassCost, runq.h:660-685: a pass of R rows takes
 * t_w f(R) + att S1 + att_x S2 seconds; cost_learn engine.c:2641 corrects the calibrated model by the measured time of each
 * pass; seg_cost :2631 forms S1 and S2).  Host wall time says nothing about work that runs asynchronously on a device, so the
 * library measures: with rq_cuda_pass_timing on, every pass is bracketed by CUDA events on the context's stream, and
 * rq_cuda_pass_time returns, for the last closed pass, the device seconds between rq_cuda_pass_begin and rq_cuda_pass_end
 * (it waits for that pass to finish) with the pass's rows, S1 = the sum of the segments' first positions and S2 = the sum of
 * the positions of every further row: `took` and the arguments of rq_pass_cost for cost_learn.
 * rq_cuda_pass_cost_measure is rq_pass_cost_measure (runq.h:678) for the attention path on the device: on a sequence of this
 * context filled with synthetic values it times (fastest of `reps`) one row at L / 2, one row at L and a segment of 16 rows at
 * L over all attention layers and solves for t_w (the part of a pass that does not depend on the context: launches), att
 * (seconds per position of context for a segment's first row) and att_x (for each further row).  The sequence is left empty. */
typedef struct {
    double seconds;    /* device time of the pass */
    int rows;          /* its rows */
    double pos_first;  /* S1 */
    double pos_more;   /* S2 */
} RqCudaPassTime;
int rq_cuda_pass_timing(RqCuda *ctx, int on);
int rq_cuda_pass_time(RqCuda *ctx, RqCudaPassTime *out);
int rq_cuda_pass_cost_measure(RqCuda *ctx, RqCudaSeq *seq, int L, int reps, double *t_w, double *att, double *att_x);

/* K and V rows of the pass into the caches of attention layer `layer`, replacing kv_store (forward.c:1901; call
 * sites :2682/:2686, :3067-3085, :3568-3578).  k, v: host fp32 [rows][kv_heads_local][head_dim], after QK-norm and
 * RoPE; either may be NULL.  f16: round to nearest even, saturating (f32_f16 :1325); q8 / q4: rotate + quantise
 * (kvq_store :1710). */
int rq_cuda_kv_store(RqCuda *ctx, int layer, const float *k, const float *v);
int rq_cuda_kv_store_dev(RqCuda *ctx, int layer, const float *k_dev, const float *v_dev);

/* The step right before the path, fused on the device (device pointers): per row of the pass, QK-norm (RMSNorm per head)
 * and NeoX-style RoPE of q and k for the row's position, then K and V into the cache tiles, replacing qk_norm_rope
 * (forward.c:1266), rope_row (:1248) and kv_store at the call sites :2679-2687, :3059-3085, :3568-3578.
 * q: [rows][heads_local][qh] raw projections, normed + rotated in place (a gate half is left untouched);
 * k, v: [rows][kv_heads_local][head_dim] raw projections; q_norm_w, k_norm_w: [head_dim] weights of the layer;
 * rope_dim: rotated dims per head (head_dim for Qwen3, 64 for Qwen3.5); rope_theta: the RoPE base (1e6).
 * The reference builds this step with -Ofast: results agree to rounding (~1e-6 relative), not bit for bit. */
int rq_cuda_qk_norm_rope_store_dev(RqCuda *ctx, int layer, float *q_dev, const float *k_dev, const float *v_dev,
                                   const float *q_norm_w_dev, const float *k_norm_w_dev, int rope_dim, float rope_theta);

/* Attention of every row of the pass over its sequence's cache of layer `layer`: split-K flash-decode over the
 * reference's fixed 256-position blocks with the partial results merged in block order, replacing the attention
 * items of decode_worker (forward.c:2691-2715) and batch_decode_worker (:3582-3616): attention_part :1806 +
 * att_combine :1405, with att_q_rot :1662 before and att_o_unrot :1672 / attn_gate :2291 after.
 * q: host fp32 [rows][heads_local][qh] (qh = head_dim, or 2 head_dim when gated), out: host fp32
 * [rows][heads_local][head_dim].  Softmax scale 1/sqrt(head_dim).  The call returns when `out` is complete.  If `out`
 * is page-locked memory the GPU can address (rq_cuda_malloc_host, cudaMallocHost, cudaHostRegister) the last kernel
 * stores into it directly; ordinary memory takes a staged copy.  The same holds for rq_cuda_attn_prefill. */
int rq_cuda_attn_decode(RqCuda *ctx, int layer, const float *q, float *out);
int rq_cuda_attn_decode_dev(RqCuda *ctx, int layer, const float *q_dev, float *out_dev);

/* (No counterpart in the reference.)  rq_cuda_attn_decode_dev for hosts that must not allocate: a server that
 * budgeted all device memory at start-up, or code running where cudaMalloc is not allowed or would stall the device.
 * The per-block partial results go to a fixed 32 MiB array inside the library (held by every GPU that loads it)
 * instead of the context's growable scratch; the call performs no cudaMalloc / cudaFree and calls no allocating
 * routine.  q_dev and out_dev are the caller's device buffers, as for rq_cuda_attn_decode_dev, and the results are
 * the same bits.  A pass whose (256-position blocks of all rows) x heads x (head_dim + 16) x 4 bytes exceed
 * rq_cuda_attn_decode_noalloc_max_bytes() is refused with RQ_CUDA_ERR_ARG and a message.  The first call on a device
 * looks up the array's device address: make that first call before any stream capture.  All calls share the one
 * array and it keeps the last call's contents: calls that overlap on the GPU (two streams, two contexts, two host
 * threads on one device) race; nothing in it needs to start at zero. */
int rq_cuda_attn_decode_noalloc(RqCuda *ctx, int layer, const float *q_dev, float *out_dev);
size_t rq_cuda_attn_decode_noalloc_max_bytes(void);

/* The same attention for passes with many rows per sequence (prompt chunks), replacing prefill_worker's items
 * (forward.c:3096-3146, attention_kv :1871): tensor-core tiles over the cached prefix plus the chunk's own rows,
 * causal per row.  Same arguments and layouts as rq_cuda_attn_decode. */
int rq_cuda_attn_prefill(RqCuda *ctx, int layer, const float *q, float *out);
int rq_cuda_attn_prefill_dev(RqCuda *ctx, int layer, const float *q_dev, float *out_dev);

/* Gated DeltaNet recurrence of linear layer `lin_layer` over the rows of the pass, replacing dn_rec_run
 * (forward.c:2224; call sites :2640-2650, :3018-3027).  rows: fp32 [rows][lw], lw = 2 nk dk + 2 nv dv + 2 nv, laid
 * out [q | k | v | z | exp(g) | beta] as dn_prep_part (:2104) leaves them; out: fp32 [rows][nv dv], the raw S^T q.
 * A segment starting at position 0 clears its state first.  The state is advanced in place. */
int rq_cuda_dn_rec(RqCuda *ctx, int lin_layer, const float *rows, float *out);
int rq_cuda_dn_rec_dev(RqCuda *ctx, int lin_layer, const float *rows_dev, float *out_dev);

/* The same recurrence for passes with many rows per sequence (prompt chunks: the dn_rec_run items of prefill_worker,
 * forward.c:3018-3027), re-associated per chunk of 64 tokens (WY / UT form) so that the work runs as dense products on
 * the tensor cores.  Same arguments, layouts and state as rq_cuda_dn_rec; operands are rounded to f16 (fp32
 * accumulation and state), so results agree with the token recurrence to ~5e-4 relative instead of bit for bit.
 * dk = dv = 128 only (RQ_CUDA_ERR_ARG otherwise). */
int rq_cuda_dn_chunk(RqCuda *ctx, int lin_layer, const float *rows, float *out);
int rq_cuda_dn_chunk_dev(RqCuda *ctx, int lin_layer, const float *rows_dev, float *out_dev);

/* The steps around the recurrence, on the device (dk = dv = 128): the layer's weights once (host pointers: conv taps in the
 * reference's per-channel-group order [conv][channels of the group] at conv * first_channel, conv * (2 nk dk + nv dv) floats;
 * ssm_a = -exp(A_log) [nv]; the dt bias [nv]; the gated RMSNorm weight [dv]; src/internal.h:166-169), then per pass
 * rq_cuda_dn_prep_dev (dn_prep_part, forward.c:2104: causal conv + SiLU, L2 norm of q / k, exp(g) and beta; raw projection
 * rows -> recurrence inputs, in place; the conv part of the state is advanced) and rq_cuda_dn_out_dev (dn_out :2280: gated
 * RMSNorm x SiLU(z), in place on the recurrence's outputs).  Same operations in the same order as the reference, except
 * the two libm calls of the gate (expf, log1pf), which agree to the last bits only. */
int rq_cuda_dn_set_weights(RqCuda *ctx, int lin_layer, const float *conv, const float *ssm_a, const float *ssm_dt, const float *ssm_norm);
int rq_cuda_dn_prep_dev(RqCuda *ctx, int lin_layer, float *rows_dev);
int rq_cuda_dn_out_dev(RqCuda *ctx, int lin_layer, const float *rows_dev, float *out_dev);

/* ---- device memory and timing helpers for hosts without a CUDA runtime of their own (ctypes, cgo, JNI) ---- */
int rq_cuda_malloc(RqCuda *ctx, size_t bytes, void **dev);
int rq_cuda_mfree(RqCuda *ctx, void *dev);
int rq_cuda_malloc_host(RqCuda *ctx, size_t bytes, void **host); /* pinned */
int rq_cuda_mfree_host(RqCuda *ctx, void *host);
int rq_cuda_memcpy_h2d(RqCuda *ctx, void *dev, const void *host, size_t bytes); /* async on the context's stream */
int rq_cuda_memcpy_d2h(RqCuda *ctx, void *host, const void *dev, size_t bytes); /* async on the context's stream */
int rq_cuda_mem_info(RqCuda *ctx, size_t *free_bytes, size_t *total_bytes);
/* CUDA events on the context's stream: start, then stop returns the milliseconds between them (stop synchronises) */
int rq_cuda_timer_start(RqCuda *ctx);
int rq_cuda_timer_stop(RqCuda *ctx, float *ms);
/* kernels launched by this context since it was created */
unsigned long long rq_cuda_launch_count(const RqCuda *ctx);
/* per-launch device time of the attention's dominant kernel (the per-block partial kernel): between _begin and _end
 * every launch is bracketed by CUDA events on the context's stream (no synchronisation is added); _end waits for the
 * stream and returns the summed milliseconds and the number of launches timed (at most max_launches) */
int rq_cuda_profile_begin(RqCuda *ctx, int max_launches);
int rq_cuda_profile_end(RqCuda *ctx, float *total_ms, int *launches);

#ifdef __cplusplus
}
#endif
#endif /* RQ_CUDA_H */
