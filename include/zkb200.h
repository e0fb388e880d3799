/* zkb200 — C ABI of the B200 prover backend for zk_ml_prover's sumcheck hot path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns an int32
 * status: 0 = ok, nonzero = one of the ZKB_E_* codes below (message via zkb_last_error).
 * The reference's GPU seam turns a failed command buffer into a panic
 * (rust/zk_ml_prover/src/gpu/metal_device.rs:36-45); a Rust shim over this ABI does the
 * same with a nonzero status.  There is no CPU fallback: without a CUDA device every call
 * that needs one fails with ZKB_E_CUDA.
 *
 * Field elements are canonical u32 in [0, 2^31-1).  Extension-field (M31^4) elements are four
 * u32 in the reference's EFElement order [re(c0), im(c0), re(c1), im(c1)]
 * (rust/zk_ml_prover/src/proving/sumcheck.rs:67-96).
 *
 * Pointer arguments named `*_dev` are device pointers of the context's GPU; everything else
 * is host memory owned by the caller.  A context owns one CUDA stream; calls on one context
 * are ordered, different contexts may be used concurrently from different threads (the
 * reference calls its GPU kernels from rayon workers, gpu/metal_kernels.rs:22-44).
 */
#ifndef ZKB200_H
#define ZKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct zkb_ctx zkb_ctx;
typedef struct zkb_transcript zkb_transcript;

enum {
    ZKB_OK = 0,
    ZKB_E_CUDA = 1,         /* CUDA runtime error (no device, out of memory, launch failure) */
    ZKB_E_ARG = 2,          /* bad argument (null pointer, size not a power of two, ...) */
    ZKB_E_LOGUP_IDENTITY = 3,   /* "LogUp identity failed — invalid lookups" (lookup.rs:572-577, 733-738) */
    ZKB_E_ALPHA_COLLISION = 4,  /* "alpha collision with lookup/table encoding" (lookup.rs:550-555, 712-717) */
    ZKB_E_NOT_QR = 5,       /* "compute_r: d/sum_sq is not a quadratic residue" (transformer/mod.rs:182) */
    ZKB_E_LENGTH = 6,       /* a length assertion of the reference failed (matmul.rs:161, 861) */
    ZKB_E_TOO_LARGE = 7,    /* request exceeds a documented fixed capacity */
    ZKB_E_TIMEOUT = 8,      /* a peer GPU of a split sumcheck did not answer within the exchange's time limit */
    ZKB_E_DIV_ZERO = 9      /* batch_inverse met a zero element: p3's `.inverse()` panics there (lookup.rs:336, 358) */
};

/* Alignment.  Host pointers need no particular alignment.  Device pointers passed by the caller
 * (the `on_device` / `w_on_device` / `*_dev` arguments) must be 4-byte aligned; those that kernels
 * read with 16-byte loads must be 16-byte aligned, and each such argument says so below.  A
 * misaligned device pointer is refused on the host with ZKB_E_ARG before anything is launched
 * (on the GPU it would be a fault that loses the whole CUDA context).  Memory from cudaMalloc or
 * zkb_buf_alloc is always aligned enough; sub-slices of a pool are the caller's responsibility. */

/* Sumcheck prover kinds; one per reference function. */
enum {
    ZKB_SC_PRODUCT = 0,              /* prove_product / _parallel / _best      sumcheck.rs:211-272, 389-482, 815-828 */
    ZKB_SC_TRIPLE = 1,               /* prove_triple / _parallel / _best       sumcheck.rs:277-354, 487-619, 831-845 */
    ZKB_SC_PRODUCT_ONES = 2,         /* prove_product_ones / _parallel / _best sumcheck.rs:857-978 */
    ZKB_SC_PRODUCT_EF = 3,           /* prove_product_ef                       sumcheck.rs:1204-1258 */
    ZKB_SC_PRODUCT_EF_FULL = 4,      /* prove_product_ef_full                  sumcheck.rs:1262-1315 */
    ZKB_SC_PRODUCT_EF_MIXED = 5,     /* prove_product_ef_mixed                 matmul.rs:889-944 */
    ZKB_SC_TRIPLE_EF_FULL = 6,       /* prove_triple_ef_full                   sumcheck.rs:1318-1384 */
    ZKB_SC_PRODUCT_ONES_EF_FULL = 7  /* prove_product_ones_ef_full             sumcheck.rs:1389-1435 */
};

/* ---- context (replaces MetalContext::get / MetalKernels::get, gpu/metal_device.rs:47-77) ---- */
int32_t zkb_ctx_create(int32_t device, zkb_ctx** out);
void zkb_ctx_destroy(zkb_ctx* ctx);
const char* zkb_last_error(const zkb_ctx* ctx);
int32_t zkb_ctx_sync(zkb_ctx* ctx);
/* A context keeps a scratch arena on the device that grows to what its largest proof needed and is
 * reused from then on (nothing is allocated per proof).  zkb_ctx_scratch_bytes reports its size;
 * zkb_ctx_trim waits for the context's stream and gives the arena back to the device - for a caller
 * that proves more layers than fit side by side (the reference bounds the same working set by
 * proving in chunks, pipeline/prove.rs:112-151). */
int32_t zkb_ctx_trim(zkb_ctx* ctx);
uint64_t zkb_ctx_scratch_bytes(const zkb_ctx* ctx);
/* Tuning options of one context, for measurements (none is needed in production; value 0 restores
 * the built-in choice).  ZKB_OPT_PLAIN_TAIL: nonzero = every sumcheck ends in the plain
 * single-CTA tail instead of the pipelined one.  ZKB_OPT_SINGLE_CTA_THREADS /
 * ZKB_OPT_PIPE_THREADS: thread counts of the single-CTA kernels and of the pipelined tail.
 * ZKB_OPT_NO_FUSED_FOLD: nonzero = product sumchecks over base-field tables fold one challenge per
 * launch (they normally fold the first two challenges in one pass over the base tables).
 * ZKB_OPT_FOLD2_VEC: pair indices per thread (1, 2 or 4) of that two-challenge pass.
 * ZKB_OPT_BASEFOLD_IN_ORDER: nonzero = a Basefold opening runs fold, tree and transcript step of
 * each round one after another on the context's stream (normally the folds and trees of all rounds
 * whose challenge is a coordinate of the point run ahead on a second stream).
 * ZKB_OPT_MATVEC_PREFETCH_ROWS: 0..8, rows per CTA that a forward matvec prefetches into L2 before it
 * waits for its input vector (default 2; 8 is the CTA's whole first pass; here 0 is a value, not "default").
 * ZKB_OPT_MATVEC_RING: nonzero = forward matvecs whose rows are a multiple of 16 bytes (at most 64 KB)
 * go through a shared-memory ring filled by bulk asynchronous copies, one persistent CTA per SM, instead of
 * the kernel that stages rows in registers (measured slower on the 4B shape: 5.49 against 5.22 ms for the
 * forward chain, so it is off unless asked for).
 * ZKB_OPT_SHARED_SM_HASH: 1 = the single-CTA kernels that advance the transcript do not reserve an SM's
 * shared memory for themselves (normally they ask for 200 KB they do not use, so that other contexts' kernels
 * do not share their SM); 16 .. 200 = they reserve that many KB.
 * ZKB_OPT_ATTENTION_THREADS: threads per (head, row) CTA of the row-attention kernels: 64, 128 or 256; 0 = chosen
 * from seq_len and d_head (fewer threads let more rows share an SM; a row's critical path is its one-thread hash chain). */
enum { ZKB_OPT_PLAIN_TAIL = 0, ZKB_OPT_SINGLE_CTA_THREADS = 1, ZKB_OPT_PIPE_THREADS = 2, ZKB_OPT_NO_FUSED_FOLD = 3, ZKB_OPT_FOLD2_VEC = 4,
       ZKB_OPT_BASEFOLD_IN_ORDER = 5, ZKB_OPT_MATVEC_PREFETCH_ROWS = 6,
       ZKB_OPT_MATVEC_RING = 7, ZKB_OPT_SHARED_SM_HASH = 8, ZKB_OPT_ATTENTION_THREADS = 9 };
int32_t zkb_ctx_set_option(zkb_ctx* ctx, int32_t option, int32_t value);
/* The context's cudaStream_t (as an opaque pointer), for callers that enqueue their own work in order with the library's. */
void* zkb_ctx_stream(zkb_ctx* ctx);
/* CUDA-event stopwatch on the context's stream (for benchmarks; device time, not wall clock). */
int32_t zkb_timer_start(zkb_ctx* ctx);
int32_t zkb_timer_stop_ms(zkb_ctx* ctx, float* ms);
/* When enabled, sumcheck calls record one CUDA event per launch; read back with
 * zkb_profile_read: ms[i] = device time of launch i of the most recent sumcheck call. */
int32_t zkb_profile_enable(zkb_ctx* ctx, int32_t on);
int32_t zkb_profile_read(zkb_ctx* ctx, float* ms, size_t cap, size_t* n);
/* While profiling is enabled the bandwidth-bound matrix kernels are bracketed by CUDA events.
 * zkb_profile_ranges sums them per tag since the last call: ms[tag], bytes[tag] (algorithmic
 * bytes = 4 m n per launch), count[tag]; arrays of ZKB_RANGE_COUNT entries.  Synchronises. */
enum { ZKB_RANGE_FOLD_EQ_MATVEC = 0, ZKB_RANGE_MATVEC_FORWARD = 1, ZKB_RANGE_COUNT = 2 };
int32_t zkb_profile_ranges(zkb_ctx* ctx, double* ms, double* bytes, uint64_t* count);
/* Launch trace (a debugging aid, off by default): while on, every launch site of the context
 * records an event behind its kernel, also inside a captured layer graph, whose replays refresh
 * the time stamps.  zkb_trace_dump waits for the context's stream and writes "index,site,ms" lines
 * (site = source file:line of the launch, ms = time since the first traced launch of `base`, or of
 * `ctx` itself when base is NULL) to `path`.  Enabling or disabling clears the log. */
int32_t zkb_trace_enable(zkb_ctx* ctx, int32_t on);
int32_t zkb_trace_dump(zkb_ctx* ctx, zkb_ctx* base, const char* path);
/* Number of kernels this context has launched since creation. */
uint64_t zkb_launch_count(const zkb_ctx* ctx);

/* ---- device buffers (replaces GpuBuffer::from_field_slice / to_field_vec, gpu/metal_buffer.rs:9-53) ---- */
int32_t zkb_buf_alloc(zkb_ctx* ctx, size_t n_u32, uint32_t** out_dev);
int32_t zkb_buf_upload_u32(zkb_ctx* ctx, const uint32_t* host, size_t n, uint32_t* dst_dev);
int32_t zkb_buf_download_u32(zkb_ctx* ctx, const uint32_t* src_dev, size_t n, uint32_t* host);
int32_t zkb_buf_free(zkb_ctx* ctx, uint32_t* dev);
/* Page-locked host memory, so that host-pointer calls copy at full PCIe rate. */
int32_t zkb_host_alloc(zkb_ctx* ctx, size_t bytes, void** out_host);
int32_t zkb_host_free(zkb_ctx* ctx, void* host);

/* ---- transcript (device-resident mirror of Transcript, sumcheck.rs:110-206) ---- */
int32_t zkb_tr_new(zkb_ctx* ctx, const uint8_t* label, size_t len, zkb_transcript** out);   /* Transcript::new   :115-119 */
void zkb_tr_free(zkb_transcript* tr);
int32_t zkb_tr_absorb_u32(zkb_transcript* tr, uint32_t v);                                  /* absorb             :121-123 */
int32_t zkb_tr_absorb_many(zkb_transcript* tr, const uint32_t* host, size_t n);              /* absorb_many        :125-129 */
int32_t zkb_tr_absorb_many_dev(zkb_transcript* tr, const uint32_t* dev, size_t n);
int32_t zkb_tr_absorb_bytes(zkb_transcript* tr, const uint8_t* bytes, size_t n);             /* absorb_bytes       :177-179 */
int32_t zkb_tr_squeeze(zkb_transcript* tr, uint32_t* out);                                  /* squeeze            :147-171 */
int32_t zkb_tr_squeeze_ef(zkb_transcript* tr, uint32_t out[4]);                              /* squeeze_ef         :182-188 */
/* Serialised SHA-256 stream state (h[8] LE u32, buflen u32, pad u32, total u64, buf[64]) so a
 * host-side Transcript and the device one can hand the stream to each other. */
#define ZKB_TR_STATE_BYTES 112
int32_t zkb_tr_export(zkb_transcript* tr, uint8_t state[ZKB_TR_STATE_BYTES]);
int32_t zkb_tr_import(zkb_transcript* tr, const uint8_t state[ZKB_TR_STATE_BYTES]);

/* ---- batch Basefold: k polynomials, possibly of different sizes, opened with one fold chain (basefold.rs:769-1590) ----
 * zkb_basefold_batch_precommit = batch_precommit_multi_height (basefold.rs:1183-1216): polynomial i has n_coeffs[i] coefficients and
 * the caller's log_ns[i] (n_coeffs[i] <= 2^log_ns[i]; ZKB_E_LENGTH otherwise).  All are encoded with the tables of the largest log_n and
 * their Merkle trees built; codewords and trees stay in device memory until zkb_basefold_batch_destroy (the transcript-independent half,
 * done once at load time).  on_device != 0: the coefficient pointers are device memory that must stay valid (they are read again for the
 * final value); otherwise they are copied.  At most 4096 polynomials.
 * zkb_basefold_batch_prove = batch_prove_with_precommit (basefold.rs:1221-1378): absorbs the roots (by size, descending; ties in input
 * order), squeezes rho, builds the rho-weighted sum of the largest codewords, squeezes the whole fold point, and runs one fold chain in
 * which smaller codewords join when the chain reaches their length, with the joined trees opened at that round's positions.
 * individual_openings != 0 (all polynomials of one size, ZKB_E_ARG otherwise) also opens every tree at the final positions: the result is
 * then batch_commit_and_prove (basefold.rs:801-956).  out = bincode(Vec<BasefoldCommitment>) in input order followed by
 * bincode(BasefoldBatchProof); poly indices inside the proof are positions in the size-sorted order, as in the reference. */
typedef struct zkb_bf_batch zkb_bf_batch;
int32_t zkb_basefold_batch_precommit(zkb_ctx* ctx, const uint32_t* const* coeffs, const size_t* n_coeffs, const uint32_t* log_ns, size_t k,
                                     int32_t on_device, int32_t node_hash, zkb_bf_batch** out);
size_t zkb_basefold_batch_count(const zkb_bf_batch* batch);
uint64_t zkb_basefold_batch_device_bytes(const zkb_bf_batch* batch);
int32_t zkb_basefold_batch_commitment(const zkb_bf_batch* batch, size_t index, uint8_t root[16], uint64_t* num_coeffs, uint64_t* log_n);
int32_t zkb_basefold_batch_prove(zkb_bf_batch* batch, zkb_transcript* tr, int32_t individual_openings, uint8_t* out, size_t cap, size_t* len);
void zkb_basefold_batch_destroy(zkb_bf_batch* batch);
/* batch_verify_opening (basefold.rs:959-1137) on those bytes: *accepted = 1 / 0.  Like the reference's verifier it checks the roots'
 * transcript, every Merkle opening and the fold relation with the joined polynomials' contributions at 24 positions per round, not the
 * final value.  ZKB_E_ARG when the bytes do not decode. */
int32_t zkb_basefold_batch_verify_opening(zkb_ctx* ctx, zkb_transcript* tr, const uint8_t* bytes, size_t len, int32_t node_hash, int32_t* accepted);

/* ---- row-decomposed attention at seq_len >= 2 ----
 * prove_row_attention (proving/attention.rs:116-276), as the op-list prover calls it for an "attention" op
 * (pipeline/prove.rs:419-425), and the op's forward pass (pipeline/forward.rs:233-276).
 *   q, k, v     (num_heads, seq_len, d_head) row-major canonical M31 values
 *   table_out   output column of the exp table in table order (65536 entries, input raw as i16 -
 *               lookup.rs build_exp_table - or 256 entries, input raw as i8, as the reference's tests build it)
 *   on_device   0: all pointers are host memory; 1: q, k, v, table_out (and attn_out / out) are device pointers
 * Forward: out[h][i] = sum_l y[l] V[h][l], y = e / sum(e), e[j] = table(Q[h][i] . K[h][j]).
 * Prove: `tr` absorbs num_heads, seq_len, d_head, every (head, row) is proved on a transcript of its own
 * ("row-attn-h{h}-r{i}": score matmul, softmax = LogUp of e + sum sumcheck + division sumcheck, output matmul),
 * one CTA per row, then `tr` absorbs every row's scores and outputs.  `out` receives bincode(RowAttentionProof)
 * with seq1_consistency = None; attn_out (may be NULL) the op's output.  seq_len <= 1024, d_head <= 256.
 * ZKB_E_ARG with a message when a score is not an input of the table or a row's sum of e is zero (the
 * reference panics on both: attention.rs:105-108).
 * tr = NULL (prover and verifier): the caller keeps its transcript.  Only the rows are proved (checked); the caller absorbs num_heads
 * [, num_kv_heads], seq_len, d_head and then every row's scores and outputs - all of them in the proof - into its own transcript, as
 * attention.rs:140-143 and 254-265 do.  That stream is 4 * rows * (seq_len + d_head) bytes of strictly serial SHA-256, which a CPU core
 * with SHA instructions hashes about twenty times faster than one GPU thread: for the 1536 rows of a 12 x 128 x 64 call the GPU-side
 * transcript costs 21 ms, the rows themselves 1.1 ms. */
int32_t zkb_row_attention_forward(zkb_ctx* ctx, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t seq_len,
                                  size_t d_head, const uint32_t* table_out, size_t n_table, int32_t on_device, uint32_t* out);
int32_t zkb_prove_row_attention(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads,
                                size_t seq_len, size_t d_head, const uint32_t* table_out, size_t n_table, int32_t on_device,
                                uint32_t* attn_out, uint8_t* out, size_t cap, size_t* len);
/* Grouped-query form, prove_row_attention_gqa (attention.rs:386-500; the "gqa_attention" op, prove.rs:572-584, forward.rs:555-660):
 * q has num_heads heads, k and v have num_kv_heads (a divisor of num_heads); query head h reads K/V head h / (num_heads / num_kv_heads);
 * the rows' transcripts are labelled "gqa-h{h}-r{i}" and `tr` absorbs num_heads, num_kv_heads, seq_len, d_head.  num_kv_heads = 0 is
 * the plain form above. */
int32_t zkb_row_attention_gqa_forward(zkb_ctx* ctx, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads, size_t num_kv_heads,
                                      size_t seq_len, size_t d_head, const uint32_t* table_out, size_t n_table, int32_t on_device, uint32_t* out);
int32_t zkb_prove_row_attention_gqa(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* q, const uint32_t* k, const uint32_t* v, size_t num_heads,
                                    size_t num_kv_heads, size_t seq_len, size_t d_head, const uint32_t* table_out, size_t n_table,
                                    int32_t on_device, uint32_t* attn_out, uint8_t* out, size_t cap, size_t* len);

/* verify_row_attention / verify_row_attention_gqa (attention.rs:279-385, 503-590) on the bytes the prover returns: *accepted = 1 / 0.  k, v as for
 * the prover (num_kv_heads = 0: the plain form).  Every row is checked by one CTA: the row's transcript replayed, the three sumchecks of the
 * softmax and the two matmul sumchecks verified, K(r, s) and V^T(r, s) recomputed from k and v; `tr` absorbs what the prover's absorbed.  As
 * in the reference neither q nor the exp table is read, the lookup's inputs are not compared with the scores, and attn_weights / y_values
 * are not looked at.  A proof whose vectors do not have the lengths the prover produces is rejected; ZKB_E_ARG when the bytes do not decode. */
int32_t zkb_verify_row_attention(zkb_ctx* ctx, zkb_transcript* tr, const uint8_t* proof, size_t len, const uint32_t* k, const uint32_t* v,
                                 size_t num_heads, size_t num_kv_heads, size_t seq_len, size_t d_head, int32_t on_device, int32_t* accepted);

/* ---- weights in the reference's wire format, kept resident ----
 * zkb_weightset_preload takes the preload block of the reference's server mode (server.rs:33-94):
 *   [count u32] then per matrix [name_len u32][name, UTF-8][m u32][n u32][m * n u32 LE]
 * copies every matrix to device memory (through pinned staging buffers, the copy to the GPU overlapping
 * the host copy of the next piece), computes its commit_weights_fast root on the GPU and keeps both by name,
 * as the server's HashMap<String, PreloadedLinear> does (a later matrix of the same name replaces the
 * earlier one).  The caps are the reference's (at most 65536 matrices, names up to 4096 bytes, dimensions up
 * to 2^24, 2^30 elements per matrix); a violation, a block that ends early or a name that is not UTF-8 gives
 * ZKB_E_ARG and nothing stays allocated.  *consumed (may be NULL) = bytes of the block that were read: the
 * requests follow from there.  Pointers from zkb_weightset_get are device pointers (row-major u32, 16-byte
 * aligned) valid until zkb_weightset_destroy; they can be passed wherever `W` with w_on_device != 0 is taken. */
typedef struct zkb_weightset zkb_weightset;
int32_t zkb_weightset_preload(zkb_ctx* ctx, const uint8_t* block, size_t len, zkb_weightset** out, size_t* consumed);
uint32_t zkb_weightset_count(const zkb_weightset* ws);
uint64_t zkb_weightset_bytes(const zkb_weightset* ws);
int32_t zkb_weightset_get(const zkb_weightset* ws, const char* name, const uint32_t** w_dev, size_t* m, size_t* n, uint8_t root[32]);
void zkb_weightset_destroy(zkb_weightset* ws);

/* ---- sumcheck provers ----
 * tables[i] holds 2^num_vars elements (u32 each for base-field inputs, 4 u32 each for EF
 * inputs; which is fixed by `kind`).  `on_device` != 0: tables are device pointers and are
 * left untouched; EF tables on the device must be 16-byte aligned (ZKB_E_ARG otherwise),
 * base-field tables only 4-byte (16-byte alignment selects the faster vectorised launches).
 * Outputs (host memory):
 *   round_polys  num_vars x (stored evals per round) x w   u32
 *   challenges   num_vars x w                               u32
 *   finals       (number of tables, min 2) x w              u32   (f(s), g(s)[, h(s)]; f(s)=1 for ONES)
 * with w = 1 for base-field kinds and 4 for EF kinds; stored evals per round: PRODUCT 3
 * [s0,s1,s2], TRIPLE 4, PRODUCT_ONES 2 [s0,s2], PRODUCT_EF 2 [s0,s2], PRODUCT_EF_FULL 3,
 * PRODUCT_EF_MIXED 3, TRIPLE_EF_FULL 3 [s0,s2,s3], PRODUCT_ONES_EF_FULL 2 [s0,s2]. */
int32_t zkb_sumcheck_prove(zkb_ctx* ctx, zkb_transcript* tr, int32_t kind, const uint32_t* const* tables,
                           uint32_t num_vars, int32_t on_device, uint32_t* round_polys, uint32_t* challenges,
                           uint32_t* finals);

/* ---- field helpers, commitments, matrix kernels ---- */
/* commit_weights_fast: blake3("weights" || LE u32 buffer)            weight_commitment.rs:82-107 */
int32_t zkb_commit_weights_fast(zkb_ctx* ctx, const uint32_t* w, size_t n, int32_t on_device, uint8_t root[32]);
/* eq_evals / eq_evals_ef: r has k (ef: 4k) words, out 2^k (ef: 4 * 2^k) words   m31_ops.rs:30-50, 175-191
 * (replaces eq_evals_gpu / MetalKernels::eq_butterfly, m31_ops.rs:54-78, gpu/metal_kernels.rs:232-253) */
int32_t zkb_eq_evals(zkb_ctx* ctx, const uint32_t* r, uint32_t k, int32_t ef, uint32_t* out);
/* mle_evaluate (m31_ops.rs:11-26): MLE of `evals` (n <= 2^k values, the rest of the hypercube is
 * zero) at `point` (k base-field coordinates, host memory, point[0] = most significant index bit).
 * on_device != 0: evals is a device pointer.  One pass over the table. */
int32_t zkb_mle_eval_base(zkb_ctx* ctx, const uint32_t* evals, size_t n, const uint32_t* point, uint32_t k, int32_t on_device,
                          uint32_t* out);
/* mle_evaluate_ef (m31_ops.rs:155-171): the same at an extension-field point (4k words).
 * evals_ef = 0: base-field evals (the reference's signature); evals_ef != 0: evals are EF elements
 * (4 words each; what the reference's verifier folds after a sumcheck).  A device pointer to EF
 * evals must be 16-byte aligned. */
int32_t zkb_mle_eval_ef(zkb_ctx* ctx, const uint32_t* evals, size_t n, int32_t evals_ef, const uint32_t* point, uint32_t k,
                        int32_t on_device, uint32_t out[4]);
/* batch_inverse / batch_inverse_ef (lookup.rs:322-368; replaces MetalKernels::batch_inverse,
 * gpu/metal_kernels.rs:212-229, called at lookup.rs:491-542): out[i] = 1 / vals[i].
 * on_device != 0: vals and out are device pointers (out may equal vals; EF: both 16-byte
 * aligned).  A zero element gives ZKB_E_DIV_ZERO (the reference panics there). */
int32_t zkb_batch_inverse_base(zkb_ctx* ctx, const uint32_t* vals, size_t n, int32_t on_device, uint32_t* out);
int32_t zkb_batch_inverse_ef(zkb_ctx* ctx, const uint32_t* vals, size_t n, int32_t on_device, uint32_t* out);
/* fold_eq_matvec / fold_eq_matvec_ef: out[j] = sum_i eq(r)[i] W[i][j], zero-padded to n_pad    matmul.rs:76-128, 743-835
 * W on the device (w_on_device != 0) with n a multiple of 4 must be 16-byte aligned; the same holds for
 * every `W` / `w_on_device` pair below. */
int32_t zkb_fold_eq_matvec(zkb_ctx* ctx, const uint32_t* W, size_t m, size_t n, const uint32_t* r, uint32_t log_m, int32_t ef,
                           int32_t w_on_device, uint32_t* out);
/* matmul_forward: y = W x mod p                                        transformer/mod.rs:140-163 */
int32_t zkb_matvec_forward(zkb_ctx* ctx, const uint32_t* W, const uint32_t* x, size_t m, size_t n, int32_t w_on_device, uint32_t* y);
/* rmsnorm_forward with the QR perturbation search                      transformer/mod.rs:245-288 */
int32_t zkb_rmsnorm_forward(zkb_ctx* ctx, const uint32_t* x, const uint32_t* gamma, size_t d, uint32_t* out, uint32_t* x_used,
                            int32_t* delta);

/* requantize_to_i16_field (transformer/mod.rs:293-324): q[i] = the int16-range requantisation of the
 * centred value raw[i] (scaled by 32767 / max |raw| when that maximum exceeds 32767), and, when a
 * table is given (device-resident output column of 65536 or 256 entries), t[i] = table[q[i]]
 * (qwen.rs:286-316).  raw: host or device; q_out, t_out: host.  A value outside the table is ZKB_E_ARG. */
int32_t zkb_requantize_lookup(zkb_ctx* ctx, const uint32_t* raw, size_t n, int32_t on_device, const uint32_t* table_out_dev,
                              uint32_t n_table, uint32_t* q_out, uint32_t* t_out);

/* ---- sub-protocol provers: host inputs, proof returned as the reference's bincode bytes.
 * *len receives the proof length; ZKB_E_TOO_LARGE if it exceeds cap. ---- */
/* prove_matmul_succinct_ef -> SuccinctMatmulProofEF                    matmul.rs:963-997 */
int32_t zkb_prove_matmul_succinct_ef(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* W, const uint32_t* x, const uint32_t* y,
                                     size_t m, size_t n, int32_t w_on_device, uint8_t* out, size_t cap, size_t* len);
/* The same prover under one of the reference's compile-time weight-binding modes
 * (bind_weights_ef, matmul.rs:360-453): ZKB_BIND_BLAKE3 = default build (identical to the call
 * above), ZKB_BIND_PCS = feature pcs (Basefold of w_partial), ZKB_BIND_PCS_FULL = feature
 * pcs-full (Basefold of the row-padded matrix W).  In the PCS modes basefold_proof is Some(..)
 * and node_hash (ZKB_NODE_*) selects the Merkle node hash. */
#define ZKB_BIND_BLAKE3 0
#define ZKB_BIND_PCS 1
#define ZKB_BIND_PCS_FULL 2
int32_t zkb_prove_matmul_succinct_ef_bind(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* W, const uint32_t* x, const uint32_t* y,
                                          size_t m, size_t n, int32_t w_on_device, int32_t bind_mode, int32_t node_hash, uint8_t* out,
                                          size_t cap, size_t* len);
/* Base-field twins (challenges in M31; the MLP / GPT-2 op-list mode of the reference):
 * prove_matmul_succinct -> SuccinctMatmulProof                          matmul.rs:134-180, 482-511 */
int32_t zkb_prove_matmul_succinct(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* W, const uint32_t* x, const uint32_t* y, size_t m,
                                  size_t n, int32_t w_on_device, uint8_t* out, size_t cap, size_t* len);
/* prove_mle_eval_no_merkle (label_len = 0) / prove_mle_eval_bound (label + 32-byte root absorbed first)
 * -> MleEvalProof; w: n <= 2^k values, point: k challenges          weight_commitment.rs:177-206, 437-447 */
int32_t zkb_prove_mle_eval(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* w, size_t n, const uint32_t* point, uint32_t k,
                           const uint8_t* label, size_t label_len, const uint8_t root[32], uint8_t* out, size_t cap, size_t* len);
/* prove_hadamard (is_add = 0) / prove_add (is_add = 1); point = k base-field challenges
 * -> HadamardProof / AddProof                                          elementwise.rs:50-98, 189-235 */
int32_t zkb_prove_elementwise(zkb_ctx* ctx, zkb_transcript* tr, int32_t is_add, const uint32_t* a, const uint32_t* b, const uint32_t* c,
                              size_t n, const uint32_t* point, uint32_t k, uint8_t* out, size_t cap, size_t* len);
/* prove_hadamard_ef (is_add = 0) / prove_add_ef (is_add = 1); point = k EF challenges    elementwise.rs:429-480, 545-595 */
int32_t zkb_prove_elementwise_ef(zkb_ctx* ctx, zkb_transcript* tr, int32_t is_add, const uint32_t* a, const uint32_t* b,
                                 const uint32_t* c, size_t n, const uint32_t* point, uint32_t k, uint8_t* out, size_t cap, size_t* len);
/* prove_rmsnorm_ef -> RmsNormProofEF                                   rmsnorm.rs:512-667 */
int32_t zkb_prove_rmsnorm_ef(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d,
                             int32_t delta, uint8_t* out, size_t cap, size_t* len);
/* prove_lookup_ef -> LookupProofEF; table_out = output column of a 65536- or 256-entry table   lookup.rs:643-762 */
int32_t zkb_prove_lookup_ef(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* table_out, size_t n_table, const uint32_t* inputs,
                            const uint32_t* outputs, size_t n, uint8_t* out, size_t cap, size_t* len);

/* prove_rmsnorm (base-field challenges) -> RmsNormProof                                        rmsnorm.rs:96-246 */
int32_t zkb_prove_rmsnorm(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* x, const uint32_t* gamma, const uint32_t* y, size_t d,
                          int32_t delta, uint8_t* out, size_t cap, size_t* len);
/* prove_lookup (base-field challenges) -> LookupProof                                          lookup.rs:432-604 */
int32_t zkb_prove_lookup(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* table_out, size_t n_table, const uint32_t* inputs,
                         const uint32_t* outputs, size_t n, uint8_t* out, size_t cap, size_t* len);

/* ---- resident Qwen-style layer (QwenLayerWeights + commit_qwen_layer + trace)   transformer/qwen.rs:62-73, 148-161 ----
 * dims = {d_model, d_ff, num_q_heads, num_kv_heads, d_head, v_num_heads, v_d_head};
 * weights = {norm1_gamma, w_q, w_k, w_v, w_o, w_g_proj, norm2_gamma, w_gate, w_up, w_down} (host, row-major);
 * the tables are the output columns of build_silu_table / build_sigmoid_table already on the device. */
typedef struct zkb_qwen_layer zkb_qwen_layer;
int32_t zkb_qwen_layer_create(zkb_ctx* ctx, const uint64_t dims[7], const uint32_t* const weights[10],
                              const uint32_t* silu_table_dev, const uint32_t* sigmoid_table_dev, uint32_t n_table,
                              zkb_qwen_layer** out);
void zkb_qwen_layer_destroy(zkb_qwen_layer* layer);
/* the eight 32-byte weight commitments in the order q, k, v, o, g_proj, gate, up, down */
int32_t zkb_qwen_layer_commitments(zkb_qwen_layer* layer, uint8_t roots[256]);
/* qwen_forward_indexed                                                  transformer/qwen.rs:211-325 */
int32_t zkb_qwen_layer_forward(zkb_qwen_layer* layer, const uint32_t* x, int32_t x_on_device, uint32_t* y, int32_t y_on_device);
/* Same forward, fully asynchronous, for a chain of layers that live on different contexts:
 * with prev != NULL the input is prev's device-resident output and this layer's stream waits
 * for prev's forward through a CUDA event (prev's forward must already have been issued);
 * with prev == NULL the input is x.  Errors surface at zkb_qwen_layer_prove_end. */
int32_t zkb_qwen_layer_forward_async(zkb_qwen_layer* layer, zkb_qwen_layer* prev, const uint32_t* x, int32_t x_on_device);
/* A model may give all its layers one shared stream for their forward passes (zkb_stream_create
 * with high_priority = 1): the forward chain then runs back to back and ahead of the proof
 * kernels of earlier layers; each layer's own stream waits for its forward before proving, and
 * a later forward waits for the layer's previous proof.  NULL returns to the layer's own stream. */
int32_t zkb_stream_create(zkb_ctx* ctx, int32_t high_priority, void** out);
void zkb_stream_destroy(void* stream);
int32_t zkb_qwen_layer_set_forward_stream(zkb_qwen_layer* layer, void* stream);
/* Waits for the layer's (asynchronous) forward pass only - not for a proof queued behind it -
 * and copies the layer output (d_model words) to the host. */
int32_t zkb_qwen_layer_read_output(zkb_qwen_layer* layer, uint32_t* y_host);
/* Host-side wait for the layer's (asynchronous) forward pass only; afterwards the output at
 * zkb_qwen_layer_output_dev may be read on any stream or sent to another GPU while the layer's
 * proof is still running. */
int32_t zkb_qwen_layer_wait_forward(zkb_qwen_layer* layer);
const uint32_t* zkb_qwen_layer_output_dev(const zkb_qwen_layer* layer);
/* The launch sequence of a layer proof depends only on the layer's shapes and binding mode, so
 * from the second proof on it is replayed from a CUDA graph captured on the layer's stream
 * (one graph launch instead of about two thousand kernel launches).  on = 0 switches that off. */
int32_t zkb_qwen_layer_use_graph(zkb_qwen_layer* layer, int32_t on);
/* What the next prove_begin will do: 0 = enqueue launch by launch, 1 = capture (once, slower),
 * 2 = replay.  A host that drives many layers from several threads can use this to let the
 * one-off captures happen one at a time. */
int32_t zkb_qwen_layer_graph_state(const zkb_qwen_layer* layer);
/* Selects what the reference fixes at compile time for the layer's eight matmul proofs: the
 * weight binding (ZKB_BIND_*, features pcs / pcs-full, matmul.rs:360-453) and the Merkle node
 * hash (ZKB_NODE_*, pcs.rs:87-135).  Default after create: ZKB_BIND_BLAKE3. */
int32_t zkb_qwen_layer_set_binding(zkb_qwen_layer* layer, int32_t bind_mode, int32_t node_hash);
/* prove_qwen_layer_precommitted_ef on a fresh transcript "qwen-layer-{idx}" || input_hash
 * (transformer/qwen.rs:795-912, pipeline/prove.rs:166-168) -> QwenLayerProofEF bincode.
 * prove_begin only enqueues GPU work; prove_end waits and serialises. */
int32_t zkb_qwen_layer_prove_begin(zkb_qwen_layer* layer, uint32_t layer_idx, const uint8_t input_hash[32]);
int32_t zkb_qwen_layer_prove_end(zkb_qwen_layer* layer, uint8_t* out, size_t cap, size_t* len);
int32_t zkb_qwen_layer_prove(zkb_qwen_layer* layer, uint32_t layer_idx, const uint8_t input_hash[32], uint8_t* out, size_t cap,
                             size_t* len);
/* verify_qwen_layer_ef_indexed (transformer/qwen.rs:932-1097) for the proof bytes zkb_qwen_layer_prove returns.
 * Like the reference's verifier it works on a forward pass of its own: call zkb_qwen_layer_forward with the
 * layer's input first; the layer object then holds the trace the proof is checked against.  y_expected
 * (d_model words, host memory; may be NULL) is compared with that pass's output.  The transcript is replayed
 * on the device (the sumcheck rounds, the MLE-eval proofs, the LogUp sums, a Basefold opening when the matmul
 * proofs carry one); *accepted = 1 / 0.  Bytes that do not decode give ZKB_E_ARG. */
int32_t zkb_qwen_layer_verify(zkb_qwen_layer* layer, uint32_t layer_idx, const uint8_t input_hash[32], const uint8_t* proof, size_t len,
                              const uint32_t* y_expected, int32_t* accepted);
/* The same in two halves, so that the layers of a model (one context each) are checked side by side: begin decodes and
 * enqueues without waiting (y_expected is read before it returns), end waits and gives the verdict. */
int32_t zkb_qwen_layer_verify_begin(zkb_qwen_layer* layer, uint32_t layer_idx, const uint8_t input_hash[32], const uint8_t* proof, size_t len,
                                    const uint32_t* y_expected);
int32_t zkb_qwen_layer_verify_end(zkb_qwen_layer* layer, int32_t* accepted);

/* Tells a context that it shares the GPU with many other contexts that run at the same time (one
 * per layer of a model).  Its kernels then leave half of every SM free: single-CTA kernels use
 * 512 threads, wide kernels two or three CTAs per SM (the weight fold one).  Without this a wide
 * kernel fills every SM's register file and every other context's single-CTA kernels - the
 * serial transcript steps - may wait for it to drain.  Off by default: a lone context is fastest
 * with the greedy shapes, and on B200 the 32-layer 4B-shape proof was measured slower with it
 * (34.9 ms against 32.7 ms), the wide kernels losing more than the small ones gain. */
int32_t zkb_ctx_set_shared(zkb_ctx* ctx, int32_t on);

/* ---- one sumcheck split over several GPUs (one process per GPU) ----------------------------
 * No counterpart in the reference, which proves on one machine's cores; this is how a table
 * too large or too slow for one GPU is proved by `world` GPUs (a power of two, at most 8).
 * Rank g holds the elements j with j mod world == g of every table, stored contiguously.
 * Folding is MSB-first, so all but the last log2(world) rounds fold pairs that live on one GPU;
 * per round only the three or four partial sums cross NVLink, written by the round kernel
 * itself into mailboxes in the peers' memory, and every rank advances an identical transcript.
 * Set-up: every rank calls zkb_xch_create and zkb_xch_handle, the caller carries the 64-byte
 * handles between the processes (e.g. an all-gather), every rank calls zkb_xch_connect with
 * all of them.  A rank whose peer does not answer within the time limit (default 4 s) gets
 * ZKB_E_TIMEOUT instead of a proof.  The time-out is sticky: every later call on that exchange
 * fails at once, so after a time-out every rank must destroy its zkb_xch and the ranks must set
 * up a new one together (the context itself stays usable). */
typedef struct zkb_xch zkb_xch;
int32_t zkb_xch_create(zkb_ctx* ctx, uint32_t world, uint32_t rank, zkb_xch** out);
int32_t zkb_xch_handle(zkb_xch* xch, uint8_t handle[64]);
int32_t zkb_xch_connect(zkb_xch* xch, const uint8_t* handles /* world x 64 bytes */);
/* Wires the peers of a multi-rank exchange to private buffers on this GPU that nobody writes:
 * the next split sumcheck then runs into the time limit and returns ZKB_E_TIMEOUT.  For testing
 * the time-out path in one process; not for production use. */
int32_t zkb_xch_connect_loopback(zkb_xch* xch);
int32_t zkb_xch_set_timeout_ms(zkb_xch* xch, uint32_t ms);
void zkb_xch_destroy(zkb_xch* xch);
/* zkb_sumcheck_prove over tables of 2^num_vars elements of which this rank passes its slice of
 * 2^num_vars / world elements.  Every rank makes the same call with transcripts in the same
 * state; every rank receives the complete proof (identical to the single-GPU one) and ends
 * with the same transcript state. */
int32_t zkb_sumcheck_prove_split(zkb_ctx* ctx, zkb_xch* xch, zkb_transcript* tr, int32_t kind, const uint32_t* const* tables,
                                 uint32_t num_vars, int32_t on_device, uint32_t* round_polys, uint32_t* challenges, uint32_t* finals);

/* ---- Merkle trees and the Basefold commitment (features pcs / pcs-full of the reference) -------
 * Digests are 16 bytes.  node_hash selects the reference's hash_node variant
 * (rust/zk_ml_prover/src/proving/pcs.rs:87-135): ZKB_NODE_BLAKE3 = blake3(L || R)[..16], what the
 * reference computes on every target except aarch64; ZKB_NODE_AES_MMO = its aarch64 AES-based
 * compression.  Leaves are the u32 values zero-padded to 16 bytes (pcs.rs:71-75); a vector of n
 * values makes a tree over 2^max(1, ceil(log2 n)) leaves, zero-padded (pcs.rs:143-153). */
#define ZKB_NODE_BLAKE3 0
#define ZKB_NODE_AES_MMO 1

/* MerkleTree::new(values).root() (pcs.rs:143-201). */
int32_t zkb_merkle_root(zkb_ctx* ctx, const uint32_t* values, size_t n, int32_t on_device, int32_t node_hash, uint8_t root[16]);
/* Every internal layer of MerkleTree::new(values), from the parents of the leaves up to the
 * root, 16 bytes per node (pcs.rs:156-196).  *len = (2^h - 1) * 16. */
int32_t zkb_merkle_layers(zkb_ctx* ctx, const uint32_t* values, size_t n, int32_t on_device, int32_t node_hash, uint8_t* out, size_t cap,
                          size_t* len);
/* MerkleTree::new(values).batch_open(indices) (pcs.rs:290-337) as bincode(BatchMerkleProof):
 * indices and values in caller order, then per level the digests of the unknown siblings. */
int32_t zkb_merkle_batch_open(zkb_ctx* ctx, const uint32_t* values, size_t n, int32_t on_device, int32_t node_hash,
                              const uint64_t* indices, size_t n_idx, uint8_t* out, size_t cap, size_t* len);

/* generate_tables(log_n, table_seed(log_n)) (basefold.rs:106-143, 323-328): t_flat and
 * w_flat = 1 / (2 t), 2^log_n - 1 words each, to host memory.  Tables are generated once per
 * (device, log_n) and stay resident, as the reference caches them (basefold.rs:377-393). */
int32_t zkb_basefold_tables(zkb_ctx* ctx, uint32_t log_n, uint32_t* t_flat, uint32_t* w_flat);
/* encode (basefold.rs:169-238) of n coefficients zero-padded to 2^log_n: 2 * 2^log_n words. */
int32_t zkb_basefold_encode(zkb_ctx* ctx, const uint32_t* coeffs, size_t n, int32_t on_device, uint32_t* codeword,
                            int32_t out_on_device);
/* commit_and_prove (basefold.rs:368-396; the _with_tables and _vec variants compute the same):
 * encode, Merkle-commit, absorb the root, then the opening at `point` (n_point words; rounds
 * beyond n_point squeeze their challenge, basefold.rs:508-513).  coeffs and point are both host
 * or both device memory.  Output: bincode(BasefoldCommitment) followed by
 * bincode(BasefoldOpeningProof).  The transcript advances exactly as in the reference. */
int32_t zkb_basefold_commit_and_prove(zkb_ctx* ctx, zkb_transcript* tr, const uint32_t* coeffs, size_t n, const uint32_t* point,
                                      uint32_t n_point, int32_t on_device, int32_t node_hash, uint8_t* out, size_t cap, size_t* len);
/* verify_opening (basefold.rs:611-748, with verify_batch_opening, pcs.rs:345-438): checks the opening
 * proof in `bytes` (bincode(BasefoldCommitment) followed by bincode(BasefoldOpeningProof), exactly what
 * zkb_basefold_commit_and_prove returns) against `claimed` = the polynomial's value at `point` (host,
 * n_point coordinates).  As with the reference function, the caller absorbs the commitment root into
 * the transcript first; the transcript then advances as the prover's did.  *accepted = 1 / 0.
 * Bytes that do not decode give ZKB_E_ARG, a batch proof with more than 256 opened positions
 * ZKB_E_TOO_LARGE (an honest one has 48 and 24). */
int32_t zkb_basefold_verify_opening(zkb_ctx* ctx, zkb_transcript* tr, const uint8_t* bytes, size_t len, const uint32_t* point,
                                    uint32_t n_point, uint32_t claimed, int32_t node_hash, int32_t* accepted);

/* ---- op-list mode (MLP / GPT-2 shaped models; base-field challenges) ----------------------------
 * The reference proves such models as a list of ops on one transcript "structured-ml-proof", in
 * reverse op order (pipeline/forward.rs:24-520, pipeline/prove.rs:36, 191-648).  A zkb_oplist keeps
 * the weights of its ops resident on the GPU (committed once when the op is added); ops are added in
 * forward order; zkb_oplist_prove runs the forward pass and the proofs on the device and returns
 * bincode(Vec<SerializedLayerProof>) (protocol.rs:653-694) in the reference's push order.
 *   linear      y = W x + b; SerializedLayerProof::Matmul(prove_matmul_succinct)          prove.rs:196-235
 *   relu        SerializedLayerProof::Relu (two triple sumchecks, MLE-eval proofs)         prove.rs:237-340
 *   layernorm   layernorm_forward_simple + prove_layernorm_sqr -> LayerNormSqr              gpt2.rs:912-953, layernorm.rs:522-695
 *   gelu        LogUp lookup of the requantised activation -> Gelu(GeluProof)               prove.rs:362-392, gelu.rs:64-72
 *               (the reference receives the requantised pairs from its Python driver; here
 *               requantize_to_i16_field and the table lookup run on the device)
 *   attention   seq_len = 1: output = V, PassThrough with the output hash absorbed            prove.rs:394-411
 *               seq_len >= 2: zkb_oplist_add_attention, row proofs                              prove.rs:419-432
 *   save / add_saved / set_input / passthrough: SaveCommitment, Add, SegmentBoundary, PassThrough (prove.rs:439-489, 635-646)
 *   set_input_requant: set_input whose new activation is requantize_to_i16_field of the current one
 *               (stands in for the float re-quantisation the reference's Python driver does between segments). */
typedef struct zkb_oplist zkb_oplist;
enum { ZKB_OP_RELU = 1, ZKB_OP_ATTENTION_SEQ1 = 2, ZKB_OP_PASSTHROUGH = 3, ZKB_OP_SAVE = 4, ZKB_OP_ADD_SAVED = 5, ZKB_OP_SET_INPUT_REQUANT = 6 };
int32_t zkb_oplist_create(zkb_ctx* ctx, uint32_t input_len, zkb_oplist** out);
void zkb_oplist_destroy(zkb_oplist* list);
int32_t zkb_oplist_add_linear(zkb_oplist* list, const char* name, const uint32_t* W, const uint32_t* bias /* or NULL */, size_t m, size_t n);
/* kind = ZKB_OP_*; aux = the buffer name of save / add_saved (the reference derives the Add proof's
 * save_name from the op name: "add_X" -> "save_X", prove.rs:445). */
int32_t zkb_oplist_add_simple(zkb_oplist* list, int32_t kind, const char* name, const char* aux);
int32_t zkb_oplist_add_layernorm(zkb_oplist* list, const char* name, const uint32_t* gamma, const uint32_t* beta, size_t d);
int32_t zkb_oplist_add_gelu(zkb_oplist* list, const char* name, const uint32_t* table_out_dev, uint32_t n_table);
/* "attention" at seq_len >= 2 (forward.rs:202-306, prove.rs:419-432): the activation is Q | K | V, each (num_heads, seq_len, d_head),
 * or starts with Q when k_values and v_values (host, num_heads * seq_len * d_head words each; both or neither) are given, as the
 * reference takes them from the request.  table_out_dev: the exp table's output column on the device (build_exp_table(exp_scale));
 * it must stay valid while the list lives.  The proof is SerializedLayerProof::Attention(RowAttentionProof), see zkb_prove_row_attention.
 * num_kv_heads != 0: the "gqa_attention" op (forward.rs:555-660, prove.rs:572-584): the activation starts with Q (num_heads heads) | K | V
 * (num_kv_heads heads each), the proof is SerializedLayerProof::GqaAttention. */
int32_t zkb_oplist_add_attention(zkb_oplist* list, const char* name, size_t num_heads, size_t num_kv_heads, size_t seq_len, size_t d_head,
                                 const uint32_t* table_out_dev, uint32_t n_table, const uint32_t* k_values, const uint32_t* v_values);
/* Replaces K and V of attention op `op_index` (0-based position in the list) that was added with k_values / v_values: the next
 * forward pass and proof use the new ones (the reference's requests carry K and V with every op, protocol.rs:714-722). */
int32_t zkb_oplist_set_attention_kv(zkb_oplist* list, uint32_t op_index, const uint32_t* k_values, const uint32_t* v_values);
int32_t zkb_oplist_add_set_input(zkb_oplist* list, const char* name, const uint32_t* values, size_t n);
uint32_t zkb_oplist_output_len(const zkb_oplist* list);
/* forward pass only (x: input_len host words); zkb_oplist_activation then reads the activation after op `op_index`. */
int32_t zkb_oplist_forward(zkb_oplist* list, const uint32_t* x);
int32_t zkb_oplist_activation(zkb_oplist* list, uint32_t op_index, uint32_t* out, size_t cap, size_t* len);
/* forward pass + all proofs */
int32_t zkb_oplist_prove(zkb_oplist* list, const uint32_t* x, uint8_t* out, size_t cap, size_t* len);

/* ---- allocation-free weight fold ----
 * No counterpart in the reference: it exists for callers that must not allocate device memory
 * once they are running (a serving loop with a fixed memory plan, a host that forbids cudaMalloc
 * after start-up, code about to be captured into a CUDA graph).  Computes
 *     out[j] = sum_{i<m} eq[i] * W[i][j]   for j < n,   out[j] = 0 for n <= j < n_pad
 * with eq an array of at least m M31^4 elements (4 u32 each), W an m x n row-major u32 matrix
 * and out n_pad M31^4 elements (n_pad = n rounded up to a power of two) - the same values as
 * zkb_fold_eq_matvec with ef = 1 fed the eq table of r.  All three pointers are device memory
 * of the CURRENT device; W_dev must be 16-byte aligned when n is a multiple of 4 (a caller that
 * carves W out of its own arena must place it so; ZKB_E_ARG otherwise); `stream` is a cudaStream_t (NULL = default stream); work is only
 * enqueued.  It calls no cudaMalloc / cudaFree: its 64-bit accumulators live in a fixed
 * 512 KiB device array inside the library (present on every GPU that loads it), which limits
 * n_pad to 16384 columns - wider matrices are refused with ZKB_E_TOO_LARGE and a message in
 * `err` (optional buffer of err_cap bytes).  The first call on each device looks up that
 * array's device address; make that first call before starting any stream capture.  All calls
 * share the one array: it is cleared at the start of each call, and two calls whose GPU work
 * overlaps (different streams, different threads) corrupt each other - serialise them. */
int32_t zkb_fold_eq_matvec_ef_noalloc(const uint32_t* W_dev, size_t m, size_t n, const uint32_t* eq_dev, uint32_t* out_dev,
                                      void* stream, char* err, size_t err_cap);

#ifdef __cplusplus
}
#endif
#endif /* ZKB200_H */
