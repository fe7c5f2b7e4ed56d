/* qwenny_b200 — C ABI of the B200-native decode / verify hot path.
 *
 * The reference (hellerchr/qwenny) has no linked native library: its Rust host loads a PTX module and launches
 * `extern "C" __global__` kernels by name (src/cuda/core.rs:42-46, src/cuda/qwen/mod.rs:350-361). The boundary a
 * replacement has to honour is therefore "one call per kernel launch site, the kernel's own argument list, the
 * device-memory layouts the host packs". Each entry point below stands for one such launch site: same argument
 * order and meaning as the kernel it replaces, plus the context (scratch, SM count) and the CUDA stream the host
 * launches on. Geometry (grid, block, shared memory), which the reference host computes, is chosen inside.
 *
 * Conventions: every pointer is a device pointer unless its name starts with `h_`; `stream` is a cudaStream_t /
 * CUstream passed as void*; every call only enqueues work (stream-capturable, no allocation, no host sync) and
 * returns 0 or a QB_ERR_* / cudaError_t code (the reference surfaces a CUresult from launch or sync the same way,
 * src/server.rs:640-650). Sizes are the 27B build's compile-time constants (kernels/qwen.cu:8-35 with QWEN_27B).
 */
#ifndef QWENNY_B200_H
#define QWENNY_B200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define QB_OK 0
#define QB_ERR_ARG 1000      /* a shape or pointer the kernels cannot take */
#define QB_ERR_DEVICE 1001   /* a bounded device-side wait ran out (see qb_device_error) */
#define QB_ERR_UNSUPPORTED 1002
#define QB_ERR_TOO_LARGE 1003 /* a size beyond a fixed capacity (qb_marlin_gemm_noalloc; a product of more than 2^31 tile stages x blocks) */

typedef struct qb_ctx qb_ctx;

/* Epilogues of a matrix product: src/cuda/core.rs:58-64 (enum Epi). */
enum { QB_EPI_PLAIN = 0, QB_EPI_SILU = 1, QB_EPI_ARGMAX = 2 };

/* ---- context: what Gemm::load allocates once (src/cuda/core.rs:437-464: SM count, Marlin's `red` and `locks`).
 * Allocates the split-K scratch and tickets on `device`; everything after creation is allocation-free. Like the
 * reference's single `red` / `locks` pair, a context serves one stream at a time: launches that share a context must
 * not overlap on the device (models that run concurrently take a context each). */
int qb_create(int device, qb_ctx** out);
void qb_destroy(qb_ctx* ctx);
/* Non-zero once a kernel gave up a bounded wait (1 producer, 2 consumer, ...); reads and clears the word (syncs). */
int qb_device_error(qb_ctx* ctx);
int qb_sm_count(const qb_ctx* ctx); /* 0 for a null context */
const char* qb_version(void);

/* ---- W4A16 product over a Marlin-packed matrix. Replaces the launches of Gemm::marlin
 * (src/cuda/core.rs:569-612) of marlin_m1_n8_{plain,silu,argmax} (kernels/marlin.cuh:588-602) for m <= 16 rows and of
 * marlin_m{1..4}_n16_* (the prompt chunks' products, kernels/qwen.cu:48) beyond: more than 16 contiguous rows with the
 * plain or SwiGLU epilogue run on the tensor-core product (tcgen05), gathered rows and the argmax epilogue as 16-row
 * slabs of the first.
 *   X      f16 [.][k]; rows row0 .. row0+m-1 are read, or rows xrows[0..m) when xrows != NULL (this folds
 *          marlin_gather, kernels/marlin.cuh:605-608, into the product)
 *   B      Marlin words, k/16 x 2n u32 (src/cuda/core.rs:262-311 pack_marlin); S f16 [k/128][n] permuted scales
 *   Y      plain/argmax: f32 [.][n]; silu: f16 [.][n/2]; rows row0 .. (xrows: rows 0..m-1)
 *   keys   argmax: u64 [.], maximised with (ordered(logit) << 32 | ~index) over outputs < n_valid
 * n a multiple of 256 and k of 128 as the reference requires (src/cuda/core.rs:160-164). Plain products are
 * complete (one part), as Marlin's. */
int qb_marlin_gemm(qb_ctx* ctx, void* stream, const void* X, const void* B, void* Y, const void* S, int m, int n,
                   int k, int row0, int epi, const int* xrows, unsigned long long* keys, int n_valid);

/* A hint for the next products of up to 16 rows on this context: how many stages of their weights (36 KB per block
 * each) they may request before they wait for the kernel enqueued before them (programmatic dependent launch). 1, the
 * default, suits a product behind another large kernel; 2 a product behind a small one (a norm), whose wait would
 * otherwise leave the memory idle; a product's ring has three stages and 3 is slower than 1. Stays until changed. The
 * reference has no counterpart (its products start when the kernel before them has ended). */
int qb_marlin_early(qb_ctx* ctx, int stages);

/* The zero-point variants marlin_*_z (kernels/marlin.cuh:126-133,588-594): same arguments; S holds the scales followed
 * by the table (8 - z) * scale (qb_pack_marlin_z). w = (q - 8) * scale + (8 - z) * scale; the second term needs only
 * the group's sum of x, which the kernel has anyway. More than 16 rows run as 16-row slabs. */
int qb_marlin_gemm_z(qb_ctx* ctx, void* stream, const void* X, const void* B, void* Y, const void* S, int m, int n,
                     int k, int row0, int epi, const int* xrows, unsigned long long* keys, int n_valid);

/* qb_marlin_gemm without a context and without any allocation, for callers that cannot call cudaMalloc (an engine
 * that gave all free device memory to its cache pool, a plugin in a process whose allocator it does not own). It has
 * no counterpart in the reference. Same arguments and results as qb_marlin_gemm for m <= 16 rows, always through the
 * stream-K path, whose scratch (split-K partials, tickets, error word) lives in a fixed array inside the library image:
 * each GPU that loads the library holds qb_static_scratch_bytes() (about 16 MiB) until exit. Limits: n <= 262144 and
 * n/64 x sharers x 2 KiB (4 KiB above 8 rows) <= 16 MiB, where sharers is the most blocks of the persistent grid that
 * meet in one column block. On a 148-SM part that admits every layer product of the 27B model at 1..16 rows
 * (16384 / 14336 x 5120, 5120 x 6144, 34816 x 5120, 5120 x 17408, 5120 x 10240) and output layers of up to 262144 rows
 * at 1..8 rows; an output layer of more than 131072 rows at 9..16 rows does not fit. Larger sizes return
 * QB_ERR_TOO_LARGE before anything is enqueued. The first call on a device resolves the array's device address and the
 * SM count for that device, and the first call of each tile shape, row-count class (1..8, 9..16) and epilogue sets
 * that kernel's attributes: make one call of every shape you will use before any stream capture, with the device
 * current. Calls on one device share the array, so two of them must not overlap on the GPU (same stream, or ordered
 * by events). A bounded wait that ran out inside such a product is reported by qb_static_device_error (current
 * device; reads and clears; waits). */
int qb_marlin_gemm_noalloc(void* stream, const void* X, const void* B, void* Y, const void* S, int m, int n, int k,
                           int row0, int epi, const int* xrows, unsigned long long* keys, int n_valid);
int qb_static_scratch_bytes(void);
int qb_static_device_error(void);

/* ---- dense f16 skinny product (the 16-bit matrices of a pre-quantized checkpoint: in_proj_b / in_proj_a).
 * Replaces gemm_f16_t{8,16,32}_plain (kernels/gemm.cuh:306-326) as Gemm::run_split launches it
 * (src/cuda/core.rs:532-560): W in mma A-fragment order (qb_pack_f16), X f16 [.][K] (rows xrows[t] if given),
 * Y f32 [K/kper splits][n][ldy] partial products which the consumer sums (any n: blocks of 32 tokens). */
int qb_gemm_f16_plain(qb_ctx* ctx, void* stream, const void* W, const void* X, const int* xrows, int K, int ntiles,
                      int n, int kper, float* Y, int ldy);
/* The dense products of checkpoints that are not int4 (gemm_{f16,i8}_t*_{plain,silu,argmax}, kernels/gemm.cuh:118-304;
 * Gemm::run_split, src/cuda/core.rs:532-560): W in the reference's tile form, wbits 16 (qb_pack_f16, S NULL) or 8
 * (qb_pack_i8: codes q + 128 and f32 scales [tile][K / 128][16 rows]); epi as qb_marlin_gemm. Plain: Y f32
 * [K / kper splits][n][ldy] partial sums; SwiGLU: Y f16 [n][ldy] (ldy >= ntiles * 8); argmax: Y f32 [n][ldy] + keys;
 * the last two need kper == K. qb_pack_i8: Mat::new with int8 (pack, src/cuda/core.rs:337-372): host f32
 * [rows][cols] -> codes [n / 16 tiles][16 * cols] and scales, rows taken in h_order (NULL: as they are). */
int qb_gemm_dec(qb_ctx* ctx, void* stream, const void* W, const float* S, int wbits, const void* X, const int* xrows,
                int K, int ntiles, int n, int kper, int epi, void* Y, int ldy, unsigned long long* keys);
int qb_pack_i8(const float* h_w, int rows, int cols, const int* h_order, int n, uint8_t* h_out, float* h_scales);

/* ---- per-token kernels. n = tokens of the step (grid size in the reference's launches).
 * qb_embed        embed, kernels/dense.cuh:6-11 (src/cuda/qwen/mod.rs:612-621): out f32 [n][5120] = E bf16 rows;
 *                 clears keys[0..nkeys)
 * qb_rmsnorm      rmsnorm, kernels/dense.cuh:14-26: y f16 = w * x / rms(x)
 * qb_add_rmsnorm  add_rmsnorm, kernels/qwen.cu:57-80: h += sum of x [splits][n][5120]; y f16 = w_next * h / rms(h)
 * qb_to_xin       to_xin, kernels/qwen.cu:136-138
 * qb_sum_parts    sum_parts, kernels/qwen.cu:141-143
 * qb_mark_seen    mark_seen, kernels/sampling.cuh:14-26 (src/cuda/core.rs:949-960); vocab = bits per slot
 * qb_marlin_gather marlin_gather, kernels/marlin.cuh:605-608 (qb_marlin_gemm's xrows makes it unnecessary) */
/* mtp_in (kernels/qwen.cu:100-133): fc's input of an MTP step, y f16 [n][10240] = [pre_e * e / rms(e); pre_h * g /
 * rms(g)], e = emb[t], g = fw * h[rows[t]] / rms(h[rows[t]]).
 * qb_draft_pick: the greedy row of draft_sample (kernels/sampling.cuh:298 with argmax_draft_row, src/sample.rs:58-62):
 * the draft of logit row i is the index in keys[i] (the argmax epilogue's), mapped through head_ids when a draft head
 * made the logits; written to next_ids[i] and chain[i * chain_ld + t]. */
int qb_mtp_in(qb_ctx* ctx, void* stream, const float* emb, const float* h, const int* rows, const float* fw,
              const float* pre_e, const float* pre_h, void* y, float eps, int n);
int qb_draft_pick(qb_ctx* ctx, void* stream, const unsigned long long* keys, const int* head_ids, int n_out,
                  int* next_ids, int* chain, int chain_ld, int t);
/* ---- a LoRA adapter applied unmerged (kernels/lora.cuh, src/cuda/qwen/lora.rs:160-207).
 * xa f32 [split][n][M]: the partial sums of the stacked A's product with the step's input (qb_gemm_f16_plain on A
 * packed by qb_pack_f16; M = adapted modules * rank padded to 16, at most 256). B f16 [rows][rank] in the product's row
 * order; tab int[8]: the ends of the stacked modules' rows (3, ascending, unused INT_MAX), one unused, then each
 * module's first column of xa (-1: not adapted). slot_scale f32 [slots]: alpha / r for slots that use the adapter, else
 * 0 (their tokens get exactly the base model's values). rank 8, 16, 32 or 64.
 * qb_lora_add   lora_add_r*: y (a plain product's first partial sums, f32 [n][ldy]) += s * B . xa
 * qb_lora_silu  lora_silu_r*: mid f16 [n][rows / 2] = SwiGLU of the plain [gate; up] product y (the SwiGLU epilogue's
 *               row order) with the delta added first, as the epilogue rounds it */
int qb_lora_add(qb_ctx* ctx, void* stream, const float* xa, int split, int M, const void* B, int rows, const int* tab,
                const int* tok_slot, const float* slot_scale, int n, float* y, int ldy, int rank);
int qb_lora_silu(qb_ctx* ctx, void* stream, const float* xa, int split, int M, const void* B, int rows, const int* tab,
                 const int* tok_slot, const float* slot_scale, int n, const float* y, int ldy, void* mid, int rank);

/* ---- the GPU sampler (kernels/sampling.cuh; host definition src/sample.rs:88-211).
 * QB_QD, QB_QCAP: drafts per chain and kept tokens per stored draft distribution (QD, QCAP, kernels/sampling.cuh:73-74).
 * qb_sample_rows   sample_rows, kernels/sampling.cuh:188-291 (Step::sample, src/cuda/core.rs:977-1005): one token per
 *                  logit row (`width` logits, rows ld floats apart; the reference's VOCAB is all three of width, ld
 *                  and vocab) in vLLM's order (repetition penalty over seen + the step's tokens of the
 *                  row's sequence, presence penalty over outs + those tokens, temperature, top-k, top-p), drawn with
 *                  the host's uniform numbers; params f32 [n_out][8] = temperature, top_k, top_p, repetition penalty,
 *                  u1, u2, draft (-1: none; d <= -2: the draft -d - 2 drawn by qb_draft_sample), presence penalty.
 *                  out_tok[row] = token, out_acc[row] = draft accepted, or -1: the row needs more candidates than
 *                  QB_QCAP and is the host's, as in the reference (top_k above QB_QCAP; top_k 0 without a top-p cut).
 *                  A top_k 0 row WITH a top-p cut is made here when the cut falls among the QB_QCAP most likely tokens
 *                  (the mass of the whole vocabulary is summed on the device), and comes back -1 only otherwise: the
 *                  reference sends every such row to the host, a full sort of the vocabulary per row. seen / outs: vocab / 32 words
 *                  per slot. Tokens are those of the reference kernel, draw for draw.
 * qb_draft_sample  draft_sample, kernels/sampling.cuh:298-352 (Step::draft_sample, src/cuda/core.rs:1036-1073): a
 *                  draft per row of a draft step from its `width` logits (rows ld apart; column i is token
 *                  head_ids[i], or i when head_ids is null) under the row's sampling, u = params[4], t = params[5] the
 *                  draft's index in its chain; drafts[row] = token, and q (qtok, qn, qid ascending, qp) is stored for
 *                  (slot, t).
 * qb_host_sample_row  sample::sample_row / sample_row_q (src/sample.rs:141-200) as Step::sample_on_host calls them
 *                  (src/cuda/core.rs:1007-1032) for the rows qb_sample_rows marks -1. HOST pointers: the row's n
 *                  logits, the slot's two sets (n / 32 words or more; null: empty), the step's tokens of the row's
 *                  sequence after its first up to the row's own, the row's eight parameters, and, for a row whose draft
 *                  is marked sampled, the stored q (ascending ids; nq 0: none, the draft counts as an argmax's). */
#define QB_QD 16
#define QB_QCAP 1024
int qb_sample_rows(qb_ctx* ctx, void* stream, const float* logits, int width, int ld, int vocab, int n_out,
                   const int* out_rows, const int* tok_slot, const int* ids, const int* row_first,
                   const unsigned* seen, const unsigned* outs, const float* params, const int* qtok, const int* qn,
                   const int* qid, const float* qp, int* out_tok, int* out_acc);
int qb_host_sample_row(const float* logits, int n, const unsigned* seen, const unsigned* outs, const int* step,
                       int nstep, const float* row, const int* q_ids, const float* q_p, int nq, int* tok, int* acc);
int qb_draft_sample(qb_ctx* ctx, void* stream, const float* logits, int width, int ld, const int* head_ids, int vocab,
                    int n_out, const int* out_rows, const int* tok_slot, const unsigned* seen, const unsigned* outs,
                    const float* params, int* drafts, int* qtok, int* qn, int* qid, float* qp);
int qb_embed(qb_ctx* ctx, void* stream, const void* E, const int* ids, float* out, unsigned long long* keys,
             int nkeys, int n);
/* embed_q8, kernels/qwen.cu:85-98: the same lookup from an int8 table as stored (codes + 128, a f32 scale per 128
 * columns, S [rows][5120 / 128]); the table may be mapped host memory. */
int qb_embed_q8(qb_ctx* ctx, void* stream, const void* E, const float* S, const int* ids, float* out,
                unsigned long long* keys, int nkeys, int n);
int qb_rmsnorm(qb_ctx* ctx, void* stream, const float* x, const float* w, void* y, float eps, int n);
int qb_add_rmsnorm(qb_ctx* ctx, void* stream, float* h, const float* x, int splits, int n, const float* w_next,
                   void* y, float eps);
int qb_to_xin(qb_ctx* ctx, void* stream, const float* x, void* y, int len);
int qb_sum_parts(qb_ctx* ctx, void* stream, const float* x, int splits, int n, int ld, float* y);
int qb_mark_seen(qb_ctx* ctx, void* stream, unsigned* seen, const int* mark, const int* mark_at, const int* seg_slot,
                 const int* seg_pos0, int segs, int vocab);
int qb_marlin_gather(qb_ctx* ctx, void* stream, const void* x, const int* rows, void* out, int k8, int n);

/* ---- gated attention over the int8 KV cache.
 * qb_attn_prep    attn_prep + kv_store, kernels/qwen.cu:156-202, kernels/attn.cuh:50-64 (launched by Attn::run,
 *                 src/cuda/qwen/attn.rs:285-302). Cache layout and quantisation are the reference's: K rows of 256
 *                 bytes in kslot order, V in 16-position blocks in vslot order, byte = code + 128, f32 scale per
 *                 (slot, kv head, position); cap a multiple of 64.
 * qb_attn_decode  attn_mq{1,2,3} + attn_combine (+ to_xin when mix_f16 != NULL), kernels/attn.cuh:77-325 as
 *                 Attn::run launches them (src/cuda/qwen/attn.rs:303-336,370-375). `out` holds the gate on entry and
 *                 the gated attention output on return. part_ml / part_acc: scratch for ndec * 24 * 64 (m, l) pairs
 *                 and accumulators of 256 floats. The split size is a function of the key count alone
 *                 and of the context's SM count alone (qb_attn_dec_splits_sm: at most one block per SM over the four kv
 *                 heads, 64 at most), as the reference's dchunk is of the key count (kernels/attn.cuh:41-46).
 *                 qb_attn_dec_splits is the same for a 148-SM part. With at most 64 decode tokens in the call
 *                 (ndec) the kernel reads the token lists (dseg, dtok, tok_slot, tok_pos) and the cache entries that
 *                 lie 64 positions or more before a segment's last key AHEAD of the kernel enqueued before it on the
 *                 stream (programmatic dependent launch): those must be complete by then, which holds when the lists
 *                 are uploaded before the step's kernels and such cache entries were written by earlier steps, as in
 *                 the reference's host. Everything else (q, the gate, the step's own keys and values) waits. */
int qb_attn_prep(qb_ctx* ctx, void* stream, const float* part, int splits, int n, const float* q_norm,
                 const float* k_norm, const float* inv_freq, float qscale, float* q, float* out, void* kc, void* vc,
                 float* ks, float* vs, const int* tok_slot, const int* tok_pos, int cap);
int qb_attn_decode(qb_ctx* ctx, void* stream, const float* q, const void* kc, const void* vc, const float* ks,
                   const float* vs, const int* dseg, const int* dtok, const int* dkeys, const int* tok_slot,
                   const int* tok_pos, int cap, int ndseg, int ndec, int dmax, int max_keys, float* part_ml,
                   float* part_acc, float* out, void* mix_f16);
int qb_attn_dec_splits(int keys);
int qb_attn_dec_splits_sm(int keys, int sms);
/* qb_attn_prefill  attn_prefill + attn_combine_tiles (+ to_xin when mix_f16 != NULL), kernels/attn.cuh:327-349,351-520,
 *                  as Attn::run launches them (src/cuda/qwen/attn.rs:338-368): ntile tiles (ptile: first token,
 *                  count; at most 64 / 6 = 10 consecutive tokens of one segment each), max_keys = tile_max_pos + 1.
 *                  The key splits are the library's (qb_attn_tile_splits, one value per step like the reference's
 *                  Attn::tile_splits, attn.rs:268-274); part_ml / part_acc hold n * 24 * splits partials, n = the
 *                  step's tokens. */
int qb_attn_prefill(qb_ctx* ctx, void* stream, const float* q, const void* kc, const void* vc, const float* ks,
                    const float* vs, const int* ptile, const int* tok_slot, const int* tok_pos, int cap, int ntile,
                    int max_keys, float* part_ml, float* part_acc, float* out, void* mix_f16);
int qb_attn_tile_splits(int ntile, int max_keys);

/* ---- Gated DeltaNet. Slot memory (sst floats per slot), metadata and the rollback plan are the reference's
 * (kernels/qwen_deltanet.cuh:12-82; host side src/cuda/qwen/deltanet.rs:83-104,181-226).
 * qb_delta_conv   delta_conv, kernels/qwen_deltanet.cuh:84-131
 * qb_delta_rule   delta_rule, kernels/qwen_deltanet.cuh:172-288
 * qb_delta_norm   delta_norm, kernels/qwen_deltanet.cuh:295-315
 * launched in this order by DeltaNet::run (src/cuda/qwen/deltanet.rs:109-160). */
int qb_delta_conv(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* ba, int ba_splits,
                  const float* cw, const float* a_log, const float* dt_bias, const float* mem, long long sst,
                  float* cv, const int* tok_slot, const int* tok_pos);
int qb_delta_rule(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* cv, float* mem,
                  long long sst, const int* meta, float* out, const int* seg_start, const int* seg_len,
                  const int* seg_slot, const int* seg_pos0, int segs);
int qb_delta_norm(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* nw, const float* out,
                  void* y, int* meta, const int* seg_len, const int* seg_slot, const int* seg_pos0, int segs);

/* The three DeltaNet kernels of a step in one launch (same arguments; `out`, the raw output before the gated norm,
 * may be NULL). Same arithmetic as qb_delta_conv + qb_delta_rule + qb_delta_norm (values agree to an f32 ulp); steps
 * of up to 29 tokens (QB_ERR_UNSUPPORTED beyond: use the three calls). The reference has no fused
 * counterpart; DeltaNet::run (src/cuda/qwen/deltanet.rs:109-160) would call this once instead of its three launches. */
int qb_delta_mixer(qb_ctx* ctx, void* stream, const float* p, int splits, int n, const float* ba, int ba_splits,
                   const float* cw, const float* a_log, const float* dt_bias, const float* nw, float* mem,
                   long long sst, int* meta, float* out, void* y, const int* seg_start, const int* seg_len,
                   const int* seg_slot, const int* seg_pos0, int segs);

/* ---- the step: the host side of Model::step for this path (src/cuda/qwen/mod.rs:1125-1143).
 * A model is the layer stack's device pointers (owned by the caller, valid for the model's life, at fixed addresses
 * as the reference's regions are: src/cuda/vmm.rs:1-4) plus the step buffers allocated by qb_model_create
 * (Bufs and Step of the reference: src/cuda/qwen/mod.rs:286-305, src/cuda/core.rs:699-760). */
typedef struct qb_model qb_model;
enum { QB_LAYER_DELTA = 0, QB_LAYER_ATTN = 1 };

/* One layer (Layer + Mixer, src/cuda/qwen/mod.rs:178-196): Marlin matrices as (words, scales) pairs, norms pre-biased
 * 1 + w, then the mixer's own tensors and per-slot caches. */
typedef struct qb_layer {
    int kind;                               /* QB_LAYER_DELTA | QB_LAYER_ATTN */
    const void *in_proj_w, *in_proj_s;      /* [in_proj_qkv; in_proj_z] 16384 x 5120 | [q; k; v] 14336 x 5120 */
    const void* in_ba;                      /* DeltaNet: [in_proj_b; in_proj_a] 96 x 5120, f16 fragment order */
    const void *out_w, *out_s;              /* out_proj | o_proj, 5120 x 6144 */
    const float *input_norm, *post_norm;
    const void *gate_up_w, *gate_up_s;      /* [gate; up] 34816 x 5120, row_order(silu) */
    const void *down_w, *down_s;            /* 5120 x 17408 */
    /* DeltaNet (src/cuda/qwen/deltanet.rs:50-70) */
    const float *conv_w, *a_log, *dt_bias, *norm_w;
    float* mem;                             /* slots x sst floats: states, banks, ring */
    long long sst;
    int* meta;                              /* slots x 4: end (-1: none), ck, ebuf, _ */
    /* attention (src/cuda/qwen/attn.rs:96-111) */
    const float *q_norm, *k_norm, *inv_freq;
    void *kc, *vc;                          /* int8 [slot][4][cap][256] */
    float *ks, *vs;                         /* f32 [slot][4][cap] */
    int cap;
} qb_layer;

/* The MTP draft layer (Mtp, src/cuda/qwen/mod.rs:648-661) */
#define QB_MAX_DRAFTS 8
typedef struct qb_mtp {
    qb_layer layer;                  /* its decoder layer (own KV cache / state) */
    const void *fc_w, *fc_s;         /* fc 5120 x 10240, Marlin */
    const float *pre_e, *pre_h;      /* the norms of fc's two inputs, f32 [5120] (1 + w) */
    const float* norm;               /* the MTP's final norm, f32 [5120] */
    const void *head_w, *head_s;     /* draft head: head_rows x 5120 Marlin rows of the output layer, or NULL (the
                                        whole output layer drafts) (src/cuda/qwen/draft.rs) */
    int head_rows, head_valid;
    const int* head_ids;             /* device: the token of each draft-head row */
    int head_zero_points;            /* non-zero: head_s holds the (8 - z) * scale table too (Mat::marlin_rows with zeros) */
} qb_mtp;

/* A layer's LoRA (LayerLora, src/cuda/qwen/lora.rs:199-205): per stacked product its A (shared by the products that
 * read the same input) and B. a == NULL: the product is not adapted. */
typedef struct qb_lora_prod {
    const void* a;       /* stacked A, qb_pack_f16 of f16 [a_tiles * 16][cols] (modules * rank rows, padded to 16) */
    int a_tiles;
    const void* b;       /* B f16 [rows][rank] in the product's row order (SwiGLU: row_order), or NULL */
    const int* tab;      /* device int[8], see qb_lora_add */
    const void* b2;      /* DeltaNet in-projection only: B of [in_proj_b; in_proj_a] (96 rows) on the same xa, or NULL */
    const int* tab2;
} qb_lora_prod;
typedef struct qb_lora_layer {
    int rank;            /* 8, 16, 32 or 64 */
    qb_lora_prod inp, out, gate_up, down;
} qb_lora_layer;

/* ---- device memory mapped on demand (src/cuda/vmm.rs): Pool (:16-128) and Region (:171-289). A region reserves device
 * addresses once (kernels and graphs see fixed pointers) and maps 2 MiB pages from the pool where data lives; the pool
 * makes pages within a budget and reuses unmapped ones. Errors of the driver come back as 2000 + CUresult.
 * qb_region_map: *ok = 0 when the pool has too few pages (nothing more is mapped); new pages are zeroed on `stream`.
 * qb_region_unmap: the pages wholly inside [from, to), after the stream's work. qb_region_read / write refuse ranges that
 * are not mapped (QB_ERR_ARG). Kernels must only be given mapped ranges: an access to an unmapped page is a GPU fault. */
typedef struct qb_pool qb_pool;
typedef struct qb_region qb_region;
int qb_pool_create(int device, qb_pool** out);
void qb_pool_destroy(qb_pool* p);
size_t qb_pool_page(const qb_pool* p);
int qb_pool_set_budget(qb_pool* p, size_t pages);
int qb_pool_fill(qb_pool* p);
int qb_pool_release(qb_pool* p, size_t n, size_t* given);
int qb_pool_usage(qb_pool* p, size_t* used, size_t* budget);
size_t qb_pool_available(qb_pool* p);
int qb_region_reserve(qb_pool* p, size_t size, qb_region** out);
void* qb_region_ptr(const qb_region* r);
size_t qb_region_size(const qb_region* r);
int qb_region_is_mapped(const qb_region* r, size_t from, size_t to);
int qb_region_map(qb_region* r, void* stream, size_t from, size_t to, int* ok);
int qb_region_unmap(qb_region* r, void* stream, size_t from, size_t to);
int qb_region_read(qb_region* r, void* stream, size_t from, void* out, size_t n);
int qb_region_write(qb_region* r, void* stream, size_t from, const void* data, size_t n);
int qb_region_free(qb_region* r, void* stream);

/* A token of a step (Tok, src/engine.rs:90-95) */
typedef struct qb_tok {
    uint32_t id, slot, pos;
} qb_tok;

int qb_model_create(qb_ctx* ctx, int nlayers, int slots, int max_ctx, int vocab_rows, int vocab_valid,
                    qb_model** out);
void qb_model_destroy(qb_model* m);
int qb_model_set_layer(qb_model* m, int i, const qb_layer* l);
/* embedding bf16 [vocab][5120], final norm (1 + w), lm_head as a Marlin matrix of vocab_rows rows of which the first
 * vocab_valid count (Mat::marlin_rows, src/cuda/core.rs:137-152) */
int qb_model_set_head(qb_model* m, const void* embed_bf16, const float* final_norm, const void* lm_w,
                      const void* lm_s);
/* Model::step = Step::upload (src/cuda/core.rs:835-926) + Graphs::run (:1151-1192) of launch_step
 * (src/cuda/qwen/mod.rs:744-766). h_toks, h_out: host arrays; sequences contiguous and in order; errors as the
 * reference's ensure!s (QB_ERR_ARG). Steps of up to 32 tokens are captured once per shape and replayed as a CUDA
 * graph; larger ones (prompt chunks of up to 2048 tokens, any mix of segments) launch their kernels directly. */
int qb_model_step(qb_model* m, void* stream, const qb_tok* h_toks, int n, const int* h_out, int n_out);
int qb_model_upload(qb_model* m, void* stream, const qb_tok* h_toks, int n, const int* h_out, int n_out);
/* Model::step with `marks` (src/cuda/qwen/mod.rs:1125-1143, Step::upload's third argument, src/cuda/core.rs:872-880):
 * segment s of the step adds h_marks[h_marks_at[s] .. h_marks_at[s + 1]] to its slot's seen set instead of its own
 * tokens (a verify step marks the history committed since the slot's last step, not its drafts). h_marks_at holds one
 * entry more than the step has segments; at most 2560 marks per step. A step that is refused (QB_ERR_ARG) leaves the
 * state of the step before it in place. */
int qb_model_step_marks(qb_model* m, void* stream, const qb_tok* h_toks, int n, const int* h_out, int n_out,
                        const uint32_t* h_marks, const int* h_marks_at);
int qb_model_upload_marks(qb_model* m, void* stream, const qb_tok* h_toks, int n, const int* h_out, int n_out,
                          const uint32_t* h_marks, const int* h_marks_at);
/* The step's host arrays alone (Step::upload without the copies; no device, no model): h_arrays takes
 * qb_step_ints() ints, of which array i starts at offsets[i], i = ids, tok_slot, tok_pos, seg_start, seg_len,
 * seg_slot, seg_pos0, dtok, dseg, dkeys, ptile, out_rows, mark, mark_at, mtp_rows, row_first (16 offsets); shape
 * takes n, n_out, segs, ndec, ntile, ndseg, dmax, max_seg, dec_max_pos, tile_max_pos (10 ints: Step's counts,
 * src/cuda/core.rs:700-727). h_marks / h_marks_at may both be null (every token of a segment is marked). */
int qb_step_arrays(const qb_tok* h_toks, int n, const int* h_out, int n_out, const uint32_t* h_marks,
                   const int* h_marks_at, int slots, int max_ctx, int vocab_valid, int* h_arrays, long long* offsets,
                   int* shape);
int qb_step_ints(void);
/* The MTP draft step (what turns steps/s into accepted tok/s). qb_model_set_mtp: Mtp::load's
 * pointers. qb_model_draft: Engine::draft with greedy rows = draft_chains (src/cuda/qwen/mod.rs:870-896): k <=
 * QB_MAX_DRAFTS drafts for each row of h_out, from the hidden states the last qb_model_step left at h_rows; h_drafts
 * host [n_out][k]. */
int qb_model_set_mtp(qb_model* m, const qb_mtp* mtp);
int qb_model_draft(qb_model* m, void* stream, const qb_tok* h_toks, int n, const int* h_rows, const int* h_out,
                   int n_out, int k, int* h_drafts);
int qb_model_learn_block(qb_model* m, void* stream, int block, const uint32_t* h_words, const uint16_t* h_sc,
                         const int* h_ids16, int* grew);
/* The sampler on the step's logits.
 * qb_model_set_outputs   Step::set_outputs: the tokens a slot's request generated so far, h_words = vocab_rows / 32
 *                        host words (the presence penalty's set; the seen set is kept by the steps themselves).
 * qb_model_sample        Step::sample (src/cuda/core.rs:977-1005): a token per logit row of the last step under
 *                        h_params [n_out][8] (see qb_sample_rows), on the device; rows with top_k 0 or above QB_QCAP
 *                        on the host from the same state (Step::sample_on_host, :1007-1032 = qb_host_sample_row).
 *                        h_tok / h_acc host [n_out]; waits for the step.
 * qb_model_draft_sampled Engine::draft with sampled rows (draft_chains + launch_drafts, src/cuda/qwen/mod.rs:866-918):
 *                        qb_model_draft whose drafts are drawn on the device by qb_draft_sample under h_sampling
 *                        [n_out][8] (Params::draft_row; temperature <= 0: the argmax row) with the draws h_u
 *                        [n_out][k]; each draft's distribution is kept for (slot, t).
 * qb_model_draft_q       Step::draft_q (src/cuda/core.rs:1088-1098): that distribution (ids ascending, host [QB_QCAP]
 *                        each) and the token drawn from it. */
int qb_model_set_outputs(qb_model* m, void* stream, int slot, const unsigned* h_words);
int qb_model_sample(qb_model* m, void* stream, const float* h_params, int n_out, int* h_tok, int* h_acc);
int qb_model_draft_sampled(qb_model* m, void* stream, const qb_tok* h_toks, int n, const int* h_rows, const int* h_out,
                           int n_out, int k, const float* h_sampling, const float* h_u, int* h_drafts);
int qb_model_draft_q(qb_model* m, void* stream, int slot, int t, int* tok, int* n, int* h_ids, float* h_p);
/* A slot's saved images, byte for byte the reference's:
 * qb_model_kv_bytes / save_kv / load_kv      Model::save_kv / load_kv (src/cuda/qwen/mod.rs:1031-1061): per attention
 *     layer (the MTP's last) and kv head the keys of positions [from, to), the values in blocks of 16 positions, the
 *     two scale rows (Attn::layout, src/cuda/qwen/attn.rs:182-196); from a multiple of 16.
 * qb_model_state_bytes / save_state / load_state  Model::save_state / load_state (:993-1029): per DeltaNet layer the end
 *     state and the conv ring's last three positions (DeltaNet::save / load, src/cuda/qwen/deltanet.rs:181-226), then
 *     the slot's seen set; *pos = the position the state is at; a loaded slot continues at `pos`.
 * One gather (scatter) kernel over all layers and one copy per call; h_* are host buffers; the calls wait. */
size_t qb_model_kv_bytes(const qb_model* m, int from, int to);
int qb_model_save_kv(qb_model* m, void* stream, int slot, int from, int to, void* h_out, size_t bytes);
int qb_model_load_kv(qb_model* m, void* stream, int slot, int from, int to, const void* h_data, size_t bytes);
size_t qb_model_state_bytes(const qb_model* m);
int qb_model_save_state(qb_model* m, void* stream, int slot, void* h_out, size_t bytes, int* pos);
int qb_model_load_state(qb_model* m, void* stream, int slot, const void* h_data, size_t bytes, int pos);
/* A LoRA adapter served unmerged (Model::set_adapter, Step::lora; src/cuda/qwen/lora.rs, mod.rs:505-575):
 * qb_model_set_adapter   layer i's LoRA (NULL: none; the MTP layer is not adapted).
 * qb_model_set_slot_scale  alpha / r for a slot whose request uses the adapter, 0 for one that does not. Steps without
 *                        tokens of adapter slots run exactly the base model's kernels; in the others every adapted
 *                        product is followed by xa = A x and qb_lora_add ([gate; up]: a plain product and qb_lora_silu). */
int qb_model_set_adapter(qb_model* m, int layer, const qb_lora_layer* lora);
int qb_model_set_slot_scale(qb_model* m, void* stream, int slot, float scale);
int qb_model_run(qb_model* m, void* stream);
/* The captured steps are a bounded cache (Graphs, src/cuda/core.rs:1105-1252): once less than 128 MiB of device memory
 * is free at a capture the cache keeps what it holds and drops the least recently used; a capture that finds no memory
 * lowers the cap to three quarters and its step runs without a graph. qb_model_set_pool names the cache pool whose free
 * pages go back to the driver when memory is shorter still (NULL: none). Setting a layer, the head, the MTP layer or an
 * adapter drops every captured step (they hold the old pointers). */
int qb_model_use_graphs(qb_model* m, int on);
int qb_model_set_pool(qb_model* m, qb_pool* pool);
int qb_model_graph_stats(const qb_model* m, long long* held, long long* cap, long long* graphless);
/* 1 (default): fused launches where the library has them (qb_delta_mixer); 0: one launch per reference kernel */
int qb_model_use_fused(qb_model* m, int on);
/* on (default): the DeltaNet layers' 16-bit in-projection runs on a second stream beside the int4 one */
int qb_model_use_fork(qb_model* m, int on);
/* Engine::argmax (src/cuda/core.rs:1100-1103): greedy token per logit row of the last step; synchronises the stream */
int qb_model_argmax(qb_model* m, void* stream, int* h_tokens, int n_out);
float* qb_model_logits(qb_model* m);   /* device f32 [n_out][vocab_rows] */
float* qb_model_hidden(qb_model* m);   /* device f32 [n][5120], the residual stream after the last layer */
void* qb_model_xn(qb_model* m);        /* device f16 [n][5120], the final norm's output */
unsigned* qb_model_seen(qb_model* m);  /* device [slots][vocab_rows / 32]: the slots' seen sets (Step::seen) */
long long qb_model_launches(const qb_model* m);  /* kernels launched or replayed so far */
int qb_model_step_kernels(const qb_model* m);    /* kernels of one step of the last shape */

/* ---- host-side weight packers (load time; host pointers). They produce the layouts the reference's loader
 * produces, which every kernel here reads unchanged.
 * qb_row_order    row_order, src/cuda/core.rs:106-114
 * qb_pack_marlin  pack_marlin + marlin_word + marlin_scale (symmetric), src/cuda/core.rs:244-311; h_q is the
 *                 stored matrix as Quant holds it (src/checkpoint.rs:20-31): u32 [rows][cols/8], q + 8 in nibbles
 * qb_pack_f16     pack (f16 branch) + frag, src/cuda/core.rs:222-227,337-391
 * qb_split_for    split_for, src/cuda/core.rs:393-398 (0 for an argument that is not positive) */
int qb_row_order(int rows, int silu, int* h_order);
int qb_pack_marlin(const uint32_t* h_q, const float* h_scales, int rows, int cols, int group, const int* h_order,
                   int n, uint32_t* h_words, uint16_t* h_scales_f16);
/* with zero points (marlin_scale with zeros, src/cuda/core.rs:255-260): h_zeros u8 [rows][cols/group]; h_scales_f16 gets
 * 2 * cols/128 rows: the scales, then (8 - z) * scale */
int qb_pack_marlin_z(const uint32_t* h_q, const float* h_scales, const uint8_t* h_zeros, int rows, int cols, int group,
                     const int* h_order, int n, uint32_t* h_words, uint16_t* h_scales_f16);
int qb_pack_f16(const float* h_w, int rows, int cols, const int* h_order, int n, uint16_t* h_out);
/* A draft head learning rows (DraftHead::learn, src/cuda/qwen/draft.rs:56-72; Gemm::put_block, src/cuda/core.rs:614-671).
 * qb_marlin_block      the host half: the 16 stored rows h_rows16 of a quantized matrix (h_q, h_scales, h_zeros as for
 *                      qb_pack_marlin_z; zero_points 0: a symmetric matrix, every stored z must be 8) -> the block's words
 *                      u32 [cols/16][32] and scales f16 [tables * cols/128][16] (tables 2 with zero points)
 * qb_marlin_put_block  marlin_put_block, kernels/marlin.cuh:614-622, its arguments plus the number of k16 steps (the
 *                      reference's grid size): writes the block as rows 16 blk .. of the 64-row group c64 of the Marlin
 *                      matrix (B, S) of n rows; words / sc are DEVICE staging buffers
 * qb_model_learn_block both for the model's draft head (set with qb_model_set_mtp), through staging buffers allocated
 *                      once, plus the block's 16 tokens into head_ids; the head's valid rows grow to cover the block */
int qb_marlin_block(const uint32_t* h_q, const float* h_scales, const uint8_t* h_zeros, int zero_points, int rows,
                    int cols, int group, const int* h_rows16, uint32_t* h_words, uint16_t* h_sc);
int qb_marlin_put_block(qb_ctx* ctx, void* stream, void* B, void* S, const void* words, const void* sc, int n, int c64,
                        int blk, int groups, int tables, int k16s);
int qb_split_for(int tiles, int cols, int bits, int kd);

/* ---- which token has which row of the draft head, and how that changes while a server runs: Rows / Adaptive of
 * src/draft_vocab.rs:22-201 (host only; the head's weights are written by qb_model_learn_block). Every committed token
 * adds 1 to its row's score, the scores halve every 20,000 committed tokens; a token without a row waits until 16 do,
 * which then get a new tile of 16 rows while the head has room (cap) and else the rows of the coldest tokens (score
 * below 1), rewritten in place.
 * qb_draft_vocab_create     Rows::new: `n` rows (a multiple of 16, at most cap, cap a multiple of 16) with their scores
 *                           (null: 0); QB_ERR_ARG for a token twice or beyond the vocabulary
 * qb_draft_vocab_load       Adaptive::load: the rows saved by an earlier run if they fit this vocabulary (else none of
 *                           them), then the seed's tokens that are new while there is room (65,536 rows); whole tiles
 * qb_draft_vocab_get        the token and score of each row (either may be null); cap >= qb_draft_vocab_rows
 * qb_draft_vocab_row_of     a token's row, -1 without one
 * qb_draft_vocab_may_change Rows::may_change: whether these tokens can change a tile
 * qb_draft_vocab_learn      Adaptive::learn: takes in the tokens a step commits; when tiles changed, publish(user, ids,
 *                           n_ids, tiles, n_tiles) is to put them into the head (tiles ascending; the tokens of tile t
 *                           are ids[16 t .. 16 t + 16]); if it returns non-zero the rows are as before and that code is
 *                           returned. *changed (optional): tiles published. publish may be null (bookkeeping only).
 * qb_draft_vocab_dirty / _saved   whether rows changed since the host last saved them (the reference writes them to
 *                           its cache directory at most once a minute; where and when is the host's choice here)
 * qb_draft_ids_pt           draft_ids (:231-268): the token ids in the bytes of a mtp_draft_vocab_ids.pt file (a zip
 *                           archive whose stored entry * /data/0 holds int64 values), repeats dropped; *n = their count
 *                           (QB_ERR_TOO_LARGE when cap is less). 1: not a zip archive or truncated, 2: no tensor data,
 *                           3: the entry is compressed or no whole int64s, 4: a token id beyond the vocabulary
 * qb_model_learn            DraftHead::learn (src/cuda/qwen/draft.rs:55-68): qb_draft_vocab_learn whose publish packs
 *                           every changed tile from the stored output layer (h_q, h_scales, h_zeros, zero_points,
 *                           rows, cols, group as for qb_marlin_block) and writes it with qb_model_learn_block; *grew:
 *                           the head's valid rows grew (the MTP steps' graphs were dropped) */
typedef struct qb_draft_vocab qb_draft_vocab;
typedef int (*qb_publish_fn)(void* user, const uint32_t* ids, int n_ids, const int* tiles, int n_tiles);
int qb_draft_vocab_create(int vocab, const uint32_t* ids, const float* score, int n, int cap, qb_draft_vocab** out);
int qb_draft_vocab_load(int vocab, const uint32_t* saved_ids, const float* saved_score, int n_saved,
                        const uint32_t* seed_ids, int n_seed, qb_draft_vocab** out);
void qb_draft_vocab_destroy(qb_draft_vocab* v);
int qb_draft_vocab_rows(const qb_draft_vocab* v);
int qb_draft_vocab_get(const qb_draft_vocab* v, uint32_t* ids, float* score, int cap);
int qb_draft_vocab_row_of(const qb_draft_vocab* v, uint32_t token);
int qb_draft_vocab_waiting(const qb_draft_vocab* v, uint32_t token);
int qb_draft_vocab_pending(const qb_draft_vocab* v);
int qb_draft_vocab_dirty(const qb_draft_vocab* v);
int qb_draft_vocab_saved(qb_draft_vocab* v);
int qb_draft_vocab_may_change(const qb_draft_vocab* v, const uint32_t* toks, int n);
int qb_draft_vocab_learn(qb_draft_vocab* v, const uint32_t* toks, int n, qb_publish_fn publish, void* user, int* changed);
int qb_draft_ids_pt(const uint8_t* bytes, size_t len, int vocab, uint32_t* ids, int cap, int* n);
int qb_model_learn(qb_model* m, void* stream, qb_draft_vocab* v, const uint32_t* toks, int n, const uint32_t* h_q,
                   const float* h_scales, const uint8_t* h_zeros, int zero_points, int rows, int cols, int group,
                   int* grew);

/* Programmatic dependent launch for the kernels that support it (their weight prefetch then overlaps the tail of
 * the previous kernel of the stream). Off by default. */
int qb_set_pdl(qb_ctx* ctx, int on);

#ifdef __cplusplus
}
#endif
#endif
