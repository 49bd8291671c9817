/*
 * lumen_b200 — C ABI of the B200 (sm_100a) implementation of the Llama inference hot path of
 * chen-197/Lumen.  The reference is pure Rust with no FFI of its own; each entry point below
 * sits directly beneath one Rust function or method of the reference and cites it (paths are
 * relative to the reference crate root).  A Rust shim binds these with an `extern "C"` block
 * and keeps the reference's `Tensor` / `Module` / `LlamaModel` / `KVCache` signatures.
 *
 * Conventions
 *  - Every call returns an int status (LUMEN_OK == 0).  Conditions the reference turns into a
 *    `panic!` are checked on the host before any kernel is launched and come back as a
 *    distinct code; device code never traps.  `lumen_last_error` gives the message.
 *  - The library owns all device memory behind opaque handles; the caller owns the host
 *    buffers it passes.  Handles are released with the matching *_free / *_destroy.
 *  - One host thread and one CUDA stream per context (the reference's Tensor is !Send).
 *    Calls are asynchronous on that stream; calls that fill a host buffer synchronise.
 *  - Plain pointers and sizes only; `size_t` shapes are row-major, outermost first.
 *  - There is no CPU fallback: without a CUDA device every call fails with LUMEN_ERR_CUDA.
 */
#ifndef LUMEN_B200_H
#define LUMEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
#define LUMEN_OK 0
#define LUMEN_ERR_INVALID 1      /* null handle / bad argument */
#define LUMEN_ERR_SHAPE 2        /* matmul shape panics: src/ops/matmul.rs:24-38 */
#define LUMEN_ERR_KV_OVERFLOW 3  /* src/layers/attention/self_attention.rs:144-149, src/kv_cache.rs:34-36 */
#define LUMEN_ERR_ROPE_RANGE 4   /* src/layers/attention/encoding.rs:62-68, :176-181 */
#define LUMEN_ERR_EMBED_RANGE 5  /* src/layers/basic/embedding.rs:55 */
#define LUMEN_ERR_CACHE_COUNT 6  /* src/models/llama.rs:182-188 */
#define LUMEN_ERR_CUDA 7
#define LUMEN_ERR_NCCL 8
#define LUMEN_ERR_TIMEOUT 9      /* a bounded device-side wait gave up */
#define LUMEN_ERR_DTYPE 10
#define LUMEN_ERR_PARAM_NAME 11  /* name not in LlamaModel::named_parameters, src/models/llama.rs:218-279 */
#define LUMEN_ERR_UNSUPPORTED 12
#define LUMEN_ERR_MISSING_PARAM 13 /* forward called before every parameter was set */

typedef enum { LUMEN_F32 = 0, LUMEN_BF16 = 1 } lumen_dtype;

typedef struct lumen_ctx lumen_ctx;
typedef struct lumen_tensor lumen_tensor;
typedef struct lumen_rope lumen_rope;
typedef struct lumen_kv_cache lumen_kv_cache;             /* KVCacheInner */
typedef struct lumen_llama_kv_cache lumen_llama_kv_cache; /* LlamaKVCache */
typedef struct lumen_self_attention lumen_self_attention;
typedef struct lumen_llama lumen_llama;

/* ---- context ------------------------------------------------------------------------------
 * No counterpart in the reference (it has no device or process boundary).  tp_size > 1 makes
 * the context one rank of a tensor-parallel group; nccl_unique_id then points at the 128 bytes
 * produced by lumen_nccl_unique_id on rank 0 and distributed by the caller. */
#define LUMEN_NCCL_ID_BYTES 128
int lumen_nccl_unique_id(void *id_out_128_bytes);
int lumen_ctx_create(int device, int tp_rank, int tp_size, const void *nccl_unique_id, lumen_ctx **out);
int lumen_ctx_destroy(lumen_ctx *ctx);
int lumen_ctx_synchronize(lumen_ctx *ctx);
void *lumen_ctx_stream(lumen_ctx *ctx); /* the context's cudaStream_t, for event timing */
/* Kernels this context has enqueued so far (a CUDA-graph replay counts its kernel nodes). */
uint64_t lumen_ctx_launch_count(const lumen_ctx *ctx);
const char *lumen_last_error(const lumen_ctx *ctx);
const char *lumen_status_string(int status);
int lumen_version(void);

/* ---- Tensor — src/autograd.rs:63-64 (data only; grad/backward are training) ---------------
 * from_host     <- Tensor::from_array_no_grad / from_data_no_grad  (autograd.rs:150-163)
 * shape/ndim    <- data_ref().shape()                              (autograd.rs:82-85)
 * to_host       <- get_raw_data / data()                           (autograd.rs:251-257, :106)
 * set           <- set_raw_data (same element count)               (autograd.rs:259-262)
 * reshape       <- ops::shape::reshape as a view (-1 allowed)      (src/ops/shape.rs:9-49)
 * bf16 tensors hold weights only (src/loader.rs:50-64 upcasts them; here they stay bf16). */
int lumen_tensor_from_host(lumen_ctx *ctx, const float *data, const size_t *shape, int ndim, lumen_tensor **out);
int lumen_tensor_from_host_bf16(lumen_ctx *ctx, const uint16_t *data, const size_t *shape, int ndim, lumen_tensor **out);
int lumen_tensor_empty(lumen_ctx *ctx, const size_t *shape, int ndim, lumen_dtype dtype, lumen_tensor **out);
int lumen_tensor_ndim(const lumen_tensor *t);
int lumen_tensor_shape(const lumen_tensor *t, size_t *shape_out);
size_t lumen_tensor_numel(const lumen_tensor *t);
lumen_dtype lumen_tensor_dtype(const lumen_tensor *t);
void *lumen_tensor_data(const lumen_tensor *t); /* device pointer */
int lumen_tensor_to_host(const lumen_tensor *t, float *out);
int lumen_tensor_set(lumen_tensor *t, const float *data);
int lumen_tensor_reshape(const lumen_tensor *t, const int64_t *shape, int ndim, lumen_tensor **out);
int lumen_tensor_free(lumen_tensor *t);

/* ---- ops ----------------------------------------------------------------------------------
 * Each allocates its result (as the reference's ops do) from the context's stream-ordered pool. */
/* ops::matmul::matmul(a[...,K], w[N,K]) -> [...,N] — src/ops/matmul.rs:10-103.  M == 1 takes the
 * vector-matrix kernel (:42-69), M > 1 the GEMM kernel (:70-92).  w may be f32 or bf16. */
int lumen_matmul(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *w, lumen_tensor **out);
/* Linear::forward — src/layers/basic/linear.rs:33-41 (bias may be NULL). */
int lumen_linear_forward(lumen_ctx *ctx, const lumen_tensor *x, const lumen_tensor *w, const lumen_tensor *bias, lumen_tensor **out);
/* RMSNorm::forward — src/layers/norm/rms_norm.rs:24-62. */
int lumen_rmsnorm(lumen_ctx *ctx, const lumen_tensor *x, const lumen_tensor *weight, float eps, lumen_tensor **out);
/* SiLU::forward — src/layers/activation.rs:139-147. */
int lumen_silu(lumen_ctx *ctx, const lumen_tensor *x, lumen_tensor **out);
/* Tensor * Tensor, Tensor + Tensor — src/ops/arithmetic.rs:105-109, :48-52.  Shapes are equal, or
 * b is a trailing-dimension vector broadcast over a (the Linear bias case). */
int lumen_mul(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *b, lumen_tensor **out);
int lumen_add(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *b, lumen_tensor **out);
/* Embedding::forward — src/layers/basic/embedding.rs:21-57.  ids hold f32 token ids. */
int lumen_embedding(lumen_ctx *ctx, const lumen_tensor *ids, const lumen_tensor *table, lumen_tensor **out);
/* ops::fused::fused_softmax forward — src/ops/fused.rs:17-83.  x[B,H,Q,K]. */
int lumen_fused_softmax(lumen_ctx *ctx, const lumen_tensor *x, float scale, int causal, lumen_tensor **out);

/* Standalone vector-matrix product on raw device pointers, for callers that manage their own
 * buffers (same arithmetic as the M == 1 branch, src/ops/matmul.rs:42-69).  layout_kn == 0: w is
 * [N,K] row-major (the reference's Linear layout, src/layers/basic/linear.rs:8); layout_kn == 1:
 * w is [K,N] row-major.  x and y are f32. */
int lumen_gemv(lumen_ctx *ctx, const float *x_dev, const void *w_dev, lumen_dtype w_dtype, int layout_kn,
               size_t k, size_t n, float *y_dev);

/* lumen_gemv with layout_kn == 1, for callers that must not allocate: the split-K partial sums live in a
 * fixed 8 MiB device array inside the library instead of a buffer obtained and released per call, and the
 * call uses no allocating or freeing routine.  No counterpart in the reference (its tensors are heap
 * arrays, src/autograd.rs:17-27).
 *  - Set-up: the first call for a device resolves the array's address (cudaGetSymbolAddress, which may load
 *    the module); make that call before any stream capture begins.
 *  - Limit: sizes whose partial sums exceed 8 MiB are refused with LUMEN_ERR_UNSUPPORTED (on 148 SMs that is
 *    beyond roughly 800k columns); nothing is truncated.  Use lumen_gemv there.
 *  - Nothing has to be zeroed: each call overwrites every partial sum it later reads.
 *  - The array is one per device: two calls in flight at once on the same device (other streams, other
 *    contexts) race on it; calls on one context's stream are ordered and safe. */
int lumen_gemv_kn_static(lumen_ctx *ctx, const float *x_dev, const void *w_dev, lumen_dtype w_dtype, size_t k,
                         size_t n, float *y_dev);

/* ---- RotaryEmbedding — src/layers/attention/encoding.rs ------------------------------------
 * new      <- RotaryEmbedding::new + precompute_freqs_cis (:17-54); tables are built on the host
 *             with the f32 recipe of :38-51 and uploaded.
 * forward  <- RotaryEmbedding::forward(x[B,H,S,D], offset)   (:56-123) */
int lumen_rope_new(lumen_ctx *ctx, size_t dim, size_t max_seq_len, float theta, lumen_rope **out);
int lumen_rope_forward(lumen_rope *rope, const lumen_tensor *x_bhsd, size_t offset, lumen_tensor **out);
int lumen_rope_free(lumen_rope *rope);

/* ---- KVCacheInner — src/layers/attention/self_attention.rs:24-44 ---------------------------
 * k,v: [B,Hkv,max_seq,D] f32 zero-initialised device slabs + len.  reset() sets len = 0 only. */
int lumen_kv_new(lumen_ctx *ctx, size_t b, size_t h_kv, size_t max_seq, size_t d, lumen_kv_cache **out);
int lumen_kv_reset(lumen_kv_cache *c);
size_t lumen_kv_len(const lumen_kv_cache *c);
int lumen_kv_free(lumen_kv_cache *c);
/* Test/bench access to the public `k`, `v`, `len` fields: whole-slab copies to/from the host. */
int lumen_kv_read(const lumen_kv_cache *c, float *k_out, float *v_out);
int lumen_kv_write(lumen_kv_cache *c, const float *k_in, const float *v_in, size_t len);

/* ---- LlamaKVCache — src/kv_cache.rs:5-59 ---------------------------------------------------
 * new(config) (:14-29) -> [1,Hkv,max_seq,D]; update(k,v,start_pos) (:31-49) copies k,v
 * [1,Hkv,S,D]; get_view(n) (:51-59) returns owned copies of the first n rows. */
int lumen_llama_kv_new(lumen_ctx *ctx, size_t kv_heads, size_t max_seq_len, size_t head_dim, lumen_llama_kv_cache **out);
int lumen_llama_kv_update(lumen_llama_kv_cache *c, const lumen_tensor *k, const lumen_tensor *v, size_t start_pos);
int lumen_llama_kv_get_view(const lumen_llama_kv_cache *c, size_t current_len, lumen_tensor **k_out, lumen_tensor **v_out);
int lumen_llama_kv_free(lumen_llama_kv_cache *c);

/* ---- SelfAttention — src/layers/attention/self_attention.rs:46-127, :299-306 ----------------
 * new          <- SelfAttention::new (:61-93); head_dim = embed_dim / n_head
 * set_weight   <- the pub fields w_q, w_k, w_v, w_o (:47-50); which = 0,1,2,3; [out,in] f32/bf16
 * forward      <- SelfAttention::forward(x[B,S,E], Option<KVCache>) in no-grad mode: S == 1
 *                 decode path (:125-306), S > 1 prefill path (:308-426).  cache == NULL creates
 *                 one (:119-122); *cache_out receives the cache used (owned by the caller when
 *                 it was created here). */
#define LUMEN_W_Q 0
#define LUMEN_W_K 1
#define LUMEN_W_V 2
#define LUMEN_W_O 3
int lumen_self_attention_new(lumen_ctx *ctx, size_t embed_dim, size_t n_head, size_t n_kv_head, size_t max_seq_len,
                             float rope_theta, int causal, lumen_self_attention **out);
int lumen_self_attention_set_weight(lumen_self_attention *attn, int which, const lumen_tensor *w);
int lumen_self_attention_forward(lumen_self_attention *attn, const lumen_tensor *x, lumen_kv_cache *cache,
                                 lumen_tensor **out, lumen_kv_cache **cache_out);
int lumen_self_attention_free(lumen_self_attention *attn);

/* Attention core on raw device pointers (the part of the decode path between the projections and
 * w_o, self_attention.rs:141-297): q[B,Hq,D], k_new/v_new[B,Hkv,D] un-rotated; rotates q and k_new
 * at position len, appends to the cache, and writes out[B,Hq,D].  rope == NULL skips the rotation. */
int lumen_attention_decode(lumen_ctx *ctx, const float *q_dev, const float *k_new_dev, const float *v_new_dev,
                           size_t n_head, lumen_kv_cache *cache, lumen_rope *rope, int causal, float *out_dev);

/* ---- LlamaModel — src/models/llama.rs -------------------------------------------------------
 * The first nine fields are LlamaConfig (:11-21).  head_dim == 0 means hidden/heads (:162).
 * qk_norm adds a per-head RMSNorm on q and k before RoPE (Qwen3; not in the reference).
 * weight_dtype is the storage type of the projection / embedding / lm_head matrices. */
typedef struct {
    size_t vocab_size;
    size_t hidden_size;
    size_t intermediate_size;
    size_t num_hidden_layers;
    size_t num_attention_heads;
    size_t num_key_value_heads;
    float rms_norm_eps;
    size_t max_seq_len;
    float rope_theta;
    size_t head_dim;
    int qk_norm;
    lumen_dtype weight_dtype;
} lumen_llama_config;

/* new                <- LlamaModel::new (:138-156), parameters left unset
 * set_param          <- filling named_parameters() by HF name (:218-279; src/loader.rs:10-80).
 *                       data is a HOST pointer to the full (unsharded) tensor, f32 or bf16; a
 *                       tensor-parallel rank keeps only its slice.
 * init_kv_caches     <- LlamaModel::init_kv_caches(batch) (:161-169): writes num_hidden_layers handles
 * reset_kv_caches    <- LlamaModel::reset_kv_caches (:172-176)
 * forward            <- LlamaModel::forward(input_ids[B,S] as f32, caches, _pos) (:181-206);
 *                       ids and logits[B,S,V] are HOST buffers; pos is ignored like the reference's.
 * forward_last       <- same, but only the last position's logits [B,V] are computed and copied (what
 *                       the reference's caller keeps, src/main.rs:155-163).
 * forward_device     <- same as forward with DEVICE ids / logits and no synchronisation. */
int lumen_llama_new(lumen_ctx *ctx, const lumen_llama_config *cfg, lumen_llama **out);
/* Tensor-parallel shard plan, host arithmetic only (needs no device): the part of the named parameter that
 * rank tp_rank of tp_size keeps.  out = {rows, cols, row0, nrows, col0, ncols}: rows [row0, row0+nrows) x
 * columns [col0, col0+ncols) of the full [rows, cols] tensor; cols == 0 means a vector kept whole.  Split:
 * q/k/v/gate/up by output rows (whole heads; a KV head is replicated when there are fewer than ranks), o/down
 * by input columns, lm_head by vocabulary rows, norms and the embedding table replicated.  set_param applies
 * exactly this plan.  No counterpart in the reference (single process). */
int lumen_tp_param_slice(const lumen_llama_config *cfg, int tp_rank, int tp_size, const char *name, size_t out[6]);
int lumen_llama_set_param(lumen_llama *m, const char *name, const void *host_data, const size_t *shape, int ndim, lumen_dtype dtype);
int lumen_llama_init_kv_caches(lumen_llama *m, size_t batch, lumen_kv_cache **caches_out);
int lumen_llama_reset_kv_caches(lumen_llama *m, lumen_kv_cache **caches, size_t n_caches);
int lumen_llama_forward(lumen_llama *m, const float *ids_host, size_t b, size_t s, lumen_kv_cache **caches,
                        size_t n_caches, size_t pos, float *logits_host);
int lumen_llama_forward_last(lumen_llama *m, const float *ids_host, size_t b, size_t s, lumen_kv_cache **caches,
                             size_t n_caches, size_t pos, float *logits_host);
int lumen_llama_forward_device(lumen_llama *m, const float *ids_dev, size_t b, size_t s, lumen_kv_cache **caches,
                               size_t n_caches, float *logits_dev);
/* sample_top_p of the reference's chat loop (src/main.rs:74-137) on the device: repetition penalty over
 * `recent_tokens` (one division per occurrence, only when the penalty is > 1), temperature (floored at 1e-5),
 * softmax, stable descending sort, nucleus cut at top_p, inverse-CDF walk with `uniform` in [0,1) (the
 * reference draws it from its thread RNG, :69-72; here the caller supplies it so that runs can be repeated).
 * recent_tokens is a HOST array of at most 256 ids.
 * lumen_sample_top_p        : logits_dev[vocab] (device) -> *token_out (host); synchronises.
 * lumen_llama_forward_sample: LlamaModel::forward on ids[1,S] followed by the sampler on the last position's
 *                             logits, as main.rs:334-372 does on the host; only the token id is copied back. */
typedef struct {
    float temperature;
    float top_p;
    float repetition_penalty;
    const int32_t *recent_tokens;
    size_t n_recent;
    float uniform;
} lumen_sample_params;
int lumen_sample_top_p(lumen_ctx *ctx, const float *logits_dev, size_t vocab, const lumen_sample_params *params,
                       int32_t *token_out);
int lumen_llama_forward_sample(lumen_llama *m, const float *ids_host, size_t s, lumen_kv_cache **caches, size_t n_caches,
                               const lumen_sample_params *params, int32_t *token_out);
int lumen_llama_free(lumen_llama *m);
/* Bytes of weights one decode step streams on this rank (for roofline accounting). */
size_t lumen_llama_weight_bytes(const lumen_llama *m);
/* Tracing (no counterpart in the reference, which has no timers): when the environment variable
 * LUMEN_DECODE_TRACE=1 was set at lumen_llama_new, the persistent batch-1 decode kernel stores, for CTA 0,
 * a nanosecond timestamp at the start of each phase, after its prologue and after its last weight tile
 * (3 per phase; phases per layer: qkv, attention, o_proj, gate/up, down; then lm_head), plus one at the
 * end, followed by one stamp per phase taken when the producer issued the phase's first weight tile.
 * Copies up to `capacity` stamps of the last step to the host. */
int lumen_llama_decode_trace(lumen_llama *m, uint64_t *out, size_t capacity, size_t *n_out);

/* ---- measurement helpers (no counterpart in the reference) ----------------------------------
 * A kernel timed as a kernel: `iters` calls of lumen_gemv (src/ops/matmul.rs:42-69) / lumen_attention_decode
 * (self_attention.rs:141-297) enqueued back to back from compiled code between two CUDA events on the context's
 * stream, after three untimed calls, rotating over the n_w weight matrices / n_caches caches given (a working set
 * larger than L2).  *us_per_call_out = microseconds per call.  Every attention call appends one row to the cache
 * it uses, so each cache needs room for (iters + 3) / n_caches + 1 more rows.  Synchronises. */
int lumen_gemv_repeat(lumen_ctx *ctx, const float *x_dev, const void *const *w_devs, size_t n_w, lumen_dtype w_dtype, int layout_kn,
                      size_t k, size_t n, float *y_dev, size_t iters, float *us_per_call_out);
int lumen_attention_decode_repeat(lumen_ctx *ctx, const float *q_dev, const float *k_new_dev, const float *v_new_dev, size_t n_head,
                                  lumen_kv_cache *const *caches, size_t n_caches, lumen_rope *rope, float *out_dev, size_t iters,
                                  float *us_per_call_out);

#ifdef __cplusplus
}
#endif
#endif /* LUMEN_B200_H */
