// C ABI: operator-level entry points (matmul, norms, activations, RoPE, caches, SelfAttention).
#include <algorithm>
#include <cmath>

#include "common.cuh"

using namespace lumen;

struct lumen_llama_kv_cache {
    lumen_ctx *ctx = nullptr;
    size_t head_num = 0, max_seq_len = 0, dim = 0;
    float *k = nullptr, *v = nullptr;  // [1, Hkv, max_seq, D]
};

struct lumen_self_attention {
    lumen_ctx *ctx = nullptr;
    size_t embed_dim = 0, n_head = 0, n_kv_head = 0, head_dim = 0, max_seq = 0;
    float scale = 0.f;
    int causal = 1;
    lumen_rope *rope = nullptr;
    lumen_tensor *w[4] = {nullptr, nullptr, nullptr, nullptr};  // views sharing the caller's storage
    float *part = nullptr;
    size_t part_bytes = 0;
};

namespace lumen {

// Shared by the op-level API and the model: y[M,N] = a[M,K] . w[N,K]^T (+ residual).
int matmul_dispatch(lumen_ctx *ctx, const float *a, const void *w, lumen_dtype wdt, float *y, size_t M, size_t K,
                    size_t N, const float *residual, cudaStream_t s, const TpSumArgs *tp) {
    if (M == 0 || N == 0) return LUMEN_OK;
    if (ctx->tp_size == 1) tp = nullptr;
    const bool fused = tp && tp_sum_usable(ctx, M, N);
    // The streaming vector-matrix kernel takes up to 8 rows over f32 weights; over bf16 weights only a single row
    // (from two rows on, the tensor-core kernel with split K is faster).
    const size_t vec_rows = (wdt == LUMEN_BF16 && gemm_tc_usable(wdt, M, K, N, w)) ? 1 : 8;
    if (M <= vec_rows && M * K * 4 <= 200 * 1024) {
        GemvArgs g;
        g.x = a; g.w = w; g.wdt = wdt; g.y = y; g.M = (int)M; g.K = K; g.N = N; g.ldy = N; g.residual = residual;
        LUMEN_TRY(launch_gemv_nk(ctx, g, s));
        if (fused) return launch_tp_sum(ctx, y, 1, nullptr, M, N, *tp, s);
    } else {
        LUMEN_TRY(launch_gemm_nk(ctx, a, w, wdt, y, M, K, N, residual, s, fused ? tp : nullptr));
        if (fused) return LUMEN_OK;
    }
    if (tp) {
        // too many rows for the fused exchange (long prefill slices are bandwidth-bound): NCCL, then the norm
        LUMEN_TRY(tp_allreduce_sum(ctx, y, M * N, s));
        if (tp->norm_w) LUMEN_TRY(launch_rmsnorm(ctx, y, tp->norm_w, tp->eps, tp->normed, M, N, s));
    }
    return LUMEN_OK;
}

int rope_tables_host(size_t dim, size_t max_seq, float theta, std::vector<float> &cos_h, std::vector<float> &sin_h) {
    // RotaryEmbedding::precompute_freqs_cis — src/layers/attention/encoding.rs:38-51, evaluated on the host
    // in f32 exactly as written there: freq = 1.0 / theta.powf((j*2)/dim); val = pos*freq; cos/sin(val).
    const size_t half = dim / 2;
    cos_h.resize(max_seq * half);
    sin_h.resize(max_seq * half);
    for (size_t i = 0; i < max_seq; ++i) {
        const float pos = (float)i;
        for (size_t j = 0; j < half; ++j) {
            const float freq = 1.0f / powf(theta, ((float)j * 2.0f) / (float)dim);
            const float val = pos * freq;
            cos_h[i * half + j] = cosf(val);
            sin_h[i * half + j] = sinf(val);
        }
    }
    return LUMEN_OK;
}

}  // namespace lumen

namespace {

int require_f32(lumen_ctx *ctx, const lumen_tensor *t, const char *what) {
    if (!t) return set_error(ctx, LUMEN_ERR_INVALID, "%s: null tensor", what);
    if (t->dtype != LUMEN_F32) return set_error(ctx, LUMEN_ERR_DTYPE, "%s: activations must be f32", what);
    return LUMEN_OK;
}

}  // namespace

namespace {
template <typename F>
int timed_repeat(lumen_ctx *ctx, size_t iters, float *us_per_call_out, F call) {
    if (iters == 0) return set_error(ctx, LUMEN_ERR_INVALID, "repeat: iters == 0");
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    LUMEN_CUDA(ctx, cudaEventCreate(&e0));
    cudaError_t ce = cudaEventCreate(&e1);
    if (ce != cudaSuccess) {
        cudaEventDestroy(e0);
        return cuda_fail(ctx, ce, "cudaEventCreate");
    }
    int rc = LUMEN_OK;
    size_t i = 0;
    for (; i < 3 && rc == LUMEN_OK; ++i) rc = call(i);
    if (rc == LUMEN_OK) rc = check_device_status(ctx);
    if (rc == LUMEN_OK && cudaEventRecord(e0, ctx->stream) != cudaSuccess) rc = LUMEN_ERR_CUDA;
    for (size_t j = 0; j < iters && rc == LUMEN_OK; ++j) rc = call(i + j);
    if (rc == LUMEN_OK && cudaEventRecord(e1, ctx->stream) != cudaSuccess) rc = LUMEN_ERR_CUDA;
    if (rc == LUMEN_OK) rc = check_device_status(ctx);
    float ms = 0.f;
    if (rc == LUMEN_OK && cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = LUMEN_ERR_CUDA;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc == LUMEN_OK) *us_per_call_out = ms * 1000.0f / (float)iters;
    return rc;
}
}  // namespace


extern "C" {

int lumen_matmul(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *w, lumen_tensor **out) {
    if (!ctx || !a || !w || !out) return set_error(ctx, LUMEN_ERR_INVALID, "matmul: null argument");
    LUMEN_TRY(require_f32(ctx, a, "matmul lhs"));
    if (w->shape.size() != 2) return set_error(ctx, LUMEN_ERR_SHAPE, "MatMul RHS must be 2D, got %zu dims", w->shape.size());
    if (a->shape.empty()) return set_error(ctx, LUMEN_ERR_SHAPE, "MatMul LHS must have at least 1 dim");
    const size_t K = a->shape.back(), N = w->shape[0], Kb = w->shape[1];
    if (K != Kb) return set_error(ctx, LUMEN_ERR_SHAPE, "MatMul shape mismatch: a K=%zu vs b K=%zu", K, Kb);
    const size_t M = K ? a->numel() / K : 0;
    std::vector<size_t> os = a->shape;
    os.back() = N;
    LUMEN_TRY(new_tensor(ctx, os.data(), (int)os.size(), LUMEN_F32, out));
    if (K == 0) {
        LUMEN_CUDA(ctx, cudaMemsetAsync((*out)->data(), 0, (*out)->numel() * 4, ctx->stream));
        return LUMEN_OK;
    }
    return matmul_dispatch(ctx, static_cast<const float *>(a->data()), w->data(), w->dtype, static_cast<float *>((*out)->data()),
                           M, K, N, nullptr, ctx->stream);
}

int lumen_linear_forward(lumen_ctx *ctx, const lumen_tensor *x, const lumen_tensor *w, const lumen_tensor *bias, lumen_tensor **out) {
    LUMEN_TRY(lumen_matmul(ctx, x, w, out));
    if (bias) {
        if (bias->dtype != LUMEN_F32 || bias->numel() != w->shape[0]) {
            lumen_tensor_free(*out);
            *out = nullptr;
            return set_error(ctx, LUMEN_ERR_SHAPE, "Linear bias must be f32 [out_features]");
        }
        float *y = static_cast<float *>((*out)->data());
        return launch_binary(ctx, y, static_cast<const float *>(bias->data()), y, (*out)->numel(), bias->numel(), 0, ctx->stream);
    }
    return LUMEN_OK;
}

int lumen_rmsnorm(lumen_ctx *ctx, const lumen_tensor *x, const lumen_tensor *weight, float eps, lumen_tensor **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    LUMEN_TRY(require_f32(ctx, x, "rmsnorm input"));
    LUMEN_TRY(require_f32(ctx, weight, "rmsnorm weight"));
    if (x->shape.empty()) return set_error(ctx, LUMEN_ERR_SHAPE, "rmsnorm: input needs at least 1 dim");
    const size_t dim = x->shape.back();
    if (weight->numel() != dim) return set_error(ctx, LUMEN_ERR_SHAPE, "rmsnorm: weight has %zu elements, dim is %zu", weight->numel(), dim);
    LUMEN_TRY(new_tensor(ctx, x->shape.data(), (int)x->shape.size(), LUMEN_F32, out));
    if (dim == 0) return LUMEN_OK;
    return launch_rmsnorm(ctx, static_cast<const float *>(x->data()), static_cast<const float *>(weight->data()), eps,
                          static_cast<float *>((*out)->data()), x->numel() / dim, dim, ctx->stream);
}

int lumen_silu(lumen_ctx *ctx, const lumen_tensor *x, lumen_tensor **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    LUMEN_TRY(require_f32(ctx, x, "silu input"));
    LUMEN_TRY(new_tensor(ctx, x->shape.data(), (int)x->shape.size(), LUMEN_F32, out));
    return launch_silu(ctx, static_cast<const float *>(x->data()), static_cast<float *>((*out)->data()), x->numel(), ctx->stream);
}

static int binary_op(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *b, lumen_tensor **out, int is_mul) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    LUMEN_TRY(require_f32(ctx, a, "binary lhs"));
    LUMEN_TRY(require_f32(ctx, b, "binary rhs"));
    const size_t n = a->numel(), nb = b->numel();
    bool same = a->shape == b->shape;
    bool trailing = false;
    if (!same && nb > 0 && b->shape.size() <= a->shape.size()) {
        trailing = std::equal(b->shape.rbegin(), b->shape.rend(), a->shape.rbegin());
    }
    if (!same && !trailing) return set_error(ctx, LUMEN_ERR_SHAPE, "elementwise op: shapes are neither equal nor trailing-broadcastable");
    LUMEN_TRY(new_tensor(ctx, a->shape.data(), (int)a->shape.size(), LUMEN_F32, out));
    return launch_binary(ctx, static_cast<const float *>(a->data()), static_cast<const float *>(b->data()),
                         static_cast<float *>((*out)->data()), n, same ? n : nb, is_mul, ctx->stream);
}

int lumen_mul(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *b, lumen_tensor **out) { return binary_op(ctx, a, b, out, 1); }
int lumen_add(lumen_ctx *ctx, const lumen_tensor *a, const lumen_tensor *b, lumen_tensor **out) { return binary_op(ctx, a, b, out, 0); }

int lumen_embedding(lumen_ctx *ctx, const lumen_tensor *ids, const lumen_tensor *table, lumen_tensor **out) {
    if (!ctx || !out || !table) return set_error(ctx, LUMEN_ERR_INVALID, "embedding: null argument");
    LUMEN_TRY(require_f32(ctx, ids, "embedding ids"));
    if (table->shape.size() != 2) return set_error(ctx, LUMEN_ERR_SHAPE, "Embedding weight must be 2D");
    std::vector<size_t> os = ids->shape;
    os.push_back(table->shape[1]);
    LUMEN_TRY(new_tensor(ctx, os.data(), (int)os.size(), LUMEN_F32, out));
    LUMEN_TRY(launch_embedding(ctx, static_cast<const float *>(ids->data()), table->data(), table->dtype,
                               static_cast<float *>((*out)->data()), ids->numel(), table->shape[0], table->shape[1], ctx->stream));
    // The reference panics on an out-of-range id before returning; surface that here.
    int rc = check_device_status(ctx);
    if (rc != LUMEN_OK) {
        lumen_tensor_free(*out);
        *out = nullptr;
    }
    return rc;
}

int lumen_fused_softmax(lumen_ctx *ctx, const lumen_tensor *x, float scale, int causal, lumen_tensor **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    LUMEN_TRY(require_f32(ctx, x, "fused_softmax input"));
    if (x->shape.size() != 4) return set_error(ctx, LUMEN_ERR_SHAPE, "Fused Softmax expects 4D input [B, H, Q, K]");
    LUMEN_TRY(new_tensor(ctx, x->shape.data(), 4, LUMEN_F32, out));
    return launch_fused_softmax(ctx, static_cast<const float *>(x->data()), static_cast<float *>((*out)->data()),
                                x->shape[0] * x->shape[1], x->shape[2], x->shape[3], scale, causal, ctx->stream);
}

int lumen_gemv(lumen_ctx *ctx, const float *x_dev, const void *w_dev, lumen_dtype w_dtype, int layout_kn, size_t k, size_t n, float *y_dev) {
    if (!ctx || !x_dev || !w_dev || !y_dev) return set_error(ctx, LUMEN_ERR_INVALID, "gemv: null argument");
    if (w_dtype != LUMEN_F32 && w_dtype != LUMEN_BF16) return set_error(ctx, LUMEN_ERR_DTYPE, "gemv: dtype %d", (int)w_dtype);
    if (k == 0 || n == 0) return LUMEN_OK;
    if (!layout_kn) {
        if (k * 4 > 200 * 1024) return launch_gemm_nk(ctx, x_dev, w_dev, w_dtype, y_dev, 1, k, n, nullptr, ctx->stream);
        GemvArgs g;
        g.x = x_dev; g.w = w_dev; g.wdt = w_dtype; g.y = y_dev; g.M = 1; g.K = k; g.N = n; g.ldy = n;
        return launch_gemv_nk(ctx, g, ctx->stream);
    }
    void *scratch = nullptr;
    LUMEN_TRY(dev_alloc(ctx, gemv_kn_scratch_bytes(k, n, ctx->num_sms), &scratch));
    int rc = launch_gemv_kn(ctx, x_dev, w_dev, w_dtype, y_dev, k, n, static_cast<float *>(scratch), ctx->stream);
    int rc2 = dev_free(ctx, scratch);
    return rc != LUMEN_OK ? rc : rc2;
}

// ---- measurement helpers: a kernel timed as a kernel ----------------------------------------------------------
// `iters` calls enqueued back to back from compiled code between two CUDA events on the context's stream (after
// three untimed calls), rotating over the given operands so that a working set larger than L2 can be used: the
// per-call cost of an interpreted host and its launch rate stay out of the number.
int lumen_gemv_repeat(lumen_ctx *ctx, const float *x_dev, const void *const *w_devs, size_t n_w, lumen_dtype w_dtype, int layout_kn,
                      size_t k, size_t n, float *y_dev, size_t iters, float *us_per_call_out) {
    if (!ctx || !w_devs || n_w == 0 || !us_per_call_out) return set_error(ctx, LUMEN_ERR_INVALID, "gemv_repeat: null argument");
    return timed_repeat(ctx, iters, us_per_call_out,
                        [&](size_t i) { return lumen_gemv(ctx, x_dev, w_devs[i % n_w], w_dtype, layout_kn, k, n, y_dev); });
}

int lumen_attention_decode_repeat(lumen_ctx *ctx, const float *q_dev, const float *k_new_dev, const float *v_new_dev, size_t n_head,
                                  lumen_kv_cache *const *caches, size_t n_caches, lumen_rope *rope, float *out_dev, size_t iters,
                                  float *us_per_call_out) {
    if (!ctx || !caches || n_caches == 0 || !us_per_call_out)
        return set_error(ctx, LUMEN_ERR_INVALID, "attention_decode_repeat: null argument");
    return timed_repeat(ctx, iters, us_per_call_out, [&](size_t i) {
        return lumen_attention_decode(ctx, q_dev, k_new_dev, v_new_dev, n_head, caches[i % n_caches], rope, 1, out_dev);
    });
}

int lumen_sample_top_p(lumen_ctx *ctx, const float *logits_dev, size_t vocab, const lumen_sample_params *sp, int32_t *token_out) {
    if (!ctx || !logits_dev || !sp || !token_out || (sp->n_recent && !sp->recent_tokens))
        return set_error(ctx, LUMEN_ERR_INVALID, "sample_top_p: null argument");
    void *tok = nullptr;
    LUMEN_TRY(dev_alloc(ctx, 256, &tok));
    int rc = launch_sample_top_p(ctx, logits_dev, vocab, sp->temperature, sp->top_p, sp->repetition_penalty, sp->recent_tokens,
                                 sp->n_recent, sp->uniform, static_cast<int *>(tok), ctx->stream);
    int32_t host = 0;
    if (rc == LUMEN_OK) {
        cudaError_t e = cudaMemcpyAsync(&host, tok, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) rc = cuda_fail(ctx, e, "cudaMemcpyAsync(token)");
    }
    if (rc == LUMEN_OK) rc = check_device_status(ctx);  // synchronises
    int rc2 = dev_free(ctx, tok);
    if (rc == LUMEN_OK) *token_out = host;
    return rc != LUMEN_OK ? rc : rc2;
}

// ---- RotaryEmbedding ---------------------------------------------------------------------------------
int lumen_rope_new(lumen_ctx *ctx, size_t dim, size_t max_seq_len, float theta, lumen_rope **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    if (dim == 0 || (dim & 1)) return set_error(ctx, LUMEN_ERR_SHAPE, "RoPE dim must be even, got %zu", dim);
    std::vector<float> ch, sh;
    rope_tables_host(dim, max_seq_len, theta, ch, sh);
    auto *r = new lumen_rope();
    r->ctx = ctx; r->dim = dim; r->max_seq = max_seq_len; r->theta = theta;
    const size_t bytes = std::max<size_t>(ch.size() * 4, 16);
    cudaError_t e;
    if ((e = cudaMalloc(&r->cos_t, bytes)) != cudaSuccess || (e = cudaMalloc(&r->sin_t, bytes)) != cudaSuccess) {
        if (r->cos_t) cudaFree(r->cos_t);
        delete r;
        return cuda_fail(ctx, e, "cudaMalloc(rope tables)");
    }
    if (!ch.empty()) {
        LUMEN_CUDA(ctx, cudaMemcpy(r->cos_t, ch.data(), ch.size() * 4, cudaMemcpyHostToDevice));
        LUMEN_CUDA(ctx, cudaMemcpy(r->sin_t, sh.data(), sh.size() * 4, cudaMemcpyHostToDevice));
    }
    *out = r;
    return LUMEN_OK;
}

int lumen_rope_forward(lumen_rope *rope, const lumen_tensor *x, size_t offset, lumen_tensor **out) {
    if (!rope || !out) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = rope->ctx;
    LUMEN_TRY(require_f32(ctx, x, "rope input"));
    if (x->shape.size() != 4) return set_error(ctx, LUMEN_ERR_SHAPE, "RoPE expects [B,H,S,D]");
    if (x->shape[3] != rope->dim) return set_error(ctx, LUMEN_ERR_SHAPE, "RoPE dimension mismatch");
    if (offset + x->shape[2] > rope->max_seq)
        return set_error(ctx, LUMEN_ERR_ROPE_RANGE, "RoPE index out of range: offset %zu + len %zu > max %zu", offset, x->shape[2], rope->max_seq);
    LUMEN_TRY(new_tensor(ctx, x->shape.data(), 4, LUMEN_F32, out));
    return launch_rope_forward(ctx, static_cast<const float *>(x->data()), static_cast<float *>((*out)->data()), x->shape[0],
                               x->shape[1], x->shape[2], x->shape[3], offset, rope->cos_t, rope->sin_t, ctx->stream);
}

int lumen_rope_free(lumen_rope *rope) {
    if (!rope) return LUMEN_ERR_INVALID;
    cudaStreamSynchronize(rope->ctx->stream);
    cudaFree(rope->cos_t);
    cudaFree(rope->sin_t);
    delete rope;
    return LUMEN_OK;
}

// ---- KVCacheInner --------------------------------------------------------------------------------------
int lumen_kv_new(lumen_ctx *ctx, size_t b, size_t h_kv, size_t max_seq, size_t d, lumen_kv_cache **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    auto *c = new lumen_kv_cache();
    c->ctx = ctx; c->b = b; c->h_kv = h_kv; c->max_seq = max_seq; c->d = d;
    const size_t n = std::max<size_t>(b * h_kv * max_seq * d, 4);
    cudaError_t e;
    if ((e = cudaMalloc(&c->k, 2 * n * sizeof(float) + 16)) != cudaSuccess) {
        delete c;
        return cuda_fail(ctx, e, "cudaMalloc(kv cache)");
    }
    c->v = c->k + n;
    c->d_len = reinterpret_cast<int *>(c->v + n);
    c->seen_abort = ctx->abort_gen;
    LUMEN_CUDA(ctx, cudaMemsetAsync(c->k, 0, 2 * n * sizeof(float) + 16, ctx->stream));
    *out = c;
    return LUMEN_OK;
}

int lumen_kv_reset(lumen_kv_cache *c) {
    if (!c) return LUMEN_ERR_INVALID;
    c->len = 0;  // contents are kept, like KVCacheInner::reset
    c->seen_abort = c->ctx->abort_gen;
    LUMEN_CUDA(c->ctx, cudaMemsetAsync(c->d_len, 0, sizeof(int), c->ctx->stream));
    return LUMEN_OK;
}

size_t lumen_kv_len(const lumen_kv_cache *c) {
    if (!c) return 0;
    kv_resync_len(const_cast<lumen_kv_cache *>(c));  // after a device-side abort the device copy is the truth
    return c->len;
}

int lumen_kv_free(lumen_kv_cache *c) {
    if (!c) return LUMEN_ERR_INVALID;
    if (c->owns_slab) {
        cudaStreamSynchronize(c->ctx->stream);
        cudaFree(c->k);
    } else if (c->slab && --c->slab->refs == 0) {
        cudaStreamSynchronize(c->ctx->stream);
        cudaFree(c->slab->ptr);
        delete c->slab;
    }
    delete c;
    return LUMEN_OK;
}

int lumen_kv_read(const lumen_kv_cache *c, float *k_out, float *v_out) {
    if (!c || !k_out || !v_out) return LUMEN_ERR_INVALID;
    const size_t bytes = c->b * c->h_kv * c->max_seq * c->d * sizeof(float);
    LUMEN_CUDA(c->ctx, cudaMemcpyAsync(k_out, c->k, bytes, cudaMemcpyDeviceToHost, c->ctx->stream));
    LUMEN_CUDA(c->ctx, cudaMemcpyAsync(v_out, c->v, bytes, cudaMemcpyDeviceToHost, c->ctx->stream));
    LUMEN_CUDA(c->ctx, cudaStreamSynchronize(c->ctx->stream));
    return LUMEN_OK;
}

int lumen_kv_write(lumen_kv_cache *c, const float *k_in, const float *v_in, size_t len) {
    if (!c || !k_in || !v_in) return LUMEN_ERR_INVALID;
    if (len > c->max_seq) return set_error(c->ctx, LUMEN_ERR_KV_OVERFLOW, "KV cache overflow: len=%zu > max_seq=%zu", len, c->max_seq);
    const size_t bytes = c->b * c->h_kv * c->max_seq * c->d * sizeof(float);
    const int ilen = (int)len;
    LUMEN_CUDA(c->ctx, cudaMemcpyAsync(c->k, k_in, bytes, cudaMemcpyHostToDevice, c->ctx->stream));
    LUMEN_CUDA(c->ctx, cudaMemcpyAsync(c->v, v_in, bytes, cudaMemcpyHostToDevice, c->ctx->stream));
    LUMEN_CUDA(c->ctx, cudaMemcpyAsync(c->d_len, &ilen, sizeof(int), cudaMemcpyHostToDevice, c->ctx->stream));
    LUMEN_CUDA(c->ctx, cudaStreamSynchronize(c->ctx->stream));
    c->len = len;
    c->seen_abort = c->ctx->abort_gen;
    return LUMEN_OK;
}

// ---- LlamaKVCache ---------------------------------------------------------------------------------------
int lumen_llama_kv_new(lumen_ctx *ctx, size_t kv_heads, size_t max_seq_len, size_t head_dim, lumen_llama_kv_cache **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    auto *c = new lumen_llama_kv_cache();
    c->ctx = ctx; c->head_num = kv_heads; c->max_seq_len = max_seq_len; c->dim = head_dim;
    const size_t n = std::max<size_t>(kv_heads * max_seq_len * head_dim, 4);
    cudaError_t e;
    if ((e = cudaMalloc(&c->k, 2 * n * sizeof(float))) != cudaSuccess) {
        delete c;
        return cuda_fail(ctx, e, "cudaMalloc(llama kv cache)");
    }
    c->v = c->k + n;
    LUMEN_CUDA(ctx, cudaMemsetAsync(c->k, 0, 2 * n * sizeof(float), ctx->stream));
    *out = c;
    return LUMEN_OK;
}

int lumen_llama_kv_update(lumen_llama_kv_cache *c, const lumen_tensor *k, const lumen_tensor *v, size_t start_pos) {
    if (!c || !k || !v) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = c->ctx;
    LUMEN_TRY(require_f32(ctx, k, "kv update k"));
    LUMEN_TRY(require_f32(ctx, v, "kv update v"));
    if (k->shape.size() != 4 || v->shape != k->shape || k->shape[0] != 1 || k->shape[1] != c->head_num || k->shape[3] != c->dim)
        return set_error(ctx, LUMEN_ERR_SHAPE, "LlamaKVCache::update expects k,v [1,%zu,S,%zu]", c->head_num, c->dim);
    const size_t s = k->shape[2];
    if (start_pos + s > c->max_seq_len)
        return set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "KV Cache overflow! Max: %zu, Current: %zu", c->max_seq_len, start_pos + s);
    LUMEN_TRY(launch_kv_slab_copy(ctx, static_cast<const float *>(k->data()), c->k, c->head_num, s, c->dim, c->max_seq_len, start_pos, 1, ctx->stream));
    return launch_kv_slab_copy(ctx, static_cast<const float *>(v->data()), c->v, c->head_num, s, c->dim, c->max_seq_len, start_pos, 1, ctx->stream);
}

int lumen_llama_kv_get_view(const lumen_llama_kv_cache *c, size_t current_len, lumen_tensor **k_out, lumen_tensor **v_out) {
    if (!c || !k_out || !v_out) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = c->ctx;
    if (current_len > c->max_seq_len) return set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "get_view: %zu > max %zu", current_len, c->max_seq_len);
    const size_t shape[4] = {1, c->head_num, current_len, c->dim};
    LUMEN_TRY(new_tensor(ctx, shape, 4, LUMEN_F32, k_out));
    int rc = new_tensor(ctx, shape, 4, LUMEN_F32, v_out);
    if (rc != LUMEN_OK) {
        lumen_tensor_free(*k_out);
        return rc;
    }
    LUMEN_TRY(launch_kv_slab_copy(ctx, c->k, static_cast<float *>((*k_out)->data()), c->head_num, current_len, c->dim, c->max_seq_len, 0, 0, ctx->stream));
    return launch_kv_slab_copy(ctx, c->v, static_cast<float *>((*v_out)->data()), c->head_num, current_len, c->dim, c->max_seq_len, 0, 0, ctx->stream);
}

int lumen_llama_kv_free(lumen_llama_kv_cache *c) {
    if (!c) return LUMEN_ERR_INVALID;
    cudaStreamSynchronize(c->ctx->stream);
    cudaFree(c->k);
    delete c;
    return LUMEN_OK;
}

// ---- attention core on raw pointers ------------------------------------------------------------------------
int lumen_attention_decode(lumen_ctx *ctx, const float *q_dev, const float *k_new_dev, const float *v_new_dev, size_t n_head,
                           lumen_kv_cache *cache, lumen_rope *rope, int causal, float *out_dev) {
    if (!ctx || !q_dev || !k_new_dev || !v_new_dev || !cache || !out_dev) return set_error(ctx, LUMEN_ERR_INVALID, "attention_decode: null argument");
    (void)causal;  // with S == 1 the causal test `j > past_len` never fires (self_attention.rs:255-258)
    LUMEN_TRY(kv_resync_len(cache));
    if (cache->len + 1 > cache->max_seq)
        return set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "KV cache overflow: new_len=%zu > max_seq=%zu", cache->len + 1, cache->max_seq);
    if (rope) {
        if (rope->dim != cache->d) return set_error(ctx, LUMEN_ERR_SHAPE, "RoPE dimension mismatch");
        if (cache->len >= rope->max_seq)
            return set_error(ctx, LUMEN_ERR_ROPE_RANGE, "RoPE index out of range: pos %zu >= max %zu", cache->len, rope->max_seq);
    }
    AttnDecodeArgs a;
    a.q = q_dev; a.k_new = k_new_dev; a.v_new = v_new_dev;
    a.q_stride = n_head * cache->d; a.kv_stride = cache->h_kv * cache->d;
    a.k_cache = cache->k; a.v_cache = cache->v; a.d_len = cache->d_len;
    a.B = cache->b; a.Hq = n_head; a.Hkv = cache->h_kv; a.D = cache->d; a.max_seq = cache->max_seq;
    a.cos_t = rope ? rope->cos_t : nullptr; a.sin_t = rope ? rope->sin_t : nullptr;
    a.scale = 1.0f / sqrtf((float)cache->d);
    a.out = out_dev;
    a.max_splits = attn_decode_pick_splits(a.B, a.Hkv, cache->len + 1, ctx->num_sms);
    a.len_hint = cache->len;
    void *part = nullptr;
    LUMEN_TRY(dev_alloc(ctx, attn_decode_scratch_bytes(a.B, a.Hq, a.D, a.max_splits), &part));
    a.part = static_cast<float *>(part);
    int rc = launch_attn_decode(ctx, a, ctx->stream);
    int rc2 = dev_free(ctx, part);
    if (rc == LUMEN_OK) cache->len += 1;
    return rc != LUMEN_OK ? rc : rc2;
}

// ---- SelfAttention -----------------------------------------------------------------------------------------
int lumen_self_attention_new(lumen_ctx *ctx, size_t embed_dim, size_t n_head, size_t n_kv_head, size_t max_seq_len,
                             float rope_theta, int causal, lumen_self_attention **out) {
    if (!ctx || !out) return LUMEN_ERR_INVALID;
    if (n_head == 0 || embed_dim % n_head) return set_error(ctx, LUMEN_ERR_SHAPE, "Embed dim must be divisible by n_head");
    if (n_kv_head == 0 || n_head % n_kv_head) return set_error(ctx, LUMEN_ERR_SHAPE, "n_head must be a multiple of n_kv_head");
    auto *a = new lumen_self_attention();
    a->ctx = ctx; a->embed_dim = embed_dim; a->n_head = n_head; a->n_kv_head = n_kv_head;
    a->head_dim = embed_dim / n_head; a->max_seq = max_seq_len; a->causal = causal;
    a->scale = 1.0f / sqrtf((float)a->head_dim);  // (head_dim as f32).sqrt().recip()
    int rc = lumen_rope_new(ctx, a->head_dim, max_seq_len, rope_theta, &a->rope);
    if (rc != LUMEN_OK) {
        delete a;
        return rc;
    }
    *out = a;
    return LUMEN_OK;
}

int lumen_self_attention_set_weight(lumen_self_attention *attn, int which, const lumen_tensor *w) {
    if (!attn || !w || which < 0 || which > 3) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = attn->ctx;
    const size_t kv_dim = attn->n_kv_head * attn->head_dim;
    const size_t rows = (which == LUMEN_W_K || which == LUMEN_W_V) ? kv_dim : attn->embed_dim;
    if (w->shape.size() != 2 || w->shape[0] != rows || w->shape[1] != attn->embed_dim)
        return set_error(ctx, LUMEN_ERR_SHAPE, "SelfAttention weight %d must be [%zu,%zu]", which, rows, attn->embed_dim);
    if (attn->w[which]) lumen_tensor_free(attn->w[which]);
    auto *view = new lumen_tensor(*w);
    view->st->refs += 1;
    attn->w[which] = view;
    return LUMEN_OK;
}

int lumen_self_attention_forward(lumen_self_attention *attn, const lumen_tensor *x, lumen_kv_cache *cache, lumen_tensor **out,
                                 lumen_kv_cache **cache_out) {
    if (!attn || !x || !out) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = attn->ctx;
    LUMEN_TRY(require_f32(ctx, x, "SelfAttention input"));
    for (int i = 0; i < 4; ++i)
        if (!attn->w[i]) return set_error(ctx, LUMEN_ERR_MISSING_PARAM, "SelfAttention weight %d not set", i);
    if (x->shape.size() != 3 || x->shape[2] != attn->embed_dim) return set_error(ctx, LUMEN_ERR_SHAPE, "SelfAttention expects x [B,S,%zu]", attn->embed_dim);
    const size_t B = x->shape[0], S = x->shape[1], E = attn->embed_dim, D = attn->head_dim;
    const size_t Hq = attn->n_head, Hkv = attn->n_kv_head, kvd = Hkv * D, M = B * S;
    bool created = false;
    if (!cache) {
        LUMEN_TRY(lumen_kv_new(ctx, B, Hkv, attn->max_seq, D, &cache));
        created = true;
    }
    auto bail = [&](int rc) {
        if (created) lumen_kv_free(cache);
        return rc;
    };
    if (cache->b != B || cache->h_kv != Hkv || cache->d != D) return bail(set_error(ctx, LUMEN_ERR_SHAPE, "KV cache geometry does not match the layer"));
    // Order of the reference's checks: prefill runs rope.forward (range panic) before the overflow assert;
    // decode asserts overflow first (self_attention.rs:144-149 vs :334-346).
    if (int rs = kv_resync_len(cache)) return bail(rs);
    const size_t past = cache->len;
    if (S == 1) {
        if (past + 1 > cache->max_seq) return bail(set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "KV cache overflow: new_len=%zu > max_seq=%zu", past + 1, cache->max_seq));
        if (past >= attn->rope->max_seq) return bail(set_error(ctx, LUMEN_ERR_ROPE_RANGE, "RoPE index out of range: pos %zu >= max %zu", past, attn->rope->max_seq));
    } else {
        if (past + S > attn->rope->max_seq) return bail(set_error(ctx, LUMEN_ERR_ROPE_RANGE, "RoPE index out of range: offset %zu + len %zu > max %zu", past, S, attn->rope->max_seq));
        if (past + S > cache->max_seq) return bail(set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "KV cache overflow: new_len=%zu > max_seq=%zu", past + S, cache->max_seq));
    }
    cudaStream_t st = ctx->stream;
    void *qb = nullptr, *kb = nullptr, *vb = nullptr, *ab = nullptr;
    int rc = dev_alloc(ctx, M * E * 4, &qb);
    if (rc == LUMEN_OK) rc = dev_alloc(ctx, M * kvd * 4, &kb);
    if (rc == LUMEN_OK) rc = dev_alloc(ctx, M * kvd * 4, &vb);
    if (rc == LUMEN_OK) rc = dev_alloc(ctx, M * E * 4, &ab);
    const float *xp = static_cast<const float *>(x->data());
    if (rc == LUMEN_OK) rc = matmul_dispatch(ctx, xp, attn->w[0]->data(), attn->w[0]->dtype, (float *)qb, M, E, E, nullptr, st);
    if (rc == LUMEN_OK) rc = matmul_dispatch(ctx, xp, attn->w[1]->data(), attn->w[1]->dtype, (float *)kb, M, E, kvd, nullptr, st);
    if (rc == LUMEN_OK) rc = matmul_dispatch(ctx, xp, attn->w[2]->data(), attn->w[2]->dtype, (float *)vb, M, E, kvd, nullptr, st);
    if (rc == LUMEN_OK && S == 1) {
        AttnDecodeArgs a;
        a.q = (float *)qb; a.k_new = (float *)kb; a.v_new = (float *)vb;
        a.q_stride = E; a.kv_stride = kvd;
        a.k_cache = cache->k; a.v_cache = cache->v; a.d_len = cache->d_len;
        a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.max_seq = cache->max_seq;
        a.cos_t = attn->rope->cos_t; a.sin_t = attn->rope->sin_t;
        a.scale = attn->scale; a.out = (float *)ab;
        a.max_splits = attn_decode_pick_splits(B, Hkv, past + 1, ctx->num_sms);
        a.len_hint = past;
        const size_t need = attn_decode_scratch_bytes(B, Hq, D, a.max_splits);
        void *part = nullptr;
        rc = dev_alloc(ctx, need, &part);
        a.part = (float *)part;
        if (rc == LUMEN_OK) rc = launch_attn_decode(ctx, a, st);
        dev_free(ctx, part);
        if (rc == LUMEN_OK) cache->len = past + 1;
    } else if (rc == LUMEN_OK) {
        AttnPrefillArgs a;
        a.q = (float *)qb; a.k = (float *)kb; a.v = (float *)vb;
        a.q_stride = E; a.kv_stride = kvd;
        a.k_cache = cache->k; a.v_cache = cache->v;
        a.past = past; a.S = S; a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.max_seq = cache->max_seq;
        a.cos_t = attn->rope->cos_t; a.sin_t = attn->rope->sin_t;
        a.scale = attn->scale; a.causal = attn->causal; a.out = (float *)ab;
        rc = launch_attn_prefill(ctx, a, st);
        if (rc == LUMEN_OK) rc = launch_bump_len(ctx, cache->d_len, (int)S, st);
        if (rc == LUMEN_OK) cache->len = past + S;
    }
    if (rc == LUMEN_OK) {
        const size_t os[3] = {B, S, E};
        rc = new_tensor(ctx, os, 3, LUMEN_F32, out);
        if (rc == LUMEN_OK)
            rc = matmul_dispatch(ctx, (float *)ab, attn->w[3]->data(), attn->w[3]->dtype, (float *)(*out)->data(), M, E, E, nullptr, st);
    }
    dev_free(ctx, qb); dev_free(ctx, kb); dev_free(ctx, vb); dev_free(ctx, ab);
    if (rc != LUMEN_OK) return bail(rc);
    if (cache_out) *cache_out = cache;
    return LUMEN_OK;
}

int lumen_self_attention_free(lumen_self_attention *attn) {
    if (!attn) return LUMEN_ERR_INVALID;
    for (auto *w : attn->w)
        if (w) lumen_tensor_free(w);
    if (attn->rope) lumen_rope_free(attn->rope);
    delete attn;
    return LUMEN_OK;
}

}  // extern "C"
