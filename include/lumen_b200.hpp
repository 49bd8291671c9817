// C++ host-side mirror of Lumen's inference interface over the lumen_b200 C ABI.
//
// The reference is a compiled (Rust) crate whose callers use `Tensor`, `Module`, `Linear`, `RMSNorm`,
// `RotaryEmbedding`, `SelfAttention`, `KVCache`, `LlamaKVCache`, `LlamaConfig` and `LlamaModel`
// (src/autograd.rs, src/module.rs, src/layers/..., src/kv_cache.rs, src/models/llama.rs).  This header
// gives a compiled host the same names, argument meanings and error behaviour: what the reference
// turns into `panic!` is thrown here as lumen_b200::Error (status code + the library's message).
// Header-only; link with -llumen_b200.  Handles are reference counted like the reference's
// `Rc<RefCell<..>>` (autograd.rs:64, self_attention.rs:30); one host thread per Context, as there.
#pragma once

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "lumen_b200.h"

namespace lumen_b200 {

class Error : public std::runtime_error {
public:
    Error(int status, const std::string &msg) : std::runtime_error(msg), code(status) {}
    int code;
};

inline void check(int status, const lumen_ctx *ctx = nullptr) {
    if (status == LUMEN_OK) return;
    std::string msg = lumen_status_string(status);
    if (ctx) {
        const char *detail = lumen_last_error(ctx);
        if (detail && detail[0]) msg += std::string(": ") + detail;
    }
    throw Error(status, msg);
}

// One GPU (or one tensor-parallel rank) with its stream.  No counterpart in the reference.
class Context {
public:
    explicit Context(int device = 0, int tp_rank = 0, int tp_size = 1, const void *nccl_id = nullptr) {
        lumen_ctx *h = nullptr;
        check(lumen_ctx_create(device, tp_rank, tp_size, nccl_id, &h));
        h_.reset(h, [](lumen_ctx *c) { lumen_ctx_destroy(c); });
    }
    lumen_ctx *get() const { return h_.get(); }
    void synchronize() const { check(lumen_ctx_synchronize(get()), get()); }
    uint64_t launch_count() const { return lumen_ctx_launch_count(get()); }

private:
    std::shared_ptr<lumen_ctx> h_;
};

// `no_grad()` guard (autograd.rs:43-51).  Only the inference branches exist here, so the guard is a
// marker: modules refuse to run outside one, as the training branches are not provided.
class NoGradGuard {
public:
    NoGradGuard() { ++depth(); }
    ~NoGradGuard() { --depth(); }
    NoGradGuard(const NoGradGuard &) = delete;
    NoGradGuard &operator=(const NoGradGuard &) = delete;
    static bool active() { return depth() > 0; }

private:
    static int &depth() {
        static thread_local int d = 0;
        return d;
    }
};
inline NoGradGuard no_grad() { return NoGradGuard(); }
inline bool is_no_grad() { return NoGradGuard::active(); }
inline void require_no_grad(const char *what) {
    if (!is_no_grad()) throw Error(LUMEN_ERR_UNSUPPORTED, std::string(what) + ": only the no_grad (inference) path is provided");
}

// Tensor (autograd.rs:63-64): shape + f32 (or bf16 weight) data on the device.
class Tensor {
public:
    Tensor() = default;
    // Tensor::from_array_no_grad (autograd.rs:161-163)
    static Tensor from_array_no_grad(const Context &ctx, const std::vector<size_t> &shape, const float *data) {
        lumen_tensor *t = nullptr;
        check(lumen_tensor_from_host(ctx.get(), data, shape.data(), (int)shape.size(), &t), ctx.get());
        return Tensor(ctx, t);
    }
    static Tensor from_bf16_bits(const Context &ctx, const std::vector<size_t> &shape, const uint16_t *bits) {
        lumen_tensor *t = nullptr;
        check(lumen_tensor_from_host_bf16(ctx.get(), bits, shape.data(), (int)shape.size(), &t), ctx.get());
        return Tensor(ctx, t);
    }
    std::vector<size_t> shape() const {
        std::vector<size_t> s((size_t)lumen_tensor_ndim(get()));
        if (!s.empty()) check(lumen_tensor_shape(get(), s.data()), ctx_.get());
        return s;
    }
    size_t numel() const { return lumen_tensor_numel(get()); }
    // data_ref / get_raw_data (autograd.rs:82-112, 251-257): a host copy
    std::vector<float> data() const {
        std::vector<float> out(numel());
        check(lumen_tensor_to_host(get(), out.data()), ctx_.get());
        return out;
    }
    // set_raw_data (autograd.rs:259-262)
    void set_raw_data(const float *data) { check(lumen_tensor_set(get(), data), ctx_.get()); }
    Tensor reshape(const std::vector<int64_t> &shape) const {
        lumen_tensor *t = nullptr;
        check(lumen_tensor_reshape(get(), shape.data(), (int)shape.size(), &t), ctx_.get());
        return Tensor(ctx_, t);
    }
    void *device_ptr() const { return lumen_tensor_data(get()); }
    lumen_tensor *get() const { return h_.get(); }
    const Context &context() const { return ctx_; }
    explicit operator bool() const { return (bool)h_; }

    Tensor(const Context &ctx, lumen_tensor *t) : ctx_(ctx), h_(t, [](lumen_tensor *p) { lumen_tensor_free(p); }) {}

private:
    Context ctx_{};
    std::shared_ptr<lumen_tensor> h_;
};

// ops::matmul (src/ops/matmul.rs:10): a[..., K] x w[N, K] -> [..., N]
inline Tensor matmul(const Tensor &a, const Tensor &w) {
    lumen_tensor *out = nullptr;
    check(lumen_matmul(a.context().get(), a.get(), w.get(), &out), a.context().get());
    return Tensor(a.context(), out);
}
// Tensor + Tensor, Tensor * Tensor (src/ops/arithmetic.rs:48-52, 105-109)
inline Tensor operator+(const Tensor &a, const Tensor &b) {
    lumen_tensor *out = nullptr;
    check(lumen_add(a.context().get(), a.get(), b.get(), &out), a.context().get());
    return Tensor(a.context(), out);
}
inline Tensor operator*(const Tensor &a, const Tensor &b) {
    lumen_tensor *out = nullptr;
    check(lumen_mul(a.context().get(), a.get(), b.get(), &out), a.context().get());
    return Tensor(a.context(), out);
}
// ops::fused::fused_softmax (src/ops/fused.rs:17)
inline Tensor fused_softmax(const Tensor &x, float scale, bool causal) {
    lumen_tensor *out = nullptr;
    check(lumen_fused_softmax(x.context().get(), x.get(), scale, causal ? 1 : 0, &out), x.context().get());
    return Tensor(x.context(), out);
}

// Module (src/module.rs:12-24): forward + named parameters.
class Module {
public:
    virtual ~Module() = default;
    virtual Tensor forward(const Tensor &x) = 0;
};

// Linear (src/layers/basic/linear.rs): weight [out, in], optional bias.
class Linear : public Module {
public:
    explicit Linear(Tensor weight, Tensor bias = Tensor()) : weight(std::move(weight)), bias(std::move(bias)) {}
    Tensor forward(const Tensor &x) override {
        require_no_grad("Linear::forward");
        lumen_tensor *out = nullptr;
        check(lumen_linear_forward(x.context().get(), x.get(), weight.get(), bias ? bias.get() : nullptr, &out), x.context().get());
        return Tensor(x.context(), out);
    }
    Tensor weight, bias;
};

// RMSNorm (src/layers/norm/rms_norm.rs:24-62)
class RMSNorm : public Module {
public:
    RMSNorm(Tensor weight, float eps) : weight(std::move(weight)), eps(eps) {}
    Tensor forward(const Tensor &x) override {
        require_no_grad("RMSNorm::forward");
        lumen_tensor *out = nullptr;
        check(lumen_rmsnorm(x.context().get(), x.get(), weight.get(), eps, &out), x.context().get());
        return Tensor(x.context(), out);
    }
    Tensor weight;
    float eps;
};

// SiLU (src/layers/activation.rs:139-147)
class SiLU : public Module {
public:
    Tensor forward(const Tensor &x) override {
        require_no_grad("SiLU::forward");
        lumen_tensor *out = nullptr;
        check(lumen_silu(x.context().get(), x.get(), &out), x.context().get());
        return Tensor(x.context(), out);
    }
};

// Embedding (src/layers/basic/embedding.rs:21-57): ids are f32 token ids.
class Embedding : public Module {
public:
    explicit Embedding(Tensor table) : weight(std::move(table)) {}
    Tensor forward(const Tensor &ids) override {
        require_no_grad("Embedding::forward");
        lumen_tensor *out = nullptr;
        check(lumen_embedding(ids.context().get(), ids.get(), weight.get(), &out), ids.context().get());
        return Tensor(ids.context(), out);
    }
    Tensor weight;
};

// RotaryEmbedding (src/layers/attention/encoding.rs:17-123)
class RotaryEmbedding {
public:
    RotaryEmbedding(const Context &ctx, size_t dim, size_t max_seq_len, float theta) : ctx_(ctx) {
        lumen_rope *r = nullptr;
        check(lumen_rope_new(ctx.get(), dim, max_seq_len, theta, &r), ctx.get());
        h_.reset(r, [](lumen_rope *p) { lumen_rope_free(p); });
    }
    Tensor forward(const Tensor &x_bhsd, size_t offset) const {
        lumen_tensor *out = nullptr;
        check(lumen_rope_forward(h_.get(), x_bhsd.get(), offset, &out), ctx_.get());
        return Tensor(ctx_, out);
    }
    lumen_rope *get() const { return h_.get(); }

private:
    Context ctx_;
    std::shared_ptr<lumen_rope> h_;
};

// KVCacheInner / KVCache (src/layers/attention/self_attention.rs:24-44): [B, Hkv, max_seq, D] slabs + len.
class KVCache {
public:
    KVCache() = default;
    KVCache(const Context &ctx, size_t b, size_t h_kv, size_t max_seq, size_t d) : ctx_(ctx) {
        lumen_kv_cache *c = nullptr;
        check(lumen_kv_new(ctx.get(), b, h_kv, max_seq, d, &c), ctx.get());
        h_.reset(c, [](lumen_kv_cache *p) { lumen_kv_free(p); });
    }
    KVCache(const Context &ctx, lumen_kv_cache *owned) : ctx_(ctx), h_(owned, [](lumen_kv_cache *p) { lumen_kv_free(p); }) {}
    void reset() { check(lumen_kv_reset(get()), ctx_.get()); }  // self_attention.rs:41-43
    size_t len() const { return lumen_kv_len(get()); }
    lumen_kv_cache *get() const { return h_.get(); }
    explicit operator bool() const { return (bool)h_; }

private:
    Context ctx_{};
    std::shared_ptr<lumen_kv_cache> h_;
};

// LlamaKVCache (src/kv_cache.rs:14-59)
class LlamaKVCache {
public:
    LlamaKVCache(const Context &ctx, size_t kv_heads, size_t max_seq_len, size_t head_dim) : ctx_(ctx) {
        lumen_llama_kv_cache *c = nullptr;
        check(lumen_llama_kv_new(ctx.get(), kv_heads, max_seq_len, head_dim, &c), ctx.get());
        h_.reset(c, [](lumen_llama_kv_cache *p) { lumen_llama_kv_free(p); });
    }
    void update(const Tensor &k, const Tensor &v, size_t start_pos) {
        check(lumen_llama_kv_update(h_.get(), k.get(), v.get(), start_pos), ctx_.get());
    }
    std::pair<Tensor, Tensor> get_view(size_t current_len) const {
        lumen_tensor *k = nullptr, *v = nullptr;
        check(lumen_llama_kv_get_view(h_.get(), current_len, &k, &v), ctx_.get());
        return {Tensor(ctx_, k), Tensor(ctx_, v)};
    }

private:
    Context ctx_;
    std::shared_ptr<lumen_llama_kv_cache> h_;
};

// SelfAttention (src/layers/attention/self_attention.rs:46-306): forward(x, Option<KVCache>) -> (out, cache)
class SelfAttention {
public:
    SelfAttention(const Context &ctx, size_t embed_dim, size_t n_head, size_t n_kv_head, size_t max_seq_len, float rope_theta,
                  bool causal)
        : ctx_(ctx) {
        lumen_self_attention *a = nullptr;
        check(lumen_self_attention_new(ctx.get(), embed_dim, n_head, n_kv_head, max_seq_len, rope_theta, causal ? 1 : 0, &a), ctx.get());
        h_.reset(a, [](lumen_self_attention *p) { lumen_self_attention_free(p); });
    }
    void set_weight(int which, const Tensor &w) { check(lumen_self_attention_set_weight(h_.get(), which, w.get()), ctx_.get()); }
    std::pair<Tensor, KVCache> forward(const Tensor &x, KVCache cache = KVCache()) {
        require_no_grad("SelfAttention::forward");
        lumen_tensor *out = nullptr;
        lumen_kv_cache *used = nullptr;
        check(lumen_self_attention_forward(h_.get(), x.get(), cache ? cache.get() : nullptr, &out, &used), ctx_.get());
        if (!cache) cache = KVCache(ctx_, used);  // created by the call (self_attention.rs:119-122): now ours
        return {Tensor(ctx_, out), cache};
    }

private:
    Context ctx_;
    std::shared_ptr<lumen_self_attention> h_;
};

// LlamaConfig (src/models/llama.rs:11-37) + head_dim / qk_norm / weight_dtype extensions.
struct LlamaConfig {
    size_t vocab_size = 32000, hidden_size = 2048, intermediate_size = 5632, num_hidden_layers = 22;
    size_t num_attention_heads = 32, num_key_value_heads = 4;
    float rms_norm_eps = 1e-5f;
    size_t max_seq_len = 2048;
    float rope_theta = 10000.0f;
    size_t head_dim = 0;
    bool qk_norm = false;
    lumen_dtype weight_dtype = LUMEN_F32;
    lumen_llama_config to_c() const {
        lumen_llama_config c{};
        c.vocab_size = vocab_size; c.hidden_size = hidden_size; c.intermediate_size = intermediate_size;
        c.num_hidden_layers = num_hidden_layers; c.num_attention_heads = num_attention_heads;
        c.num_key_value_heads = num_key_value_heads; c.rms_norm_eps = rms_norm_eps; c.max_seq_len = max_seq_len;
        c.rope_theta = rope_theta; c.head_dim = head_dim; c.qk_norm = qk_norm ? 1 : 0; c.weight_dtype = weight_dtype;
        return c;
    }
};

// LlamaModel (src/models/llama.rs:129-216)
class LlamaModel {
public:
    LlamaModel(const Context &ctx, const LlamaConfig &config) : config(config), ctx_(ctx) {
        const lumen_llama_config c = config.to_c();
        lumen_llama *m = nullptr;
        check(lumen_llama_new(ctx.get(), &c, &m), ctx.get());
        h_.reset(m, [](lumen_llama *p) { lumen_llama_free(p); });
    }
    // What a loader does with named_parameters() (llama.rs:218-279, src/loader.rs:10-80): the full tensor by
    // its Hugging Face name; a tensor-parallel rank keeps its slice.
    void set_param(const std::string &name, const std::vector<size_t> &shape, const float *data) {
        check(lumen_llama_set_param(h_.get(), name.c_str(), data, shape.data(), (int)shape.size(), LUMEN_F32), ctx_.get());
    }
    void set_param_bf16(const std::string &name, const std::vector<size_t> &shape, const uint16_t *bits) {
        check(lumen_llama_set_param(h_.get(), name.c_str(), bits, shape.data(), (int)shape.size(), LUMEN_BF16), ctx_.get());
    }
    // init_kv_caches (llama.rs:161-169)
    std::vector<KVCache> init_kv_caches(size_t batch_size) const {
        std::vector<lumen_kv_cache *> raw(config.num_hidden_layers, nullptr);
        check(lumen_llama_init_kv_caches(h_.get(), batch_size, raw.data()), ctx_.get());
        std::vector<KVCache> out;
        out.reserve(raw.size());
        for (lumen_kv_cache *c : raw) out.emplace_back(ctx_, c);
        return out;
    }
    // reset_kv_caches (llama.rs:172-176)
    void reset_kv_caches(std::vector<KVCache> &caches) const {
        for (KVCache &c : caches) c.reset();
    }
    // forward(input_ids[B,S] as f32, caches, _pos) -> logits[B,S,V] (llama.rs:181-206); pos is ignored like
    // the reference's.
    std::vector<float> forward(const float *ids, size_t b, size_t s, std::vector<KVCache> &caches, size_t pos = 0) const {
        require_no_grad("LlamaModel::forward");
        std::vector<lumen_kv_cache *> raw;
        for (const KVCache &c : caches) raw.push_back(c.get());
        std::vector<float> logits(b * s * config.vocab_size);
        check(lumen_llama_forward(h_.get(), ids, b, s, raw.data(), raw.size(), pos, logits.data()), ctx_.get());
        return logits;
    }
    // Same, keeping only the last position's logits [B,V] (what the reference's caller uses, src/main.rs:155-163).
    std::vector<float> forward_last(const float *ids, size_t b, size_t s, std::vector<KVCache> &caches) const {
        require_no_grad("LlamaModel::forward_last");
        std::vector<lumen_kv_cache *> raw;
        for (const KVCache &c : caches) raw.push_back(c.get());
        std::vector<float> logits(b * config.vocab_size);
        check(lumen_llama_forward_last(h_.get(), ids, b, s, raw.data(), raw.size(), 0, logits.data()), ctx_.get());
        return logits;
    }
    size_t weight_bytes_per_step() const { return lumen_llama_weight_bytes(h_.get()); }
    LlamaConfig config;

private:
    Context ctx_;
    std::shared_ptr<lumen_llama> h_;
};

}  // namespace lumen_b200
