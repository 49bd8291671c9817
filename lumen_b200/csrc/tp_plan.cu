// Tensor-parallel shard plan: which part of each named parameter a rank keeps.  Host arithmetic only (no
// CUDA call), shared by lumen_llama_new / lumen_llama_set_param and exported so that a host can plan its
// loads (and so that the plan can be checked without a GPU).
//
// Split (Megatron style, one exchange per block): q/k/v/gate/up by output rows - whole heads per rank, the
// KV cache goes with the KV heads - o/down by input columns (the columns produced by this rank's heads /
// intermediate rows), lm_head by vocabulary rows; norms and the embedding table are replicated.  With fewer
// KV heads than ranks each KV head is replicated on tp_size / Hkv consecutive ranks.
#include <cstdio>
#include <cstring>

#include "tp_plan.cuh"

namespace lumen {

int tp_head_plan(const lumen_llama_config &cfg, size_t T, size_t r, TpHeads &h) {
    const size_t Hq = cfg.num_attention_heads, Hkv = cfg.num_key_value_heads;
    if (T == 0 || r >= T) return LUMEN_ERR_INVALID;
    if (Hq == 0 || Hkv == 0 || Hq % T || cfg.intermediate_size % T || cfg.vocab_size % T) return LUMEN_ERR_UNSUPPORTED;
    h.hq_l = Hq / T;
    h.q_head0 = r * h.hq_l;
    if (Hkv % T == 0) {
        h.hkv_l = Hkv / T;
        h.kv_head0 = r * h.hkv_l;
    } else if (T % Hkv == 0) {
        h.hkv_l = 1;
        h.kv_head0 = r / (T / Hkv);
    } else {
        return LUMEN_ERR_UNSUPPORTED;
    }
    if (h.hq_l % h.hkv_l) return LUMEN_ERR_UNSUPPORTED;
    // every local q head must map to a local KV head: q head g uses KV head g / (Hq / Hkv)
    const size_t n_rep = Hq / Hkv;
    if (Hq % Hkv || h.q_head0 / n_rep < h.kv_head0 || (h.q_head0 + h.hq_l - 1) / n_rep >= h.kv_head0 + h.hkv_l)
        return LUMEN_ERR_UNSUPPORTED;
    h.inter_l = cfg.intermediate_size / T;
    h.inter0 = r * h.inter_l;
    h.vocab_l = cfg.vocab_size / T;
    h.vocab0 = r * h.vocab_l;
    return LUMEN_OK;
}

int tp_param_slice(const lumen_llama_config &cfg, size_t T, size_t r, const char *name, TpSlice &s, long *layer,
                   const char **leaf) {
    TpHeads h;
    int rc = tp_head_plan(cfg, T, r, h);
    if (rc != LUMEN_OK) return rc;
    const size_t H = cfg.hidden_size, V = cfg.vocab_size, I = cfg.intermediate_size;
    const size_t D = cfg.head_dim ? cfg.head_dim : H / cfg.num_attention_heads;
    const size_t Hq = cfg.num_attention_heads, Hkv = cfg.num_key_value_heads;
    auto whole = [&](size_t rows, size_t cols) { s = TpSlice{rows, cols, 0, rows, 0, cols}; };
    auto by_rows = [&](size_t rows, size_t cols, size_t r0, size_t n) { s = TpSlice{rows, cols, r0, n, 0, cols}; };
    auto by_cols = [&](size_t rows, size_t cols, size_t c0, size_t n) { s = TpSlice{rows, cols, 0, rows, c0, n}; };
    if (layer) *layer = -1;
    if (leaf) *leaf = name;
    if (!strcmp(name, "model.embed_tokens.weight")) { whole(V, H); return LUMEN_OK; }
    if (!strcmp(name, "model.norm.weight")) { whole(H, 0); return LUMEN_OK; }
    if (!strcmp(name, "lm_head.weight")) { by_rows(V, H, h.vocab0, h.vocab_l); return LUMEN_OK; }
    long li = -1;
    int consumed = 0;
    if (sscanf(name, "model.layers.%ld.%n", &li, &consumed) != 1 || consumed == 0 || li < 0 ||
        (size_t)li >= cfg.num_hidden_layers)
        return LUMEN_ERR_PARAM_NAME;
    const char *rest = name + consumed;
    if (layer) *layer = li;
    if (leaf) *leaf = rest;
    if (!strcmp(rest, "self_attn.q_proj.weight")) by_rows(Hq * D, H, h.q_head0 * D, h.hq_l * D);
    else if (!strcmp(rest, "self_attn.k_proj.weight") || !strcmp(rest, "self_attn.v_proj.weight"))
        by_rows(Hkv * D, H, h.kv_head0 * D, h.hkv_l * D);
    else if (!strcmp(rest, "self_attn.o_proj.weight")) by_cols(H, Hq * D, h.q_head0 * D, h.hq_l * D);
    else if (!strcmp(rest, "mlp.gate_proj.weight") || !strcmp(rest, "mlp.up_proj.weight")) by_rows(I, H, h.inter0, h.inter_l);
    else if (!strcmp(rest, "mlp.down_proj.weight")) by_cols(H, I, h.inter0, h.inter_l);
    else if (!strcmp(rest, "input_layernorm.weight") || !strcmp(rest, "post_attention_layernorm.weight")) whole(H, 0);
    else if (cfg.qk_norm && (!strcmp(rest, "self_attn.q_norm.weight") || !strcmp(rest, "self_attn.k_norm.weight"))) whole(D, 0);
    else return LUMEN_ERR_PARAM_NAME;
    return LUMEN_OK;
}

}  // namespace lumen

extern "C" int lumen_tp_param_slice(const lumen_llama_config *cfg, int tp_rank, int tp_size, const char *name,
                                    size_t out[6]) {
    if (!cfg || !name || !out || tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return LUMEN_ERR_INVALID;
    lumen::TpSlice s;
    int rc = lumen::tp_param_slice(*cfg, (size_t)tp_size, (size_t)tp_rank, name, s, nullptr, nullptr);
    if (rc != LUMEN_OK) return rc;
    out[0] = s.rows; out[1] = s.cols; out[2] = s.row0; out[3] = s.nrows; out[4] = s.col0; out[5] = s.ncols;
    return LUMEN_OK;
}
