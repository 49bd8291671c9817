// Drives the C++ host mirror (include/lumen_b200.hpp) the way the reference's chat loop drives its model
// (src/main.rs:220-221, 334-336, 367-372): init_kv_caches(1) once, prefill with [1,S], then one
// forward([1,1]) per token.  Inputs come from files written by the test; logits go back to a file.
//
//   host_mirror_check <dir>      reads <dir>/cfg.txt, params.bin, ids.bin; writes <dir>/logits.bin
//   host_mirror_check --no-gpu   only checks that a missing device surfaces as lumen_b200::Error
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "lumen_b200.hpp"

namespace L = lumen_b200;

static std::vector<std::pair<std::string, std::vector<size_t>>> param_shapes(const L::LlamaConfig &c) {
    const size_t H = c.hidden_size, D = c.head_dim ? c.head_dim : H / c.num_attention_heads;
    std::vector<std::pair<std::string, std::vector<size_t>>> out;
    out.push_back({"model.embed_tokens.weight", {c.vocab_size, H}});
    for (size_t l = 0; l < c.num_hidden_layers; ++l) {
        const std::string p = "model.layers." + std::to_string(l) + ".";
        out.push_back({p + "self_attn.q_proj.weight", {c.num_attention_heads * D, H}});
        out.push_back({p + "self_attn.k_proj.weight", {c.num_key_value_heads * D, H}});
        out.push_back({p + "self_attn.v_proj.weight", {c.num_key_value_heads * D, H}});
        out.push_back({p + "self_attn.o_proj.weight", {H, c.num_attention_heads * D}});
        out.push_back({p + "mlp.gate_proj.weight", {c.intermediate_size, H}});
        out.push_back({p + "mlp.up_proj.weight", {c.intermediate_size, H}});
        out.push_back({p + "mlp.down_proj.weight", {H, c.intermediate_size}});
        out.push_back({p + "input_layernorm.weight", {H}});
        out.push_back({p + "post_attention_layernorm.weight", {H}});
    }
    out.push_back({"model.norm.weight", {H}});
    out.push_back({"lm_head.weight", {c.vocab_size, H}});
    return out;
}

static std::vector<float> read_floats(const std::string &path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) throw std::runtime_error("cannot open " + path);
    const std::streamsize n = f.tellg();
    f.seekg(0);
    std::vector<float> v((size_t)n / sizeof(float));
    f.read(reinterpret_cast<char *>(v.data()), n);
    return v;
}

int main(int argc, char **argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: host_mirror_check <dir> | --no-gpu\n");
        return 2;
    }
    if (!std::strcmp(argv[1], "--no-gpu")) {
        try {
            L::Context ctx(0);
            std::puts("context created");
        } catch (const L::Error &e) {
            std::printf("Error code=%d what=%s\n", e.code, e.what());
            return e.code == LUMEN_ERR_CUDA ? 0 : 1;
        }
        return 0;
    }
    try {
        const std::string dir = argv[1];
        L::LlamaConfig cfg;
        size_t prompt = 0, steps = 0;
        {
            std::ifstream f(dir + "/cfg.txt");
            if (!(f >> cfg.vocab_size >> cfg.hidden_size >> cfg.intermediate_size >> cfg.num_hidden_layers >> cfg.num_attention_heads >>
                  cfg.num_key_value_heads >> cfg.rms_norm_eps >> cfg.max_seq_len >> cfg.rope_theta >> prompt >> steps))
                throw std::runtime_error("bad cfg.txt");
        }
        const std::vector<float> params = read_floats(dir + "/params.bin");
        const std::vector<float> ids = read_floats(dir + "/ids.bin");
        L::Context ctx(0);
        L::LlamaModel model(ctx, cfg);
        size_t off = 0;
        for (const auto &ps : param_shapes(cfg)) {
            size_t n = 1;
            for (size_t d : ps.second) n *= d;
            if (off + n > params.size()) throw std::runtime_error("params.bin too short at " + ps.first);
            model.set_param(ps.first, ps.second, params.data() + off);
            off += n;
        }
        std::vector<L::KVCache> caches = model.init_kv_caches(1);
        std::vector<float> all;
        {
            // calling a module outside no_grad is refused: only the inference branches exist
            bool refused = false;
            try {
                model.forward(ids.data(), 1, prompt, caches);
            } catch (const L::Error &e) {
                refused = e.code == LUMEN_ERR_UNSUPPORTED;
            }
            if (!refused) throw std::runtime_error("forward outside no_grad was not refused");
        }
        {
            L::NoGradGuard guard;
            std::vector<float> lg = model.forward(ids.data(), 1, prompt, caches);  // prefill: logits [1,S,V]
            all.insert(all.end(), lg.end() - (std::ptrdiff_t)cfg.vocab_size, lg.end());
            for (size_t t = 0; t < steps; ++t) {  // teacher-forced decode, one [1,1] call per token
                lg = model.forward(ids.data() + prompt + t, 1, 1, caches);
                all.insert(all.end(), lg.begin(), lg.end());
            }
            if (caches[0].len() != prompt + steps) throw std::runtime_error("cache length mismatch");
            // KV overflow comes back as the reference's assert (self_attention.rs:144-149)
            model.reset_kv_caches(caches);
            if (caches[0].len() != 0) throw std::runtime_error("reset_kv_caches did not reset");
        }
        std::ofstream o(dir + "/logits.bin", std::ios::binary);
        o.write(reinterpret_cast<const char *>(all.data()), (std::streamsize)(all.size() * sizeof(float)));
        std::printf("ok %zu logits, %llu kernel launches\n", all.size(), (unsigned long long)ctx.launch_count());
        return 0;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "host_mirror_check failed: %s\n", e.what());
        return 1;
    }
}
