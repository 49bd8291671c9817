// Tensor-parallel shard plan (host arithmetic only); see tp_plan.cu.
#pragma once

#include <cstddef>

#include "../../include/lumen_b200.h"

namespace lumen {

// Heads, intermediate rows and vocabulary rows owned by one rank.
struct TpHeads {
    size_t hq_l = 0, q_head0 = 0;    // local query heads and the first one's global index
    size_t hkv_l = 0, kv_head0 = 0;  // local KV heads (a replicated head counts on every rank holding it)
    size_t inter_l = 0, inter0 = 0;
    size_t vocab_l = 0, vocab0 = 0;
};

// A rank's part of one parameter: rows [row0, row0+nrows) x columns [col0, col0+ncols) of the full
// [rows, cols] tensor (cols == 0: a vector of `rows` elements, always kept whole).
struct TpSlice {
    size_t rows = 0, cols = 0, row0 = 0, nrows = 0, col0 = 0, ncols = 0;
};

int tp_head_plan(const lumen_llama_config &cfg, size_t tp_size, size_t tp_rank, TpHeads &out);
// `layer` receives the layer index (-1 for model-level tensors) and `leaf` the name below the layer prefix.
int tp_param_slice(const lumen_llama_config &cfg, size_t tp_size, size_t tp_rank, const char *name, TpSlice &out,
                   long *layer, const char **leaf);

}  // namespace lumen
