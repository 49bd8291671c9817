// Parameters of the whole-token persistent decode kernel (decode_mega.cu).
#pragma once

#include "common.cuh"

namespace lumen {

constexpr int kMegaMaxStages = 7;

struct MegaLayer {
    const char *wqkv, *wo, *wgate, *wup, *wdown;  // [rows, K] row-major, f32 or bf16
    const float *norm1, *norm2, *qn, *kn;         // RMSNorm gains (qn/kn may be null)
    float *k_cache, *v_cache;                     // [1, Hkv, max_seq, D]
    int *d_len;                                   // device copy of the cache length
};

struct MegaParams {
    const MegaLayer *layers;  // device array [L]
    int L, H, I, V, vocab, Hq, Hkv, D, qkv_rows, qd, kvd, max_seq;  // V = lm_head rows on this rank
    int wbf16;
    const char *embed;        // [vocab, H]
    const float *final_norm;
    const char *lm_head;      // [V, H]
    const float *cos_t, *sin_t;
    float eps, scale;
    const float *ids;         // [1] f32 token id
    float *x, *qkv, *act, *logits;
    float *part_m, *part_l, *part_ctx;  // attention partials [Hq, nsplit], [Hq, nsplit], [Hq, nsplit, D]
    int nsplit;
    unsigned long long *bar_counter;    // monotonically increasing arrival counter of the grid barrier
    unsigned long long bar_base;        // its value when this launch starts
    int *abort_flag;
    DeviceStatus *status;
    int stages, stage_bytes;            // filled by the launcher
    // Optional trace: CTA 0 stores a nanosecond timestamp at the start of each phase, after its prologue
    // and after its last tile (3 per phase), then one at the end.  Null = off.
    unsigned long long *trace;
};

size_t decode_mega_smem_bytes(int stages, int stage_bytes, int head_dim);
int decode_mega_supported(const MegaParams &p, char *why, size_t why_len);
int decode_mega_barriers_per_launch(int layers);
int decode_mega_max_splits();
int launch_decode_mega(lumen_ctx *ctx, MegaParams &p, cudaStream_t s);

}  // namespace lumen
