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
    float *logits;            // [V]
    // Activations that cross CTAs are exchanged as 8-byte {f32 bits, epoch tag} words: a consumer polls the
    // words it needs until they carry the tag of the producing phase, so the data is its own signal and no
    // grid barrier is needed.  tag(phase) = epoch_base + phase + 1; epoch_base grows with every launch.
    uint2 *xT;                // [H]          residual stream (o_proj and down outputs)
    uint2 *qkvT;              // [qkv_rows]   q | k | v projections
    uint2 *actT;              // [I]          SiLU(gate) * up
    uint2 *partT;             // [Hq, nsplit, 2 + D]: {max}, {sum}, ctx[D] of every attention work item
    unsigned int epoch_base;
    int nsplit;
    int *abort_flag;
    DeviceStatus *status;
    int stages, stage_bytes;            // filled by the launcher
    // Optional trace: CTA 0 stores a nanosecond timestamp at the start of each phase, after its prologue
    // and after its last tile (3 per phase), then one at the end.  Null = off.
    unsigned long long *trace;
    int l2_ahead;  // tiles the producer's L2 prefetch cursor runs ahead of the shared-memory ring
    int debug_flags;  // bit 0: stream no weight tiles (measures the sync + prologue chain alone; results are wrong)
};

size_t decode_mega_smem_bytes(int stages, int stage_bytes, int head_dim, int kmax);
int decode_mega_supported(const MegaParams &p, char *why, size_t why_len);
unsigned int decode_mega_epochs_per_launch(int layers);
size_t decode_mega_exchange_words(const MegaParams &p);  // uint2 words of the four exchange buffers
int decode_mega_max_splits();
int launch_decode_mega(lumen_ctx *ctx, MegaParams &p, cudaStream_t s);

}  // namespace lumen
