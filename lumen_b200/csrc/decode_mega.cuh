// Parameters of the whole-token persistent decode kernel (decode_mega.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace lumen {

// The ring: many small stages rather than few large ones.  A consumer warp holds the stage it works on, and a held
// stage is not in flight: with four warps at work, what bounds the streaming rate of an SM is (stages - 4) x stage
// bytes / memory latency.  One stage = four rows x 4 KB (rows longer than 4 KB are cut into segments).
constexpr int kMegaMaxStages = 13;
constexpr int kMegaStageBytes = 16 * 1024;

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
    float *logits;            // [V] (one GPU), or this rank's view of its own gathered logits [vocab] (tensor parallel)
    // Tensor parallelism: a rank stores its slice of the logits straight into every rank's gathered-logits area
    // (plain peer stores over NVLink), then raises its flag (the launch's tag) in every rank; the last CTA of a rank
    // to finish waits for all flags, so that when the kernel ends the rank's logits are complete.
    float *logits_peer[8];    // rank r's gathered logits [vocab] as seen from this device
    unsigned int *flag_peer[8];  // rank r's flag array [tp_size] as seen from this device
    unsigned int *done_count; // CTAs of this rank that have stored their logits rows (reset by the last one)
    // Activations that cross CTAs are exchanged as 8-byte {f32 bits, epoch tag} words: a consumer polls the
    // words it needs until they carry the tag of the producing phase, so the data is its own signal and no
    // grid barrier is needed.  tag(phase) = epoch_base + phase + 1; epoch_base grows with every launch.
    // Tensor parallelism: the o_proj and down outputs are partial sums over this rank's heads / intermediate
    // rows.  A rank stores its partial row values into slot tp_rank of EVERY rank's x buffer (plain peer
    // stores over NVLink; rank 0's partial carries the residual), and every CTA of every rank sums the
    // tp_size slots in rank order when it stages x: the all-reduce is part of the exchange the kernel does
    // anyway, and all ranks compute bit-identical sums.  Two buffers alternate between the two exchanges of a
    // layer so that a fast rank cannot overwrite a value a slow rank has not read yet.
    int tp_rank, tp_size;
    uint2 *x_peer[8];         // x_peer[r] = rank r's xT as seen from this device (x_peer[tp_rank] == xT)
    int x_slot_words;         // words per slot: H rounded up to even
    uint2 *xT;                // [2][tp_size][x_slot_words]  residual stream (o_proj -> buffer 0, down -> buffer 1)
    // Tensor parallelism with many ranks: summing tp_size slots while staging x takes tp_size times the loads of a
    // plain staging pass, in several passes (each a round trip through L2).  Instead the CTA that owns a row of the
    // residual stream sums the ranks' partial values of that row (in rank order, so every rank gets the same bits) and
    // publishes the sum in xrT; everybody then stages xrT in one pass like on a single GPU.
    uint2 *xrT;               // [2][x_slot_words] the summed residual stream (null: sum while staging)
    uint2 *qkvT;              // [qkv_rows]   q | k | v projections
    uint2 *actT;              // [I]          SiLU(gate) * up
    uint2 *partT;             // [Hq, nsplit, 2 + D]: {max}, {sum}, ctx[D] of every attention work item
    unsigned int epoch_base;
    int nsplit;
    int *abort_flag;
    DeviceStatus *status;
    int stages, stage_bytes;            // filled by the launcher
    // Optional trace written by CTA 0 (null = off); decode_mega_trace_words() 64-bit words, nph = 5L+1:
    //   [0, 3nph]        ns timestamps: start of each phase, after its prologue, after its last tile; then
    //                    one at the end of the token
    //   [3nph+1, +nph)   producer: ns timestamp of the first copy of each phase
    //   [4nph+1, +nph)   consumers: ns timestamp when the phase's input vector had arrived
    //   [5nph+1, +nph)   warp 0: clock cycles spent waiting for weight tiles of the phase
    //   [6nph+1, +nph)   warp 0: clock cycles spent on the tiles of the phase (loads, FMAs, reductions)
    //   [7nph+1, +512)   producer: ns timestamp of the issue of each of the first 512 tiles
    //   [7nph+513, +512) consumers: ns timestamp of the release of each of those tiles
    //   then, written by every CTA c < kMegaTraceCtas: [nph][kMegaTraceCtas] ns timestamp when the phase's input
    //   had arrived, and [nph][kMegaTraceCtas] ns timestamp when the CTA had published the phase's results
    unsigned long long *trace;
    // Producer schedule: for CTA c the bulk copies of one token in issue order, sched[c * sched_stride + i],
    // i < sched_count[c].  Entry = {src address lo, hi, copy bytes | phase << 16, tile bytes}; tile bytes is
    // non-zero on the first copy of a tile (= the transaction count of its stage) and 0 on the following ones.
    // The schedule depends only on the model's shapes and addresses, so it is built once on the host
    // (decode_mega_build_schedule) and the producer does no address arithmetic at all.
    // A copy is either a plain 1-D bulk copy, entry = {src address lo, hi, copy bytes | phase << 16, w},
    // or (bit 31 of w set) a 3-D tiled TMA copy of a box of rows x one segment of the row length out of a
    // row-major matrix, entry = {tensor map index | first 256-byte unit of the segment << 16, first row,
    // copy bytes | phase << 16, w}.  w = tile bytes (bits 0-15, non-zero on the first copy of a tile only) |
    // offset of the copy inside its ring stage / 16 (bits 16-27) | bit 31.  A segment tile of four rows is ONE box.
    const uint4 *sched;
    const int *sched_count;
    int sched_stride;
    const CUtensorMap *tmaps;  // device array of the tensor maps the schedule refers to (64-byte aligned)
    int l2_ahead;  // tiles the producer hands to the L2, one at a time, while the ring is full (0 = off)
    int pf_pace, pf_grace;  // cycles between two such prefetches, and how long the ring must have been full before the first
    // bit 0: stream no weight tiles (measures the exchange + prologue chain alone; results are wrong)
    // bit 2: wait for the weight tiles but skip the arithmetic on them
    // bit 3: the first phase publishes nothing: every wait on it gives up after its limit (time-out test)
    int debug_flags;
};

size_t decode_mega_smem_bytes(int stages, int stage_bytes, int head_dim, int kmax);
int decode_mega_supported(const MegaParams &p, char *why, size_t why_len);
unsigned int decode_mega_epochs_per_launch(int layers);
size_t decode_mega_exchange_words(const MegaParams &p);  // uint2 words of the four exchange buffers (+ gathered logits and flags)
size_t decode_mega_logits_offset_words(const MegaParams &p);  // where the gathered logits start (then tp_size flags)
size_t decode_mega_x_words(const MegaParams &p);         // of which the x buffers, at the start (needs tp_size, H)
int decode_mega_max_splits();
constexpr int kMegaTileTrace = 512;
constexpr int kMegaTraceCtas = 160;  // per-CTA part of the trace: [2][nph][kMegaTraceCtas] after the words above
__host__ __device__ inline size_t decode_mega_trace_base_words(size_t layers) { return 7 * (5 * layers + 1) + 1 + 2 * kMegaTileTrace; }
inline size_t decode_mega_trace_words(size_t layers) {
    return decode_mega_trace_base_words(layers) + 2 * (5 * layers + 1) * kMegaTraceCtas;
}
int decode_mega_debug_flags();  // from the environment (LUMEN_MEGA_DEBUG), read once
// Builds the producer schedule for `grid` CTAs from the shapes in p and the HOST copy of the layer table.
// entries.size() == grid * stride afterwards.
// tmaps receives the tensor maps of the matrices whose rows are cut into segments (two per matrix: a box of four
// rows and a box of one row); it stays empty when the driver offers no tensor-map encoder, and segments then
// arrive as one plain copy per row.
void decode_mega_build_schedule(const MegaParams &p, const MegaLayer *host_layers, int grid, std::vector<uint4> &entries,
                                std::vector<int> &counts, int &stride, std::vector<CUtensorMap> &tmaps);
int launch_decode_mega(lumen_ctx *ctx, MegaParams &p, cudaStream_t s);

}  // namespace lumen
