// Internal definitions shared by the kernels and the C-ABI layer of lumen_b200.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/lumen_b200.h"

namespace lumen {

constexpr int kNumSMsFallback = 148;

// Device-side status word: kernels never trap; they record the first problem here and the host
// reads it at the next synchronising call.
struct DeviceStatus {
    int code;      // LUMEN_* code, 0 = ok
    int detail0;   // kernel-specific (e.g. the offending index)
    int detail1;
    int pad;
};

}  // namespace lumen

struct lumen_ctx {
    int device = 0;
    int tp_rank = 0;
    int tp_size = 1;
    int num_sms = lumen::kNumSMsFallback;
    cudaStream_t stream = nullptr;
    void *nccl_comm = nullptr;  // ncclComm_t when tp_size > 1
    lumen::DeviceStatus *d_status = nullptr;
    lumen::DeviceStatus *h_status = nullptr;  // pinned mirror
    char err[512] = {0};
    unsigned long long launches = 0;  // kernels enqueued so far (graph replays add their node count)
    // Persistent decode kernel: 16 device bytes whose second word is the cross-CTA abort flag, and the
    // epoch from which the next launch derives the tags of its exchanged activations.
    unsigned long long *d_mega_sync = nullptr;
    unsigned int mega_epoch = 1;
    // Counts the device-side aborts the host has read (check_device_status).  A kernel that gave up did not
    // advance the device copy of the cache lengths although the host mirror was bumped at enqueue time, so
    // every cache re-reads its device length the first time it is used after an abort (kv_resync_len).
    unsigned int abort_gen = 0;
    // Tagged activation exchange buffers of the persistent kernel.  They belong to the context, not to a model: with
    // tensor parallelism every rank maps every other rank's buffer (CUDA IPC), and a mapping outlives the model that
    // asked for it.  Models on one context run one after the other on its stream and share the buffer.
    void *d_exchange = nullptr;
    size_t exchange_bytes = 0;
    void *x_peers[8] = {nullptr};  // every rank's d_exchange as seen from this device (x_peers[tp_rank] == d_exchange)
    // Buffer of the fused tensor-parallel row sum (control words, flags, two sets of per-rank slots), mapped by every
    // rank like d_exchange; fixed size, allocated once per context.
    void *d_tp_sum = nullptr;
    void *tp_sum_peers[8] = {nullptr};
    void *sampler_ws = nullptr;    // scratch of the device sampler (probabilities, indices, sort space)
    size_t sampler_ws_bytes = 0;
};

struct lumen_storage {
    void *ptr = nullptr;
    size_t bytes = 0;
    int refs = 1;
    lumen_ctx *ctx = nullptr;
};

struct lumen_tensor {
    lumen_ctx *ctx = nullptr;
    lumen_storage *st = nullptr;
    size_t offset_bytes = 0;
    std::vector<size_t> shape;
    lumen_dtype dtype = LUMEN_F32;
    size_t numel() const {
        size_t n = 1;
        for (size_t s : shape) n *= s;
        return n;
    }
    void *data() const { return st ? static_cast<char *>(st->ptr) + offset_bytes : nullptr; }
    size_t elem_size() const { return dtype == LUMEN_F32 ? 4 : 2; }
};

struct lumen_rope {
    lumen_ctx *ctx = nullptr;
    size_t dim = 0, max_seq = 0;
    float theta = 0.f;
    float *cos_t = nullptr;  // [max_seq, dim/2]: both halves of the reference table hold the same value
    float *sin_t = nullptr;
};

struct lumen_kv_cache {
    lumen_ctx *ctx = nullptr;
    size_t b = 0, h_kv = 0, max_seq = 0, d = 0;
    size_t len = 0;        // host mirror of the cache length
    int *d_len = nullptr;  // device copy read by replayable kernels
    float *k = nullptr;    // [B,Hkv,max_seq,D]
    float *v = nullptr;
    unsigned int seen_abort = 0;  // ctx->abort_gen at the last time `len` was known to equal *d_len
    bool owns_slab = true;  // false when carved out of a model-wide slab
    lumen_storage *slab = nullptr;  // shared slab (reference counted) when !owns_slab
};

namespace lumen {

int set_error(lumen_ctx *ctx, int code, const char *fmt, ...);
int cuda_fail(lumen_ctx *ctx, cudaError_t e, const char *what);

#define LUMEN_CUDA(ctx, call)                                         \
    do {                                                              \
        cudaError_t e__ = (call);                                     \
        if (e__ != cudaSuccess) return lumen::cuda_fail((ctx), e__, #call); \
    } while (0)

// After every kernel launch: surface a launch error and count the launch.
#define LUMEN_LAUNCHED(ctx)                                                     \
    do {                                                                        \
        cudaError_t e__ = cudaGetLastError();                                   \
        if (e__ != cudaSuccess) return lumen::cuda_fail((ctx), e__, "kernel launch"); \
        (ctx)->launches += 1;                                                   \
    } while (0)

#define LUMEN_TRY(call)                 \
    do {                                \
        int rc__ = (call);              \
        if (rc__ != LUMEN_OK) return rc__; \
    } while (0)

int check_device_status(lumen_ctx *ctx);
// Brings the host mirror of a cache's length back in line with the device copy after a device-side abort
// (one 4-byte synchronising read, only on the first use after the abort).
int kv_resync_len(lumen_kv_cache *c);

// What a row-parallel product (o_proj, down) of a tensor-parallel rank asks for behind its own sum: the sum over the
// ranks, in rank order, of (product + residual), written to `out` on every rank, and optionally the RMSNorm of the summed
// rows (gains norm_w) written to `normed`.
struct TpSumArgs {
    float *out = nullptr;
    const float *norm_w = nullptr;
    float *normed = nullptr;
    float eps = 0.f;
    __nv_bfloat16 *next_hi = nullptr, *next_lo = nullptr;  // bf16 hi/lo split of RMSNorm(sum) for a tensor-core product that follows
};

// y[M,N] = a[M,K] . w[N,K]^T (+ residual): vector-matrix kernel for M <= 8, tiled GEMM otherwise.  With `tp` (and
// tp_size > 1) y becomes the sum over the ranks: fused into one kernel over peer memory when the rows fit its buffer
// (launch_tp_sum), through NCCL otherwise; tp->out must be y.
int matmul_dispatch(lumen_ctx *ctx, const float *a, const void *w, lumen_dtype wdt, float *y, size_t M, size_t K,
                    size_t N, const float *residual, cudaStream_t s, const TpSumArgs *tp = nullptr);
// cos/sin tables [max_seq, dim/2] computed on the host in f32.
int rope_tables_host(size_t dim, size_t max_seq, float theta, std::vector<float> &cos_h, std::vector<float> &sin_h);

// Tensor parallelism over NCCL (loaded with dlopen so the library has no link-time NCCL dependency).
int tp_init(lumen_ctx *ctx, const void *unique_id);
void tp_shutdown(lumen_ctx *ctx);
int tp_allreduce_sum(lumen_ctx *ctx, float *buf, size_t n, cudaStream_t s);          // in place
int tp_allgather(lumen_ctx *ctx, const float *send, float *recv, size_t n_per_rank, cudaStream_t s);
// Maps a cudaMalloc'ed buffer of every rank into every rank (CUDA IPC, handles traded over NCCL):
// peers_out[r] = rank r's buffer as seen from this device.
int tp_share_buffer(lumen_ctx *ctx, void *local, void **peers_out);
// Closes the mappings of the other ranks' buffers made by tp_share_buffer.
void tp_unshare_buffer(lumen_ctx *ctx, void **peers);
// The context's exchange buffer with room for `bytes` (zeroed when (re)allocated; collective when tp_size > 1: every
// rank must ask for the same size at the same point).
int ensure_exchange(lumen_ctx *ctx, size_t bytes);

// Fused tensor-parallel row sum (tp_sum.cu).  Limits of one call: kTpSumMaxRows rows, kTpSumSlotFloats elements.
constexpr size_t kTpSumMaxRows = 512;
constexpr size_t kTpSumSlotFloats = (size_t)512 * 1024;  // 2 MB per rank and buffer
constexpr size_t kTpSumCtlBytes = 256;
// Allocates and shares the buffer (collective, synchronises; not inside a stream capture).  No-op when tp_size == 1.
int ensure_tp_sum(lumen_ctx *ctx);
bool tp_sum_usable(const lumen_ctx *ctx, size_t rows, size_t dim);
// out = sum over ranks of (sum over `splits` slices of part (+ residual)); see TpSumArgs.  part and residual may alias out.
int launch_tp_sum(lumen_ctx *ctx, const float *part, int splits, const float *residual, size_t rows, size_t dim,
                  const TpSumArgs &a, cudaStream_t s);

// Stream-ordered allocation from the device's default memory pool.
int dev_alloc(lumen_ctx *ctx, size_t bytes, void **out);
int dev_free(lumen_ctx *ctx, void *p);
int new_tensor(lumen_ctx *ctx, const size_t *shape, int ndim, lumen_dtype dt, lumen_tensor **out);

// ---- kernel launchers (all asynchronous on `s`) ---------------------------------------------

// y[m, n] = sum_k w[n, k] * x[m, k], m in [0, M), M <= 8.  w is [N,K] row-major f32 or bf16.
// Optional fusions used by the decode step:
//   norm_w != nullptr : x is RMS-normalised on the fly ((x*inv)*norm_w, rms over K) before the product
//   residual != nullptr: y += residual (same shape as y)
// ldy is the row stride of y/residual (>= N).
struct GemvArgs {
    const float *x = nullptr;   // [M, K]
    const void *w = nullptr;    // [N, K]
    lumen_dtype wdt = LUMEN_F32;
    float *y = nullptr;         // [M, ldy]
    int M = 1;
    size_t K = 0, N = 0, ldy = 0;
    const float *norm_w = nullptr;
    float norm_eps = 0.f;
    const float *residual = nullptr;
};
int launch_gemv_nk(lumen_ctx *ctx, const GemvArgs &a, cudaStream_t s);

// SwiGLU front half: out[m, i] = silu(w_gate[i,:] . xn[m,:]) * (w_up[i,:] . xn[m,:]), where xn is the
// RMS-normalised x when norm_w != nullptr.  w_gate/w_up are [I,K].
int launch_gemv_gate_up(lumen_ctx *ctx, const float *x, const void *w_gate, const void *w_up, lumen_dtype wdt,
                        float *out, int M, size_t K, size_t I, const float *norm_w, float norm_eps, cudaStream_t s);

// y[n] = sum_k w[k, n] * x[k]; w is [K,N] row-major.  Uses `scratch` (>= gemv_kn_scratch_bytes) for
// split-K partial sums.
size_t gemv_kn_scratch_bytes(size_t K, size_t N, int num_sms);                           // either weight type
size_t gemv_kn_scratch_bytes_for(size_t K, size_t N, lumen_dtype wdt, int num_sms);    // the plan of this weight type
int launch_gemv_kn(lumen_ctx *ctx, const float *x, const void *w, lumen_dtype wdt, float *y, size_t K, size_t N,
                   float *scratch, cudaStream_t s);

// C[M,N] = A[M,K] . W[N,K]^T, any M (f32 SIMT tiles; bf16 weights are widened on load).
// With `tp` usable for M x N the product leaves its result to launch_tp_sum (split-K slices included).
int launch_gemm_nk(lumen_ctx *ctx, const float *a, const void *w, lumen_dtype wdt, float *c, size_t M, size_t K,
                   size_t N, const float *residual, cudaStream_t s, const TpSumArgs *tp = nullptr);
// The same product on the tensor cores (tcgen05, accumulator in tensor memory) for M >= 2 (callers keep up to 8
// rows over f32 weights on the streaming kernel);
// launch_gemm_nk takes this path whenever gemm_tc_usable says so.
bool gemm_tc_usable(lumen_dtype wdt, size_t M, size_t K, size_t N, const void *w);
// Fusions around the tensor-core product inside a model step.  Input side: the activations arrive already split into
// bf16 hi + lo by the kernel that produced them (then `a` is not read).  Output side: the kernel that adds the split-K
// slices also produces what the next product reads (gemm_finish.cu):
//   kPostNorm    c = sum (+ residual); (next_hi, next_lo) = split of RMSNorm(c) * norm_w  (norm_w null: c only)
//   kPostSwiglu  the product ran over the concatenated gate and up weights (N = 2 * intermediate):
//                (next_hi, next_lo) = split of silu(c[:, :N/2]) * c[:, N/2:]; c is scratch for [M, N] floats
struct GemmFuse {
    enum Post { kPostNone = 0, kPostNorm = 1, kPostSwiglu = 2 };
    const __nv_bfloat16 *a_hi = nullptr, *a_lo = nullptr;
    const __nv_bfloat16 *w_hi = nullptr, *w_lo = nullptr;  // f32 weights split once by the model (else split on every call)
    Post post = kPostNone;
    const float *norm_w = nullptr;
    float eps = 0.f;
    __nv_bfloat16 *next_hi = nullptr, *next_lo = nullptr;
};
int launch_gemm_tc(lumen_ctx *ctx, const float *a, const void *w, lumen_dtype wdt, float *c, size_t M, size_t K, size_t N,
                   const float *residual, cudaStream_t s, const TpSumArgs *tp = nullptr, const GemmFuse *fuse = nullptr);
// hi = bf16(a), lo = bf16(a - hi), n elements (the operand form of the tensor-core product).
int launch_split_bf16(lumen_ctx *ctx, const float *a, __nv_bfloat16 *hi, __nv_bfloat16 *lo, size_t n, cudaStream_t s);
// Row finishers (gemm_finish.cu).  Rows of up to 8192 elements, a multiple of 8.
bool row_finish_usable(size_t dim);
// out = sum over `splits` slices of part (+ residual) (out may be null or alias part / residual); with gains also the bf16
// hi/lo split of RMSNorm(out).
int launch_sum_norm_split(lumen_ctx *ctx, const float *part, int splits, const float *residual, size_t rows, size_t dim, float *out,
                          const float *norm_w, float eps, __nv_bfloat16 *hi, __nv_bfloat16 *lo, cudaStream_t s);
// part: [splits][rows][2 * inter] (gate columns, then up columns) -> bf16 hi/lo split of silu(gate) * up, [rows, inter].
int launch_sum_swiglu_split(lumen_ctx *ctx, const float *part, int splits, size_t rows, size_t inter, __nv_bfloat16 *hi,
                            __nv_bfloat16 *lo, cudaStream_t s);

int launch_rmsnorm(lumen_ctx *ctx, const float *x, const float *w, float eps, float *out, size_t rows, size_t dim,
                   cudaStream_t s);
int launch_silu(lumen_ctx *ctx, const float *x, float *out, size_t n, cudaStream_t s);
int launch_silu_mul(lumen_ctx *ctx, const float *gate, const float *up, float *out, size_t n, cudaStream_t s);
// out = a (op) b, b broadcast with period nb (nb == n for same-shape).
int launch_binary(lumen_ctx *ctx, const float *a, const float *b, float *out, size_t n, size_t nb, int is_mul,
                  cudaStream_t s);
// ids are f32 token ids; an id >= vocab records LUMEN_ERR_EMBED_RANGE in the device status and writes zeros.
int launch_embedding(lumen_ctx *ctx, const float *ids, const void *table, lumen_dtype tdt, float *out, size_t n_ids,
                     size_t vocab, size_t dim, cudaStream_t s);
int launch_rope_forward(lumen_ctx *ctx, const float *x, float *out, size_t b, size_t h, size_t s_len, size_t d,
                        size_t offset, const float *cos_t, const float *sin_t, cudaStream_t s);
int launch_fused_softmax(lumen_ctx *ctx, const float *x, float *out, size_t rows_bh, size_t q, size_t k, float scale,
                         int causal, cudaStream_t s);

// Decode attention (S == 1).  q[B,Hq,D], k_new/v_new[B,Hkv,D] (strides given in floats between batch
// rows so that q/k/v may live in one fused projection buffer).  Position = *d_len (device) so the
// launch is replayable; writes the rotated k and v into the cache row, computes out[B,Hq,D] and
// (when bump_len) increments *d_len.  part is scratch of attn_decode_scratch_bytes().
struct AttnDecodeArgs {
    const float *q = nullptr, *k_new = nullptr, *v_new = nullptr;
    size_t q_stride = 0, kv_stride = 0;  // floats between consecutive batch rows
    float *k_cache = nullptr, *v_cache = nullptr;
    const int *d_len = nullptr;
    size_t B = 0, Hq = 0, Hkv = 0, D = 0, max_seq = 0;
    const float *cos_t = nullptr, *sin_t = nullptr;  // [rope_max, D/2] or nullptr (no rotation)
    const float *q_norm = nullptr, *k_norm = nullptr;  // per-head RMSNorm gains [D] or nullptr
    float norm_eps = 0.f;
    float scale = 0.f;
    float *out = nullptr;  // [B, Hq*D]
    float *part = nullptr;
    int max_splits = 1;  // splits of the context baked into the launch (>= 1)
    size_t len_hint = 0; // host's view of the context length, used to size the split count
};
size_t attn_decode_scratch_bytes(size_t B, size_t Hq, size_t D, int max_splits);
int attn_decode_pick_splits(size_t B, size_t Hkv, size_t len, int num_sms);
int launch_attn_decode(lumen_ctx *ctx, const AttnDecodeArgs &a, cudaStream_t s);
int launch_bump_len(lumen_ctx *ctx, int *d_len, int delta, cudaStream_t s);

// Prefill attention (S > 1): q[B,S,Hq*D] is rotated on the fly, k/v[B,S,Hkv*D] are rotated/copied
// into the cache at rows past..past+S first; out[B,S,Hq*D].
struct AttnPrefillArgs {
    const float *q = nullptr, *k = nullptr, *v = nullptr;
    size_t q_stride = 0, kv_stride = 0;  // floats between consecutive (b,s) rows
    float *k_cache = nullptr, *v_cache = nullptr;
    size_t past = 0, S = 0, B = 0, Hq = 0, Hkv = 0, D = 0, max_seq = 0;
    const float *cos_t = nullptr, *sin_t = nullptr;
    const float *q_norm = nullptr, *k_norm = nullptr;
    float norm_eps = 0.f;
    float scale = 0.f;
    int causal = 1;
    float *out = nullptr;
};
int launch_attn_prefill(lumen_ctx *ctx, const AttnPrefillArgs &a, cudaStream_t s);
// Tensor-core prefill attention (attn_prefill_tc.cu): q_rot holds the rotated queries [B, S, Hq, D] and the
// cache rows 0 .. past + S - 1 are already written.
bool attn_prefill_tc_usable(const AttnPrefillArgs &a);
int launch_attn_prefill_tc(lumen_ctx *ctx, const AttnPrefillArgs &a, const float *q_rot, cudaStream_t s);

// Nucleus sampling of one logits vector on the device (sampler.cu); *token_dev is a device int.
int launch_sample_top_p(lumen_ctx *ctx, const float *logits_dev, size_t vocab, float temperature, float top_p, float penalty,
                        const int *recent_host, size_t n_recent, float r, int *token_dev, cudaStream_t s);

// LlamaKVCache::update: dst[h, start+s, :] = src[h, s, :].
int launch_kv_slab_copy(lumen_ctx *ctx, const float *src, float *dst, size_t heads, size_t s_len, size_t d,
                        size_t dst_seq_stride_rows, size_t start, int to_slab, cudaStream_t s);

}  // namespace lumen
