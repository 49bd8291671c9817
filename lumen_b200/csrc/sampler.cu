// Nucleus sampling on the device: `sample_top_p` of the reference's chat loop (src/main.rs:74-137), so that
// one token id crosses PCIe per step instead of the logits vector.
//
// Same steps as the reference: repetition penalty over the recent tokens (one division per occurrence),
// temperature (floored at 1e-5), softmax with 1/(sum + 1e-9), stable descending sort, nucleus cut at the
// first rank where the cumulative probability reaches top_p (clamped to [1e-6, 1]), inverse-CDF walk over
// probs[i] / cumulative with the caller's uniform draw.  The cumulative sums are added sequentially in f32 like
// the reference's loops; the softmax denominator is a tree sum (the reference adds it sequentially), which
// moves every probability by the same last-ulp factor and the result only when the draw sits on a boundary.
// The sort is cub::DeviceRadixSort (a library sort: this is not a hot loop).
#include <cub/cub.cuh>

#include "common.cuh"

namespace lumen {
namespace {

constexpr int kPrepThreads = 1024;
constexpr int kMaxRecent = 256;  // the reference keeps a window of 96 tokens (src/main.rs:300-313)

__device__ __forceinline__ float block_reduce(float v, float *red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float t = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? fmaxf(v, t) : v + t;
    }
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float x = lane < (int)(blockDim.x >> 5) ? red[lane] : (is_max ? -INFINITY : 0.f);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float t = __shfl_xor_sync(0xffffffffu, x, o);
            x = is_max ? fmaxf(x, t) : x + t;
        }
        if (lane == 0) red[32] = x;
    }
    __syncthreads();
    const float out = red[32];
    __syncthreads();
    return out;
}

// One CTA: probabilities of the adjusted logits and the identity permutation.
__global__ void __launch_bounds__(kPrepThreads)
sample_prep_kernel(const float *__restrict__ logits, int n, float temperature, float penalty, const int *__restrict__ recent,
                   int n_recent, float *__restrict__ probs, int *__restrict__ idx) {
    __shared__ float red[33];
    __shared__ int rec[kMaxRecent];
    const int tid = threadIdx.x;
    for (int i = tid; i < n; i += kPrepThreads) probs[i] = logits[i];
    for (int i = tid; i < n_recent; i += kPrepThreads) rec[i] = recent[i];
    __syncthreads();
    if (penalty > 1.0f && tid < n_recent) {
        // the first occurrence of a token applies one division per occurrence (main.rs:83-89)
        const int t = rec[tid];
        bool first = t >= 0 && t < n;
        for (int k = 0; k < tid && first; ++k) first = rec[k] != t;
        if (first) {
            float x = probs[t];
            for (int k = tid; k < n_recent; ++k)
                if (rec[k] == t) x = __fdiv_rn(x, penalty);
            probs[t] = x;
        }
    }
    __syncthreads();
    const float temp = fmaxf(temperature, 1e-5f);
    float mx = -INFINITY;
    for (int i = tid; i < n; i += kPrepThreads) {
        const float x = __fdiv_rn(probs[i], temp);
        probs[i] = x;
        mx = fmaxf(mx, x);
    }
    mx = block_reduce(mx, red, true);
    float sum = 0.f;
    for (int i = tid; i < n; i += kPrepThreads) {
        const float e = expf(__fsub_rn(probs[i], mx));
        probs[i] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);
    const float inv = __fdiv_rn(1.0f, __fadd_rn(sum, 1e-9f));
    for (int i = tid; i < n; i += kPrepThreads) {
        probs[i] = __fmul_rn(probs[i], inv);
        idx[i] = i;
    }
}

// The reference adds the sorted probabilities one by one in f32 and stops at the first index where the
// running sum reaches a threshold (main.rs:113-121 and :126-134).  With a flat distribution the rounding of
// that sequential sum decides the index, so the order of the additions is kept: one thread adds the values in
// order, 32 per test of the threshold (the block of 32 that crosses is then walked value by value), reading them
// from shared memory, while the other three warps of the CTA stage the next 2048 values into the other half of a
// double buffer (dividing by `scale` on the way: 1 for the cumulative probability, the nucleus mass for the
// inverse-CDF walk).  What the walk costs is then the dependent chain of additions alone.  Returns the first
// index < n whose running sum is >= threshold (n if none) and that running sum (the total if none).
constexpr int kPickThreads = 128;
constexpr int kPickChunk = 2048;

struct PickShared {
    __align__(16) float buf[2][kPickChunk];
    int found;
    float run;
};

__device__ __forceinline__ void stage_chunk(const float *__restrict__ vals, int n, int c0, float scale, float *dst, int first, int step) {
    const int m = min(kPickChunk, n - c0);
    for (int i = first; i < kPickChunk; i += step) dst[i] = i < m ? __fdiv_rn(vals[c0 + i], scale) : 0.f;  // zeros change no sum
}

__device__ __forceinline__ int first_reaching(const float *__restrict__ vals, int n, float scale, float threshold, PickShared &sh,
                                              float *sum_out) {
    const int tid = threadIdx.x;
    stage_chunk(vals, n, 0, scale, sh.buf[0], tid, kPickThreads);
    if (tid == 0) {
        sh.found = n;
        sh.run = 0.f;
    }
    __syncthreads();
    const int chunks = (n + kPickChunk - 1) / kPickChunk;
    for (int c = 0; c < chunks; ++c) {
        if (tid >= 32) {
            if (c + 1 < chunks) stage_chunk(vals, n, (c + 1) * kPickChunk, scale, sh.buf[(c + 1) & 1], tid - 32, kPickThreads - 32);
        } else if (tid == 0) {
            const float *buf = sh.buf[c & 1];
            const int c0 = c * kPickChunk, m = min(kPickChunk, n - c0);
            float run = sh.run;
            int found = n;
            // 32 values per test of the threshold: eight 128-bit loads, then the dependent chain of 32 additions
            for (int i = 0; i < m; i += 32) {
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = *reinterpret_cast<const float4 *>(buf + i + 4 * j);
                float t = run;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    t = __fadd_rn(t, v[j].x);
                    t = __fadd_rn(t, v[j].y);
                    t = __fadd_rn(t, v[j].z);
                    t = __fadd_rn(t, v[j].w);
                }
                if (t >= threshold) {  // the sums only grow: the crossing is inside these 32 (or in their zero padding)
                    for (int j = 0; j < 32 && i + j < m; ++j) {
                        run = __fadd_rn(run, buf[i + j]);
                        if (run >= threshold) {
                            found = c0 + i + j;
                            break;
                        }
                    }
                    if (found != n) break;
                    continue;  // (only zero padding was left: t == run, and that was below the threshold)
                }
                run = t;
            }
            sh.run = run;
            sh.found = found;
        }
        __syncthreads();
        const int f = sh.found;
        __syncthreads();  // everybody has read the word before the walker writes it again
        if (f != n) break;
    }
    const int found = sh.found;
    *sum_out = sh.run;
    __syncthreads();  // the buffers and the two words are reused by the next walk
    return found;
}

__global__ void __launch_bounds__(kPickThreads)
sample_pick_kernel(const float *__restrict__ sorted_p, const int *__restrict__ sorted_i, int n, float top_p, float r,
                   int *__restrict__ token_out) {
    __shared__ PickShared sh;
    const float target = fmaxf(fminf(fmaxf(top_p, 0.f), 1.f), 1e-6f);
    float cumulative;
    const int at = first_reaching(sorted_p, n, 1.0f, target, sh, &cumulative);  // main.rs:113-121
    const int cut = max(1, min(n, at + 1));
    float acc;
    // main.rs:126-134: acc += probs[i] / cumulative; the first i with r <= acc, else the last of the nucleus
    const int pick = first_reaching(sorted_p, cut, cumulative, r, sh, &acc);
    if (threadIdx.x == 0) *token_out = sorted_i[min(pick, cut - 1)];
}

}  // namespace

// logits_dev[vocab] -> *token_dev (device int).  Asynchronous on `s`.
int launch_sample_top_p(lumen_ctx *ctx, const float *logits_dev, size_t vocab, float temperature, float top_p, float penalty,
                        const int *recent_host, size_t n_recent, float r, int *token_dev, cudaStream_t s) {
    if (vocab == 0 || vocab > (size_t)1 << 30) return set_error(ctx, LUMEN_ERR_SHAPE, "sample: vocabulary of %zu", vocab);
    if (n_recent > (size_t)kMaxRecent) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "sample: %zu recent tokens, at most %d", n_recent, kMaxRecent);
    const int n = (int)vocab;
    size_t sort_bytes = 0;
    cub::DeviceRadixSort::SortPairsDescending(nullptr, sort_bytes, (const float *)nullptr, (float *)nullptr, (const int *)nullptr,
                                              (int *)nullptr, n, 0, 32, s);
    const size_t nf = ((size_t)n + 63) & ~(size_t)63;
    const size_t bytes = 4 * nf * 4 + kMaxRecent * sizeof(int) + ((sort_bytes + 255) & ~(size_t)255);
    // scratch kept with the context (grown when a larger vocabulary comes along): no allocation per token
    if (ctx->sampler_ws_bytes < bytes) {
        LUMEN_CUDA(ctx, cudaStreamSynchronize(s));
        if (ctx->sampler_ws) cudaFree(ctx->sampler_ws);
        ctx->sampler_ws = nullptr;
        ctx->sampler_ws_bytes = 0;
        LUMEN_CUDA(ctx, cudaMalloc(&ctx->sampler_ws, bytes));
        ctx->sampler_ws_bytes = bytes;
    }
    void *ws = ctx->sampler_ws;
    float *probs = static_cast<float *>(ws), *probs_sorted = probs + nf;
    int *idx = reinterpret_cast<int *>(probs_sorted + nf), *idx_sorted = idx + nf;
    int *recent_dev = idx_sorted + nf;
    void *sort_ws = recent_dev + kMaxRecent;
    int rc = LUMEN_OK;
    cudaError_t e = cudaSuccess;
    if (n_recent) e = cudaMemcpyAsync(recent_dev, recent_host, n_recent * sizeof(int), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) {
        sample_prep_kernel<<<1, kPrepThreads, 0, s>>>(logits_dev, n, temperature, penalty, recent_dev, (int)n_recent, probs, idx);
        e = cudaGetLastError();
        if (e == cudaSuccess) ctx->launches += 1;
    }
    if (e == cudaSuccess)
        e = cub::DeviceRadixSort::SortPairsDescending(sort_ws, sort_bytes, probs, probs_sorted, idx, idx_sorted, n, 0, 32, s);
    if (e == cudaSuccess) {
        sample_pick_kernel<<<1, kPickThreads, 0, s>>>(probs_sorted, idx_sorted, n, top_p, r, token_dev);
        e = cudaGetLastError();
        if (e == cudaSuccess) ctx->launches += 1;
    }
    if (e != cudaSuccess) rc = cuda_fail(ctx, e, "sample_top_p");
    return rc;
}

}  // namespace lumen
