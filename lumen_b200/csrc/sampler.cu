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

// One warp: walks the sorted probabilities in chunks staged through shared memory; lane 0 adds them
// sequentially (the reference's rounding), first to find the cut, then to find the drawn token.
__global__ void __launch_bounds__(32)
sample_pick_kernel(const float *__restrict__ sorted_p, const int *__restrict__ sorted_i, int n, float top_p, float r,
                   int *__restrict__ token_out) {
    constexpr int kChunk = 1024;
    __shared__ float buf[kChunk];
    __shared__ int s_cut, s_done;
    __shared__ float s_cum;
    const int lane = threadIdx.x;
    const float target = fmaxf(fminf(fmaxf(top_p, 0.f), 1.f), 1e-6f);
    if (lane == 0) {
        s_cut = 0;
        s_done = 0;
        s_cum = 0.f;
    }
    __syncwarp();
    for (int base = 0; base < n && !s_done; base += kChunk) {
        const int m = min(kChunk, n - base);
        for (int i = lane; i < m; i += 32) buf[i] = sorted_p[base + i];
        __syncwarp();
        if (lane == 0) {
            float cum = s_cum;
            int cut = s_cut;
            for (int i = 0; i < m; ++i) {
                cum = __fadd_rn(cum, buf[i]);
                cut = base + i + 1;
                if (cum >= target) {
                    s_done = 1;
                    break;
                }
            }
            s_cum = cum;
            s_cut = cut;
        }
        __syncwarp();
    }
    const int cut = max(s_cut, 1);
    const float cumulative = s_cum;
    if (lane == 0) s_done = 0;
    __shared__ int s_pick;
    __shared__ float s_acc;
    if (lane == 0) {
        s_pick = cut - 1;  // `*idxs.last()` when the walk never reaches r
        s_acc = 0.f;
    }
    __syncwarp();
    for (int base = 0; base < cut && !s_done; base += kChunk) {
        const int m = min(kChunk, cut - base);
        for (int i = lane; i < m; i += 32) buf[i] = sorted_p[base + i];
        __syncwarp();
        if (lane == 0) {
            float acc = s_acc;
            for (int i = 0; i < m; ++i) {
                acc = __fadd_rn(acc, __fdiv_rn(buf[i], cumulative));
                if (r <= acc) {
                    s_pick = base + i;
                    s_done = 1;
                    break;
                }
            }
            s_acc = acc;
        }
        __syncwarp();
    }
    if (lane == 0) *token_out = sorted_i[s_pick];
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
    void *ws = nullptr;
    LUMEN_TRY(dev_alloc(ctx, bytes, &ws));
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
        sample_pick_kernel<<<1, 32, 0, s>>>(probs_sorted, idx_sorted, n, top_p, r, token_dev);
        e = cudaGetLastError();
        if (e == cudaSuccess) ctx->launches += 1;
    }
    if (e != cudaSuccess) rc = cuda_fail(ctx, e, "sample_top_p");
    int rc2 = dev_free(ctx, ws);
    return rc != LUMEN_OK ? rc : rc2;
}

}  // namespace lumen
