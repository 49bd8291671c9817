// Small per-token ops of the Llama path: RMSNorm, SiLU, add/mul, embedding gather, RoPE, the
// training-path fused softmax, and KV slab copies.  All are a few KB per token; they use explicit
// round-to-nearest mul/add intrinsics (no FMA contraction) so that element-wise results match the
// reference's separate f32 multiplies and adds bit for bit wherever no reduction is involved.
#include "common.cuh"

namespace lumen {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

template <int T>
__device__ float block_sum(float v, float *red) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < T / 32; ++w) t += red[w];
    __syncthreads();
    return t;
}
template <int T>
__device__ float block_max(float v, float *red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = -INFINITY;
#pragma unroll
    for (int w = 0; w < T / 32; ++w) t = fmaxf(t, red[w]);
    __syncthreads();
    return t;
}

// RMSNorm::forward — src/layers/norm/rms_norm.rs:49-56: rms = sqrt(ss/dim + eps); o = (x*inv)*w.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                      float eps, float *__restrict__ out, size_t dim) {
    __shared__ float red[8];
    const float *xr = x + (size_t)blockIdx.x * dim;
    float *o = out + (size_t)blockIdx.x * dim;
    float ss = 0.f;
    for (size_t i = threadIdx.x; i < dim; i += 256) ss = fmaf(xr[i], xr[i], ss);
    ss = block_sum<256>(ss, red);
    float rms = sqrtf(__fadd_rn(__fdiv_rn(ss, (float)dim), eps));
    float inv = __fdiv_rn(1.0f, rms);
    for (size_t i = threadIdx.x; i < dim; i += 256) o[i] = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
}

// SiLU::forward — src/layers/activation.rs:143-146.
__device__ __forceinline__ float silu1(float x) {
    float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
    return __fmul_rn(x, sig);
}
__global__ void silu_kernel(const float *__restrict__ x, float *__restrict__ out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = silu1(x[i]);
}
__global__ void silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ out,
                                size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(silu1(g[i]), u[i]);
}

// Tensor + Tensor / Tensor * Tensor — src/ops/arithmetic.rs:48-52, :105-109.
__global__ void binary_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                              size_t n, size_t nb, int is_mul) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float bv = b[nb == n ? i : i % nb];
    out[i] = is_mul ? __fmul_rn(a[i], bv) : __fadd_rn(a[i], bv);
}

// Embedding::forward — src/layers/basic/embedding.rs:47-57.  `as usize` on an f32 saturates:
// NaN and negatives become 0; an id >= vocab is the reference's panic -> status word + zeros.
template <typename TT>
__global__ void __launch_bounds__(256) embedding_kernel(const float *__restrict__ ids, const TT *__restrict__ table,
                                                        float *__restrict__ out, size_t vocab, size_t dim,
                                                        DeviceStatus *status) {
    const float f = ids[blockIdx.x];
    unsigned long long idx = (f != f || f <= 0.f) ? 0ull : (f >= 1.8e19f ? ~0ull : (unsigned long long)f);
    float *o = out + (size_t)blockIdx.x * dim;
    if (idx >= vocab) {
        if (threadIdx.x == 0 && atomicCAS(&status->code, 0, LUMEN_ERR_EMBED_RANGE) == 0) {
            status->detail0 = (int)blockIdx.x;
            status->detail1 = (int)min(idx, (unsigned long long)0x7fffffff);
        }
        for (size_t i = threadIdx.x; i < dim; i += 256) o[i] = 0.f;
        return;
    }
    const TT *row = table + idx * dim;
    for (size_t i = threadIdx.x; i < dim; i += 256) {
        if constexpr (sizeof(TT) == 4) o[i] = row[i];
        else o[i] = __bfloat162float(row[i]);
    }
}

// RotaryEmbedding::forward — src/layers/attention/encoding.rs:101-116: x[B,H,S,D] at positions
// offset..offset+S; out[j] = x1*c - x2*s; out[j+half] = x2*c + x1*s.  Tables are [max_seq, D/2].
__global__ void rope_forward_kernel(const float *__restrict__ x, float *__restrict__ out, size_t s_len, size_t d,
                                    size_t offset, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                    size_t total_pairs) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total_pairs) return;
    const size_t half = d / 2;
    size_t j = i % half, row = i / half;  // row indexes (b,h,s)
    size_t ss = row % s_len;
    float c = cos_t[(offset + ss) * half + j], sn = sin_t[(offset + ss) * half + j];
    float x1 = x[row * d + j], x2 = x[row * d + j + half];
    out[row * d + j] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, sn));
    out[row * d + j + half] = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn));
}

// ops::fused::fused_softmax forward — src/ops/fused.rs:45-80.  One CTA per (b,h,i) row.
__global__ void __launch_bounds__(256) fused_softmax_kernel(const float *__restrict__ x, float *__restrict__ out,
                                                            size_t q, size_t k, float scale, int masking) {
    __shared__ float red[8];
    const size_t row = blockIdx.x;
    const size_t i = row % q;
    const float *xr = x + row * k;
    float *o = out + row * k;
    const size_t lim = masking ? min(k, i + 1) : k;  // unmasked columns are j <= i
    float mx = -INFINITY;
    for (size_t j = threadIdx.x; j < lim; j += 256) mx = fmaxf(mx, __fmul_rn(xr[j], scale));
    mx = block_max<256>(mx, red);
    float sum = 0.f;
    for (size_t j = threadIdx.x; j < k; j += 256) {
        float e = 0.f;
        if (j < lim) {
            e = expf(__fsub_rn(__fmul_rn(xr[j], scale), mx));
            sum += e;
        }
        o[j] = e;
    }
    sum = block_sum<256>(sum, red);
    const float inv = __fdiv_rn(1.0f, __fadd_rn(sum, 1e-10f));
    for (size_t j = threadIdx.x; j < k; j += 256) o[j] = __fmul_rn(o[j], inv);
}

// LlamaKVCache::update / get_view — src/kv_cache.rs:31-59: rows of [heads, S, D] <-> [heads, max_seq, D].
__global__ void kv_slab_copy_kernel(const float *__restrict__ src, float *__restrict__ dst, size_t s_len, size_t d,
                                    size_t slab_rows, size_t start, int to_slab, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    size_t e = i % d, r = (i / d) % s_len, h = i / (d * s_len);
    size_t slab_idx = (h * slab_rows + start + r) * d + e;
    if (to_slab) dst[slab_idx] = src[i];
    else dst[i] = src[slab_idx];
}

__global__ void bump_len_kernel(int *len, int delta) { *len += delta; }

inline unsigned blocks(size_t n, int t) { return (unsigned)((n + t - 1) / t); }

}  // namespace

int launch_rmsnorm(lumen_ctx *ctx, const float *x, const float *w, float eps, float *out, size_t rows, size_t dim,
                   cudaStream_t s) {
    if (rows == 0) return LUMEN_OK;
    rmsnorm_kernel<<<(unsigned)rows, 256, 0, s>>>(x, w, eps, out, dim);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_silu(lumen_ctx *ctx, const float *x, float *out, size_t n, cudaStream_t s) {
    if (n == 0) return LUMEN_OK;
    silu_kernel<<<blocks(n, 256), 256, 0, s>>>(x, out, n);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_silu_mul(lumen_ctx *ctx, const float *gate, const float *up, float *out, size_t n, cudaStream_t s) {
    if (n == 0) return LUMEN_OK;
    silu_mul_kernel<<<blocks(n, 256), 256, 0, s>>>(gate, up, out, n);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_binary(lumen_ctx *ctx, const float *a, const float *b, float *out, size_t n, size_t nb, int is_mul,
                  cudaStream_t s) {
    if (n == 0) return LUMEN_OK;
    binary_kernel<<<blocks(n, 256), 256, 0, s>>>(a, b, out, n, nb, is_mul);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_embedding(lumen_ctx *ctx, const float *ids, const void *table, lumen_dtype tdt, float *out, size_t n_ids,
                     size_t vocab, size_t dim, cudaStream_t s) {
    if (n_ids == 0) return LUMEN_OK;
    if (tdt == LUMEN_F32)
        embedding_kernel<float><<<(unsigned)n_ids, 256, 0, s>>>(ids, static_cast<const float *>(table), out, vocab, dim,
                                                                 ctx->d_status);
    else
        embedding_kernel<__nv_bfloat16><<<(unsigned)n_ids, 256, 0, s>>>(
            ids, static_cast<const __nv_bfloat16 *>(table), out, vocab, dim, ctx->d_status);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_rope_forward(lumen_ctx *ctx, const float *x, float *out, size_t b, size_t h, size_t s_len, size_t d,
                        size_t offset, const float *cos_t, const float *sin_t, cudaStream_t s) {
    size_t pairs = b * h * s_len * (d / 2);
    if (pairs == 0) return LUMEN_OK;
    rope_forward_kernel<<<blocks(pairs, 256), 256, 0, s>>>(x, out, s_len, d, offset, cos_t, sin_t, pairs);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_fused_softmax(lumen_ctx *ctx, const float *x, float *out, size_t rows_bh, size_t q, size_t k, float scale,
                         int causal, cudaStream_t s) {
    size_t rows = rows_bh * q;
    if (rows == 0 || k == 0) return LUMEN_OK;
    fused_softmax_kernel<<<(unsigned)rows, 256, 0, s>>>(x, out, q, k, scale, (causal && q > 1) ? 1 : 0);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_kv_slab_copy(lumen_ctx *ctx, const float *src, float *dst, size_t heads, size_t s_len, size_t d,
                        size_t slab_rows, size_t start, int to_slab, cudaStream_t s) {
    size_t total = heads * s_len * d;
    if (total == 0) return LUMEN_OK;
    kv_slab_copy_kernel<<<blocks(total, 256), 256, 0, s>>>(src, dst, s_len, d, slab_rows, start, to_slab, total);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_bump_len(lumen_ctx *ctx, int *d_len, int delta, cudaStream_t s) {
    bump_len_kernel<<<1, 1, 0, s>>>(d_len, delta);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace lumen
