// M = 1 (and small-M) vector-matrix kernels: y = W . x with W streamed once from HBM.
//
// Restates the M == 1 branch of ops::matmul::matmul (src/ops/matmul.rs:42-69 of the reference):
// one output element per weight row, f32 accumulation.  The reference sums in k order on one
// core; here a warp owns a row, every lane accumulates a strided slice with FMAs and the 32
// partial sums are combined by a shuffle tree, so results agree to rounding, not bitwise.
//
// Bandwidth design: each lane issues 128-bit streaming loads (ld.global.cs) and keeps
// kUnroll x kRowsPerWarp of them in flight; the activation vector is staged once per CTA in
// shared memory and read back as conflict-free 128-bit words.
#include <algorithm>

#include "common.cuh"

namespace lumen {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float4 ld_stream_f4(const float4 *p) { return __ldcs(p); }
__device__ __forceinline__ uint4 ld_stream_u4(const uint4 *p) { return __ldcs(p); }

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// Stage x[M,K] into shared memory, optionally RMS-normalised: xs = (x * inv_rms) * norm_w, which is
// the element the reference's RMSNorm produces (src/layers/norm/rms_norm.rs:49-56) before its Linear.
template <int MB>
__device__ void stage_x(float *xs, const float *__restrict__ x, int M, size_t K, const float *__restrict__ norm_w,
                        float eps, float *red /* [MB][kWarps] */) {
    const int tid = threadIdx.x;
    for (size_t i = tid; i < (size_t)MB * K; i += kThreads) {
        size_t m = i / K;
        xs[i] = (m < (size_t)M) ? x[i] : 0.f;
    }
    __syncthreads();
    if (norm_w == nullptr) return;
    const int lane = tid & 31, warp = tid >> 5;
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        float ss = 0.f;
        for (size_t k = tid; k < K; k += kThreads) {
            float v = xs[(size_t)m * K + k];
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) red[m * kWarps + warp] = ss;
    }
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        float ss = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) ss += red[m * kWarps + w];
        float rms = sqrtf(__fadd_rn(__fdiv_rn(ss, (float)K), eps));
        float inv = __fdiv_rn(1.0f, rms);
        for (size_t k = tid; k < K; k += kThreads) {
            float v = xs[(size_t)m * K + k];
            xs[(size_t)m * K + k] = __fmul_rn(__fmul_rn(v, inv), norm_w[k]);
        }
    }
    __syncthreads();
}

// Accumulate one row (`wrow`, K elements) against MB staged vectors.  Vector path needs K % VEC == 0
// and a 16-byte aligned row; otherwise the scalar path runs.
template <typename WT, int MB>
__device__ __forceinline__ void row_dot(const WT *__restrict__ wrow, const float *xs, size_t K, int lane, bool vec_ok,
                                        float (&acc)[MB]) {
    constexpr int kUnroll = 8;
    if constexpr (sizeof(WT) == 4) {
        if (vec_ok) {
            const float4 *w4 = reinterpret_cast<const float4 *>(wrow);
            const size_t n4 = K / 4;
            for (size_t base = 0; base < n4; base += 32 * kUnroll) {
                float4 wv[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    size_t i = base + (size_t)u * 32 + lane;
                    wv[u] = (i < n4) ? ld_stream_f4(w4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    size_t i = base + (size_t)u * 32 + lane;
                    if (i < n4) {
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            float4 xv = *reinterpret_cast<const float4 *>(xs + (size_t)m * K + i * 4);
                            acc[m] = fmaf(wv[u].x, xv.x, acc[m]);
                            acc[m] = fmaf(wv[u].y, xv.y, acc[m]);
                            acc[m] = fmaf(wv[u].z, xv.z, acc[m]);
                            acc[m] = fmaf(wv[u].w, xv.w, acc[m]);
                        }
                    }
                }
            }
            return;
        }
        for (size_t k = lane; k < K; k += 32) {
            float w = reinterpret_cast<const float *>(wrow)[k];
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[m] = fmaf(w, xs[(size_t)m * K + k], acc[m]);
        }
    } else {
        if (vec_ok) {
            const uint4 *w8 = reinterpret_cast<const uint4 *>(wrow);
            const size_t n8 = K / 8;
            for (size_t base = 0; base < n8; base += 32 * kUnroll) {
                uint4 wv[kUnroll];
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    size_t i = base + (size_t)u * 32 + lane;
                    wv[u] = (i < n8) ? ld_stream_u4(w8 + i) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    size_t i = base + (size_t)u * 32 + lane;
                    if (i < n8) {
#pragma unroll
                        for (int m = 0; m < MB; ++m) {
                            const float4 *xp = reinterpret_cast<const float4 *>(xs + (size_t)m * K + i * 8);
                            float4 x0 = xp[0], x1 = xp[1];
                            acc[m] = fmaf(bf16_lo(wv[u].x), x0.x, acc[m]);
                            acc[m] = fmaf(bf16_hi(wv[u].x), x0.y, acc[m]);
                            acc[m] = fmaf(bf16_lo(wv[u].y), x0.z, acc[m]);
                            acc[m] = fmaf(bf16_hi(wv[u].y), x0.w, acc[m]);
                            acc[m] = fmaf(bf16_lo(wv[u].z), x1.x, acc[m]);
                            acc[m] = fmaf(bf16_hi(wv[u].z), x1.y, acc[m]);
                            acc[m] = fmaf(bf16_lo(wv[u].w), x1.z, acc[m]);
                            acc[m] = fmaf(bf16_hi(wv[u].w), x1.w, acc[m]);
                        }
                    }
                }
            }
            return;
        }
        for (size_t k = lane; k < K; k += 32) {
            float w = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(wrow)[k]);
#pragma unroll
            for (int m = 0; m < MB; ++m) acc[m] = fmaf(w, xs[(size_t)m * K + k], acc[m]);
        }
    }
}

// RR rows of W against MB staged vectors at once: every 16 bytes of x read from shared memory feed RR rows, so
// the shared-memory traffic per weight byte is MB / RR instead of MB (with MB = 8 and one row at a time the
// kernel was bound by shared memory, not by HBM).  Vector path only (K % VEC == 0, 16-byte aligned rows).
template <typename WT, int MB, int RR>
__device__ __forceinline__ void rows_dot(const WT *const (&rows)[RR], const float *xs, size_t K, int lane, float (&acc)[RR][MB]) {
    constexpr int VEC = 16 / sizeof(WT);
    constexpr int kUnroll = 4;
    const size_t nv = K / VEC;
    for (size_t base = 0; base < nv; base += 32 * kUnroll) {
        uint4 wv[RR][kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = base + (size_t)u * 32 + lane;
#pragma unroll
            for (int r = 0; r < RR; ++r)
                wv[r][u] = (i < nv) ? ld_stream_u4(reinterpret_cast<const uint4 *>(rows[r]) + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t i = base + (size_t)u * 32 + lane;
            if (i < nv) {
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const float4 *xp = reinterpret_cast<const float4 *>(xs + (size_t)m * K + i * VEC);
                    const float4 x0 = xp[0];
                    if constexpr (sizeof(WT) == 4) {
#pragma unroll
                        for (int r = 0; r < RR; ++r) {
                            acc[r][m] = fmaf(__uint_as_float(wv[r][u].x), x0.x, acc[r][m]);
                            acc[r][m] = fmaf(__uint_as_float(wv[r][u].y), x0.y, acc[r][m]);
                            acc[r][m] = fmaf(__uint_as_float(wv[r][u].z), x0.z, acc[r][m]);
                            acc[r][m] = fmaf(__uint_as_float(wv[r][u].w), x0.w, acc[r][m]);
                        }
                    } else {
                        const float4 x1 = xp[1];
#pragma unroll
                        for (int r = 0; r < RR; ++r) {
                            acc[r][m] = fmaf(bf16_lo(wv[r][u].x), x0.x, acc[r][m]);
                            acc[r][m] = fmaf(bf16_hi(wv[r][u].x), x0.y, acc[r][m]);
                            acc[r][m] = fmaf(bf16_lo(wv[r][u].y), x0.z, acc[r][m]);
                            acc[r][m] = fmaf(bf16_hi(wv[r][u].y), x0.w, acc[r][m]);
                            acc[r][m] = fmaf(bf16_lo(wv[r][u].z), x1.x, acc[r][m]);
                            acc[r][m] = fmaf(bf16_hi(wv[r][u].z), x1.y, acc[r][m]);
                            acc[r][m] = fmaf(bf16_lo(wv[r][u].w), x1.z, acc[r][m]);
                            acc[r][m] = fmaf(bf16_hi(wv[r][u].w), x1.w, acc[r][m]);
                        }
                    }
                }
            }
        }
    }
}

template <typename WT, int MB>
__global__ void __launch_bounds__(kThreads)
gemv_nk_kernel(const float *__restrict__ x, const WT *__restrict__ w, float *__restrict__ y, int M, size_t K, size_t N,
               size_t ldy, const float *__restrict__ norm_w, float eps, const float *__restrict__ residual) {
    extern __shared__ __align__(16) float smem[];
    float *xs = smem;
    float *red = smem + (size_t)MB * K;
    stage_x<MB>(xs, x, M, K, norm_w, eps, red);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int VEC = 16 / sizeof(WT);
    const bool vec_ok = (K % VEC == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    if constexpr (MB > 1) {
        if (vec_ok) {  // several vectors: rows are taken RR at a time so that x is read once per RR rows
            constexpr int RR = MB >= 8 ? 2 : 4;
            for (size_t row0 = ((size_t)blockIdx.x * kWarps + warp) * RR; row0 < N; row0 += (size_t)gridDim.x * kWarps * RR) {
                const WT *rows[RR];
                float acc[RR][MB];
#pragma unroll
                for (int r = 0; r < RR; ++r) {
                    rows[r] = w + (row0 + r < N ? row0 + r : N - 1) * K;  // rows past the end repeat the last one (not stored)
#pragma unroll
                    for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
                }
                rows_dot<WT, MB, RR>(rows, xs, K, lane, acc);
#pragma unroll
                for (int r = 0; r < RR; ++r) {
#pragma unroll
                    for (int m = 0; m < MB; ++m) {
                        const float v = warp_sum(acc[r][m]);
                        if (lane == 0 && m < M && row0 + r < N) {
                            const size_t o = (size_t)m * ldy + row0 + r;
                            y[o] = residual ? __fadd_rn(residual[o], v) : v;
                        }
                    }
                }
            }
            return;
        }
    }
    for (size_t row = (size_t)blockIdx.x * kWarps + warp; row < N; row += (size_t)gridDim.x * kWarps) {
        float acc[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) acc[m] = 0.f;
        row_dot<WT, MB>(w + row * K, xs, K, lane, vec_ok, acc);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            float v = warp_sum(acc[m]);
            if (lane == 0 && m < M) {
                size_t o = (size_t)m * ldy + row;
                y[o] = residual ? __fadd_rn(residual[o], v) : v;
            }
        }
    }
}

// gate/up pair: out[m,i] = silu(gate_i . x_m) * (up_i . x_m)  (src/models/llama.rs:59-63,
// src/layers/activation.rs:143-146: sig = 1/(1+exp(-g)); g*sig).
template <typename WT, int MB>
__global__ void __launch_bounds__(kThreads)
gemv_gate_up_kernel(const float *__restrict__ x, const WT *__restrict__ wg, const WT *__restrict__ wu,
                    float *__restrict__ out, int M, size_t K, size_t I, const float *__restrict__ norm_w, float eps) {
    extern __shared__ __align__(16) float smem[];
    float *xs = smem;
    float *red = smem + (size_t)MB * K;
    stage_x<MB>(xs, x, M, K, norm_w, eps, red);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int VEC = 16 / sizeof(WT);
    const bool vec_ok = (K % VEC == 0) && ((reinterpret_cast<uintptr_t>(wg) & 15) == 0) &&
                        ((reinterpret_cast<uintptr_t>(wu) & 15) == 0);
    if constexpr (MB > 1) {
        if (vec_ok) {  // the gate row and the up row of an output share every read of x
            for (size_t row = (size_t)blockIdx.x * kWarps + warp; row < I; row += (size_t)gridDim.x * kWarps) {
                const WT *rows[2] = {wg + row * K, wu + row * K};
                float acc[2][MB];
#pragma unroll
                for (int m = 0; m < MB; ++m) acc[0][m] = acc[1][m] = 0.f;
                rows_dot<WT, MB, 2>(rows, xs, K, lane, acc);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    const float g = warp_sum(acc[0][m]);
                    const float u = warp_sum(acc[1][m]);
                    if (lane == 0 && m < M) {
                        const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
                        out[(size_t)m * I + row] = __fmul_rn(__fmul_rn(g, sig), u);
                    }
                }
            }
            return;
        }
    }
    for (size_t row = (size_t)blockIdx.x * kWarps + warp; row < I; row += (size_t)gridDim.x * kWarps) {
        float ag[MB], au[MB];
#pragma unroll
        for (int m = 0; m < MB; ++m) ag[m] = au[m] = 0.f;
        row_dot<WT, MB>(wg + row * K, xs, K, lane, vec_ok, ag);
        row_dot<WT, MB>(wu + row * K, xs, K, lane, vec_ok, au);
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            float g = warp_sum(ag[m]);
            float u = warp_sum(au[m]);
            if (lane == 0 && m < M) {
                float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
                out[(size_t)m * I + row] = __fmul_rn(__fmul_rn(g, sig), u);
            }
        }
    }
}

// ---- [K,N] row-major layout ---------------------------------------------------------------------
// y[n] = sum_k w[k,n] x[k].  A thread owns VEC adjacent columns and walks a slice of k; slices are
// summed by a second kernel in slice order (deterministic, no atomics).
constexpr int kKnThreads = 128;

template <typename WT>
__global__ void __launch_bounds__(kKnThreads)
gemv_kn_partial_kernel(const float *__restrict__ x, const WT *__restrict__ w, float *__restrict__ part, size_t K,
                       size_t N, size_t k_per_split) {
    constexpr int VEC = 16 / sizeof(WT);
    const size_t col0 = ((size_t)blockIdx.x * kKnThreads + threadIdx.x) * VEC;
    const size_t k0 = (size_t)blockIdx.y * k_per_split;
    const size_t k1 = min(K, k0 + k_per_split);
    __shared__ float xs[1024];
    float acc[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
    const bool vec_ok = (N % VEC == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    for (size_t kb = k0; kb < k1; kb += 1024) {
        const size_t kn = min((size_t)1024, k1 - kb);
        __syncthreads();
        for (size_t i = threadIdx.x; i < kn; i += kKnThreads) xs[i] = x[kb + i];
        __syncthreads();
        if (col0 >= N) continue;
        if (vec_ok) {
            constexpr int U = 8;
            for (size_t kk = 0; kk < kn; kk += U) {
                uint4 wv[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    wv[u] = (kk + u < kn) ? __ldcs(reinterpret_cast<const uint4 *>(w + (kb + kk + u) * N + col0))
                                          : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float xv = (kk + u < kn) ? xs[kk + u] : 0.f;
                    if constexpr (sizeof(WT) == 4) {
                        acc[0] = fmaf(__uint_as_float(wv[u].x), xv, acc[0]);
                        acc[1] = fmaf(__uint_as_float(wv[u].y), xv, acc[1]);
                        acc[2] = fmaf(__uint_as_float(wv[u].z), xv, acc[2]);
                        acc[3] = fmaf(__uint_as_float(wv[u].w), xv, acc[3]);
                    } else {
                        acc[0] = fmaf(bf16_lo(wv[u].x), xv, acc[0]);
                        acc[1] = fmaf(bf16_hi(wv[u].x), xv, acc[1]);
                        acc[2] = fmaf(bf16_lo(wv[u].y), xv, acc[2]);
                        acc[3] = fmaf(bf16_hi(wv[u].y), xv, acc[3]);
                        acc[4] = fmaf(bf16_lo(wv[u].z), xv, acc[4]);
                        acc[5] = fmaf(bf16_hi(wv[u].z), xv, acc[5]);
                        acc[6] = fmaf(bf16_lo(wv[u].w), xv, acc[6]);
                        acc[7] = fmaf(bf16_hi(wv[u].w), xv, acc[7]);
                    }
                }
            }
        } else {
            for (size_t kk = 0; kk < kn; ++kk) {
#pragma unroll
                for (int v = 0; v < VEC; ++v) {
                    if (col0 + v < N) {
                        float wv;
                        if constexpr (sizeof(WT) == 4) wv = reinterpret_cast<const float *>(w)[(kb + kk) * N + col0 + v];
                        else wv = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(w)[(kb + kk) * N + col0 + v]);
                        acc[v] = fmaf(wv, xs[kk], acc[v]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v)
        if (col0 + v < N) part[(size_t)blockIdx.y * N + col0 + v] = acc[v];
}

__global__ void gemv_kn_reduce_kernel(const float *__restrict__ part, float *__restrict__ y, size_t N, int splits) {
    size_t n = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float s = 0.f;
    for (int i = 0; i < splits; ++i) s += part[(size_t)i * N + n];
    y[n] = s;
}

struct KnPlan {
    int col_blocks, splits;
    size_t k_per_split;
};

KnPlan plan_kn(size_t K, size_t N, int vec, int num_sms) {
    KnPlan p;
    p.col_blocks = (int)((N + (size_t)kKnThreads * vec - 1) / ((size_t)kKnThreads * vec));
    int want = (num_sms * 8 + p.col_blocks - 1) / p.col_blocks;  // aim at ~8 CTAs per SM
    size_t max_splits = (K + 31) / 32;                            // at least 32 k per slice
    int splits = (int)std::min<size_t>((size_t)std::max(want, 1), max_splits);
    splits = std::min(splits, 256);
    p.k_per_split = (K + splits - 1) / splits;
    p.splits = (int)((K + p.k_per_split - 1) / p.k_per_split);
    return p;
}

template <typename K>
int set_smem(lumen_ctx *ctx, K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        LUMEN_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    return LUMEN_OK;
}

int pick_grid(lumen_ctx *ctx, size_t rows, size_t smem_bytes) {
    // Resident CTAs per SM limited by shared memory (227 KB) and by 2048 threads.
    int per_sm = (int)std::min<size_t>(8, (227 * 1024) / std::max<size_t>(smem_bytes + 1024, 1));
    per_sm = std::max(per_sm, 1);
    size_t want = (rows + kWarps - 1) / kWarps;
    size_t cap = (size_t)ctx->num_sms * per_sm;
    return (int)std::max<size_t>(1, std::min(want, cap));
}

template <typename WT, int MB>
int launch_nk_t(lumen_ctx *ctx, const GemvArgs &a, cudaStream_t s) {
    size_t smem = ((size_t)MB * a.K + MB * kWarps) * sizeof(float);
    auto kern = gemv_nk_kernel<WT, MB>;
    LUMEN_TRY(set_smem(ctx, kern, smem));
    int grid = pick_grid(ctx, a.N, smem);
    kern<<<grid, kThreads, smem, s>>>(a.x, static_cast<const WT *>(a.w), a.y, a.M, a.K, a.N, a.ldy, a.norm_w,
                                      a.norm_eps, a.residual);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

template <typename WT, int MB>
int launch_gate_up_t(lumen_ctx *ctx, const float *x, const void *wg, const void *wu, float *out, int M, size_t K,
                     size_t I, const float *norm_w, float eps, cudaStream_t s) {
    size_t smem = ((size_t)MB * K + MB * kWarps) * sizeof(float);
    auto kern = gemv_gate_up_kernel<WT, MB>;
    LUMEN_TRY(set_smem(ctx, kern, smem));
    int grid = pick_grid(ctx, I, smem);
    kern<<<grid, kThreads, smem, s>>>(x, static_cast<const WT *>(wg), static_cast<const WT *>(wu), out, M, K, I, norm_w,
                                      eps);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace

int launch_gemv_nk(lumen_ctx *ctx, const GemvArgs &a, cudaStream_t s) {
    if (a.M < 1 || a.M > 8) return set_error(ctx, LUMEN_ERR_INVALID, "gemv: M=%d outside 1..8", a.M);
    if ((size_t)a.M * a.K * 4 > 200 * 1024) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "gemv: M*K too large for staging");
    const int mb = a.M == 1 ? 1 : a.M == 2 ? 2 : a.M <= 4 ? 4 : 8;
    const bool f32 = a.wdt == LUMEN_F32;
    switch (mb) {
        case 1: return f32 ? launch_nk_t<float, 1>(ctx, a, s) : launch_nk_t<__nv_bfloat16, 1>(ctx, a, s);
        case 2: return f32 ? launch_nk_t<float, 2>(ctx, a, s) : launch_nk_t<__nv_bfloat16, 2>(ctx, a, s);
        case 4: return f32 ? launch_nk_t<float, 4>(ctx, a, s) : launch_nk_t<__nv_bfloat16, 4>(ctx, a, s);
        default: return f32 ? launch_nk_t<float, 8>(ctx, a, s) : launch_nk_t<__nv_bfloat16, 8>(ctx, a, s);
    }
}

int launch_gemv_gate_up(lumen_ctx *ctx, const float *x, const void *w_gate, const void *w_up, lumen_dtype wdt,
                        float *out, int M, size_t K, size_t I, const float *norm_w, float norm_eps, cudaStream_t s) {
    if (M < 1 || M > 8) return set_error(ctx, LUMEN_ERR_INVALID, "gate_up: M=%d outside 1..8", M);
    if ((size_t)M * K * 4 > 200 * 1024) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "gate_up: M*K too large for staging");
    const int mb = M == 1 ? 1 : M == 2 ? 2 : M <= 4 ? 4 : 8;
    const bool f32 = wdt == LUMEN_F32;
#define GU(T, B) launch_gate_up_t<T, B>(ctx, x, w_gate, w_up, out, M, K, I, norm_w, norm_eps, s)
    switch (mb) {
        case 1: return f32 ? GU(float, 1) : GU(__nv_bfloat16, 1);
        case 2: return f32 ? GU(float, 2) : GU(__nv_bfloat16, 2);
        case 4: return f32 ? GU(float, 4) : GU(__nv_bfloat16, 4);
        default: return f32 ? GU(float, 8) : GU(__nv_bfloat16, 8);
    }
#undef GU
}

size_t gemv_kn_scratch_bytes_for(size_t K, size_t N, lumen_dtype wdt, int num_sms) {
    return (size_t)plan_kn(K, N, wdt == LUMEN_F32 ? 4 : 8, num_sms).splits * N * sizeof(float);
}

size_t gemv_kn_scratch_bytes(size_t K, size_t N, int num_sms) {
    KnPlan p4 = plan_kn(K, N, 4, num_sms), p8 = plan_kn(K, N, 8, num_sms);
    return (size_t)std::max(p4.splits, p8.splits) * N * sizeof(float);
}

int launch_gemv_kn(lumen_ctx *ctx, const float *x, const void *w, lumen_dtype wdt, float *y, size_t K, size_t N,
                   float *scratch, cudaStream_t s) {
    const int vec = wdt == LUMEN_F32 ? 4 : 8;
    KnPlan p = plan_kn(K, N, vec, ctx->num_sms);
    dim3 grid(p.col_blocks, p.splits);
    if (wdt == LUMEN_F32)
        gemv_kn_partial_kernel<float><<<grid, kKnThreads, 0, s>>>(x, static_cast<const float *>(w), scratch, K, N,
                                                                   p.k_per_split);
    else
        gemv_kn_partial_kernel<__nv_bfloat16>
            <<<grid, kKnThreads, 0, s>>>(x, static_cast<const __nv_bfloat16 *>(w), scratch, K, N, p.k_per_split);
    LUMEN_LAUNCHED(ctx);
    gemv_kn_reduce_kernel<<<(unsigned)((N + 255) / 256), 256, 0, s>>>(scratch, y, N, p.splits);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace lumen
