// M > 1 product C[M,N] = A[M,K] . W[N,K]^T in f32 (SIMT register tiles).
//
// Restates the M > 1 branch of ops::matmul::matmul (src/ops/matmul.rs:70-92 of the reference), which
// hands the product to ndarray's general_mat_mul.  That routine's summation order is third-party and
// unpinned, so parity is to f32 rounding.  Used for prefill and for batches too large for the
// vector-matrix kernel when the weights are f32 (bf16 weights are widened on load).
#include <algorithm>

#include "common.cuh"

namespace lumen {
namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
constexpr int kThreads = (BM / TM) * (BN / TN);  // 256

template <typename WT>
__device__ __forceinline__ float w_to_f32(WT v) {
    if constexpr (sizeof(WT) == 4) return v;
    else return __bfloat162float(v);
}

template <typename WT>
__global__ void __launch_bounds__(kThreads)
gemm_nk_kernel(const float *__restrict__ a, const WT *__restrict__ w, float *__restrict__ c, size_t M, size_t K,
               size_t N, const float *__restrict__ residual) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const size_t m0 = (size_t)blockIdx.y * BM, n0 = (size_t)blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // Each thread loads 4 consecutive k of one row of A and of W per tile: 64 rows x 16 k = 256 x 4.
    const int lr = tid / (BK / 4), lk = (tid % (BK / 4)) * 4;
    for (size_t k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const size_t kk = k0 + lk + t;
            const size_t am = m0 + lr, wn = n0 + lr;
            as[lk + t][lr] = (am < M && kk < K) ? a[am * K + kk] : 0.f;
            ws[lk + t][lr] = (wn < N && kk < K) ? w_to_f32<WT>(w[wn * K + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4 *>(&as[kk][ty * TM]);
            const float4 wv = *reinterpret_cast<const float4 *>(&ws[kk][tx * TN]);
            const float ar[TM] = {av.x, av.y, av.z, av.w};
            const float wr[TN] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const size_t m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const size_t n = n0 + tx * TN + j;
            if (n >= N) continue;
            const size_t o = m * N + n;
            c[o] = residual ? __fadd_rn(residual[o], acc[i][j]) : acc[i][j];
        }
    }
}

}  // namespace

int launch_gemm_nk(lumen_ctx *ctx, const float *a, const void *w, lumen_dtype wdt, float *c, size_t M, size_t K,
                   size_t N, const float *residual, cudaStream_t s, const TpSumArgs *tp) {
    if (M == 0 || N == 0) return LUMEN_OK;
    if (gemm_tc_usable(wdt, M, K, N, w)) return launch_gemm_tc(ctx, a, w, wdt, c, M, K, N, residual, s, tp);
    dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM));
    if (wdt == LUMEN_F32)
        gemm_nk_kernel<float><<<grid, kThreads, 0, s>>>(a, static_cast<const float *>(w), c, M, K, N, residual);
    else
        gemm_nk_kernel<__nv_bfloat16>
            <<<grid, kThreads, 0, s>>>(a, static_cast<const __nv_bfloat16 *>(w), c, M, K, N, residual);
    LUMEN_LAUNCHED(ctx);
    if (tp) return launch_tp_sum(ctx, c, 1, nullptr, M, N, *tp, s);
    return LUMEN_OK;
}

}  // namespace lumen
