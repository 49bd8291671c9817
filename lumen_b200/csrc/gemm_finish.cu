// Kernels that finish a tensor-core product of a batched step or a prefill slice in one pass over its split-K slices,
// producing what the NEXT product reads, so that a block of LlamaBlock::forward (src/models/llama.rs:107-115, :59-65)
// needs 11 launches instead of 20:
//   sum_norm_split_kernel  x = sum of slices + residual;  (hi, lo) = bf16 split of RMSNorm(x) * gains
//                          (replaces split-K sum + RMSNorm + hi/lo split)
//   sum_swiglu_split_kernel  (hi, lo) = bf16 split of silu(gate) * up, gate and up being the column halves of one product
//                          over the concatenated gate and up weights (replaces two split-K sums + SiLU*mul + hi/lo split)
#include <algorithm>

#include "row_finish.cuh"

namespace lumen {
namespace {

__global__ void __launch_bounds__(256) sum_norm_split_kernel(const float *__restrict__ part, int splits, const float *residual, int rows,
                                                             int dim, RowFinish f) {
    __shared__ float red[8];
    const int tid = threadIdx.x, nvec = dim >> 2;
    const size_t mn = (size_t)rows * dim;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * dim;
        float4 v[kRowVecs];
        row_load_sum(v, part, splits, mn, residual, base, nvec, tid);
        row_finish(v, f, base, dim, nvec, tid, red);
    }
}

// SiLU::forward — src/layers/activation.rs:143-146
__device__ __forceinline__ float silu_mul1(float g, float u) {
    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(__fmul_rn(g, sig), u);
}

// part: [splits][rows][2 * inter]; thread = 4 adjacent columns of one row
__global__ void __launch_bounds__(256) sum_swiglu_split_kernel(const float *__restrict__ part, int splits, size_t rows, size_t inter,
                                                               __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo) {
    const size_t q = (size_t)blockIdx.x * 256 + threadIdx.x, per_row = inter >> 2;
    if (q >= rows * per_row) return;
    const size_t row = q / per_row, col = (q - row * per_row) << 2;
    const size_t mn = rows * 2 * inter, at = row * 2 * inter + col;
    float4 g = *reinterpret_cast<const float4 *>(part + at), u = *reinterpret_cast<const float4 *>(part + at + inter);
#pragma unroll 4
    for (int sl = 1; sl < splits; ++sl) {
        const float4 g2 = *reinterpret_cast<const float4 *>(part + (size_t)sl * mn + at);
        const float4 u2 = *reinterpret_cast<const float4 *>(part + (size_t)sl * mn + at + inter);
        g = add4(g, g2);
        u = add4(u, u2);
    }
    const float4 a = make_float4(silu_mul1(g.x, u.x), silu_mul1(g.y, u.y), silu_mul1(g.z, u.z), silu_mul1(g.w, u.w));
    uint2 h, l;
    split4(a, &h, &l);
    *reinterpret_cast<uint2 *>(hi + row * inter + col) = h;
    *reinterpret_cast<uint2 *>(lo + row * inter + col) = l;
}

}  // namespace

bool row_finish_usable(size_t dim) { return dim % 8 == 0 && dim <= (size_t)kRowVecs * 1024; }

int launch_sum_norm_split(lumen_ctx *ctx, const float *part, int splits, const float *residual, size_t rows, size_t dim, float *out,
                          const float *norm_w, float eps, __nv_bfloat16 *hi, __nv_bfloat16 *lo, cudaStream_t s) {
    if (rows == 0) return LUMEN_OK;
    if (!row_finish_usable(dim)) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "row finisher: row length %zu", dim);
    RowFinish f{out, norm_w, eps, nullptr, hi, lo};
    const unsigned grid = (unsigned)std::min<size_t>(rows, (size_t)ctx->num_sms * 8);
    sum_norm_split_kernel<<<grid, 256, 0, s>>>(part, splits, residual, (int)rows, (int)dim, f);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_sum_swiglu_split(lumen_ctx *ctx, const float *part, int splits, size_t rows, size_t inter, __nv_bfloat16 *hi,
                            __nv_bfloat16 *lo, cudaStream_t s) {
    if (rows == 0 || inter == 0) return LUMEN_OK;
    if (inter % 8) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "SwiGLU finisher: intermediate size %zu", inter);
    const size_t quads = rows * (inter >> 2);
    sum_swiglu_split_kernel<<<(unsigned)((quads + 255) / 256), 256, 0, s>>>(part, splits, rows, inter, hi, lo);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace lumen
