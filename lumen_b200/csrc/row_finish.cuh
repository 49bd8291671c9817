// Device helpers shared by the kernels that finish a matrix product row by row (gemm_finish.cu, tp_sum.cu): a CTA of
// 256 threads holds one output row of up to kRowVecs * 1024 elements in registers (thread t owns the float4 at
// t + 256 k), so the split-K sum, the residual, the RMSNorm of the row and the bf16 hi/lo split the next tensor-core
// product wants are passes over registers, and every pass over memory is one batch of independent 128-bit accesses.
#pragma once

#include "common.cuh"

namespace lumen {

constexpr int kRowVecs = 8;  // float4 per thread: rows of up to 8192 elements

__device__ __forceinline__ float4 add4(float4 a, float4 b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}

// hi = bf16(x), lo = bf16(x - hi) for four values, packed for one 8-byte store each
__device__ __forceinline__ void split4(float4 v, uint2 *hi, uint2 *lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y), h2 = __float2bfloat16_rn(v.z),
                        h3 = __float2bfloat16_rn(v.w);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(v.x - __bfloat162float(h0)), l1 = __float2bfloat16_rn(v.y - __bfloat162float(h1)),
                        l2 = __float2bfloat16_rn(v.z - __bfloat162float(h2)), l3 = __float2bfloat16_rn(v.w - __bfloat162float(h3));
    hi->x = (unsigned)__bfloat16_as_ushort(h0) | ((unsigned)__bfloat16_as_ushort(h1) << 16);
    hi->y = (unsigned)__bfloat16_as_ushort(h2) | ((unsigned)__bfloat16_as_ushort(h3) << 16);
    lo->x = (unsigned)__bfloat16_as_ushort(l0) | ((unsigned)__bfloat16_as_ushort(l1) << 16);
    lo->y = (unsigned)__bfloat16_as_ushort(l2) | ((unsigned)__bfloat16_as_ushort(l3) << 16);
}

// What follows the sum of a row.
struct RowFinish {
    float *out;            // [rows, dim] the summed row (null: not stored)
    const float *norm_w;   // RMSNorm gains (null: no norm outputs)
    float eps;
    float *normed;         // [rows, dim] f32 Norm(row) (null: not stored)
    __nv_bfloat16 *hi, *lo;  // [rows, dim] bf16 split of Norm(row) (null: not stored)
};

// acc[k] = sum over `splits` slices (added in slice order) of part[slice][row] (+ residual[row]): the thread's share of a row.
__device__ __forceinline__ void row_load_sum(float4 (&acc)[kRowVecs], const float *part, int splits, size_t mn, const float *residual,
                                             size_t base, int nvec, int tid) {
    {
        const float4 *p0 = reinterpret_cast<const float4 *>(part + base);
#pragma unroll
        for (int k = 0; k < kRowVecs; ++k)
            if (tid + 256 * k < nvec) acc[k] = p0[tid + 256 * k];
    }
#pragma unroll 4
    for (int sl = 1; sl < splits; ++sl) {
        const float4 *ps = reinterpret_cast<const float4 *>(part + (size_t)sl * mn + base);
        float4 t[kRowVecs];
#pragma unroll
        for (int k = 0; k < kRowVecs; ++k)
            if (tid + 256 * k < nvec) t[k] = ps[tid + 256 * k];
#pragma unroll
        for (int k = 0; k < kRowVecs; ++k)
            if (tid + 256 * k < nvec) acc[k] = add4(acc[k], t[k]);
    }
    if (residual) {
        const float4 *pr = reinterpret_cast<const float4 *>(residual + base);
        float4 t[kRowVecs];
#pragma unroll
        for (int k = 0; k < kRowVecs; ++k)
            if (tid + 256 * k < nvec) t[k] = pr[tid + 256 * k];
#pragma unroll
        for (int k = 0; k < kRowVecs; ++k)
            if (tid + 256 * k < nvec) acc[k] = add4(t[k], acc[k]);
    }
}

// Stores the row and, with gains, RMSNorm::forward of it (src/layers/norm/rms_norm.rs:49-56: rms = sqrt(ss/dim + eps),
// o = (x * (1/rms)) * w) as f32 and/or as the bf16 hi/lo pair.  `red` is 8 floats of shared memory; all 256 threads call.
__device__ __forceinline__ void row_finish(const float4 (&v)[kRowVecs], const RowFinish &f, size_t base, int dim, int nvec, int tid,
                                           float *red) {
    float ss = 0.f;
    float4 *o4 = f.out ? reinterpret_cast<float4 *>(f.out + base) : nullptr;
#pragma unroll
    for (int k = 0; k < kRowVecs; ++k)
        if (tid + 256 * k < nvec) {
            if (o4) o4[tid + 256 * k] = v[k];
            ss = fmaf(v[k].x, v[k].x, ss);
            ss = fmaf(v[k].y, v[k].y, ss);
            ss = fmaf(v[k].z, v[k].z, ss);
            ss = fmaf(v[k].w, v[k].w, ss);
        }
    if (!f.norm_w) return;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    __syncthreads();
    const float rms = sqrtf(__fadd_rn(__fdiv_rn(t, (float)dim), f.eps));
    const float inv = __fdiv_rn(1.0f, rms);
    const float4 *g4 = reinterpret_cast<const float4 *>(f.norm_w);
    float4 *n4 = f.normed ? reinterpret_cast<float4 *>(f.normed + base) : nullptr;
    uint2 *h2 = f.hi ? reinterpret_cast<uint2 *>(f.hi + base) : nullptr;
    uint2 *l2 = f.hi ? reinterpret_cast<uint2 *>(f.lo + base) : nullptr;
#pragma unroll
    for (int k = 0; k < kRowVecs; ++k)
        if (tid + 256 * k < nvec) {
            const float4 g = g4[tid + 256 * k];
            const float4 n = make_float4(__fmul_rn(__fmul_rn(v[k].x, inv), g.x), __fmul_rn(__fmul_rn(v[k].y, inv), g.y),
                                         __fmul_rn(__fmul_rn(v[k].z, inv), g.z), __fmul_rn(__fmul_rn(v[k].w, inv), g.w));
            if (n4) n4[tid + 256 * k] = n;
            if (h2) {
                uint2 h, l;
                split4(n, &h, &l);
                h2[tid + 256 * k] = h;
                l2[tid + 256 * k] = l;
            }
        }
}

}  // namespace lumen
