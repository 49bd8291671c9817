// C[M,N] = A[M,K] . W[N,K]^T (+ residual) on the 5th-generation tensor cores, for the M > 8 branch of
// ops::matmul (src/ops/matmul.rs:70-92: prefill and batched decode), for bf16 and for f32 weights.
//
// sm_100a structure: one CTA per 128 x 128 output tile (for at most 64 output rows: 128 weight rows x 64 output rows, the
// operands swapped so that the weights fill the 128-row side of the MMA); thread 0 is the TMA producer (2-D tiled copies
// with 128-byte swizzle into a 4-stage shared-memory ring, mbarrier transaction counts), thread 32 issues
// tcgen05.mma (kind::f16, bf16 operands, f32 accumulation) with the accumulator in tensor memory (128
// lanes x 128 columns) and releases each stage with tcgen05.commit; afterwards the four warps read the
// accumulator back with tcgen05.ld (32 lanes each) and store f32 rows.
//
// The activations are f32 in the reference.  They are split into two bf16 matrices, hi = bf16(a) and
// lo = bf16(a - hi), and both products accumulate into the same tensor-memory tile: a = hi + lo to about
// 2^-17 relative, so the result stays within ~1e-5 of the f32 product instead of the ~4e-3 a single bf16
// rounding of the activations would cost, at twice the (cheap) tensor-core work.  f32 weights (the
// reference's own dtype) are split the same way on the fly and three cross products are accumulated
// (a_hi.w_hi + a_lo.w_hi + a_hi.w_lo; the dropped a_lo.w_lo term is ~2^-18).
//
// Every wait is bounded; a wait that gives up records LUMEN_ERR_TIMEOUT, the CTA stops issuing, lets the
// copies in flight land, frees its tensor memory and returns.
#include <algorithm>

#include "tc_common.cuh"

namespace lumen {
namespace {

using namespace tc;

constexpr int kBM = 128;  // tile rows of A
constexpr int kTcThreads = 128;
constexpr uint32_t kABytes = kBM * kBK * 2;
// The tile is 128 x BN: BN = 128, or 64 / 32 for outputs narrower than that.  The 128-row side ("A") and the BN-row
// side ("B") each arrive as one or two bf16 matrices (a bf16 matrix, or the hi and lo parts of an f32 one):
//   plain:   A = activations (hi, lo), B = weights (bf16: one part; f32: hi, lo)   -> tile rows are output rows
//   swapped: A = weights (bf16: one part; f32: hi, lo), B = activations (hi, lo)   -> tile rows are output columns
// The swapped form serves few output rows (M <= 64, batched decode): the 128-row side of the MMA is filled with
// weight rows instead of mostly empty activation rows, so an MMA does useful work on all of its rows.
template <int NA, int NB, int BN>
struct TcGeom {
    static constexpr uint32_t kBBytes = BN * kBK * 2;
    static constexpr uint32_t kStageBytes = NA * kABytes + NB * kBBytes;
    static constexpr int kStages = (200 * 1024 / kStageBytes) > 6 ? 6 : (200 * 1024 / kStageBytes);
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    // Instruction descriptor: f32 accumulator, bf16 A and B, both K-major, N and M of the tile.
    static constexpr uint32_t kIdesc = idesc_bf16(kBM, BN);
};

struct TcParams {
    float *c;               // output, or the [splits][M][N] partial sums when the K range is split over blockIdx.z
    const float *residual;  // added in the epilogue (null with split K: the reduction kernel adds it)
    int M, N, K;
    int kb_per_split;       // 64-element K blocks per blockIdx.z
    DeviceStatus *status;
};

template <int NA, int NB, int BN, bool SWAP>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
               const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_blo, const TcParams p) {
    using Geom = TcGeom<NA, NB, BN>;
    constexpr int kStages = Geom::kStages, kBN = BN, kTmemCols = Geom::kTmemCols;
    constexpr uint32_t kStageBytes = Geom::kStageBytes, kBBytes = Geom::kBBytes, kIdesc = Geom::kIdesc;
    extern __shared__ unsigned char smem_raw[];
    // the 128-byte swizzle pattern repeats every 1024 bytes: tiles must start on that boundary
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full[kStages], empty[kStages], done;
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // first row of this CTA's tile on the 128-row side and on the BN-row side (blockIdx.x walks the weight rows)
    const int a0 = (SWAP ? blockIdx.x : blockIdx.y) * kBM, b0 = (SWAP ? blockIdx.y : blockIdx.x) * kBN;
    // This CTA's range of 64-element K blocks: all of them, or slice blockIdx.z when K is split over the grid
    // (few output tiles and a long K: more CTAs stream the weights).  kb below counts from the slice's start.
    const int kb_all = (p.K + kBK - 1) / kBK;
    const int kb0 = (int)blockIdx.z * p.kb_per_split;
    const int nkb = max(0, min(kb_all, kb0 + p.kb_per_split) - kb0);

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            bar_init(&full[s], 1);
            bar_init(&empty[s], 1);
        }
        bar_init(&done, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {  // tensor memory: kBN (at least 32) columns of 128 lanes x 32 bits
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (tid == 0) {
        // ---- producer ----
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % kStages;
            if (kb >= kStages && !bar_wait(&empty[s], (uint32_t)((kb / kStages - 1) & 1), p.status, 500)) {
                failed = 1;
                break;
            }
            unsigned char *st = tiles + (size_t)s * kStageBytes;
            bar_expect(&full[s], kStageBytes);
            const int kx = (kb0 + kb) * kBK;
            tma_load_2d(st, &map_ahi, kx, a0, &full[s]);
            if (NA == 2) tma_load_2d(st + kABytes, &map_alo, kx, a0, &full[s]);
            tma_load_2d(st + NA * kABytes, &map_b, kx, b0, &full[s]);
            if (NB == 2) tma_load_2d(st + NA * kABytes + kBBytes, &map_blo, kx, b0, &full[s]);
        }
    } else if (tid == 32) {
        // ---- MMA issuer ----
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; ++kb) {
            const int s = kb % kStages;
            ok = bar_wait(&full[s], (uint32_t)((kb / kStages) & 1), p.status, 510);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t st = saddr(tiles + (size_t)s * kStageBytes);
            const uint64_t dhi = smem_desc(st), dlo = smem_desc(st + kABytes), db = smem_desc(st + NA * kABytes);
            const uint64_t dblo = smem_desc(st + NA * kABytes + kBBytes);
#pragma unroll
            for (int kk = 0; kk < kBK / 16; ++kk) {  // UMMA K = 16 bf16 = 32 bytes = 2 descriptor units
                umma_bf16(tmem_base, dhi + 2 * kk, db + 2 * kk, kIdesc, (kb > 0 || kk > 0) ? 1u : 0u);
                if (NA == 2) umma_bf16(tmem_base, dlo + 2 * kk, db + 2 * kk, kIdesc, 1u);
                if (NB == 2) umma_bf16(tmem_base, dhi + 2 * kk, dblo + 2 * kk, kIdesc, 1u);  // (lo . lo ~ 2^-18: dropped)
            }
            umma_commit(&empty[s]);  // arrives when the MMAs above have finished reading the stage
        }
        if (!ok) failed = 1;
        umma_commit(&done);  // arrives when every MMA issued so far has completed
    }
    __syncwarp();
    // ---- epilogue: all four warps ----
    const bool have = bar_wait(&done, 0, p.status, 520);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    if (have && !failed) {
        const int arow = a0 + warp * 32 + lane;  // this thread's row of the tile's 128-row side
        const bool empty_slice = nkb == 0;       // nothing was accumulated: the tile's contribution is zero
        float *cbase = p.c + (size_t)blockIdx.z * p.M * p.N;
#pragma unroll 1
        for (int c0 = 0; c0 < kBN; c0 += 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
            tmem_ld32(taddr, v);
            if (!SWAP) {
                if (arow < p.M) {  // output row arow, columns b0 + c0 ..
                    float *crow = cbase + (size_t)arow * p.N + b0 + c0;
                    const float *rrow = p.residual ? p.residual + (size_t)arow * p.N + b0 + c0 : nullptr;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (b0 + c0 + j < p.N) {
                            float x = empty_slice ? 0.f : __uint_as_float(v[j]);
                            if (rrow) x = __fadd_rn(rrow[j], x);  // x + residual as `Tensor + Tensor` (arithmetic.rs:48-52)
                            crow[j] = x;
                        }
                    }
                }
            } else if (arow < p.N) {  // output column arow, rows b0 + c0 ..: a warp writes 32 adjacent columns of one row
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int m = b0 + c0 + j;
                    if (m < p.M) {
                        float x = empty_slice ? 0.f : __uint_as_float(v[j]);
                        if (p.residual) x = __fadd_rn(p.residual[(size_t)m * p.N + arow], x);
                        cbase[(size_t)m * p.N + arow] = x;
                    }
                }
            }
        }
    } else if (tid == 0) {
        // A wait gave up: let the copies that are still in flight land before the CTA exits (bounded).
        for (int s = 0; s < kStages; ++s) {
            const long long t0 = clock64();
            while (!bar_try(&full[s], 0) && !bar_try(&full[s], 1) && clock64() - t0 < kTcWaitCycles) {}
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// c[m, n] = sum over splits of part[s][m][n] (+ residual), splits added in order
__global__ void splitk_reduce_kernel(const float *__restrict__ part, const float *__restrict__ residual, float *__restrict__ c,
                                     size_t mn, int splits) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float s = part[i];
    for (int k = 1; k < splits; ++k) s = __fadd_rn(s, part[(size_t)k * mn + i]);
    c[i] = residual ? __fadd_rn(residual[i], s) : s;
}

// hi = bf16(a), lo = bf16(a - hi)
__global__ void split_bf16_kernel(const float *__restrict__ a, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = a[i];
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(x - __bfloat162float(h));
}

}  // namespace

bool gemm_tc_usable(lumen_dtype wdt, size_t M, size_t K, size_t N, const void *w) {
    static const int mode = [] {  // LUMEN_NO_TC=1: never; LUMEN_NO_TC=f32: bf16 weights only
        const char *e = getenv("LUMEN_NO_TC");
        return !e ? 0 : (e[0] == '1' ? 1 : 2);
    }();
    if (mode == 1 || (mode == 2 && wdt == LUMEN_F32)) return false;
    // TMA: 16-byte aligned base and row pitch (K * 2 bytes)
    return M > 1 && N >= 8 && K % 8 == 0 && K >= 8 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
}

namespace {

template <int NA, int NB, int BN, bool SWAP>
int launch_tc_kernel(lumen_ctx *ctx, const CUtensorMap &mhi, const CUtensorMap &mlo, const CUtensorMap &mb, const CUtensorMap &mblo,
                     const TcParams &p, size_t M, size_t N, cudaStream_t s) {
    using Geom = TcGeom<NA, NB, BN>;
    constexpr size_t smem = (size_t)Geom::kStages * Geom::kStageBytes + 1024;  // + slack for the alignment
    static bool attr_set[64] = {false};
    const int dev = ctx->device >= 0 && ctx->device < 64 ? ctx->device : 0;
    if (!attr_set[dev]) {
        LUMEN_CUDA(ctx, cudaFuncSetAttribute(gemm_tc_kernel<NA, NB, BN, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    const int kb_all = (p.K + kBK - 1) / kBK;
    const int splits = (kb_all + p.kb_per_split - 1) / p.kb_per_split;
    const dim3 grid = SWAP ? dim3((unsigned)((N + kBM - 1) / kBM), (unsigned)((M + BN - 1) / BN), (unsigned)splits)
                           : dim3((unsigned)((N + BN - 1) / BN), (unsigned)((M + kBM - 1) / kBM), (unsigned)splits);
    gemm_tc_kernel<NA, NB, BN, SWAP><<<grid, kTcThreads, smem, s>>>(mhi, mlo, mb, mblo, p);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

// 128-wide tiles measured fastest even when they leave SMs without a CTA (M = 512, N = 4096: 331 TFLOP/s
// with 128 CTAs of 128 x 128 against 228 with 256 CTAs of 128 x 64); narrower tiles only for narrow outputs.
int pick_bn(size_t M, size_t N, int num_sms) {
    (void)M;
    (void)num_sms;
    return N > 64 ? 128 : (N > 32 ? 64 : 32);
}

}  // namespace

int launch_split_bf16(lumen_ctx *ctx, const float *a, __nv_bfloat16 *hi, __nv_bfloat16 *lo, size_t n, cudaStream_t s) {
    if (n == 0) return LUMEN_OK;
    split_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, hi, lo, n);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

// wdt == LUMEN_F32: the weights are split into hi + lo bf16 matrices on the fly as well (one streaming pass
// over W per call) and three of the four cross products are accumulated.
int launch_gemm_tc(lumen_ctx *ctx, const float *a, const void *w, lumen_dtype wdt, float *c, size_t M, size_t K, size_t N,
                   const float *residual, cudaStream_t s, const TpSumArgs *tp, const GemmFuse *fuse) {
    const bool wsplit = wdt == LUMEN_F32;
    const bool presplit = fuse && fuse->a_hi && fuse->a_lo;  // the producer of the activations split them already
    void *split = nullptr;
    const bool wpre = wsplit && fuse && fuse->w_hi && fuse->w_lo;  // the model keeps the split of its f32 weights
    const size_t na = presplit ? 0 : M * K, nap = (na + 7) & ~(size_t)7, nw = (wsplit && !wpre) ? N * K : 0, nwp = (nw + 7) & ~(size_t)7;
    LUMEN_TRY(dev_alloc(ctx, (2 * nap + 2 * nwp) * sizeof(__nv_bfloat16) + 32, &split));
    __nv_bfloat16 *hi = static_cast<__nv_bfloat16 *>(split);
    __nv_bfloat16 *lo = hi + nap;  // every matrix stays 16-byte aligned
    __nv_bfloat16 *whi = lo + nap, *wlo = whi + nwp;
    int rc = LUMEN_OK;
    if (presplit) {
        hi = const_cast<__nv_bfloat16 *>(fuse->a_hi);
        lo = const_cast<__nv_bfloat16 *>(fuse->a_lo);
    } else {
        split_bf16_kernel<<<(unsigned)((na + 255) / 256), 256, 0, s>>>(a, hi, lo, na);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = cuda_fail(ctx, e, "split_bf16_kernel launch");
        else ctx->launches += 1;
    }
    if (wpre) {
        whi = const_cast<__nv_bfloat16 *>(fuse->w_hi);
        wlo = const_cast<__nv_bfloat16 *>(fuse->w_lo);
    } else if (rc == LUMEN_OK && wsplit) {
        split_bf16_kernel<<<(unsigned)((nw + 255) / 256), 256, 0, s>>>(static_cast<const float *>(w), whi, wlo, nw);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = cuda_fail(ctx, e, "split_bf16_kernel launch");
        else ctx->launches += 1;
    }
    // Few output rows: the weights take the 128-row side of the tile and the activations the 64-row side.
    static const bool no_swap = [] {
        const char *e = getenv("LUMEN_NO_TC_SWAP");
        return e && e[0] == '1';
    }();
    const bool swap = M <= 64 && !no_swap;
    CUtensorMap map_hi, map_lo, map_b, map_blo;  // 128-row side (hi, lo), BN-row side (hi, lo)
    const int bn = swap ? 64 : pick_bn(M, N, ctx->num_sms);
    if (!swap) {
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_hi, hi, M, K, kBM);
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_lo, lo, M, K, kBM);
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_b, wsplit ? (const void *)whi : w, N, K, bn);
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_blo, wsplit ? (const void *)wlo : w, N, K, bn);
    } else {
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_hi, wsplit ? (const void *)whi : w, N, K, kBM);
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_lo, wsplit ? (const void *)wlo : w, N, K, kBM);
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_b, hi, M, K, bn);
        if (rc == LUMEN_OK) rc = make_map(ctx, &map_blo, lo, M, K, bn);
    }
    // Few output tiles (one row of tiles: M <= 128) and many K blocks: split K over blockIdx.z so that about
    // every SM streams a share of W; the slices' partial tiles are summed in slice order by a second kernel.
    const int kb_all = (int)((K + kBK - 1) / kBK);
    int splits = 1;
    if (M <= (size_t)kBM) {
        const int tiles = (int)((N + (swap ? kBM : bn) - 1) / (swap ? kBM : bn));
        splits = std::max(1, std::min(std::min(ctx->num_sms / std::max(tiles, 1), kb_all / 4), 16));
    }
    const int kb_per_split = (kb_all + splits - 1) / splits;
    splits = (kb_all + kb_per_split - 1) / kb_per_split;
    void *partial = nullptr;
    if (rc == LUMEN_OK && splits > 1) rc = dev_alloc(ctx, (size_t)splits * M * N * sizeof(float), &partial);
    if (rc == LUMEN_OK) {
        TcParams p{splits > 1 ? static_cast<float *>(partial) : c, splits > 1 ? nullptr : residual, (int)M, (int)N, (int)K,
                   kb_per_split, ctx->d_status};
#define LUMEN_TC(NA_, NB_, BN_, SW_) launch_tc_kernel<NA_, NB_, BN_, SW_>(ctx, map_hi, map_lo, map_b, map_blo, p, M, N, s)
        if (swap) rc = wsplit ? LUMEN_TC(2, 2, 64, true) : LUMEN_TC(1, 2, 64, true);
        else if (wsplit) rc = bn == 128 ? LUMEN_TC(2, 2, 128, false) : bn == 64 ? LUMEN_TC(2, 2, 64, false) : LUMEN_TC(2, 2, 32, false);
        else rc = bn == 128 ? LUMEN_TC(2, 1, 128, false) : bn == 64 ? LUMEN_TC(2, 1, 64, false) : LUMEN_TC(2, 1, 32, false);
#undef LUMEN_TC
        if (rc == LUMEN_OK && tp) {
            // the sum over the ranks takes the slices (or the finished product) from here
            rc = splits > 1 ? launch_tp_sum(ctx, static_cast<const float *>(partial), splits, residual, M, N, *tp, s)
                            : launch_tp_sum(ctx, c, 1, nullptr, M, N, *tp, s);
        } else if (rc == LUMEN_OK && fuse && fuse->post == GemmFuse::kPostNorm) {
            if (splits > 1)
                rc = launch_sum_norm_split(ctx, static_cast<const float *>(partial), splits, residual, M, N, c, fuse->norm_w, fuse->eps,
                                           fuse->next_hi, fuse->next_lo, s);
            else if (fuse->norm_w)  // c is complete (the product's epilogue added the residual): only the norm outputs are missing
                rc = launch_sum_norm_split(ctx, c, 1, nullptr, M, N, nullptr, fuse->norm_w, fuse->eps, fuse->next_hi, fuse->next_lo, s);
        } else if (rc == LUMEN_OK && fuse && fuse->post == GemmFuse::kPostSwiglu) {
            rc = launch_sum_swiglu_split(ctx, splits > 1 ? static_cast<const float *>(partial) : c, splits, M, N / 2, fuse->next_hi,
                                         fuse->next_lo, s);
        } else if (rc == LUMEN_OK && splits > 1) {
            const size_t mn = M * N;
            splitk_reduce_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(static_cast<const float *>(partial), residual, c, mn, splits);
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) rc = cuda_fail(ctx, e, "splitk_reduce_kernel launch");
            else ctx->launches += 1;
        }
    }
    if (partial) {
        int rc3 = dev_free(ctx, partial);
        if (rc == LUMEN_OK) rc = rc3;
    }
    int rc2 = dev_free(ctx, split);
    return rc != LUMEN_OK ? rc : rc2;
}

}  // namespace lumen
