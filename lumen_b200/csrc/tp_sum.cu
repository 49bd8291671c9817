// Tensor-parallel sum of a row-parallel product for batched steps and short prefills, as ONE kernel over peer memory:
// the rank's split-K slices are added (the product's own last step), the rank's partial rows are stored into a slot of
// every rank's buffer over NVLink, a per-row flag follows, and each rank adds the ranks' slots in rank order (so every
// rank holds bit-identical sums), optionally applying the next block's RMSNorm to the summed row.  It replaces
// split-K sum + NCCL all-reduce + RMSNorm (three launches, one of them a collective) on the o_proj and down products of
// LlamaBlock::forward (src/models/llama.rs:107-115); the reference is a single process and has no counterpart.
//
// Protocol.  Every rank owns {control words, flags[2][T][kTpSumMaxRows], slots[2][T][kTpSumSlotFloats]} and maps the
// other ranks' copies (CUDA IPC).  A launch reads the epoch e from its control word (all ranks run the same sequence of
// launches, so their epochs agree), uses buffer e & 1, and the last CTA to finish advances the epoch for the next
// launch on the stream; that keeps the kernel replayable inside a CUDA graph.  A rank can be at most one exchange ahead
// of another (it needs that rank's rows of exchange k before it finishes k), so two buffers are enough: when a rank
// writes for k + 2 every rank has finished reading k.  Every CTA first stores all its rows and only then waits, and
// the grid is small enough to be co-resident, so no CTA waits for one that cannot run.  Waits are bounded: on expiry
// the CTA records LUMEN_ERR_TIMEOUT in the status word and carries on without the missing rows.
#include <algorithm>
#include <cstdlib>

#include "row_finish.cuh"

namespace lumen {
namespace {

constexpr long long kTpSumWaitCycles = 4000000000LL;  // ~2 s: ranks are launched by different host processes

struct TpSumParams {
    const float *part;      // [splits][rows*dim] partial products of this rank
    const float *residual;  // added once (rank 0 passes the residual stream) or null
    RowFinish fin;          // where the sum over the ranks goes: the row, and optionally RMSNorm of it (f32 and/or bf16 hi/lo)
    int splits, rows, dim, rank;
    float *slots[8];
    unsigned *flags[8];
    unsigned *ctl;          // {epoch, finished CTAs}
    DeviceStatus *status;
};

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <int T>
__global__ void __launch_bounds__(256) tp_sum_kernel(TpSumParams p) {
    __shared__ float red[8];
    const int tid = threadIdx.x;
    const unsigned e = *reinterpret_cast<volatile unsigned *>(p.ctl) + 1u;
    const size_t buf = e & 1u;
    const size_t mn = (size_t)p.rows * p.dim;
    const int nvec = p.dim >> 2;
    const size_t my_slot = (buf * T + p.rank) * kTpSumSlotFloats;
    const size_t my_flag = (buf * T + p.rank) * kTpSumMaxRows;

    // 1. this rank's partial rows (split-K slices added in order, residual last) into everybody's slot `rank`
    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        const size_t base = (size_t)row * p.dim;
        float4 acc[kRowVecs];
        row_load_sum(acc, p.part, p.splits, mn, p.residual, base, nvec, tid);
#pragma unroll
        for (int r = 0; r < T; ++r) {
            float4 *dst = reinterpret_cast<float4 *>(p.slots[r] + my_slot + base);
#pragma unroll
            for (int k = 0; k < kRowVecs; ++k)
                if (tid + 256 * k < nvec) dst[tid + 256 * k] = acc[k];
        }
        __syncthreads();
        if (tid < T) {
            __threadfence_system();
            st_release_sys(p.flags[tid] + my_flag + row, e);
        }
    }

    // 2. wait for the ranks' rows, add them in rank order
    const float *mine = p.slots[p.rank] + buf * T * kTpSumSlotFloats;
    const unsigned *flg = p.flags[p.rank] + buf * T * kTpSumMaxRows;
    for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
        if (tid < T) {
            const unsigned *f = flg + (size_t)tid * kTpSumMaxRows + row;
            const long long t0 = clock64();
            while (ld_acquire_sys(f) != e) {
                if (clock64() - t0 > kTpSumWaitCycles) {
                    if (atomicCAS(&p.status->code, 0, LUMEN_ERR_TIMEOUT) == 0) {
                        p.status->detail0 = 700 + tid;
                        p.status->detail1 = row;
                    }
                    break;
                }
            }
        }
        __syncthreads();
        const size_t base = (size_t)row * p.dim;
        float4 v[kRowVecs];
        {
            const float4 *s0 = reinterpret_cast<const float4 *>(mine + base);
#pragma unroll
            for (int k = 0; k < kRowVecs; ++k)
                if (tid + 256 * k < nvec) v[k] = __ldcg(s0 + tid + 256 * k);
        }
#pragma unroll
        for (int t = 1; t < T; ++t) {
            const float4 *st = reinterpret_cast<const float4 *>(mine + (size_t)t * kTpSumSlotFloats + base);
            float4 u[kRowVecs];
#pragma unroll
            for (int k = 0; k < kRowVecs; ++k)
                if (tid + 256 * k < nvec) u[k] = __ldcg(st + tid + 256 * k);
#pragma unroll
            for (int k = 0; k < kRowVecs; ++k)
                if (tid + 256 * k < nvec) v[k] = add4(v[k], u[k]);
        }
        row_finish(v, p.fin, base, p.dim, nvec, tid, red);
    }

    // 3. the last CTA advances the epoch for the next launch on this stream
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(p.ctl + 1, 1u) == gridDim.x - 1) {
            p.ctl[1] = 0;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(p.ctl) = e;
        }
    }
}

size_t tp_sum_buffer_bytes(int T) {
    return kTpSumCtlBytes + (size_t)2 * T * kTpSumMaxRows * sizeof(unsigned) + (size_t)2 * T * kTpSumSlotFloats * sizeof(float);
}

}  // namespace

bool tp_sum_usable(const lumen_ctx *ctx, size_t rows, size_t dim) {
    static const bool off = [] {
        const char *e = getenv("LUMEN_TP_NCCL");
        return e && e[0] == '1';
    }();
    const int T = ctx->tp_size;
    return !off && (T == 2 || T == 4 || T == 8) && ctx->d_tp_sum && rows >= 1 && rows <= kTpSumMaxRows && dim % 4 == 0 &&
           dim % 8 == 0 && dim <= (size_t)kRowVecs * 1024 && rows * dim <= kTpSumSlotFloats;
}

int ensure_tp_sum(lumen_ctx *ctx) {
    if (ctx->tp_size <= 1 || ctx->tp_size > 8 || ctx->d_tp_sum) return LUMEN_OK;
    const size_t bytes = tp_sum_buffer_bytes(ctx->tp_size);
    LUMEN_CUDA(ctx, cudaMalloc(&ctx->d_tp_sum, bytes));
    // only the control words and the flags need a defined start
    LUMEN_CUDA(ctx, cudaMemsetAsync(ctx->d_tp_sum, 0, kTpSumCtlBytes + (size_t)2 * ctx->tp_size * kTpSumMaxRows * sizeof(unsigned),
                                    ctx->stream));
    const int rc = tp_share_buffer(ctx, ctx->d_tp_sum, ctx->tp_sum_peers);  // (collective: also orders the memsets)
    if (rc != LUMEN_OK) {
        tp_unshare_buffer(ctx, ctx->tp_sum_peers);
        cudaFree(ctx->d_tp_sum);
        ctx->d_tp_sum = nullptr;
    }
    return rc;
}

int launch_tp_sum(lumen_ctx *ctx, const float *part, int splits, const float *residual, size_t rows, size_t dim,
                  const TpSumArgs &a, cudaStream_t s) {
    if (!tp_sum_usable(ctx, rows, dim)) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "tensor-parallel sum: %zu x %zu does not fit the exchange buffer", rows, dim);
    TpSumParams p{};
    p.part = part; p.residual = residual;
    p.fin = RowFinish{a.out, a.norm_w, a.eps, a.normed, a.next_hi, a.next_lo};
    p.splits = splits; p.rows = (int)rows; p.dim = (int)dim; p.rank = ctx->tp_rank;
    const size_t flag_words = (size_t)2 * ctx->tp_size * kTpSumMaxRows;
    for (int r = 0; r < ctx->tp_size; ++r) {
        char *b = static_cast<char *>(ctx->tp_sum_peers[r]);
        p.flags[r] = reinterpret_cast<unsigned *>(b + kTpSumCtlBytes);
        p.slots[r] = reinterpret_cast<float *>(b + kTpSumCtlBytes + flag_words * sizeof(unsigned));
    }
    p.ctl = static_cast<unsigned *>(ctx->d_tp_sum);
    p.status = ctx->d_status;
    const unsigned grid = (unsigned)std::min<size_t>(rows, (size_t)ctx->num_sms);  // co-resident: at most one CTA per SM
    if (ctx->tp_size == 2) tp_sum_kernel<2><<<grid, 256, 0, s>>>(p);
    else if (ctx->tp_size == 4) tp_sum_kernel<4><<<grid, 256, 0, s>>>(p);
    else tp_sum_kernel<8><<<grid, 256, 0, s>>>(p);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace lumen
