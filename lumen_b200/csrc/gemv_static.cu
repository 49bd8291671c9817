// lumen_gemv_kn_static: the [K,N]-layout vector-matrix product of lumen_gemv with its split-K partial
// sums kept in a fixed device array of this module instead of a per-call allocation.  The entry point
// calls no allocating or freeing routine of the CUDA runtime (and no host allocator).
#include <mutex>

#include "common.cuh"

namespace {

// Room for the partial sums: splits * N floats.  The launcher aims at about 8 CTAs per SM, which puts
// splits * N near 1184 * 1024 floats (4.7 MB) whatever N is, so 8 MiB covers N up to several hundred
// thousand columns on a 148-SM part; larger requests are refused, never truncated.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) float g_kn_scratch[kStaticScratchBytes / sizeof(float)];

// Address of g_kn_scratch per device ordinal, looked up on the first call made for that device.
constexpr int kMaxDevices = 64;
float *g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mu;

}  // namespace

using namespace lumen;

extern "C" {

int lumen_gemv_kn_static(lumen_ctx *ctx, const float *x_dev, const void *w_dev, lumen_dtype w_dtype, size_t k, size_t n,
                         float *y_dev) {
    if (!ctx || !x_dev || !w_dev || !y_dev) return set_error(ctx, LUMEN_ERR_INVALID, "gemv_kn_static: null argument");
    if (w_dtype != LUMEN_F32 && w_dtype != LUMEN_BF16)
        return set_error(ctx, LUMEN_ERR_DTYPE, "gemv_kn_static: dtype %d", (int)w_dtype);
    if (k == 0 || n == 0) return LUMEN_OK;
    const size_t need = gemv_kn_scratch_bytes_for(k, n, w_dtype, ctx->num_sms);  // what this launch will write
    if (need > kStaticScratchBytes)
        return set_error(ctx, LUMEN_ERR_UNSUPPORTED,
                         "gemv_kn_static: k=%zu n=%zu needs %zu bytes of partial sums, the fixed scratch holds %zu; "
                         "use lumen_gemv for this size",
                         k, n, need, (size_t)kStaticScratchBytes);
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "gemv_kn_static: device ordinal %d beyond %d", ctx->device, kMaxDevices);
    int cur = -1;
    LUMEN_CUDA(ctx, cudaGetDevice(&cur));
    if (cur != ctx->device)
        return set_error(ctx, LUMEN_ERR_INVALID, "gemv_kn_static: current device %d is not the context's device %d", cur,
                         ctx->device);
    float *scratch;
    {
        std::lock_guard<std::mutex> lock(g_scratch_mu);
        scratch = g_scratch_ptr[cur];
        if (!scratch) {
            // First call on this device: resolve the array's address (this may load the module).
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_kn_scratch);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaGetSymbolAddress(g_kn_scratch)");
            if (!p || (reinterpret_cast<uintptr_t>(p) & 255) != 0)
                return set_error(ctx, LUMEN_ERR_CUDA, "gemv_kn_static: scratch address %p is not 256-byte aligned", p);
            scratch = g_scratch_ptr[cur] = static_cast<float *>(p);
        }
    }
    // Nothing has to start at zero: the first kernel writes every partial sum that the second one reads.
    return launch_gemv_kn(ctx, x_dev, w_dev, w_dtype, y_dev, k, n, scratch, ctx->stream);
}

}  // extern "C"
