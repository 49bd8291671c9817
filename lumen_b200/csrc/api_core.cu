// C ABI: context, error reporting, device memory and the Tensor handle.
#include <dlfcn.h>

#include <algorithm>
#include <cmath>

#include "common.cuh"

namespace lumen {

int set_error(lumen_ctx *ctx, int code, const char *fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

int cuda_fail(lumen_ctx *ctx, cudaError_t e, const char *what) {
    return set_error(ctx, LUMEN_ERR_CUDA, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

int dev_alloc(lumen_ctx *ctx, size_t bytes, void **out) {
    *out = nullptr;
    if (bytes == 0) bytes = 16;
    LUMEN_CUDA(ctx, cudaMallocAsync(out, bytes, ctx->stream));
    return LUMEN_OK;
}

int dev_free(lumen_ctx *ctx, void *p) {
    if (!p) return LUMEN_OK;
    LUMEN_CUDA(ctx, cudaFreeAsync(p, ctx->stream));
    return LUMEN_OK;
}

int new_tensor(lumen_ctx *ctx, const size_t *shape, int ndim, lumen_dtype dt, lumen_tensor **out) {
    if (!ctx || !out || ndim < 0 || (ndim > 0 && !shape)) return set_error(ctx, LUMEN_ERR_INVALID, "new_tensor: bad argument");
    auto *t = new lumen_tensor();
    t->ctx = ctx;
    t->dtype = dt;
    t->shape.assign(shape, shape + ndim);
    auto *st = new lumen_storage();
    st->ctx = ctx;
    st->bytes = t->numel() * t->elem_size();
    int rc = dev_alloc(ctx, st->bytes, &st->ptr);
    if (rc != LUMEN_OK) {
        delete st;
        delete t;
        return rc;
    }
    t->st = st;
    *out = t;
    return LUMEN_OK;
}

// Reads the device status word; called by the synchronising entry points.
int check_device_status(lumen_ctx *ctx) {
    LUMEN_CUDA(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(DeviceStatus), cudaMemcpyDeviceToHost, ctx->stream));
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->h_status->code != 0) {
        int code = ctx->h_status->code, d0 = ctx->h_status->detail0, d1 = ctx->h_status->detail1;
        ctx->abort_gen += 1;  // host mirrors of the cache lengths may be ahead of the device: see kv_resync_len
        LUMEN_CUDA(ctx, cudaMemsetAsync(ctx->d_status, 0, sizeof(DeviceStatus), ctx->stream));
        // A persistent decode kernel that gave up leaves its abort flag raised: clear it.
        LUMEN_CUDA(ctx, cudaMemsetAsync(ctx->d_mega_sync, 0, 16, ctx->stream));
        if (code == LUMEN_ERR_EMBED_RANGE) return set_error(ctx, code, "Embedding index out of bounds: id %d at position %d", d1, d0);
        if (code == LUMEN_ERR_TIMEOUT) return set_error(ctx, code, "device-side wait gave up (site %d, value %d)", d0, d1);
        return set_error(ctx, code, "device status %d (%d, %d)", code, d0, d1);
    }
    return LUMEN_OK;
}

int kv_resync_len(lumen_kv_cache *c) {
    if (!c || !c->ctx || c->seen_abort == c->ctx->abort_gen) return LUMEN_OK;
    lumen_ctx *ctx = c->ctx;
    int dev_len = 0;
    LUMEN_CUDA(ctx, cudaMemcpyAsync(&dev_len, c->d_len, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    c->len = dev_len < 0 ? 0 : (size_t)dev_len;
    c->seen_abort = ctx->abort_gen;
    return LUMEN_OK;
}

}  // namespace lumen

using namespace lumen;

extern "C" {

int lumen_version(void) { return 100; }

const char *lumen_status_string(int status) {
    switch (status) {
        case LUMEN_OK: return "ok";
        case LUMEN_ERR_INVALID: return "invalid argument";
        case LUMEN_ERR_SHAPE: return "shape mismatch";
        case LUMEN_ERR_KV_OVERFLOW: return "KV cache overflow";
        case LUMEN_ERR_ROPE_RANGE: return "RoPE index out of range";
        case LUMEN_ERR_EMBED_RANGE: return "Embedding index out of bounds";
        case LUMEN_ERR_CACHE_COUNT: return "KV cache count mismatch";
        case LUMEN_ERR_CUDA: return "CUDA failure";
        case LUMEN_ERR_NCCL: return "NCCL failure";
        case LUMEN_ERR_TIMEOUT: return "bounded wait timed out";
        case LUMEN_ERR_DTYPE: return "unsupported dtype";
        case LUMEN_ERR_PARAM_NAME: return "unknown parameter name";
        case LUMEN_ERR_UNSUPPORTED: return "unsupported configuration";
        case LUMEN_ERR_MISSING_PARAM: return "parameter not set";
        default: return "unknown status";
    }
}

const char *lumen_last_error(const lumen_ctx *ctx) { return ctx ? ctx->err : "null context"; }

int lumen_ctx_create(int device, int tp_rank, int tp_size, const void *nccl_unique_id, lumen_ctx **out) {
    if (!out) return LUMEN_ERR_INVALID;
    *out = nullptr;
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return LUMEN_ERR_INVALID;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0 || device < 0 || device >= count) return LUMEN_ERR_CUDA;  // no CPU fallback
    auto *ctx = new lumen_ctx();
    ctx->device = device;
    ctx->tp_rank = tp_rank;
    ctx->tp_size = tp_size;
    auto fail = [&](cudaError_t err, const char *what) {
        fprintf(stderr, "lumen_ctx_create: %s: %s\n", what, cudaGetErrorString(err));
        lumen_ctx_destroy(ctx);  // frees whatever was created so far
        return LUMEN_ERR_CUDA;
    };
    if ((e = cudaSetDevice(device)) != cudaSuccess) return fail(e, "cudaSetDevice");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return fail(e, "cudaGetDeviceProperties");
    if (prop.major != 10) {
        fprintf(stderr, "lumen_ctx_create: device %d is sm_%d%d; this library is built for sm_100a only\n", device,
                prop.major, prop.minor);
        lumen_ctx_destroy(ctx);
        return LUMEN_ERR_UNSUPPORTED;
    }
    ctx->num_sms = prop.multiProcessorCount;
    if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e, "cudaStreamCreate");
    cudaMemPool_t pool;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
        uint64_t keep = ~0ull;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    if ((e = cudaMalloc(&ctx->d_status, sizeof(DeviceStatus))) != cudaSuccess) return fail(e, "cudaMalloc(status)");
    if ((e = cudaMemset(ctx->d_status, 0, sizeof(DeviceStatus))) != cudaSuccess) return fail(e, "cudaMemset(status)");
    if ((e = cudaMallocHost(&ctx->h_status, sizeof(DeviceStatus))) != cudaSuccess) return fail(e, "cudaMallocHost(status)");
    if ((e = cudaMalloc(&ctx->d_mega_sync, 16)) != cudaSuccess) return fail(e, "cudaMalloc(barrier)");
    if ((e = cudaMemset(ctx->d_mega_sync, 0, 16)) != cudaSuccess) return fail(e, "cudaMemset(barrier)");
    if (tp_size > 1) {
        int rc = tp_init(ctx, nccl_unique_id);
        if (rc != LUMEN_OK) {
            fprintf(stderr, "lumen_ctx_create: %s\n", ctx->err);
            lumen_ctx_destroy(ctx);
            return rc;
        }
    }
    *out = ctx;
    return LUMEN_OK;
}

int lumen_ctx_destroy(lumen_ctx *ctx) {
    if (!ctx) return LUMEN_ERR_INVALID;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->sampler_ws) cudaFree(ctx->sampler_ws);
    if (ctx->d_exchange) {
        tp_unshare_buffer(ctx, ctx->x_peers);
        cudaFree(ctx->d_exchange);
    }
    if (ctx->d_tp_sum) {
        tp_unshare_buffer(ctx, ctx->tp_sum_peers);
        cudaFree(ctx->d_tp_sum);
    }
    if (ctx->nccl_comm) {
        tp_shutdown(ctx);
    }
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_mega_sync) cudaFree(ctx->d_mega_sync);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return LUMEN_OK;
}

int lumen_ctx_synchronize(lumen_ctx *ctx) {
    if (!ctx) return LUMEN_ERR_INVALID;
    return check_device_status(ctx);
}

void *lumen_ctx_stream(lumen_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

uint64_t lumen_ctx_launch_count(const lumen_ctx *ctx) { return ctx ? ctx->launches : 0; }

// ---- tensors ---------------------------------------------------------------------------------------
int lumen_tensor_from_host(lumen_ctx *ctx, const float *data, const size_t *shape, int ndim, lumen_tensor **out) {
    if (!ctx || !data) return set_error(ctx, LUMEN_ERR_INVALID, "tensor_from_host: null argument");
    LUMEN_TRY(new_tensor(ctx, shape, ndim, LUMEN_F32, out));
    size_t bytes = (*out)->numel() * 4;
    if (bytes) LUMEN_CUDA(ctx, cudaMemcpyAsync((*out)->data(), data, bytes, cudaMemcpyHostToDevice, ctx->stream));
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the host buffer may be reused on return
    return LUMEN_OK;
}

int lumen_tensor_from_host_bf16(lumen_ctx *ctx, const uint16_t *data, const size_t *shape, int ndim, lumen_tensor **out) {
    if (!ctx || !data) return set_error(ctx, LUMEN_ERR_INVALID, "tensor_from_host_bf16: null argument");
    LUMEN_TRY(new_tensor(ctx, shape, ndim, LUMEN_BF16, out));
    size_t bytes = (*out)->numel() * 2;
    if (bytes) LUMEN_CUDA(ctx, cudaMemcpyAsync((*out)->data(), data, bytes, cudaMemcpyHostToDevice, ctx->stream));
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return LUMEN_OK;
}

int lumen_tensor_empty(lumen_ctx *ctx, const size_t *shape, int ndim, lumen_dtype dtype, lumen_tensor **out) {
    if (dtype != LUMEN_F32 && dtype != LUMEN_BF16) return set_error(ctx, LUMEN_ERR_DTYPE, "tensor_empty: dtype %d", (int)dtype);
    return new_tensor(ctx, shape, ndim, dtype, out);
}

int lumen_tensor_ndim(const lumen_tensor *t) { return t ? (int)t->shape.size() : -1; }

int lumen_tensor_shape(const lumen_tensor *t, size_t *shape_out) {
    if (!t || !shape_out) return LUMEN_ERR_INVALID;
    std::copy(t->shape.begin(), t->shape.end(), shape_out);
    return LUMEN_OK;
}

size_t lumen_tensor_numel(const lumen_tensor *t) { return t ? t->numel() : 0; }
lumen_dtype lumen_tensor_dtype(const lumen_tensor *t) { return t ? t->dtype : LUMEN_F32; }
void *lumen_tensor_data(const lumen_tensor *t) { return t ? t->data() : nullptr; }

namespace {
__global__ void bf16_to_f32_kernel(const __nv_bfloat16 *in, float *out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __bfloat162float(in[i]);
}
}  // namespace

int lumen_tensor_to_host(const lumen_tensor *t, float *out) {
    if (!t || !out) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = t->ctx;
    size_t n = t->numel();
    if (n == 0) return LUMEN_OK;
    if (t->dtype == LUMEN_F32) {
        LUMEN_CUDA(ctx, cudaMemcpyAsync(out, t->data(), n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    } else {
        void *tmp = nullptr;
        LUMEN_TRY(dev_alloc(ctx, n * 4, &tmp));
        bf16_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, ctx->stream>>>(
            static_cast<const __nv_bfloat16 *>(t->data()), static_cast<float *>(tmp), n);
        LUMEN_LAUNCHED(ctx);
        LUMEN_CUDA(ctx, cudaMemcpyAsync(out, tmp, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        LUMEN_TRY(dev_free(ctx, tmp));
    }
    return check_device_status(ctx);
}

int lumen_tensor_set(lumen_tensor *t, const float *data) {
    if (!t || !data) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = t->ctx;
    if (t->dtype != LUMEN_F32) return set_error(ctx, LUMEN_ERR_DTYPE, "tensor_set: only f32 tensors can be set from f32 data");
    if (t->numel()) LUMEN_CUDA(ctx, cudaMemcpyAsync(t->data(), data, t->numel() * 4, cudaMemcpyHostToDevice, ctx->stream));
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return LUMEN_OK;
}

int lumen_tensor_reshape(const lumen_tensor *t, const int64_t *shape, int ndim, lumen_tensor **out) {
    if (!t || !out || ndim < 0 || (ndim > 0 && !shape)) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = t->ctx;
    std::vector<size_t> ns(ndim);
    size_t known = 1;
    int infer = -1;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] == -1) {
            if (infer >= 0) return set_error(ctx, LUMEN_ERR_SHAPE, "reshape: more than one -1");
            infer = i;
        } else if (shape[i] < 0) {
            return set_error(ctx, LUMEN_ERR_SHAPE, "reshape: negative dimension");
        } else {
            ns[i] = (size_t)shape[i];
            known *= ns[i];
        }
    }
    size_t n = t->numel();
    if (infer >= 0) {
        if (known == 0 || n % known) return set_error(ctx, LUMEN_ERR_SHAPE, "reshape: cannot infer dimension");
        ns[infer] = n / known;
        known *= ns[infer];
    }
    if (known != n) return set_error(ctx, LUMEN_ERR_SHAPE, "reshape: %zu elements into %zu", n, known);
    auto *r = new lumen_tensor(*t);
    r->shape = ns;
    r->st->refs += 1;
    *out = r;
    return LUMEN_OK;
}

int lumen_tensor_free(lumen_tensor *t) {
    if (!t) return LUMEN_ERR_INVALID;
    int rc = LUMEN_OK;
    if (t->st && --t->st->refs == 0) {
        rc = dev_free(t->ctx, t->st->ptr);
        delete t->st;
    }
    delete t;
    return rc;
}

}  // extern "C"
