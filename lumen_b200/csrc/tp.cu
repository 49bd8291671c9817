// Tensor-parallel plumbing: one context = one rank = one GPU; collectives go through NCCL over
// NVLink.  NCCL is bound at run time with dlopen("libnccl.so.2") so that the library carries no
// link-time dependency and shares the NCCL already loaded by the host process when there is one.
// The reference has no multi-device code; the sharding layout (row-split q/k/v/gate/up, column-split
// o/down, one sum-allreduce after each) is described where the model applies it.
#include <dlfcn.h>

#include "common.cuh"

namespace lumen {
namespace {

struct NcclId {
    char bytes[LUMEN_NCCL_ID_BYTES];
};
typedef int (*fn_get_unique_id)(NcclId *);
typedef int (*fn_comm_init_rank)(void **, int, NcclId, int);
typedef int (*fn_comm_destroy)(void *);
typedef int (*fn_all_reduce)(const void *, void *, size_t, int, int, void *, cudaStream_t);
typedef int (*fn_all_gather)(const void *, void *, size_t, int, void *, cudaStream_t);
typedef const char *(*fn_error_string)(int);

struct NcclApi {
    void *handle = nullptr;
    fn_get_unique_id get_unique_id = nullptr;
    fn_comm_init_rank comm_init_rank = nullptr;
    fn_comm_destroy comm_destroy = nullptr;
    fn_all_reduce all_reduce = nullptr;
    fn_all_gather all_gather = nullptr;
    fn_error_string error_string = nullptr;
    bool ok = false;
};

NcclApi &api() {
    static NcclApi a;
    if (a.handle) return a;
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) a.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) return a;
    a.get_unique_id = (fn_get_unique_id)dlsym(a.handle, "ncclGetUniqueId");
    a.comm_init_rank = (fn_comm_init_rank)dlsym(a.handle, "ncclCommInitRank");
    a.comm_destroy = (fn_comm_destroy)dlsym(a.handle, "ncclCommDestroy");
    a.all_reduce = (fn_all_reduce)dlsym(a.handle, "ncclAllReduce");
    a.all_gather = (fn_all_gather)dlsym(a.handle, "ncclAllGather");
    a.error_string = (fn_error_string)dlsym(a.handle, "ncclGetErrorString");
    a.ok = a.get_unique_id && a.comm_init_rank && a.comm_destroy && a.all_reduce && a.all_gather && a.error_string;
    return a;
}

constexpr int kNcclFloat32 = 7;  // ncclFloat32 in nccl.h's ncclDataType_t
constexpr int kNcclSum = 0;      // ncclSum in ncclRedOp_t

int nccl_fail(lumen_ctx *ctx, int rc, const char *what) {
    return set_error(ctx, LUMEN_ERR_NCCL, "NCCL error %d (%s) in %s", rc, api().error_string ? api().error_string(rc) : "?", what);
}

}  // namespace

int tp_init(lumen_ctx *ctx, const void *unique_id) {
    if (!unique_id) return set_error(ctx, LUMEN_ERR_INVALID, "tp_size > 1 needs an NCCL unique id");
    NcclApi &a = api();
    if (!a.ok) return set_error(ctx, LUMEN_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
    NcclId id;
    memcpy(id.bytes, unique_id, sizeof(id.bytes));
    int rc = a.comm_init_rank(&ctx->nccl_comm, ctx->tp_size, id, ctx->tp_rank);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclCommInitRank");
    return LUMEN_OK;
}

void tp_shutdown(lumen_ctx *ctx) {
    if (ctx->nccl_comm && api().ok) api().comm_destroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
}

int tp_allreduce_sum(lumen_ctx *ctx, float *buf, size_t n, cudaStream_t s) {
    if (ctx->tp_size == 1) return LUMEN_OK;
    int rc = api().all_reduce(buf, buf, n, kNcclFloat32, kNcclSum, ctx->nccl_comm, s);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclAllReduce");
    return LUMEN_OK;
}

int tp_allgather(lumen_ctx *ctx, const float *send, float *recv, size_t n_per_rank, cudaStream_t s) {
    if (ctx->tp_size == 1) {
        if (send != recv) LUMEN_CUDA(ctx, cudaMemcpyAsync(recv, send, n_per_rank * 4, cudaMemcpyDeviceToDevice, s));
        return LUMEN_OK;
    }
    int rc = api().all_gather(send, recv, n_per_rank, kNcclFloat32, ctx->nccl_comm, s);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclAllGather");
    return LUMEN_OK;
}

// Makes `local` (a cudaMalloc'ed buffer of this rank) addressable by every rank of the group: the ranks
// trade CUDA IPC handles through an NCCL all-gather and map each other's buffer.  peers_out[r] is a
// pointer valid on THIS device to rank r's buffer (peers_out[tp_rank] == local).  One process per GPU.
// Synchronises the stream.  The mappings stay open for the life of the process.
int tp_share_buffer(lumen_ctx *ctx, void *local, void **peers_out) {
    const int T = ctx->tp_size;
    if (T == 1) {
        peers_out[0] = local;
        return LUMEN_OK;
    }
    if (T > 8) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "peer sharing supports at most 8 ranks, got %d", T);
    cudaIpcMemHandle_t mine;
    LUMEN_CUDA(ctx, cudaIpcGetMemHandle(&mine, local));
    static_assert(sizeof(cudaIpcMemHandle_t) % 4 == 0, "handle is gathered as f32 words");
    constexpr size_t kWords = sizeof(cudaIpcMemHandle_t) / 4;
    float *d_all = nullptr;
    LUMEN_CUDA(ctx, cudaMalloc(&d_all, T * sizeof(cudaIpcMemHandle_t)));
    LUMEN_CUDA(ctx, cudaMemcpyAsync(reinterpret_cast<char *>(d_all) + ctx->tp_rank * sizeof(cudaIpcMemHandle_t), &mine,
                                    sizeof(mine), cudaMemcpyHostToDevice, ctx->stream));
    int rc = tp_allgather(ctx, d_all + ctx->tp_rank * kWords, d_all, kWords, ctx->stream);
    std::vector<cudaIpcMemHandle_t> all(T);
    cudaError_t e = cudaSuccess;
    if (rc == LUMEN_OK) e = cudaMemcpyAsync(all.data(), d_all, T * sizeof(cudaIpcMemHandle_t), cudaMemcpyDeviceToHost, ctx->stream);
    if (rc == LUMEN_OK && e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(d_all);
    if (rc != LUMEN_OK) return rc;
    if (e != cudaSuccess) return cuda_fail(ctx, e, "exchange of IPC handles");
    for (int r = 0; r < T; ++r) {
        if (r == ctx->tp_rank) {
            peers_out[r] = local;
            continue;
        }
        void *p = nullptr;
        e = cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaIpcOpenMemHandle (peer access between the ranks' GPUs is required)");
        peers_out[r] = p;
    }
    return LUMEN_OK;
}

void tp_unshare_buffer(lumen_ctx *ctx, void **peers) {
    for (int r = 0; r < ctx->tp_size && r < 8; ++r) {
        if (r != ctx->tp_rank && peers[r]) cudaIpcCloseMemHandle(peers[r]);
        peers[r] = nullptr;
    }
}

int ensure_exchange(lumen_ctx *ctx, size_t bytes) {
    if (ctx->d_exchange && ctx->exchange_bytes >= bytes) return LUMEN_OK;
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->d_exchange) {
        // every rank drops its mappings of the old buffers before anybody frees one
        tp_unshare_buffer(ctx, ctx->x_peers);
        if (ctx->tp_size > 1) {
            LUMEN_TRY(tp_allreduce_sum(ctx, static_cast<float *>(ctx->d_exchange), 1, ctx->stream));
            LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        }
        cudaFree(ctx->d_exchange);
        ctx->d_exchange = nullptr;
        ctx->exchange_bytes = 0;
    }
    LUMEN_CUDA(ctx, cudaMalloc(&ctx->d_exchange, bytes));
    ctx->exchange_bytes = bytes;
    LUMEN_CUDA(ctx, cudaMemsetAsync(ctx->d_exchange, 0, bytes, ctx->stream));
    ctx->mega_epoch = 1;  // clean buffers: the tags start over
    return tp_share_buffer(ctx, ctx->d_exchange, ctx->x_peers);  // (collective: also orders the memsets)
}

}  // namespace lumen

extern "C" int lumen_nccl_unique_id(void *id_out_128_bytes) {
    if (!id_out_128_bytes) return LUMEN_ERR_INVALID;
    auto &a = lumen::api();
    if (!a.ok) return LUMEN_ERR_NCCL;
    lumen::NcclId id;
    int rc = a.get_unique_id(&id);
    if (rc != 0) return LUMEN_ERR_NCCL;
    memcpy(id_out_128_bytes, id.bytes, sizeof(id.bytes));
    return LUMEN_OK;
}
