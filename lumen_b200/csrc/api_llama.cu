// C ABI: LlamaModel (src/models/llama.rs of the reference) on one GPU or one tensor-parallel rank.
//
// Memory: one device slab holds every weight of the rank (q/k/v rows of a layer are stored back to
// back so the three projections are one vector-matrix launch), one slab holds the KV caches of all
// layers, one workspace holds the activations of the largest batch seen.  A decode step allocates
// nothing.  Decode steps (S == 1) are captured once per batch size into a CUDA graph and replayed;
// the context length is read from device memory so the same graph serves every position.
//
// Tensor parallelism (new; the reference is single-process): q/k/v/gate/up are split by output row
// (whole heads per rank, KV heads replicated when there are fewer than ranks), o/down by input
// column with a sum-allreduce after each, lm_head by vocabulary row with an allgather.
#include <algorithm>
#include <cmath>
#include <map>
#include <tuple>

#include "common.cuh"
#include "decode_mega.cuh"
#include "tp_plan.cuh"

using namespace lumen;

namespace {

struct LayerW {
    char *wqkv = nullptr;  // [(qd_l + 2*kvd_l), H]
    char *wo = nullptr;    // [H, qd_l]
    char *wgate = nullptr; // [I_l, H]
    char *wup = nullptr;   // [I_l, H]
    char *wdown = nullptr; // [H, I_l]
    float *norm1 = nullptr, *norm2 = nullptr, *qn = nullptr, *kn = nullptr;
};

struct Workspace {
    size_t M = 0;
    char *base = nullptr;
    float *x = nullptr, *nx = nullptr, *qkv = nullptr, *att = nullptr, *act = nullptr, *gate = nullptr, *up = nullptr;
    float *logits = nullptr, *logits_local = nullptr, *last_x = nullptr, *part = nullptr, *ids = nullptr;
    // bf16 hi/lo split of the activations the next tensor-core product reads (written by the kernel that finishes the
    // previous product): [M, max(H, I_l)] each
    __nv_bfloat16 *p_hi = nullptr, *p_lo = nullptr;
    size_t part_bytes = 0;
    float *h_ids = nullptr;     // pinned
    float *h_logits = nullptr;  // pinned
    size_t h_logits_elems = 0;
};

constexpr int kMaxSplits = 64;

__global__ void f32_to_bf16_kernel(const float *in, __nv_bfloat16 *out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void bf16_to_f32_kernel2(const __nv_bfloat16 *in, float *out, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __bfloat162float(in[i]);
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct lumen_llama {
    lumen_ctx *ctx = nullptr;
    lumen_llama_config cfg{};
    size_t D = 0, H = 0, V = 0, I = 0, L = 0;
    size_t hq_l = 0, hkv_l = 0, qd_l = 0, kvd_l = 0, inter_l = 0, vocab_l = 0, qkv_rows = 0;
    size_t kv_head0 = 0, q_head0 = 0;  // first global head owned by this rank
    size_t esz = 4;
    char *wslab = nullptr;
    // f32 weights only: bf16 hi and lo halves of the whole slab (same layout at half the offsets), built before the first
    // tensor-core product and dropped when a parameter changes, so that prefill and batched steps do not split the
    // weights again on every call.  Costs as many bytes as the weights; absent (null) when that allocation fails.
    __nv_bfloat16 *wsplit = nullptr;
    bool wsplit_valid = false, wsplit_failed = false;
    size_t wbytes = 0, stream_bytes = 0;
    std::vector<LayerW> layers;
    char *embed = nullptr, *lm_head = nullptr;
    float *final_norm = nullptr;
    float *cos_t = nullptr, *sin_t = nullptr;
    std::map<std::string, bool> is_set;
    size_t n_expected = 0;
    Workspace ws;
    // decode graphs keyed by (batch, splits, first cache's k pointer)
    std::map<std::tuple<size_t, int, const void *>, cudaGraphExec_t> graphs;
    std::map<std::tuple<size_t, int, const void *>, int> eager_runs;
    std::map<std::tuple<size_t, int, const void *>, unsigned long long> graph_nodes;
    bool use_graph = true;
    // persistent whole-step decode kernel (batch 1)
    bool use_mega = true;
    MegaLayer *d_mega_layers = nullptr;
    uint4 *d_sched = nullptr;      // producer schedule of the persistent kernel (see MegaParams::sched)
    int *d_sched_count = nullptr;
    size_t sched_capacity = 0;
    int sched_stride = 0;
    CUtensorMap *d_tmaps = nullptr;   // tensor maps of the segmented matrices (see MegaParams::tmaps); null when there are none
    size_t tmaps_capacity = 0;
    const void *mega_key = nullptr;  // first cache's k pointer the layer table was built for
    unsigned long long *d_trace = nullptr;  // phase timestamps of the last persistent step (LUMEN_DECODE_TRACE=1)
};

namespace {

void drop_graphs(lumen_llama *m) {
    for (auto &kv : m->graphs) cudaGraphExecDestroy(kv.second);
    m->graphs.clear();
    m->eager_runs.clear();
}

int ensure_workspace(lumen_llama *m, size_t M) {
    Workspace &w = m->ws;
    lumen_ctx *ctx = m->ctx;
    LUMEN_TRY(ensure_tp_sum(ctx));  // (every rank passes here at the same points; no-op after the first time)
    if (M <= w.M) return LUMEN_OK;
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    drop_graphs(m);
    if (w.base) cudaFree(w.base);
    if (w.h_ids) cudaFreeHost(w.h_ids);
    if (w.h_logits) cudaFreeHost(w.h_logits);
    w = Workspace();
    const size_t T = ctx->tp_size;
    const size_t qkvd = m->qkv_rows;
    // Decode batches never exceed M; the attention scratch is sized for the largest split count.
    w.part_bytes = attn_decode_scratch_bytes(M, m->hq_l, m->D, kMaxSplits);
    size_t off = 0;
    auto take = [&](size_t elems) {
        size_t o = off;
        off += align_up(elems * sizeof(float), 256);
        return o;
    };
    size_t o_x = take(M * m->H), o_nx = take(M * m->H), o_qkv = take(M * qkvd), o_att = take(M * m->qd_l);
    // gate and up are adjacent: the fused step runs them as one product into [M, 2 * I_l]
    size_t o_act = take(M * m->inter_l), o_gate = take(2 * M * m->inter_l);
    const size_t pair_floats = (M * std::max(m->H, m->inter_l) + 1) / 2 + 8;
    size_t o_phi = take(pair_floats), o_plo = take(pair_floats);
    size_t o_logits = take(M * m->V), o_ll = take(T > 1 ? T * M * m->vocab_l : 0), o_last = take(M * m->H);
    size_t o_part = take(w.part_bytes / sizeof(float)), o_ids = take(M);
    LUMEN_CUDA(ctx, cudaMalloc(&w.base, off));
    auto at = [&](size_t o) { return reinterpret_cast<float *>(w.base + o); };
    w.x = at(o_x); w.nx = at(o_nx); w.qkv = at(o_qkv); w.att = at(o_att); w.act = at(o_act); w.gate = at(o_gate);
    w.up = w.gate + M * m->inter_l; w.p_hi = reinterpret_cast<__nv_bfloat16 *>(at(o_phi)); w.p_lo = reinterpret_cast<__nv_bfloat16 *>(at(o_plo));
    w.logits = at(o_logits); w.logits_local = at(o_ll); w.last_x = at(o_last); w.part = at(o_part);
    w.ids = at(o_ids);
    LUMEN_CUDA(ctx, cudaMallocHost(&w.h_ids, std::max<size_t>(M, 1) * sizeof(float)));
    w.h_logits_elems = std::min<size_t>(M * m->V, (size_t)16 << 20);  // pinned staging up to 64 MB
    LUMEN_CUDA(ctx, cudaMallocHost(&w.h_logits, std::max<size_t>(w.h_logits_elems, 1) * sizeof(float)));
    w.M = M;
    return LUMEN_OK;
}

// Copies the [rows x ncols] block starting at column col0 of a row-major host matrix with `cols_total`
// columns into a dense device matrix of dtype dst_dt, converting between f32 and bf16 when needed.
int upload_block(lumen_ctx *ctx, void *dst, lumen_dtype dst_dt, const void *src_host, lumen_dtype src_dt, size_t rows,
                 size_t cols_total, size_t col0, size_t ncols) {
    if (rows == 0 || ncols == 0) return LUMEN_OK;
    const size_t se = src_dt == LUMEN_F32 ? 4 : 2;
    const char *src = static_cast<const char *>(src_host) + col0 * se;
    cudaStream_t s = ctx->stream;
    if (src_dt == dst_dt) {
        LUMEN_CUDA(ctx, cudaMemcpy2DAsync(dst, ncols * se, src, cols_total * se, ncols * se, rows, cudaMemcpyHostToDevice, s));
        LUMEN_CUDA(ctx, cudaStreamSynchronize(s));
        return LUMEN_OK;
    }
    // Convert in row chunks to bound the staging buffer.
    const size_t chunk_rows = std::max<size_t>(1, ((size_t)64 << 20) / (ncols * se));
    void *tmp = nullptr;
    LUMEN_CUDA(ctx, cudaMalloc(&tmp, std::min(rows, chunk_rows) * ncols * se));
    const size_t de = dst_dt == LUMEN_F32 ? 4 : 2;
    int rc = LUMEN_OK;
    for (size_t r0 = 0; r0 < rows && rc == LUMEN_OK; r0 += chunk_rows) {
        const size_t nr = std::min(chunk_rows, rows - r0), n = nr * ncols;
        cudaError_t e = cudaMemcpy2DAsync(tmp, ncols * se, src + r0 * cols_total * se, cols_total * se, ncols * se, nr,
                                          cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) { rc = cuda_fail(ctx, e, "cudaMemcpy2DAsync"); break; }
        char *d = static_cast<char *>(dst) + r0 * ncols * de;
        if (dst_dt == LUMEN_BF16)
            f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const float *)tmp, (__nv_bfloat16 *)d, n);
        else
            bf16_to_f32_kernel2<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const __nv_bfloat16 *)tmp, (float *)d, n);
        e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) rc = cuda_fail(ctx, e, "convert upload");
    }
    cudaFree(tmp);
    return rc;
}

int ensure_weight_split(lumen_llama *m) {
    if (m->cfg.weight_dtype != LUMEN_F32 || m->wsplit_valid || m->wsplit_failed) return LUMEN_OK;
    static const bool off = [] {
        const char *e = getenv("LUMEN_NO_WEIGHT_SPLIT_CACHE");
        return e && e[0] == '1';
    }();
    if (off) return LUMEN_OK;
    lumen_ctx *ctx = m->ctx;
    const size_t n = m->wbytes / 4;
    if (!m->wsplit) {
        void *p = nullptr;
        if (cudaMalloc(&p, 2 * n * sizeof(__nv_bfloat16)) != cudaSuccess) {
            cudaGetLastError();  // no room: the products keep splitting per call
            m->wsplit_failed = true;
            return LUMEN_OK;
        }
        m->wsplit = static_cast<__nv_bfloat16 *>(p);
    }
    LUMEN_TRY(launch_split_bf16(ctx, reinterpret_cast<const float *>(m->wslab), m->wsplit, m->wsplit + n, n, ctx->stream));
    m->wsplit_valid = true;
    return LUMEN_OK;
}

// Points a product's fusion record at the kept split of the f32 weight matrix `wp` (no-op without one).
void use_weight_split(const lumen_llama *m, const void *wp, GemmFuse &f) {
    if (!m->wsplit_valid) return;
    const size_t at = (size_t)(static_cast<const char *>(wp) - m->wslab) / 4;
    f.w_hi = m->wsplit + at;
    f.w_lo = m->wsplit + m->wbytes / 4 + at;
}

struct StepPlan {
    size_t B, S, M;
    bool decode;
    int nsplit;
};

// Enqueues one forward pass over ws.ids[M] on the context stream.  `last_only` restricts the final norm
// and lm_head to the last position of each sequence.  Logits land in ws.logits ([M,V] or [B,V]).
int enqueue_forward(lumen_llama *m, const StepPlan &p, lumen_kv_cache **caches, bool last_only) {
    lumen_ctx *ctx = m->ctx;
    cudaStream_t s = ctx->stream;
    Workspace &w = m->ws;
    const size_t M = p.M, H = m->H, qkvd = m->qkv_rows;
    const lumen_dtype wdt = m->cfg.weight_dtype;
    // Row counts that take the streaming vector-matrix kernels: up to 8 rows over f32 weights, a single row over
    // bf16 weights (from two rows on the tensor-core kernel with split K is faster there).
    const size_t vec_rows = (wdt == LUMEN_BF16 && gemm_tc_usable(wdt, 2, H, H, m->lm_head)) ? 1 : 8;
    const bool vec = M <= vec_rows && M * std::max(H, std::max(m->inter_l, m->qd_l)) * 4 <= 200 * 1024;
    const bool tp = ctx->tp_size > 1;
    const float eps = m->cfg.rms_norm_eps;
    const float scale = 1.0f / sqrtf((float)m->D);  // (head_dim as f32).sqrt().recip(), self_attention.rs:89
    const float *res_x = (!tp || ctx->tp_rank == 0) ? w.x : nullptr;

    // Fused step (tiled products only): every product's finishing kernel writes what the next product reads, as the bf16
    // hi/lo pair in w.p_hi / w.p_lo, and gate and up run as one product over their adjacent weights.  Per block:
    // qkv product + split-K sum, attention, o_proj (split + product + finisher), gate/up (product + finisher),
    // down (product + finisher) = 11 launches instead of 20.
    static const bool no_fuse = [] {
        const char *e = getenv("LUMEN_NO_STEP_FUSE");
        return e && e[0] == '1';
    }();
    bool fuse = !vec && !no_fuse && row_finish_usable(H) && m->inter_l % 8 == 0 && m->qd_l % 8 == 0 && m->L > 0;
    for (size_t l = 0; fuse && l < m->L; ++l) {
        const LayerW &lw = m->layers[l];
        fuse = lw.wup == lw.wgate + m->inter_l * H * m->esz && gemm_tc_usable(wdt, M, H, qkvd, lw.wqkv) &&
               gemm_tc_usable(wdt, M, m->qd_l, H, lw.wo) && gemm_tc_usable(wdt, M, H, 2 * m->inter_l, lw.wgate) &&
               gemm_tc_usable(wdt, M, m->inter_l, H, lw.wdown);
    }

    auto attend = [&](const LayerW &lw, lumen_kv_cache *c) -> int {
        if (p.decode) {
            AttnDecodeArgs a;
            a.q = w.qkv; a.k_new = w.qkv + m->qd_l; a.v_new = w.qkv + m->qd_l + m->kvd_l;
            a.q_stride = qkvd; a.kv_stride = qkvd;
            a.k_cache = c->k; a.v_cache = c->v; a.d_len = c->d_len;
            a.B = p.B; a.Hq = m->hq_l; a.Hkv = m->hkv_l; a.D = m->D; a.max_seq = c->max_seq;
            a.cos_t = m->cos_t; a.sin_t = m->sin_t;
            a.q_norm = lw.qn; a.k_norm = lw.kn; a.norm_eps = eps;
            a.scale = scale; a.out = w.att; a.part = w.part; a.max_splits = p.nsplit; a.len_hint = c->len;
            return launch_attn_decode(ctx, a, s);
        }
        AttnPrefillArgs a;
        a.q = w.qkv; a.k = w.qkv + m->qd_l; a.v = w.qkv + m->qd_l + m->kvd_l;
        a.q_stride = qkvd; a.kv_stride = qkvd;
        a.k_cache = c->k; a.v_cache = c->v;
        a.past = c->len; a.S = p.S; a.B = p.B; a.Hq = m->hq_l; a.Hkv = m->hkv_l; a.D = m->D; a.max_seq = c->max_seq;
        a.cos_t = m->cos_t; a.sin_t = m->sin_t;
        a.q_norm = lw.qn; a.k_norm = lw.kn; a.norm_eps = eps;
        a.scale = scale; a.causal = 1; a.out = w.att;
        LUMEN_TRY(launch_attn_prefill(ctx, a, s));
        return launch_bump_len(ctx, c->d_len, (int)p.S, s);
    };
    // Row-parallel product of the fused step: x = x + a . W^T summed over the ranks, and the split of RMSNorm(x) * norm_w
    // for the next product (norm_w null after the last block).  `a` null: the activations are the pair already.
    auto row_parallel = [&](const float *a, const void *wmat, size_t K, const float *norm_w) -> int {
        GemmFuse f;
        use_weight_split(m, wmat, f);
        if (!a) { f.a_hi = w.p_hi; f.a_lo = w.p_lo; }
        if (!tp) {
            f.post = GemmFuse::kPostNorm; f.norm_w = norm_w; f.eps = eps; f.next_hi = w.p_hi; f.next_lo = w.p_lo;
            return launch_gemm_tc(ctx, a, wmat, wdt, w.x, M, K, H, res_x, s, nullptr, &f);
        }
        if (tp_sum_usable(ctx, M, H)) {
            TpSumArgs t;
            t.out = w.x; t.norm_w = norm_w; t.eps = eps;
            if (norm_w) { t.next_hi = w.p_hi; t.next_lo = w.p_lo; }
            return launch_gemm_tc(ctx, a, wmat, wdt, w.x, M, K, H, res_x, s, &t, &f);
        }
        // too many rows for the fused exchange (long prefill slices are bandwidth-bound): NCCL, then the norm + split
        LUMEN_TRY(launch_gemm_tc(ctx, a, wmat, wdt, w.x, M, K, H, res_x, s, nullptr, &f));
        LUMEN_TRY(tp_allreduce_sum(ctx, w.x, M * H, s));
        if (norm_w) return launch_sum_norm_split(ctx, w.x, 1, nullptr, M, H, nullptr, norm_w, eps, w.p_hi, w.p_lo, s);
        return LUMEN_OK;
    };

    LUMEN_TRY(launch_embedding(ctx, w.ids, m->embed, wdt, w.x, M, m->V, H, s));
    bool nx_ready = false;  // w.nx (or, fused, the pair) already holds Norm(x) of the block about to run
    for (size_t l = 0; l < m->L; ++l) {
        const LayerW &lw = m->layers[l];
        lumen_kv_cache *c = caches[l];
        if (fuse) {
            if (!nx_ready) LUMEN_TRY(launch_sum_norm_split(ctx, w.x, 1, nullptr, M, H, nullptr, lw.norm1, eps, w.p_hi, w.p_lo, s));
            GemmFuse fq;
            fq.a_hi = w.p_hi; fq.a_lo = w.p_lo;
            use_weight_split(m, lw.wqkv, fq);
            LUMEN_TRY(launch_gemm_tc(ctx, nullptr, lw.wqkv, wdt, w.qkv, M, H, qkvd, nullptr, s, nullptr, &fq));
            LUMEN_TRY(attend(lw, c));
            LUMEN_TRY(row_parallel(w.att, lw.wo, m->qd_l, lw.norm2));
            GemmFuse fg;
            fg.a_hi = w.p_hi; fg.a_lo = w.p_lo; fg.post = GemmFuse::kPostSwiglu; fg.next_hi = w.p_hi; fg.next_lo = w.p_lo;
            use_weight_split(m, lw.wgate, fg);
            LUMEN_TRY(launch_gemm_tc(ctx, nullptr, lw.wgate, wdt, w.gate, M, H, 2 * m->inter_l, nullptr, s, nullptr, &fg));
            nx_ready = l + 1 < m->L;
            LUMEN_TRY(row_parallel(nullptr, lw.wdown, m->inter_l, nx_ready ? m->layers[l + 1].norm1 : nullptr));
            continue;
        }
        // h = x + Attention(Norm(x))                                   llama.rs:107-110
        if (vec) {
            GemvArgs g;
            g.x = w.x; g.w = lw.wqkv; g.wdt = wdt; g.y = w.qkv; g.M = (int)M; g.K = H; g.N = qkvd; g.ldy = qkvd;
            g.norm_w = lw.norm1; g.norm_eps = eps;
            LUMEN_TRY(launch_gemv_nk(ctx, g, s));
        } else {
            if (!nx_ready) LUMEN_TRY(launch_rmsnorm(ctx, w.x, lw.norm1, eps, w.nx, M, H, s));
            LUMEN_TRY(launch_gemm_nk(ctx, w.nx, lw.wqkv, wdt, w.qkv, M, H, qkvd, nullptr, s));
        }
        LUMEN_TRY(attend(lw, c));
        // With tensor parallelism the sum over the ranks follows the product in the same call, and (outside the
        // vector path, which folds the norm into its next product) leaves Norm(x) for the next product in w.nx.
        TpSumArgs sum_o;
        sum_o.out = w.x;
        if (tp && !vec) { sum_o.norm_w = lw.norm2; sum_o.normed = w.nx; sum_o.eps = eps; }
        LUMEN_TRY(matmul_dispatch(ctx, w.att, lw.wo, wdt, w.x, M, m->qd_l, H, res_x, s, tp ? &sum_o : nullptr));
        // out = h + MLP(Norm(h))                                       llama.rs:113-115, :59-65
        if (vec) {
            LUMEN_TRY(launch_gemv_gate_up(ctx, w.x, lw.wgate, lw.wup, wdt, w.act, (int)M, H, m->inter_l, lw.norm2, eps, s));
        } else {
            if (!tp) LUMEN_TRY(launch_rmsnorm(ctx, w.x, lw.norm2, eps, w.nx, M, H, s));
            LUMEN_TRY(launch_gemm_nk(ctx, w.nx, lw.wgate, wdt, w.gate, M, H, m->inter_l, nullptr, s));
            LUMEN_TRY(launch_gemm_nk(ctx, w.nx, lw.wup, wdt, w.up, M, H, m->inter_l, nullptr, s));
            LUMEN_TRY(launch_silu_mul(ctx, w.gate, w.up, w.act, M * m->inter_l, s));
        }
        TpSumArgs sum_d;
        sum_d.out = w.x;
        nx_ready = tp && !vec && l + 1 < m->L;
        if (nx_ready) { sum_d.norm_w = m->layers[l + 1].norm1; sum_d.normed = w.nx; sum_d.eps = eps; }
        LUMEN_TRY(matmul_dispatch(ctx, w.act, lw.wdown, wdt, w.x, M, m->inter_l, H, res_x, s, tp ? &sum_d : nullptr));
    }
    // Final norm + lm_head                                             llama.rs:202-205
    const float *xin = w.x;
    size_t rows = M;
    if (last_only && p.S > 1) {
        LUMEN_CUDA(ctx, cudaMemcpy2DAsync(w.last_x, H * 4, w.x + (p.S - 1) * H, p.S * H * 4, H * 4, p.B, cudaMemcpyDeviceToDevice, s));
        xin = w.last_x;
        rows = p.B;
    }
    float *lg = tp ? w.logits_local + (size_t)ctx->tp_rank * rows * m->vocab_l : w.logits;
    if (rows <= vec_rows && rows * H * 4 <= 200 * 1024) {
        GemvArgs g;
        g.x = xin; g.w = m->lm_head; g.wdt = wdt; g.y = lg; g.M = (int)rows; g.K = H; g.N = m->vocab_l; g.ldy = m->vocab_l;
        g.norm_w = m->final_norm; g.norm_eps = eps;
        LUMEN_TRY(launch_gemv_nk(ctx, g, s));
    } else {
        LUMEN_TRY(launch_rmsnorm(ctx, xin, m->final_norm, eps, w.nx, rows, H, s));
        if (m->wsplit_valid && gemm_tc_usable(wdt, rows, H, m->vocab_l, m->lm_head)) {
            GemmFuse fl;
            use_weight_split(m, m->lm_head, fl);
            LUMEN_TRY(launch_gemm_tc(ctx, w.nx, m->lm_head, wdt, lg, rows, H, m->vocab_l, nullptr, s, nullptr, &fl));
        } else {
            LUMEN_TRY(launch_gemm_nk(ctx, w.nx, m->lm_head, wdt, lg, rows, H, m->vocab_l, nullptr, s));
        }
    }
    if (tp) {
        LUMEN_TRY(tp_allgather(ctx, lg, w.logits_local, rows * m->vocab_l, s));
        for (int r = 0; r < ctx->tp_size; ++r)
            LUMEN_CUDA(ctx, cudaMemcpy2DAsync(w.logits + (size_t)r * m->vocab_l, m->V * 4, w.logits_local + (size_t)r * rows * m->vocab_l,
                                              m->vocab_l * 4, m->vocab_l * 4, rows, cudaMemcpyDeviceToDevice, s));
    }
    return LUMEN_OK;
}

int pick_decode_splits(const lumen_llama *m, size_t B, size_t len) {
    // Power-of-two buckets so that a handful of graphs cover every context length.
    int want = attn_decode_pick_splits(B, m->hkv_l, len, m->ctx->num_sms);
    int n = 1;
    while (n < want && n < kMaxSplits) n <<= 1;
    return n;
}

int check_caches(lumen_llama *m, size_t b, size_t s, lumen_kv_cache **caches, size_t n_caches) {
    lumen_ctx *ctx = m->ctx;
    if (n_caches != m->L || !caches)
        return set_error(ctx, LUMEN_ERR_CACHE_COUNT, "KV cache count mismatch: got %zu, expected %zu", n_caches, m->L);
    for (size_t l = 0; l < m->L; ++l) {
        lumen_kv_cache *c = caches[l];
        if (!c) return set_error(ctx, LUMEN_ERR_INVALID, "null KV cache for layer %zu", l);
        LUMEN_TRY(kv_resync_len(c));
        if (c->b != b || c->h_kv != m->hkv_l || c->d != m->D)
            return set_error(ctx, LUMEN_ERR_SHAPE, "KV cache %zu geometry [%zu,%zu,%zu,%zu] does not match batch %zu / model", l, c->b, c->h_kv, c->max_seq, c->d, b);
        if (c->len != caches[0]->len) return set_error(ctx, LUMEN_ERR_INVALID, "KV caches have different lengths");
        if (s == 1) {  // decode asserts overflow before touching RoPE (self_attention.rs:144-149)
            if (c->len + 1 > c->max_seq) return set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "KV cache overflow: new_len=%zu > max_seq=%zu", c->len + 1, c->max_seq);
            if (c->len >= m->cfg.max_seq_len) return set_error(ctx, LUMEN_ERR_ROPE_RANGE, "RoPE index out of range: pos %zu >= max %zu", c->len, m->cfg.max_seq_len);
        } else {       // prefill rotates first (self_attention.rs:334-346)
            if (c->len + s > m->cfg.max_seq_len) return set_error(ctx, LUMEN_ERR_ROPE_RANGE, "RoPE index out of range: offset %zu + len %zu > max %zu", c->len, s, m->cfg.max_seq_len);
            if (c->len + s > c->max_seq) return set_error(ctx, LUMEN_ERR_KV_OVERFLOW, "KV cache overflow: new_len=%zu > max_seq=%zu", c->len + s, c->max_seq);
        }
    }
    return LUMEN_OK;
}

// Batch-1 decode through the persistent kernel: one launch per token.
int run_mega(lumen_llama *m, lumen_kv_cache **caches) {
    lumen_ctx *ctx = m->ctx;
    Workspace &w = m->ws;
    MegaParams p{};
    p.L = (int)m->L; p.H = (int)m->H; p.I = (int)m->inter_l; p.V = (int)m->vocab_l; p.vocab = (int)m->V;
    p.Hq = (int)m->hq_l; p.Hkv = (int)m->hkv_l; p.D = (int)m->D;
    p.qkv_rows = (int)m->qkv_rows; p.qd = (int)m->qd_l; p.kvd = (int)m->kvd_l; p.max_seq = (int)caches[0]->max_seq;
    p.wbf16 = m->cfg.weight_dtype == LUMEN_BF16;
    p.embed = m->embed; p.final_norm = m->final_norm; p.lm_head = m->lm_head;
    if (m->mega_key != (const void *)caches[0]->k || !m->d_mega_layers) {
        // (Re)build what depends on addresses: the layer table and the producer's copy schedule.
        std::vector<MegaLayer> host(m->L);
        for (size_t l = 0; l < m->L; ++l) {
            const LayerW &lw = m->layers[l];
            host[l] = MegaLayer{lw.wqkv, lw.wo, lw.wgate, lw.wup, lw.wdown, lw.norm1, lw.norm2, lw.qn, lw.kn,
                                caches[l]->k, caches[l]->v, caches[l]->d_len};
        }
        std::vector<uint4> entries;
        std::vector<int> counts;
        int stride = 0;
        std::vector<CUtensorMap> tmaps;
        decode_mega_build_schedule(p, host.data(), ctx->num_sms, entries, counts, stride, tmaps);
        LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // earlier launches may still read the tables
        if (!m->d_mega_layers) LUMEN_CUDA(ctx, cudaMalloc(&m->d_mega_layers, std::max<size_t>(m->L, 1) * sizeof(MegaLayer)));
        if (m->d_sched && m->sched_capacity < entries.size()) {
            cudaFree(m->d_sched);
            m->d_sched = nullptr;
        }
        if (!m->d_sched) {
            LUMEN_CUDA(ctx, cudaMalloc(&m->d_sched, entries.size() * sizeof(uint4)));
            m->sched_capacity = entries.size();
        }
        if (!m->d_sched_count) LUMEN_CUDA(ctx, cudaMalloc(&m->d_sched_count, counts.size() * sizeof(int)));
        if (m->d_tmaps && m->tmaps_capacity < tmaps.size()) {
            cudaFree(m->d_tmaps);
            m->d_tmaps = nullptr;
        }
        if (!tmaps.empty()) {
            if (!m->d_tmaps) {
                LUMEN_CUDA(ctx, cudaMalloc(&m->d_tmaps, tmaps.size() * sizeof(CUtensorMap)));
                m->tmaps_capacity = tmaps.size();
            }
            LUMEN_CUDA(ctx, cudaMemcpy(m->d_tmaps, tmaps.data(), tmaps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice));
        } else if (m->d_tmaps) {
            cudaFree(m->d_tmaps);
            m->d_tmaps = nullptr;
            m->tmaps_capacity = 0;
        }
        LUMEN_CUDA(ctx, cudaMemcpy(m->d_mega_layers, host.data(), m->L * sizeof(MegaLayer), cudaMemcpyHostToDevice));
        LUMEN_CUDA(ctx, cudaMemcpy(m->d_sched, entries.data(), entries.size() * sizeof(uint4), cudaMemcpyHostToDevice));
        LUMEN_CUDA(ctx, cudaMemcpy(m->d_sched_count, counts.data(), counts.size() * sizeof(int), cudaMemcpyHostToDevice));
        m->sched_stride = stride;
        m->mega_key = caches[0]->k;
    }
    p.layers = m->d_mega_layers;
    p.sched = m->d_sched; p.sched_count = m->d_sched_count; p.sched_stride = m->sched_stride;
    p.tmaps = m->d_tmaps;
    p.cos_t = m->cos_t; p.sin_t = m->sin_t;
    p.eps = m->cfg.rms_norm_eps;
    p.scale = 1.0f / sqrtf((float)m->D);
    const bool tp = ctx->tp_size > 1;
    p.tp_rank = ctx->tp_rank; p.tp_size = ctx->tp_size;
    p.x_slot_words = (p.H + 1) & ~1;
    // A rank computes its slice of the vocabulary; the slices are gathered after the kernel.
    p.ids = w.ids;
    p.logits = w.logits;  // (tensor parallel: set below, once the exchange buffer exists)
    // Exchange buffers of tagged words (zeroed once; tag 0 is never used).  With tensor parallelism the x
    // buffers at their start are written by every rank: the ranks map each other's buffer once.
    const size_t words = decode_mega_exchange_words(p);
    LUMEN_TRY(ensure_exchange(ctx, words * sizeof(uint2)));
    const unsigned int per_launch = decode_mega_epochs_per_launch(p.L);
    if (ctx->mega_epoch > 0xf0000000u - per_launch) {  // tags are about to wrap: start over from clean buffers
        LUMEN_CUDA(ctx, cudaMemsetAsync(ctx->d_exchange, 0, ctx->exchange_bytes, ctx->stream));
        // no rank may write into a peer's buffer before that peer has cleared it
        if (tp) LUMEN_TRY(tp_allreduce_sum(ctx, w.logits_local, 1, ctx->stream));
        ctx->mega_epoch = 1;
    }
    p.xT = static_cast<uint2 *>(ctx->d_exchange);
    for (int r = 0; r < ctx->tp_size; ++r) p.x_peer[r] = static_cast<uint2 *>(ctx->x_peers[r]);
    p.xrT = nullptr;
    if (tp) {
        // Two forms of the exchange.  One hop: every CTA sums the ranks' slots while it stages x (tp_size times the loads
        // of a plain staging pass, in several passes of what fits the registers).  Two hops: the row owners sum the
        // ranks' partial values and publish the sums, then everybody stages them in one pass.  Measured on TinyLlama f32
        // the single hop wins at 2 ranks (1353 against 1272 tok/s) and at 4 (1604 against 1405); at 8 ranks the single hop
        // needs 5 passes (10 at hidden size 4096), so the two hops are the default there.  LUMEN_MEGA_TP_REDUCE=0/1 forces one.
        static const int reduce_env = [] { const char *e = getenv("LUMEN_MEGA_TP_REDUCE"); return e ? atoi(e) : -1; }();
        const size_t lo = decode_mega_logits_offset_words(p);
        if (reduce_env == 1 || (reduce_env < 0 && ctx->tp_size >= 8)) p.xrT = p.xT + lo - 2 * (size_t)p.x_slot_words;
        for (int r = 0; r < ctx->tp_size; ++r) {
            p.logits_peer[r] = reinterpret_cast<float *>(static_cast<uint2 *>(ctx->x_peers[r]) + lo);
            p.flag_peer[r] = reinterpret_cast<unsigned int *>(p.logits_peer[r] + ((p.vocab + 1) & ~1));
        }
        p.logits = p.logits_peer[ctx->tp_rank];
        p.done_count = reinterpret_cast<unsigned int *>(ctx->d_mega_sync);
    }
    p.qkvT = p.xT + decode_mega_x_words(p);
    p.actT = p.qkvT + ((p.qkv_rows + 1) & ~1);
    p.partT = p.actT + ((p.I + 1) & ~1);
    p.epoch_base = ctx->mega_epoch;
    // Attention work items = heads x splits, at most one per SM, with at least 128 rows per split.
    const size_t len = caches[0]->len + 1;
    int nsplit = std::max(1, std::min(decode_mega_max_splits(), ctx->num_sms / std::max(1, p.Hq)));
    nsplit = (int)std::max<size_t>(1, std::min<size_t>(nsplit, len / 128));
    p.nsplit = nsplit;
    p.abort_flag = reinterpret_cast<int *>(ctx->d_mega_sync + 1);
    p.status = ctx->d_status;
    p.trace = m->d_trace;
    LUMEN_TRY(launch_decode_mega(ctx, p, ctx->stream));
    ctx->mega_epoch += per_launch;
    if (tp)  // the kernel gathered the vocabulary slices of all ranks into this rank's exchange buffer
        LUMEN_CUDA(ctx, cudaMemcpyAsync(w.logits, p.logits, m->V * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return LUMEN_OK;
}

bool mega_usable(lumen_llama *m, size_t b, size_t s) {
    if (!m->use_mega || b != 1 || s != 1 || m->L == 0) return false;
    // the kernel's fused all-reduce has forms for 2, 4 and 8 ranks; other rank counts take the per-operator path + NCCL
    const int T = m->ctx->tp_size;
    if (T != 1 && T != 2 && T != 4 && T != 8) return false;
    MegaParams p{};
    p.H = (int)m->H; p.I = (int)m->inter_l; p.qd = (int)m->qd_l; p.D = (int)m->D;
    p.qkv_rows = (int)m->qkv_rows; p.kvd = (int)m->kvd_l;
    p.wbf16 = m->cfg.weight_dtype == LUMEN_BF16;
    char why[128];
    return decode_mega_supported(p, why, sizeof(why)) != 0;
}

// Runs one forward over ws.ids; batch-1 decode steps take the persistent kernel, other decode steps go
// through a captured graph after the first call.
int run_forward(lumen_llama *m, size_t b, size_t s, lumen_kv_cache **caches, bool last_only) {
    lumen_ctx *ctx = m->ctx;
    if (mega_usable(m, b, s)) {
        LUMEN_TRY(run_mega(m, caches));
        for (size_t l = 0; l < m->L; ++l) caches[l]->len += 1;
        return LUMEN_OK;
    }
    StepPlan p{b, s, b * s, s == 1, 1};
    if (p.M > 8) LUMEN_TRY(ensure_weight_split(m));  // (outside any stream capture; the streaming kernels of <= 8 rows read f32)
    if (p.decode) p.nsplit = pick_decode_splits(m, b, caches[0]->len + 1);
    int rc = LUMEN_OK;
    if (p.decode && m->use_graph) {
        auto key = std::make_tuple(b, p.nsplit, (const void *)caches[0]->k);
        auto it = m->graphs.find(key);
        if (it == m->graphs.end() && m->eager_runs[key]++ >= 1) {
            cudaGraph_t graph = nullptr;
            const unsigned long long before = ctx->launches;
            LUMEN_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
            rc = enqueue_forward(m, p, caches, last_only);
            cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
            m->graph_nodes[key] = ctx->launches - before;  // captured, not run
            ctx->launches = before;
            if (rc != LUMEN_OK) {
                if (graph) cudaGraphDestroy(graph);
                return rc;
            }
            if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaStreamEndCapture");
            cudaGraphExec_t exec = nullptr;
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaGraphInstantiate");
            it = m->graphs.emplace(key, exec).first;
        }
        if (it != m->graphs.end()) {
            LUMEN_CUDA(ctx, cudaGraphLaunch(it->second, ctx->stream));
            ctx->launches += m->graph_nodes[key];
        } else {
            rc = enqueue_forward(m, p, caches, last_only);
        }
    } else {
        rc = enqueue_forward(m, p, caches, last_only);
    }
    if (rc == LUMEN_OK)
        for (size_t l = 0; l < m->L; ++l) caches[l]->len += s;
    return rc;
}

int forward_host(lumen_llama *m, const float *ids_host, size_t b, size_t s, lumen_kv_cache **caches, size_t n_caches,
                 float *logits_host, bool last_only) {
    if (!m || !ids_host || !logits_host) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = m->ctx;
    if (m->is_set.size() < m->n_expected) return set_error(ctx, LUMEN_ERR_MISSING_PARAM, "%zu of %zu parameters set", m->is_set.size(), m->n_expected);
    const size_t M = b * s;
    if (M == 0) return LUMEN_OK;
    LUMEN_TRY(check_caches(m, b, s, caches, n_caches));
    // Embedding range check on the host (src/layers/basic/embedding.rs:50-56) before anything is launched.
    for (size_t i = 0; i < M; ++i) {
        const float f = ids_host[i];
        if (f >= (float)m->V && f == f) return set_error(ctx, LUMEN_ERR_EMBED_RANGE, "Embedding index out of bounds: %.0f >= %zu", (double)f, m->V);
    }
    LUMEN_TRY(ensure_workspace(m, M));
    Workspace &w = m->ws;
    // The pinned staging buffers are reused every step: wait for the previous step's copies first.
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    memcpy(w.h_ids, ids_host, M * sizeof(float));
    LUMEN_CUDA(ctx, cudaMemcpyAsync(w.ids, w.h_ids, M * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    LUMEN_TRY(run_forward(m, b, s, caches, last_only));
    const size_t rows = (last_only && s > 1) ? b : M;
    const size_t n = rows * m->V;
    if (n <= w.h_logits_elems) {
        LUMEN_CUDA(ctx, cudaMemcpyAsync(w.h_logits, w.logits, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        LUMEN_TRY(check_device_status(ctx));
        memcpy(logits_host, w.h_logits, n * 4);
    } else {
        LUMEN_CUDA(ctx, cudaMemcpyAsync(logits_host, w.logits, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        LUMEN_TRY(check_device_status(ctx));
    }
    return LUMEN_OK;
}

}  // namespace

extern "C" {

int lumen_llama_new(lumen_ctx *ctx, const lumen_llama_config *cfg, lumen_llama **out) {
    if (!ctx || !cfg || !out) return set_error(ctx, LUMEN_ERR_INVALID, "llama_new: null argument");
    if (cfg->weight_dtype != LUMEN_F32 && cfg->weight_dtype != LUMEN_BF16) return set_error(ctx, LUMEN_ERR_DTYPE, "weight_dtype %d", (int)cfg->weight_dtype);
    if (!cfg->num_attention_heads || !cfg->num_key_value_heads || cfg->num_attention_heads % cfg->num_key_value_heads)
        return set_error(ctx, LUMEN_ERR_SHAPE, "num_attention_heads must be a positive multiple of num_key_value_heads");
    if (!cfg->head_dim && cfg->hidden_size % cfg->num_attention_heads) return set_error(ctx, LUMEN_ERR_SHAPE, "Embed dim must be divisible by n_head");
    auto *m = new lumen_llama();
    m->ctx = ctx;
    m->cfg = *cfg;
    m->H = cfg->hidden_size; m->V = cfg->vocab_size; m->I = cfg->intermediate_size; m->L = cfg->num_hidden_layers;
    m->D = cfg->head_dim ? cfg->head_dim : cfg->hidden_size / cfg->num_attention_heads;
    m->esz = cfg->weight_dtype == LUMEN_F32 ? 4 : 2;
    const size_t T = ctx->tp_size, r = ctx->tp_rank, Hq = cfg->num_attention_heads, Hkv = cfg->num_key_value_heads;
    if (m->D == 0 || (m->D & 1) || m->D > 256) { delete m; return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "head_dim %zu (need even, <= 256)", m->D); }
    TpHeads th;
    if (tp_head_plan(*cfg, T, r, th) != LUMEN_OK) {
        delete m;
        return set_error(ctx, LUMEN_ERR_UNSUPPORTED,
                         "tp_size %zu does not divide heads %zu / kv heads %zu / intermediate %zu / vocab %zu", T, Hq, Hkv,
                         cfg->intermediate_size, cfg->vocab_size);
    }
    m->hq_l = th.hq_l; m->q_head0 = th.q_head0; m->hkv_l = th.hkv_l; m->kv_head0 = th.kv_head0;
    m->qd_l = m->hq_l * m->D; m->kvd_l = m->hkv_l * m->D; m->inter_l = m->I / T; m->vocab_l = m->V / T;
    m->qkv_rows = m->qd_l + 2 * m->kvd_l;

    // Slab layout.
    const size_t e = m->esz, H = m->H;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align_up(bytes, 256); return o; };
    struct Off { size_t qkv, o, g, u, d, n1, n2, qn, kn; };
    std::vector<Off> lo(m->L);
    size_t o_embed = take(m->V * H * e);
    for (size_t l = 0; l < m->L; ++l) {
        lo[l].n1 = take(H * 4);
        lo[l].qkv = take(m->qkv_rows * H * e);
        lo[l].qn = take(cfg->qk_norm ? m->D * 4 : 0);
        lo[l].kn = take(cfg->qk_norm ? m->D * 4 : 0);
        lo[l].o = take(H * m->qd_l * e);
        lo[l].n2 = take(H * 4);
        lo[l].g = take(m->inter_l * H * e);
        lo[l].u = take(m->inter_l * H * e);
        lo[l].d = take(H * m->inter_l * e);
    }
    size_t o_fn = take(H * 4), o_lm = take(m->vocab_l * H * e);
    const size_t half = m->D / 2;
    size_t o_cos = take(cfg->max_seq_len * half * 4), o_sin = take(cfg->max_seq_len * half * 4);
    m->wbytes = off;
    cudaError_t ce = cudaMalloc(&m->wslab, std::max<size_t>(off, 256));
    if (ce != cudaSuccess) { delete m; return cuda_fail(ctx, ce, "cudaMalloc(weight slab)"); }
    m->embed = m->wslab + o_embed;
    m->layers.resize(m->L);
    for (size_t l = 0; l < m->L; ++l) {
        LayerW &w = m->layers[l];
        w.wqkv = m->wslab + lo[l].qkv; w.wo = m->wslab + lo[l].o; w.wgate = m->wslab + lo[l].g;
        w.wup = m->wslab + lo[l].u; w.wdown = m->wslab + lo[l].d;
        w.norm1 = (float *)(m->wslab + lo[l].n1); w.norm2 = (float *)(m->wslab + lo[l].n2);
        if (cfg->qk_norm) { w.qn = (float *)(m->wslab + lo[l].qn); w.kn = (float *)(m->wslab + lo[l].kn); }
    }
    m->final_norm = (float *)(m->wslab + o_fn);
    m->lm_head = m->wslab + o_lm;
    m->cos_t = (float *)(m->wslab + o_cos);
    m->sin_t = (float *)(m->wslab + o_sin);
    std::vector<float> ch, sh;
    rope_tables_host(m->D, cfg->max_seq_len, cfg->rope_theta, ch, sh);
    if (!ch.empty()) {
        cudaMemcpy(m->cos_t, ch.data(), ch.size() * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(m->sin_t, sh.data(), sh.size() * 4, cudaMemcpyHostToDevice);
    }
    m->n_expected = 3 + m->L * (cfg->qk_norm ? 11 : 9);
    // Weights one decode step reads on this rank (the embedding contributes one row per token).
    m->stream_bytes = m->L * ((m->qkv_rows * H + H * m->qd_l + 3 * m->inter_l * H) * e + 2 * H * 4 + (cfg->qk_norm ? 2 * m->D * 4 : 0)) +
                      H * 4 + m->vocab_l * H * e;
    const char *ng = getenv("LUMEN_NO_GRAPH");
    m->use_graph = !(ng && ng[0] == '1');
    const char *nm = getenv("LUMEN_NO_MEGA");
    m->use_mega = !(nm && nm[0] == '1');
    const char *tr = getenv("LUMEN_DECODE_TRACE");
    if (tr && tr[0] == '1') {
        const size_t n = decode_mega_trace_words(m->L);
        if (cudaMalloc(&m->d_trace, n * sizeof(unsigned long long)) == cudaSuccess) cudaMemset(m->d_trace, 0, n * sizeof(unsigned long long));
        else m->d_trace = nullptr;
    }
    *out = m;
    return LUMEN_OK;
}

int lumen_llama_set_param(lumen_llama *m, const char *name, const void *host_data, const size_t *shape, int ndim, lumen_dtype dtype) {
    if (!m || !name || !host_data || !shape) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = m->ctx;
    if (dtype != LUMEN_F32 && dtype != LUMEN_BF16) return set_error(ctx, LUMEN_ERR_DTYPE, "set_param: dtype %d", (int)dtype);
    const lumen_dtype wdt = m->cfg.weight_dtype;
    const size_t se = dtype == LUMEN_F32 ? 4 : 2, e = m->esz, H = m->H;
    m->wsplit_valid = false;  // (the kept bf16 split of the f32 weights is rebuilt before its next use)
    // Which part of the tensor this rank keeps comes from the shard plan; what is left here is where it goes.
    TpSlice sl;
    long li = -1;
    const char *leaf = name;
    int rc = tp_param_slice(m->cfg, ctx->tp_size, ctx->tp_rank, name, sl, &li, &leaf);
    if (rc != LUMEN_OK) return set_error(ctx, rc, "unknown parameter '%s'", name);
    if (sl.cols == 0) {
        if (ndim != 1 || shape[0] != sl.rows) return set_error(ctx, LUMEN_ERR_SHAPE, "%s: expected [%zu]", name, sl.rows);
    } else if (ndim != 2 || shape[0] != sl.rows || shape[1] != sl.cols) {
        return set_error(ctx, LUMEN_ERR_SHAPE, "%s: expected [%zu,%zu]", name, sl.rows, sl.cols);
    }
    char *dst = nullptr;
    lumen_dtype ddt = wdt;
    if (li < 0) {
        if (!strcmp(leaf, "model.embed_tokens.weight")) dst = m->embed;
        else if (!strcmp(leaf, "lm_head.weight")) dst = m->lm_head;
        else { dst = reinterpret_cast<char *>(m->final_norm); ddt = LUMEN_F32; }
    } else {
        LayerW &w = m->layers[li];
        if (!strcmp(leaf, "self_attn.q_proj.weight")) dst = w.wqkv;
        else if (!strcmp(leaf, "self_attn.k_proj.weight")) dst = w.wqkv + m->qd_l * H * e;
        else if (!strcmp(leaf, "self_attn.v_proj.weight")) dst = w.wqkv + (m->qd_l + m->kvd_l) * H * e;
        else if (!strcmp(leaf, "self_attn.o_proj.weight")) dst = w.wo;
        else if (!strcmp(leaf, "mlp.gate_proj.weight")) dst = w.wgate;
        else if (!strcmp(leaf, "mlp.up_proj.weight")) dst = w.wup;
        else if (!strcmp(leaf, "mlp.down_proj.weight")) dst = w.wdown;
        else {
            ddt = LUMEN_F32;
            if (!strcmp(leaf, "input_layernorm.weight")) dst = reinterpret_cast<char *>(w.norm1);
            else if (!strcmp(leaf, "post_attention_layernorm.weight")) dst = reinterpret_cast<char *>(w.norm2);
            else if (!strcmp(leaf, "self_attn.q_norm.weight")) dst = reinterpret_cast<char *>(w.qn);
            else dst = reinterpret_cast<char *>(w.kn);
        }
    }
    if (sl.cols == 0) {
        rc = upload_block(ctx, dst, ddt, host_data, dtype, 1, sl.rows, 0, sl.rows);
    } else {
        const char *src = static_cast<const char *>(host_data) + sl.row0 * sl.cols * se;
        rc = upload_block(ctx, dst, ddt, src, dtype, sl.nrows, sl.cols, sl.col0, sl.ncols);
    }
    if (rc == LUMEN_ERR_PARAM_NAME) return set_error(ctx, rc, "unknown parameter '%s'", name);
    if (rc == LUMEN_OK) m->is_set[name] = true;
    return rc;
}

int lumen_llama_init_kv_caches(lumen_llama *m, size_t batch, lumen_kv_cache **caches_out) {
    if (!m || !caches_out) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = m->ctx;
    const size_t per = batch * m->hkv_l * m->cfg.max_seq_len * m->D;  // floats per k (or v) slab of a layer
    const size_t bytes = m->L * 2 * per * sizeof(float) + align_up(m->L * sizeof(int), 256);
    auto *slab = new lumen_storage();
    slab->ctx = ctx;
    slab->bytes = bytes;
    slab->refs = 0;
    cudaError_t e = cudaMalloc(&slab->ptr, std::max<size_t>(bytes, 256));
    if (e != cudaSuccess) { delete slab; return cuda_fail(ctx, e, "cudaMalloc(kv slab)"); }
    LUMEN_CUDA(ctx, cudaMemsetAsync(slab->ptr, 0, bytes, ctx->stream));  // Array4::zeros, self_attention.rs:35-36
    float *base = static_cast<float *>(slab->ptr);
    int *lens = reinterpret_cast<int *>(base + m->L * 2 * per);
    for (size_t l = 0; l < m->L; ++l) {
        auto *c = new lumen_kv_cache();
        c->ctx = ctx; c->b = batch; c->h_kv = m->hkv_l; c->max_seq = m->cfg.max_seq_len; c->d = m->D;
        c->k = base + (2 * l) * per;
        c->v = base + (2 * l + 1) * per;
        c->d_len = lens + l;
        c->seen_abort = ctx->abort_gen;
        c->owns_slab = false;
        c->slab = slab;
        slab->refs += 1;
        caches_out[l] = c;
    }
    if (m->L == 0) { cudaFree(slab->ptr); delete slab; }
    return LUMEN_OK;
}

int lumen_llama_reset_kv_caches(lumen_llama *m, lumen_kv_cache **caches, size_t n_caches) {
    if (!m || (!caches && n_caches)) return LUMEN_ERR_INVALID;
    for (size_t i = 0; i < n_caches; ++i) LUMEN_TRY(lumen_kv_reset(caches[i]));
    return LUMEN_OK;
}

int lumen_llama_forward(lumen_llama *m, const float *ids_host, size_t b, size_t s, lumen_kv_cache **caches, size_t n_caches,
                        size_t pos, float *logits_host) {
    (void)pos;  // `_pos` is ignored by the reference too (llama.rs:180-181)
    return forward_host(m, ids_host, b, s, caches, n_caches, logits_host, false);
}

int lumen_llama_forward_last(lumen_llama *m, const float *ids_host, size_t b, size_t s, lumen_kv_cache **caches, size_t n_caches,
                             size_t pos, float *logits_host) {
    (void)pos;
    return forward_host(m, ids_host, b, s, caches, n_caches, logits_host, true);
}

int lumen_llama_forward_sample(lumen_llama *m, const float *ids_host, size_t s, lumen_kv_cache **caches, size_t n_caches,
                               const lumen_sample_params *sp, int32_t *token_out) {
    if (!m || !ids_host || !sp || !token_out || (sp->n_recent && !sp->recent_tokens)) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = m->ctx;
    if (m->is_set.size() < m->n_expected) return set_error(ctx, LUMEN_ERR_MISSING_PARAM, "%zu of %zu parameters set", m->is_set.size(), m->n_expected);
    if (s == 0) return set_error(ctx, LUMEN_ERR_SHAPE, "forward_sample: empty input");
    LUMEN_TRY(check_caches(m, 1, s, caches, n_caches));
    for (size_t i = 0; i < s; ++i) {
        const float f = ids_host[i];
        if (f >= (float)m->V && f == f) return set_error(ctx, LUMEN_ERR_EMBED_RANGE, "Embedding index out of bounds: %.0f >= %zu", (double)f, m->V);
    }
    LUMEN_TRY(ensure_workspace(m, s));
    Workspace &w = m->ws;
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the pinned staging buffer is reused every step
    memcpy(w.h_ids, ids_host, s * sizeof(float));
    LUMEN_CUDA(ctx, cudaMemcpyAsync(w.ids, w.h_ids, s * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    LUMEN_TRY(run_forward(m, 1, s, caches, true));  // last position's logits in w.logits[V]
    int *token_dev = reinterpret_cast<int *>(w.ids);  // the id buffer is free again once the forward is enqueued behind it
    LUMEN_TRY(launch_sample_top_p(ctx, w.logits, m->V, sp->temperature, sp->top_p, sp->repetition_penalty, sp->recent_tokens,
                                  sp->n_recent, sp->uniform, token_dev, ctx->stream));
    LUMEN_CUDA(ctx, cudaMemcpyAsync(w.h_ids, token_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    LUMEN_TRY(check_device_status(ctx));
    memcpy(token_out, w.h_ids, sizeof(int));
    return LUMEN_OK;
}

int lumen_llama_forward_device(lumen_llama *m, const float *ids_dev, size_t b, size_t s, lumen_kv_cache **caches, size_t n_caches,
                               float *logits_dev) {
    if (!m || !ids_dev || !logits_dev) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = m->ctx;
    if (m->is_set.size() < m->n_expected) return set_error(ctx, LUMEN_ERR_MISSING_PARAM, "%zu of %zu parameters set", m->is_set.size(), m->n_expected);
    const size_t M = b * s;
    if (M == 0) return LUMEN_OK;
    LUMEN_TRY(check_caches(m, b, s, caches, n_caches));
    LUMEN_TRY(ensure_workspace(m, M));
    LUMEN_CUDA(ctx, cudaMemcpyAsync(m->ws.ids, ids_dev, M * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    LUMEN_TRY(run_forward(m, b, s, caches, false));
    LUMEN_CUDA(ctx, cudaMemcpyAsync(logits_dev, m->ws.logits, M * m->V * sizeof(float), cudaMemcpyDeviceToDevice, ctx->stream));
    return LUMEN_OK;
}

size_t lumen_llama_weight_bytes(const lumen_llama *m) { return m ? m->stream_bytes : 0; }

int lumen_llama_decode_trace(lumen_llama *m, uint64_t *out, size_t capacity, size_t *n_out) {
    if (!m || !out || !n_out) return LUMEN_ERR_INVALID;
    lumen_ctx *ctx = m->ctx;
    if (!m->d_trace) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "decode trace is off (set LUMEN_DECODE_TRACE=1 before creating the model)");
    const size_t n = std::min<size_t>(capacity, decode_mega_trace_words(m->L));
    LUMEN_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    LUMEN_CUDA(ctx, cudaMemcpy(out, m->d_trace, n * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    *n_out = n;
    return LUMEN_OK;
}

int lumen_llama_free(lumen_llama *m) {
    if (!m) return LUMEN_ERR_INVALID;
    cudaStreamSynchronize(m->ctx->stream);
    drop_graphs(m);
    if (m->d_mega_layers) cudaFree(m->d_mega_layers);
    if (m->d_sched) cudaFree(m->d_sched);
    if (m->d_sched_count) cudaFree(m->d_sched_count);
    if (m->d_tmaps) cudaFree(m->d_tmaps);
    if (m->d_trace) cudaFree(m->d_trace);
    if (m->ws.base) cudaFree(m->ws.base);
    if (m->ws.h_ids) cudaFreeHost(m->ws.h_ids);
    if (m->ws.h_logits) cudaFreeHost(m->ws.h_logits);
    if (m->wslab) cudaFree(m->wslab);
    if (m->wsplit) cudaFree(m->wsplit);
    delete m;
    return LUMEN_OK;
}

}  // extern "C"
