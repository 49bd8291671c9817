// GQA attention over the static KV cache: stand-alone decode kernels (split over the context, then a
// merge) and the prefill path.
//
// Decode (S == 1): see attn_decode.cuh.  One CTA serves all query heads of its KV head (up to 8), so
// K/V rows are read once per KV head instead of once per query head.
//
// Prefill (S > 1) restates src/layers/attention/self_attention.rs:308-426, :519-535, :621-678 of the
// reference: rotate q/k at positions past..past+S, slab write, causal mask j > past+i, softmax with
// `1/(sum + 1e-9)`, P.V, output in [B,S,H,D] order.
#include "attn_decode.cuh"

namespace lumen {
namespace {

constexpr int kThreads = kAttnThreads;
constexpr int kWarps = kAttnWarps;

struct SyncThreads {
    __device__ __forceinline__ void operator()() const { __syncthreads(); }
};

// grid (nsplit, Hkv * (G/GT), B)
template <int GT, int NI>
__global__ void __launch_bounds__(kThreads) attn_decode_kernel(DecodeParams p) {
    extern __shared__ __align__(16) float smem[];
    attn_decode_item<GT, NI, false, kWarps>(p, smem, blockIdx.z, blockIdx.y, blockIdx.x, threadIdx.x, *p.d_len, SyncThreads(),
                                    PartOut{&p}, NoStage());
}

// Merge the splits; grid (B*Hq).  Thread 0 of block 0 advances the cache length afterwards
// (c.len = new_len, self_attention.rs:179).
__global__ void attn_decode_combine_kernel(const float *part_m, const float *part_l, const float *part_ctx,
                                           float *__restrict__ out, int D, int nsplit, int *d_len_bump) {
    const size_t row = blockIdx.x;
    for (int e = threadIdx.x; e < D; e += blockDim.x)
        out[row * D + e] = attn_combine_elem(part_m, part_l, part_ctx, row, e, D, nsplit);
    if (d_len_bump && blockIdx.x == 0 && threadIdx.x == 0) *d_len_bump += 1;
}

// ---- prefill ------------------------------------------------------------------------------------
struct PrefillParams {
    const float *q, *k, *v;
    size_t q_stride, kv_stride;
    float *k_cache, *v_cache;
    int past, S, Hq, Hkv, D, max_seq;
    const float *cos_t, *sin_t, *q_norm, *k_norm;
    float norm_eps, scale;
    int causal;
    float *q_rot;  // [B,S,Hq,D]
    float *out;    // [B,S,Hq,D]
};

// One warp per head vector of (b, s): heads 0..Hq-1 are q (rotated into q_rot), Hq..Hq+Hkv-1 are k
// (rotated into the cache) with v copied beside it.  grid (S, B), dynamic smem kWarps*D floats.
__global__ void __launch_bounds__(kThreads) attn_prefill_prep_kernel(PrefillParams p) {
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = blockIdx.x, b = blockIdx.y, D = p.D, half = D / 2;
    float *buf = smem + warp * D;
    const int pos = p.past + s;
    const float *cos_row = p.cos_t ? p.cos_t + (size_t)pos * half : nullptr;
    const float *sin_row = p.sin_t ? p.sin_t + (size_t)pos * half : nullptr;
    const size_t row = (size_t)b * p.S + s;
    for (int h = warp; h < p.Hq + p.Hkv; h += kWarps) {
        const bool is_q = h < p.Hq;
        const float *src = is_q ? p.q + row * p.q_stride + (size_t)h * D
                                : p.k + row * p.kv_stride + (size_t)(h - p.Hq) * D;
        for (int i = lane; i < D; i += 32) buf[i] = src[i];
        __syncwarp();
        head_norm_rope(buf, D, is_q ? p.q_norm : p.k_norm, p.norm_eps, cos_row, sin_row, lane);
        if (is_q) {
            float *dst = p.q_rot + (row * p.Hq + h) * D;
            for (int i = lane; i < D; i += 32) dst[i] = buf[i];
        } else {
            const int hk = h - p.Hq;
            const size_t crow = (((size_t)b * p.Hkv + hk) * p.max_seq + pos) * D;
            const float *vsrc = p.v + row * p.kv_stride + (size_t)hk * D;
            for (int i = lane; i < D; i += 32) {
                p.k_cache[crow + i] = buf[i];
                p.v_cache[crow + i] = vsrc[i];
            }
        }
        __syncwarp();
    }
}

// One warp per query row; grid (ceil(S/kWarps), Hq, B).
template <int NI>
__global__ void __launch_bounds__(kThreads) attn_prefill_kernel(PrefillParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i_q = blockIdx.x * kWarps + warp;
    if (i_q >= p.S) return;
    const int h = blockIdx.y, b = blockIdx.z, D = p.D;
    const int hk = h / (p.Hq / p.Hkv);
    const int total = p.past + p.S;
    const int last = p.causal ? min(total - 1, p.past + i_q) : total - 1;  // mask j > past + i
    const float *qr = p.q_rot + (((size_t)b * p.S + i_q) * p.Hq + h) * D;
    const float *kbase = p.k_cache + ((size_t)b * p.Hkv + hk) * p.max_seq * D;
    const float *vbase = p.v_cache + ((size_t)b * p.Hkv + hk) * p.max_seq * D;
    float q[NI], ctx[NI];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        int e = lane + 32 * i;
        q[i] = (e < D) ? qr[e] : 0.f;
        ctx[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    constexpr int UN = 4;
    for (int jb = 0; jb <= last; jb += UN) {
        float kr[UN][NI], vr[UN][NI];
#pragma unroll
        for (int u = 0; u < UN; ++u)
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int e = lane + 32 * i, j = jb + u;
                const bool ok = (j <= last) && (e < D);
                kr[u][i] = ok ? kbase[(size_t)j * D + e] : 0.f;
                vr[u][i] = ok ? vbase[(size_t)j * D + e] : 0.f;
            }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            if (jb + u > last) break;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < NI; ++i) dot = fmaf(q[i], kr[u][i], dot);
            dot = attn_warp_sum(dot);
            const float sc = __fmul_rn(dot, p.scale);
            const float mn = fmaxf(m, sc);
            const float r = expf(m - mn);
            const float w = expf(sc - mn);
            l = fmaf(l, r, w);
#pragma unroll
            for (int i = 0; i < NI; ++i) ctx[i] = fmaf(w, vr[u][i], ctx[i] * r);
            m = mn;
        }
    }
    const float inv = __fdiv_rn(1.0f, __fadd_rn(l, 1e-9f));
    float *o = p.out + (((size_t)b * p.S + i_q) * p.Hq + h) * D;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        int e = lane + 32 * i;
        if (e < D) o[e] = __fmul_rn(ctx[i], inv);
    }
}

int pick_gt(int G) { return (G % 8 == 0) ? 8 : (G % 4 == 0) ? 4 : (G % 2 == 0) ? 2 : 1; }
int pick_ni(size_t D) { return D <= 32 ? 1 : D <= 64 ? 2 : D <= 128 ? 4 : 8; }

template <int GT>
int launch_decode_gt(lumen_ctx *ctx, const DecodeParams &p, int ni, dim3 grid, size_t smem, cudaStream_t s) {
#define LD(NI_)                                                                                                       \
    do {                                                                                                              \
        auto kern = attn_decode_kernel<GT, NI_>;                                                                      \
        if (smem > 48 * 1024)                                                                                         \
            LUMEN_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));      \
        kern<<<grid, kThreads, smem, s>>>(p);                                                                         \
    } while (0)
    switch (ni) {
        case 1: LD(1); break;
        case 2: LD(2); break;
        case 4: LD(4); break;
        default: LD(8); break;
    }
#undef LD
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace

size_t attn_decode_scratch_bytes(size_t B, size_t Hq, size_t D, int max_splits) {
    return B * Hq * (size_t)max_splits * (D + 2) * sizeof(float);
}

int attn_decode_pick_splits(size_t B, size_t Hkv, size_t len, int num_sms) {
    // The grid is (B * Hkv) x splits CTAs and an SM holds about one of them (the 8-head kernel uses the
    // whole register file), so the step takes waves x rows-per-split: pick the split count that minimises
    // that product (plus a fixed cost per wave for staging q and merging), with at least 64 rows per split.
    const size_t base = std::max<size_t>(1, B * Hkv);
    const size_t max_ns = std::max<size_t>(1, std::min<size_t>(64, (len + 63) / 64));
    size_t best = 1, best_cost = ~(size_t)0;
    for (size_t ns = 1; ns <= max_ns; ++ns) {
        const size_t waves = (base * ns + (size_t)num_sms - 1) / (size_t)num_sms;
        const size_t rows = (len + ns - 1) / ns;
        const size_t cost = waves * (rows + 48);
        if (cost < best_cost) {
            best_cost = cost;
            best = ns;
        }
    }
    return (int)best;
}

int launch_attn_decode(lumen_ctx *ctx, const AttnDecodeArgs &a, cudaStream_t s) {
    if (a.D == 0 || a.D > 256 || (a.D & 1)) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "attention: head_dim %zu", a.D);
    if (a.Hkv == 0 || a.Hq % a.Hkv) return set_error(ctx, LUMEN_ERR_SHAPE, "attention: Hq %zu not a multiple of Hkv %zu", a.Hq, a.Hkv);
    const int G = (int)(a.Hq / a.Hkv), GT = pick_gt(G), ni = pick_ni(a.D);
    const int nsplit = std::max(1, a.max_splits);
    DecodeParams p;
    p.q = a.q; p.k_new = a.k_new; p.v_new = a.v_new;
    p.q_stride = a.q_stride; p.kv_stride = a.kv_stride;
    p.k_cache = a.k_cache; p.v_cache = a.v_cache; p.d_len = a.d_len;
    p.Hq = (int)a.Hq; p.Hkv = (int)a.Hkv; p.D = (int)a.D; p.max_seq = (int)a.max_seq;
    p.cos_t = a.cos_t; p.sin_t = a.sin_t; p.q_norm = a.q_norm; p.k_norm = a.k_norm;
    p.norm_eps = a.norm_eps; p.scale = a.scale;
    p.nsplit = nsplit;
    const size_t rows = a.B * a.Hq * (size_t)nsplit;
    p.part_m = a.part;
    p.part_l = a.part + rows;
    p.part_ctx = a.part + 2 * rows;
    dim3 grid(nsplit, (unsigned)(a.Hkv * (G / GT)), (unsigned)a.B);
    size_t smem = attn_decode_smem_floats(GT, (int)a.D) * sizeof(float);
    int rc;
    switch (GT) {
        case 8: rc = launch_decode_gt<8>(ctx, p, ni, grid, smem, s); break;
        case 4: rc = launch_decode_gt<4>(ctx, p, ni, grid, smem, s); break;
        case 2: rc = launch_decode_gt<2>(ctx, p, ni, grid, smem, s); break;
        default: rc = launch_decode_gt<1>(ctx, p, ni, grid, smem, s); break;
    }
    LUMEN_TRY(rc);
    attn_decode_combine_kernel<<<(unsigned)(a.B * a.Hq), 64, 0, s>>>(p.part_m, p.part_l, p.part_ctx, a.out, (int)a.D,
                                                                      nsplit, const_cast<int *>(a.d_len));
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

int launch_attn_prefill(lumen_ctx *ctx, const AttnPrefillArgs &a, cudaStream_t s) {
    if (a.D == 0 || a.D > 256 || (a.D & 1)) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "attention: head_dim %zu", a.D);
    if (a.Hkv == 0 || a.Hq % a.Hkv) return set_error(ctx, LUMEN_ERR_SHAPE, "attention: Hq %zu not a multiple of Hkv %zu", a.Hq, a.Hkv);
    PrefillParams p;
    p.q = a.q; p.k = a.k; p.v = a.v; p.q_stride = a.q_stride; p.kv_stride = a.kv_stride;
    p.k_cache = a.k_cache; p.v_cache = a.v_cache;
    p.past = (int)a.past; p.S = (int)a.S; p.Hq = (int)a.Hq; p.Hkv = (int)a.Hkv; p.D = (int)a.D; p.max_seq = (int)a.max_seq;
    p.cos_t = a.cos_t; p.sin_t = a.sin_t; p.q_norm = a.q_norm; p.k_norm = a.k_norm;
    p.norm_eps = a.norm_eps; p.scale = a.scale; p.causal = a.causal;
    p.out = a.out;
    void *qrot = nullptr;
    LUMEN_TRY(dev_alloc(ctx, a.B * a.S * a.Hq * a.D * sizeof(float), &qrot));
    p.q_rot = static_cast<float *>(qrot);
    attn_prefill_prep_kernel<<<dim3((unsigned)a.S, (unsigned)a.B), kThreads, kWarps * a.D * sizeof(float), s>>>(p);
    LUMEN_LAUNCHED(ctx);
    dim3 grid((unsigned)((a.S + kWarps - 1) / kWarps), (unsigned)a.Hq, (unsigned)a.B);
    switch (pick_ni(a.D)) {
        case 1: attn_prefill_kernel<1><<<grid, kThreads, 0, s>>>(p); break;
        case 2: attn_prefill_kernel<2><<<grid, kThreads, 0, s>>>(p); break;
        case 4: attn_prefill_kernel<4><<<grid, kThreads, 0, s>>>(p); break;
        default: attn_prefill_kernel<8><<<grid, kThreads, 0, s>>>(p); break;
    }
    LUMEN_LAUNCHED(ctx);
    LUMEN_TRY(dev_free(ctx, qrot));
    return LUMEN_OK;
}

}  // namespace lumen
