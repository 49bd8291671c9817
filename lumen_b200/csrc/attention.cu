// GQA attention over the static KV cache.
//
// Decode (S == 1) restates src/layers/attention/self_attention.rs:141-297 of the reference: rotate the
// new k into cache row `len`, copy v, rotate q, then softmax(q.K^T * scale).V over rows 0..=len with
// the `1/(l + 1e-9)` normalisation.  The reference walks the rows serially per (b,h) with a
// branching online softmax; here the rows are split over CTAs and warps (flash-decoding), each keeps
// a running (max, sum, ctx) and the pieces are merged with the usual log-sum-exp rescale, so results
// agree to rounding.  One CTA serves all query heads of its KV head, so K/V rows are read once per
// KV head instead of once per query head.
//
// Prefill (S > 1) restates :308-426, :519-535, :621-678: rotate q/k at positions past..past+S, slab
// write, causal mask j > past+i, softmax with `1/(sum + 1e-9)`, P.V, output in [B,S,H,D] order.
#include "common.cuh"

namespace lumen {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Normalise (optional) and rotate one head vector held in shared memory `buf[D]` in place.
// Called by one warp.  RoPE as encoding.rs:195-203: dst[j] = x1*c - x2*s; dst[j+half] = x2*c + x1*s.
__device__ void head_norm_rope(float *buf, int D, const float *norm_w, float eps, const float *cos_row,
                               const float *sin_row, int lane) {
    if (norm_w) {
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) ss = fmaf(buf[i], buf[i], ss);
        ss = warp_sum(ss);
        float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)D), eps)));
        for (int i = lane; i < D; i += 32) buf[i] = __fmul_rn(__fmul_rn(buf[i], inv), norm_w[i]);
        __syncwarp();
    }
    if (cos_row) {
        const int half = D / 2;
        for (int j = lane; j < half; j += 32) {
            float x1 = buf[j], x2 = buf[j + half];
            float c = cos_row[j], s = sin_row[j];
            buf[j] = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
            buf[j + half] = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
        }
        __syncwarp();
    }
}

struct DecodeParams {
    const float *q, *k_new, *v_new;
    size_t q_stride, kv_stride;
    float *k_cache, *v_cache;
    const int *d_len;
    int Hq, Hkv, D, max_seq;
    const float *cos_t, *sin_t, *q_norm, *k_norm;
    float norm_eps, scale;
    float *part_m, *part_l, *part_ctx;  // [B,Hq,nsplit], [B,Hq,nsplit], [B,Hq,nsplit,D]
    int nsplit;
};

// grid (nsplit, Hkv * (G/GT), B).  GT query heads per CTA, NI = ceil(D/32) elements per lane.
template <int GT, int NI>
__global__ void __launch_bounds__(kThreads) attn_decode_kernel(DecodeParams p) {
    extern __shared__ __align__(16) float smem[];
    const int D = p.D;
    float *qs = smem;                       // [GT][D]
    float *knew = qs + GT * D;              // [D]
    float *wm = knew + D;                   // [kWarps][GT]
    float *wl = wm + kWarps * GT;           // [kWarps][GT]
    float *wctx = wl + kWarps * GT;         // [kWarps][GT][D]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int G = p.Hq / p.Hkv;
    const int groups_per_kv = G / GT;
    const int hk = blockIdx.y / groups_per_kv;
    const int h0 = hk * G + (blockIdx.y % groups_per_kv) * GT;
    const int b = blockIdx.z;
    const int split = blockIdx.x;

    const int past = *p.d_len;
    const int total = past + 1;
    const int chunk = (total + p.nsplit - 1) / p.nsplit;
    const int j0 = split * chunk;
    const int j1 = min(total, j0 + chunk);
    const int half = D / 2;
    const float *cos_row = p.cos_t ? p.cos_t + (size_t)past * half : nullptr;
    const float *sin_row = p.sin_t ? p.sin_t + (size_t)past * half : nullptr;

    // Stage and rotate the GT query heads (one warp per head, round robin).
    for (int g = warp; g < GT; g += kWarps) {
        const float *src = p.q + (size_t)b * p.q_stride + (size_t)(h0 + g) * D;
        for (int i = lane; i < D; i += 32) qs[g * D + i] = src[i];
        __syncwarp();
        head_norm_rope(qs + g * D, D, p.q_norm, p.norm_eps, cos_row, sin_row, lane);
    }
    // The CTA whose range holds row `past` appends the new k (rotated) and v to the cache.
    // Only the first head group of a KV head writes; the others read what it wrote?  No: they would
    // race.  Every group whose range holds `past` keeps the new row in shared memory and uses that
    // copy, so nobody reads the freshly written global row inside this kernel.
    const bool owns_new = (past >= j0 && past < j1);
    float *k_row_cache = p.k_cache + (((size_t)b * p.Hkv + hk) * p.max_seq + past) * D;
    float *v_row_cache = p.v_cache + (((size_t)b * p.Hkv + hk) * p.max_seq + past) * D;
    if (owns_new && warp == kWarps - 1) {
        const float *ksrc = p.k_new + (size_t)b * p.kv_stride + (size_t)hk * D;
        for (int i = lane; i < D; i += 32) knew[i] = ksrc[i];
        __syncwarp();
        head_norm_rope(knew, D, p.k_norm, p.norm_eps, cos_row, sin_row, lane);
        if (blockIdx.y % groups_per_kv == 0) {
            const float *vsrc = p.v_new + (size_t)b * p.kv_stride + (size_t)hk * D;
            for (int i = lane; i < D; i += 32) {
                k_row_cache[i] = knew[i];
                v_row_cache[i] = vsrc[i];
            }
        }
    }
    __syncthreads();

    float q[GT][NI], ctx[GT][NI], m[GT], l[GT];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            int e = lane + 32 * i;
            q[g][i] = (e < D) ? qs[g * D + e] : 0.f;
            ctx[g][i] = 0.f;
        }
    }

    const float *kbase = p.k_cache + ((size_t)b * p.Hkv + hk) * p.max_seq * D;
    const float *vbase = p.v_cache + ((size_t)b * p.Hkv + hk) * p.max_seq * D;
    const float *vnew_src = p.v_new + (size_t)b * p.kv_stride + (size_t)hk * D;
    constexpr int UN = 4;
    for (int jb = j0 + warp * UN; jb < j1; jb += kWarps * UN) {
        float kr[UN][NI], vr[UN][NI];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int j = jb + u;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int e = lane + 32 * i;
                float kv = 0.f, vv = 0.f;
                if (j < j1 && e < D) {
                    if (j == past) {  // the row appended by this step: use the staged copy
                        kv = knew[e];
                        vv = vnew_src[e];
                    } else {
                        kv = __ldcg(kbase + (size_t)j * D + e);
                        vv = __ldcg(vbase + (size_t)j * D + e);
                    }
                }
                kr[u][i] = kv;
                vr[u][i] = vv;
            }
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            if (jb + u >= j1) break;
#pragma unroll
            for (int g = 0; g < GT; ++g) {
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < NI; ++i) dot = fmaf(q[g][i], kr[u][i], dot);
                dot = warp_sum(dot);
                const float sc = __fmul_rn(dot, p.scale);
                const float mn = fmaxf(m[g], sc);
                const float r = expf(m[g] - mn);  // exp(-inf) = 0 on the first row
                const float w = expf(sc - mn);
                l[g] = fmaf(l[g], r, w);
#pragma unroll
                for (int i = 0; i < NI; ++i) ctx[g][i] = fmaf(w, vr[u][i], ctx[g][i] * r);
                m[g] = mn;
            }
        }
    }

    // Merge the warps of this CTA.
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        if (lane == 0) {
            wm[warp * GT + g] = m[g];
            wl[warp * GT + g] = l[g];
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            int e = lane + 32 * i;
            if (e < D) wctx[(warp * GT + g) * D + e] = ctx[g][i];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < GT * D; idx += kThreads) {
        const int g = idx / D, e = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) M = fmaxf(M, wm[w * GT + g]);
        float L = 0.f, c = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const float mw = wm[w * GT + g];
            const float f = (mw == -INFINITY) ? 0.f : expf(mw - M);
            L = fmaf(wl[w * GT + g], f, L);
            c = fmaf(wctx[(w * GT + g) * D + e], f, c);
        }
        const size_t o = ((size_t)b * p.Hq + h0 + g) * p.nsplit + split;
        p.part_ctx[o * D + e] = c;
        if (e == 0) {
            p.part_m[o] = M;
            p.part_l[o] = L;
        }
    }
}

// Merge the splits: out = ctx * (1/(l + 1e-9))  (self_attention.rs:287-290).  grid (B*Hq).
// Thread 0 of block 0 advances the cache length afterwards (c.len = new_len, :179).
__global__ void attn_decode_combine_kernel(const float *__restrict__ part_m, const float *__restrict__ part_l,
                                           const float *__restrict__ part_ctx, float *__restrict__ out, int D,
                                           int nsplit, int *d_len_bump) {
    const size_t row = blockIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_m[row * nsplit + s]);
    float L = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = part_m[row * nsplit + s];
        if (ms != -INFINITY) L = fmaf(part_l[row * nsplit + s], expf(ms - M), L);
    }
    const float inv = __fdiv_rn(1.0f, __fadd_rn(L, 1e-9f));
    for (int e = threadIdx.x; e < D; e += blockDim.x) {
        float c = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float ms = part_m[row * nsplit + s];
            if (ms != -INFINITY) c = fmaf(part_ctx[(row * nsplit + s) * D + e], expf(ms - M), c);
        }
        out[row * D + e] = __fmul_rn(c, inv);
    }
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
            dot = warp_sum(dot);
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
    // Enough CTAs to cover the SMs about twice, but at least 64 rows per split.
    size_t base = std::max<size_t>(1, B * Hkv);
    size_t want = ((size_t)num_sms * 2 + base - 1) / base;
    size_t by_len = std::max<size_t>(1, (len + 63) / 64);
    return (int)std::max<size_t>(1, std::min<size_t>(std::min(want, by_len), 64));
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
    size_t smem = ((size_t)GT * a.D + a.D + 2 * kWarps * GT + (size_t)kWarps * GT * a.D) * sizeof(float);
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
