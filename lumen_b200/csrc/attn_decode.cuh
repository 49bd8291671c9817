// Device code of the decode (S == 1) attention step, shared by the stand-alone kernel and the
// whole-step persistent kernel.
//
// Restates src/layers/attention/self_attention.rs:141-297 of the reference: rotate the new k into cache
// row `len`, copy v, rotate q, then softmax(q.K^T * scale).V over rows 0..=len with the
// `1/(l + 1e-9)` normalisation.  The reference walks the rows serially per (b,h) with a branching online
// softmax; here the rows are split over CTAs and warps, each keeps a running (max, sum, ctx) and the
// pieces are merged with the log-sum-exp rescale, so results agree to rounding.
#pragma once

#include "common.cuh"

namespace lumen {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;

__device__ __forceinline__ float attn_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Normalise (optional) and rotate one head vector held in shared memory `buf[D]` in place; called by
// one warp.  RoPE as encoding.rs:195-203: dst[j] = x1*c - x2*s; dst[j+half] = x2*c + x1*s.
__device__ __forceinline__ void head_norm_rope(float *buf, int D, const float *norm_w, float eps,
                                               const float *cos_row, const float *sin_row, int lane) {
    if (norm_w) {
        float ss = 0.f;
        for (int i = lane; i < D; i += 32) ss = fmaf(buf[i], buf[i], ss);
        ss = attn_warp_sum(ss);
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

// Loads one head vector (D <= 256) together with its cos/sin row in one batch of independent loads,
// then normalises (optional) and rotates it into shared memory `buf[D]`.  Same arithmetic as
// head_norm_rope; the loads are issued before anything depends on them so the whole step costs one
// memory round trip.  Called by one warp.
template <bool LOCAL = false>
__device__ __forceinline__ void load_norm_rope(float *buf, const float *src, int D, const float *norm_w, float eps,
                                               const float *cos_row, const float *sin_row, int lane) {
    const int half = D / 2;
    float v[8], nw[8], c[4], s[4];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int i = lane + 32 * t;
        v[t] = (i < D) ? (LOCAL ? src[i] : __ldcg(src + i)) : 0.f;  // LOCAL: src is already in shared memory
        nw[t] = (norm_w && i < D) ? __ldg(norm_w + i) : 1.f;
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int j = lane + 32 * t;
        c[t] = (cos_row && j < half) ? __ldg(cos_row + j) : 1.f;
        s[t] = (sin_row && j < half) ? __ldg(sin_row + j) : 0.f;
    }
    if (norm_w) {
        float ss = 0.f;
#pragma unroll
        for (int t = 0; t < 8; ++t) ss = fmaf(v[t], v[t], ss);
        ss = attn_warp_sum(ss);
        const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)D), eps)));
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = __fmul_rn(__fmul_rn(v[t], inv), nw[t]);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const int i = lane + 32 * t;
        if (i < D) buf[i] = v[t];
    }
    __syncwarp();
    if (cos_row) {
        float lo[4], hi[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int j = lane + 32 * t;
            lo[t] = (j < half) ? buf[j] : 0.f;
            hi[t] = (j < half) ? buf[j + half] : 0.f;
        }
        __syncwarp();
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            const int j = lane + 32 * t;
            if (j < half) {
                buf[j] = __fsub_rn(__fmul_rn(lo[t], c[t]), __fmul_rn(hi[t], s[t]));
                buf[j + half] = __fadd_rn(__fmul_rn(hi[t], c[t]), __fmul_rn(lo[t], s[t]));
            }
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
    DeviceStatus *status = nullptr;  // where a bounded wait that gave up is recorded (may be null)
};

// Rows of K and V a warp keeps in flight, as a function of the elements per lane NI = ceil(D / 32).
__host__ __device__ constexpr int attn_rows_in_flight(int NI) { return NI <= 2 ? 8 : (NI == 4 ? 4 : 2); }

__host__ __device__ inline size_t attn_decode_smem_floats(int GT, int D, int warps = kAttnWarps) {
    // q heads, rotated new k, per-warp (max, sum), per-warp ctx, per-warp softmax weights of one chunk + rescale factors
    return (size_t)GT * D + D + 2 * warps * GT + (size_t)warps * GT * D + (size_t)warps * (8 * GT + GT);
}

// Sums NV values over the 32 lanes at once: at every step a lane keeps half of the values it still
// carries and trades the other half with its partner, so NV = 64 costs 62 shuffles instead of 320.
// Afterwards a lane holds the complete sums of values [idx0, idx0 + max(1, NV/32)), idx0 =
// NV >= 32 ? lane * (NV/32) : lane / (32/NV), in a[0..].
template <int NV>
__device__ __forceinline__ void attn_reduce_multi(float (&a)[NV], int lane) {
    int n = NV;
#pragma unroll
    for (int bit = 16; bit > 0; bit >>= 1) {
        if (n > 1) {
            const bool up = (lane & bit) != 0;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                if (i < n / 2) {
                    const float send = up ? a[i] : a[i + n / 2];
                    const float keep = up ? a[i + n / 2] : a[i];
                    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
                }
            }
            n >>= 1;
        } else {
            a[0] += __shfl_xor_sync(0xffffffffu, a[0], bit);
        }
    }
}

// Default sink of an item's result: the plain partial arrays of DecodeParams.
struct PartOut {
    const DecodeParams *p;
    __device__ __forceinline__ void operator()(size_t row, int split, int e, float c, float M, float L) const {
        const size_t o = row * p->nsplit + split;
        p->part_ctx[o * p->D + e] = c;
        if (e == 0) {
            p->part_m[o] = M;
            p->part_l[o] = L;
        }
    }
};

// One work item: batch row b, KV head group `ygroup` (= hk * (G/GT) + group), context split `split`.
// Executed by NW warps (tid = 0 .. 32*NW-1) that share `smem` and the barrier `bar()`.
// GT query heads per item, NI = ceil(D/32) elements per lane.
// LOCAL_IN: p.q / p.k_new / p.v_new point at this item's vectors already staged in shared memory
// ([GT*D], [D], [D]) instead of the global projection buffer.
// out(row = b*Hq + head, split, e, ctx_e, max, sum) receives the item's partial result.
// The first K/V rows of every warp are requested before q is staged: cached rows do not depend on this
// step's projections, so their round trip overlaps the wait for q.
// stage() runs after those requests are issued and before q is read: the persistent kernel waits there
// for the projections of this step (and copies them to shared memory); elsewhere it is a no-op.
struct NoStage {
    __device__ __forceinline__ void operator()() const {}
};
template <int GT, int NI, bool LOCAL_IN, int NW, typename Bar, typename Out, typename Stage>
__device__ __forceinline__ void attn_decode_item(const DecodeParams &p, float *smem, int b, int ygroup, int split, int tid,
                                                 int past, Bar bar, Out out, Stage stage) {
    const int D = p.D;
    float *qs = smem;                        // [GT][D]
    float *knew = qs + GT * D;               // [D]
    float *wm = knew + D;                    // [warps][GT]
    float *wl = wm + NW * GT;        // [warps][GT]
    float *wctx = wl + NW * GT;      // [warps][GT][D]
    float *wsoft = wctx + (size_t)NW * GT * D;  // [warps][UN*GT + GT] softmax weights of a chunk, then rescale factors

    const int lane = tid & 31, warp = tid >> 5;
    const int G = p.Hq / p.Hkv;
    const int groups_per_kv = G / GT;
    const int hk = ygroup / groups_per_kv;
    const int h0 = hk * G + (ygroup % groups_per_kv) * GT;

    const int total = past + 1;
    const int chunk = (total + p.nsplit - 1) / p.nsplit;
    const int j0 = split * chunk;
    const int j1 = min(total, j0 + chunk);
    const int half = D / 2;
    const float *cos_row = p.cos_t ? p.cos_t + (size_t)past * half : nullptr;
    const float *sin_row = p.sin_t ? p.sin_t + (size_t)past * half : nullptr;
    const float *kbase = p.k_cache + ((size_t)b * p.Hkv + hk) * p.max_seq * D;
    const float *vbase = p.v_cache + ((size_t)b * p.Hkv + hk) * p.max_seq * D;

    constexpr int UN = attn_rows_in_flight(NI);  // rows whose K and V loads are in flight together
    // Two register buffers of UN rows each: the loads of the next chunk are issued before the arithmetic
    // of the current one, so a warp always has a chunk in flight.
    float kra[UN][NI], vra[UN][NI], krb[UN][NI], vrb[UN][NI];
    // Rows other than `past` come from the cache (row `past` is patched in from shared memory later).
    auto load_chunk = [&](int jb, float (&kr)[UN][NI], float (&vr)[UN][NI]) {
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int j = jb + u;
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                const int e = lane + 32 * i;
                const bool ok = j < j1 && j != past && e < D;
                kr[u][i] = ok ? __ldcg(kbase + (size_t)j * D + e) : 0.f;
                vr[u][i] = ok ? __ldcg(vbase + (size_t)j * D + e) : 0.f;
            }
        }
    };
    int jb = j0 + warp * UN;
    if (jb < j1) load_chunk(jb, kra, vra);
    stage();

    // Stage and rotate the GT query heads (one warp per head, round robin).
    for (int g = warp; g < GT; g += NW) {
        const float *src = LOCAL_IN ? p.q + (size_t)g * D : p.q + (size_t)b * p.q_stride + (size_t)(h0 + g) * D;
        load_norm_rope<LOCAL_IN>(qs + g * D, src, D, p.q_norm, p.norm_eps, cos_row, sin_row, lane);
    }
    // Every item whose range holds row `past` rotates the new k into shared memory and uses that copy
    // (and v_new straight from the projection), so no item reads the cache row written during this step;
    // the first head group of each KV head also stores the row into the cache.
    const bool owns_new = (past >= j0 && past < j1);
    const float *vnew_src = LOCAL_IN ? p.v_new : p.v_new + (size_t)b * p.kv_stride + (size_t)hk * D;
    if (owns_new && warp == NW - 1) {
        const float *ksrc = LOCAL_IN ? p.k_new : p.k_new + (size_t)b * p.kv_stride + (size_t)hk * D;
        load_norm_rope<LOCAL_IN>(knew, ksrc, D, p.k_norm, p.norm_eps, cos_row, sin_row, lane);
        if (ygroup % groups_per_kv == 0) {
            float *k_row = p.k_cache + (((size_t)b * p.Hkv + hk) * p.max_seq + past) * D;
            float *v_row = p.v_cache + (((size_t)b * p.Hkv + hk) * p.max_seq + past) * D;
            for (int i = lane; i < D; i += 32) {
                k_row[i] = knew[i];
                v_row[i] = LOCAL_IN ? vnew_src[i] : __ldcg(vnew_src + i);
            }
        }
    }
    bar();

    // A chunk of UN rows x GT heads is handled at once: the UN*GT dot products are summed across the lanes
    // by one butterfly, after which each score lives in one lane (value g*UN + u in lane idx0 .. ), the
    // lanes of a head (GS of them) agree on the chunk's maximum with log2(GS) shuffles, every lane
    // exponentiates only the scores it holds, and the weights reach all lanes through shared memory for the
    // P.V update.  Same online softmax as the reference's row-by-row form up to rounding.
    constexpr int NV = UN * GT;
    constexpr int HELD = NV >= 32 ? NV / 32 : 1;  // scores a lane holds after the butterfly
    constexpr int DUP = NV >= 32 ? 1 : 32 / NV;   // lanes that hold the same score
    constexpr int GS = 32 / GT;                   // lanes that hold scores of the same head
    const int idx0 = NV >= 32 ? lane * HELD : lane / DUP;
    const int g_l = idx0 / UN;                    // the head whose running (max, sum) this lane carries
    const bool canonical = (lane % DUP) == 0;
    float *ws = wsoft + (size_t)warp * (NV + GT);
    float q[GT][NI], ctx[GT][NI];
    float m_h = -INFINITY, l_h = 0.f;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            int e = lane + 32 * i;
            q[g][i] = (e < D) ? qs[g * D + e] : 0.f;
            ctx[g][i] = 0.f;
        }
    }

    auto do_chunk = [&](int jb, float (&kr)[UN][NI], float (&vr)[UN][NI]) {
        if (past >= jb && past < jb + UN) {  // the row appended by this step: use the staged copies
            const int u_new = past - jb;
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                if (u == u_new) {
#pragma unroll
                    for (int i = 0; i < NI; ++i) {
                        const int e = lane + 32 * i;
                        kr[u][i] = (e < D) ? knew[e] : 0.f;
                        vr[u][i] = (e < D) ? (LOCAL_IN ? vnew_src[e] : __ldcg(vnew_src + e)) : 0.f;
                    }
                }
            }
        }
        float d[NV];
#pragma unroll
        for (int g = 0; g < GT; ++g) {
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < NI; ++i) dot = fmaf(q[g][i], kr[u][i], dot);
                d[g * UN + u] = dot;
            }
        }
        attn_reduce_multi<NV>(d, lane);
        float sc[HELD];
        float cmax = -INFINITY;
#pragma unroll
        for (int k = 0; k < HELD; ++k) {
            const int u = (idx0 + k) % UN;
            sc[k] = (jb + u < j1) ? __fmul_rn(d[k], p.scale) : -INFINITY;  // rows past the range weigh nothing
            cmax = fmaxf(cmax, sc[k]);
        }
#pragma unroll
        for (int b2 = 1; b2 < GS; b2 <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, b2));
        const float mn = fmaxf(m_h, cmax);  // finite: the chunk's first row is always inside the range
        const float r = expf(m_h - mn);     // exp(-inf) = 0 on the first chunk
        float wsum = 0.f;
#pragma unroll
        for (int k = 0; k < HELD; ++k) {
            const float w = expf(sc[k] - mn);
            if (canonical) ws[idx0 + k] = w;
            wsum += w;
        }
        l_h = fmaf(l_h, r, canonical ? wsum : 0.f);
        m_h = mn;
        if ((lane & (GS - 1)) == 0) ws[NV + g_l] = r;
        __syncwarp();
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            const float rg = ws[NV + g];
#pragma unroll
            for (int i = 0; i < NI; ++i) ctx[g][i] *= rg;
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const float w = ws[g * UN + u];
#pragma unroll
                for (int i = 0; i < NI; ++i) ctx[g][i] = fmaf(w, vr[u][i], ctx[g][i]);
            }
        }
        __syncwarp();  // the weights are overwritten by the next chunk
    };
    constexpr int kStep = NW * UN;
    while (jb < j1) {
        if (jb + kStep < j1) load_chunk(jb + kStep, krb, vrb);
        do_chunk(jb, kra, vra);
        jb += kStep;
        if (jb >= j1) break;
        if (jb + kStep < j1) load_chunk(jb + kStep, kra, vra);
        do_chunk(jb, krb, vrb);
        jb += kStep;
    }

    // Merge the warps of this item.  The running sum of a head is spread over its GS lanes.
#pragma unroll
    for (int b2 = 1; b2 < GS; b2 <<= 1) l_h += __shfl_xor_sync(0xffffffffu, l_h, b2);
    if ((lane & (GS - 1)) == 0) {
        wm[warp * GT + g_l] = m_h;
        wl[warp * GT + g_l] = l_h;
    }
#pragma unroll
    for (int g = 0; g < GT; ++g) {
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            int e = lane + 32 * i;
            if (e < D) wctx[(warp * GT + g) * D + e] = ctx[g][i];
        }
    }
    bar();
    for (int idx = tid; idx < GT * D; idx += (NW * 32)) {
        const int g = idx / D, e = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, wm[w * GT + g]);
        float L = 0.f, c = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float mw = wm[w * GT + g];
            const float f = (mw == -INFINITY) ? 0.f : expf(mw - M);
            L = fmaf(wl[w * GT + g], f, L);
            c = fmaf(wctx[(w * GT + g) * D + e], f, c);
        }
        out((size_t)b * p.Hq + h0 + g, split, e, c, M, L);
    }
    bar();  // shared memory may be reused by the caller's next item
}

// Merges the splits of one (b, head) row: element e of out = ctx * (1/(l + 1e-9)) (self_attention.rs:287-290).
__device__ __forceinline__ float attn_combine_elem(const float *part_m, const float *part_l, const float *part_ctx,
                                                   size_t row, int e, int D, int nsplit) {
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, __ldcg(part_m + row * nsplit + s));
    float L = 0.f, c = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = __ldcg(part_m + row * nsplit + s);
        if (ms != -INFINITY) {
            const float f = expf(ms - M);
            L = fmaf(__ldcg(part_l + row * nsplit + s), f, L);
            c = fmaf(__ldcg(part_ctx + (row * nsplit + s) * D + e), f, c);
        }
    }
    return __fmul_rn(c, __fdiv_rn(1.0f, __fadd_rn(L, 1e-9f)));
}

}  // namespace lumen
