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

// ---- decode, long contexts: tiled kernel ------------------------------------------------------------
// For GQA groups of 4 or 8 query heads and head dimensions 64 / 128.  A CTA still owns (batch row, KV head,
// context split) and serves the whole query group from one read of K and V, but the work of a warp is
// organised as two small register-tiled products per tile of TR cached rows instead of one shuffle-reduced
// dot product per row and head:
//   - the warp brings a K tile and a V tile (TR rows = 8 KB each, contiguous in the cache) into shared
//     memory with one TMA bulk copy each (cp.async.bulk + an mbarrier per warp and stage, three stages:
//     two tiles in flight behind the one in use; bounded waits);
//   - scores S[GT][TR] = q . K^T: lane (hg, rg) accumulates HT = GT/2 heads x RPL = TR/16 rows over the D/4
//     chunks, each lane walking the chunks in an order rotated by rg so that the 16 rows read by one load
//     fall into different banks;
//   - online softmax per tile: the tile maximum of a head needs 4 shuffles, every score is exponentiated
//     once, the weights go to a TR x GT table in shared memory;
//   - ctx[GT][D] += P^T . V: lane (hg, dg) accumulates HT heads x D/16 dimensions over the TR rows (one
//     128-bit load of V per D/64 and one broadcast load of the HT weights per row).
// About 90 instructions per KB of cache read instead of 150, almost all independent FMAs.  The partial
// results leave through the same (max, sum, ctx) records as the other kernel, so the merge is shared.
constexpr int kTiledStages = 3;  // tiles of K and of V per warp in shared memory: two in flight behind the one in use

template <int D>
__host__ __device__ constexpr int tiled_rows() { return 2048 / D; }  // rows per tile: 8 KB of K, 8 KB of V
template <int D>
__host__ __device__ constexpr int tiled_warps() { return 4; }

template <int D, int GT>
__host__ __device__ constexpr size_t tiled_smem_floats() {
    // q heads | rotated new k | per warp: K and V tiles of every stage and the weight table | per-warp (max, sum)
    return (size_t)GT * D + D + (size_t)tiled_warps<D>() * (2 * kTiledStages * tiled_rows<D>() * D + tiled_rows<D>() * GT) +
           2 * tiled_warps<D>() * GT;
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tile_bar_init(uint64_t *bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tile_bar_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tile_bar_try(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_addr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared (TMA), completion counted in bytes on `bar`.
__device__ __forceinline__ void tile_bulk_load(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_addr(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// Bounded wait: gives up after ~0.1 s of clock cycles and reports it (the kernel then finishes with whatever
// it has; the host sees LUMEN_ERR_TIMEOUT at its next synchronising call).
__device__ __forceinline__ bool tile_bar_wait(uint64_t *bar, uint32_t parity, DeviceStatus *status) {
    if (tile_bar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!tile_bar_try(bar, parity)) {
        if (clock64() - t0 > 200000000LL) {
            if (status && atomicCAS(&status->code, 0, LUMEN_ERR_TIMEOUT) == 0) status->detail0 = 400;
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ float dot4(const float4 a, const float4 b, float acc) {
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc);
    acc = fmaf(a.w, b.w, acc);
    return acc;
}

// grid (nsplit, Hkv * (G/GT), B), (tiled_warps<D>() * 32) threads
template <int D, int GT>
__global__ void __launch_bounds__((tiled_warps<D>() * 32), 1) attn_decode_tiled_kernel(DecodeParams p) {
    constexpr int NW = tiled_warps<D>();
    constexpr int TR = tiled_rows<D>();  // 32 (D = 64) or 16 (D = 128)
    constexpr int CH = D / 4;            // 16-byte chunks per row
    constexpr int HT = GT / 2;           // heads per lane
    constexpr int RPL = TR / 16;         // rows per lane in the score product
    constexpr int DQ = D / 64;           // float4s of ctx per lane and head
    extern __shared__ __align__(16) float smem[];
    float *qs = smem;                          // [GT][D]
    float *knew = qs + GT * D;                 // [D]
    float *wbase = knew + D;                   // per warp: K tiles, V tiles, P
    constexpr int NS = kTiledStages;
    constexpr int kPerWarp = 2 * NS * TR * D + TR * GT;
    float *wm = wbase + NW * kPerWarp;         // [NW][GT]
    float *wl = wm + NW * GT;                  // [NW][GT]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hg = lane >> 4, rg = lane & 15;
    const int b = blockIdx.z, ygroup = blockIdx.y, split = blockIdx.x;
    const int past = *p.d_len;
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
    float *ktile = wbase + warp * kPerWarp;             // [NS][TR][D], chunks swizzled
    float *vtile = ktile + NS * TR * D;                 // [NS][TR][D]
    float *pt = vtile + NS * TR * D;                    // [TR][GT]

    // Tiles arrive by TMA: the TR rows of a tile are contiguous in the cache, so a tile is one bulk copy for K
    // and one for V, counted on the (warp, stage) mbarrier.  The last tile of the range copies only its valid
    // rows.  Issued by lane 0 of the warp that will consume the tile.
    __shared__ uint64_t bars[NW * NS];
    if (tid == 0) {
        for (int i = 0; i < NW * NS; ++i) tile_bar_init(&bars[i]);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto load_tile = [&](int jt, int buf) {
        if (jt < j1 && lane == 0) {
            const uint32_t bytes = (uint32_t)min(TR, j1 - jt) * D * sizeof(float);
            uint64_t *bar = &bars[warp * NS + buf];
            tile_bar_expect(bar, 2 * bytes);
            tile_bulk_load(ktile + buf * TR * D, kbase + (size_t)jt * D, bytes, bar);
            tile_bulk_load(vtile + buf * TR * D, vbase + (size_t)jt * D, bytes, bar);
        }
    };
    const int jw0 = j0 + warp * TR;  // first tile of this warp; the next ones follow every NW * TR rows
    constexpr int kStep = NW * TR;
#pragma unroll
    for (int st = 0; st < NS - 1; ++st) load_tile(jw0 + st * kStep, st);

    // Stage and rotate the query heads and this step's k (as in the other kernel).
    for (int g = warp; g < GT; g += NW) {
        const float *src = p.q + (size_t)b * p.q_stride + (size_t)(h0 + g) * D;
        load_norm_rope<false>(qs + g * D, src, D, p.q_norm, p.norm_eps, cos_row, sin_row, lane);
    }
    const bool owns_new = (past >= j0 && past < j1);
    const float *vnew_src = p.v_new + (size_t)b * p.kv_stride + (size_t)hk * D;
    if (owns_new && warp == NW - 1) {
        const float *ksrc = p.k_new + (size_t)b * p.kv_stride + (size_t)hk * D;
        load_norm_rope<false>(knew, ksrc, D, p.k_norm, p.norm_eps, cos_row, sin_row, lane);
        if (ygroup % groups_per_kv == 0) {
            float *k_row = p.k_cache + (((size_t)b * p.Hkv + hk) * p.max_seq + past) * D;
            float *v_row = p.v_cache + (((size_t)b * p.Hkv + hk) * p.max_seq + past) * D;
            for (int i = lane; i < D; i += 32) {
                k_row[i] = knew[i];
                v_row[i] = __ldcg(vnew_src + i);
            }
        }
    }
    __syncthreads();

    float m[HT], l[HT];
    float4 ctx[HT][DQ];
#pragma unroll
    for (int i = 0; i < HT; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int q4 = 0; q4 < DQ; ++q4) ctx[i][q4] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const float4 *qs4 = reinterpret_cast<const float4 *>(qs);

    int buf = 0, it = 0;
    bool alive = true;
    for (int jt = jw0; jt < j1 && alive; jt += kStep, buf = (buf + 1 == NS ? 0 : buf + 1), ++it) {
        load_tile(jt + (NS - 1) * kStep, buf == 0 ? NS - 1 : buf - 1);  // into the stage released by the previous iteration
        alive = tile_bar_wait(&bars[warp * NS + buf], (uint32_t)(it / NS) & 1u, p.status);
        float4 *k4 = reinterpret_cast<float4 *>(ktile + buf * TR * D);
        float4 *v4 = reinterpret_cast<float4 *>(vtile + buf * TR * D);
        const int nvalid = min(TR, j1 - jt);
        // Rows past the range weigh nothing, but what they are multiplied with must be finite: clear V there.
        for (int i = nvalid * CH + lane; i < TR * CH; i += 32) v4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (past >= jt && past < jt + TR) {  // the row appended by this step: take it from the staged copies
            const int r = past - jt;
            if (lane < CH) {
                k4[r * CH + lane] = reinterpret_cast<const float4 *>(knew)[lane];
                v4[r * CH + lane] = __ldcg(reinterpret_cast<const float4 *>(vnew_src) + lane);
            }
        }
        __syncwarp();
        // ---- scores ------------------------------------------------------------------------------------
        float s[RPL][HT];
#pragma unroll
        for (int rr = 0; rr < RPL; ++rr)
#pragma unroll
            for (int i = 0; i < HT; ++i) s[rr][i] = 0.f;
        // The 16 row lanes of a load read 16 different rows, whose chunks of equal index share their banks:
        // every lane therefore walks the chunks in an order rotated by its own index (a sum does not care).
#pragma unroll 4
        for (int cc = 0; cc < CH; ++cc) {
            const int c = (cc + rg) & (CH - 1);
            float4 qv[HT];
#pragma unroll
            for (int i = 0; i < HT; ++i) qv[i] = qs4[(HT * hg + i) * CH + c];
#pragma unroll
            for (int rr = 0; rr < RPL; ++rr) {
                const int r = RPL * rg + rr;
                const float4 kv = k4[r * CH + c];
#pragma unroll
                for (int i = 0; i < HT; ++i) s[rr][i] = dot4(kv, qv[i], s[rr][i]);
            }
        }
        // ---- online softmax of the tile -----------------------------------------------------------------
        float rs[HT];
#pragma unroll
        for (int i = 0; i < HT; ++i) {
            float tmax = -INFINITY;
#pragma unroll
            for (int rr = 0; rr < RPL; ++rr) {
                const bool ok = jt + RPL * rg + rr < j1;
                s[rr][i] = ok ? __fmul_rn(s[rr][i], p.scale) : -INFINITY;
                tmax = fmaxf(tmax, s[rr][i]);
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
            const float mn = fmaxf(m[i], tmax);  // finite: the tile's first row is inside the range
            rs[i] = expf(m[i] - mn);
            float wsum = 0.f;
#pragma unroll
            for (int rr = 0; rr < RPL; ++rr) {
                const float w = expf(s[rr][i] - mn);
                s[rr][i] = w;
                wsum += w;
            }
            l[i] = fmaf(l[i], rs[i], wsum);
            m[i] = mn;
        }
#pragma unroll
        for (int rr = 0; rr < RPL; ++rr)
#pragma unroll
            for (int i = 0; i < HT; ++i) pt[(RPL * rg + rr) * GT + HT * hg + i] = s[rr][i];
        __syncwarp();
        // ---- ctx = ctx * r + P^T . V ----------------------------------------------------------------------
#pragma unroll
        for (int i = 0; i < HT; ++i)
#pragma unroll
            for (int q4 = 0; q4 < DQ; ++q4) {
                ctx[i][q4].x *= rs[i]; ctx[i][q4].y *= rs[i]; ctx[i][q4].z *= rs[i]; ctx[i][q4].w *= rs[i];
            }
#pragma unroll 4
        for (int r = 0; r < TR; ++r) {
            float w[HT];
            if (HT == 4) {
                const float4 w4 = *reinterpret_cast<const float4 *>(pt + r * GT + 4 * hg);
                w[0] = w4.x; w[1] = w4.y; w[HT - 2] = w4.z; w[HT - 1] = w4.w;
            } else {
                const float2 w2 = *reinterpret_cast<const float2 *>(pt + r * GT + 2 * hg);
                w[0] = w2.x; w[HT - 1] = w2.y;
            }
#pragma unroll
            for (int q4 = 0; q4 < DQ; ++q4) {
                const float4 vv = v4[r * CH + q4 * 16 + rg];  // dimensions 4 * (q4 * 16 + rg) ..
#pragma unroll
                for (int i = 0; i < HT; ++i) {
                    ctx[i][q4].x = fmaf(w[i], vv.x, ctx[i][q4].x);
                    ctx[i][q4].y = fmaf(w[i], vv.y, ctx[i][q4].y);
                    ctx[i][q4].z = fmaf(w[i], vv.z, ctx[i][q4].z);
                    ctx[i][q4].w = fmaf(w[i], vv.w, ctx[i][q4].w);
                }
            }
        }
        __syncwarp();  // the weight table and this tile's buffers are rewritten by the next iterations
    }

    // Merge the warps of this CTA.  A head's running sum is spread over its 16 row lanes.
#pragma unroll
    for (int i = 0; i < HT; ++i) {
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) l[i] += __shfl_xor_sync(0xffffffffu, l[i], o);
        if (rg == 0) {
            wm[warp * GT + HT * hg + i] = m[i];
            wl[warp * GT + HT * hg + i] = l[i];
        }
    }
    if (!alive) {  // a wait gave up: let this warp's copies that are still in flight land before the CTA exits
        for (int sb = 0; sb < NS; ++sb) {
            const long long t0 = clock64();
            while (!tile_bar_try(&bars[warp * NS + sb], 0) && !tile_bar_try(&bars[warp * NS + sb], 1) && clock64() - t0 < 200000000LL) {}
        }
    }
    float *wctx = ktile;  // this warp's first K tile is free now: [GT][D]
#pragma unroll
    for (int i = 0; i < HT; ++i)
#pragma unroll
        for (int q4 = 0; q4 < DQ; ++q4)
            reinterpret_cast<float4 *>(wctx)[(HT * hg + i) * CH + q4 * 16 + rg] = ctx[i][q4];
    __syncthreads();
    for (int idx = tid; idx < GT * D; idx += (tiled_warps<D>() * 32)) {
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
            c = fmaf(wbase[w * kPerWarp + g * D + e], f, c);
        }
        const size_t o = ((size_t)b * p.Hq + h0 + g) * p.nsplit + split;
        p.part_ctx[o * D + e] = c;
        if (e == 0) {
            p.part_m[o] = M;
            p.part_l[o] = L;
        }
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

template <int D, int GT>
int launch_decode_tiled(lumen_ctx *ctx, const DecodeParams &p, dim3 grid, cudaStream_t s) {
    auto kern = attn_decode_tiled_kernel<D, GT>;
    constexpr size_t smem = tiled_smem_floats<D, GT>() * sizeof(float);
    static bool attr_set[64] = {false};  // per device ordinal
    const int dev = ctx->device >= 0 && ctx->device < 64 ? ctx->device : 0;
    if (!attr_set[dev]) {
        LUMEN_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    kern<<<grid, (tiled_warps<D>() * 32), smem, s>>>(p);
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
    static const size_t wave_rows = [] {
        const char *e = getenv("LUMEN_ATTN_WAVE_ROWS");
        return e ? (size_t)atoi(e) : (size_t)256;
    }();
    size_t best = 1, best_cost = ~(size_t)0;
    for (size_t ns = 1; ns <= max_ns; ++ns) {
        const size_t waves = (base * ns + (size_t)num_sms - 1) / (size_t)num_sms;
        const size_t rows = (len + ns - 1) / ns;
        const size_t cost = waves * (rows + wave_rows);
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
    p.status = ctx->d_status;
    const size_t rows = a.B * a.Hq * (size_t)nsplit;
    p.part_m = a.part;
    p.part_l = a.part + rows;
    p.part_ctx = a.part + 2 * rows;
    dim3 grid(nsplit, (unsigned)(a.Hkv * (G / GT)), (unsigned)a.B);
    size_t smem = attn_decode_smem_floats(GT, (int)a.D) * sizeof(float);
    int rc;
    // Long contexts of grouped-query models take the tiled kernel (at least four tiles of rows per split).
    const size_t rows_per_split = (a.len_hint + 1 + nsplit - 1) / nsplit;
    const bool tiled = (GT == 8 || GT == 4) && (a.D == 64 || a.D == 128) && rows_per_split >= 128 && !getenv("LUMEN_NO_TILED_ATTN");
    if (tiled) {
        if (a.D == 64) rc = GT == 8 ? launch_decode_tiled<64, 8>(ctx, p, grid, s) : launch_decode_tiled<64, 4>(ctx, p, grid, s);
        else rc = GT == 8 ? launch_decode_tiled<128, 8>(ctx, p, grid, s) : launch_decode_tiled<128, 4>(ctx, p, grid, s);
    } else
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
    if (attn_prefill_tc_usable(a)) {
        const int rc = launch_attn_prefill_tc(ctx, a, p.q_rot, s);
        const int rc2 = dev_free(ctx, qrot);
        return rc != LUMEN_OK ? rc : rc2;
    }
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
