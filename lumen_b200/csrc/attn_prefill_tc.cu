// Prefill attention (S > 1 query positions, src/layers/attention/self_attention.rs:519-678) on the 5th-generation
// tensor cores: scores = Q.K^T, causal mask j > past + i, softmax with 1/(sum + 1e-9), ctx = P.V, without the
// reference's S x L score scratch (the softmax runs tile by tile with a running maximum, like its decode path).
//
// One CTA of 128 threads owns 128 query positions of one (batch row, query head) and walks the cached rows in
// tiles of 64:
//   - thread 0 brings the tile of K (64 rows x D) and of V^T (D x 64 rows) into a two-stage shared-memory ring
//     with TMA (128-byte swizzle, mbarrier transaction counts) and issues the tcgen05.mma instructions;
//   - S[128 x 64] = Q.K^T accumulates in tensor memory; thread r reads row r back (tcgen05.ld: lane r of
//     tensor memory is row r of the tile), applies scale and mask, updates the row maximum and sum, and writes
//     the weights P[r, 0..63] into shared memory in the swizzled K-major layout the tensor core reads;
//   - O_tile[128 x D] = P.V^T accumulates in tensor memory; thread r folds its row into the running context
//     held in registers: ctx = ctx * exp(m_old - m_new) + O_tile.
// f32 values go through the tensor cores as hi + lo bf16 pairs (hi = bf16(x), lo = bf16(x - hi)) and three of the
// four cross products are accumulated in f32, which keeps products to ~2^-17 relative: the result agrees with
// the f32 reference to ~1e-5.  Q, K and V^T are split (and V transposed) by small kernels beforehand; rows
// beyond the context are zero so that masked weights (exactly 0) meet finite values.
//
// Every wait is bounded; a wait that gives up records LUMEN_ERR_TIMEOUT, the CTA leaves its loop at the next
// block-wide barrier, lets the copies in flight land, frees its tensor memory and returns.
#include "tc_common.cuh"

namespace lumen {
namespace {

using namespace tc;

constexpr int kBQ = 128;   // query rows per CTA
constexpr int kBKV = 64;   // cached rows per tile
constexpr int kFaWorkers = 256;             // 8 warps: two threads per query row
constexpr int kFaThreads = kFaWorkers + 64;  // + a warp whose first lane issues the MMAs + a warp whose first lane issues the copies

template <int D>
struct FaGeom {
    static constexpr int kKB = D / kBK;                      // 64-element blocks along the head dimension
    static constexpr uint32_t kQTile = kBQ * kBK * 2;        // one (hi | lo, block) tile of Q: 128 rows of 128 bytes
    static constexpr uint32_t kQBytes = 2 * kKB * kQTile;    // hi blocks, then lo blocks
    static constexpr uint32_t kKTile = kBKV * kBK * 2;       // 64 rows of 128 bytes
    static constexpr uint32_t kKBytes = 2 * kKB * kKTile;    // hi blocks, then lo blocks
    static constexpr uint32_t kVTile = D * kBK * 2;          // V^T: D rows of 64 cached rows
    static constexpr uint32_t kVBytes = 2 * kVTile;          // hi, lo
    static constexpr uint32_t kStageBytes = kKBytes + kVBytes;
    static constexpr uint32_t kPTile = kBQ * kBK * 2;
    static constexpr uint32_t kPBytes = 2 * kPTile;          // hi, lo
    static constexpr int kStages = 2;
    static constexpr size_t kSmem = kQBytes + kStages * kStageBytes + kPBytes + 1024;  // + slack for the alignment
    // S of even tiles: columns 0..63, S of odd tiles: 64..127, O of even tiles: 128..128+D-1, O of odd tiles after it
    static constexpr int kTmemCols = D > 64 ? 512 : 256;
    static constexpr uint32_t kIdescS = idesc_bf16(kBQ, kBKV);
    static constexpr uint32_t kIdescO = idesc_bf16(kBQ, D);
};

struct FaParams {
    float *out;  // [B, S, Hq, D]
    int S, Hq, Hkv, past, total, causal;
    int s_pad, l_pad;  // padded extents of the split copies
    float scale;
    DeviceStatus *status;
};

__device__ __forceinline__ float ex2(float x) {  // 2^x, one MUFU operation (relative error 2^-22; -inf -> 0)
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// A wait that also ends when another thread of the CTA has given up (nobody leaves the tile loop early, so
// every barrier keeps its full set of participants; after a failure the remaining iterations do not wait).
__device__ __forceinline__ bool wait_or_failed(uint64_t *bar, uint32_t parity, volatile int *failed, DeviceStatus *status, int site) {
    if (*failed) return false;
    if (bar_try(bar, parity)) return true;
    const long long t0 = clock64();
    while (!bar_try(bar, parity)) {
        if (*failed) return false;
        if (clock64() - t0 > kTcWaitCycles) {
            if (status && atomicCAS(&status->code, 0, LUMEN_ERR_TIMEOUT) == 0) status->detail0 = site;
            *failed = 1;
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void bar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}

// grid (s_pad / 128, Hq, B); 8 worker warps, warp 8 (first lane) issues the MMAs, warp 9 (first lane) the copies
template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_qhi, const __grid_constant__ CUtensorMap map_qlo,
                       const __grid_constant__ CUtensorMap map_khi, const __grid_constant__ CUtensorMap map_klo,
                       const __grid_constant__ CUtensorMap map_vhi, const __grid_constant__ CUtensorMap map_vlo, const FaParams p) {
    using G = FaGeom<D>;
    constexpr int kKB = G::kKB, kDH = D / 2;  // a worker thread owns half a row of the context
    extern __shared__ unsigned char smem_raw[];
    // the 128-byte swizzle pattern repeats every 1024 bytes: tiles must start on that boundary
    unsigned char *q_s = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *ring = q_s + G::kQBytes;
    unsigned char *p_s = ring + G::kStages * G::kStageBytes;
    __shared__ uint64_t q_bar, k_full[G::kStages], v_full[G::kStages], k_free[G::kStages], v_free[G::kStages], s_bar[2], o_bar, p_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;
    // [column half][row]: row maxima, at the end the row sums.  One copy is enough: a thread writes its next value
    // only after P.V of this tile, which is issued after its partner announced its weights (and so has read).
    __shared__ float xch[2][kBQ];
    volatile int *failed = &failed_s;
    const int tid = threadIdx.x, warp = tid >> 5;
    // the last tiles of a causal prompt walk the most rows: they go first
    const int qt = (int)(gridDim.x - 1 - blockIdx.x);
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (p.Hq / p.Hkv);
    const int i0 = qt * kBQ;
    // cached rows this tile can see: up to the diagonal of its last query row
    const int i_hi = min(i0 + kBQ, p.S) - 1;
    const int visible = p.causal ? min(p.total, p.past + i_hi + 1) : p.total;
    const int nt = (visible + kBKV - 1) / kBKV;

    if (tid == 0) {
        bar_init(&q_bar, 1);
        for (int s = 0; s < G::kStages; ++s) {
            bar_init(&k_full[s], 1);
            bar_init(&v_full[s], 1);
            bar_init(&k_free[s], 1);
            bar_init(&v_free[s], 1);
        }
        bar_init(&s_bar[0], 1);
        bar_init(&s_bar[1], 1);
        bar_init(&o_bar, 1);
        bar_init(&p_bar, kFaWorkers);
        failed_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kFaWorkers / 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_s)), "r"(G::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // tensor memory: scores of even tiles | scores of odd tiles | O of even tiles | O of odd tiles
    const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + 2 * kBKV;

    float ctx[kDH];
    float l = 0.f;
    if (warp == kFaWorkers / 32 + 1) {
        if ((tid & 31) == 0) {
            // ---- TMA producer: Q once, then K and V^T of tile j + 2 as soon as tile j has released its half stage ----
            const int q_row0 = (b * p.Hq + h) * p.s_pad + i0;
            const int k_row0 = (b * p.Hkv + hk) * p.l_pad;
            const int v_row0 = (b * p.Hkv + hk) * D;
            // A stage holds K (hi, lo) and V^T (hi, lo) of one tile; the two halves are refilled separately: K as
            // soon as the tile's scores are done, V^T after its P.V.
            auto load_k = [&](int j) {
                const int s = j % G::kStages;
                unsigned char *st = ring + (size_t)s * G::kStageBytes;
                bar_expect(&k_full[s], G::kKBytes);
#pragma unroll
                for (int kb = 0; kb < kKB; ++kb) {
                    tma_load_2d(st + kb * G::kKTile, &map_khi, kb * kBK, k_row0 + j * kBKV, &k_full[s]);
                    tma_load_2d(st + (kKB + kb) * G::kKTile, &map_klo, kb * kBK, k_row0 + j * kBKV, &k_full[s]);
                }
            };
            auto load_v = [&](int j) {
                const int s = j % G::kStages;
                unsigned char *st = ring + (size_t)s * G::kStageBytes;
                bar_expect(&v_full[s], G::kVBytes);
                tma_load_2d(st + G::kKBytes, &map_vhi, j * kBKV, v_row0, &v_full[s]);
                tma_load_2d(st + G::kKBytes + G::kVTile, &map_vlo, j * kBKV, v_row0, &v_full[s]);
            };
            bar_expect(&q_bar, G::kQBytes);
#pragma unroll
            for (int kb = 0; kb < kKB; ++kb) {
                tma_load_2d(q_s + kb * G::kQTile, &map_qhi, kb * kBK, q_row0, &q_bar);
                tma_load_2d(q_s + (kKB + kb) * G::kQTile, &map_qlo, kb * kBK, q_row0, &q_bar);
            }
            for (int j = 0; j < nt && j < G::kStages; ++j) {
                load_k(j);
                load_v(j);
            }
#pragma unroll 1
            for (int j = 0; j + G::kStages < nt; ++j) {
                const int s = j % G::kStages;
                const uint32_t par = (uint32_t)((j / G::kStages) & 1);
                if (wait_or_failed(&k_free[s], par, failed, p.status, 640)) load_k(j + G::kStages);
                if (wait_or_failed(&v_free[s], par, failed, p.status, 641)) load_v(j + G::kStages);
            }
        }
        __syncwarp();
    } else if (warp == kFaWorkers / 32) {
        if ((tid & 31) == 0) {
            // ---- MMA issuer: never waits for a result, only for operands ----------------------------------
            // S = Q.K^T of tile j (three hi/lo products per 16-element K step) into the score buffer j % 2
            auto issue_scores = [&](int j) {
                const int s = j % G::kStages;
                bool ok = wait_or_failed(&k_full[s], (uint32_t)((j / G::kStages) & 1), failed, p.status, 600);
                if (ok && j == 0) ok = wait_or_failed(&q_bar, 0, failed, p.status, 601);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ok) {
                    const uint32_t qa = saddr(q_s), st = saddr(ring + (size_t)s * G::kStageBytes);
                    const uint32_t acc = tmem_s + (uint32_t)((j & 1) * kBKV);
#pragma unroll
                    for (int kb = 0; kb < kKB; ++kb) {
                        const uint64_t qhi = smem_desc(qa + kb * G::kQTile), qlo = smem_desc(qa + (kKB + kb) * G::kQTile);
                        const uint64_t khi = smem_desc(st + kb * G::kKTile), klo = smem_desc(st + (kKB + kb) * G::kKTile);
#pragma unroll
                        for (int kk = 0; kk < kBK / 16; ++kk) {  // UMMA K = 16 bf16 = 32 bytes = 2 descriptor units
                            umma_bf16(acc, qhi + 2 * kk, khi + 2 * kk, G::kIdescS, (kb > 0 || kk > 0) ? 1u : 0u);
                            umma_bf16(acc, qlo + 2 * kk, khi + 2 * kk, G::kIdescS, 1u);
                            umma_bf16(acc, qhi + 2 * kk, klo + 2 * kk, G::kIdescS, 1u);
                        }
                    }
                }
                // both arrive when the MMAs above have completed (at once if none was issued): the workers may read
                // the scores, the producer may refill the K half of the stage
                umma_commit(&s_bar[j & 1]);
                umma_commit(&k_free[s]);
            };
            issue_scores(0);
#pragma unroll 1
            for (int j = 0; j < nt; ++j) {
                // The next tile's scores run while the workers turn this tile's scores into weights.  Its score
                // buffer was last read for tile j - 1, whose weights were announced on p_bar before P.V of
                // tile j - 1 was issued below.
                if (j + 1 < nt) issue_scores(j + 1);
                const int s = j % G::kStages;
                bool ok = wait_or_failed(&p_bar, (uint32_t)(j & 1), failed, p.status, 630);
                if (ok) ok = wait_or_failed(&v_full[s], (uint32_t)((j / G::kStages) & 1), failed, p.status, 635);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ok) {
                    const uint32_t st = saddr(ring + (size_t)s * G::kStageBytes), pa = saddr(p_s);
                    const uint64_t phi = smem_desc(pa), plo = smem_desc(pa + G::kPTile);
                    const uint64_t vhi = smem_desc(st + G::kKBytes), vlo = smem_desc(st + G::kKBytes + G::kVTile);
                    const uint32_t acc = tmem_o + (uint32_t)((j & 1) * D);
#pragma unroll
                    for (int kk = 0; kk < kBKV / 16; ++kk) {
                        umma_bf16(acc, phi + 2 * kk, vhi + 2 * kk, G::kIdescO, kk > 0 ? 1u : 0u);
                        umma_bf16(acc, plo + 2 * kk, vhi + 2 * kk, G::kIdescO, 1u);
                        umma_bf16(acc, phi + 2 * kk, vlo + 2 * kk, G::kIdescO, 1u);
                    }
                }
                // P.V of this tile has completed when these flip: the workers may read O and rewrite the weights, the
                // producer may refill the V^T half of the stage
                umma_commit(&o_bar);
                umma_commit(&v_free[s]);
            }
        }
        __syncwarp();
    } else {
        // ---- workers: thread (row, half) owns 32 of the 64 scores of its row and D/2 of its context values ----
        const int row = tid & (kBQ - 1), half = tid >> 7, quad = warp & 3;
        const uint32_t lane_off = (uint32_t)(quad * 32) << 16;  // warps w and w + 4 read the same 32 lanes of tensor memory
        const int i_row = min(i0 + row, p.S - 1);
        const int last = p.causal ? min(p.total - 1, p.past + i_row) : p.total - 1;
        const int last_min = p.causal ? min(p.total - 1, p.past + i0) : p.total - 1;  // the smallest `last` of the CTA
        // exp(s * scale - m) = 2^(s * scale * log2(e) - m'): the maximum is kept in the base-2 domain
        const float scale2 = p.scale * 1.4426950408889634f;
#pragma unroll
        for (int e = 0; e < kDH; ++e) ctx[e] = 0.f;
        float m = -INFINITY;
        unsigned char *prow_hi = p_s + (size_t)row * 128, *prow_lo = prow_hi + G::kPTile;

        // ctx = ctx * factor + O of tile j (the accumulator of odd tiles sits D columns after that of even tiles)
        auto fold = [&](int j, float factor) {
            uint32_t v[kDH / 32][32];  // every load is issued before the one wait
#pragma unroll
            for (int q = 0; q < kDH / 32; ++q) tmem_ld32_issue(tmem_o + (uint32_t)((j & 1) * D) + lane_off + half * kDH + 32 * q, v[q]);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < kDH / 32; ++q)
#pragma unroll
                for (int c = 0; c < 32; ++c) ctx[32 * q + c] = fmaf(ctx[32 * q + c], factor, __uint_as_float(v[q][c]));
        };
        float r_prev = 0.f;  // the factor that goes with the O tile not folded in yet
#pragma unroll 1
        for (int j = 0; j < nt; ++j) {
            wait_or_failed(&s_bar[j & 1], (uint32_t)((j >> 1) & 1), failed, p.status, 610);
            __syncwarp();  // the tensor-memory loads below are warp-wide
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc[32];
            {
                uint32_t v[32];
                tmem_ld32(tmem_s + (uint32_t)((j & 1) * kBKV) + lane_off + 32 * half, v);
#pragma unroll
                for (int c = 0; c < 32; ++c) sc[c] = __uint_as_float(v[c]);
            }
            const int key0 = j * kBKV + 32 * half;
            float mx = -INFINITY;
            if (j * kBKV + kBKV - 1 > last_min) {  // the tile crosses the diagonal or the end of the context (same for the CTA)
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    sc[c] = key0 + c <= last ? sc[c] * scale2 : -INFINITY;
                    mx = fmaxf(mx, sc[c]);
                }
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    sc[c] *= scale2;
                    mx = fmaxf(mx, sc[c]);
                }
            }
            // the row maximum needs the other half's: exchanged between warps w and w + 4 (64-thread named barriers:
            // one after the writes, one after the reads so that the next tile's write cannot overtake a read)
            xch[half][row] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
            const float mt = fmaxf(m, fmaxf(mx, xch[half ^ 1][row]));
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
            const float r = ex2(m - mt);  // 0 for the first tile (m = -inf; row 0 of the cache is visible to every query)
            m = mt;
            float lsum = 0.f;
            uint32_t hi[16], lo[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const float w0 = ex2(sc[2 * u] - mt), w1 = ex2(sc[2 * u + 1] - mt);
                lsum += w0 + w1;
                hi[u] = pack_bf16(w0, w1);  // low half: w0
                lo[u] = pack_bf16(w0 - __uint_as_float(hi[u] << 16), w1 - __uint_as_float(hi[u] & 0xffff0000u));
            }
            l = fmaf(l, r, lsum);  // this half's share of the row sum: both halves scale by the same factors
            // Everything above overlapped P.V of the previous tile; the weights buffer is free once that has completed.
            if (j > 0) {
                wait_or_failed(&o_bar, (uint32_t)((j - 1) & 1), failed, p.status, 620);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
#pragma unroll
            for (int c8 = 0; c8 < 4; ++c8) {
                // 128-byte swizzle: 16-byte chunk c of row r sits at chunk position c ^ (r & 7)
                const int off = (((4 * half + c8) ^ (row & 7)) << 4);
                *reinterpret_cast<uint4 *>(prow_hi + off) = make_uint4(hi[4 * c8], hi[4 * c8 + 1], hi[4 * c8 + 2], hi[4 * c8 + 3]);
                *reinterpret_cast<uint4 *>(prow_lo + off) = make_uint4(lo[4 * c8], lo[4 * c8 + 1], lo[4 * c8 + 2], lo[4 * c8 + 3]);
            }
            // the weights were written through the generic proxy; the tensor core reads through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            bar_arrive(&p_bar);
            // while P.V of this tile runs: fold in the previous tile's O (its accumulator is rewritten by the tile after
            // this one, whose P.V is not issued before this thread has announced that tile's weights)
            if (j > 0) {
                __syncwarp();  // the tensor-memory loads are warp-wide
                fold(j - 1, r_prev);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            r_prev = r;
        }
        wait_or_failed(&o_bar, (uint32_t)((nt - 1) & 1), failed, p.status, 621);
        __syncwarp();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        fold(nt - 1, r_prev);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        xch[half][row] = l;
    }
    __syncthreads();
    if (!*failed) {
        if (warp < kFaWorkers / 32) {
            const int row = tid & (kBQ - 1), half = tid >> 7;
            if (i0 + row < p.S) {
                const float inv = __fdiv_rn(1.0f, __fadd_rn(xch[0][row] + xch[1][row], 1e-9f));
                float *o = p.out + (((size_t)b * p.S + (i0 + row)) * p.Hq + h) * D + half * kDH;
#pragma unroll
                for (int e = 0; e < kDH; e += 4)
                    *reinterpret_cast<float4 *>(o + e) = make_float4(__fmul_rn(ctx[e], inv), __fmul_rn(ctx[e + 1], inv),
                                                                     __fmul_rn(ctx[e + 2], inv), __fmul_rn(ctx[e + 3], inv));
            }
        }
    } else if (tid == kFaWorkers + 32) {
        // A wait gave up: let the copies that are still in flight land before the CTA exits (bounded).
        const long long t0 = clock64();
        while (!bar_try(&q_bar, 0) && clock64() - t0 < kTcWaitCycles) {}
        for (int s = 0; s < G::kStages; ++s) {
            const long long t1 = clock64();
            while (!bar_try(&k_full[s], 0) && !bar_try(&k_full[s], 1) && clock64() - t1 < kTcWaitCycles) {}
            while (!bar_try(&v_full[s], 0) && !bar_try(&v_full[s], 1) && clock64() - t1 < kTcWaitCycles) {}
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kFaWorkers / 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(G::kTmemCols) : "memory");
}

__device__ __forceinline__ void split_store(float x, __nv_bfloat16 *hi, __nv_bfloat16 *lo, size_t i) {
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(x - __bfloat162float(h));
}

// q_rot [B, S, Hq, D] f32 -> hi / lo [B, Hq, s_pad, D] bf16, rows s >= S zero.  One thread per element.
__global__ void fa_split_q_kernel(const float *__restrict__ q_rot, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
                                  int S, int Hq, int D, int s_pad, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = (int)(i % D);
    const size_t row = i / D;
    const int s = (int)(row % s_pad);
    const size_t bh = row / s_pad;
    const size_t b = bh / Hq, h = bh % Hq;
    split_store(s < S ? q_rot[((b * S + s) * Hq + h) * D + e] : 0.f, hi, lo, i);
}

// K cache [B*Hkv, max_seq, D] f32 -> hi / lo [B*Hkv, l_pad, D] bf16, rows >= total zero.
__global__ void fa_split_k_kernel(const float *__restrict__ k_cache, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
                                  int total, int max_seq, int D, int l_pad, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int e = (int)(i % D);
    const size_t row = i / D;
    const int j = (int)(row % l_pad);
    const size_t bh = row / l_pad;
    split_store(j < total ? k_cache[(bh * max_seq + j) * D + e] : 0.f, hi, lo, i);
}

// V cache [B*Hkv, max_seq, D] f32 -> transposed hi / lo [B*Hkv, D, l_pad] bf16, columns >= total zero.
// grid (l_pad / 64, B*Hkv); a CTA transposes 64 cached rows through shared memory.
template <int D>
__global__ void __launch_bounds__(256)
fa_split_vt_kernel(const float *__restrict__ v_cache, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo, int total,
                   int max_seq, int l_pad) {
    __shared__ float tile[64][D + 1];
    const int j0 = blockIdx.x * 64;
    const size_t bh = blockIdx.y;
    for (int i = threadIdx.x; i < 64 * D; i += 256) {
        const int jr = i / D, e = i % D;
        tile[jr][e] = j0 + jr < total ? v_cache[(bh * max_seq + j0 + jr) * D + e] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * D; i += 256) {
        const int e = i / 64, jr = i % 64;
        split_store(tile[jr][e], hi, lo, (bh * D + e) * (size_t)l_pad + j0 + jr);
    }
}

template <int D>
int launch_fa(lumen_ctx *ctx, const CUtensorMap *maps, const FaParams &p, dim3 grid, cudaStream_t s) {
    static bool attr_set[64] = {false};
    const int dev = ctx->device >= 0 && ctx->device < 64 ? ctx->device : 0;
    if (!attr_set[dev]) {
        LUMEN_CUDA(ctx, cudaFuncSetAttribute(attn_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FaGeom<D>::kSmem));
        attr_set[dev] = true;
    }
    attn_prefill_tc_kernel<D><<<grid, kFaThreads, FaGeom<D>::kSmem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
    LUMEN_LAUNCHED(ctx);
    return LUMEN_OK;
}

}  // namespace

// Head dimensions 64 and 128, prompts of at least 64 positions (shorter ones leave most of a 128-row tile empty
// and stay on the warp-per-row kernel).  LUMEN_NO_TC_ATTN=1 switches the path off.
bool attn_prefill_tc_usable(const AttnPrefillArgs &a) {
    static const bool off = [] {
        const char *e = getenv("LUMEN_NO_TC_ATTN");
        return e && e[0] == '1';
    }();
    if (off || (a.D != 64 && a.D != 128) || a.S < 64) return false;
    const size_t l_pad = (a.past + a.S + 63) / 64 * 64, s_pad = (a.S + 127) / 128 * 128;
    // tensor-map coordinates are 32-bit row numbers
    return a.B * a.Hq * s_pad < ((size_t)1 << 31) && a.B * a.Hkv * l_pad < ((size_t)1 << 31) && a.B <= 65535 && a.Hq <= 65535;
}

// q_rot: the rotated queries [B, S, Hq, D]; the cache already holds rows 0 .. past + S - 1.
int launch_attn_prefill_tc(lumen_ctx *ctx, const AttnPrefillArgs &a, const float *q_rot, cudaStream_t s) {
    const size_t total = a.past + a.S;
    const size_t l_pad = (total + 63) / 64 * 64, s_pad = (a.S + kBQ - 1) / kBQ * kBQ;
    const size_t nq = a.B * a.Hq * s_pad * a.D, nkv = a.B * a.Hkv * l_pad * a.D;
    void *ws = nullptr;
    LUMEN_TRY(dev_alloc(ctx, (2 * nq + 4 * nkv) * sizeof(__nv_bfloat16), &ws));  // every count is a multiple of 64 * 64
    __nv_bfloat16 *qhi = static_cast<__nv_bfloat16 *>(ws), *qlo = qhi + nq;
    __nv_bfloat16 *khi = qlo + nq, *klo = khi + nkv, *vhi = klo + nkv, *vlo = vhi + nkv;
    int rc = LUMEN_OK;
    auto launched = [&](const char *what) {
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = cuda_fail(ctx, e, what);
        else ctx->launches += 1;
    };
    fa_split_q_kernel<<<(unsigned)((nq + 255) / 256), 256, 0, s>>>(q_rot, qhi, qlo, (int)a.S, (int)a.Hq, (int)a.D, (int)s_pad, nq);
    launched("fa_split_q_kernel launch");
    if (rc == LUMEN_OK) {
        fa_split_k_kernel<<<(unsigned)((nkv + 255) / 256), 256, 0, s>>>(a.k_cache, khi, klo, (int)total, (int)a.max_seq, (int)a.D, (int)l_pad, nkv);
        launched("fa_split_k_kernel launch");
    }
    if (rc == LUMEN_OK) {
        const dim3 g((unsigned)(l_pad / 64), (unsigned)(a.B * a.Hkv));
        if (a.D == 64) fa_split_vt_kernel<64><<<g, 256, 0, s>>>(a.v_cache, vhi, vlo, (int)total, (int)a.max_seq, (int)l_pad);
        else fa_split_vt_kernel<128><<<g, 256, 0, s>>>(a.v_cache, vhi, vlo, (int)total, (int)a.max_seq, (int)l_pad);
        launched("fa_split_vt_kernel launch");
    }
    CUtensorMap maps[6];
    if (rc == LUMEN_OK) rc = make_map(ctx, &maps[0], qhi, a.B * a.Hq * s_pad, a.D, kBQ);
    if (rc == LUMEN_OK) rc = make_map(ctx, &maps[1], qlo, a.B * a.Hq * s_pad, a.D, kBQ);
    if (rc == LUMEN_OK) rc = make_map(ctx, &maps[2], khi, a.B * a.Hkv * l_pad, a.D, kBKV);
    if (rc == LUMEN_OK) rc = make_map(ctx, &maps[3], klo, a.B * a.Hkv * l_pad, a.D, kBKV);
    if (rc == LUMEN_OK) rc = make_map(ctx, &maps[4], vhi, a.B * a.Hkv * a.D, l_pad, (int)a.D);
    if (rc == LUMEN_OK) rc = make_map(ctx, &maps[5], vlo, a.B * a.Hkv * a.D, l_pad, (int)a.D);
    if (rc == LUMEN_OK) {
        FaParams p{a.out, (int)a.S, (int)a.Hq, (int)a.Hkv, (int)a.past, (int)total, a.causal, (int)s_pad, (int)l_pad, a.scale, ctx->d_status};
        const dim3 grid((unsigned)(s_pad / kBQ), (unsigned)a.Hq, (unsigned)a.B);
        rc = a.D == 64 ? launch_fa<64>(ctx, maps, p, grid, s) : launch_fa<128>(ctx, maps, p, grid, s);
    }
    const int rc2 = dev_free(ctx, ws);
    return rc != LUMEN_OK ? rc : rc2;
}

}  // namespace lumen
