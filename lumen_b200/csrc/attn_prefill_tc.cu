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
constexpr int kFaThreads = 128;

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
    static constexpr int kTmemCols = D > 64 ? 256 : 128;     // S: columns 0..63, O: columns 64..64+D-1
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

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&v);
}

// grid (s_pad / 128, Hq, B)
template <int D>
__global__ void __launch_bounds__(kFaThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_qhi, const __grid_constant__ CUtensorMap map_qlo,
                       const __grid_constant__ CUtensorMap map_khi, const __grid_constant__ CUtensorMap map_klo,
                       const __grid_constant__ CUtensorMap map_vhi, const __grid_constant__ CUtensorMap map_vlo, const FaParams p) {
    using G = FaGeom<D>;
    constexpr int kKB = G::kKB;
    extern __shared__ unsigned char smem_raw[];
    // the 128-byte swizzle pattern repeats every 1024 bytes: tiles must start on that boundary
    unsigned char *q_s = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char *ring = q_s + G::kQBytes;
    unsigned char *p_s = ring + G::kStages * G::kStageBytes;
    __shared__ uint64_t q_bar, full[G::kStages], s_bar, o_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed;
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
    const int q_row0 = (b * p.Hq + h) * p.s_pad + i0;
    const int k_row0 = (b * p.Hkv + hk) * p.l_pad;
    const int v_row0 = (b * p.Hkv + hk) * D;

    if (tid == 0) {
        bar_init(&q_bar, 1);
        for (int s = 0; s < G::kStages; ++s) bar_init(&full[s], 1);
        bar_init(&s_bar, 1);
        bar_init(&o_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_base_s)), "r"(G::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_base_s, tmem_o = tmem_base_s + kBKV;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

    auto load_tile = [&](int j) {  // thread 0: K and V^T of tile j into stage j % 2
        const int s = j % G::kStages;
        unsigned char *st = ring + (size_t)s * G::kStageBytes;
        bar_expect(&full[s], G::kStageBytes);
#pragma unroll
        for (int kb = 0; kb < kKB; ++kb) {
            tma_load_2d(st + kb * G::kKTile, &map_khi, kb * kBK, k_row0 + j * kBKV, &full[s]);
            tma_load_2d(st + (kKB + kb) * G::kKTile, &map_klo, kb * kBK, k_row0 + j * kBKV, &full[s]);
        }
        tma_load_2d(st + G::kKBytes, &map_vhi, j * kBKV, v_row0, &full[s]);
        tma_load_2d(st + G::kKBytes + G::kVTile, &map_vlo, j * kBKV, v_row0, &full[s]);
    };

    int in_flight = 0;  // thread 0: tiles whose copies were issued
    if (tid == 0) {
        bar_expect(&q_bar, G::kQBytes);
#pragma unroll
        for (int kb = 0; kb < kKB; ++kb) {
            tma_load_2d(q_s + kb * G::kQTile, &map_qhi, kb * kBK, q_row0, &q_bar);
            tma_load_2d(q_s + (kKB + kb) * G::kQTile, &map_qlo, kb * kBK, q_row0, &q_bar);
        }
        for (; in_flight < nt && in_flight < G::kStages; ++in_flight) load_tile(in_flight);
    }
    __syncwarp();

    // this thread's query row: position, last visible cached row
    const int i_row = min(i0 + tid, p.S - 1);
    const int last = p.causal ? min(p.total - 1, p.past + i_row) : p.total - 1;
    float ctx[D];
#pragma unroll
    for (int e = 0; e < D; ++e) ctx[e] = 0.f;
    float m = -INFINITY, l = 0.f;

#pragma unroll 1
    for (int j = 0; j < nt; ++j) {
        const int s = j % G::kStages;
        const uint32_t st = saddr(ring + (size_t)s * G::kStageBytes);
        if (tid == 0) {
            bool ok = bar_wait(&full[s], (uint32_t)((j / G::kStages) & 1), p.status, 600);
            if (ok && j == 0) ok = bar_wait(&q_bar, 0, p.status, 601);
            if (!ok) failed = 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok) {
                const uint32_t qa = saddr(q_s);
#pragma unroll
                for (int kb = 0; kb < kKB; ++kb) {
                    const uint64_t qhi = smem_desc(qa + kb * G::kQTile), qlo = smem_desc(qa + (kKB + kb) * G::kQTile);
                    const uint64_t khi = smem_desc(st + kb * G::kKTile), klo = smem_desc(st + (kKB + kb) * G::kKTile);
#pragma unroll
                    for (int kk = 0; kk < kBK / 16; ++kk) {  // UMMA K = 16 bf16 = 32 bytes = 2 descriptor units
                        umma_bf16(tmem_s, qhi + 2 * kk, khi + 2 * kk, G::kIdescS, (kb > 0 || kk > 0) ? 1u : 0u);
                        umma_bf16(tmem_s, qlo + 2 * kk, khi + 2 * kk, G::kIdescS, 1u);
                        umma_bf16(tmem_s, qhi + 2 * kk, klo + 2 * kk, G::kIdescS, 1u);
                    }
                }
            }
            umma_commit(&s_bar);  // arrives when the MMAs above have completed (at once if none was issued)
        }
        __syncwarp();
        if (!bar_wait(&s_bar, (uint32_t)(j & 1), p.status, 610)) failed = 1;
        __syncwarp();  // the tensor-memory loads below are warp-wide
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- scores of row `tid`: scale, mask, running maximum, weights -------------------------------
        float sc[kBKV];
        {
            uint32_t v[32];
            tmem_ld32(tmem_s + lane_off, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) sc[c] = __uint_as_float(v[c]);
            tmem_ld32(tmem_s + lane_off + 32, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) sc[32 + c] = __uint_as_float(v[c]);
        }
        const int key0 = j * kBKV;
        float mt = m;
#pragma unroll
        for (int c = 0; c < kBKV; ++c) {
            sc[c] = key0 + c <= last ? __fmul_rn(sc[c], p.scale) : -INFINITY;
            mt = fmaxf(mt, sc[c]);
        }
        const float r = expf(m - mt);  // 0 for the first tile (m = -inf; row 0 of the cache is visible to every query)
        m = mt;
        float lsum = 0.f;
        unsigned char *prow_hi = p_s + (size_t)tid * 128, *prow_lo = prow_hi + G::kPTile;
#pragma unroll
        for (int c8 = 0; c8 < kBKV / 8; ++c8) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float w0 = expf(sc[c8 * 8 + 2 * u] - mt), w1 = expf(sc[c8 * 8 + 2 * u + 1] - mt);
                lsum += w0 + w1;
                const __nv_bfloat16 h0 = __float2bfloat16_rn(w0), h1 = __float2bfloat16_rn(w1);
                hi[u] = pack_bf16(__bfloat162float(h0), __bfloat162float(h1));
                lo[u] = pack_bf16(w0 - __bfloat162float(h0), w1 - __bfloat162float(h1));
            }
            // 128-byte swizzle: 16-byte chunk c8 of row r sits at chunk position c8 ^ (r & 7)
            const int off = ((c8 ^ (tid & 7)) << 4);
            *reinterpret_cast<uint4 *>(prow_hi + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4 *>(prow_lo + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
        l = fmaf(l, r, lsum);
        // the weights were written through the generic proxy; the tensor core reads through the async proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (__syncthreads_or(failed)) break;  // the same answer in every thread

        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t pa = saddr(p_s);
            const uint64_t phi = smem_desc(pa), plo = smem_desc(pa + G::kPTile);
            const uint64_t vhi = smem_desc(st + G::kKBytes), vlo = smem_desc(st + G::kKBytes + G::kVTile);
#pragma unroll
            for (int kk = 0; kk < kBKV / 16; ++kk) {
                umma_bf16(tmem_o, phi + 2 * kk, vhi + 2 * kk, G::kIdescO, kk > 0 ? 1u : 0u);
                umma_bf16(tmem_o, plo + 2 * kk, vhi + 2 * kk, G::kIdescO, 1u);
                umma_bf16(tmem_o, phi + 2 * kk, vlo + 2 * kk, G::kIdescO, 1u);
            }
            umma_commit(&o_bar);
        }
        __syncwarp();
        if (!bar_wait(&o_bar, (uint32_t)(j & 1), p.status, 620)) failed = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // every MMA that read stage s has completed: refill it with the tile after next
        if (tid == 0 && in_flight < nt && !failed) load_tile(in_flight++);
        __syncwarp();  // the tensor-memory loads below are warp-wide
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(tmem_o + lane_off + c0, v);
#pragma unroll
            for (int c = 0; c < 32; ++c) ctx[c0 + c] = fmaf(ctx[c0 + c], r, __uint_as_float(v[c]));
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (!failed) {
        if (i0 + tid < p.S) {
            const float inv = __fdiv_rn(1.0f, __fadd_rn(l, 1e-9f));
            float *o = p.out + (((size_t)b * p.S + (i0 + tid)) * p.Hq + h) * D;
#pragma unroll
            for (int e = 0; e < D; e += 4)
                *reinterpret_cast<float4 *>(o + e) = make_float4(__fmul_rn(ctx[e], inv), __fmul_rn(ctx[e + 1], inv),
                                                                 __fmul_rn(ctx[e + 2], inv), __fmul_rn(ctx[e + 3], inv));
        }
    } else if (tid == 0) {
        // A wait gave up: let the copies that are still in flight land before the CTA exits (bounded).
        const long long t0 = clock64();
        while (!bar_try(&q_bar, 0) && clock64() - t0 < kTcWaitCycles) {}
        for (int s = 0; s < G::kStages; ++s) {
            const long long t1 = clock64();
            while (!bar_try(&full[s], 0) && !bar_try(&full[s], 1) && clock64() - t1 < kTcWaitCycles) {}
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(G::kTmemCols) : "memory");
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
