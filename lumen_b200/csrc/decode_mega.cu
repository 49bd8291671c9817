// Whole-token persistent decode kernel (batch 1): one launch runs LlamaModel::forward for one new
// token (src/models/llama.rs:181-206 of the reference; layer body :104-116, MLP :59-65, decode
// attention self_attention.rs:141-297, vector-matrix products src/ops/matmul.rs:42-69).
//
// Design for B200: one CTA per SM (launched cooperatively so that all CTAs are co-resident).  The
// last warp of each CTA is a producer: one elected lane walks a static schedule of weight tiles (the
// CTA's rows of every matrix of every layer, in execution order) and streams them from HBM into a
// shared-memory ring with 1-D bulk TMA copies (cp.async.bulk + mbarrier transaction counts, L2
// evict-first).  The schedule does not depend on the activations, so the producer keeps HBM busy across
// phase boundaries while the consumer warps wait for activations or run the (weight-free) attention.
//
// Consumers: the 4 consumer warps form G independent groups (G = 4, 2 or 1, chosen per matrix from its
// row length); group g owns every G-th tile, so several tiles are processed at once and no CTA-wide
// barrier sits between tiles.  Within a group every thread keeps its slice of the input vector in
// registers (4 warps leave each thread the full 255 registers), reads its 128-bit words of each weight
// row from shared memory, and the warp's partial sum per row goes to a small shared table; once per row
// block the table is reduced and the fused epilogue runs (RMSNorm in the prologue, residual add,
// SiLU*mul).  Phases of a layer: qkv | attention | o_proj(+residual) | gate/up(+SiLU*mul) |
// down(+residual).
//
// Activations cross CTAs through global memory (L2) as tagged words {f32 bits, tag}: a consumer polls
// the words it needs until their tag equals the one of the producing phase of this launch, so there is
// no grid-wide barrier and a CTA starts a phase as soon as ITS inputs exist.  Everything between two
// exchanges is arranged as one batch of independent loads, since an L2 round trip (~1 us under load)
// is the unit of cost on the critical path.
//
// Every wait (mbarrier, data poll) is bounded: on expiry the CTA records LUMEN_ERR_TIMEOUT in the
// device status word, raises an abort flag that the other CTAs poll, waits (bounded) for its own bulk
// copies still in flight and returns; the kernel never traps or spins forever.
#include <algorithm>
#include <cstdlib>

#include "attn_decode.cuh"
#include "decode_mega.cuh"

namespace lumen {
namespace {

// 4 consumer warps + 1 producer warp: at most two warps per SM sub-partition, so every thread may use up
// to 255 registers (a ninth warp would cap the kernel at 168 and the spills, with the L1 squeezed by
// ~200 KB of shared memory, turn into L2 round trips on the critical path).
constexpr int kConsumers = 128;
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kThreads = kConsumers + 32;  // + producer warp
constexpr int kMaxRowsPerTile = 8;
constexpr int kRowBlock = 128;             // rows reduced together (one per consumer thread)
constexpr int kMaxSplit = 4;               // attention splits merged in the o_proj prologue
constexpr int kTileTrace = 512;            // tiles of CTA 0 whose issue / arrival times the trace keeps
constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s at 1.9 GHz

// Floats of the shared table that holds the per-warp partial sums of a row block ([2][kRowBlock][8]) and,
// during a phase's prologue, the staged input vector (up to kmax floats).
__host__ __device__ inline size_t mega_table_floats(int kmax) {
    const size_t part = 2 * (size_t)kRowBlock * kConsumerWarps;
    return part > (size_t)kmax ? part : (((size_t)kmax + 3) / 4) * 4;
}

// ---- PTX helpers -------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cnt(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t make_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// 1-D bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }
struct ConsumerBar {
    __device__ __forceinline__ void operator()() const { consumer_bar(); }
};
// A consumer barrier after which all consumer threads agree on whether the CTA is aborting.  Exits must be
// uniform (a thread that left would make the next bar.sync wait forever), so the flag is sampled by
// thread 0 before the barrier into a slot that alternates with `k`, and read by everyone after it.
__device__ __forceinline__ bool consumer_bar_ok(volatile int *abort, volatile int *decision, int tid, int &k) {
    if (tid == 0) decision[k & 1] = *abort;
    consumer_bar();
    const bool ok = decision[k & 1] == 0;
    ++k;
    return ok;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void trace_stamp(const MegaParams &p, int cta, int tid, int slot) {
    if (p.trace && cta == 0 && tid == 0) p.trace[slot] = globaltimer_ns();
}
__device__ __forceinline__ int ld_volatile_int(const int *p) { return *reinterpret_cast<const volatile int *>(p); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// ---- shared state ------------------------------------------------------------------------------------
struct Shared {
    unsigned char *stages;
    float *part;       // [2][kRowBlock][kConsumerWarps] per-warp partial sums of the rows of one block
    float *red;        // [kConsumerWarps]
    float *attn;       // scratch of the attention item
    uint64_t *full;    // [S]
    uint64_t *empty;   // [S]
    volatile int *abort;
    volatile int *decision;  // [2] abort flag sampled by thread 0 before a barrier, read by all after it
    volatile int *seen;      // [S] number of uses of each stage whose data a consumer has seen land
    int S, stage_bytes;
};

__device__ __forceinline__ void raise_abort(const MegaParams &p, volatile int *abort, int site, int value) {
    *abort = 1;
    atomicExch(p.abort_flag, 1);
    if (atomicCAS(&p.status->code, 0, LUMEN_ERR_TIMEOUT) == 0) {
        p.status->detail0 = site;
        p.status->detail1 = value;
    }
}

// Bounded mbarrier wait; false = gave up (abort raised) or somebody else aborted.
__device__ __forceinline__ bool mbar_wait(const MegaParams &p, Shared &sh, uint64_t *bar, uint32_t parity, int site) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 63) == 0) {
            if (*sh.abort) return false;
            if (clock64() - t0 > kWaitCycles) {
                raise_abort(p, sh.abort, site, (int)parity);
                return false;
            }
        }
    }
    return true;
}

// Bounded wait until `uses` fills of stage s are known to have landed (written by the groups that
// consumed them).  In steady state this is already true and costs one shared-memory read.
__device__ __forceinline__ bool stage_use_seen(const MegaParams &p, Shared &sh, int s, int uses, int site) {
    if (sh.seen[s] >= uses) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (sh.seen[s] < uses) {
        if ((++spins & 63) == 0) {
            if (*sh.abort) return false;
            if (clock64() - t0 > kWaitCycles) {
                raise_abort(p, sh.abort, site, uses);
                return false;
            }
        }
    }
    return true;
}

// ---- phases and tiles --------------------------------------------------------------------------------
enum PhaseKind { PH_QKV = 0, PH_ATT = 1, PH_O = 2, PH_GATEUP = 3, PH_DOWN = 4, PH_LMHEAD = 5 };

struct Phase {
    int kind, layer, nmat, N, K;
    const char *w0, *w1;
};

__device__ __forceinline__ Phase get_phase(const MegaParams &p, int ph) {
    Phase g;
    g.nmat = 1;
    g.w1 = nullptr;
    if (ph >= 5 * p.L) {
        g.kind = PH_LMHEAD; g.layer = p.L; g.N = p.V; g.K = p.H; g.w0 = p.lm_head;
        return g;
    }
    g.layer = ph / 5;
    g.kind = ph % 5;
    const MegaLayer &l = p.layers[g.layer];
    switch (g.kind) {
        case PH_QKV: g.N = p.qkv_rows; g.K = p.H; g.w0 = l.wqkv; break;
        case PH_O: g.N = p.H; g.K = p.qd; g.w0 = l.wo; break;
        case PH_GATEUP: g.N = p.I; g.K = p.H; g.w0 = l.wgate; g.w1 = l.wup; g.nmat = 2; break;
        case PH_DOWN: g.N = p.H; g.K = p.I; g.w0 = l.wdown; break;
        default: g.N = 0; g.K = 0; g.w0 = nullptr; break;  // PH_ATT streams no weights
    }
    return g;
}

// The CTA's tiles of one phase, in the order both the producer and the consumers walk them: chunks of up
// to R whole rows; per chunk one tile per matrix (gate rows, then the same rows of up).
struct TileIter {
    long r, r0, r1;
    int nmat, R, rowbytes, mat;
    __device__ TileIter(const Phase &g, int esz, int stage_bytes, int cta, int nctas, bool skip_tiles = false) {
        rowbytes = g.K * esz;
        nmat = g.nmat;
        r0 = r = (long)g.N * cta / nctas;
        r1 = (long)g.N * (cta + 1) / nctas;
        R = max(1, min(kMaxRowsPerTile, stage_bytes / max(rowbytes, 1)));
        mat = 0;
        if (skip_tiles) r = r1;  // debug: keep the row range, stream nothing
    }
    __device__ bool valid() const { return r < r1; }
    __device__ int rows() const { return (int)min((long)R, r1 - r); }
    __device__ void advance() {
        if (++mat == nmat) {
            mat = 0;
            r += R;
        }
    }
};

// ---- producer ----------------------------------------------------------------------------------------
// Walks the CTA's weight tiles of the whole token in execution order.
struct TileWalker {
    int ph, nphases, esz, stage_bytes, cta, nctas;
    Phase g;
    TileIter ti;
    __device__ TileWalker(const MegaParams &p, int esz_, int stage_bytes_, int cta_, int nctas_)
        : ph(-1), nphases(5 * p.L + 1), esz(esz_), stage_bytes(stage_bytes_), cta(cta_), nctas(nctas_),
          g(get_phase(p, 0)), ti(g, esz_, stage_bytes_, cta_, nctas_) {
        ti.r = ti.r1;  // forces the first call of next() to open phase 0
    }
    // Moves to the next tile; false when the token's schedule is exhausted.
    __device__ bool next(const MegaParams &p, bool first_call) {
        if (!first_call && ti.valid()) ti.advance();
        while (!ti.valid()) {
            if (++ph >= nphases) return false;
            g = get_phase(p, ph);
            if (g.kind == PH_ATT) continue;
            ti = TileIter(g, esz, stage_bytes, cta, nctas, (p.debug_flags & 1) != 0);
        }
        return true;
    }
    __device__ const char *src() const { return (ti.mat == 0 ? g.w0 : g.w1) + (size_t)ti.r * ti.rowbytes; }
    __device__ uint32_t bytes() const { return (uint32_t)ti.rows() * (uint32_t)ti.rowbytes; }
};

__device__ __forceinline__ void prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// One elected thread.  Two cursors run over the same schedule: `ld` feeds the shared-memory ring and
// blocks when the ring is full; `pf` runs `p.l2_ahead` tiles in front of it and only asks the L2 to fetch
// the tile (cp.async.bulk.prefetch.L2).  While the consumers sit in barriers or in the attention phase the
// ring fills up within a few microseconds, but HBM keeps streaming the prefetched tiles into the 126 MB
// L2, and the ring later refills from L2 faster than HBM could deliver.
__device__ __forceinline__ void producer_loop(const MegaParams &p, Shared &sh, int cta, int nctas, int esz) {
    const uint64_t pol = make_evict_first_policy();
    const int nphases = 5 * p.L + 1;
    int s = 0;          // stage of the next tile
    uint32_t use = 0;   // how many times the ring has wrapped
    long issued = 0, prefetched = 0;
    bool ok = true;
    TileWalker ld(p, esz, sh.stage_bytes, cta, nctas), pf(p, esz, sh.stage_bytes, cta, nctas);
    bool pf_more = pf.next(p, true);
    int last_ph = -1;
    for (bool more = ld.next(p, true); more; more = ld.next(p, false)) {
        // keep the L2 cursor ahead (the tiles the ring itself holds need no L2 copy)
        while (pf_more && prefetched < issued + sh.S + p.l2_ahead) {
            if (prefetched >= issued + sh.S) prefetch_l2(pf.src(), pf.bytes());
            ++prefetched;
            pf_more = pf.next(p, false);
        }
        if (ld.ph != last_ph) {
            if (p.trace && cta == 0) p.trace[3 * nphases + 1 + ld.ph] = globaltimer_ns();
            last_ph = ld.ph;
        }
        if (use > 0 && !mbar_wait(p, sh, &sh.empty[s], (use - 1) & 1, 100 + ld.g.kind)) {
            ok = false;
            break;
        }
        const uint32_t bytes = ld.bytes();
        mbar_expect_tx(&sh.full[s], bytes);
        bulk_load(sh.stages + (size_t)s * sh.stage_bytes, ld.src(), bytes, &sh.full[s], pol);
        if (p.trace && cta == 0 && issued < kTileTrace) p.trace[4 * nphases + 1 + issued] = globaltimer_ns();
        ++issued;
        if (++s == sh.S) {
            s = 0;
            ++use;
        }
    }
    if (!ok) {
        // Wait (bounded) for the copies still in flight before the CTA may exit: the last min(issued, S) tiles.
        const long n = issued < sh.S ? issued : sh.S;
        for (long i = 0; i < n; ++i) {
            const long idx = issued - 1 - i;
            uint64_t *bar = &sh.full[idx % sh.S];
            const uint32_t parity = (uint32_t)((idx / sh.S) & 1);
            const long long t0 = clock64();
            while (!mbar_try_wait(bar, parity) && clock64() - t0 < kWaitCycles) {}
        }
    }
}

// ---- consumers ---------------------------------------------------------------------------------------
// Tagged exchange words.  An aligned 8-byte store is single-copy atomic, so a reader that sees the tag
// also sees the value; 16-byte loads fetch two such words (each half is checked on its own).
__device__ __forceinline__ void st_tagged(uint2 *dst, float v, uint32_t tag) {
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2(const uint4 *src) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src)
                 : "memory");
    return v;
}
__device__ __forceinline__ uint32_t phase_tag(const MegaParams &p, int ph) { return p.epoch_base + (uint32_t)ph + 1u; }

// Bookkeeping shared by every bounded poll loop: true = keep polling.
__device__ __forceinline__ bool poll_continue(const MegaParams &p, volatile int *abort, int &spins, long long t0, int site,
                                              int value) {
    if ((++spins & 7) != 0) return true;
    if (*abort) return false;
    if (ld_volatile_int(p.abort_flag)) {
        *abort = 1;
        return false;
    }
    if (clock64() - t0 > kWaitCycles) {
        raise_abort(p, abort, site, value);
        return false;
    }
    return true;
}

// All consumer threads: wait until the `n` tagged words at `src` (n even) carry `tag`, and leave their
// values as floats in shared memory `xs[n]`.  Returns false (uniformly) when the CTA is aborting.
__device__ __forceinline__ bool poll_vector(const MegaParams &p, Shared &sh, const uint2 *src, int n, uint32_t tag, float *xs,
                                            int tid, int &bk, int site) {
    constexpr int kBatch = 4;  // 16-byte loads in flight per thread and pass
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
    const int npairs = n / 2;
    for (int base = 0; base < npairs; base += kConsumers * kBatch) {
        uint4 v[kBatch];
        const long long t0 = clock64();
        int spins = 0;
        bool done = false, alive = true;
        while (!done && alive) {
            done = true;
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int idx = base + tid + kConsumers * u;
                v[u] = idx < npairs ? ld_tagged2(s4 + idx) : make_uint4(0u, tag, 0u, tag);
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) done = done && v[u].y == tag && v[u].w == tag;
            if (!done) alive = poll_continue(p, sh.abort, spins, t0, site, base);
        }
        if (done) {
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int idx = base + tid + kConsumers * u;
                if (idx < npairs) *reinterpret_cast<float2 *>(xs + 2 * idx) = make_float2(__uint_as_float(v[u].x), __uint_as_float(v[u].z));
            }
        }
    }
    return consumer_bar_ok(sh.abort, sh.decision, tid, bk);
}

template <typename WT>
struct VecTraits;
template <>
struct VecTraits<float> {
    static constexpr int XPV = 4;  // x elements per 16-byte weight vector
    static constexpr int XQ = 1;   // float4 registers of x per weight vector
    __device__ static __forceinline__ float dot(const uint4 &w, const float4 *x, float a) {
        a = fmaf(__uint_as_float(w.x), x[0].x, a);
        a = fmaf(__uint_as_float(w.y), x[0].y, a);
        a = fmaf(__uint_as_float(w.z), x[0].z, a);
        a = fmaf(__uint_as_float(w.w), x[0].w, a);
        return a;
    }
};
template <>
struct VecTraits<__nv_bfloat16> {
    static constexpr int XPV = 8;
    static constexpr int XQ = 2;
    __device__ static __forceinline__ float dot(const uint4 &w, const float4 *x, float a) {
        a = fmaf(bf16_lo(w.x), x[0].x, a);
        a = fmaf(bf16_hi(w.x), x[0].y, a);
        a = fmaf(bf16_lo(w.y), x[0].z, a);
        a = fmaf(bf16_hi(w.y), x[0].w, a);
        a = fmaf(bf16_lo(w.z), x[1].x, a);
        a = fmaf(bf16_hi(w.z), x[1].y, a);
        a = fmaf(bf16_lo(w.w), x[1].z, a);
        a = fmaf(bf16_hi(w.w), x[1].w, a);
        return a;
    }
};

__device__ __forceinline__ float embed_elem(const MegaParams &p, long id, int k) {
    if (p.wbf16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.embed)[id * p.H + k]);
    return __ldg(reinterpret_cast<const float *>(p.embed) + id * p.H + k);
}

// Stage / parity bookkeeping of the consumer side of the ring.
struct RingPos {
    int s;
    uint32_t use;
    __device__ void next(int S) {
        if (++s == S) {
            s = 0;
            ++use;
        }
    }
};

// o_proj prologue: wait for the partial results of every attention work item and merge the splits,
// out = ctx * (1/(l + 1e-9)) (self_attention.rs:287-290), into shared memory xs[qd].
__device__ __forceinline__ bool poll_attention(const MegaParams &p, Shared &sh, uint32_t tag, float *xs, int tid, int &bk) {
    const int nv4 = p.qd / 4;
    const int rec_words = 2 + p.D;  // uint2 words per (head, split) record
    for (int v = tid; v < nv4; v += kConsumers) {
        const int k0 = v * 4, h = k0 / p.D, e0 = k0 % p.D;
        uint4 ml[kMaxSplit], c01[kMaxSplit], c23[kMaxSplit];
        const long long t0 = clock64();
        int spins = 0;
        bool done = false, alive = true;
        while (!done && alive) {
            done = true;
#pragma unroll
            for (int s = 0; s < kMaxSplit; ++s) {
                const bool oks = s < p.nsplit;
                const uint4 *rec = reinterpret_cast<const uint4 *>(p.partT + ((size_t)h * p.nsplit + (oks ? s : 0)) * rec_words);
                const uint4 ok_word = make_uint4(0xff800000u, tag, 0u, tag);  // {max = -inf, sum = 0}
                ml[s] = oks ? ld_tagged2(rec) : ok_word;
                c01[s] = oks ? ld_tagged2(rec + 1 + e0 / 2) : make_uint4(0u, tag, 0u, tag);
                c23[s] = oks ? ld_tagged2(rec + 2 + e0 / 2) : make_uint4(0u, tag, 0u, tag);
            }
#pragma unroll
            for (int s = 0; s < kMaxSplit; ++s)
                done = done && ml[s].y == tag && ml[s].w == tag && c01[s].y == tag && c01[s].w == tag && c23[s].y == tag &&
                       c23[s].w == tag;
            if (!done) alive = poll_continue(p, sh.abort, spins, t0, 320, v);
        }
        if (done) {
            float M = -INFINITY;
#pragma unroll
            for (int s = 0; s < kMaxSplit; ++s) M = fmaxf(M, __uint_as_float(ml[s].x));
            float L = 0.f;
            float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < kMaxSplit; ++s) {
                const float ms = __uint_as_float(ml[s].x);
                if (ms != -INFINITY) {
                    const float f = expf(ms - M);
                    L = fmaf(__uint_as_float(ml[s].z), f, L);
                    c.x = fmaf(__uint_as_float(c01[s].x), f, c.x);
                    c.y = fmaf(__uint_as_float(c01[s].z), f, c.y);
                    c.z = fmaf(__uint_as_float(c23[s].x), f, c.z);
                    c.w = fmaf(__uint_as_float(c23[s].z), f, c.w);
                }
            }
            const float inv = __fdiv_rn(1.0f, __fadd_rn(L, 1e-9f));
            reinterpret_cast<float4 *>(xs)[v] =
                make_float4(__fmul_rn(c.x, inv), __fmul_rn(c.y, inv), __fmul_rn(c.z, inv), __fmul_rn(c.w, inv));
        }
    }
    return consumer_bar_ok(sh.abort, sh.decision, tid, bk);
}

// One vector-matrix phase for the consumer threads.
//   NXV = 16-byte weight vectors per thread per row, G = warp groups (each owns every G-th tile).
//   xres = the residual-stream value of the row this thread finishes in the o_proj / down phases (the row
//   split of those two phases is the same, so the value never leaves the thread).
template <typename WT, int NXV, int G>
__device__ __forceinline__ bool gemv_phase(const MegaParams &p, Shared &sh, const Phase &g, long id, RingPos &rp, int cta, int nctas,
                                           int tid, int &bk, int ph, float &xres) {
    constexpr int XPV = VecTraits<WT>::XPV;
    constexpr int XQ = VecTraits<WT>::XQ;
    constexpr int T = kConsumers / G;       // threads per group
    constexpr int WG = kConsumerWarps / G;  // warps per group
    const int lane = tid & 31, warp = tid >> 5;
    const int grp = tid / T, gtid = tid % T, gwarp = warp % WG;
    const int nvec = g.K / XPV;  // vectors per row
    const MegaLayer *lw = g.layer < p.L ? &p.layers[g.layer] : nullptr;
    TileIter ti(g, (int)sizeof(WT), sh.stage_bytes, cta, nctas, (p.debug_flags & 1) != 0);
    if (ti.r0 == ti.r1) return true;  // no rows of this matrix here: nothing to read, nothing to publish

    // ---- prologue: this thread's slice of the input vector, in registers ---------------------------------
    float4 xr[NXV * XQ];
    const float *norm_w = nullptr;
    if (g.kind == PH_QKV) norm_w = lw->norm1;
    else if (g.kind == PH_GATEUP) norm_w = lw->norm2;
    else if (g.kind == PH_LMHEAD) norm_w = p.final_norm;
    // RMSNorm gains are fetched first so that they share the wait for x.  (When x alone already takes 64
    // registers they are fetched after the reduction instead.)
    constexpr bool kEarlyGains = NXV * XQ <= 8;
    float4 nw[NXV * XQ];
    const float4 *n4 = reinterpret_cast<const float4 *>(norm_w);
    if (norm_w && kEarlyGains) {
#pragma unroll
        for (int j = 0; j < NXV; ++j) {
            const int v = gtid + T * j;
#pragma unroll
            for (int q = 0; q < XQ; ++q)
                nw[j * XQ + q] = v < nvec ? __ldg(n4 + (size_t)v * XQ + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    float *xs = sh.part;  // the partial-sum table is idle during the prologue: stage the input vector there
    if (g.kind == PH_QKV && g.layer == 0) {
        // Embedding::forward (embedding.rs:47-57): the token's row is the first layer's input
#pragma unroll
        for (int j = 0; j < NXV; ++j) {
            const int v = gtid + T * j;
#pragma unroll
            for (int q = 0; q < XQ; ++q) {
                const int k = v * XPV + 4 * q;
                xr[j * XQ + q] = (v < nvec) ? make_float4(embed_elem(p, id, k), embed_elem(p, id, k + 1),
                                                          embed_elem(p, id, k + 2), embed_elem(p, id, k + 3))
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    } else {
        const uint32_t tag = phase_tag(p, ph - 1);  // every phase consumes what the phase before it published
        bool ok;
        if (g.kind == PH_O) ok = poll_attention(p, sh, tag, xs, tid, bk);
        else ok = poll_vector(p, sh, g.kind == PH_DOWN ? p.actT : p.xT, g.K, tag, xs, tid, bk, 330 + g.kind);
        if (!ok) return false;
        if (p.trace && cta == 0 && tid == 0) p.trace[4 * (5 * p.L + 1) + 1 + kTileTrace + ph] = globaltimer_ns();
#pragma unroll
        for (int j = 0; j < NXV; ++j) {
            const int v = gtid + T * j;
#pragma unroll
            for (int q = 0; q < XQ; ++q)
                xr[j * XQ + q] = (v < nvec) ? reinterpret_cast<const float4 *>(xs)[(size_t)v * XQ + q]
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (norm_w) {
        // RMSNorm::forward (rms_norm.rs:49-56): rms = sqrt(ss/dim + eps); x = (x * (1/rms)) * w
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NXV * XQ; ++i) {
            ss = fmaf(xr[i].x, xr[i].x, ss);
            ss = fmaf(xr[i].y, xr[i].y, ss);
            ss = fmaf(xr[i].z, xr[i].z, ss);
            ss = fmaf(xr[i].w, xr[i].w, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) sh.red[warp] = ss;
        consumer_bar();  // also: everybody has copied its slice out of xs before partial sums land there
        float tot = 0.f;  // every group holds the whole vector: sum the warps of this thread's group
#pragma unroll
        for (int w = 0; w < WG; ++w) tot += sh.red[grp * WG + w];
        const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)g.K), p.eps)));
        if (!kEarlyGains) {
#pragma unroll
            for (int j = 0; j < NXV; ++j) {
                const int v = gtid + T * j;
#pragma unroll
                for (int q = 0; q < XQ; ++q)
                    nw[j * XQ + q] = v < nvec ? __ldg(n4 + (size_t)v * XQ + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int i = 0; i < NXV * XQ; ++i) {
            xr[i].x = __fmul_rn(__fmul_rn(xr[i].x, inv), nw[i].x);
            xr[i].y = __fmul_rn(__fmul_rn(xr[i].y, inv), nw[i].y);
            xr[i].z = __fmul_rn(__fmul_rn(xr[i].z, inv), nw[i].z);
            xr[i].w = __fmul_rn(__fmul_rn(xr[i].w, inv), nw[i].w);
        }
    } else {
        consumer_bar();  // everybody has copied its slice out of xs before partial sums land there
    }
    trace_stamp(p, cta, tid, 3 * ph + 1);
    // ---- tiles ---------------------------------------------------------------------------------------
    // Branch-free inner loop: vector indices are clamped into the row (x is zero there, so the extra
    // products vanish) and rows are taken in static blocks of RB with the row index clamped to the last
    // valid row, so every block issues its 128-bit shared loads back to back and the RB shuffle
    // reductions interleave.  Guarded, fully unrolled row/vector slots would serialise into one
    // load -> FMA chain per slot.
    const int vlast = nvec - 1;
    const int rows_per_block = ti.R * (kRowBlock / ti.R);  // a block never splits a tile
    long blk0 = ti.r0;                                     // first row of the current block
    int tile = 0;
    for (; ti.valid(); ti.advance(), ++tile) {
        const int nr = ti.rows();
        if (tile % G == grp) {
            // A parity test tells two phases apart, not three: before testing for use `u` of this stage,
            // use `u-1` (owned by another group) must be known to have landed.  Its owner publishes that.
            // A failed wait must not leave early (see consumer_bar_ok): skip the math, keep the sequence.
            bool have = (G == 1) || stage_use_seen(p, sh, rp.s, (int)rp.use, 310 + g.kind);
            have = have && mbar_wait(p, sh, &sh.full[rp.s], rp.use & 1, 300 + g.kind);
            if (have && lane == 0) sh.seen[rp.s] = (int)rp.use + 1;  // also when G == 1: a later phase may need it
            const uint4 *st = reinterpret_cast<const uint4 *>(sh.stages + (size_t)rp.s * sh.stage_bytes);
            float *part = sh.part + ((size_t)ti.mat * kRowBlock + (size_t)(ti.r - blk0)) * kConsumerWarps + gwarp;
            if (ti.R >= 4) {
                for (int rb = 0; rb < nr; rb += 4) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint4 *rp0 = st + (size_t)min(rb + 0, nr - 1) * nvec, *rp1 = st + (size_t)min(rb + 1, nr - 1) * nvec;
                    const uint4 *rp2 = st + (size_t)min(rb + 2, nr - 1) * nvec, *rp3 = st + (size_t)min(rb + 3, nr - 1) * nvec;
                    if (have) {
                        // The empty asm every fourth vector keeps the compiler from hoisting every load of
                        // the tile to the top, which would need more registers than exist.
#pragma unroll
                        for (int j = 0; j < NXV; ++j) {
                            const int v = min(gtid + T * j, vlast);
                            const uint4 w0 = rp0[v], w1 = rp1[v], w2 = rp2[v], w3 = rp3[v];
                            acc[0] = VecTraits<WT>::dot(w0, &xr[j * XQ], acc[0]);
                            acc[1] = VecTraits<WT>::dot(w1, &xr[j * XQ], acc[1]);
                            acc[2] = VecTraits<WT>::dot(w2, &xr[j * XQ], acc[2]);
                            acc[3] = VecTraits<WT>::dot(w3, &xr[j * XQ], acc[3]);
                            if ((j & 3) == 3) asm volatile("" ::: "memory");
                        }
                    }
                    if (rb + 4 >= nr) {  // last block of the tile: the stage can go back to the producer
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cnt(&sh.empty[rp.s], G);  // the G-th share of the 4 arrivals
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float v = warp_sum(acc[i]);
                        if (lane == 0 && rb + i < nr) part[(rb + i) * kConsumerWarps] = v;
                    }
                }
            } else if (ti.R >= 2) {
                for (int rb = 0; rb < nr; rb += 2) {
                    float acc[2] = {0.f, 0.f};
                    const uint4 *rp0 = st + (size_t)rb * nvec, *rp1 = st + (size_t)min(rb + 1, nr - 1) * nvec;
                    if (have) {
#pragma unroll
                        for (int j = 0; j < NXV; ++j) {
                            const int v = min(gtid + T * j, vlast);
                            const uint4 w0 = rp0[v], w1 = rp1[v];
                            acc[0] = VecTraits<WT>::dot(w0, &xr[j * XQ], acc[0]);
                            acc[1] = VecTraits<WT>::dot(w1, &xr[j * XQ], acc[1]);
                            if ((j & 7) == 7) asm volatile("" ::: "memory");
                        }
                    }
                    if (rb + 2 >= nr) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cnt(&sh.empty[rp.s], G);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float v = warp_sum(acc[i]);
                        if (lane == 0 && rb + i < nr) part[(rb + i) * kConsumerWarps] = v;
                    }
                }
            } else {
                // One row per tile (long rows): two accumulators keep the FMA chains short.
                float a0 = 0.f, a1 = 0.f;
                if (have) {
#pragma unroll
                    for (int j = 0; j < NXV; j += 2) {
                        const uint4 w0 = st[min(gtid + T * j, vlast)];
                        const uint4 w1 = st[min(gtid + T * (j + 1), vlast)];
                        a0 = VecTraits<WT>::dot(w0, &xr[j * XQ], a0);
                        a1 = VecTraits<WT>::dot(w1, &xr[(j + 1) * XQ], a1);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive_cnt(&sh.empty[rp.s], G);
                const float v = warp_sum(a0 + a1);
                if (lane == 0) part[0] = v;
            }
        }
        rp.next(sh.S);
        // End of a row block (or of the phase): reduce the per-warp partials, run the epilogue and publish.
        const bool last_of_chunk = ti.mat == ti.nmat - 1;
        const long next_r = ti.r + ti.R;
        if (last_of_chunk && (next_r >= ti.r1 || next_r - blk0 >= rows_per_block)) {
            const int nrows = (int)(min(next_r, ti.r1) - blk0);
            if (!consumer_bar_ok(sh.abort, sh.decision, tid, bk)) return false;
            if (tid < nrows) {
                const float *p0 = sh.part + (size_t)tid * kConsumerWarps;
                float tot = 0.f, tot1 = 0.f;
#pragma unroll
                for (int w = 0; w < WG; ++w) tot += p0[w];
                if (g.nmat == 2) {
#pragma unroll
                    for (int w = 0; w < WG; ++w) tot1 += p0[(size_t)kRowBlock * kConsumerWarps + w];
                }
                const long row = blk0 + tid;
                const uint32_t tag = phase_tag(p, ph);
                switch (g.kind) {
                    case PH_QKV: st_tagged(p.qkvT + row, tot, tag); break;
                    case PH_O:      // h = x + attn_out                                   llama.rs:110
                    case PH_DOWN:   // out = h + mlp_out                                  llama.rs:115
                        xres = __fadd_rn(xres, tot);  // (these phases have a single row block: see the launcher)
                        st_tagged(p.xT + row, xres, tag);
                        break;
                    case PH_GATEUP: {  // SiLU (activation.rs:143-146) then gate_act * up (llama.rs:61-63)
                        const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-tot)));
                        st_tagged(p.actT + row, __fmul_rn(__fmul_rn(tot, sig), tot1), tag);
                        break;
                    }
                    default: p.logits[row] = tot; break;
                }
            }
            blk0 = next_r;
            if (next_r < ti.r1) consumer_bar();  // the table is rewritten by the next block
        }
    }
    if ((p.debug_flags & 1) && ti.r0 + tid < ti.r1) {  // debug (no tiles streamed): publish zeros so that the chain runs
        const uint32_t tag = phase_tag(p, ph);
        uint2 *dst = g.kind == PH_QKV ? p.qkvT : g.kind == PH_GATEUP ? p.actT : p.xT;
        if (g.kind != PH_LMHEAD) st_tagged(dst + ti.r0 + tid, 0.f, tag);
    }
    trace_stamp(p, cta, tid, 3 * ph + 2);
    return true;
}

template <typename WT, int G>
__device__ __forceinline__ bool gemv_phase_nxv(const MegaParams &p, Shared &sh, const Phase &g, long id, RingPos &rp, int cta,
                                               int nctas, int tid, int &bk, int ph, float &xres, int need) {
    if (need <= 4) return gemv_phase<WT, 4, G>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres);
    if (need <= 8) return gemv_phase<WT, 8, G>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres);
    if constexpr (VecTraits<WT>::XPV == 4) {
        if (need > 12) return gemv_phase<WT, 16, G>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres);
    }
    return gemv_phase<WT, 12, G>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres);  // the launcher rejects more
}

// Picks the number of warp groups: the most groups whose threads still hold their input slice in
// registers (<= 16 vectors per thread for f32 weights, <= 8 preferred for bf16 whose vectors are twice
// as wide in x).
template <typename WT>
__device__ __forceinline__ bool gemv_phase_dispatch(const MegaParams &p, Shared &sh, const Phase &g, long id, RingPos &rp, int cta,
                                                    int nctas, int tid, int &bk, int ph, float &xres) {
    constexpr int XPV = VecTraits<WT>::XPV;
    constexpr int kPrefer = XPV == 4 ? 16 : 8;
    const int nvec = g.K / XPV;
    const int need4 = (nvec + kConsumers / 4 - 1) / (kConsumers / 4);
    const int need2 = (nvec + kConsumers / 2 - 1) / (kConsumers / 2);
    const int need1 = (nvec + kConsumers - 1) / kConsumers;
    if (need4 <= kPrefer) return gemv_phase_nxv<WT, 4>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres, need4);
    if (need2 <= kPrefer) return gemv_phase_nxv<WT, 2>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres, need2);
    return gemv_phase_nxv<WT, 1>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres, need1);
}

// Sink of an attention work item in the persistent kernel: tagged record {max}, {sum}, ctx[D].
struct TaggedPartOut {
    uint2 *partT;
    int rec_words, nsplit;
    uint32_t tag;
    __device__ __forceinline__ void operator()(size_t row, int split, int e, float c, float M, float L) const {
        uint2 *rec = partT + (row * nsplit + split) * rec_words;
        st_tagged(rec + 2 + e, c, tag);
        if (e == 0) {
            st_tagged(rec, M, tag);
            st_tagged(rec + 1, L, tag);
        }
    }
};

// Waits for this step's q (head h), k and v (KV head hk) projections and copies them to shared memory
// raw[3*D]; runs inside the attention item after its first K/V row requests are in flight.
struct StageQKV {
    const MegaParams *p;  // the kernel's __grid_constant__ block: taking its address costs nothing
    volatile int *abort;  // (a pointer to the Shared struct itself would force it into local memory)
    float *raw;
    int h, hk, tid;
    uint32_t tag;
    __device__ __forceinline__ void operator()() const {
        const int D = p->D, half = D / 2;
        for (int t = tid; t < 3 * half; t += kConsumers) {
            const int which = t / half, i = t % half;
            const uint2 *src = which == 0 ? p->qkvT + (size_t)h * D
                                          : p->qkvT + p->qd + (which == 2 ? p->kvd : 0) + (size_t)hk * D;
            const uint4 *s4 = reinterpret_cast<const uint4 *>(src) + i;
            const long long t0 = clock64();
            int spins = 0;
            uint4 v = ld_tagged2(s4);
            while ((v.y != tag || v.w != tag) && poll_continue(*p, abort, spins, t0, 340, t)) v = ld_tagged2(s4);
            *reinterpret_cast<float2 *>(raw + which * D + 2 * i) = make_float2(__uint_as_float(v.x), __uint_as_float(v.z));
        }
        consumer_bar();
    }
};

// Receives plain values only: a reference to the kernel's Shared struct inside the functors below would
// push that struct into local memory.
__device__ __forceinline__ void attention_items(const MegaParams &p, float *attn_smem, volatile int *abort, int layer, int ph, int past,
                                             int cta, int nctas, int tid) {
    const int items = p.Hq * p.nsplit;
    const MegaLayer &l = p.layers[layer];
    float *raw = attn_smem + attn_decode_smem_floats(1, p.D, kConsumerWarps);
    DecodeParams dp;
    dp.q = raw; dp.k_new = raw + p.D; dp.v_new = raw + 2 * p.D;
    dp.q_stride = 0; dp.kv_stride = 0;
    dp.k_cache = l.k_cache; dp.v_cache = l.v_cache; dp.d_len = l.d_len;
    dp.Hq = p.Hq; dp.Hkv = p.Hkv; dp.D = p.D; dp.max_seq = p.max_seq;
    dp.cos_t = p.cos_t; dp.sin_t = p.sin_t; dp.q_norm = l.qn; dp.k_norm = l.kn;
    dp.norm_eps = p.eps; dp.scale = p.scale;
    dp.part_m = nullptr; dp.part_l = nullptr; dp.part_ctx = nullptr;
    dp.nsplit = p.nsplit;
    const TaggedPartOut out{p.partT, 2 + p.D, p.nsplit, phase_tag(p, ph)};
    for (int item = cta; item < items; item += nctas) {
        const int h = item / p.nsplit, split = item % p.nsplit;
        const StageQKV stage{&p, abort, raw, h, h / (p.Hq / p.Hkv), tid, phase_tag(p, ph - 1)};
        // two lane layouts cover head_dim <= 128 (the launcher rejects larger heads)
        if (p.D <= 64) attn_decode_item<1, 2, true, kConsumerWarps>(dp, attn_smem, 0, h, split, tid, past, ConsumerBar(), out, stage);
        else attn_decode_item<1, 4, true, kConsumerWarps>(dp, attn_smem, 0, h, split, tid, past, ConsumerBar(), out, stage);
    }
}

__device__ __forceinline__ bool attention_phase(const MegaParams &p, Shared &sh, int layer, int ph, int past, int cta, int nctas,
                                                int tid, int &bk) {
    if (cta >= p.Hq * p.nsplit) return true;  // no work item here: nothing to wait for
    attention_items(p, sh.attn, sh.abort, layer, ph, past, cta, nctas, tid);
    return consumer_bar_ok(sh.abort, sh.decision, tid, bk);
}

template <typename WT>
__device__ __forceinline__ void consumer_loop(const MegaParams &p, Shared &sh, int cta, int nctas, int tid) {
    // Token id: f32 -> usize with Rust's saturating cast (embedding.rs:50); id >= vocab is the reference's
    // panic: record it and run nothing (every CTA takes the same branch).
    const float f = __ldcg(p.ids);
    const int past = __ldcg(p.layers[0].d_len);  // context length before this token, the same for every layer
    const unsigned long long uid = (f != f || f <= 0.f) ? 0ull : (f >= 1.8e19f ? ~0ull : (unsigned long long)f);
    if (uid >= (unsigned long long)p.vocab) {
        if (cta == 0 && tid == 0 && atomicCAS(&p.status->code, 0, LUMEN_ERR_EMBED_RANGE) == 0) {
            p.status->detail0 = 0;
            p.status->detail1 = (int)min(uid, (unsigned long long)0x7fffffff);
        }
        if (tid == 0) *sh.abort = 1;  // releases the producer
        return;
    }
    const long id = (long)uid;
    // The residual stream starts as the embedding row.  The rows of the hidden vector this CTA finishes in
    // the o_proj and down phases are the same, so each value stays in the register of the thread that
    // owns its row for the whole token.
    float xres = 0.f;
    {
        const long r0 = (long)p.H * cta / nctas, r1 = (long)p.H * (cta + 1) / nctas;
        if (r0 + tid < r1) xres = embed_elem(p, id, (int)(r0 + tid));
    }
    const int nphases = 5 * p.L + 1;
    RingPos rp{0, 0};
    int bk = 0;
    for (int ph = 0; ph < nphases; ++ph) {
        const Phase g = get_phase(p, ph);
        trace_stamp(p, cta, tid, 3 * ph);
        if (g.kind == PH_ATT) {
            if (!attention_phase(p, sh, g.layer, ph, past, cta, nctas, tid, bk)) return;
            trace_stamp(p, cta, tid, 3 * ph + 1);
            trace_stamp(p, cta, tid, 3 * ph + 2);
        } else {
            if (!gemv_phase_dispatch<WT>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres)) return;
        }
    }
    trace_stamp(p, cta, tid, 3 * nphases);
    // c.len = new_len (self_attention.rs:179) for every layer's cache.  Every CTA read `past` before it did
    // anything else, and the next launch starts only after this one has ended.
    for (int l = tid; cta == 0 && l < p.L; l += kConsumers) *p.layers[l].d_len = past + 1;
}

// The parameter block is __grid_constant__ so that helpers can take it by reference without the compiler
// materialising a per-thread copy in local memory: with ~200 KB of shared memory in use the L1 is tiny,
// and every stack access would become an L2 round trip on the critical path.
// One kernel per weight type: the bf16 variants hold twice as many activation registers per weight
// vector, and fusing both into one kernel makes the f32 path spill.
template <typename WT>
__global__ void __launch_bounds__(kThreads, 1) decode_mega_kernel(const __grid_constant__ MegaParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ uint64_t bars[2 * kMegaMaxStages];
    __shared__ int abort_flag;
    __shared__ int decision[2];
    __shared__ int seen[kMegaMaxStages];
    Shared sh;
    sh.S = p.stages;
    sh.stage_bytes = p.stage_bytes;
    sh.stages = smem_raw;
    float *fl = reinterpret_cast<float *>(smem_raw + (size_t)p.stages * p.stage_bytes);
    sh.part = fl;
    sh.red = sh.part + mega_table_floats(max(p.H, max(p.qd, p.I)));
    sh.attn = sh.red + kConsumerWarps;
    sh.full = bars;
    sh.empty = bars + kMegaMaxStages;
    sh.abort = &abort_flag;
    sh.decision = decision;
    sh.seen = seen;
    const int tid = threadIdx.x;
    if (tid == 0) {
        abort_flag = 0;
        decision[0] = decision[1] = 0;
        for (int s = 0; s < kMegaMaxStages; ++s) seen[s] = 0;
        for (int s = 0; s < sh.S; ++s) {
            mbar_init(&sh.full[s], 1);                 // the producer's arrive.expect_tx
            mbar_init(&sh.empty[s], kConsumerWarps);   // 4 arrivals: the owning group's warps, G each
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int cta = blockIdx.x, nctas = gridDim.x;
    if (tid >= kConsumers) {
        if (tid == kConsumers) producer_loop(p, sh, cta, nctas, (int)sizeof(WT));
    } else {
        consumer_loop<WT>(p, sh, cta, nctas, tid);
    }
}

}  // namespace

size_t decode_mega_smem_bytes(int stages, int stage_bytes, int head_dim, int kmax) {
    return (size_t)stages * stage_bytes +
           (mega_table_floats(kmax) + kConsumerWarps + attn_decode_smem_floats(1, head_dim, kConsumerWarps) + 3 * (size_t)head_dim) * sizeof(float);
}

int decode_mega_max_splits() { return kMaxSplit; }
unsigned int decode_mega_epochs_per_launch(int layers) { return 5u * (unsigned)layers + 2u; }

size_t decode_mega_exchange_words(const MegaParams &p) {
    return (size_t)p.H + p.qkv_rows + p.I + (size_t)p.Hq * kMaxSplit * (2 + p.D) + 8;
}

int decode_mega_supported(const MegaParams &p, char *why, size_t why_len) {
    const int esz = p.wbf16 ? 2 : 4;
    const int ks[3] = {p.H, p.qd, p.I};
    for (int k : ks) {
        if ((k * esz) % 16) {
            snprintf(why, why_len, "row of %d elements is not a multiple of 16 bytes", k);
            return 0;
        }
        const int nvec = k * esz / 16;
        if ((nvec + kConsumers - 1) / kConsumers > (p.wbf16 ? 12 : 16)) {
            snprintf(why, why_len, "K=%d too large for the register-resident input slice", k);
            return 0;
        }
    }
    if (p.D > 128 || (p.D % 4)) {
        snprintf(why, why_len, "head_dim %d is not a multiple of 4 up to 128", p.D);
        return 0;
    }
    if (p.qkv_rows % 2 || p.qd % 4 || p.kvd % 2) {
        snprintf(why, why_len, "projection widths must be even");
        return 0;
    }
    return 1;
}

int launch_decode_mega(lumen_ctx *ctx, MegaParams &p, cudaStream_t s) {
    // All CTAs must be resident at once (they wait for each other's results): one per SM, cooperative launch.
    const int grid = ctx->num_sms;
    if ((p.H + grid - 1) / grid + 1 > kRowBlock)
        return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "hidden size %d needs more than %d rows per CTA", p.H, kRowBlock);
    // Ring geometry: 32 KB stages (a row of every supported matrix fits), as many as fit beside the
    // scratch areas in the 227 KB a CTA may use.
    p.stage_bytes = 32 * 1024;
    const int kmax = std::max(p.H, std::max(p.qd, p.I));
    const size_t budget = 227 * 1024 - 1024;  // static shared (barriers, flags) and alignment slack
    int stages = kMegaMaxStages;
    while (stages > 2 && decode_mega_smem_bytes(stages, p.stage_bytes, p.D, kmax) > budget) --stages;
    p.stages = stages;
    // L2 look-ahead of the producer, in tiles per CTA (6 x 32 KB x 148 CTAs = 28 MB of the 126 MB L2).
    p.l2_ahead = 6;
    p.debug_flags = 0;
    if (const char *e = getenv("LUMEN_MEGA_DEBUG")) p.debug_flags = atoi(e);
    if (const char *e = getenv("LUMEN_MEGA_L2_AHEAD")) p.l2_ahead = std::max(0, std::min(64, atoi(e)));
    const size_t smem = decode_mega_smem_bytes(stages, p.stage_bytes, p.D, kmax);
    if (smem > budget) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "shared memory: %zu bytes needed", smem);
    const void *kern = p.wbf16 ? (const void *)decode_mega_kernel<__nv_bfloat16> : (const void *)decode_mega_kernel<float>;
    static bool attr_set[2] = {false, false};
    if (!attr_set[p.wbf16 ? 1 : 0]) {  // once, for the largest ring any shape can ask for
        LUMEN_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
        attr_set[p.wbf16 ? 1 : 0] = true;
    }
    void *args[] = {&p};
    LUMEN_CUDA(ctx, cudaLaunchCooperativeKernel(kern, dim3(grid), dim3(kThreads), args, smem, s));
    ctx->launches += 1;
    return LUMEN_OK;
}

}  // namespace lumen
