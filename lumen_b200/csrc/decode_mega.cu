// Whole-token persistent decode kernel (batch 1): one launch runs LlamaModel::forward for one new
// token (src/models/llama.rs:181-206 of the reference; layer body :104-116, MLP :59-65, decode
// attention self_attention.rs:141-297, vector-matrix products src/ops/matmul.rs:42-69).
//
// Design for B200: one CTA per SM (launched cooperatively so that all CTAs are co-resident).  The
// last warp of each CTA is a producer: it walks a schedule of bulk copies that the host built once (the
// CTA's rows of every matrix of every layer, in execution order) and streams the weight tiles from HBM
// into a shared-memory ring with 1-D bulk TMA copies (cp.async.bulk + mbarrier transaction counts, L2
// evict-first, a short cp.async.bulk.prefetch.L2 look-ahead).  The schedule does not depend on the
// activations, so the producer keeps HBM busy across phase boundaries while the consumer warps wait for
// activations or run the (weight-free) attention.
//
// Consumers: a phase's input vector is staged in shared memory (RMSNorm applied in place), tiles go
// round-robin to the 4 consumer warps, and a warp works through its own tiles alone: per 16-byte step
// a lane reads one vector of x and the matching vector of up to 4 weight rows with conflict-free 128-bit
// shared loads, the row sums are folded across lanes by one butterfly, and the only CTA-wide barrier is
// at the end of a row block, where the fused epilogue runs (residual add, SiLU*mul) and the results are
// published.  Phases of a layer: qkv | attention | o_proj(+residual) | gate/up(+SiLU*mul) |
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
constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s at 1.9 GHz

// Floats of the staged input vector of a phase (up to kmax elements, zero-padded to four whole steps of a
// warp through a row: 4 x 32 lanes x 8 elements) and of the table of row sums of a row block ([2][kRowBlock][4]).
__host__ __device__ inline size_t mega_xs_floats(int kmax) { return (((size_t)kmax + 1023) / 1024) * 1024; }
__host__ __device__ inline size_t mega_table_floats(int kmax) {
    return mega_xs_floats(kmax) + 2 * (size_t)kRowBlock * kConsumerWarps;
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
    float *xs;         // the phase's input vector (zero-padded)
    float *part;       // [2][kRowBlock][kConsumerWarps]: row sums of one block (first slot of each row)
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

__host__ __device__ __forceinline__ Phase get_phase(const MegaParams &p, const MegaLayer *layers, int ph) {
    Phase g;
    g.nmat = 1;
    g.w1 = nullptr;
    if (ph >= 5 * p.L) {
        g.kind = PH_LMHEAD; g.layer = p.L; g.N = p.V; g.K = p.H; g.w0 = p.lm_head;
        return g;
    }
    g.layer = ph / 5;
    g.kind = ph % 5;
    const MegaLayer &l = layers[g.layer];
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
    __host__ __device__ TileIter(const Phase &g, int esz, int stage_bytes, int cta, int nctas, bool skip_tiles = false) {
        rowbytes = g.K * esz;
        nmat = g.nmat;
        r0 = r = (long)g.N * cta / nctas;
        r1 = (long)g.N * (cta + 1) / nctas;
        R = stage_bytes / (rowbytes > 0 ? rowbytes : 1);
        R = R < 1 ? 1 : (R > kMaxRowsPerTile ? kMaxRowsPerTile : R);
        if (R > 4 && R < 8) R = 4;  // the consumers take rows four at a time
        mat = 0;
        if (skip_tiles) r = r1;  // debug: keep the row range, stream nothing
    }
    __host__ __device__ bool valid() const { return r < r1; }
    __host__ __device__ int rows() const { return (int)((long)R < r1 - r ? (long)R : r1 - r); }
    __host__ __device__ void advance() {
        if (++mat == nmat) {
            mat = 0;
            r += R;
        }
    }
};

__device__ __forceinline__ void prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// ---- producer ----------------------------------------------------------------------------------------
// The producer warp walks the CTA's precomputed schedule of bulk copies (MegaParams::sched).  All 32 lanes
// fetch a batch of 32 entries with one coalesced load (the next batch is requested before the current one
// is issued, so its latency is hidden); lane 0 then issues the copies: on the first copy of a tile it waits
// for the stage to be free and arms the stage's mbarrier with the tile's byte count.  A tile made of row
// segments is one copy per row, packed back to back in the stage.
__device__ __forceinline__ void producer_loop(const MegaParams &p, Shared &sh, int cta, int lane) {
    const uint64_t pol = make_evict_first_policy();
    const int nphases = 5 * p.L + 1;
    const uint4 *sched = p.sched + (size_t)cta * p.sched_stride;
    const int n = p.sched_count[cta];
    int s = -1;          // stage of the current tile
    uint32_t use = 0;    // how many times the ring has wrapped
    uint32_t off = 0;    // bytes of the current tile already requested
    long tiles = 0;
    int last_ph = -1;
    bool ok = true;
    uint4 nxt = lane < n ? sched[lane] : make_uint4(0u, 0u, 0u, 0u);
    for (int base = 0; base < n; base += 32) {
        const uint4 cur = nxt;
        if (base + 32 + lane < n) nxt = sched[base + 32 + lane];
        const int cnt = min(32, n - base);
        for (int i = 0; i < cnt; ++i) {
            // L2 look-ahead: the lane that holds the entry `ahead` copies further on (in this batch or the
            // next) asks the L2 to fetch it.  While the consumers wait for activations the ring fills up
            // within a few microseconds, but HBM keeps streaming into the 126 MB L2, and the ring later
            // refills from there faster than HBM could deliver.
            if (p.l2_ahead > 0) {
                const int j = i + p.l2_ahead;
                if (lane == (j & 31) && j < 64 && base + j < n) {
                    const uint4 f = j < 32 ? cur : nxt;
                    prefetch_l2(reinterpret_cast<const char *>(((unsigned long long)f.y << 32) | f.x), f.z & 0xffffu);
                }
            }
            uint4 e;
            e.x = __shfl_sync(0xffffffffu, cur.x, i);
            e.y = __shfl_sync(0xffffffffu, cur.y, i);
            e.z = __shfl_sync(0xffffffffu, cur.z, i);
            e.w = __shfl_sync(0xffffffffu, cur.w, i);
            if (lane != 0 || !ok) continue;
            if (e.w) {  // first copy of a tile: next stage
                if (++s == sh.S) {
                    s = 0;
                    ++use;
                }
                const int ph = (int)(e.z >> 16);
                if (p.trace && cta == 0 && ph != last_ph) {
                    p.trace[3 * nphases + 1 + ph] = globaltimer_ns();
                    last_ph = ph;
                }
                if (use > 0 && !mbar_wait(p, sh, &sh.empty[s], (use - 1) & 1, 100)) {
                    ok = false;
                    --s;  // this tile was not issued (s == -1 cannot occur here: use > 0)
                    continue;
                }
                mbar_expect_tx(&sh.full[s], e.w);
                off = 0;
                if (p.trace && cta == 0 && tiles < kMegaTileTrace) p.trace[7 * nphases + 1 + tiles] = globaltimer_ns();
                ++tiles;
            }
            const uint32_t bytes = e.z & 0xffffu;
            const char *src = reinterpret_cast<const char *>(((unsigned long long)e.y << 32) | e.x);
            bulk_load(sh.stages + (size_t)s * sh.stage_bytes + off, src, bytes, &sh.full[s], pol);
            off += bytes;
        }
    }
    if (lane == 0 && !ok) {
        // Wait (bounded) for the copies still in flight before the CTA may exit: the last min(tiles, S) tiles.
        const long m = tiles < sh.S ? tiles : sh.S;
        for (long i = 0; i < m; ++i) {
            const long idx = tiles - 1 - i;
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
// The same at system scope, for words that another GPU writes or reads over NVLink.
__device__ __forceinline__ void st_tagged_sys(uint2 *dst, float v, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2_sys(const uint4 *src) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
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
template <int kBatch>  // 16-byte loads in flight per thread and pass
__device__ __forceinline__ void poll_vector_pass(const MegaParams &p, Shared &sh, const uint4 *s4, int npairs, int base, uint32_t tag,
                                                 float *xs, int tid, int site) {
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

// The whole vector is requested in one pass whenever it fits 24 loads per thread (6144 words): every pass
// costs a round trip through L2, which is what this wait is made of.
__device__ __forceinline__ bool poll_vector(const MegaParams &p, Shared &sh, const uint2 *src, int n, uint32_t tag, float *xs,
                                            int tid, int &bk, int site) {
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
    const int npairs = n / 2;
    const int per_thread = (npairs + kConsumers - 1) / kConsumers;
    if (per_thread <= 4) poll_vector_pass<4>(p, sh, s4, npairs, 0, tag, xs, tid, site);
    else if (per_thread <= 8) poll_vector_pass<8>(p, sh, s4, npairs, 0, tag, xs, tid, site);
    else if (per_thread <= 16) poll_vector_pass<16>(p, sh, s4, npairs, 0, tag, xs, tid, site);
    else
        for (int base = 0; base < npairs; base += kConsumers * 16) poll_vector_pass<16>(p, sh, s4, npairs, base, tag, xs, tid, site);
    return consumer_bar_ok(sh.abort, sh.decision, tid, bk);
}

// Tensor-parallel form of poll_vector for the residual stream: waits for the T ranks' partial vectors
// (slots of `n` words, `slot_words` apart) and stages their sum, added in rank order.
template <int T, int KB>
__device__ __forceinline__ void poll_x_sum_pass(const MegaParams &p, Shared &sh, const uint2 *src, int slot_words, int npairs, int base,
                                                uint32_t tag, float *xs, int tid) {
    uint4 v[T][KB];
    const long long t0 = clock64();
    int spins = 0;
    bool done = false, alive = true;
    while (!done && alive) {
        done = true;
#pragma unroll
        for (int r = 0; r < T; ++r) {
            const uint4 *s4 = reinterpret_cast<const uint4 *>(src + (size_t)r * slot_words);
#pragma unroll
            for (int u = 0; u < KB; ++u) {
                const int idx = base + tid + kConsumers * u;
                v[r][u] = idx < npairs ? ld_tagged2_sys(s4 + idx) : make_uint4(0u, tag, 0u, tag);
            }
        }
#pragma unroll
        for (int r = 0; r < T; ++r)
#pragma unroll
            for (int u = 0; u < KB; ++u) done = done && v[r][u].y == tag && v[r][u].w == tag;
        if (!done) alive = poll_continue(p, sh.abort, spins, t0, 350, base);
    }
    if (!done) return;
#pragma unroll
    for (int u = 0; u < KB; ++u) {
        const int idx = base + tid + kConsumers * u;
        if (idx >= npairs) continue;
        float a = __uint_as_float(v[0][u].x), b = __uint_as_float(v[0][u].z);
#pragma unroll
        for (int r = 1; r < T; ++r) {
            a = __fadd_rn(a, __uint_as_float(v[r][u].x));
            b = __fadd_rn(b, __uint_as_float(v[r][u].z));
        }
        *reinterpret_cast<float2 *>(xs + 2 * idx) = make_float2(a, b);
    }
}

__device__ __forceinline__ bool poll_x_sum(const MegaParams &p, Shared &sh, const uint2 *src, int n, uint32_t tag, float *xs, int tid,
                                           int &bk) {
    const int npairs = n / 2, sw = p.x_slot_words;
    if (p.tp_size == 2)
        for (int base = 0; base < npairs; base += kConsumers * 8) poll_x_sum_pass<2, 8>(p, sh, src, sw, npairs, base, tag, xs, tid);
    else if (p.tp_size == 4)
        for (int base = 0; base < npairs; base += kConsumers * 4) poll_x_sum_pass<4, 4>(p, sh, src, sw, npairs, base, tag, xs, tid);
    else
        for (int base = 0; base < npairs; base += kConsumers * 2) poll_x_sum_pass<8, 2>(p, sh, src, sw, npairs, base, tag, xs, tid);
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
// Hands a stage back to the producer (this warp's share of the stage's arrivals) and, when tracing,
// notes the time the first warp did so.
__device__ __forceinline__ void release_stage(const MegaParams &p, Shared &sh, int rs, int count, uint32_t slot, int cta, int gwarp) {
    mbar_arrive_cnt(&sh.empty[rs], count);
    if (p.trace && cta == 0 && gwarp == 0 && slot < (uint32_t)kMegaTileTrace)
        p.trace[7 * (5 * p.L + 1) + 1 + kMegaTileTrace + slot] = globaltimer_ns();
}

// Tiles this CTA has consumed so far in the token: tile n of the CTA's schedule sits in ring stage n % S,
// and it is use n / S of that stage.
struct RingPos {
    uint32_t n;
};

// o_proj prologue: wait for the partial results of every attention work item and merge the splits,
// out = ctx * (1/(l + 1e-9)) (self_attention.rs:287-290), into shared memory xs[qd].
template <int NS, int VB>  // NS = context splits handled, VB = output vectors per thread and pass
__device__ __forceinline__ void poll_attention_pass(const MegaParams &p, Shared &sh, uint32_t tag, float *xs, int tid, int vbase) {
    const int nv4 = p.qd / 4;
    const int rec_words = 2 + p.D;  // uint2 words per (head, split) record
    uint4 ml[VB][NS], c01[VB][NS], c23[VB][NS];
    const long long t0 = clock64();
    int spins = 0;
    bool done = false, alive = true;
    while (!done && alive) {
        done = true;
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int v = vbase + tid + kConsumers * b;
            const int k0 = v * 4, h = k0 / p.D, e0 = k0 % p.D;
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const bool oks = s < p.nsplit && v < nv4;
                const uint4 *rec = reinterpret_cast<const uint4 *>(p.partT + ((size_t)(oks ? h : 0) * p.nsplit + (oks ? s : 0)) * rec_words);
                const uint4 ok_word = make_uint4(0xff800000u, tag, 0u, tag);  // {max = -inf, sum = 0}
                ml[b][s] = oks ? ld_tagged2(rec) : ok_word;
                c01[b][s] = oks ? ld_tagged2(rec + 1 + e0 / 2) : make_uint4(0u, tag, 0u, tag);
                c23[b][s] = oks ? ld_tagged2(rec + 2 + e0 / 2) : make_uint4(0u, tag, 0u, tag);
            }
        }
#pragma unroll
        for (int b = 0; b < VB; ++b)
#pragma unroll
            for (int s = 0; s < NS; ++s)
                done = done && ml[b][s].y == tag && ml[b][s].w == tag && c01[b][s].y == tag && c01[b][s].w == tag &&
                       c23[b][s].y == tag && c23[b][s].w == tag;
        if (!done) alive = poll_continue(p, sh.abort, spins, t0, 320, vbase);
    }
    if (!done) return;
#pragma unroll
    for (int b = 0; b < VB; ++b) {
        const int v = vbase + tid + kConsumers * b;
        if (v >= nv4) continue;
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < NS; ++s) M = fmaxf(M, __uint_as_float(ml[b][s].x));
        float L = 0.f;
        float4 c = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const float ms = __uint_as_float(ml[b][s].x);
            if (ms != -INFINITY) {
                const float f = expf(ms - M);
                L = fmaf(__uint_as_float(ml[b][s].z), f, L);
                c.x = fmaf(__uint_as_float(c01[b][s].x), f, c.x);
                c.y = fmaf(__uint_as_float(c01[b][s].z), f, c.y);
                c.z = fmaf(__uint_as_float(c23[b][s].x), f, c.z);
                c.w = fmaf(__uint_as_float(c23[b][s].z), f, c.w);
            }
        }
        const float inv = __fdiv_rn(1.0f, __fadd_rn(L, 1e-9f));
        reinterpret_cast<float4 *>(xs)[v] =
            make_float4(__fmul_rn(c.x, inv), __fmul_rn(c.y, inv), __fmul_rn(c.z, inv), __fmul_rn(c.w, inv));
    }
}

// As many of a thread's vectors as registers allow are requested per pass (each pass is a round trip
// through L2): four with one context split, two with two, one with up to kMaxSplit.
__device__ __forceinline__ bool poll_attention(const MegaParams &p, Shared &sh, uint32_t tag, float *xs, int tid, int &bk) {
    const int nv4 = p.qd / 4;
    if (p.nsplit == 1)
        for (int vb = 0; vb < nv4; vb += 4 * kConsumers) poll_attention_pass<1, 4>(p, sh, tag, xs, tid, vb);
    else if (p.nsplit == 2)
        for (int vb = 0; vb < nv4; vb += 2 * kConsumers) poll_attention_pass<2, 2>(p, sh, tag, xs, tid, vb);
    else
        for (int vb = 0; vb < nv4; vb += kConsumers) poll_attention_pass<kMaxSplit, 1>(p, sh, tag, xs, tid, vb);
    return consumer_bar_ok(sh.abort, sh.decision, tid, bk);
}

// One vector-matrix phase for the consumer threads.
//
// The input vector lives in shared memory for the whole phase (normalised in place when the phase starts
// with an RMSNorm), so a warp needs no registers for it and any warp can take any tile: tiles go
// round-robin to the four consumer warps, each warp works through its own tiles without ever meeting the
// others, and the only CTA-wide synchronisation is at the end of a row block.  Per 16-byte step a lane
// reads one vector of x and the matching vector of RB weight rows (all conflict-free 128-bit shared loads)
// and feeds RB accumulators; the RB cross-lane sums are folded into one butterfly (reduce_rows).
//   xres = the residual-stream value of the row this thread finishes in the o_proj / down phases (the row
//   split of those two phases is the same, so the value never leaves the thread).

// Sum over the 32 lanes of RB accumulators at once: every step halves the number of values a lane still
// carries by trading the other half with its partner, so RB = 4 costs 6 shuffles instead of 20.  The sum of
// row reduce_row_of<RB>(lane) ends up in lanes that are multiples of 32 / RB.
template <int RB>
__device__ __forceinline__ float reduce_rows(float (&a)[RB], int lane) {
    int bit = 16;
#pragma unroll
    for (int n = RB; n > 1; n >>= 1) {
        const bool up = (lane & bit) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = up ? a[i] : a[i + n / 2];
            const float keep = up ? a[i + n / 2] : a[i];
            a[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
        }
        bit >>= 1;
    }
#pragma unroll
    for (int b = 16 / RB; b > 0; b >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], b);
    return a[0];
}
template <int RB>
__device__ __forceinline__ int reduce_row_of(int lane) {
    if (lane % (32 / RB) != 0) return -1;
    int row = 0, bit = 16;
#pragma unroll
    for (int n = RB; n > 1; n >>= 1) {
        if (lane & bit) row += n / 2;
        bit >>= 1;
    }
    return row;
}

// Rows [rb, rb + RB) of one tile (row indices clamped to the tile's last row; x is zero-padded so that the
// clamped vector index of the last lanes contributes nothing).
template <typename WT, int RB>
__device__ __forceinline__ void tile_rows(const uint4 *st, const float4 *xs4, int nvec, int njl, int lane, int nr, int rb,
                                          float (&acc)[RB]) {
    constexpr int XQ = VecTraits<WT>::XQ;
    constexpr int NA = RB >= 4 ? 1 : 4 / RB;  // accumulators per row: four independent FMA chains in all
    const uint4 *row[RB];
    float a[RB][NA];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
        row[i] = st + (size_t)min(rb + i, nr - 1) * nvec;
#pragma unroll
        for (int c = 0; c < NA; ++c) a[i][c] = 0.f;
    }
    const int vlast = nvec - 1;
    for (int j0 = 0; j0 < njl; j0 += 4) {  // four steps at a time (x is zero-padded to a whole four steps)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int vx = lane + 32 * (j0 + jj);
            const int v = min(vx, vlast);
            float4 x[XQ];
#pragma unroll
            for (int q = 0; q < XQ; ++q) x[q] = xs4[vx * XQ + q];
#pragma unroll
            for (int i = 0; i < RB; ++i) a[i][jj % NA] = VecTraits<WT>::dot(row[i][v], x, a[i][jj % NA]);
        }
    }
#pragma unroll
    for (int i = 0; i < RB; ++i) {
        float t = a[i][0];
#pragma unroll
        for (int c = 1; c < NA; ++c) t += a[i][c];
        acc[i] = t;
    }
}

template <typename WT, int RB>
__device__ __forceinline__ void consume_tile(const MegaParams &p, Shared &sh, const uint4 *st, const float4 *xs4, int nvec, int njl,
                                             int lane, int nr, bool have, float *part, int rs, uint32_t slot, int cta) {
    for (int rb = 0; rb < nr; rb += RB) {
        float acc[RB];
        if (have) {
            tile_rows<WT, RB>(st, xs4, nvec, njl, lane, nr, rb, acc);
        } else {
#pragma unroll
            for (int i = 0; i < RB; ++i) acc[i] = 0.f;
        }
        if (rb + RB >= nr) {  // the tile's last loads are done: the stage can go back to the producer
            __syncwarp();
            if (lane == 0) release_stage(p, sh, rs, kConsumerWarps, slot, cta, 0);  // all 4 arrivals of the stage
        }
        const float s = reduce_rows<RB>(acc, lane);
        const int r = reduce_row_of<RB>(lane);
        if (r >= 0 && rb + r < nr) part[(rb + r) * kConsumerWarps] = s;
    }
}

template <typename WT>
__device__ __forceinline__ bool gemv_phase(const MegaParams &p, Shared &sh, const Phase &g, long id, RingPos &rp, int cta, int nctas,
                                           int tid, int &bk, int ph, float &xres) {
    constexpr int XPV = VecTraits<WT>::XPV;
    constexpr int XQ = VecTraits<WT>::XQ;
    const int lane = tid & 31, warp = tid >> 5;
    const MegaLayer *lw = g.layer < p.L ? &p.layers[g.layer] : nullptr;
    const TileIter ti(g, (int)sizeof(WT), sh.stage_bytes, cta, nctas, (p.debug_flags & 1) != 0);
    // No rows of this matrix here: nothing to read, nothing to publish - except that the phases which stage
    // the residual stream also refresh the residual value this thread carries for the o_proj / down epilogues.
    const bool has_rows = ti.r0 != ti.r1;
    const bool stages_x = g.kind == PH_QKV || g.kind == PH_GATEUP;
    if (!has_rows && !stages_x) return true;
    const int nvec = g.K / XPV;          // 16-byte weight vectors per row
    const int njl = (nvec + 31) / 32;    // steps of a lane through a row

    // ---- prologue: the input vector, in shared memory ---------------------------------------------------
    float *xs = sh.xs;
    float4 *xs4 = reinterpret_cast<float4 *>(xs);
    // RMSNorm gains of the phase are requested before the wait for x, so that their trip to L2 is not added
    // to the critical path (up to 4 vectors per thread: K <= 2048; longer rows fetch them afterwards).
    const float *norm_w = nullptr;
    if (g.kind == PH_QKV) norm_w = lw->norm1;
    else if (g.kind == PH_GATEUP) norm_w = lw->norm2;
    else if (g.kind == PH_LMHEAD) norm_w = p.final_norm;
    constexpr int kEarlyGains = 4;
    const int n4s = g.K / 4;
    const bool early = norm_w != nullptr && n4s <= kEarlyGains * kConsumers;
    float4 gains[kEarlyGains];
    if (early) {
#pragma unroll
        for (int u = 0; u < kEarlyGains; ++u) {
            const int i = tid + kConsumers * u;
            gains[u] = i < n4s ? __ldg(reinterpret_cast<const float4 *>(norm_w) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    const int njl4 = (njl + 3) & ~3;     // the inner loop takes four steps at a time
    for (int k = g.K + tid; k < njl4 * 32 * XPV; k += kConsumers) xs[k] = 0.f;  // zero padding up to whole steps
    if (g.kind == PH_QKV && g.layer == 0) {
        // Embedding::forward (embedding.rs:47-57): the token's row is the first layer's input
        for (int k = tid; k < g.K; k += kConsumers) xs[k] = embed_elem(p, id, k);
        consumer_bar();
    } else {
        const uint32_t tag = phase_tag(p, ph - 1);  // every phase consumes what the phase before it published
        bool ok;
        // o_proj outputs travel in x buffer 0 (read by gate/up), down outputs in buffer 1 (read by qkv, lm_head)
        const uint2 *xsrc = p.xT + (size_t)(g.kind == PH_GATEUP ? 0 : 1) * p.tp_size * p.x_slot_words;
        if (g.kind == PH_O) ok = poll_attention(p, sh, tag, xs, tid, bk);
        else if (g.kind == PH_DOWN) ok = poll_vector(p, sh, p.actT, g.K, tag, xs, tid, bk, 330 + g.kind);
        else if (p.tp_size == 1) ok = poll_vector(p, sh, xsrc, g.K, tag, xs, tid, bk, 330 + g.kind);
        else ok = poll_x_sum(p, sh, xsrc, g.K, tag, xs, tid, bk);
        if (!ok) return false;
        if (p.trace && cta == 0 && tid == 0) p.trace[4 * (5 * p.L + 1) + 1 + ph] = globaltimer_ns();
    }
    if (stages_x) {
        // xs holds the whole residual stream (all ranks' partial sums added): keep this thread's row of it
        const long r0h = (long)p.H * cta / nctas, r1h = (long)p.H * (cta + 1) / nctas;
        if (tid < r1h - r0h) xres = xs[r0h + tid];
        if (!has_rows) {
            trace_stamp(p, cta, tid, 3 * ph + 1);
            trace_stamp(p, cta, tid, 3 * ph + 2);
            return true;
        }
    }
    if (norm_w) {
        // RMSNorm::forward (rms_norm.rs:49-56): rms = sqrt(ss/dim + eps); x = (x * (1/rms)) * w, in place
        const float4 *n4 = reinterpret_cast<const float4 *>(norm_w);
        float ss = 0.f;
        for (int i = tid; i < n4s; i += kConsumers) {
            const float4 v = xs4[i];
            ss = fmaf(v.x, v.x, ss);
            ss = fmaf(v.y, v.y, ss);
            ss = fmaf(v.z, v.z, ss);
            ss = fmaf(v.w, v.w, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) sh.red[warp] = ss;
        consumer_bar();
        const float tot = (sh.red[0] + sh.red[1]) + (sh.red[2] + sh.red[3]);
        const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)g.K), p.eps)));
        auto rescale = [&](int i, const float4 w) {
            float4 v = xs4[i];
            v.x = __fmul_rn(__fmul_rn(v.x, inv), w.x);
            v.y = __fmul_rn(__fmul_rn(v.y, inv), w.y);
            v.z = __fmul_rn(__fmul_rn(v.z, inv), w.z);
            v.w = __fmul_rn(__fmul_rn(v.w, inv), w.w);
            xs4[i] = v;
        };
        if (early) {
#pragma unroll
            for (int u = 0; u < kEarlyGains; ++u) {
                const int i = tid + kConsumers * u;
                if (i < n4s) rescale(i, gains[u]);
            }
        } else {
            for (int i = tid; i < n4s; i += kConsumers) rescale(i, __ldg(n4 + i));
        }
        consumer_bar();
    }
    trace_stamp(p, cta, tid, 3 * ph + 1);

    // ---- tiles ------------------------------------------------------------------------------------------
    // Tiles are addressed in closed form: tile t of the phase covers rows [R * (t / nmat), +R) of the CTA's
    // range in matrix t % nmat (gate rows, then the same rows of up) and sits in ring slot (tiles consumed
    // so far + t).  Warp w owns tiles w, w + 4, ...  Rows are reduced and published in blocks of at most
    // kRowBlock (a block never splits a tile).
    const int R = ti.R, nmat = ti.nmat;
    const int nrows_cta = (int)(ti.r1 - ti.r0);
    const int chunks = (p.debug_flags & 1) ? 0 : (nrows_cta + R - 1) / R;
    const int chunks_per_block = kRowBlock / R;
    for (int cb = 0; cb < chunks; cb += chunks_per_block) {
        const int cend = min(chunks, cb + chunks_per_block);
        const int t0 = cb * nmat, t1 = cend * nmat;
        const int row0_blk = cb * R;  // first row of the block, relative to the CTA's first row
        for (int t = t0 + ((warp - t0) & (kConsumerWarps - 1)); t < t1; t += kConsumerWarps) {
            const int chunk = t / nmat, mat = t - chunk * nmat;
            const int rrel = chunk * R;
            const int nr = min(R, nrows_cta - rrel);
            const uint32_t slot = rp.n + (uint32_t)t;
            const int rs = (int)(slot % (uint32_t)sh.S);
            const uint32_t use = slot / (uint32_t)sh.S;
            // A parity test tells two phases apart, not three: before testing for use `u` of this stage,
            // use `u-1` (owned by another warp) must be known to have landed.  Its owner publishes that.
            // A failed wait must not leave early (see consumer_bar_ok): skip the math, keep the sequence.
            bool have = stage_use_seen(p, sh, rs, (int)use, 310 + g.kind);
            have = have && mbar_wait(p, sh, &sh.full[rs], use & 1, 300 + g.kind);
            if (have && lane == 0) sh.seen[rs] = (int)use + 1;
            if (p.debug_flags & 4) have = false;  // debug: wait for the tiles but skip the arithmetic
            const uint4 *st = reinterpret_cast<const uint4 *>(sh.stages + (size_t)rs * sh.stage_bytes);
            float *part = sh.part + ((size_t)mat * kRowBlock + (size_t)(rrel - row0_blk)) * kConsumerWarps;
            if (R >= 4) consume_tile<WT, 4>(p, sh, st, xs4, nvec, njl, lane, nr, have, part, rs, slot, cta);
            else if (R >= 2) consume_tile<WT, 2>(p, sh, st, xs4, nvec, njl, lane, nr, have, part, rs, slot, cta);
            else consume_tile<WT, 1>(p, sh, st, xs4, nvec, njl, lane, nr, have, part, rs, slot, cta);
        }
        // End of a row block: run the epilogue on the row sums and publish.
        const int nrows = min(cend * R, nrows_cta) - row0_blk;
        if (!consumer_bar_ok(sh.abort, sh.decision, tid, bk)) return false;
        if (tid < nrows) {
            const float tot = sh.part[(size_t)tid * kConsumerWarps];
            const long row = ti.r0 + row0_blk + tid;
            const uint32_t tag = phase_tag(p, ph);
            switch (g.kind) {
                case PH_QKV:
                    // debug bit 3: the first phase of the token publishes nothing, so that every wait on it
                    // runs into its limit (used to test the time-out path; nothing faults or hangs)
                    if (!((p.debug_flags & 8) && ph == 0)) st_tagged(p.qkvT + row, tot, tag);
                    break;
                case PH_O:      // h = x + attn_out                                   llama.rs:110
                case PH_DOWN: { // out = h + mlp_out                                  llama.rs:115
                    // (these phases have a single row block: see the launcher)
                    const size_t slot = (size_t)((g.kind == PH_O ? 0 : 1) * p.tp_size + p.tp_rank) * p.x_slot_words + row;
                    if (p.tp_size == 1) {
                        st_tagged(p.xT + slot, __fadd_rn(xres, tot), tag);
                    } else {
                        // this rank's partial sum (rank 0 adds the residual) goes to every rank's copy
                        const float val = p.tp_rank == 0 ? __fadd_rn(xres, tot) : tot;
                        for (int r = 0; r < p.tp_size; ++r) st_tagged_sys(p.x_peer[r] + slot, val, tag);
                    }
                    break;
                }
                case PH_GATEUP: {  // SiLU (activation.rs:143-146) then gate_act * up (llama.rs:61-63)
                    const float up = sh.part[((size_t)kRowBlock + tid) * kConsumerWarps];
                    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-tot)));
                    st_tagged(p.actT + row, __fmul_rn(__fmul_rn(tot, sig), up), tag);
                    break;
                }
                default: p.logits[row] = tot; break;
            }
        }
        if (cend < chunks) consumer_bar();  // the table is rewritten by the next block
    }
    rp.n += (uint32_t)(chunks * nmat);
    if ((p.debug_flags & 1) && ti.r0 + tid < ti.r1) {  // debug (no tiles streamed): publish zeros so that the chain runs
        const uint32_t tag = phase_tag(p, ph);
        uint2 *dst = g.kind == PH_QKV ? p.qkvT : g.kind == PH_GATEUP ? p.actT : p.xT + (size_t)(g.kind == PH_O ? 0 : 1) * p.x_slot_words;
        if (g.kind != PH_LMHEAD) st_tagged(dst + ti.r0 + tid, 0.f, tag);
    }
    trace_stamp(p, cta, tid, 3 * ph + 2);
    return true;
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
    RingPos rp{0};
    int bk = 0;
    for (int ph = 0; ph < nphases; ++ph) {
        const Phase g = get_phase(p, p.layers, ph);
        trace_stamp(p, cta, tid, 3 * ph);
        if (g.kind == PH_ATT) {
            if (!attention_phase(p, sh, g.layer, ph, past, cta, nctas, tid, bk)) return;
            trace_stamp(p, cta, tid, 3 * ph + 1);
            trace_stamp(p, cta, tid, 3 * ph + 2);
        } else {
            if (!gemv_phase<WT>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres)) return;
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
    sh.xs = fl;
    sh.part = fl + mega_xs_floats(max(p.H, max(p.qd, p.I)));
    sh.red = fl + mega_table_floats(max(p.H, max(p.qd, p.I)));
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
        producer_loop(p, sh, cta, tid - kConsumers);
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

int decode_mega_debug_flags() {
    static const int flags = [] {
        const char *e = getenv("LUMEN_MEGA_DEBUG");
        return e ? atoi(e) : 0;
    }();
    return flags;
}

void decode_mega_build_schedule(const MegaParams &p_in, const MegaLayer *host_layers, int grid, std::vector<uint4> &entries,
                                std::vector<int> &counts, int &stride) {
    MegaParams p = p_in;
    p.debug_flags = decode_mega_debug_flags();
    const int esz = p.wbf16 ? 2 : 4, nphases = 5 * p.L + 1;
    std::vector<std::vector<uint4>> per(grid);
    for (int cta = 0; cta < grid; ++cta) {
        for (int ph = 0; ph < nphases; ++ph) {
            const Phase g = get_phase(p, host_layers, ph);
            if (g.kind == PH_ATT) continue;
            for (TileIter ti(g, esz, kMegaStageBytes, cta, grid, (p.debug_flags & 1) != 0); ti.valid(); ti.advance()) {
                // whole rows are one contiguous block: one copy per tile
                const unsigned long long a = (unsigned long long)(uintptr_t)((ti.mat == 0 ? g.w0 : g.w1) + (size_t)ti.r * ti.rowbytes);
                const uint32_t tile_bytes = (uint32_t)ti.rows() * (uint32_t)ti.rowbytes;
                per[cta].push_back(make_uint4((uint32_t)a, (uint32_t)(a >> 32), tile_bytes | ((uint32_t)ph << 16), tile_bytes));
            }
        }
    }
    size_t mx = 1;
    for (auto &v : per) mx = std::max(mx, v.size());
    stride = (int)((mx + 31) / 32 * 32);
    entries.assign((size_t)grid * stride, make_uint4(0u, 0u, 0u, 0u));
    counts.resize(grid);
    for (int cta = 0; cta < grid; ++cta) {
        counts[cta] = (int)per[cta].size();
        std::copy(per[cta].begin(), per[cta].end(), entries.begin() + (size_t)cta * stride);
    }
}
unsigned int decode_mega_epochs_per_launch(int layers) { return 5u * (unsigned)layers + 2u; }

size_t decode_mega_x_words(const MegaParams &p) { return 2 * (size_t)p.tp_size * (size_t)((p.H + 1) & ~1); }

size_t decode_mega_exchange_words(const MegaParams &p) {
    return decode_mega_x_words(p) + p.qkv_rows + p.I + (size_t)p.Hq * kMaxSplit * (2 + p.D) + 8;
}

int decode_mega_supported(const MegaParams &p, char *why, size_t why_len) {
    const int esz = p.wbf16 ? 2 : 4;
    const int ks[3] = {p.H, p.qd, p.I};
    for (int k : ks) {
        if ((k * esz) % 16) {
            snprintf(why, why_len, "row of %d elements is not a multiple of 16 bytes", k);
            return 0;
        }
        if (k * esz > kMegaStageBytes) {
            snprintf(why, why_len, "a row of %d elements does not fit one %d-byte ring stage", k, kMegaStageBytes);
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
    p.stage_bytes = kMegaStageBytes;
    const int kmax = std::max(p.H, std::max(p.qd, p.I));
    const size_t budget = 227 * 1024 - 1024;  // static shared (barriers, flags) and alignment slack
    int stages = kMegaMaxStages;
    while (stages > 2 && decode_mega_smem_bytes(stages, p.stage_bytes, p.D, kmax) > budget) --stages;
    p.stages = stages;
    p.debug_flags = decode_mega_debug_flags();
    // L2 look-ahead of the producer in copies per CTA, counted from the copy being issued (the ring itself
    // holds `stages` of them): 0 = off, at most 56.
    p.l2_ahead = 8;  // measured: +2 % at 8, no gain at 12, a loss from 20 on (the look-ahead competes with the exchanges)
    if (const char *e = getenv("LUMEN_MEGA_L2_AHEAD")) p.l2_ahead = std::max(0, std::min(56, atoi(e)));
    if (!p.sched || !p.sched_count) return set_error(ctx, LUMEN_ERR_INVALID, "persistent decode kernel: no producer schedule");
    const size_t smem = decode_mega_smem_bytes(stages, p.stage_bytes, p.D, kmax);
    if (smem > budget) return set_error(ctx, LUMEN_ERR_UNSUPPORTED, "shared memory: %zu bytes needed", smem);
    const void *kern = p.wbf16 ? (const void *)decode_mega_kernel<__nv_bfloat16> : (const void *)decode_mega_kernel<float>;
    static bool attr_set[64][2] = {};  // per device ordinal and weight type
    const int dev = ctx->device >= 0 && ctx->device < 64 ? ctx->device : 0;
    if (!attr_set[dev][p.wbf16 ? 1 : 0]) {  // once, for the largest ring any shape can ask for
        LUMEN_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget));
        attr_set[dev][p.wbf16 ? 1 : 0] = true;
    }
    void *args[] = {&p};
    LUMEN_CUDA(ctx, cudaLaunchCooperativeKernel(kern, dim3(grid), dim3(kThreads), args, smem, s));
    ctx->launches += 1;
    return LUMEN_OK;
}

}  // namespace lumen
