// Whole-token persistent decode kernel (batch 1): one launch runs LlamaModel::forward for one new
// token (src/models/llama.rs:181-206 of the reference; layer body :104-116, MLP :59-65, decode
// attention self_attention.rs:141-297, vector-matrix products src/ops/matmul.rs:42-69).
//
// Design for B200: one CTA per SM (launched cooperatively so that all CTAs are co-resident).  The
// last warp of each CTA is a producer: it walks a schedule of copies that the host built once (the CTA's
// rows of every matrix of every layer, in execution order) and streams the weight tiles from HBM into a
// shared-memory ring of 16 KB stages with TMA copies (mbarrier transaction counts, L2 evict-first).  A tile
// is four rows x 4 KB: rows of up to 4 KB travel whole (1-D bulk copy of the contiguous rows), longer rows
// are cut into segments and a tile is ONE 3-D tiled copy (cp.async.bulk.tensor: a box of four rows x one
// segment out of the row-major matrix).  Each producer lane issues one copy of a batch of 32, so the fixed
// cost of a copy is paid once per batch.  The schedule does not depend on the activations, so the producer
// keeps HBM busy across phase boundaries while the consumer warps wait for activations or run the
// (weight-free) attention.
//
// Consumers: a phase's input vector is staged in shared memory (multiplied by the RMSNorm gains on the
// way in; the 1/rms factor is a scalar and is applied to the row sums).  Tiles go round-robin to the seven
// consumer warps and a warp works through a tile alone: per 16-byte step a lane reads one vector of x and the
// matching vector of four weight rows with conflict-free 128-bit shared loads, the four row sums are folded
// across lanes by one butterfly and land in the row's column (one per segment) of a table of partial sums.
// The only CTA-wide barrier is at the end of a row block, where the partial sums of a row are added, the
// fused epilogue runs (1/rms, residual add, SiLU*mul) and the results are published.  Phases of a layer:
// qkv | attention | o_proj(+residual) | gate/up(+SiLU*mul) | down(+residual).
// The arithmetic on tiles that already sit in shared memory is what the token's time is made of (measured
// with the copies switched off), so the kernel is kept free of register spills: with the L1 squeezed by
// ~220 KB of shared memory a spill reload inside the tile loop is a round trip through L2.
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

// 7 consumer warps + 1 producer warp: two warps per SM sub-partition, so every thread may use up to 255 registers
// (with three warps on a sub-partition the limit is 168) and each scheduler has a second warp to cover the
// shared-memory and shuffle latencies of the first.  The kernel must not spill: the L1 is squeezed by ~220 KB of
// shared memory, and a spill reload inside the tile loop is a round trip through L2.
constexpr int kConsumers = 224;
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kThreads = kConsumers + 32;   // + producer warp
constexpr int kMaxRowsPerTile = 8;
constexpr int kRowBlock = 64;              // rows reduced together (one per consumer thread, half of them idle)
constexpr int kMaxSeg = 8;                 // segments a row is cut into at most
constexpr int kPartCols = kMaxSeg;         // columns of the table of partial row sums: one per segment
constexpr int kMaxSplit = 4;               // attention splits merged in the o_proj prologue
constexpr long long kWaitCycles = 400000000LL;  // ~0.2 s at 1.9 GHz
constexpr long long kPrefetchGrace = 1000;      // a ring that has been full for this long is a stall, not back-pressure
constexpr long long kPrefetchPace = 600;        // cycles between the L2 prefetches of consecutive 16 KB tiles (~54 KB/us)

// Floats of the staged input vector of a phase (up to kmax elements, zero-padded to four whole steps of a
// warp through a row: 4 x 32 lanes x 8 elements) and of the table of row sums of a row block ([2][kRowBlock][4]).
__host__ __device__ inline size_t mega_xs_floats(int kmax) { return (((size_t)kmax + 1023) / 1024) * 1024; }
__host__ __device__ inline size_t mega_table_floats(int kmax) {
    return mega_xs_floats(kmax) + 2 * (size_t)kRowBlock * kPartCols;
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
// Non-blocking test of a barrier phase (try_wait may suspend the thread for an implementation-defined time).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
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
// 3-D tiled TMA copy: box of the map at (0, unit, row) -> this CTA's shared memory.  The innermost coordinate is
// always 0, so the 16-byte start rule of TMA holds.
__device__ __forceinline__ void tensor_load(void *dst_smem, const CUtensorMap *map, int unit, int row, uint64_t *bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(smem_u32(dst_smem)), "l"(map), "r"(0), "r"(unit), "r"(row), "r"(smem_u32(bar)), "l"(pol)
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
// Per-CTA stamps: which = 0 (input arrived) or 1 (results published).
__device__ __forceinline__ void trace_cta(const MegaParams &p, int cta, int tid, int which, int ph) {
    if (p.trace && tid == 0 && cta < kMegaTraceCtas) {
        const size_t nph = 5 * (size_t)p.L + 1;
        p.trace[decode_mega_trace_base_words(p.L) + ((size_t)which * nph + ph) * kMegaTraceCtas + cta] = globaltimer_ns();
    }
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
    float *part;       // [2][kRowBlock][kPartCols]: partial row sums of one block, one column per (segment, half) of the row
    float *red;        // [kConsumerWarps] partial sums of squares of the staged vector
    float *xraw;       // [kRowBlock] the residual-stream values of this CTA's rows, before the gains
    float *attn;       // scratch of the attention item
    uint64_t *full;    // [S]
    uint64_t *empty;   // [S]
    volatile int *abort;
    volatile int *decision;  // [2] abort flag sampled by thread 0 before a barrier, read by all after it
    volatile int *issued;    // [S] producer: the last use of each stage whose copies have been issued (-1: none yet)
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

#ifdef LUMEN_MEGA_TRYWAIT
#define MEGA_WAIT mbar_try_wait
#else
#define MEGA_WAIT mbar_test_wait
#endif
// Bounded mbarrier wait; false = gave up (abort raised) or somebody else aborted.
__device__ __forceinline__ bool mbar_wait(const MegaParams &p, Shared &sh, uint64_t *bar, uint32_t parity, int site) {
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!(MEGA_WAIT(bar, parity))) {
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

// Bounded wait until `uses` fills of stage s are known to have landed (written by the
// warps that consumed them).  In steady state this is already true and costs one shared-memory read.
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

// The CTA's tiles of one phase, in the order both the producer and the consumers walk them.
// A tile is up to R rows (4, or 8 for very short rows) x one segment of the row length.  Rows longer than a
// quarter of a ring stage are cut into nseg = 2 or 4 segments of whole steps (a step = 32 consecutive 16-byte
// vectors, one per lane), so that every tile holds four rows and each 16-byte vector of x read from shared
// memory feeds four weight rows; a segmented tile arrives as one bulk copy per row, packed back to back in the
// stage.  Tile t of the phase = (chunk of R rows, matrix, segment): t = (chunk * nmat + mat) * nseg + seg.
// The partial row sums of the segments of a row land in different columns of the row-sum table.
struct PhaseTiles {
    long r0, r1;  // the CTA's rows of the matrix (or matrices)
    int nmat, R, nseg, per, njl, rowbytes, nrows, chunks;
    __host__ __device__ PhaseTiles(const Phase &g, int esz, int stage_bytes, int cta, int nctas) {
        rowbytes = g.K * esz;
        nmat = g.nmat;
        r0 = (long)g.N * cta / nctas;
        r1 = (long)g.N * (cta + 1) / nctas;
        nrows = (int)(r1 - r0);
        njl = (rowbytes / 16 + 31) / 32;  // steps of a lane through a whole row
        // Four whole rows per stage where they fit; otherwise four rows x segments of stage_bytes / 4 bytes each (a
        // whole number of blocks of four steps, the unit of the consumers' inner loop).
        nseg = 1;
        per = njl;
        if (4 * rowbytes > stage_bytes) {
            per = (stage_bytes / 4 / 512) & ~3;
            nseg = (njl + per - 1) / per;
        }
        R = (nseg == 1 && 8 * rowbytes <= stage_bytes) ? 8 : 4;
        chunks = (nrows + R - 1) / R;
    }
    __host__ __device__ int tiles() const { return chunks * nmat * nseg; }
    __host__ __device__ int seg_steps(int seg) const { return (njl < (seg + 1) * per ? njl : (seg + 1) * per) - seg * per; }
    __host__ __device__ int seg_bytes(int seg) const {
        const int b1 = (seg + 1) * per * 512;
        return (b1 < rowbytes ? b1 : rowbytes) - seg * per * 512;
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
__device__ __forceinline__ void prefetch_tensor_l2(const CUtensorMap *map, int unit, int row) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];" ::"l"(map), "r"(0), "r"(unit), "r"(row) : "memory");
}
__device__ __forceinline__ void prefetch_entry(const MegaParams &p, const uint4 &f) {
    if (f.w & 0x80000000u) prefetch_tensor_l2(p.tmaps + (f.x & 0xffffu), (int)(f.x >> 16), (int)f.y);
    else prefetch_l2(reinterpret_cast<const char *>(((unsigned long long)f.y << 32) | f.x), f.z & 0xffffu);
}

// The producer warp.  Each lane owns one entry of a batch of 32 schedule entries (one coalesced load; the next
// batch is requested before the current one is issued) and issues that copy by itself: it waits until the ring
// stage of its tile is free, arms the stage's barrier with the tile's byte count if the copy is the first of
// its tile, and issues the copy.  The lanes run in lockstep, so the fixed cost of a copy (barrier test, address
// set-up, the TMA instruction) is paid once per pass for all the copies whose stages are free, instead of once
// per copy by a single thread, which capped the stream at one tile per ~0.33 us.  A batch is issued in passes of
// at most S tiles: within a pass no two tiles share a stage, so a stage's barrier is never tested for a use
// before the use before it has been issued (a parity test tells two uses apart, not three).
__device__ __forceinline__ void producer_loop(const MegaParams &p, Shared &sh, int cta, int lane) {
    const uint64_t pol = make_evict_first_policy();
    const int nphases = 5 * p.L + 1;
    const uint4 *sched = p.sched + (size_t)cta * p.sched_stride;
    const int n = p.sched_count[cta];
    const uint32_t S = (uint32_t)sh.S;
    uint32_t tiles = 0;  // tiles before the current batch (the same in every lane)
    int last_ph = -1;    // trace: phase of the last entry of the previous batch
    bool carry_pf = false;
    bool ok = true;
    uint4 nxt = lane < n ? sched[lane] : make_uint4(0u, 0u, 0u, 0u);
    for (int base = 0; base < n && ok; base += 32) {
        const uint4 e = nxt;
        if (base + 32 + lane < n) nxt = sched[base + 32 + lane];
        const bool valid = base + lane < n;
        const bool first = valid && (e.w & 0xffffu) != 0;  // first copy of a tile
        const uint32_t firsts = __ballot_sync(0xffffffffu, first);
        // tile of this lane's copy: a continuation copy belongs to the tile of the nearest first copy before it
        const uint32_t tile = tiles + (uint32_t)__popc(firsts & (0xffffffffu >> (31 - lane))) - 1u;
        const uint32_t slot = tile % S, use = tile / S;
        unsigned char *dst = sh.stages + (size_t)slot * sh.stage_bytes + (size_t)((e.w >> 16) & 0xfffu) * 16;
        if (p.trace && cta == 0) {  // (uniform: every lane takes part in the shuffles)
            const int ph = valid ? (int)(e.z >> 16) : -1;
            int ph_prev = __shfl_up_sync(0xffffffffu, ph, 1);
            if (lane == 0) ph_prev = last_ph;
            last_ph = __shfl_sync(0xffffffffu, ph, min(31, n - base - 1));
            if (first && tile < (uint32_t)kMegaTileTrace) p.trace[7 * nphases + 1 + tile] = globaltimer_ns();
            if (valid && ph_prev != ph) p.trace[3 * nphases + 1 + ph] = globaltimer_ns();  // first copy of a phase
        }
        bool pending = valid, prefetched = carry_pf;  // (this entry may have gone to the L2 while it was the next batch)
        const uint32_t ntiles_batch = (uint32_t)__popc(firsts);
        // the entry of the NEXT batch this lane already holds, and its tile (for the look-ahead below)
        const bool valid_n = base + 32 + lane < n;
        const uint32_t firsts_n = __ballot_sync(0xffffffffu, valid_n && (nxt.w & 0xffffu) != 0);
        const uint32_t tile_n = tiles + ntiles_batch + (uint32_t)__popc(firsts_n & (0xffffffffu >> (31 - lane))) - 1u;
        bool prefetched_n = !valid_n;
        for (uint32_t t0 = tiles; __any_sync(0xffffffffu, pending) && ok; t0 += S) {
            const bool mine = pending && tile < t0 + S;  // this pass: tiles [t0, t0 + S)
            const long long c0 = clock64();
            int spins = 0;
            bool waiting = mine;
            while (__any_sync(0xffffffffu, waiting)) {
                if (waiting && (use == 0 || mbar_try_wait(&sh.empty[slot], (use - 1) & 1))) {
                    if (first) mbar_expect_tx(&sh.full[slot], e.w & 0xffffu);
                    if (e.w & 0x80000000u) {  // box of rows x one segment of the row length (3-D tiled copy)
                        tensor_load(dst, p.tmaps + (e.x & 0xffffu), (int)(e.x >> 16), (int)e.y, &sh.full[slot], pol);
                    } else {
                        bulk_load(dst, reinterpret_cast<const char *>(((unsigned long long)e.y << 32) | e.x), e.z & 0xffffu, &sh.full[slot], pol);
                    }
                    if (first) sh.issued[slot] = (int)use;
                    waiting = false;
                    pending = false;
                }
                // The ring is full and the stall has lasted a while (the consumers wait for activations): hand the next
                // copies to the L2, ONE tile per `pace` cycles, in order.  HBM then keeps streaming at about its fair
                // share while the ring cannot take more, without the burst of requests that would queue up in front
                // of the consumers' polls; the ring later refills from the L2.
                if (p.l2_ahead > 0 && pending && !prefetched && tile >= t0 && tile - t0 < (uint32_t)p.l2_ahead &&
                    clock64() - c0 > (long long)p.pf_grace + (long long)(tile - t0) * p.pf_pace) {
                    prefetch_entry(p, e);
                    prefetched = true;
                }
                if (p.l2_ahead > 32 && !prefetched_n && tile_n >= t0 && tile_n - t0 < (uint32_t)p.l2_ahead &&
                    clock64() - c0 > (long long)p.pf_grace + (long long)(tile_n - t0) * p.pf_pace) {
                    prefetch_entry(p, nxt);
                    prefetched_n = true;
                }
                if ((++spins & 63) == 0) {
                    bool give_up = *sh.abort != 0;
                    if (!give_up && clock64() - c0 > kWaitCycles) {
                        if (waiting) raise_abort(p, sh.abort, 100, (int)slot);
                        give_up = true;
                    }
                    if (__any_sync(0xffffffffu, give_up)) {
                        ok = false;
                        break;
                    }
                }
            }
        }
        tiles += ntiles_batch;
        carry_pf = valid_n && prefetched_n;
    }
    if (!ok && lane < (int)S) {
        // Wait (bounded) for this stage's last copies still in flight before the CTA may exit.
        const int u = sh.issued[lane];
        if (u >= 0) {
            const long long t0 = clock64();
            while (!mbar_try_wait(&sh.full[lane], (uint32_t)u & 1) && clock64() - t0 < kWaitCycles) {}
        }
    }
}

// ---- consumers ---------------------------------------------------------------------------------------
// Tagged exchange words {f32 bits, tag}.  A word is written and read as ONE 64-bit access (b64 stores, v2.b64
// loads: each 64-bit element is single-copy atomic in the PTX memory model), so a reader that sees the tag
// also sees the value that was stored with it.  A 16-byte load fetches two such words; each is checked on its own.
__device__ __forceinline__ void st_tagged(uint2 *dst, float v, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2(const uint4 *src) {
    unsigned long long a, b;
    asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(src) : "memory");
    return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
}
// The same at system scope, for words that another GPU writes or reads over NVLink.
__device__ __forceinline__ void st_tagged_sys(uint2 *dst, float v, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(dst), "l"(w) : "memory");
}
__device__ __forceinline__ uint4 ld_tagged2_sys(const uint4 *src) {
    unsigned long long a, b;
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(src) : "memory");
    return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
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

// What the staging of a phase's input vector does besides copying it (all optional):
//   gains   RMSNorm gains: xs[k] = x[k] * gains[k].  RMSNorm::forward (rms_norm.rs:49-56) is (x * inv) * w with
//           the scalar inv = 1 / sqrt(mean(x^2) + eps); inv multiplies the finished row sums instead.
//   ss      this thread's share of sum(x^2), accumulated over the raw values
//   xraw    the raw values of elements [r0, r1) are kept aside (the residual stream of this CTA's rows)
struct StageOpts {
    const float *gains = nullptr;
    float *xraw = nullptr;
    int r0 = 0, r1 = 0;
};
__device__ __forceinline__ void stage_pair(const StageOpts o, float *xs, int idx, float a, float b, float2 g, float &ss) {
    ss = fmaf(a, a, ss);
    ss = fmaf(b, b, ss);
    if (o.xraw) {
        const int e = 2 * idx;
        if (e >= o.r0 && e < o.r1) o.xraw[e - o.r0] = a;
        if (e + 1 >= o.r0 && e + 1 < o.r1) o.xraw[e + 1 - o.r0] = b;
    }
    *reinterpret_cast<float2 *>(xs + 2 * idx) = make_float2(__fmul_rn(a, g.x), __fmul_rn(b, g.y));
}

// All consumer threads: wait until the `n` tagged words at `src` (n even) carry `tag`, and leave their
// values as floats in shared memory `xs[n]`.  The gains are requested before the first poll so that their trip
// to L2 is not added to the critical path.
template <int kBatch>  // 16-byte loads in flight per thread and pass
__device__ __forceinline__ void poll_vector_pass(const MegaParams &p, Shared &sh, const uint4 *s4, int npairs, int base, uint32_t tag,
                                                 float *xs, int tid, int site, const StageOpts o, float &ss) {
    uint4 v[kBatch];
    // up to 8 loads per thread the gains wait in registers; longer vectors fetch them after the wait instead
    constexpr bool kEarlyGains = kBatch <= 8;
    float2 g[kEarlyGains ? kBatch : 1];
    if (kEarlyGains) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int idx = base + tid + kConsumers * u;
            g[u] = (o.gains && idx < npairs) ? __ldg(reinterpret_cast<const float2 *>(o.gains) + idx) : make_float2(1.f, 1.f);
        }
    }
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
            if (idx >= npairs) continue;
            const float2 gu = kEarlyGains ? g[kEarlyGains ? u : 0]
                                          : (o.gains ? __ldg(reinterpret_cast<const float2 *>(o.gains) + idx) : make_float2(1.f, 1.f));
            stage_pair(o, xs, idx, __uint_as_float(v[u].x), __uint_as_float(v[u].z), gu, ss);
        }
    }
}

// Leaves this warp's share of sum(x^2) in red[warp] (read by everybody after the next consumer barrier).
__device__ __forceinline__ void publish_ss(Shared &sh, float ss, int tid) {
    ss = warp_sum(ss);
    if ((tid & 31) == 0) sh.red[tid >> 5] = ss;
}

// The whole vector is requested in one pass whenever it fits 16 loads per thread (4096 words): every pass
// costs a round trip through L2, which is what this wait is made of.
__device__ __forceinline__ bool poll_vector(const MegaParams &p, Shared &sh, const uint2 *src, int n, uint32_t tag, float *xs,
                                            int tid, int &bk, int site, const StageOpts o = StageOpts()) {
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
    const int npairs = n / 2;
    const int per_thread = (npairs + kConsumers - 1) / kConsumers;
    float ss = 0.f;
    // At most 13 loads per thread and pass (a 5632-element vector in one pass of 224 threads): more words in flight
    // would push the kernel's hot loops into spilling, and with the L1 squeezed by the shared-memory ring a spill
    // costs a round trip through L2.  Every pass is such a round trip too.
    if (per_thread <= 4) poll_vector_pass<4>(p, sh, s4, npairs, 0, tag, xs, tid, site, o, ss);
    else if (per_thread <= 8) poll_vector_pass<8>(p, sh, s4, npairs, 0, tag, xs, tid, site, o, ss);
    else
        for (int base = 0; base < npairs; base += kConsumers * 13) poll_vector_pass<13>(p, sh, s4, npairs, base, tag, xs, tid, site, o, ss);
    publish_ss(sh, ss, tid);
    return consumer_bar_ok(sh.abort, sh.decision, tid, bk);
}

// Tensor-parallel form of poll_vector for the residual stream: waits for the T ranks' partial vectors
// (slots of `n` words, `slot_words` apart) and stages their sum, added in rank order.
template <int T, int KB>
__device__ __forceinline__ void poll_x_sum_pass(const MegaParams &p, Shared &sh, const uint2 *src, int slot_words, int npairs, int base,
                                                uint32_t tag, float *xs, int tid, const StageOpts o, float &ss) {
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
        // (the T * KB words in flight leave no registers to hold the gains through the wait)
        const float2 gu = o.gains ? __ldg(reinterpret_cast<const float2 *>(o.gains) + idx) : make_float2(1.f, 1.f);
        stage_pair(o, xs, idx, a, b, gu, ss);
    }
}

// Two-step form of the same exchange: the threads that own rows [r0, r1) of the residual stream wait for the ranks'
// partial values of their row, add them in rank order and publish the sum in `dst` (this GPU's xrT buffer); then
// every thread stages dst like a single-GPU vector.
__device__ __forceinline__ bool reduce_then_poll_x(const MegaParams &p, Shared &sh, const uint2 *src, uint2 *dst, int n, uint32_t tag,
                                                   float *xs, int tid, int &bk, int r0, int r1, const StageOpts o) {
    if (tid < r1 - r0) {
        const int row = r0 + tid;
        const long long t0 = clock64();
        int spins = 0;
        float sum = 0.f;
        bool done = false, alive = true;
        while (!done && alive) {
            done = true;
            unsigned long long w[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
                if (r < p.tp_size) asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w[r]) : "l"(src + (size_t)r * p.x_slot_words + row) : "memory");
            sum = 0.f;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < p.tp_size) {
                    done = done && (uint32_t)(w[r] >> 32) == tag;
                    const float v = __uint_as_float((uint32_t)w[r]);
                    sum = r == 0 ? v : __fadd_rn(sum, v);
                }
            }
            if (!done) alive = poll_continue(p, sh.abort, spins, t0, 355, row);
        }
        if (done) st_tagged(dst + row, sum, tag);
    }
    return poll_vector(p, sh, dst, n, tag, xs, tid, bk, 356, o);
}

__device__ __forceinline__ bool poll_x_sum(const MegaParams &p, Shared &sh, const uint2 *src, int n, uint32_t tag, float *xs, int tid,
                                           int &bk, const StageOpts o) {
    const int npairs = n / 2, sw = p.x_slot_words;
    float ss = 0.f;
    if (p.tp_size == 2)
        for (int base = 0; base < npairs; base += kConsumers * 5) poll_x_sum_pass<2, 5>(p, sh, src, sw, npairs, base, tag, xs, tid, o, ss);
    else if (p.tp_size == 4)
        for (int base = 0; base < npairs; base += kConsumers * 3) poll_x_sum_pass<4, 3>(p, sh, src, sw, npairs, base, tag, xs, tid, o, ss);
    else  // 8 ranks (the launcher admits 1, 2, 4 and 8)
        for (int base = 0; base < npairs; base += kConsumers) poll_x_sum_pass<8, 1>(p, sh, src, sw, npairs, base, tag, xs, tid, o, ss);
    publish_ss(sh, ss, tid);
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
// The input vector lives in shared memory for the whole phase (already multiplied by the RMSNorm gains when
// the phase starts with an RMSNorm).  All four consumer warps walk the CTA's tiles in order and each takes
// its own quarter of the row length of every tile: per 16-byte step a lane reads one vector of x and the
// matching vector of RB weight rows (all conflict-free 128-bit shared loads) and feeds RB accumulators; the
// RB cross-lane sums are folded into one butterfly (reduce_rows) and land in the warp's column of the
// table of partial row sums.  A warp hands its share of the stage back as soon as its loads are done.
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

// Steps [s0, s1) of a lane through rows [rb, rb + RB) of one tile: a step is 32 consecutive 16-byte vectors of
// the row, one per lane.  Row indices are clamped to the tile's last row, vector indices to the row's last
// vector (x is zero-padded to whole steps, so a clamped vector contributes nothing).
template <typename WT, int RB>
__device__ __forceinline__ void tile_rows(const uint4 *st, const float4 *xs4, int stride, int nvec, int s0, int s1, int lane, int nr,
                                          int rb, float (&acc)[RB]) {
    constexpr int XQ = VecTraits<WT>::XQ;
    // accumulators per row: two FMA chains per row measured 24 % faster than one on tiles resident in shared memory
    // (904 against 1194 cycles per 16 KB tile and warp), the dependent chain of one being 32 FMAs long
    constexpr int NA = RB >= 4 ? 2 : 4 / RB;
    const uint4 *row[RB];
    float a[RB][NA];
#pragma unroll
    for (int i = 0; i < RB; ++i) {
        row[i] = st + (size_t)min(rb + i, nr - 1) * stride;
#pragma unroll
        for (int c = 0; c < NA; ++c) a[i][c] = 0.f;
    }
    const int vlast = nvec - 1;
    for (int j = s0; j < s1; j += 4) {  // four steps at a time (x is zero-padded to a whole four steps past the row end)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int vx = lane + 32 * (j + jj);
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

// One tile, worked through by one warp: nr rows of seg_nvec vectors each (row groups of RB), against the
// matching part of x; part points at the tile's first row in the table of partial sums (column = segment).
template <typename WT, int RB>
__device__ __forceinline__ void consume_tile(const MegaParams &p, Shared &sh, const uint4 *st, const float4 *xs4, int stride, int seg_nvec,
                                             int s0, int s1, int lane, int nr, bool have, float *part, int rs, uint32_t slot, int cta) {
    for (int rb = 0; rb < nr; rb += RB) {
        float acc[RB];
        if (have) {
            tile_rows<WT, RB>(st, xs4, stride, seg_nvec, s0, s1, lane, nr, rb, acc);
        } else {
#pragma unroll
            for (int i = 0; i < RB; ++i) acc[i] = 0.f;
        }
        if (rb + RB >= nr) {  // the tile's last loads are done: the stage can go back to the producer
            __syncwarp();
            if (lane == 0 && !(p.debug_flags & 16)) release_stage(p, sh, rs, 1, slot, cta, 0);
        }
        const float s = reduce_rows<RB>(acc, lane);
        const int r = reduce_row_of<RB>(lane);
        if (r >= 0 && rb + r < nr) part[(rb + r) * kPartCols] = s;
    }
}

template <typename WT>
__device__ __forceinline__ bool gemv_phase(const MegaParams &p, Shared &sh, const Phase &g, long id, RingPos &rp, int cta, int nctas,
                                           int tid, int &bk, int ph, float &xres) {
    constexpr int XPV = VecTraits<WT>::XPV;
    const int lane = tid & 31, warp = tid >> 5;
    const MegaLayer *lw = g.layer < p.L ? &p.layers[g.layer] : nullptr;
    const PhaseTiles ti(g, (int)sizeof(WT), sh.stage_bytes, cta, nctas);
    // No rows of this matrix here: nothing to read, nothing to publish - except that the phases which stage
    // the residual stream also refresh the residual value this thread carries for the o_proj / down epilogues.
    const bool has_rows = ti.r0 != ti.r1;
    const bool stages_x = g.kind == PH_QKV || g.kind == PH_GATEUP;
    // (with the two-step tensor-parallel exchange every CTA owes the others the sums of its rows of the residual
    // stream, also in the lm_head phase, where it may have no rows of the matrix)
    const bool owes_sums = p.xrT != nullptr && g.kind == PH_LMHEAD;
    if (!has_rows && !stages_x && !owes_sums) return true;
    const int njl = ti.njl;  // steps of a lane through a whole row

    // ---- prologue: the input vector, in shared memory ---------------------------------------------------
    float *xs = sh.xs;
    float4 *xs4 = reinterpret_cast<float4 *>(xs);
    StageOpts so;
    if (g.kind == PH_QKV) so.gains = lw->norm1;
    else if (g.kind == PH_GATEUP) so.gains = lw->norm2;
    else if (g.kind == PH_LMHEAD) so.gains = p.final_norm;
    const bool normed = so.gains != nullptr;
    const long r0h = (long)p.H * cta / nctas, r1h = (long)p.H * (cta + 1) / nctas;
    if (stages_x) {
        so.xraw = sh.xraw;
        so.r0 = (int)r0h;
        so.r1 = (int)r1h;
    }
    const int njl4 = (njl + 3) & ~3;  // the inner loop takes four steps at a time
    for (int k = g.K + tid; k < njl4 * 32 * XPV; k += kConsumers) xs[k] = 0.f;  // zero padding up to whole blocks of steps
    if (g.kind == PH_QKV && g.layer == 0) {
        // Embedding::forward (embedding.rs:47-57): the token's row is the first layer's input
        float ss = 0.f;
        for (int k = tid; k < g.K / 2; k += kConsumers)
            stage_pair(so, xs, k, embed_elem(p, id, 2 * k), embed_elem(p, id, 2 * k + 1),
                       __ldg(reinterpret_cast<const float2 *>(so.gains) + k), ss);
        publish_ss(sh, ss, tid);
        consumer_bar();
    } else {
        const uint32_t tag = phase_tag(p, ph - 1);  // every phase consumes what the phase before it published
        bool ok;
        // o_proj outputs travel in x buffer 0 (read by gate/up), down outputs in buffer 1 (read by qkv, lm_head)
        const uint2 *xsrc = p.xT + (size_t)(g.kind == PH_GATEUP ? 0 : 1) * p.tp_size * p.x_slot_words;
        if (g.kind == PH_O) ok = poll_attention(p, sh, tag, xs, tid, bk);
        else if (g.kind == PH_DOWN) ok = poll_vector(p, sh, p.actT, g.K, tag, xs, tid, bk, 330 + g.kind);
        else if (p.tp_size == 1) ok = poll_vector(p, sh, xsrc, g.K, tag, xs, tid, bk, 330 + g.kind, so);
        else if (p.xrT)
            ok = reduce_then_poll_x(p, sh, xsrc, p.xrT + (size_t)(g.kind == PH_GATEUP ? 0 : 1) * p.x_slot_words, g.K, tag, xs, tid, bk, (int)r0h,
                                    (int)r1h, so);
        else ok = poll_x_sum(p, sh, xsrc, g.K, tag, xs, tid, bk, so);
        if (!ok) return false;
        if (p.trace && cta == 0 && tid == 0) p.trace[4 * (5 * p.L + 1) + 1 + ph] = globaltimer_ns();
    }
    // RMSNorm::forward (rms_norm.rs:49-56): rms = sqrt(ss/dim + eps), inv = 1/rms.  The vector in shared memory
    // carries the gains; inv multiplies the row sums in the epilogue.
    float inv = 1.f;
    if (normed) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) tot += sh.red[w];
        inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(tot, (float)g.K), p.eps)));
    }
    if (stages_x || owes_sums) {
        // keep this thread's row of the residual stream (all ranks' partial sums added, before the gains)
        if (stages_x && tid < r1h - r0h) xres = sh.xraw[tid];
        if (!has_rows) {
            trace_stamp(p, cta, tid, 3 * ph + 1);
            trace_stamp(p, cta, tid, 3 * ph + 2);
            return true;
        }
    }
    trace_stamp(p, cta, tid, 3 * ph + 1);
    trace_cta(p, cta, tid, 0, ph);

    // ---- tiles ------------------------------------------------------------------------------------------
    // Tiles are addressed in closed form (see PhaseTiles) and sit in ring slot (tiles consumed so far + t).
    // Warp w owns tiles w, w + 4, ...  Rows are reduced and published in blocks of at most kRowBlock (a block
    // never splits a chunk of rows).
    constexpr int XQ = VecTraits<WT>::XQ;
    const int R = ti.R, nmat = ti.nmat, nseg = ti.nseg;
    const int nrows_cta = ti.nrows;
    const int chunks = ((p.debug_flags & 1) && !(p.debug_flags & 16)) ? 0 : ti.chunks;
    const bool dry = (p.debug_flags & 16) != 0;  // debug: no copies are issued (bit 0); run the arithmetic on whatever the ring holds
    const int chunks_per_block = kRowBlock / R;
    const int tpc = nmat * nseg;  // tiles per chunk of rows
    // rows of a segment tile that came as a box sit a whole segment slot apart (the box is zero-filled past the row end)
    const bool boxed = nseg > 1 && p.tmaps != nullptr;
    for (int cb = 0; cb < chunks; cb += chunks_per_block) {
        const int cend = min(chunks, cb + chunks_per_block);
        const int t0 = cb * tpc, t1 = cend * tpc;
        const int row0_blk = cb * R;  // first row of the block, relative to the CTA's first row
        // Warp w owns tiles w, w + W, ... of the phase.  The tile's coordinates and its ring position are carried
        // along incrementally (no divisions in the loop).
        int t = t0 + (warp + kConsumerWarps - t0 % kConsumerWarps) % kConsumerWarps;
        int chunk = t / tpc, mat = (t - chunk * tpc) / nseg, seg = t - chunk * tpc - mat * nseg;
        uint32_t slot = rp.n + (uint32_t)t;
        int rs = (int)(slot % (uint32_t)sh.S);
        uint32_t use = slot / (uint32_t)sh.S;
        for (; t < t1; t += kConsumerWarps) {
            const int rrel = chunk * R;
            const int nr = min(R, nrows_cta - rrel);
            // A parity test tells two phases apart, not three: before testing for use `u` of this stage,
            // use `u-1` (owned by another warp) must be known to have landed.  Its owner publishes that.
            // A failed wait must not leave early (see consumer_bar_ok): skip the math, keep the sequence.
            bool have = dry || stage_use_seen(p, sh, rs, (int)use, 310 + g.kind);
            have = have && (dry || mbar_wait(p, sh, &sh.full[rs], use & 1, 300 + g.kind));
            if (have && lane == 0 && !dry) sh.seen[rs] = (int)use + 1;
            if (p.debug_flags & 4) have = false;  // debug: wait for the tiles but skip the arithmetic
            const uint4 *st = reinterpret_cast<const uint4 *>(sh.stages + (size_t)rs * sh.stage_bytes);
            float *part = sh.part + ((size_t)mat * kRowBlock + (size_t)(rrel - row0_blk)) * kPartCols + seg;
            const int seg_nvec = ti.seg_bytes(seg) / 16;  // valid 16-byte vectors of a row of this tile
            consume_tile<WT, 4>(p, sh, st, xs4 + (size_t)seg * ti.per * 32 * XQ, boxed ? ti.per * 32 : seg_nvec, seg_nvec, 0, ti.seg_steps(seg),
                                lane, nr, have, part, rs, slot, cta);
            // the next tile of this warp
            slot += kConsumerWarps;
            rs += kConsumerWarps;
            while (rs >= sh.S) {
                rs -= sh.S;
                ++use;
            }
            seg += kConsumerWarps;
            while (seg >= nseg) {
                seg -= nseg;
                if (++mat == nmat) {
                    mat = 0;
                    ++chunk;
                }
            }
        }
        // End of a row block: add the warps' partial sums, run the epilogue and publish.
        const int nrows = min(cend * R, nrows_cta) - row0_blk;
        if (!consumer_bar_ok(sh.abort, sh.decision, tid, bk)) return false;
        if (tid < nrows) {
            // the segments of the row, added in order
            const float *pr = sh.part + (size_t)tid * kPartCols;
            float acc = pr[0];
            for (int c = 1; c < nseg; ++c) acc += pr[c];
            const float tot = __fmul_rn(acc, inv);
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
                    const float *pu = sh.part + ((size_t)kRowBlock + tid) * kPartCols;
                    float accu = pu[0];
                    for (int c = 1; c < nseg; ++c) accu += pu[c];
                    const float up = __fmul_rn(accu, inv);
                    const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-tot)));
                    st_tagged(p.actT + row, __fmul_rn(__fmul_rn(tot, sig), up), tag);
                    break;
                }
                default:  // lm_head: this rank's rows of the logits, stored into every rank's gathered copy
                    if (p.tp_size == 1) {
                        p.logits[row] = tot;
                    } else {
                        const size_t grow = (size_t)p.tp_rank * p.V + row;
                        for (int r = 0; r < p.tp_size; ++r) p.logits_peer[r][grow] = tot;
                    }
                    break;
            }
        }
        if (cend < chunks) consumer_bar();  // the table is rewritten by the next block
    }
    rp.n += (uint32_t)(chunks * tpc);
    if ((p.debug_flags & 1) && !dry && ti.r0 + tid < ti.r1) {  // debug (no tiles streamed): publish zeros so that the chain runs
        const uint32_t tag = phase_tag(p, ph);
        uint2 *dst = g.kind == PH_QKV ? p.qkvT : g.kind == PH_GATEUP ? p.actT : p.xT + (size_t)(g.kind == PH_O ? 0 : 1) * p.x_slot_words;
        if (g.kind != PH_LMHEAD) st_tagged(dst + ti.r0 + tid, 0.f, tag);
    }
    trace_stamp(p, cta, tid, 3 * ph + 2);
    trace_cta(p, cta, tid, 1, ph);
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
            if (cta < p.Hq * p.nsplit) trace_cta(p, cta, tid, 1, ph);
        } else {
            if (!gemv_phase<WT>(p, sh, g, id, rp, cta, nctas, tid, bk, ph, xres)) return;
        }
    }
    trace_stamp(p, cta, tid, 3 * nphases);
    if (p.tp_size > 1) {
        // The logits rows of this CTA are on their way to every rank.  The last CTA of the rank to get here tells
        // every rank that this rank's slice is complete, and waits (bounded) for the slices of the others.
        consumer_bar();
        if (tid == 0) {
            __threadfence_system();
            if (atomicAdd(p.done_count, 1u) == (unsigned)nctas - 1u) {
                atomicExch(p.done_count, 0u);
                const uint32_t tag = phase_tag(p, nphases - 1);
                for (int r = 0; r < p.tp_size; ++r)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag_peer[r] + p.tp_rank), "r"(tag) : "memory");
                const long long t0 = clock64();
                for (int r = 0; r < p.tp_size; ++r) {
                    uint32_t v;
                    do {
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.flag_peer[p.tp_rank] + r) : "memory");
                    } while (v != tag && !*sh.abort && clock64() - t0 < kWaitCycles);
                    if (v != tag) {
                        raise_abort(p, sh.abort, 360, r);
                        break;
                    }
                }
            }
        }
    }
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
    __shared__ int issued[kMegaMaxStages];
    Shared sh;
    sh.S = p.stages;
    sh.stage_bytes = p.stage_bytes;
    sh.stages = smem_raw;
    float *fl = reinterpret_cast<float *>(smem_raw + (size_t)p.stages * p.stage_bytes);
    sh.xs = fl;
    sh.part = fl + mega_xs_floats(max(p.H, max(p.qd, p.I)));
    sh.red = fl + mega_table_floats(max(p.H, max(p.qd, p.I)));
    sh.xraw = sh.red + kConsumerWarps;
    sh.attn = sh.xraw + kRowBlock;
    sh.full = bars;
    sh.empty = bars + kMegaMaxStages;
    sh.abort = &abort_flag;
    sh.decision = decision;
    sh.seen = seen;
    sh.issued = issued;
    const int tid = threadIdx.x;
    if (tid == 0) {
        abort_flag = 0;
        decision[0] = decision[1] = 0;
        for (int s = 0; s < kMegaMaxStages; ++s) {
            seen[s] = 0;
            issued[s] = -1;
        }
        for (int s = 0; s < sh.S; ++s) {
            mbar_init(&sh.full[s], 1);                 // the producer's arrive.expect_tx
            mbar_init(&sh.empty[s], 1);                // the warp that worked on the tile
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
           (mega_table_floats(kmax) + kConsumerWarps + kRowBlock + attn_decode_smem_floats(1, head_dim, kConsumerWarps) + 3 * (size_t)head_dim) *
               sizeof(float);
}

int decode_mega_max_splits() { return kMaxSplit; }

int decode_mega_debug_flags() {
    static const int flags = [] {
        const char *e = getenv("LUMEN_MEGA_DEBUG");
        return e ? atoi(e) : 0;
    }();
    return flags;
}

namespace {
// Tensor map over a row-major matrix [rows, rowbytes] seen as 32-bit words [rows][rowbytes / 256][64]: a box of
// box_rows rows x `units` 256-byte units (one segment of the row length), no swizzle, zero fill past the edges.
bool make_segment_map(CUtensorMap *map, const void *base, size_t rows, size_t rowbytes, int units, int box_rows) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = [] {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeFn>(f);
    }();
    if (!fn || rowbytes % 256 || units < 1 || units > 256) return false;
    const cuuint64_t dims[3] = {64, (cuuint64_t)(rowbytes / 256), (cuuint64_t)rows};
    const cuuint64_t strides[2] = {256, (cuuint64_t)rowbytes};
    const cuuint32_t box[3] = {64, (cuuint32_t)units, (cuuint32_t)box_rows};
    const cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

void decode_mega_build_schedule(const MegaParams &p_in, const MegaLayer *host_layers, int grid, std::vector<uint4> &entries,
                                std::vector<int> &counts, int &stride, std::vector<CUtensorMap> &tmaps) {
    MegaParams p = p_in;
    p.debug_flags = decode_mega_debug_flags();
    const int esz = p.wbf16 ? 2 : 4, nphases = 5 * p.L + 1;
    // Tensor maps are all or nothing (the consumers derive the layout of a segment tile from `tmaps != nullptr`):
    // if one cannot be made, the schedule is built again without any.
    bool no_tensor = getenv("LUMEN_MEGA_NO_TENSOR_COPY") != nullptr;
    bool retry = false;
    std::vector<std::vector<uint4>> per;
build:
    tmaps.clear();
    per.assign(grid, std::vector<uint4>());
    for (int ph = 0; ph < nphases; ++ph) {
        const Phase g = get_phase(p, host_layers, ph);
        if (g.kind == PH_ATT) continue;
        // Matrices whose rows are cut into segments get two tensor maps each (boxes of 4 rows and of 1 row).
        int map0[2] = {-1, -1};
        {
            const PhaseTiles pt(g, esz, kMegaStageBytes, 0, grid);
            if (pt.nseg > 1 && !no_tensor) {
                for (int mat = 0; mat < pt.nmat; ++mat) {
                    CUtensorMap m4, m1;
                    const char *w = mat == 0 ? g.w0 : g.w1;
                    if (make_segment_map(&m4, w, (size_t)g.N, (size_t)pt.rowbytes, pt.per * 2, 4) &&
                        make_segment_map(&m1, w, (size_t)g.N, (size_t)pt.rowbytes, pt.per * 2, 1)) {
                        map0[mat] = (int)tmaps.size();
                        tmaps.push_back(m4);
                        tmaps.push_back(m1);
                    } else {
                        retry = true;
                    }
                }
                if (retry) break;
            }
        }
        for (int cta = 0; cta < grid; ++cta) {
            const PhaseTiles pt(g, esz, kMegaStageBytes, cta, grid);
            const int ntiles = (p.debug_flags & 1) ? 0 : pt.tiles();  // debug: stream nothing
            for (int t = 0; t < ntiles; ++t) {
                const int seg = t % pt.nseg, mat = (t / pt.nseg) % pt.nmat, chunk = t / (pt.nseg * pt.nmat);
                const int nr = std::min(pt.R, pt.nrows - chunk * pt.R);
                const long row = pt.r0 + (long)chunk * pt.R;
                const uint32_t phz = (uint32_t)ph << 16;
                if (pt.nseg == 1) {  // whole rows are one contiguous block: one plain copy per tile
                    const unsigned long long a = (unsigned long long)(uintptr_t)((mat == 0 ? g.w0 : g.w1) + (size_t)row * pt.rowbytes);
                    const uint32_t tile_bytes = (uint32_t)nr * (uint32_t)pt.rowbytes;
                    per[cta].push_back(make_uint4((uint32_t)a, (uint32_t)(a >> 32), tile_bytes | phz, tile_bytes));
                    continue;
                }
                // Segments: the rows of a tile sit pt.per * 512 bytes apart in the stage, whatever the segment's length.
                const uint32_t slot_bytes = (uint32_t)pt.per * 512u;
                if (map0[mat] >= 0) {  // one box of four rows, or one box per row for a shorter last chunk
                    const uint32_t unit0 = (uint32_t)(seg * pt.per * 2);
                    if (nr == 4) {
                        per[cta].push_back(make_uint4((uint32_t)map0[mat] | (unit0 << 16), (uint32_t)row, 4u * slot_bytes | phz,
                                                      4u * slot_bytes | 0x80000000u));
                    } else {
                        for (int c = 0; c < nr; ++c)
                            per[cta].push_back(make_uint4((uint32_t)(map0[mat] + 1) | (unit0 << 16), (uint32_t)(row + c), slot_bytes | phz,
                                                          (c == 0 ? (uint32_t)nr * slot_bytes : 0u) | (((uint32_t)c * slot_bytes / 16u) << 16) |
                                                              0x80000000u));
                    }
                } else {  // no tensor maps: one plain copy per row
                    const uint32_t sb = (uint32_t)pt.seg_bytes(seg);
                    const char *w = (mat == 0 ? g.w0 : g.w1) + (size_t)row * pt.rowbytes + (size_t)seg * pt.per * 512;
                    for (int c = 0; c < nr; ++c) {
                        const unsigned long long a = (unsigned long long)(uintptr_t)(w + (size_t)c * pt.rowbytes);
                        per[cta].push_back(make_uint4((uint32_t)a, (uint32_t)(a >> 32), sb | phz,
                                                      (c == 0 ? (uint32_t)nr * sb : 0u) | (((uint32_t)c * sb / 16u) << 16)));
                    }
                }
            }
        }
    }
    if (retry && !no_tensor) {
        no_tensor = true;
        retry = false;
        goto build;
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

size_t decode_mega_logits_offset_words(const MegaParams &p) {
    size_t w = decode_mega_x_words(p) + p.qkv_rows + p.I + (size_t)p.Hq * kMaxSplit * (2 + p.D) + 8;
    if (p.tp_size > 1) w = ((w + 1) & ~(size_t)1) + 2 * (size_t)((p.H + 1) & ~1);  // + the summed residual stream (xrT)
    return (w + 15) & ~(size_t)15;  // 128-byte aligned
}
size_t decode_mega_exchange_words(const MegaParams &p) {
    // tensor parallel: + the gathered logits (f32 [vocab]) and one flag word per rank
    const size_t extra = p.tp_size > 1 ? ((size_t)p.vocab + 1) / 2 + 8 : 0;
    return decode_mega_logits_offset_words(p) + extra;
}

int decode_mega_supported(const MegaParams &p, char *why, size_t why_len) {
    const int esz = p.wbf16 ? 2 : 4;
    const int ks[3] = {p.H, p.qd, p.I};
    for (int k : ks) {
        if ((k * esz) % 16) {
            snprintf(why, why_len, "row of %d elements is not a multiple of 16 bytes", k);
            return 0;
        }
        if (k * esz > kMaxSeg * (kMegaStageBytes / 4)) {
            snprintf(why, why_len, "a row of %d elements is longer than %d segments of %d bytes", k, kMaxSeg, kMegaStageBytes / 4);
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
    // Ring geometry: 16 KB stages (four rows x 4 KB; longer rows arrive in segments), as many as fit beside the
    // scratch areas in the 227 KB a CTA may use.
    p.stage_bytes = kMegaStageBytes;
    const int kmax = std::max(p.H, std::max(p.qd, p.I));
    const size_t budget = 227 * 1024 - 1024;  // static shared (barriers, flags) and alignment slack
    int stages = kMegaMaxStages;
    while (stages > 2 && decode_mega_smem_bytes(stages, p.stage_bytes, p.D, kmax) > budget) --stages;
    p.stages = stages;
    p.debug_flags = decode_mega_debug_flags();
    // Tiles handed to the L2, one at a time, while the ring is full (0: none; at most 64, the entries the producer
    // holds).  Measured on TinyLlama f32, 20 steps after a 32-token prompt: 0 -> 1040 tok/s, 24 -> 1076 (64 steps),
    // 48 -> 1115; a pace of 450 cycles instead of 600 loses again (the prefetches queue up in front of the polls).
    // With 4 or more tensor-parallel ranks the token is bound by the cross-GPU exchanges, a rank's share of the weights is
    // small, and the prefetches only get in the way of the polls: 4 ranks 1466 tok/s with 48, 1599 with none.
    p.l2_ahead = p.tp_size >= 4 ? 0 : 48;
    if (const char *e = getenv("LUMEN_MEGA_L2_AHEAD")) p.l2_ahead = std::max(0, std::min(64, atoi(e)));
    p.pf_pace = (int)kPrefetchPace;
    p.pf_grace = (int)kPrefetchGrace;
    if (const char *e = getenv("LUMEN_MEGA_PF_PACE")) p.pf_pace = std::max(0, atoi(e));
    if (const char *e = getenv("LUMEN_MEGA_PF_GRACE")) p.pf_grace = std::max(0, atoi(e));
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
