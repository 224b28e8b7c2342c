// The fused row-sampling kernel: one launch does penalties -> grammar mask -> row max /
// log-sum-exp -> top-k -> temperature -> min-p -> top-p -> inverse-CDF draw.
//
// Work decomposition.  A row of the [batch, vocab] logits is cut into S contiguous slices;
// CTA (slice, row) streams its slice from HBM exactly once.  One producer warp keeps a ring
// of kStages shared-memory tiles full with 1-D bulk copies (TMA, non-multicast) that
// complete on mbarriers; kThreads compute threads read the tiles with 128-bit shared loads and
// hand each tile back through a second mbarrier.  While streaming the compute threads keep
//   * the running maximum (NaN-propagating) and an online log-sum-exp per thread,
//   * a candidate buffer of rank keys that still can be among the k best.
// A vector group enters the slow path only when its maximum reaches the current threshold
// tau (one compare per 16 bytes); the hits of a warp are collected with ballots into slots
// the warp reserves 32 at a time.  When the buffer fills up, a radix select (shared-memory
// histograms, digit located with a warp scan and ballot) finds the exact k-th best entry,
// the buffer is compacted to k and tau rises.  Since the kept set of every filter is a
// prefix of the rank order, the k best entries of a slice are all that the rest of the
// pipeline needs.
// Each slice leaves a record (max, lse partial, <= k entries) in scratch memory; the last
// CTA of a row to finish (atomic ticket, no spinning) merges the records and runs the
// selection and the draw on exact integer masses.
//
// Greedy selection keeps the reference's tie rule -- the first maximum wins
// (born: internal/nn/cross_entropy.go:241-251) -- through the rank key (value, -index).
#pragma once
#include <float.h>
#include "../../include/born_sampler.h"
#include "spec.cuh"

namespace born {

enum : int { kModeFull = 0, kModeLocal = 1, kModeMerge = 2 };

constexpr int kBlockThreads = kThreads + 32;  // compute threads + the producer warp
constexpr int kHistBuckets = 128;             // history ids are bucketed by tile
constexpr int kPrivPerLane = 4;               // candidate slots every compute thread owns
constexpr int kSmallSet = 256;                // candidate sets up to this size are finished by all-pairs ranking
constexpr int kPrivCap = kPrivPerLane * kThreads;

struct RecordHdr {  // 32 bytes, precedes the entries of a slice / shard record
    float m;        // maximum of the slice (NaN if a NaN was seen)
    float lse_s;    // sum of 2^((z - m) * c2) over the slice
    uint32_t count; // entries that follow
    uint32_t flags; // bit 0: entries were dropped (more than k candidates existed)
    float bound;    // at least k tokens of the slice are at or above this value (-inf: no bound)
    uint32_t pad[3];
};
static_assert(sizeof(RecordHdr) == kRecordHdrBytes, "record header size");

struct SampleKernelArgs {
    const void* logits;
    int64_t row_stride;  // elements
    const uint32_t* mask;
    int64_t mask_stride;  // words
    const int32_t* history;
    const int32_t* history_len;
    int history_stride;
    int B, V;
    const born_row_params* row_params;
    born_row_params params;
    const float* uniforms;
    int32_t* out_token;
    float* out_prob;
    float* out_lse;
    int32_t* out_status;
    int32_t* out_kept_ids;
    int32_t* out_kept_count;
    int kept_stride;
    int mode;
    int S;             // slices (or shards when merging) per row
    int slice_len;     // elements per slice
    int segment_mode;  // 1: each slice keeps its own top-k, the merge takes the union
    int idx_offset;    // added to token indices written to records (shard offset)
    int tma_logits, tma_mask;
    const unsigned long long* ext_total;  // per row: total mass of all survivors (top-p without top-k), or null
    uint8_t* records;  // record (row, slice) at row*rec_row_stride + slice*rec_slice_stride
    int64_t rec_row_stride, rec_slice_stride;
    uint32_t* tickets;
    int* dev_error;
    unsigned long long* prof;  // phase time stamps per CTA (profiling builds only)
};

#ifdef BORN_PROFILE
#define BORN_PROF(i)                                                                                   \
    do {                                                                                               \
        if (A.prof && threadIdx.x == 0)                                                                \
            A.prof[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32 + (i)] = (unsigned long long)clock64(); \
    } while (0)
#define BORN_PROF_T0() long long pt0_ = clock64()
#define BORN_PROF_ACC(var) do { long long pt1_ = clock64(); (var) += pt1_ - pt0_; pt0_ = pt1_; } while (0)
#else
#define BORN_PROF(i) do { } while (0)
#define BORN_PROF_T0() do { } while (0)
#define BORN_PROF_ACC(var) do { } while (0)
#endif

// A pipeline stage holds kTileBytes of logits whatever their type: 4096 fp32 or 8192 bf16.
template <typename T>
struct TileOf { static constexpr int n = kTileBytes / (int)sizeof(T); };

template <typename T>
struct VecOf;
template <>
struct VecOf<float> { static constexpr int n = 4; };
template <>
struct VecOf<uint16_t> { static constexpr int n = 8; };

// Shared-memory layout, computed identically on host and device.
struct SmemLayout {
    int tiles, masks, cand, search, pairs, hist, total;
};
__host__ __device__ inline SmemLayout smem_layout(int elem_bytes, bool has_mask, bool has_hist) {
    SmemLayout L;
    int off = 0;
    L.tiles = off; off += kStages * kTileBytes;
    L.masks = off; off += has_mask ? kStages * (kTileBytes / elem_bytes / 32) * 4 : 0;
    L.cand = off; off += kCandCap * 8;
    // the radix-search scratch and the pairing lists of the compaction are never live together
    L.search = off;
    L.pairs = off;
    {
        const int a = (int)((sizeof(SearchScratch) + 127) / 128 * 128), b = kMaxK * 2 * 2;  // also 2 * kSmallSet * 8
        off += a > b ? a : b;
    }
    L.hist = off; off += has_hist ? kHistCap * 10 : 0;  // ids, replay values, multiplicities
    L.total = off;
    return L;
}

struct BlockShared {  // static shared state of a CTA
    unsigned long long full_bar[kStages];
    unsigned long long empty_bar[kStages];
    unsigned long long ready_bar[kStages];  // tile patched by the producer warp (fp32 rows with penalties)
    unsigned long long tau_ck;
    unsigned long long red64[kThreads / 32];
    unsigned long long acc[4];  // block-wide integer sums of the final selection (shared-memory atomics)
    float redf[kThreads / 32];
    float redf2[kThreads / 32];
    float wbound[kThreads / 32];  // per warp: a lower bound of the k-th largest value (lane maxima)
    uint32_t taubits;  // key of tau; only ever raised (red.max)
    uint32_t maxbits;
    float u_row;     // the row's uniform variate, fetched at the start
    int count;
    int event;       // a compaction is wanted: warps meet at the rendezvous
    int done_warps;  // warps that have finished their tiles
    int fail;
    int dropped;
    int nh;
    int nl, nw, nsw;
    int trig;        // fill of the shared area that asks for a compaction
    int hist_ready;  // the history buckets are built (read by the producer warp)
    int last;
    int hoff[kHistBuckets + 1];
    int hcur[kHistBuckets];
#ifdef BORN_PROFILE
    long long pf_search, pf_pair, pf_calls;
#endif
};

struct ThreadStats {
    float mx;   // running maximum (NaN-propagating)
    float R;    // reference of the online log-sum-exp (z domain)
    float nRc;  // -R * c2
    float2 s;   // two partial sums of 2^((z - R) * c2) (packed fp32x2 arithmetic)
    float pub;  // largest maximum this thread has published for the min-p prune
#ifdef BORN_PROFILE
    long long pf_hit;
#endif
};

struct Ctx {  // per-CTA pointers and row constants, all block-uniform
    uint64_t* cand;
    SearchScratch* sc;
    uint16_t* lslot;
    uint16_t* wpos;
    int32_t* hlist;
    float* hval;
    uint16_t* hcnt;  // multiplicity of a history id, 0 for repeats of an id already listed
    BlockShared* bs;
    int k_eff;
    int trigger;
    int psize;  // entries of the buffer that are thread-private slots (kPrivCap while streaming, 0 after)
    int hshift;  // history bucket of tile c is c >> hshift
    float c2;
    float delta_minp;
    bool minp_on;
    born_row_params rp;
#ifdef BORN_PROFILE
    unsigned long long* pr;  // this CTA's profiling record
#endif
};

// The candidate buffer.  The first cx.psize entries are private slots: thread t owns entries
// t, t+kThreads, ... and fills them in that order, counting in a register (no atomic, no
// waiting for a slot number); the rest is a shared area filled through the atomic counter
// bs.count, used by lanes whose private slots are full.  A thread that walks the buffer as
// i = tid, tid+kThreads, ... meets exactly its own private slots, so it can tell the filled ones
// from its register.  Unfilled slots read as dead entries (value part 0, unique low bits).
// Private slots are not filtered by the exact rank-key threshold when they are written (the
// hot path only compares values); what does not belong is dropped when the buffer is read.
struct LanePriv {
    int pcnt;  // filled private slots of this thread
};

// Private slots hold the raw pair (float bits << 32 | token index) exactly as the hot loop
// stored it; the rank key is formed when a slot is read (cold paths only).
__device__ __forceinline__ uint64_t raw_to_ck(uint64_t raw) {
    return make_ck(__uint_as_float((uint32_t)(raw >> 32)), (int)(uint32_t)raw);
}
__device__ __forceinline__ uint64_t slot_key(const Ctx& cx, const LanePriv& lp, int i, int scount) {
    if (i < cx.psize) return ((i / kThreads) < lp.pcnt) ? raw_to_ck(cx.cand[i]) : (uint64_t)i;
    return (i - cx.psize < scount) ? cx.cand[i] : (uint64_t)i;
}

// Keep the k best entries of the buffer (exact, by rank key) and raise tau.  Private entries
// stay with their owners, the shared area is compacted in place.  Returns true when entries
// were dropped.
__device__ __forceinline__ bool compact_to_k_body(Ctx& cx, LanePriv& lp, int k) {
    BlockShared& bs = *cx.bs;
    const int tid = threadIdx.x;
    cta_sync();
    const int sc = min(bs.count, kCandCap - cx.psize);
    if (tid == 0) { bs.nl = 0; bs.nw = 0; bs.nsw = 0; }
    cta_sync();
    if (lp.pcnt) smem_red_add(&bs.nl, (uint32_t)lp.pcnt);
    cta_sync();
    const int total = bs.nl + sc;
    cta_sync();
    if (total <= k) {
        if (tid == 0 && bs.count > sc) bs.count = sc;  // refused appends only inflated the counter
        cta_sync();
        return false;
    }
    uint64_t* cand = cx.cand;
#ifdef BORN_PROFILE
    long long pf0 = clock64();
#endif
    const uint64_t T = block_radix_search<true, 56, true>(
        kCandCap, (unsigned long long)(k - 1), [&](int i) { return slot_key(cx, lp, i, sc); },
        [&](int) { return 1ull; }, *cx.sc);
#ifdef BORN_PROFILE
    long long pf1 = clock64();
#endif
    // private entries: every thread filters its own
    int np = 0;
    for (int s = 0; s < lp.pcnt; ++s) {
        const uint64_t raw = cand[s * kThreads + tid];
        if (raw_to_ck(raw) >= T) cand[(np++) * kThreads + tid] = raw;
    }
    lp.pcnt = np;
    // shared area: survivors to the front
    uint64_t* sh = cand + cx.psize;
    if (tid == 0) { bs.nl = 0; bs.nw = 0; }
    for (int i = tid; i < sc; i += kThreads)
        if (sh[i] >= T) smem_red_add(&bs.nsw, 1u);
    cta_sync();
    const int w = bs.nsw;
    for (int i = tid; i < sc; i += kThreads) {
        const uint64_t c = sh[i];
        if (i < w) {
            if (c < T) cx.lslot[smem_atom_add(&bs.nl, 1u)] = (uint16_t)i;
        } else if (c >= T) {
            cx.wpos[smem_atom_add(&bs.nw, 1u)] = (uint16_t)i;
        }
    }
    cta_sync();
    const int nl = bs.nl;
    for (int j = tid; j < nl; j += kThreads) sh[cx.lslot[j]] = sh[cx.wpos[j]];
    if (tid == 0) {
        bs.count = w;
        bs.trig = min(max(w + 256, cx.trigger), kCandCap - cx.psize - 64);
        if (ck_alive(T)) {
            bs.tau_ck = T;
            smem_red_max(&bs.taubits, (uint32_t)(T >> 24));
        }
        bs.dropped = 1;
#ifdef BORN_PROFILE
        bs.pf_search += pf1 - pf0; bs.pf_pair += clock64() - pf1; bs.pf_calls += 1000000 + total;
#endif
    }
    cta_sync();
    return true;
}

// The compaction takes its state by value -- the few pointers it needs, and the thread's
// count of filled private slots in and out.  (Measured: as a real out-of-line function it
// shrinks the kernel by 140 KB of code but the call ABI costs the streaming loop 15 %.)
__device__ __forceinline__ uint32_t compact_to_k_cold(BlockShared* bs, uint64_t* cand, SearchScratch* sc, uint16_t* lslot,
                                                   int psize, int trigger, int pcnt, int k) {
    Ctx cx;
    cx.bs = bs; cx.cand = cand; cx.sc = sc; cx.lslot = lslot; cx.wpos = lslot + kMaxK;
    cx.psize = psize; cx.trigger = trigger;
    LanePriv lp;
    lp.pcnt = pcnt;
    const bool dropped = compact_to_k_body(cx, lp, k);
    return (uint32_t)lp.pcnt | (dropped ? 0x100u : 0u);
}
__device__ __forceinline__ bool compact_to_k(const Ctx& cx, LanePriv& lp, int k) {
    const uint32_t r = compact_to_k_cold(cx.bs, cx.cand, cx.sc, cx.lslot, cx.psize, cx.trigger, lp.pcnt, k);
    lp.pcnt = (int)(r & 0xffu);
    return (r >> 8) != 0;
}

template <bool kLse>
__device__ __forceinline__ void stats_one(ThreadStats& st, float z, float c2) {
    st.mx = max_nan(st.mx, z);
    if (kLse) {
        if (z > st.R) {
            { const float f = ex2_approx(__fmul_rn(st.R - z, c2)); st.s.x *= f; st.s.y *= f; }
            st.R = z;
            st.nRc = -z * c2;
        }
        st.s.x += ex2_approx(fmaf(z, c2, st.nRc));
    }
}

// 16 bytes of the tile as floats, grammar mask applied.
template <typename T, bool kHasMask>
__device__ __forceinline__ void load_group(const T* tile, const uint32_t* smask, int g, int nvalid,
                                           float (&v)[VecOf<T>::n]) {
    constexpr int VEC = VecOf<T>::n;
    if constexpr (VEC == 4) {
        float4 q = reinterpret_cast<const float4*>(tile)[g];
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
        uint4 q = reinterpret_cast<const uint4*>(tile)[g];
        v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xFFFF0000u);
        v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xFFFF0000u);
        v[4] = __uint_as_float(q.z << 16); v[5] = __uint_as_float(q.z & 0xFFFF0000u);
        v[6] = __uint_as_float(q.w << 16); v[7] = __uint_as_float(q.w & 0xFFFF0000u);
    }
    if constexpr (kHasMask) {
        const int e = g * VEC;
        uint32_t bits = smask[e >> 5] >> (e & 31);
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = ((bits >> i) & 1u) ? v[i] : -INFINITY;
    }
    if (nvalid < TileOf<T>::n) {  // last tile of the row: nothing beyond the row counts
#pragma unroll
        for (int i = 0; i < VEC; ++i)
            if (g * VEC + i >= nvalid) v[i] = -INFINITY;
    }
}

__device__ __forceinline__ float max3_nan(float a, float b, float c) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Maximum of one vector group (NaN-propagating).
template <int VEC>
__device__ __forceinline__ float group_max(const float (&v)[VEC]) {
    if constexpr (VEC == 4) {
        return max_nan(max3_nan(v[0], v[1], v[2]), v[3]);
    } else {
        return max3_nan(max3_nan(v[0], v[1], v[2]), max3_nan(v[3], v[4], v[5]), max_nan(v[6], v[7]));
    }
}

// Online log-sum-exp of a thread's share of one tile.  The running reference st.R moves at
// most once per tile (to the share's maximum mt), then every term is formed two at a time
// with packed fp32x2 multiply-adds and adds, in two independent chains.  It feeds no decision.
template <int ITER, int VEC>
__device__ __forceinline__ void tile_lse(ThreadStats& st, const float (&v)[ITER][VEC], float mt, float c2) {
    if (mt > st.R) {
        const float f = ex2_approx(__fmul_rn(st.R - mt, c2));
        st.s = __fmul2_rn(st.s, make_float2(f, f));
        st.R = mt;
        st.nRc = -mt * c2;
    }
    const float2 cc = make_float2(c2, c2), rr = make_float2(st.nRc, st.nRc);
    float2 s1 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < ITER; ++j) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
            const float2 t0 = __ffma2_rn(make_float2(v[j][i], v[j][i + 1]), cc, rr);
            const float2 t1 = __ffma2_rn(make_float2(v[j][i + 2], v[j][i + 3]), cc, rr);
            st.s = __fadd2_rn(st.s, make_float2(ex2_approx(t0.x), ex2_approx(t0.y)));
            s1 = __fadd2_rn(s1, make_float2(ex2_approx(t1.x), ex2_approx(t1.y)));
        }
    }
    st.s = __fadd2_rn(st.s, s1);
}

// Rendezvous of the compute threads.  Warps stream their tiles without any block-wide
// barrier; only a rare event (the candidate buffer reached its trigger or is full) brings
// them together.  A warp comes here when it sees bs.event at a tile boundary, when one of
// its lanes cannot get buffer space, or when it has finished all its tiles; the buffer is
// compacted if an event is pending.  Returns true when every warp has finished and no event
// was pending.
__device__ __forceinline__ bool rendezvous_body(Ctx& cx, LanePriv& lp) {
    BlockShared& bs = *cx.bs;
    cta_sync();
    const int ev = bs.event, dn = bs.done_warps;
    cta_sync();
    if (ev) {
        compact_to_k(cx, lp, cx.k_eff);
        if (threadIdx.x == 0) bs.event = 0;
        cta_sync();
    }
    return !ev && dn == kThreads / 32;
}
// Wrappers that pass the per-thread state by value (the count of filled private slots goes in
// and comes back in the return value), so that nothing of the caller's registers has its
// address taken should the compiler decide not to inline the body.
__device__ __forceinline__ uint32_t rendezvous_cold(const Ctx* sh, int pcnt) {
    Ctx cx = *sh;
    LanePriv lp;
    lp.pcnt = pcnt;
    const bool done = rendezvous_body(cx, lp);
    return (uint32_t)lp.pcnt | (done ? 0x100u : 0u);
}
__device__ __forceinline__ bool rendezvous(const Ctx& cx, LanePriv& lp) {
    const uint32_t r = rendezvous_cold(&cx, lp.pcnt);
    lp.pcnt = (int)(r & 0xffu);
    return (r >> 8) != 0;
}

// One candidate from the lane that found it: exact rank-key test, then a store into the
// lane's next private slot -- no atomic, nothing to wait for.  A lane whose private slots are
// full takes a slot of the shared area with a shared-memory atomic.  Returns false when that
// area is full too (the caller keeps the element for the retry after the compaction).
__device__ __forceinline__ bool lane_put_shared(const Ctx* sh, uint64_t ck) {
    BlockShared* bs = sh->bs;
    if (!(ck > bs->tau_ck)) return true;  // cannot be among the k best any more
    const int psize = sh->psize;
    const int scap = kCandCap - psize;
    const int pos = (int)smem_atom_add(&bs->count, 1u);
    if (pos < scap) {
        sh->cand[psize + pos] = ck;
        if (pos + 1 > bs->trig) bs->event = 1;  // compaction at the next tile boundary
        return true;
    }
    bs->event = 1;
    return false;
}
// The hot-path store: value bits and token index as one 8-byte shared store into the lane's
// next private slot; only a lane whose slots are full goes through the shared area.
__device__ __forceinline__ bool lane_put(Ctx& cx, LanePriv& lp, float z, int idx) {
    if (lp.pcnt < kPrivPerLane && cx.psize) {
        reinterpret_cast<uint2*>(cx.cand)[lp.pcnt * kThreads + threadIdx.x] = make_uint2((uint32_t)idx, __float_as_uint(z));
        ++lp.pcnt;
        return true;
    }
    return lane_put_shared(&cx, make_ck(z, idx));
}
__device__ __forceinline__ bool lane_put_ck(Ctx& cx, LanePriv& lp, uint64_t ck) {
    // history tokens (cold): straight to the shared area, which holds rank keys
    (void)lp;
    return lane_put_shared(&cx, ck);
}

// One offer per lane, called by the whole warp (history tokens): lanes that find the buffer
// full take the warp to the rendezvous and try again after the compaction.
__device__ __forceinline__ void settle_one(Ctx& cx, LanePriv& lp, bool pending, uint64_t ck) {
    for (;;) {
        if (pending && lane_put_ck(cx, lp, ck)) pending = false;
        if (!__any_sync(0xffffffffu, pending)) break;
        rendezvous(cx, lp);
    }
}

// Rare path: some lane found the buffer full.  The warp goes to the rendezvous for the
// compaction; the lanes then offer the elements they kept back (bit j*VEC+i of `ovf`), read
// again from the tile the warp still holds.
template <typename T>
__device__ __forceinline__ void warp_retry_body(Ctx& cx, LanePriv& lp, const T* tile, uint32_t ovf, int c0) {
    constexpr int VEC = VecOf<T>::n;
    for (;;) {
        uint32_t m = ovf;
        ovf = 0;
        while (m) {
            const int b = __ffs(m) - 1;
            m &= m - 1;
            const int e = (threadIdx.x + kThreads * (b / VEC)) * VEC + (b % VEC);
            float z;
            if constexpr (sizeof(T) == 4) z = reinterpret_cast<const float*>(tile)[e];
            else z = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(tile)[e]);
            if (!lane_put(cx, lp, z, c0 + e)) ovf |= 1u << b;
        }
        if (!__any_sync(0xffffffffu, ovf != 0)) break;
        rendezvous(cx, lp);  // the buffer is full: compaction, then offer again
    }
}

template <typename T>
__device__ __forceinline__ uint32_t warp_retry_cold(const Ctx* sh, int pcnt, const T* tile, uint32_t ovf, int c0) {
    Ctx cx = *sh;
    LanePriv lp;
    lp.pcnt = pcnt;
    warp_retry_body<T>(cx, lp, tile, ovf, c0);
    return (uint32_t)lp.pcnt;
}
template <typename T>
__device__ __forceinline__ void warp_retry(const Ctx& cx, LanePriv& lp, const T* tile, uint32_t ovf, int c0) {
    lp.pcnt = (int)warp_retry_cold<T>(&cx, lp.pcnt, tile, ovf, c0);
}

// Penalised logit of a history token (once per distinct token, `cnt` = its multiplicity).
__device__ __forceinline__ float penalise(const born_row_params& rp, float z, int cnt) {
    if (rp.repetition_penalty != 1.0f && rp.repetition_penalty != 0.0f)
        z = (z > 0.0f) ? __fdiv_rn(z, rp.repetition_penalty) : __fmul_rn(z, rp.repetition_penalty);
    if (rp.frequency_penalty != 0.0f || rp.presence_penalty != 0.0f) {
        float pen = __fmul_rn(rp.frequency_penalty, (float)cnt);
        pen = __fadd_rn(pen, rp.presence_penalty);
        z = __fsub_rn(z, pen);
    }
    return z;
}

// History tokens of this tile that fall on elements this warp owns (the warp that reads a
// vector group is the only one that ever touches it, so no other warp is involved): the
// token's logit is penalised once per distinct token, the token is taken out of the tile
// (-inf) and its new value goes through the statistics and the candidate test on its own.
// Entries are bucketed by tile and carry their multiplicity (repeats carry 0).
template <typename T, bool kHasMask, bool kLse>
__device__ __forceinline__ void warp_patch_body(Ctx& cx, ThreadStats& st, LanePriv& lp, T* tile, const uint32_t* smask,
                                                int c, int c0, int nvalid, float tau, bool stats, bool collect,
                                                int replay) {
    // replay: 0 = patch, take statistics and collect in one go; 1 = patch and take statistics,
    // remember the new values; 2 = collect from the remembered values (first tile of a slice,
    // whose candidates are collected only after the threshold bootstrap)
    constexpr int VEC = VecOf<T>::n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = c >> cx.hshift;
    const int lo = cx.bs->hoff[b], hi = cx.bs->hoff[b + 1];
    bool wrote = false;
    for (int base = lo; base < hi; base += 32) {
        const int i = base + lane;
        float z = -INFINITY;
        int id = -1;
        bool first = false;
        if (i < hi) {
            id = cx.hlist[i];
            const int off = id - c0;
            const int cnt = cx.hcnt[i];  // 0: a repeat of an id listed earlier
            if (cnt > 0 && off >= 0 && off < nvalid && (((off / VEC) % kThreads) >> 5) == warp) {
                first = true;
                if (first && replay == 2) {
                    z = cx.hval[i];
                } else if (first) {
                    if constexpr (sizeof(T) == 4) z = reinterpret_cast<float*>(tile)[off];
                    else z = bf16_bits_to_f32(reinterpret_cast<uint16_t*>(tile)[off]);
                    z = penalise(cx.rp, z, cnt);
                    if constexpr (kHasMask) {
                        if (!((smask[off >> 5] >> (off & 31)) & 1u)) z = -INFINITY;
                    }
                    if constexpr (sizeof(T) == 4) reinterpret_cast<float*>(tile)[off] = -INFINITY;
                    else reinterpret_cast<uint16_t*>(tile)[off] = 0xFF80u;
                    wrote = true;
                    if (replay == 1) cx.hval[i] = z;
                }
            }
        }
        if (first && stats) stats_one<kLse>(st, z, cx.c2);
        if (collect) {
            uint64_t ck = 0;
            bool pred = first && z >= tau;
            if (pred) { ck = make_ck(z, id); pred = ck > cx.bs->tau_ck; }
            settle_one(cx, lp, pred, ck);
        }
    }
    if (wrote) fence_proxy_async();
    __syncwarp();
}

// Tiles that hold history tokens of a row whose tiles the producer cannot patch.  The
// statistics of the patched values come back as (their maximum, the sum of
// 2^((z - maximum) * c2)) and are merged by the caller.
template <typename T, bool kHasMask, bool kLse>
__device__ __forceinline__ unsigned long long warp_patch_cold(const Ctx* sh, LanePriv& lp, T* tile, const uint32_t* smask,
                                                           int c, int c0, int nvalid, float tau, int flags) {
    Ctx cx = *sh;
    ThreadStats ps;
    ps.mx = -INFINITY; ps.R = -1e30f; ps.nRc = 1e30f * cx.c2; ps.s = make_float2(0.0f, 0.0f); ps.pub = -INFINITY;
    warp_patch_body<T, kHasMask, kLse>(cx, ps, lp, tile, smask, c, c0, nvalid, tau, (flags & 1) != 0, (flags & 2) != 0, flags >> 2);
    // the sum is relative to the largest patched value when that is above -1e30 (else it is 0)
    return ((unsigned long long)__float_as_uint(ps.s.x + ps.s.y) << 32) | __float_as_uint(ps.mx);
}
template <typename T, bool kHasMask, bool kLse>
__device__ __forceinline__ void warp_patch(const Ctx& cx, ThreadStats& st, LanePriv& lp, T* tile, const uint32_t* smask,
                                           int c, int c0, int nvalid, float tau, bool stats, bool collect, int replay) {
    const unsigned long long r = warp_patch_cold<T, kHasMask, kLse>(&cx, lp, tile, smask, c, c0, nvalid, tau,
                                                                    (stats ? 1 : 0) | (collect ? 2 : 0) | (replay << 2));
    if (stats) {
        const float pm = __uint_as_float((uint32_t)r), psum = __uint_as_float((uint32_t)(r >> 32));
        st.mx = max_nan(st.mx, pm);
        if constexpr (kLse) {
            if (pm > -1e30f) {  // some patched value is finite (NaN fails the test, the row fails anyway)
                if (pm > st.R) {
                    const float f = ex2_approx(__fmul_rn(st.R - pm, cx.c2));
                    st.s = __fmul2_rn(st.s, make_float2(f, f));
                    st.R = pm;
                    st.nRc = -pm * cx.c2;
                }
                st.s.x += psum * ex2_approx(fmaf(pm, cx.c2, st.nRc));
            }
        }
    }
}

__device__ __forceinline__ float current_tau(const Ctx& cx) {
    float tau = zkey_to_float(*reinterpret_cast<const volatile uint32_t*>(&cx.bs->taubits));
    if (cx.minp_on) tau = fmaxf(tau, zkey_to_float(*reinterpret_cast<const volatile uint32_t*>(&cx.bs->maxbits)) + cx.delta_minp);
    return tau;
}

// Running maximum for the min-p prune: a thread publishes only when its own maximum has
// grown past what it published before (rare after the first tiles).
__device__ __forceinline__ void publish_max(Ctx& cx, ThreadStats& st) {
    if (st.mx > st.pub) {
        st.pub = st.mx;
        smem_red_max(&cx.bs->maxbits, zkey(st.mx));
    }
}

// One tile for one warp, no block synchronisation: history patches on the warp's own
// elements, one pass over the thread's vector groups for the statistics and a
// one-compare-per-group candidate test, then at most one collection step.
template <typename T, bool kHasMask, bool kLse>
__device__ __forceinline__ void process_tile(Ctx& cx, ThreadStats& st, LanePriv& lp, T* tile, const uint32_t* smask,
                                             int c, int c0, int nvalid, bool tile_hist, bool stats, bool collect,
                                             int replay = 0) {
    constexpr int VEC = VecOf<T>::n;
    constexpr int ITER = TileOf<T>::n / VEC / kThreads;
    const float tau = current_tau(cx);
    if (tile_hist) warp_patch<T, kHasMask, kLse>(cx, st, lp, tile, smask, c, c0, nvalid, tau, stats, collect, replay);
    uint32_t ovf = 0;  // elements that found the buffer full (bit j*VEC+i)
    // the thread's groups are taken GB at a time (16 values in registers): all of a batch is
    // loaded before anything depends on it, and it costs one statistics update and one
    // candidate test
    constexpr int GB = 16 / VEC, NB = ITER / GB;
#ifdef BORN_PROFILE
    const long long ph0 = clock64();
#endif
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        float v[GB][VEC], m[GB];
#pragma unroll
        for (int j = 0; j < GB; ++j) load_group<T, kHasMask>(tile, smask, threadIdx.x + kThreads * (h * GB + j), nvalid, v[j]);
#pragma unroll
        for (int j = 0; j < GB; ++j) m[j] = group_max<VEC>(v[j]);
        float mt = m[0];
#pragma unroll
        for (int j = 1; j < GB; ++j) mt = max_nan(mt, m[j]);
        if (stats) {
            st.mx = max_nan(st.mx, mt);
            if constexpr (kLse) tile_lse<GB, VEC>(st, v, mt, cx.c2);
        }
        if (collect && mt >= tau) {  // rare per lane
#pragma unroll
            for (int j = 0; j < GB; ++j) {
                if (m[j] >= tau) {
                    const int g = threadIdx.x + kThreads * (h * GB + j);
#pragma unroll
                    for (int i = 0; i < VEC; ++i)
                        if (v[j][i] >= tau && !lane_put(cx, lp, v[j][i], c0 + g * VEC + i)) ovf |= 1u << ((h * GB + j) * VEC + i);
                }
            }
        }
        __syncwarp();
    }
#ifdef BORN_PROFILE
    st.pf_hit += clock64() - ph0;
#endif
    if (collect && __any_sync(0xffffffffu, ovf != 0)) warp_retry<T>(cx, lp, tile, ovf, c0);
}

// The streaming loop's tile: full tiles of rows whose history (if any) the producer has
// already applied.  Straight-line code -- loads, maxima, log-sum-exp, and a candidate test
// that fails for almost every thread; a hit goes into the lane's private slots and only
// when those are full is the element reported back (bit j*VEC+i of the result) for the
// caller to settle outside the loop.
template <typename T, bool kHasMask, bool kLse>
__device__ __forceinline__ uint32_t fast_tile(const Ctx& cx, ThreadStats& st, LanePriv& lp, const T* tile,
                                              const uint32_t* smask, int c0, float tau) {
    constexpr int VEC = VecOf<T>::n;
    constexpr int ITER = TileOf<T>::n / VEC / kThreads;
    constexpr int GB = 16 / VEC, NB = ITER / GB;  // groups per batch of 16 values, batches per tile
    uint32_t ovf = 0;
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        float v[GB][VEC], m[GB];
#pragma unroll
        for (int j = 0; j < GB; ++j)
            load_group<T, kHasMask>(tile, smask, threadIdx.x + kThreads * (h * GB + j), TileOf<T>::n, v[j]);
#pragma unroll
        for (int j = 0; j < GB; ++j) m[j] = group_max<VEC>(v[j]);
        float mt = m[0];
#pragma unroll
        for (int j = 1; j < GB; ++j) mt = max_nan(mt, m[j]);
        st.mx = max_nan(st.mx, mt);
        if constexpr (kLse) tile_lse<GB, VEC>(st, v, mt, cx.c2);
        if (mt >= tau) {  // rare per lane
#pragma unroll
            for (int j = 0; j < GB; ++j) {
                if (m[j] >= tau) {
                    const int g = threadIdx.x + kThreads * (h * GB + j);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        if (v[j][i] >= tau) {
                            if (lp.pcnt < kPrivPerLane) {
                                reinterpret_cast<uint2*>(cx.cand)[lp.pcnt * kThreads + threadIdx.x] =
                                    make_uint2((uint32_t)(c0 + g * VEC + i), __float_as_uint(v[j][i]));
                                ++lp.pcnt;
                            } else {
                                ovf |= 1u << ((h * GB + j) * VEC + i);
                            }
                        }
                    }
                }
            }
        }
    }
    __syncwarp();
    return ovf;
}

// Lane-maxima bound.  Every lane's running maximum belongs to a different token, so the
// j-th largest of a warp's 32 lane maxima has at least j tokens at or above it; with
// j = ceil(k / #warps) the smallest of the warps' values has at least k tokens at or above
// it and is a valid lower bound of the row's k-th largest value -- no sorting, no barrier.
// It tracks the true k-th value closely because the best k tokens rarely share a lane.
// Each warp publishes its value; tau is raised to the minimum over the warps (values of
// warps that have not caught up are older, hence lower, hence still valid).
__device__ __forceinline__ void publish_lane_bound_cold(BlockShared* bsp, int k_eff, float mx) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float v = (mx == mx) ? mx : -INFINITY;
    uint32_t key = zkey(v);
    const int j = (k_eff + kThreads / 32 - 1) / (kThreads / 32);
    uint32_t kj;
    if (j == 1) {
        kj = __reduce_max_sync(0xffffffffu, key);
    } else {
        // warp bitonic sort, descending by lane: 15 compare-exchange steps, one shuffle each
#pragma unroll
        for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
            for (int d = k >> 1; d > 0; d >>= 1) {
                const uint32_t other = __shfl_xor_sync(0xffffffffu, key, d);
                const bool up = ((lane & k) == 0);          // this run is sorted descending
                const bool lower = ((lane & d) == 0);        // lower lane of the pair
                key = (up == lower) ? max(key, other) : min(key, other);
            }
        }
        kj = __shfl_sync(0xffffffffu, key, j - 1);
    }
    const float w = zkey_to_float(kj);
    if (k_eff == 1) {  // any single token is a bound for k = 1: take the best one
        if (lane == 0 && w > -FLT_MAX) smem_red_max(&bsp->taubits, kj);
        return;
    }
    if (lane == 0) *reinterpret_cast<volatile float*>(&bsp->wbound[warp]) = w;
    __syncwarp();
    float m = *reinterpret_cast<const volatile float*>(&bsp->wbound[0]);
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) m = fminf(m, *reinterpret_cast<const volatile float*>(&bsp->wbound[i]));
    if (lane == 0 && m > -FLT_MAX) smem_red_max(&bsp->taubits, zkey(m));
}

__device__ __forceinline__ void publish_lane_bound(const Ctx& cx, const ThreadStats& st) {
    publish_lane_bound_cold(cx.bs, cx.k_eff, st.mx);
}

// After the statistics of the first tile (block-wide, once per slice): open the threshold
// from the lane maxima and the min-p prune from the tile's maximum.
__device__ __forceinline__ void bootstrap_threshold(Ctx& cx, ThreadStats& st) {
    if (cx.minp_on) publish_max(cx, st);
    if (cx.k_eff <= kThreads) {
        publish_lane_bound(cx, st);
        cta_sync();
        publish_lane_bound(cx, st);  // now every warp's value is there
        if (threadIdx.x == 0) cx.bs->dropped = 1;
    }
    cta_sync();
}

// Token history of this slice, bucketed by tile (counting sort: histogram, scan, scatter).
__device__ __forceinline__ int bucket_history_body(Ctx& cx, const int (&hid)[kHistCap / kThreads], int len, int e_begin, int e_end, int tile_elems) {
    // the ids are in registers already (thread t holds ids t, t + kThreads, ...); the bucket
    // counters were cleared before the CTA's first barrier
    BlockShared& bs = *cx.bs;
    const int tid = threadIdx.x;
    int bkt[kHistCap / kThreads];
#pragma unroll
    for (int k = 0; k < kHistCap / kThreads; ++k) {
        const int id = hid[k];
        const bool in = (tid + k * kThreads < len) && (id >= e_begin && id < e_end);
        bkt[k] = in ? (((id - e_begin) / tile_elems) >> cx.hshift) : -1;
        if (in) smem_red_add(&bs.hcur[bkt[k]], 1u);
    }
    cta_sync();
    if (tid < 32) {  // exclusive scan over the 128 bucket counts, 4 per lane
        int v[4], s = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) { v[j] = bs.hcur[4 * tid + j]; s += v[j]; }
        int incl = s;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int up = __shfl_up_sync(0xffffffffu, incl, d);
            if (tid >= d) incl += up;
        }
        int run = incl - s;
#pragma unroll
        for (int j = 0; j < 4; ++j) { bs.hoff[4 * tid + j] = run; bs.hcur[4 * tid + j] = run; run += v[j]; }
        if (tid == 31) bs.hoff[kHistBuckets] = run;
    }
    cta_sync();
#pragma unroll
    for (int k = 0; k < kHistCap / kThreads; ++k)
        if (bkt[k] >= 0) cx.hlist[smem_atom_add(&bs.hcur[bkt[k]], 1u)] = hid[k];
    cta_sync();
    // multiplicity of every id within its bucket; repeats of an id are marked with 0
    const int total = bs.hoff[kHistBuckets];
    for (int i = tid; i < total; i += kThreads) {
        const int id = cx.hlist[i];
        const int b = ((id - e_begin) / tile_elems) >> cx.hshift;
        const int lo = bs.hoff[b], hi = bs.hoff[b + 1];
        int cnt = 0;
        bool first = true;
        for (int j = lo; j < hi; ++j) {
            const bool eq = (cx.hlist[j] == id);
            cnt += eq ? 1 : 0;
            if (eq && j < i) first = false;
        }
        cx.hcnt[i] = first ? (uint16_t)cnt : (uint16_t)0;
    }
    cta_sync();
    return total;
}

__device__ __forceinline__ int bucket_history(const Ctx* sh, const int (&hid)[kHistCap / kThreads], int len, int e_begin, int e_end, int tile_elems) {
    Ctx cx = *sh;
    return bucket_history_body(cx, hid, len, e_begin, e_end, tile_elems);
}

template <typename T, bool kHasMask, bool kLse>
__global__ void __launch_bounds__(kBlockThreads, 2) sample_kernel(const SampleKernelArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ BlockShared bs;
    const int tid = threadIdx.x;
    const int row = blockIdx.y, slice = blockIdx.x;
    const bool hist_arg = A.history != nullptr;
    const SmemLayout L = smem_layout((int)sizeof(T), kHasMask, hist_arg);

    // geometry of this CTA's slice (needed by the producer warp as well)
    const int e_begin = slice * A.slice_len;
    const int e_end = min(A.V, e_begin + A.slice_len);
    const int nelem = max(0, e_end - e_begin);
    constexpr int kChunk = TileOf<T>::n;  // logits per pipeline stage
    const int nchunks = (A.mode == kModeMerge) ? 0 : (nelem + kChunk - 1) / kChunk;
    const T* grow = reinterpret_cast<const T*>(A.logits) + (int64_t)row * A.row_stride + e_begin;
    const uint32_t* gmask = kHasMask ? A.mask + (int64_t)row * A.mask_stride + (e_begin >> 5) : nullptr;
    T* tiles = reinterpret_cast<T*>(smem + L.tiles);
    uint32_t* masks = reinterpret_cast<uint32_t*>(smem + L.masks);
    const bool tma_l = A.tma_logits != 0, tma_m = kHasMask && A.tma_mask != 0;
    const bool use_bar = (A.mode != kModeMerge) && (tma_l || tma_m);

    // Everything the CTA needs from global memory besides the logits is asked for now, so
    // that the round trips overlap each other and the barrier set-up instead of queueing up
    // in front of the first tile and behind the last one.
    const born_row_params rp0 = A.row_params ? A.row_params[row] : A.params;
    const float u_row0 = (A.uniforms && tid == 0) ? A.uniforms[row] : 0.0f;  // parked in shared memory below
    int hist_len0 = 0;
    int hid[kHistCap / kThreads];
#pragma unroll
    for (int k = 0; k < kHistCap / kThreads; ++k) hid[k] = -1;
    if (hist_arg && tid < kThreads && A.mode != kModeMerge) {
        hist_len0 = A.history_len ? A.history_len[row] : A.history_stride;
        const int32_t* gh = A.history + (int64_t)row * A.history_stride;
        const int cap = min(A.history_stride, kHistCap);
#pragma unroll
        for (int k = 0; k < kHistCap / kThreads; ++k)
            if (tid + k * kThreads < cap) hid[k] = gh[tid + k * kThreads];
    }
    if (tid < kHistBuckets) { bs.hoff[tid] = 0; bs.hcur[tid] = 0; }
    if (tid == 0) {
        bs.u_row = u_row0;
        bs.hoff[kHistBuckets] = 0;
        bs.taubits = zkey(-FLT_MAX);
        for (int w = 0; w < kThreads / 32; ++w) bs.wbound[w] = -FLT_MAX;
        bs.tau_ck = 0;
        bs.maxbits = zkey(-INFINITY);
        bs.count = 0;
        bs.event = 0;
        bs.hist_ready = 0;
        bs.trig = kCandCap;
#ifdef BORN_PROFILE
        bs.pf_search = bs.pf_pair = bs.pf_calls = 0;
#endif
        bs.done_warps = 0;
        bs.fail = 0;
        bs.dropped = 0;
        bs.nh = 0;
        bs.last = 0;
        if (use_bar) {
            for (int s = 0; s < kStages; ++s) {
                mbar_init(reinterpret_cast<uint64_t*>(&bs.full_bar[s]), 1);
                mbar_init(reinterpret_cast<uint64_t*>(&bs.empty_bar[s]), kThreads / 32);
                mbar_init(reinterpret_cast<uint64_t*>(&bs.ready_bar[s]), 1);
            }
            mbar_fence_init();
        }
    }
    __syncthreads();  // the only barrier all 288 threads share

    const bool greedy0 = (rp0.flags & BORN_FLAG_GREEDY) || rp0.temperature == 0.0f;
    (void)greedy0;
    const bool pen_on = (rp0.repetition_penalty != 1.0f && rp0.repetition_penalty != 0.0f) ||
                        rp0.frequency_penalty != 0.0f || rp0.presence_penalty != 0.0f;
    // fp32 tiles can hold a penalised logit, so for them the otherwise idle producer warp
    // applies the history penalties in place before it releases the tile to the compute warps
    const bool producer_patches = hist_arg && pen_on && sizeof(T) == 4 && tma_l && A.mode != kModeMerge;
    int hshift0 = 0;
    while ((nchunks >> hshift0) > kHistBuckets) ++hshift0;

    if (tid >= kThreads) {
        // ------------------------------------------------------------------ producer warp
        if (!use_bar) return;
        const int lane = tid - kThreads;
        const int lag = 2;  // a tile is patched this many iterations after it was issued
        const int32_t* hlist = reinterpret_cast<const int32_t*>(smem + L.hist);
        const uint16_t* hcnt = reinterpret_cast<const uint16_t*>(smem + L.hist + kHistCap * 8);
        const int iters = nchunks + (producer_patches ? lag : 0);
        for (int it = 0; it < iters; ++it) {
            int stop = 0;
            if (it < nchunks && lane == 0) {
                const int c = it, st = c % kStages;
                if (c >= kStages) {
                    // the compute warps hand the tile back when they are done with it
                    if (!mbar_wait_or_abort(reinterpret_cast<uint64_t*>(&bs.empty_bar[st]),
                                            (uint32_t)(c / kStages - 1) & 1u, &bs.fail))
                        stop = 1;
                }
                if (!stop) {
                    const int n = min(kChunk, nelem - c * kChunk);
                    const uint32_t bytes_l = tma_l ? (((uint32_t)n * (uint32_t)sizeof(T) + 15u) & ~15u) : 0u;
                    const uint32_t bytes_m = tma_m ? ((((uint32_t)(n + 31) >> 5) * 4u + 15u) & ~15u) : 0u;
                    uint64_t* bar = reinterpret_cast<uint64_t*>(&bs.full_bar[st]);
                    mbar_expect_tx(bar, bytes_l + bytes_m);
                    if (tma_l) bulk_load(tiles + (size_t)st * kChunk, grow + (size_t)c * kChunk, bytes_l, bar);
                    if (tma_m) bulk_load(masks + st * (kChunk / 32), gmask + c * (kChunk / 32), bytes_m, bar);
                }
            }
            if (__any_sync(0xffffffffu, stop)) break;
            if (producer_patches && it >= lag) {
                if (it == lag) {
                    // the first copies are in flight; now wait (bounded) for the compute
                    // threads to finish bucketing the history
                    unsigned long long t0 = global_timer_ns();
                    int bad = 0;
                    while (!*reinterpret_cast<const volatile int*>(&bs.hist_ready)) {
                        if (*reinterpret_cast<const volatile int*>(&bs.fail)) { bad = 1; break; }
                        if (global_timer_ns() - t0 > kMbarTimeoutNs) { bs.fail = 1; bad = 1; break; }
                    }
                    if (__any_sync(0xffffffffu, bad)) break;
                }
                const int c = it - lag, st = c % kStages;
                const bool ok = mbar_wait_or_abort(reinterpret_cast<uint64_t*>(&bs.full_bar[st]),
                                                   (uint32_t)(c / kStages) & 1u, &bs.fail);
                if (!__all_sync(0xffffffffu, ok)) {
                    bs.fail = 1;
                    break;
                }
                float* tile = reinterpret_cast<float*>(tiles) + (size_t)st * kChunk;
                const int c0 = e_begin + c * kChunk, nvalid = min(kChunk, e_end - c0);
                const int b = c >> hshift0;
                const int lo = bs.hoff[b], hi = bs.hoff[b + 1];
                bool wrote = false;
                for (int i = lo + lane; i < hi; i += 32) {
                    const int cnt = hcnt[i];
                    const int off = hlist[i] - c0;
                    if (cnt > 0 && off >= 0 && off < nvalid) {
                        float z = tile[off];
                        if (rp0.repetition_penalty != 1.0f && rp0.repetition_penalty != 0.0f)
                            z = (z > 0.0f) ? __fdiv_rn(z, rp0.repetition_penalty) : __fmul_rn(z, rp0.repetition_penalty);
                        if (rp0.frequency_penalty != 0.0f || rp0.presence_penalty != 0.0f) {
                            float pen = __fmul_rn(rp0.frequency_penalty, (float)cnt);
                            pen = __fadd_rn(pen, rp0.presence_penalty);
                            z = __fsub_rn(z, pen);
                        }
                        tile[off] = z;
                        wrote = true;
                    }
                }
                if (wrote) fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&bs.ready_bar[st]));
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- compute threads
    Ctx cx;
    cx.cand = reinterpret_cast<uint64_t*>(smem + L.cand);
    cx.sc = reinterpret_cast<SearchScratch*>(smem + L.search);
    cx.lslot = reinterpret_cast<uint16_t*>(smem + L.pairs);
    cx.wpos = cx.lslot + kMaxK;
    cx.hlist = reinterpret_cast<int32_t*>(smem + L.hist);
    cx.hval = reinterpret_cast<float*>(smem + L.hist + kHistCap * 4);
    cx.hcnt = reinterpret_cast<uint16_t*>(smem + L.hist + kHistCap * 8);
    cx.bs = &bs;
#ifdef BORN_PROFILE
    cx.pr = A.prof ? A.prof + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32 : nullptr;
#endif
    cx.rp = rp0;
    const born_row_params& rp = cx.rp;
    const bool greedy = (rp.flags & BORN_FLAG_GREEDY) || rp.temperature == 0.0f;
    const float inv_T = greedy ? 1.0f : __fdiv_rn(1.0f, rp.temperature);
    cx.c2 = inv_T * 1.44269504f;
    cx.minp_on = !greedy && rp.min_p > 0.0f;
    cx.delta_minp = cx.minp_on ? (__logf(rp.min_p) - 0.05f) * rp.temperature : 0.0f;
    if (A.ext_total && !greedy && rp.top_k <= 0 && rp.top_p > 0.0f && rp.top_p < 1.0f) {
        // Top-p against the known total S of all survivors: the tokens lighter than
        // (1 - P) * S / V weigh less than (1 - P) * S together, so the nucleus lies among the
        // others -- a cut of the same kind as min-p (relative to the running maximum, with a
        // margin), which spares the candidate buffer nearly the whole row.
        const float s_all = (float)__ldcg(&A.ext_total[row]) * (1.0f / 1099511627776.0f);
        if (s_all > 0.0f) {
            const float d = (__logf((1.0f - rp.top_p) * s_all / (float)A.V) - 0.05f) * rp.temperature;
            cx.delta_minp = cx.minp_on ? fmaxf(cx.delta_minp, d) : d;
            cx.minp_on = true;
        }
    }
    cx.k_eff = greedy ? 1 : (rp.top_k > 0 ? min(rp.top_k, kMaxK) : kMaxK);
    cx.psize = (A.mode == kModeMerge) ? 0 : kPrivCap;
    cx.trigger = min(max(2 * cx.k_eff, 512), kCandCap - kPrivCap - 128);  // fill of the shared area that asks for a compaction
    if (tid == 0) bs.trig = cx.trigger;
    cx.hshift = 0;
    while ((nchunks >> cx.hshift) > kHistBuckets) ++cx.hshift;

    LanePriv lp;
    lp.pcnt = 0;
    BORN_PROF(0);
    float m_row = -INFINITY;  // maximum over the whole row (known after the merge)
    float lse_sum = 0.0f;     // sum of 2^((z - m_row) * c2) over the whole row
    int dropped = 0;

    if (A.mode != kModeMerge) {
        // ------------------------------------------------------------------ streaming pass
        bool has_hist = false;
        if (hist_arg && pen_on) {
            const int len = max(0, min(min(hist_len0, A.history_stride), kHistCap));
            const int nh = bucket_history(&cx, hid, len, e_begin, e_end, kChunk);
            has_hist = nh > 0 && !producer_patches;  // otherwise the tiles arrive patched
            if (producer_patches && tid == 0) {
                __threadfence_block();
                *reinterpret_cast<volatile int*>(&bs.hist_ready) = 1;
            }
        }

        BORN_PROF(1);
        ThreadStats st;
        st.mx = -INFINITY;
        st.R = -1e30f;
        st.nRc = 1e30f * cx.c2;
        st.s = make_float2(0.0f, 0.0f);
        st.pub = -INFINITY;
#ifdef BORN_PROFILE
        st.pf_hit = 0;
#endif

        // Warps stream their share of every tile on their own: they wait for the tile's bulk
        // copy, work on the vector groups they own, and hand the tile back with one mbarrier
        // arrival per warp.  The only block-wide meetings are the threshold bootstrap after
        // the first tile and the rendezvous for rare events.
        const int lane = tid & 31;
        bool failed = false;
        long long pa_wait = 0, pa_proc = 0, pa_rdv = 0;
        (void)pa_wait; (void)pa_proc; (void)pa_rdv;
        // wait for tile c; a warp parked here must still answer a rendezvous, or the warp
        // that called it (and holds an older tile) would never hand that tile back
        auto wait_tile = [&](int c, int stg) {
            if (!use_bar || failed) return;
            uint64_t* bar = reinterpret_cast<uint64_t*>(producer_patches ? &bs.ready_bar[stg] : &bs.full_bar[stg]);
            for (;;) {
                const int w = mbar_wait_or_event(bar, (uint32_t)(c / kStages) & 1u, &bs.event);
                if (w == 1) return;
                if (w == 2 && c > 0) { rendezvous(cx, lp); continue; }
                if (w == 2) continue;  // before the bootstrap nobody can have raised an event
                bs.fail = 1;
                failed = true;
                return;
            }
        };
        // rows that are not 16-byte aligned: each thread fetches its own groups
        auto fetch_tile = [&](int c, T* tile, int nvalid) {
            constexpr int VEC = VecOf<T>::n;
            const T* src = grow + (size_t)c * kChunk;
            for (int j = 0; j < kChunk / VEC / kThreads; ++j)
                for (int i = 0; i < VEC; ++i) {
                    const int e = (tid + kThreads * j) * VEC + i;
                    if (e < nvalid) tile[e] = src[e];
                }
            __syncwarp();
        };
        if (nchunks > 0) {
            // first tile: statistics, then the threshold bootstrap (block-wide), then the
            // tile's candidates under the new threshold
            BORN_PROF_T0();
            const int nvalid = min(kChunk, e_end - e_begin);
            const uint32_t* smask = tma_m ? masks : gmask;
            wait_tile(0, 0);
            BORN_PROF_ACC(pa_wait);
            if (!failed) {
                if (!tma_l) fetch_tile(0, tiles, nvalid);
                const bool tile_hist = has_hist && (bs.hoff[1] > bs.hoff[0]);
                process_tile<T, kHasMask, kLse>(cx, st, lp, tiles, smask, 0, e_begin, nvalid, tile_hist, true, false, 1);
                bootstrap_threshold(cx, st);
                process_tile<T, kHasMask, kLse>(cx, st, lp, tiles, smask, 0, e_begin, nvalid, tile_hist, false, true, 2);
                if (cx.minp_on) publish_max(cx, st);
            } else {
                bootstrap_threshold(cx, st);  // keep the block-wide step in lockstep
            }
            __syncwarp();
            if (lane == 0 && use_bar) mbar_arrive(reinterpret_cast<uint64_t*>(&bs.empty_bar[0]));
            BORN_PROF_ACC(pa_proc);
            BORN_PROF(2);
        }
        // The streaming loop proper holds only the common case -- a full tile that needs no
        // consumer-side history patch, every hit fitting the lane's private slots -- so that
        // its code stays small enough for the instruction cache.  Everything else leaves the
        // loop with a reason, is dealt with below it, and the loop is entered again.
        enum : int { kGoOn = 0, kEvent, kSlowTile, kOverflow, kRefresh, kFail, kDone };
        int c = 1, stg = 1 % kStages;
        uint32_t ovf = 0;
        // tiles that take the slow route: the last partial tile, rows fetched by the threads
        // themselves, tiles whose history tokens the compute warps must patch
        const bool slow_all = !tma_l || !use_bar;
        const int c_full = (nelem % kChunk) ? nchunks - 1 : nchunks;  // tiles [0, c_full) are full
        for (;;) {
            int why = kDone;
#pragma unroll 1
            while (c < nchunks && !failed) {
                BORN_PROF_T0();
                if (*reinterpret_cast<const volatile int*>(&bs.event)) { why = kEvent; break; }
                if (use_bar) {
                    uint64_t* bar = reinterpret_cast<uint64_t*>(producer_patches ? &bs.ready_bar[stg] : &bs.full_bar[stg]);
                    const int w = mbar_wait_or_event(bar, (uint32_t)(c / kStages) & 1u, &bs.event);
                    if (w != 1) { why = (w == 2) ? kEvent : kFail; break; }
                }
                BORN_PROF_ACC(pa_wait);
                if (slow_all || c >= c_full ||
                    (has_hist && bs.hoff[(c >> cx.hshift) + 1] > bs.hoff[c >> cx.hshift])) { why = kSlowTile; break; }
                const T* tile = tiles + (size_t)stg * kChunk;
                const uint32_t* smask = tma_m ? masks + stg * (kChunk / 32) : gmask + c * (kChunk / 32);
                ovf = fast_tile<T, kHasMask, kLse>(cx, st, lp, tile, smask, e_begin + c * kChunk, current_tau(cx));
                if (cx.minp_on) publish_max(cx, st);  // running maximum for the min-p prune
                if (__any_sync(0xffffffffu, ovf != 0)) { why = kOverflow; break; }
                if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&bs.empty_bar[stg]));  // tile back to the producer
                stg = (stg + 1 == kStages) ? 0 : stg + 1;
                ++c;
                BORN_PROF_ACC(pa_proc);
                if ((c & (c - 1)) == 0) { why = kRefresh; break; }
            }
            if (why == kDone || failed) break;
            if (why == kFail) {
                bs.fail = 1;
                failed = true;
                break;
            }
            if (why == kEvent) {
                rendezvous(cx, lp);  // then the same tile again
                continue;
            }
            if (why == kSlowTile || why == kOverflow) {
                const int c0 = e_begin + c * kChunk;
                const int nvalid = min(kChunk, e_end - c0);
                T* tile = tiles + (size_t)stg * kChunk;
                const uint32_t* smask = tma_m ? masks + stg * (kChunk / 32) : gmask + c * (kChunk / 32);
                if (why == kSlowTile) {
                    if (!tma_l) fetch_tile(c, tile, nvalid);
                    const bool tile_hist = has_hist && (bs.hoff[(c >> cx.hshift) + 1] > bs.hoff[c >> cx.hshift]);
                    process_tile<T, kHasMask, kLse>(cx, st, lp, tile, smask, c, c0, nvalid, tile_hist, true, true);
                    if (cx.minp_on) publish_max(cx, st);
                } else {
                    warp_retry<T>(cx, lp, tile, ovf, c0);  // the hits that found the private slots full
                }
                __syncwarp();
                if (lane == 0 && use_bar) mbar_arrive(reinterpret_cast<uint64_t*>(&bs.empty_bar[stg]));
                stg = (stg + 1 == kStages) ? 0 : stg + 1;
                ++c;
                if ((c & (c - 1)) != 0) continue;
            }
            // tighten tau from the lane maxima once per doubling of the tiles seen
            if (cx.k_eff <= kThreads) publish_lane_bound(cx, st);
        }
        // finished: one last bound from the lane maxima, then stay available for rendezvous
        // until every warp is through
        if (cx.k_eff <= kThreads && !failed && nchunks > 0) publish_lane_bound(cx, st);
        __syncwarp();
        if (lane == 0) smem_red_add(&bs.done_warps, 1u);
        while (!rendezvous(cx, lp)) { }
        BORN_PROF(3);
#ifdef BORN_PROFILE
        if (A.prof && tid == 0) {
            unsigned long long* pr = A.prof + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32;
            pr[8] = pa_wait; pr[9] = pa_rdv; pr[10] = pa_proc;
        }
        if (A.prof && lane == 0) {
            unsigned long long* pr = A.prof + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32;
            pr[16 + (tid >> 5)] = pa_proc;
        }
#endif
        if (bs.fail) {
            // A bulk copy never arrived.  The producer sees bs.fail and stops issuing; thread 0
            // waits (bounded) for copies that may still be in flight so that this CTA's shared
            // memory is quiet before it exits, then reports.
            if (tid == 0) {
                for (int s = 0; s < kStages; ++s) {
                    uint64_t* fb = reinterpret_cast<uint64_t*>(&bs.full_bar[s]);
                    mbar_wait(fb, 0);
                }
                atomicExch(A.dev_error, 1);
                if (A.out_status) A.out_status[row] = 100 + BORN_ERR_DEVICE_TIMEOUT;
                if (A.out_token) A.out_token[row] = -1;
            }
            cta_sync();
            return;
        }
        // A record that stands for a vocabulary shard or segment holds exactly its k best (that
        // is the algorithm's definition); a plain slice record of a row that is finished on this
        // GPU may hold any superset of them that fits.
        const bool exact_rec = (A.mode == kModeLocal) || A.segment_mode;
        const int rec_cap = exact_rec ? cx.k_eff : kMaxK;
        cta_sync();

        // slice statistics: every warp reduces its maximum and, relative to that, its share of
        // the log-sum-exp by shuffles; the eight pairs meet in shared memory behind one barrier
        float wm = st.mx;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) wm = max_nan(wm, __shfl_xor_sync(0xffffffffu, wm, d));
        float wsum = 0.0f;
        if (kLse) {
            const float ssum = st.s.x + st.s.y;
            wsum = ssum * ex2_approx(__fmul_rn(st.R - wm, cx.c2));
            if (!(ssum > 0.0f) || !(wm == wm)) wsum = 0.0f;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, d);
        }
        if ((tid & 31) == 0) {
            bs.redf[tid >> 5] = wm;
            bs.redf2[tid >> 5] = wsum;
        }
        cta_sync();
        float m_slice = bs.redf[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) m_slice = max_nan(m_slice, bs.redf[w]);
        float s_slice = 0.0f;
        if (kLse) {
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) {
                const float ws = bs.redf2[w];
                if (ws > 0.0f) s_slice += ws * ex2_approx(__fmul_rn(bs.redf[w] - m_slice, cx.c2));
            }
        }
        cta_sync();
        BORN_PROF(4);

        if (A.mode == kModeFull && A.S == 1) {
            m_row = m_slice;
            lse_sum = s_slice;
            dropped = bs.dropped;
        } else {
            // leave the record, then take a ticket; only the last CTA of the row goes on
            uint8_t* rec = A.records + (int64_t)row * A.rec_row_stride + (int64_t)slice * A.rec_slice_stride;
            uint64_t* ent = reinterpret_cast<uint64_t*>(rec + kRecordHdrBytes);
            int n = -1;
            uint32_t rec_flags = 0;
            if (exact_rec && cx.k_eff <= kThreads) {
                // Exactly the k best, without a radix select: the entries at or above the final
                // lane-maxima bound (a few more than k) are ranked against each other, several
                // threads to an entry, and an entry of rank r < k goes to position r.
                uint64_t* sel = reinterpret_cast<uint64_t*>(smem + L.search);
                const float tb = zkey_to_float(bs.taubits);
                const int scx = min(bs.count, kCandCap - cx.psize);
                if (tid == 0) bs.nl = 0;
                cta_sync();
                if (cx.psize) {
                    for (int s = 0; s < lp.pcnt; ++s) {
                        const uint64_t raw = cx.cand[s * kThreads + tid];
                        if (__uint_as_float((uint32_t)(raw >> 32)) >= tb) {
                            const int pos = (int)smem_atom_add(&bs.nl, 1u);
                            if (pos < kSmallSet) sel[pos] = raw_to_ck(raw);
                        }
                    }
                }
                for (int i = tid; i < scx; i += kThreads) {
                    const uint64_t e = cx.cand[cx.psize + i];
                    if (ck_alive(e) && ck_z(e) >= tb) {
                        const int pos = (int)smem_atom_add(&bs.nl, 1u);
                        if (pos < kSmallSet) sel[pos] = e;
                    }
                }
                cta_sync();
                const int na = bs.nl;
                if (na <= kSmallSet) {
                    int lg = 0;
                    while (lg < 5 && (na << (lg + 1)) <= kThreads) ++lg;
                    const int P = 1 << lg, part = tid & (P - 1), e_i = tid >> lg;
                    const uint64_t ck = (e_i < na) ? sel[e_i] : 0ull;
                    int rank = 0;
                    for (int j2 = part; j2 < na; j2 += P) rank += (sel[j2] > ck) ? 1 : 0;
                    for (int d = 1; d < P; d <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, d);
                    if (e_i < na && part == 0 && rank < cx.k_eff) ent[rank] = ck - (uint64_t)A.idx_offset;
                    n = min(na, cx.k_eff);
                    rec_flags = (uint32_t)(bs.dropped | (na > cx.k_eff ? 1 : 0));
                }
                cta_sync();
            }
            if (n < 0) {
                compact_to_k(cx, lp, rec_cap);
                cta_sync();
                const int sc = min(bs.count, kCandCap - cx.psize);
                // nothing below the slice's final bounds can be among the row's k best or pass min-p
                float tau_rec = (cx.k_eff <= kThreads) ? zkey_to_float(bs.taubits) : -INFINITY;
                if (cx.minp_on && m_slice == m_slice && !(rp.top_k <= 0 && bs.dropped)) tau_rec = fmaxf(tau_rec, m_slice + cx.delta_minp);
                if (exact_rec) tau_rec = -INFINITY;  // after the compaction: exactly the k best
                if (tid == 0) bs.nl = 0;
                cta_sync();
                for (int i = tid; i < kCandCap; i += kThreads) {
                    const uint64_t e = slot_key(cx, lp, i, sc);
                    if (ck_alive(e) && ck_z(e) >= tau_rec) {
                        const int pos = (int)smem_atom_add(&bs.nl, 1u);
                        if (pos < rec_cap) ent[pos] = e - (uint64_t)A.idx_offset;
                    }
                }
                cta_sync();
                n = min(bs.nl, rec_cap);
                rec_flags = (uint32_t)bs.dropped;
            }
            if (tid == 0) {
                RecordHdr h;
                h.m = m_slice; h.lse_s = s_slice; h.count = (uint32_t)n; h.flags = rec_flags;
                h.bound = (cx.k_eff <= kThreads && !greedy) ? zkey_to_float(bs.taubits) : -INFINITY;
                h.pad[0] = h.pad[1] = h.pad[2] = 0;
                *reinterpret_cast<RecordHdr*>(rec) = h;
            }
            if (A.mode == kModeLocal) return;
            __threadfence();
            cta_sync();
            if (tid == 0) {
                uint32_t t = atomicAdd(&A.tickets[row], 1u);
                bs.last = (t == (uint32_t)(A.S - 1));
                if (bs.last) A.tickets[row] = 0;  // ready for the next launch
            }
            cta_sync();
            if (!bs.last) return;
            __threadfence();
        }
    }

    // ---------------------------------------------------------------------- merge records
    if (A.mode == kModeMerge || A.S > 1) {
        cta_sync();
        if (tid == 0) bs.count = 0;
        lp.pcnt = 0;
        cx.psize = 0;  // the whole buffer is one shared area from here on
        cta_sync();
        // Headers first (all of them at once: the loads are independent), then the entries of
        // every record in one sweep without a barrier in between.  Entries below the best of
        // the slices' own bounds, or below the min-p cut of the row maximum, are left out.
        m_row = -INFINITY;
        float tau_row = -INFINITY;
        int total = 0;
#pragma unroll 4
        for (int s = 0; s < A.S; ++s) {
            const uint8_t* rec = A.records + (int64_t)row * A.rec_row_stride + (int64_t)s * A.rec_slice_stride;
            const uint4 h0 = __ldcg(reinterpret_cast<const uint4*>(rec));
            const float b0 = __ldcg(reinterpret_cast<const float*>(rec) + 4);
            m_row = max_nan(m_row, __uint_as_float(h0.x));
            tau_row = fmaxf(tau_row, b0);
            total += (int)h0.z;
            dropped |= (int)(h0.w & 1u);
        }
        if (A.segment_mode) tau_row = -INFINITY;  // segments keep exactly their k best
        else if (cx.minp_on && m_row == m_row && !(rp.top_k <= 0 && dropped))
            tau_row = fmaxf(tau_row, m_row + cx.delta_minp);  // (a row that lost entries must show its lowest one)
        if (tid == 0) bs.nw = 0;
        cta_sync();
#pragma unroll 2
        for (int s = 0; s < A.S; ++s) {
            const uint8_t* rec = A.records + (int64_t)row * A.rec_row_stride + (int64_t)s * A.rec_slice_stride;
            const uint4 h0 = __ldcg(reinterpret_cast<const uint4*>(rec));
            const float ms_ = __uint_as_float(h0.x), ss_ = __uint_as_float(h0.y);
            const int cnt = (int)h0.z;
            if (kLse && ss_ > 0.0f) lse_sum += ss_ * ex2_approx(__fmul_rn(ms_ - m_row, cx.c2));
            const unsigned long long* ent = reinterpret_cast<const unsigned long long*>(rec + kRecordHdrBytes);
            for (int i = tid; i < cnt; i += kThreads) {
                const uint64_t e = __ldcg(ent + i);
                if (ck_alive(e) && ck_z(e) >= tau_row) {
                    const int pos = (int)smem_atom_add(&bs.count, 1u);
                    if (pos < kCandCap) cx.cand[pos] = e;
                    else bs.nw = 1;  // does not fit: redo record by record with compactions
                }
            }
        }
        cta_sync();
        const bool refill = bs.nw != 0;
        cta_sync();
        if (refill) {
            if (tid == 0) bs.count = 0;
            cta_sync();
            for (int s = 0; s < A.S; ++s) {
                const uint8_t* rec = A.records + (int64_t)row * A.rec_row_stride + (int64_t)s * A.rec_slice_stride;
                const int cnt = (int)__ldcg(reinterpret_cast<const uint32_t*>(rec) + 2);
                if (!A.segment_mode && bs.count + cnt > kCandCap) compact_to_k(cx, lp, cx.k_eff);
                const int base = bs.count;
                const unsigned long long* ent = reinterpret_cast<const unsigned long long*>(rec + kRecordHdrBytes);
                for (int i = tid; i < cnt && base + i < kCandCap; i += kThreads) {
                    const uint64_t e = __ldcg(ent + i);
                    cx.cand[base + i] = ck_alive(e) ? e : (uint64_t)(base + i);  // dead slots stay unique
                }
                cta_sync();
                if (tid == 0) bs.count = min(base + cnt, kCandCap);
                cta_sync();
            }
        }
        (void)total;
    }

    // ------------------------------------------------------------- selection and draw
    cta_sync();
    BORN_PROF(5);
    const int sc_fin = min(bs.count, kCandCap - cx.psize);  // filled part of the shared area
    int n = kCandCap;                                      // walk the whole buffer; unfilled slots read as dead
    auto ent_at = [&](int i) { return slot_key(cx, lp, i, sc_fin); };
    int status = BORN_ROW_OK;
    if (m_row != m_row) status = BORN_ROW_NAN;
    else if (m_row == INFINITY) status = BORN_ROW_POS_INF;
    else if (m_row == -INFINITY) status = BORN_ROW_ALL_MASKED;
    else if (!greedy && rp.top_k > kMaxK) status = BORN_ROW_OVERFLOW;
    if (kLse && A.out_lse && tid == 0)
        A.out_lse[row] = (status == BORN_ROW_OK) ? m_row * inv_T + __log2f(lse_sum) * 0.69314718f : NAN;
    if (status != BORN_ROW_OK) {
        if (tid == 0) {
            A.out_token[row] = -1;
            A.out_status[row] = status;
            if (A.out_prob) A.out_prob[row] = 0.0f;
            if (A.out_kept_count) A.out_kept_count[row] = 0;
        }
        return;
    }
    dropped |= bs.dropped;
    uint64_t* cand = cx.cand;
    unsigned long long* qbuf = reinterpret_cast<unsigned long long*>(smem + L.tiles);  // tiles are idle now

    if (greedy) {
        uint64_t best = 0;
        for (int i = tid; i < n; i += kThreads) best = max(best, ent_at(i));
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) best = max(best, shfl_xor_u64(best, d));
        if ((tid & 31) == 0) bs.red64[tid >> 5] = best;
        cta_sync();
        if (tid == 0) {
            for (int w = 1; w < kThreads / 32; ++w) best = max(best, (uint64_t)bs.red64[w]);
            int tok = ck_idx(best);
            A.out_token[row] = tok;
            A.out_status[row] = BORN_ROW_OK;
            if (A.out_prob) A.out_prob[row] = 1.0f;
            if (A.out_kept_count) A.out_kept_count[row] = 1;
            if (A.out_kept_ids && A.kept_stride > 0) A.out_kept_ids[(int64_t)row * A.kept_stride] = tok;
        }
        return;
    }

    // Gather the entries that can still matter: alive, not below the final lane-maxima bound
    // when this CTA streamed the whole row itself, and not below the min-p cut taken from the
    // row's final maximum (an entry below it has a mass below min_p times the largest one).
    // Each thread looks at the private slots it filled and at its share of the shared area.
    const uint64_t Qa = cx.minp_on ? __double2ull_ru((double)rp.min_p * 1099511627776.0) : 0ull;
    const float u = bs.u_row;
    uint64_t* sel = reinterpret_cast<uint64_t*>(smem + L.search);  // kSmallSet keys, then kSmallSet masses
    unsigned long long* selq = reinterpret_cast<unsigned long long*>(sel + kSmallSet);
    const bool own_row = (A.mode == kModeFull && A.S == 1);
    // With top-k off and entries dropped the kept set is exact only if min-p cuts inside the
    // buffer -- unless the caller supplied the total mass of all survivors: then top-p is taken
    // against that total and the row is exact whenever its nucleus fits into the buffer.
    const bool have_total = A.ext_total != nullptr && rp.top_k <= 0 && rp.top_p > 0.0f && rp.top_p < 1.0f;
    const bool need_low = (rp.top_k <= 0 && dropped && !have_total);  // the set's lowest entry must be seen unpruned
    const uint64_t S_all = have_total ? __ldcg(&A.ext_total[row]) : 0ull;
    float tau_g = (own_row && cx.k_eff <= kThreads) ? zkey_to_float(bs.taubits) : -INFINITY;
    if (cx.minp_on && !need_low && !A.segment_mode) tau_g = fmaxf(tau_g, m_row + cx.delta_minp);
    // a merged row whose records hold far more than k entries is cut to its k best first
    if (!own_row && !A.segment_mode && cx.k_eff <= kSmallSet && bs.count > kSmallSet) compact_to_k(cx, lp, cx.k_eff);
    const int sc_g = min(bs.count, kCandCap - cx.psize);
    if (tid == 0) { bs.nl = 0; bs.acc[0] = 0; bs.acc[1] = 0; bs.acc[2] = 0; }
    cta_sync();
    if (cx.psize) {
        for (int s = 0; s < lp.pcnt; ++s) {
            const uint64_t raw = cand[s * kThreads + tid];
            const float z = __uint_as_float((uint32_t)(raw >> 32));
            if (z >= tau_g) {
                const int pos = (int)smem_atom_add(&bs.nl, 1u);
                if (pos < kSmallSet) sel[pos] = raw_to_ck(raw);
            }
        }
    }
    for (int i = tid; i < sc_g; i += kThreads) {
        const uint64_t c = cand[cx.psize + i];
        if (ck_alive(c) && ck_z(c) >= tau_g) {
            const int pos = (int)smem_atom_add(&bs.nl, 1u);
            if (pos < kSmallSet) sel[pos] = c;
        }
    }
    cta_sync();
    const int na = bs.nl;
    BORN_PROF(24);
#ifdef BORN_PROFILE
    if (A.prof && tid == 0) A.prof[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32 + 14] = (unsigned long long)na;
#endif
    if (na <= kSmallSet) {
        // ---- small set: everything by all-pairs comparison (no sort, no histogram): rank for
        // top-k, mass ahead in rank order for top-p, mass ahead in index order for the draw.
        // An entry is shared by P = 2^lg adjacent threads (as many as fit into the block), each
        // walking every P-th entry; the partial counts meet by shuffles.  Sums are exact integers.
        int lg = 0;
        while (lg < 5 && (na << (lg + 1)) <= kThreads) ++lg;
        const int P = 1 << lg, part = tid & (P - 1), ent = tid >> lg;
        const bool mine = ent < na;
        const bool lead = mine && part == 0;
        const uint64_t ck = mine ? sel[ent] : 0ull;
        auto group_sum = [&](uint64_t v) {
            for (int d = 1; d < P; d <<= 1) v += shfl_xor_u64(v, d);
            return v;
        };
        auto block_add = [&](uint64_t v, int slot) {  // v counts once per entry (its leading thread)
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += shfl_xor_u64(v, d);
            if ((tid & 31) == 0 && v) atomicAdd(&bs.acc[slot], (unsigned long long)v);
        };
        // (the all-pairs passes read two entries per 16-byte shared load)
        const ulonglong2* sel2 = reinterpret_cast<const ulonglong2*>(sel);
        const ulonglong2* selq2 = reinterpret_cast<const ulonglong2*>(selq);
        int rank = 0;
        for (int jj = part; jj < (na >> 1); jj += P) {
            const ulonglong2 k2 = sel2[jj];
            rank += (k2.x > ck ? 1 : 0) + (k2.y > ck ? 1 : 0);
        }
        if ((na & 1) && part == 0) rank += (sel[na - 1] > ck) ? 1 : 0;
        rank = (int)group_sum((uint64_t)rank);
        bool kept = mine && (A.segment_mode || rank < cx.k_eff);
        uint64_t q = 0;
        if (kept) {
            const float x = scaled_shift(ck_z(ck), m_row, inv_T);
            q = (x < -30.0f) ? 0ull : mass_of(x);
        }
        if (need_low) {
            // survivor limit reached with top-k off: exact only if min-p cuts inside the set
            uint64_t low = mine ? ck : ~0ull;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) low = min(low, shfl_xor_u64(low, d));
            if ((tid & 31) == 0) bs.red64[tid >> 5] = low;
            cta_sync();
            for (int w = 0; w < kThreads / 32; ++w) low = min(low, (uint64_t)bs.red64[w]);
            cta_sync();
            const float xl = scaled_shift(ck_z(low), m_row, inv_T);
            const uint64_t ql = (xl < -30.0f) ? 0ull : mass_of(xl);
            if (!(cx.minp_on && (ql + (ql >> 18) + 4ull < Qa))) {
                if (tid == 0) {
                    A.out_token[row] = -1;
                    A.out_status[row] = BORN_ROW_OVERFLOW;
                    if (A.out_prob) A.out_prob[row] = 0.0f;
                    if (A.out_kept_count) A.out_kept_count[row] = 0;
                }
                return;
            }
        }
        if (Qa && q < Qa) { kept = false; q = 0; }
        BORN_PROF(25);
        cta_sync();  // every thread has read sel[] for its rank
        // The nk best entries (all of them in segment mode) go to sel[0..nk) in rank order;
        // an entry that min-p removed stays in place as a dead one with no mass.
        const int nk = A.segment_mode ? na : min(na, cx.k_eff);
        if (lead && rank < nk) {
            sel[rank] = kept ? ck : (ck & (uint64_t)kIdxMask);
            selq[rank] = q;
        }
        block_add(lead ? q : 0ull, 0);
        cta_sync();
        uint64_t S = bs.acc[0];
        // the threads are dealt out again, over the nk entries that are left
        int lg2 = 0;
        while (lg2 < 5 && (nk << (lg2 + 1)) <= kThreads) ++lg2;
        const int P2 = 1 << lg2, part2 = tid & (P2 - 1), ent2 = tid >> lg2;
        const bool mine2 = ent2 < nk;
        const bool lead2 = mine2 && part2 == 0;
        const uint64_t ck2 = mine2 ? sel[ent2] : 0ull;
        uint64_t q2 = mine2 ? (uint64_t)selq[ent2] : 0ull;
        bool kept2 = mine2 && ck_alive(ck2);
        auto group_sum2 = [&](uint64_t v) {
            for (int d = 1; d < P2; d <<= 1) v += shfl_xor_u64(v, d);
            return v;
        };
        if (rp.top_p > 0.0f && rp.top_p < 1.0f) {
            uint64_t before = 0;  // mass ahead in rank order = mass of the entries in front
            const int lim = min(ent2, nk);
            for (int jj = part2; jj < (lim >> 1); jj += P2) {
                const ulonglong2 v2 = selq2[jj];
                before += v2.x + v2.y;
            }
            if ((lim & 1) && part2 == 0) before += selq[lim - 1];
            before = group_sum2(before);
            uint64_t Tp = __double2ull_rz(__dmul_rn((double)rp.top_p, __ull2double_rn(have_total ? S_all : S)));
            if (Tp < 1) Tp = 1;
            if (have_total && dropped && S < Tp) {  // the nucleus does not fit into the buffer
                if (tid == 0) {
                    A.out_token[row] = -1;
                    A.out_status[row] = BORN_ROW_OVERFLOW;
                    if (A.out_prob) A.out_prob[row] = 0.0f;
                    if (A.out_kept_count) A.out_kept_count[row] = 0;
                }
                return;
            }
            if (kept2 && !(before < Tp)) { kept2 = false; q2 = 0; }
            cta_sync();
            if (lead2) {
                sel[ent2] = kept2 ? ck2 : (ck2 & (uint64_t)kIdxMask);
                selq[ent2] = q2;
            }
            block_add(lead2 ? q2 : 0ull, 1);
            cta_sync();
            S = bs.acc[1];
        }
        BORN_PROF(26);
        const uint32_t my_low = (uint32_t)(ck2 & kIdxMask);  // larger low bits = smaller token index
        uint64_t pre = 0;
        for (int jj = part2; jj < (nk >> 1); jj += P2) {
            const ulonglong2 k2 = sel2[jj], v2 = selq2[jj];
            pre += (((uint32_t)(k2.x & kIdxMask) > my_low) ? v2.x : 0ull) + (((uint32_t)(k2.y & kIdxMask) > my_low) ? v2.y : 0ull);
        }
        if ((nk & 1) && part2 == 0) pre += ((uint32_t)(sel[nk - 1] & kIdxMask) > my_low) ? selq[nk - 1] : 0ull;
        pre = group_sum2(pre);
        if (S == 0) {  // cannot happen while the row maximum is finite; never divide by it
            if (tid == 0) { A.out_token[row] = -1; A.out_status[row] = BORN_ROW_ALL_MASKED; }
            return;
        }
        uint64_t t = __double2ull_rz(__dmul_rn((double)u, __ull2double_rn(S)));
        if (t > S - 1) t = S - 1;
        if (lead2 && kept2 && pre <= t && t < pre + q2) {
            A.out_token[row] = ck_idx(ck2);
            A.out_status[row] = BORN_ROW_OK;
            if (A.out_prob) A.out_prob[row] = __double2float_rn(__ddiv_rn(__ull2double_rn(q2), __ull2double_rn(S)));
        }
        BORN_PROF(6);
        if (A.out_kept_count || A.out_kept_ids) {
            if (A.out_kept_ids) {
                int kr = 0;  // kept entries ahead in rank order
                const int lim = min(ent2, nk);
                for (int jj = part2; jj < (lim >> 1); jj += P2) {
                    const ulonglong2 k2 = sel2[jj];
                    kr += (ck_alive(k2.x) ? 1 : 0) + (ck_alive(k2.y) ? 1 : 0);
                }
                if ((lim & 1) && part2 == 0) kr += ck_alive(sel[lim - 1]) ? 1 : 0;
                kr = (int)group_sum2((uint64_t)kr);
                if (lead2 && kept2 && kr < A.kept_stride) A.out_kept_ids[(int64_t)row * A.kept_stride + kr] = ck_idx(ck2);
            }
            if (A.out_kept_count) {
                block_add((lead2 && kept2) ? 1ull : 0ull, 2);
                cta_sync();
                if (tid == 0) A.out_kept_count[row] = (int)bs.acc[2];
            }
        }
        return;
    }

    // ---- large set: radix select, then radix threshold searches over a flat copy
    if (!A.segment_mode) compact_to_k(cx, lp, cx.k_eff);
    dropped |= bs.dropped;
    {
        // flatten the surviving entries (private slots and shared area) into the idle tiles
        const int sc2 = min(bs.count, kCandCap - cx.psize);
        uint64_t* flat = reinterpret_cast<uint64_t*>(smem + L.tiles);
        if (tid == 0) bs.nl = 0;
        cta_sync();
        for (int i = tid; i < kCandCap; i += kThreads) {
            const uint64_t e = slot_key(cx, lp, i, sc2);
            if (ck_alive(e)) flat[smem_atom_add(&bs.nl, 1u)] = e;
        }
        cta_sync();
        n = bs.nl;
        cand = flat;
        qbuf = reinterpret_cast<unsigned long long*>(flat + kCandCap);
    }
    // fixed-point masses relative to the row maximum
    uint64_t low_ck = ~0ull;
    for (int i = tid; i < n; i += kThreads) {
        uint64_t c = cand[i];
        if (ck_alive(c)) {
            float x = scaled_shift(ck_z(c), m_row, inv_T);
            qbuf[i] = (x < -30.0f) ? 0ull : mass_of(x);
            low_ck = min(low_ck, c);
        } else {
            qbuf[i] = 0ull;
        }
    }
    if (rp.top_k <= 0 && dropped && !have_total) {
        // survivor limit reached with top-k off: exact only if min-p cuts inside the buffer
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) low_ck = min(low_ck, shfl_xor_u64(low_ck, d));
        cta_sync();
        if ((tid & 31) == 0) bs.red64[tid >> 5] = low_ck;
        cta_sync();
        for (int w = 0; w < kThreads / 32; ++w) low_ck = min(low_ck, (uint64_t)bs.red64[w]);
        float xl = scaled_shift(ck_z(low_ck), m_row, inv_T);
        uint64_t ql = (xl < -30.0f) ? 0ull : mass_of(xl);
        bool exact = cx.minp_on && (ql + (ql >> 18) + 4ull < Qa);
        if (!exact) {
            if (tid == 0) {
                A.out_token[row] = -1;
                A.out_status[row] = BORN_ROW_OVERFLOW;
                if (A.out_prob) A.out_prob[row] = 0.0f;
                if (A.out_kept_count) A.out_kept_count[row] = 0;
            }
            return;
        }
    }
    cta_sync();
    if (Qa) {
        for (int i = tid; i < n; i += kThreads)
            if (qbuf[i] < Qa && ck_alive(cand[i])) { qbuf[i] = 0; cand[i] &= (uint64_t)kIdxMask; }
        cta_sync();
    }
    if (rp.top_p > 0.0f && rp.top_p < 1.0f) {
        uint64_t part = 0;
        for (int i = tid; i < n; i += kThreads) part += qbuf[i];
        uint64_t S = block_sum_u64(part, bs.red64);
        uint64_t Tp = __double2ull_rz(__dmul_rn((double)rp.top_p, __ull2double_rn(have_total ? S_all : S)));
        if (Tp < 1) Tp = 1;
        if (have_total && dropped && S < Tp) {  // the nucleus does not fit into the buffer
            if (tid == 0) {
                A.out_token[row] = -1;
                A.out_status[row] = BORN_ROW_OVERFLOW;
                if (A.out_prob) A.out_prob[row] = 0.0f;
                if (A.out_kept_count) A.out_kept_count[row] = 0;
            }
            return;
        }
        uint64_t C = block_radix_search<true, 56, false>(
            n, Tp - 1, [&](int i) { return cand[i]; }, [&](int i) { return qbuf[i]; }, *cx.sc);
        for (int i = tid; i < n; i += kThreads)
            if (cand[i] < C && ck_alive(cand[i])) { qbuf[i] = 0; cand[i] &= (uint64_t)kIdxMask; }
        cta_sync();
    }
    uint64_t part = 0;
    for (int i = tid; i < n; i += kThreads) part += qbuf[i];
    const uint64_t S = block_sum_u64(part, bs.red64);
    uint64_t t = __double2ull_rz(__dmul_rn((double)u, __ull2double_rn(S)));
    if (t > S - 1) t = S - 1;
    const uint64_t tok64 = block_radix_search<false, 24, false>(
        n, t, [&](int i) { return (uint64_t)ck_idx(cand[i]); }, [&](int i) { return qbuf[i]; }, *cx.sc);
    const int tok = (int)tok64;
    for (int i = tid; i < n; i += kThreads) {
        if (ck_idx(cand[i]) == tok && ck_alive(cand[i])) {
            A.out_token[row] = tok;
            A.out_status[row] = BORN_ROW_OK;
            if (A.out_prob)
                A.out_prob[row] = __double2float_rn(__ddiv_rn(__ull2double_rn(qbuf[i]), __ull2double_rn(S)));
        }
    }
    BORN_PROF(6);
#ifdef BORN_PROFILE
    if (A.prof && tid == 0) {
        unsigned long long* pr = A.prof + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 32;
        pr[11] = bs.pf_search; pr[12] = bs.pf_pair; pr[13] = bs.pf_calls; pr[15] = (unsigned long long)n;
    }
#endif
    if (A.out_kept_count || A.out_kept_ids) {
        int alive = 0;
        for (int i = tid; i < n; i += kThreads) {
            uint64_t c = cand[i];
            if (!ck_alive(c)) continue;
            ++alive;
            if (A.out_kept_ids) {
                int rank = 0;
                for (int j = 0; j < n; ++j) rank += (cand[j] > c) ? 1 : 0;
                if (rank < A.kept_stride) A.out_kept_ids[(int64_t)row * A.kept_stride + rank] = ck_idx(c);
            }
        }
        uint64_t tot = block_sum_u64((uint64_t)alive, bs.red64);
        if (tid == 0 && A.out_kept_count) A.out_kept_count[row] = (int)tot;
    }
}

}  // namespace born
