// Shared definitions of the streaming sampler: work decomposition, scratch records and the
// arguments of scan_kernel / merge_kernel.
//
// Work decomposition.  The [rows, vocab] logits are cut into tiles of 16 KB (4096 fp32 or
// 8192 bf16 logits, counted from the 16-byte boundary at or below each row's first logit).
// All tiles of all rows form one sequence; CTA c of a grid of G streams the contiguous
// range [c*T/G, (c+1)*T/G) of it, so every CTA moves the same number of bytes whatever the
// batch and vocabulary sizes are.  The part of a row that falls into one CTA's range is a
// *segment*; a segment leaves a record (maximum, log-sum-exp share, candidates) in scratch
// memory, and the CTA that completes a row (atomic ticket, no spinning) finishes it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/born_sampler.h"
#include "spec.cuh"

namespace born {

constexpr int kScanStages = 4;              // bulk-copy stages in flight per CTA: what every instantiation has ...
constexpr int kScanStagesMax = 5;           // ... and what those without a mask have whose token-history list is absent or short:
                                            // their shared memory has room for one more at two CTAs per SM, and the stream
                                            // is bound by the bytes a CTA keeps in flight
constexpr int kHistShort = 512;             // history ids per row up to which the list counts as short
// hist_cap: entries the history list has room for (kHistShort or BORN_MAX_HISTORY; ignored without a history)
__host__ __device__ constexpr int scan_stages(bool has_mask, bool has_hist, int hist_cap) {
    return (!has_mask && (!has_hist || hist_cap <= kHistShort)) ? kScanStagesMax : kScanStages;
}
constexpr int kScanWarps = kThreads / 32;   // compute warps
constexpr int kScanThreads = kThreads + 32; // compute threads + the producer warp
constexpr int kWarpCand = 256;              // candidate slots per compute warp and segment
constexpr int kMassBlock = 512;             // tokens per mass block of the whole-vocabulary routes
constexpr int kSelCap = 1024;               // candidates the in-shared-memory selection handles
constexpr int kHashSlots = 2048;            // open-addressing table for the distinct history ids
constexpr int kHdrCache = 32;                // segment headers of a row that the finish keeps in shared memory
constexpr float kNucleusWindow = 10.0f;     // top-p alone: candidates are collected this far (in units of
                                            // scaled logits) below the running maximum, then verified

enum : int { kScanFull = 0, kScanLocal = 1 };

template <typename T>
struct TileOf { static constexpr int n = kTileBytes / (int)sizeof(T); };
template <typename T>
struct VecOf { static constexpr int n = 16 / (int)sizeof(T); };

struct SegHdr {        // 32 bytes, precedes the entries of a segment record
    float m;           // maximum of the segment (NaN if a NaN was seen)
    float lse_sum;     // sum of 2^((z - m) * c2) over the segment
    float tau_excl;    // the entries are complete only at or above this value (-inf: complete)
    float bound_k;     // at least k tokens of the segment are at or above this value (-inf: unknown)
    uint32_t count;    // entries that follow: (value bits << 32) | token id
    uint32_t pad[3];
};
static_assert(sizeof(SegHdr) == kRecordHdrBytes, "segment header size");

struct MassBlock {     // one per kMassBlock tokens of a row, aligned to the row start
    float m;           // maximum of the block (-inf: nothing above -inf)
    uint32_t pad;      // tokens of the block above -inf
    unsigned long long M;  // exact sum of rne(exp_det((z - m) * inv_T) * 2^40) over the block
};

struct ScanArgs {
    const void* logits;
    int64_t row_stride;   // elements between caller rows
    const uint32_t* mask;
    int64_t mask_stride;  // words between caller rows
    const int32_t* history;
    const int32_t* history_len;
    int history_stride;
    // device-resident history (born_history_*): the finished row appends its token here
    int32_t* ring;            // [rows, ring_cap] the last ring_cap tokens of every row; NULL: off
    int32_t* ring_total;      // [rows] tokens appended since the reset
    int32_t* ring_len;        // [rows] min(total, ring_cap): what the next call reads as history_len
    int32_t* ring_finished;   // [rows] non-zero once the row has sampled a stop token
    int ring_cap, n_stop;
    int32_t stop_ids[8];
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
    int B;         // caller rows
    int G;         // contiguous vocabulary segments per caller row (1: none); a (row, segment) pair is
                   // streamed as a row of its own ("virtual row" r = b * G + g)
    int V;         // tokens per virtual row
    int tpr;       // tiles per virtual row
    int fast;      // every virtual row (and its mask words) starts on a 16-byte boundary
    int mode;      // kScanFull: sample; kScanLocal: leave the k best of every virtual row in `packed`
    int want_lse;
    int idx_base;  // added to the token ids written in kScanLocal mode
    uint8_t* packed;            // kScanLocal: record of virtual row (b, g) at g*packed_seg_stride + b*packed_row_stride
    int64_t packed_row_stride, packed_seg_stride;
    uint8_t* records;           // segment records, rec_stride bytes apart, indexed by row + cta
    int64_t rec_stride;
    int rec_cap;                // entries per record
    MassBlock* blocks;          // [rows, nblk]
    int nblk;
    uint32_t* tickets;          // [rows] zero between launches
    uint32_t* deferred;         // [rows] zero between launches: cta+1 that owes the row its exact fallback
    int* dev_error;                 // [0] error word, [1] rows that took the exact search, [8..16] ... by reason
    unsigned long long timeout_ns;  // limit of every on-device wait
    long long debug_skip_tile;      // test hook: the bulk copy of this tile is never issued (-1: none)
};

// ---- geometry -----------------------------------------------------------------------------
struct RowGeom {
    int b, g;              // caller row, vocabulary segment
    int lead;              // elements between the 16-byte boundary below the row and its first logit
    const uint8_t* abase;  // that boundary
};
// kOneSeg: the launch has no vocabulary segments (G == 1)
template <typename T, bool kOneSeg = false>
__device__ __forceinline__ RowGeom row_geom(const ScanArgs& A, int r) {
    RowGeom q;
    q.b = kOneSeg ? r : r / A.G;
    q.g = kOneSeg ? 0 : r - q.b * A.G;
    const uint8_t* base = reinterpret_cast<const uint8_t*>(A.logits) +
                          ((int64_t)q.b * A.row_stride + (int64_t)q.g * A.V) * (int64_t)sizeof(T);
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(base) & 15u);
    q.lead = (int)(mis / sizeof(T));
    q.abase = base - mis;
    return q;
}
// the mask words a tile needs: first word loaded (16-byte aligned address) and word count
struct MaskTile {
    int64_t w0a;   // first word of the row's mask that is loaded
    int nw;        // words loaded (multiple of 4; 0: none)
    int64_t mb0;   // bit index (within the caller row's mask) of element 0 of the tile
};
template <typename T>
__device__ __forceinline__ MaskTile mask_tile(const ScanArgs& A, const RowGeom& q, int j, int lo, int n_el) {
    MaskTile m;
    m.mb0 = (int64_t)q.g * A.V + (int64_t)j * TileOf<T>::n - q.lead;
    m.w0a = 0;
    m.nw = 0;
    if (n_el <= lo) return m;
    const uint32_t* mrow = A.mask + (int64_t)q.b * A.mask_stride;
    const int64_t w0 = (m.mb0 + lo) >> 5;
    const int64_t w1 = (m.mb0 + n_el - 1) >> 5;
    const int sub = (int)((reinterpret_cast<uintptr_t>(mrow + w0) & 15u) >> 2);
    m.w0a = w0 - sub;
    int64_t nw = (w1 - m.w0a + 1 + 3) & ~(int64_t)3;
    // never read past the 16-byte granule that holds the row's last valid mask word
    const int64_t valid = ((int64_t)A.G * A.V + 31) >> 5;
    const uintptr_t end = (reinterpret_cast<uintptr_t>(mrow + valid) + 15u) & ~(uintptr_t)15u;
    const int64_t wsafe = (int64_t)((end - reinterpret_cast<uintptr_t>(mrow)) >> 2);
    if (m.w0a + nw > wsafe) nw = wsafe - m.w0a;
    m.nw = (int)nw;
    return m;
}
template <typename T>
__host__ __device__ constexpr int mask_stage_words() { return TileOf<T>::n / 32 + 8; }

// CTA that streams tile t of a sequence of T tiles cut into G ranges [c*T/G, (c+1)*T/G)
__host__ __device__ inline long long range_begin(long long c, long long T, long long G) { return c * T / G; }
__host__ __device__ inline int cta_of_tile(long long t, long long T, long long G) {
    return (int)(((t + 1) * G + T - 1) / T - 1);
}

// Shared-memory layout (dynamic part), computed identically on host and device.
struct ScanSmem {
    int tiles, masks, cand, sel, hist, total;
};
__host__ __device__ inline ScanSmem scan_smem_layout(int elem_bytes, bool has_mask, bool has_hist, int hist_cap = BORN_MAX_HISTORY) {
    ScanSmem L;
    int off = 0;
    const int stages = scan_stages(has_mask, has_hist, hist_cap);
    L.tiles = off; off += stages * kTileBytes;
    L.masks = off; off += has_mask ? stages * ((kTileBytes / elem_bytes / 32 + 8) * 4) : 0;
    off = (off + 127) & ~127;
    L.cand = off; off += kScanWarps * kWarpCand * 8;  // the warps' candidate buffers; the selection's masses once they are read
    L.sel = off; off += kSelCap * 8;                   // the selection's rank keys
    L.hist = off; off += has_hist ? hist_cap * 8 : 0;  // the segment's distinct history tokens, by tile
    L.total = off;
    return L;
}
static_assert(kScanWarps * kWarpCand * 8 >= kSelCap * 8, "the selection's masses alias the candidate buffers");

// Static shared state of a CTA of scan_kernel (and of merge_kernel, which uses the selection part).
struct ScanShared {
    unsigned long long full_bar[kScanStagesMax];
    unsigned long long empty_bar[kScanStagesMax];
    unsigned long long ready_bar[kScanStagesMax];  // fp32 launches with token histories: the producer has patched the tile
    // segment state of the compute threads
    uint32_t maxbits;               // key of the running maximum (only ever raised)
    uint32_t excl_bits;             // key of the exclusion level (only ever raised)
    uint32_t rec_count;
    uint32_t defer;             // one-row launches: the row's `deferred` word (0: finished)
    float wbound[kScanWarps];       // per warp: its share of the lane-maxima bound
    uint32_t wcount[kScanWarps];    // candidates in each warp's buffer
    float wmax[kScanWarps], wsum[kScanWarps];
    int fail;
    int hist_seq;                   // segments of this CTA whose history list is built (read by the producer warp)
    int hist_n;                     // ... entries of the latest one
    born_row_params hist_rp;        // ... and its row's parameters
    int prod_done;                  // the producer warp has left its loop
    long long issued;               // ... having issued the tiles below this one
    int last, c_first, c_last;
    // finish / selection scratch
    unsigned long long red64[kScanWarps];
    unsigned long long acc[4];
    float redf[kScanWarps], redf2[kScanWarps], redf3[kScanWarps];
    int nl, nw, flag;
    float4 hdr[kHdrCache];
    uint32_t hdr_cnt[kHdrCache];
    int found;
    unsigned long long before;
    SearchScratch sc;
};

__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase (try_wait may suspend the thread for a while; a polling loop
// that has other work to look at must not).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait with a caller-chosen limit; also gives up when *abort becomes non-zero.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, unsigned long long limit_ns,
                                                const volatile int* abort) {
    if (mbar_try(bar, parity)) return true;
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < kMbarSpinLimit; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 15u) == 15u) {
            if (abort && *abort) return false;
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
    return false;
}

__device__ __forceinline__ float max3_nan(float a, float b, float c) {
    float r;
    asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ float warp_max_nan(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = max_nan(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
// smallest float above v (v finite or -inf), through the order-preserving key
__device__ __forceinline__ uint32_t key_above(float v) { return zkey(v) + 1u; }

// Penalised logit of a history token (once per distinct token, `cnt` = its multiplicity):
// repetition z>0 ? z/r : z*r, then z -= (f*cnt + p) as three separately rounded operations.
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
// The range check that the host applies to uniform parameters (params_ok in capi.cu), for
// per-row parameter arrays that live on the device and so reach the kernel unchecked.
__device__ __forceinline__ bool row_params_ok(const born_row_params& p) {
    const bool fin = isfinite(p.temperature) && isfinite(p.top_p) && isfinite(p.repetition_penalty) &&
                     isfinite(p.frequency_penalty) && isfinite(p.presence_penalty);
    return fin && p.temperature >= 0.0f && (p.temperature == 0.0f || p.temperature >= 1e-4f) && p.top_p >= 0.0f &&
           p.min_p >= 0.0f && p.min_p <= 1.0f && p.top_k >= 0 && p.top_k <= BORN_MAX_TOP_K && p.repetition_penalty >= 0.0f;
}
__device__ __forceinline__ bool penalties_on(const born_row_params& rp) {
    return (rp.repetition_penalty != 1.0f && rp.repetition_penalty != 0.0f) || rp.frequency_penalty != 0.0f ||
           rp.presence_penalty != 0.0f;
}

// Route classes the streaming kernel is instantiated for, so that a launch whose rows all take
// the same kind of route does not carry (and pay, in registers and instruction fetches) the code
// of the others: 0 any route (decided per row at run time: per-row parameter arrays, and the
// whole-vocabulary routes), 1 running-maximum thresholds only (greedy, min-p with or without
// top-p), 2 top-k (lane-maxima bound, with or without min-p).
template <int kRoute>
struct RouteOf {
    static constexpr bool mass = kRoute == 0;  // rows may take their total from the mass blocks
    static constexpr bool lane = kRoute != 1;  // rows may use the lane-maxima bound
};

// What a row's parameters ask of the streaming pass.
struct RowPlan {
    bool greedy;
    bool lane_bound;   // top-k with k <= kThreads: threshold from the lane maxima
    bool no_bound;     // top-k beyond that: nothing is collected, the row takes the exact fallback
    bool use_max;      // threshold follows the running maximum (greedy, min-p, nucleus window)
    bool window;       // ... and that threshold is a guess that the finish verifies (top-p alone)
    bool need_mass;    // no top-k and no min-p: the row total comes from the mass blocks
    bool collect;
    int k;             // top-k (0: off)
    float inv_T, c2, delta;
};
__device__ __forceinline__ RowPlan row_plan(const born_row_params& rp) {
    RowPlan p;
    p.greedy = (rp.flags & BORN_FLAG_GREEDY) || rp.temperature == 0.0f;
    p.inv_T = p.greedy ? 1.0f : __fdiv_rn(1.0f, rp.temperature);
    p.c2 = p.inv_T * 1.44269504f;
    p.k = (!p.greedy && rp.top_k > 0) ? rp.top_k : 0;
    const bool minp = !p.greedy && rp.min_p > 0.0f;
    const bool topp = !p.greedy && rp.top_p > 0.0f && rp.top_p < 1.0f;
    p.lane_bound = p.k > 0 && p.k <= kThreads;
    p.no_bound = p.k > kThreads;
    p.need_mass = !p.greedy && p.k == 0 && !minp;
    p.window = p.need_mass && topp;
    p.use_max = p.greedy || minp || p.window;
    p.delta = 0.0f;
    if (minp) p.delta = (__logf(rp.min_p) - 0.05f) * rp.temperature;
    else if (p.window) p.delta = -kNucleusWindow * rp.temperature;
    p.collect = p.greedy || p.k > 0 || minp || p.window;
    return p;
}

}  // namespace born
