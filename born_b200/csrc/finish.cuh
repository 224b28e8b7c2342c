// Finishing a row: merge the segment records, select (top-k -> min-p -> top-p on exact
// integer masses) and draw by inverse CDF in ascending token index.  Runs in the CTA that
// completes the row (scan_kernel) or in merge_kernel over all-gathered shard records.
//
// Every decision sum is an exact integer sum of fixed-point masses
// q = rne(exp_det((z - m) * inv_T) * 2^40), so thread order cannot matter.  Rank order is
// (value descending, token index ascending): the first maximum wins, as in the reference's
// argmax (born: internal/nn/cross_entropy.go:241-251).
#pragma once
#include "scan_common.cuh"

namespace born {

struct PackedHdr {  // 32 bytes: header of a packed shard / segment record (the all-gather payload)
    float m;        // maximum of the shard's row (NaN if a NaN was seen)
    float lse_s;    // sum of 2^((z - m) * c2)
    uint32_t count; // entries that follow: rank keys, best first
    uint32_t flags; // bit 0: the shard held more than `count` candidates; bit 1: the record is not exact
    float bound;
    uint32_t pad[3];
};
static_assert(sizeof(PackedHdr) == kRecordHdrBytes, "packed header size");

struct RowOut {   // where a finished row reports
    int32_t* token; float* prob; float* lse; int32_t* status; int32_t* kept_ids; int32_t* kept_count;
    int kept_stride;
    int row;
};
__device__ __forceinline__ void row_fail(const RowOut& o, int status) {
    if (threadIdx.x == 0) {
        o.token[o.row] = -1;
        o.status[o.row] = status;
        if (o.prob) o.prob[o.row] = 0.0f;
        if (o.kept_count) o.kept_count[o.row] = 0;
    }
}

struct SelectIn {
    int n;          // entries in sel[]: rank keys, all alive
    int k;          // keep the k best first (0: keep all)
    unsigned long long Qa;     // min-p threshold on the masses (0: off)
    float top_p;    // (0,1): on
    unsigned long long S_ext;  // top-p total when the candidates are only the heavy part of the row (0: their own sum)
    bool complete;  // the candidates hold every token the row can keep
    float m_row, inv_T, u;
};

// Selection and draw over n <= kThreads candidates in shared memory (sel: rank keys, all alive;
// selq: scratch for their masses), one candidate per thread.  The rank of a candidate is the
// number of larger keys (keys are unique: the token index is part of them); candidates and
// masses are then re-written in rank order, and since a mass never grows along that order the
// kept set of every filter is a prefix of it, which every thread finds by walking the sorted
// masses itself.  Returns false when the nucleus is not inside the candidates (the caller then
// takes the exact fallback); all threads get the same answer.
__device__ __forceinline__ bool select_small(const SelectIn& in, uint64_t* sel, unsigned long long* selq, ScanShared& sh,
                                             const RowOut& o) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = in.n;
    const int k_eff = in.k > 0 ? in.k : 0x7fffffff;
    const bool topp = in.top_p > 0.0f && in.top_p < 1.0f;
    const bool mine = tid < n;
    uint64_t ck = mine ? sel[tid] : 0ull;
    int rank = 0;
    {   // (eight broadcast loads in flight: the loop is bound by latency otherwise)
        int j = 0;
        for (; j + 8 <= n; j += 8) {
            uint64_t v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = sel[j + i];
#pragma unroll
            for (int i = 0; i < 8; ++i) rank += (v[i] > ck) ? 1 : 0;
        }
        for (; j < n; ++j) rank += (sel[j] > ck) ? 1 : 0;
    }
    uint64_t q = 0;
    if (mine && rank < k_eff) {
        const float x = scaled_shift(ck_z(ck), in.m_row, in.inv_T);
        q = (x < -30.0f) ? 0ull : mass_of(x);
        if (in.Qa && q < in.Qa) { q = 0; ck &= (uint64_t)kIdxMask; }  // min-p: a dead entry keeps its index only
    }
    cta_sync();  // every thread has read sel[] for its rank
    const int nk = min(n, k_eff);
    if (mine && rank < nk) { sel[rank] = ck; selq[rank] = q; }
    if (tid == 0) { sh.acc[0] = 0; sh.nw = 0; }
    cta_sync();
    // the entry of rank `tid`, and the mass ahead of it
    const uint64_t c2 = tid < nk ? sel[tid] : 0ull;
    const uint64_t q2 = tid < nk ? (uint64_t)selq[tid] : 0ull;
    uint64_t incl = q2;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint64_t up = shfl_up_u64(incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) sh.red64[warp] = incl;
    cta_sync();
    uint64_t off = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w) {
        const uint64_t x = sh.red64[w];
        if (w < warp) off += x;
        tot += x;
    }
    const uint64_t before = off + incl - q2;
    uint64_t Tp = ~0ull;
    if (topp) {
        Tp = __double2ull_rz(__dmul_rn((double)in.top_p, __ull2double_rn(in.S_ext ? in.S_ext : tot)));
        if (Tp < 1) Tp = 1;
    }
    // kept: alive and the mass ahead still short of the nucleus -- a prefix of the rank order;
    // its last entry of every warp reports the prefix's length and mass
    const bool kept = tid < nk && ck_alive(c2) && before < Tp;
    const uint32_t kb = __ballot_sync(0xffffffffu, kept);
    if (kb && lane == 31 - __clz(kb)) {
        atomicMax(&sh.nw, tid + 1);
        atomicMax(&sh.acc[0], (unsigned long long)(before + q2));
    }
    cta_sync();
    const int R = sh.nw;
    const uint64_t S = sh.acc[0];
    if (topp && in.S_ext && !in.complete && S < Tp) return false;  // (uniform)
    if (S == 0) {  // cannot happen while the row maximum is finite; never divide by it
        row_fail(o, BORN_ROW_ALL_MASKED);
        return true;
    }
    uint64_t t = __double2ull_rz(__dmul_rn((double)in.u, __ull2double_rn(S)));
    if (t > S - 1) t = S - 1;
    if (tid < R) {
        const uint32_t my_low = (uint32_t)(c2 & kIdxMask);  // larger low bits = smaller token index
        uint64_t pre = 0;
        int j = 0;
        for (; j + 8 <= R; j += 8) {
            uint64_t cj[8], qj[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { cj[i] = sel[j + i]; qj[i] = selq[j + i]; }
#pragma unroll
            for (int i = 0; i < 8; ++i) pre += ((uint32_t)(cj[i] & kIdxMask) > my_low) ? qj[i] : 0ull;
        }
        for (; j < R; ++j) pre += ((uint32_t)(sel[j] & kIdxMask) > my_low) ? (uint64_t)selq[j] : 0ull;
        if (pre <= t && t < pre + q2) {
            o.token[o.row] = ck_idx(c2);
            o.status[o.row] = BORN_ROW_OK;
            if (o.prob) o.prob[o.row] = __double2float_rn(__ddiv_rn(__ull2double_rn(q2), __ull2double_rn(S)));
        }
        if (o.kept_ids && tid < o.kept_stride) o.kept_ids[(int64_t)o.row * o.kept_stride + tid] = ck_idx(c2);
    }
    if (o.kept_count && tid == 0) o.kept_count[o.row] = R;
    return true;
}

// Selection and draw over kThreads < n <= kSelCap candidates: radix select, then mass-weighted
// radix threshold searches.  Same rules, same answer convention as select_small.
static __device__ __noinline__ bool select_and_draw(const SelectIn in, uint64_t* sel, unsigned long long* selq, ScanShared& sh,
                                             const RowOut o) {
    const int tid = threadIdx.x;
    const int n = in.n;
    const int k_eff = in.k > 0 ? in.k : 0x7fffffff;
    const bool topp = in.top_p > 0.0f && in.top_p < 1.0f;
    cta_sync();
    // ---- large set: radix select, then mass-weighted radix threshold searches
    if (n > k_eff) {
        const uint64_t T = block_radix_search<true, 56, true>(
            n, (unsigned long long)(k_eff - 1), [&](int i) { return sel[i]; }, [&](int) { return 1ull; }, sh.sc);
        for (int i = tid; i < n; i += kThreads)
            if (sel[i] < T) sel[i] &= (uint64_t)kIdxMask;
        cta_sync();
    }
    for (int i = tid; i < n; i += kThreads) {
        const uint64_t c = sel[i];
        uint64_t q = 0;
        if (ck_alive(c)) {
            const float x = scaled_shift(ck_z(c), in.m_row, in.inv_T);
            q = (x < -30.0f) ? 0ull : mass_of(x);
            if (in.Qa && q < in.Qa) { q = 0; sel[i] = c & (uint64_t)kIdxMask; }
        }
        selq[i] = q;
    }
    cta_sync();
    if (topp) {
        uint64_t part = 0;
        for (int i = tid; i < n; i += kThreads) part += selq[i];
        const uint64_t S = block_sum_u64(part, sh.red64);
        uint64_t Tp = __double2ull_rz(__dmul_rn((double)in.top_p, __ull2double_rn(in.S_ext ? in.S_ext : S)));
        if (Tp < 1) Tp = 1;
        if (in.S_ext && !in.complete && S < Tp) return false;
        if (S >= Tp) {
            // dead entries take part with weight 0 (their keys are unique small numbers)
            const uint64_t C = block_radix_search<true, 56, false>(
                n, Tp - 1, [&](int i) { return sel[i]; }, [&](int i) { return selq[i]; }, sh.sc);
            for (int i = tid; i < n; i += kThreads)
                if (sel[i] < C && ck_alive(sel[i])) { selq[i] = 0; sel[i] &= (uint64_t)kIdxMask; }
            cta_sync();
        }
    }
    uint64_t part = 0;
    for (int i = tid; i < n; i += kThreads) part += selq[i];
    const uint64_t S = block_sum_u64(part, sh.red64);
    if (S == 0) {
        row_fail(o, BORN_ROW_ALL_MASKED);
        return true;
    }
    uint64_t t = __double2ull_rz(__dmul_rn((double)in.u, __ull2double_rn(S)));
    if (t > S - 1) t = S - 1;
    // walk in ascending token index: key = index; dead entries weigh nothing but need unique keys
    const uint64_t tok64 = block_radix_search<false, 25, false>(
        n, t, [&](int i) { return ck_alive(sel[i]) ? (uint64_t)ck_idx(sel[i]) : ((1ull << 24) | (uint64_t)i); },
        [&](int i) { return selq[i]; }, sh.sc);
    const int tok = (int)tok64;
    for (int i = tid; i < n; i += kThreads) {
        if (ck_alive(sel[i]) && ck_idx(sel[i]) == tok) {
            o.token[o.row] = tok;
            o.status[o.row] = BORN_ROW_OK;
            if (o.prob) o.prob[o.row] = __double2float_rn(__ddiv_rn(__ull2double_rn(selq[i]), __ull2double_rn(S)));
        }
    }
    if (o.kept_count || o.kept_ids) {
        int alive = 0;
        for (int i = tid; i < n; i += kThreads) {
            const uint64_t c = sel[i];
            if (!ck_alive(c)) continue;
            ++alive;
            if (o.kept_ids) {
                int rank = 0;
                for (int j = 0; j < n; ++j) rank += (sel[j] > c) ? 1 : 0;
                if (rank < o.kept_stride) o.kept_ids[(int64_t)o.row * o.kept_stride + rank] = ck_idx(c);
            }
        }
        const uint64_t tot = block_sum_u64((uint64_t)alive, sh.red64);
        if (tid == 0 && o.kept_count) o.kept_count[o.row] = (int)tot;
    }
    return true;
}

// Block-wide reductions of the compute threads (results to every thread).
__device__ __forceinline__ float block_max_nan(float v, float* buf) {
    v = warp_max_nan(v);
    cta_sync();
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    cta_sync();
    float r = buf[0];
#pragma unroll
    for (int w = 1; w < kScanWarps; ++w) r = max_nan(r, buf[w]);
    return r;
}
__device__ __forceinline__ float block_sum_f32(float v, float* buf) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    cta_sync();
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    cta_sync();
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w) r += buf[w];
    return r;
}

__device__ __forceinline__ MassBlock load_block(const MassBlock* p) {
    const ulonglong2 v = __ldcg(reinterpret_cast<const ulonglong2*>(p));
    MassBlock b;
    b.m = __uint_as_float((uint32_t)v.x);
    b.pad = (uint32_t)(v.x >> 32);
    b.M = v.y;
    return b;
}

// One mass block's contribution to the row total: rne_u64((double)M_c * (double)exp_det((m_c - m) * inv_T)).
__device__ __forceinline__ unsigned long long block_share(const MassBlock& bk, float m, float inv_T) {
    if (!(bk.m > -INFINITY) || bk.M == 0) return 0ull;
    const float ef = exp_det(scaled_shift(bk.m, m, inv_T));
    return __double2ull_rn(__dmul_rn(__ull2double_rn(bk.M), (double)ef));
}

// Logit of token `tok` of virtual row (b, g) as the sampler sees it: upcast, history
// penalties, grammar mask.  O(history) per call; used by the paths that look at few tokens.
template <typename T>
__device__ __forceinline__ float token_logit(const ScanArgs& A, const born_row_params& rp, int b, int g, int tok) {
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)b * A.row_stride + (int64_t)g * A.V;
    float z;
    if constexpr (sizeof(T) == 4) z = __ldg(reinterpret_cast<const float*>(row) + tok);
    else z = bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(row) + tok));
    if (A.history && penalties_on(rp)) {
        int len = A.history_len ? A.history_len[b] : A.history_stride;
        len = max(0, min(min(len, A.history_stride), BORN_MAX_HISTORY));
        const int32_t* gh = A.history + (int64_t)b * A.history_stride;
        const int id = g * A.V + tok;
        int cnt = 0;
        for (int p = 0; p < len; ++p) cnt += (__ldg(gh + p) == id) ? 1 : 0;
        if (cnt > 0) z = penalise(rp, z, cnt);
    }
    if (A.mask) {
        const int64_t bi = (int64_t)g * A.V + tok;
        if (!((__ldg(A.mask + (int64_t)b * A.mask_stride + (bi >> 5)) >> (bi & 31)) & 1u)) z = -INFINITY;
    }
    return z;
}

// Temperature-only rows: the draw descends the mass blocks.  t = min(floor(u * S), S - 1)
// picks the block (ascending order, shares S_c), then the token inside it by the block's own
// masses: t'' = min(floor((t - before) * M_c / S_c), M_c - 1) in float64.
template <typename T>
__device__ __forceinline__ void draw_whole_row(const ScanArgs& A, ScanShared& sh, uint8_t* scratch, const RowOut& o,
                                               const born_row_params& rp, int b, int g, int row, float m, float inv_T,
                                               unsigned long long S, float u) {
    const int tid = threadIdx.x;
    const MassBlock* blocks = A.blocks + (int64_t)row * A.nblk;
    unsigned long long t = __double2ull_rz(__dmul_rn((double)u, __ull2double_rn(S)));
    if (t > S - 1) t = S - 1;
    unsigned long long run = 0;
    if (tid == 0) sh.found = -1;
    cta_sync();
    for (int base = 0; base < A.nblk; base += kThreads) {
        const int c = base + tid;
        MassBlock bk;
        bk.m = -INFINITY; bk.M = 0; bk.pad = 0;
        if (c < A.nblk) bk = load_block(blocks + c);
        const unsigned long long v = block_share(bk, m, inv_T);
        unsigned long long incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long up = shfl_up_u64(incl, d);
            if ((tid & 31) >= d) incl += up;
        }
        cta_sync();
        if ((tid & 31) == 31) sh.red64[tid >> 5] = incl;
        cta_sync();
        unsigned long long off = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kScanWarps; ++w) {
            const unsigned long long x = sh.red64[w];
            if (w < (tid >> 5)) off += x;
            total += x;
        }
        incl += off;
        if (run + total > t) {  // the block is in this chunk (uniform)
            if (run + incl > t && run + incl - v <= t) {
                sh.found = c;
                sh.before = run + incl - v;
            }
            cta_sync();
            break;
        }
        run += total;
    }
    cta_sync();
    const int c = sh.found;
    if (c < 0) {  // cannot happen: S is the sum of the shares
        row_fail(o, BORN_ROW_ALL_MASKED);
        return;
    }
    const MassBlock bk = load_block(blocks + c);
    const unsigned long long Sc = block_share(bk, m, inv_T);
    const unsigned long long tb = t - sh.before;
    unsigned long long tt = __double2ull_rz(__ddiv_rn(__dmul_rn(__ull2double_rn(tb), __ull2double_rn(bk.M)), __ull2double_rn(Sc)));
    if (tt > bk.M - 1) tt = bk.M - 1;
    // the block's tokens again, two consecutive ones per thread
    unsigned long long q[2];
    const int tok0 = c * kMassBlock + 2 * tid;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        q[i] = 0;
        if (tok0 + i < A.V) {
            const float z = token_logit<T>(A, rp, b, g, tok0 + i);
            q[i] = mass_of(scaled_shift(z, bk.m, inv_T));
        }
    }
    const unsigned long long v = q[0] + q[1];
    unsigned long long incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long up = shfl_up_u64(incl, d);
        if ((tid & 31) >= d) incl += up;
    }
    cta_sync();
    if ((tid & 31) == 31) sh.red64[tid >> 5] = incl;
    cta_sync();
    unsigned long long off = 0;
    for (int w = 0; w < (tid >> 5); ++w) off += sh.red64[w];
    incl += off;
    if (incl > tt && incl - v <= tt) {
        const int i = (incl - v + q[0] > tt) ? 0 : 1;
        o.token[o.row] = g * A.V + tok0 + i;
        o.status[o.row] = BORN_ROW_OK;
        if (o.prob) {
            const double p = __dmul_rn(__ddiv_rn(__ull2double_rn(q[i]), __ull2double_rn(bk.M)),
                                       __ddiv_rn(__ull2double_rn(Sc), __ull2double_rn(S)));
            o.prob[o.row] = __double2float_rn(p);
        }
    }
    (void)scratch;
}

template <typename T>
__device__ __noinline__ void fallback_row(const ScanArgs& A, ScanShared& sh, uint8_t* smem, int row);

// Exactly the k best of a virtual row, in rank order, into its packed record.
__device__ __forceinline__ void write_packed(const ScanArgs& A, ScanShared& sh, uint64_t* sel, unsigned long long* tmp_mem, int n, int k, int b, int g,
                                             float m, float lse_s, float bound, bool exact) {
    const int tid = threadIdx.x;
    uint8_t* rec = A.packed + (int64_t)g * A.packed_seg_stride + (int64_t)b * A.packed_row_stride;
    uint64_t* ent = reinterpret_cast<uint64_t*>(rec + kRecordHdrBytes);
    int nk = 0;
    if (exact && n > 0) {
        if (n > kThreads) {
            // cut to the k best first (k <= kThreads here), survivors to the front
            const uint64_t Tk = block_radix_search<true, 56, true>(
                n, (unsigned long long)(min(k, n) - 1), [&](int i) { return sel[i]; }, [&](int) { return 1ull; }, sh.sc);
            uint64_t* tmp = reinterpret_cast<uint64_t*>(tmp_mem);  // the mass array is idle here
            if (tid == 0) sh.nl = 0;
            cta_sync();
            for (int i = tid; i < n; i += kThreads)
                if (sel[i] >= Tk) tmp[smem_atom_add(&sh.nl, 1u)] = sel[i];
            cta_sync();
            n = sh.nl;
            for (int i = tid; i < n; i += kThreads) sel[i] = tmp[i];
            cta_sync();
        }
        const uint64_t ck = tid < n ? sel[tid] : 0ull;
        int rank = 0;
        for (int j = 0; j < n; ++j) rank += (sel[j] > ck) ? 1 : 0;
        nk = min(n, k);
        if (tid < n && rank < nk) ent[rank] = ck;
    }
    if (tid == 0) {
        PackedHdr h;
        h.m = m; h.lse_s = lse_s; h.count = (uint32_t)nk;
        h.flags = (exact ? 0u : 2u) | ((n > k) ? 1u : 0u);
        h.bound = bound;
        h.pad[0] = h.pad[1] = h.pad[2] = 0;
        memcpy(rec, &h, sizeof h);
    }
}

// Where a finished row's statistics and candidates come from: the segment records in scratch
// (a row streamed by several CTAs), or -- when one CTA streamed the whole row -- that CTA's
// own shared memory, without a round trip through L2.
struct RowSrc {
    bool direct;
    float m, ls, taux, bk;       // direct: the row's maximum, log-sum-exp sum, exclusion level, lane-maxima bound
    const uint64_t* wbuf;        // direct: the warps' candidate buffers (kScanWarps x kWarpCand raw entries)
    const uint32_t* wcount;
    int c_first, nseg;           // records: CTAs that hold a segment of the row
    int b, g;                    // the row: caller row and vocabulary segment
    float u;                     // the caller row's uniform, fetched while the row was streamed
    born_row_params rp;
    RowPlan plan;
};

// Hands row `row` to the exact search that its CTA runs once the ring is idle.  The reason goes in
// the upper byte.  A CTA that streams exactly one row keeps the word in shared memory (and spares
// every CTA a round trip to global memory at its end).
template <bool kOneRow>
__device__ __forceinline__ void defer_row(const ScanArgs& A, ScanShared& sh, int row, uint32_t why) {
    const uint32_t word = (why << 24) | (blockIdx.x + 1u);
    if constexpr (kOneRow) sh.defer = word;
    else A.deferred[row] = word;
}

// A row is complete: merge its statistics, select, draw.
// kOneRow: the instantiation only ever finishes rows straight from the shared memory of the CTA
// that streamed them, in sampling mode -- the record path and the k-best mode are left out of it.
template <typename T, int kRoute, bool kOneRow>
__device__ __forceinline__ void finish_row(const ScanArgs& A, ScanShared& sh, uint64_t* sel, unsigned long long* selq, int row,
                                           const RowSrc& src) {
    const int tid = threadIdx.x;
    const bool direct = kOneRow || src.direct;
    const bool local_mode = !kOneRow && A.mode == kScanLocal;
    const int nseg = src.nseg, c_first = src.c_first;
    const int b = src.b, g = src.g;
    const born_row_params& rp = src.rp;
    const RowPlan& pl = src.plan;
    auto rec_of = [&](int s) { return A.records + (int64_t)(row + c_first + s) * A.rec_stride; };

    // statistics: row maximum, exclusion level, best lane-maxima bound, log-sum-exp sum
    float m = src.m, taux = src.taux, bk = src.bk, ls = src.ls;
    const bool cached = nseg <= kHdrCache;
    if (!direct) {
        m = -INFINITY; taux = -INFINITY; bk = -INFINITY; ls = 0.0f;
        if (cached) {  // the headers are fetched once (one round trip to L2) and shared
            cta_sync();
            if (tid < nseg) {
                const uint8_t* rec = rec_of(tid);
                const float4 h = __ldcg(reinterpret_cast<const float4*>(rec));
                sh.hdr[tid] = h;
                sh.hdr_cnt[tid] = __ldcg(reinterpret_cast<const uint32_t*>(rec) + 4);
            }
            cta_sync();
            for (int s = 0; s < nseg; ++s) {
                const float4 h = sh.hdr[s];
                m = max_nan(m, h.x);
                taux = fmaxf(taux, h.z);
                bk = fmaxf(bk, h.w);
            }
            if (!(RouteOf<kRoute>::mass && pl.need_mass))
                for (int s = 0; s < nseg; ++s) {
                    const float4 h = sh.hdr[s];
                    if (h.y > 0.0f) ls += h.y * ex2_approx(__fmul_rn(h.x - m, pl.c2));
                }
        } else {
            for (int s = tid; s < nseg; s += kThreads) {
                const float4 h = __ldcg(reinterpret_cast<const float4*>(rec_of(s)));
                m = max_nan(m, h.x);
                taux = fmaxf(taux, h.z);
                bk = fmaxf(bk, h.w);
            }
            m = block_max_nan(m, sh.redf);
            taux = block_max_nan(taux, sh.redf2);
            bk = block_max_nan(bk, sh.redf3);
            if (!(RouteOf<kRoute>::mass && pl.need_mass)) {
                for (int s = tid; s < nseg; s += kThreads) {
                    const float4 h = __ldcg(reinterpret_cast<const float4*>(rec_of(s)));
                    if (h.y > 0.0f) ls += h.y * ex2_approx(__fmul_rn(h.x - m, pl.c2));
                }
                ls = block_sum_f32(ls, sh.redf);
            }
        }
    }
    auto count_of = [&](int s) { return cached ? (int)sh.hdr_cnt[s] : (int)__ldcg(reinterpret_cast<const uint32_t*>(rec_of(s)) + 4); };
    // every raw entry (value bits << 32 | token id) of the row, dealt over the threads
    auto for_entries = [&](auto f) {
        if (direct) {
            for (int idx = tid; idx < kScanWarps * kWarpCand; idx += kThreads) {
                const int w = idx / kWarpCand, i = idx - w * kWarpCand;
                if (i < (int)min(src.wcount[w], (uint32_t)kWarpCand)) f(src.wbuf[idx]);
            }
        } else {
            for (int s = 0; s < nseg; ++s) {
                const int cnt = count_of(s);
                const unsigned long long* ent = reinterpret_cast<const unsigned long long*>(rec_of(s) + kRecordHdrBytes);
                for (int i = tid; i < cnt; i += kThreads) f(__ldcg(ent + i));
            }
        }
    };
    int status = BORN_ROW_OK;
    if (m != m) status = BORN_ROW_NAN;
    else if (m == INFINITY) status = BORN_ROW_POS_INF;
    else if (m == -INFINITY) status = BORN_ROW_ALL_MASKED;

    if (local_mode) {
        // ---- the k best of the virtual row, in rank order
        int n = 0;
        if (status == BORN_ROW_OK) {
            if (tid == 0) sh.nl = 0;
            cta_sync();
            for_entries([&](unsigned long long e) {
                const float z = __uint_as_float((uint32_t)(e >> 32));
                if (z >= bk && z >= taux) {
                    const int pos = (int)smem_atom_add(&sh.nl, 1u);
                    if (pos < kSelCap) sel[pos] = make_ck(z, (int)(uint32_t)e);
                }
            });
            cta_sync();
            n = sh.nl;
            // complete above max(bk, taux); the k best are inside iff there are k of them (or nothing was excluded)
            if (n > kSelCap || (taux > bk && n < pl.k) || (RouteOf<kRoute>::lane && pl.no_bound)) {
                // the exact search over the row writes the record instead
                if (tid == 0) defer_row<kOneRow>(A, sh, row, 8u);
                return;
            }
        }
        write_packed(A, sh, sel, selq, n, pl.k, b, g, m, ls, bk, true);
        return;
    }

    RowOut o;
    o.token = A.out_token; o.prob = A.out_prob; o.lse = A.out_lse; o.status = A.out_status;
    o.kept_ids = A.out_kept_ids; o.kept_count = A.out_kept_count; o.kept_stride = A.kept_stride;
    o.row = b;
    if (A.row_params != nullptr && !row_params_ok(rp)) status = BORN_ROW_BAD_PARAMS;  // (device arrays are not checked on the host)
    if (status != BORN_ROW_OK) {
        if (tid == 0 && A.out_lse) A.out_lse[b] = NAN;
        row_fail(o, status);
        return;
    }
    if (!(RouteOf<kRoute>::mass && pl.need_mass) && A.out_lse && tid == 0) A.out_lse[b] = m * pl.inv_T + __log2f(ls) * 0.69314718f;

    if (pl.greedy) {
        if (taux > m) {  // a token equal to the maximum may have been lost to a full buffer
            if (tid == 0) defer_row<kOneRow>(A, sh, row, 1u);
            return;
        }
        uint64_t best = 0;
        for_entries([&](unsigned long long e) {
            const float z = __uint_as_float((uint32_t)(e >> 32));
            if (z >= m) best = max(best, make_ck(z, (int)(uint32_t)e));
        });
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) best = max(best, shfl_xor_u64(best, d));
        cta_sync();
        if ((tid & 31) == 0) sh.red64[tid >> 5] = best;
        cta_sync();
        if (tid == 0) {
            for (int w = 1; w < kScanWarps; ++w) best = max(best, (uint64_t)sh.red64[w]);
            const int tok = ck_idx(best);
            A.out_token[b] = tok;
            A.out_status[b] = BORN_ROW_OK;
            if (A.out_prob) A.out_prob[b] = 1.0f;
            if (A.out_kept_count) A.out_kept_count[b] = 1;
            if (A.out_kept_ids && A.kept_stride > 0) A.out_kept_ids[(int64_t)b * A.kept_stride] = tok;
        }
        return;
    }

    const float u = src.u;
    unsigned long long S_tot = 0;
    if ((RouteOf<kRoute>::mass && pl.need_mass)) {
        // row total from the mass blocks; log-sum-exp from it
        const MassBlock* blocks = A.blocks + (int64_t)row * A.nblk;
        unsigned long long part = 0;
        int fin = 0;
        for (int c = tid; c < A.nblk; c += kThreads) {
            const MassBlock bkc = load_block(blocks + c);
            part += block_share(bkc, m, pl.inv_T);
            fin += (int)bkc.pad;
        }
        S_tot = block_sum_u64(part, sh.red64);
        const int nfin = (int)block_sum_u64((uint64_t)fin, sh.red64);
        if (S_tot == 0) {
            row_fail(o, BORN_ROW_ALL_MASKED);
            return;
        }
        if (A.out_lse && tid == 0)
            A.out_lse[b] = (float)((double)m * (double)pl.inv_T + log(__ull2double_rn(S_tot) * (1.0 / 1099511627776.0)));
        if (!(RouteOf<kRoute>::mass && pl.window)) {
            if (A.out_kept_count && tid == 0) A.out_kept_count[b] = nfin;
            if (A.out_kept_ids) {  // the kept set is the whole row: no list of a useful size exists
                if (tid == 0) defer_row<kOneRow>(A, sh, row, 2u);
                return;
            }
            draw_whole_row<T>(A, sh, nullptr, o, rp, b, g, row, m, pl.inv_T, S_tot, u);
            return;
        }
    }

    // ---- candidates at or above the valid cut
    float cut = -INFINITY;
    if ((RouteOf<kRoute>::lane && pl.lane_bound)) cut = bk;
    if (rp.min_p > 0.0f) cut = fmaxf(cut, m + pl.delta);
    if ((RouteOf<kRoute>::mass && pl.window)) {
        // tokens lighter than (1 - P) * S / V weigh less than (1 - P) * S together: outside the nucleus
        const float s_all = (float)S_tot * (1.0f / 1099511627776.0f);
        cut = m + (__logf((1.0f - rp.top_p) * s_all / (float)A.V) - 0.05f) * rp.temperature;
    }
    bool complete = !(taux > cut);
    float lowest = complete ? cut : taux;  // below it the entries are not all there: not used
    // (sh.nl is zero on entry: the caller's last barrier saw to it)
    auto gather = [&](float low) {
        if (direct) {
            // a warp compacts its own buffer: one reservation per 32 entries
            const int lane = tid & 31, w = tid >> 5;
            const uint32_t cnt = min(src.wcount[w], (uint32_t)kWarpCand);
            const uint64_t* buf = src.wbuf + w * kWarpCand;
            for (uint32_t base = 0; base < cnt; base += 32) {
                const uint32_t i = base + lane;
                const uint64_t e = i < cnt ? buf[i] : 0ull;
                const float z = __uint_as_float((uint32_t)(e >> 32));
                const bool ok = i < cnt && z >= low;
                const uint32_t okb = __ballot_sync(0xffffffffu, ok);
                if (!okb) continue;
                uint32_t pos0 = 0;
                if (lane == 0) pos0 = smem_atom_add(&sh.nl, (uint32_t)__popc(okb));
                pos0 = __shfl_sync(0xffffffffu, pos0, 0);
                const uint32_t pos = pos0 + __popc(okb & ((1u << lane) - 1u));
                if (ok && pos < (uint32_t)kSelCap) sel[pos] = make_ck(z, (int)(uint32_t)e);
            }
        } else {
            for_entries([&](unsigned long long e) {
                const float z = __uint_as_float((uint32_t)(e >> 32));
                if (z >= low) {
                    const int pos = (int)smem_atom_add(&sh.nl, 1u);
                    if (pos < kSelCap) sel[pos] = make_ck(z, (int)(uint32_t)e);
                }
            });
        }
        cta_sync();
        return (int)sh.nl;
    };
    int n = gather(lowest);
    if (n > kSelCap && !(RouteOf<kRoute>::lane && pl.no_bound)) {
        // More candidates than the selection takes (a wide nucleus window, many ties).  Use only
        // the part above a higher level -- the lowest of a fixed ladder (in scaled-logit units
        // below the row maximum) that leaves at most kSelCap entries; that part is complete, and
        // the checks below decide whether the kept set lies inside it.
        constexpr int NL = 8;
        const float ladder[NL] = {8.0f, 6.5f, 5.0f, 4.0f, 3.0f, 2.0f, 1.0f, 0.5f};
        if (tid < NL) sh.sc.c[tid] = 0;
        cta_sync();
        for_entries([&](unsigned long long e) {
            const float z = __uint_as_float((uint32_t)(e >> 32));
            if (!(z >= lowest)) return;
            const float d = (m - z) * pl.inv_T;
            int lvl = -1;  // narrowest level that still holds the entry
#pragma unroll
            for (int l = 0; l < NL; ++l)
                if (d <= ladder[l]) lvl = l;
            if (lvl >= 0) smem_red_add(&sh.sc.c[lvl], 1u);
        });
        cta_sync();
        int pick = -1;
        uint32_t cum = 0;
        // entries inside level l = those whose narrowest level is >= l: cumulative from the narrow end
        for (int l = NL - 1; l >= 0; --l) {
            cum += sh.sc.c[l];
            if (cum <= (uint32_t)kSelCap) pick = l;
        }
        cta_sync();
        if (pick >= 0) {
            const float low2 = m - ladder[pick] * rp.temperature;
            if (low2 > lowest) {
                lowest = low2;
                complete = false;
                if (tid == 0) sh.nl = 0;
                cta_sync();
                n = gather(lowest);
            }
        }
    }
    // why a row goes to the exact search (kept in the upper byte of its `deferred` word)
    uint32_t why = 0;
    if ((RouteOf<kRoute>::lane && pl.no_bound)) why = 4;
    else if (n > kSelCap) why = 3;
    else if (!complete) {
        if (pl.k > 0) { if (n < pl.k) why = 5; }   // the k best are all at or above taux iff k tokens are
        else if (!(RouteOf<kRoute>::mass && pl.window)) why = 6;              // min-p survivors may lie below taux
    }
    bool defer = why != 0;
    if (!defer) {
        SelectIn in;
        in.n = n;
        in.k = pl.k;
        in.Qa = (rp.min_p > 0.0f) ? __double2ull_ru((double)rp.min_p * 1099511627776.0) : 0ull;
        in.top_p = rp.top_p;
        in.S_ext = (RouteOf<kRoute>::mass && pl.window) ? S_tot : 0ull;
        in.complete = complete;
        in.m_row = m; in.inv_T = pl.inv_T; in.u = u;
        if (n <= kThreads) defer = !select_small(in, sel, selq, sh, o);
        else defer = !select_and_draw(in, sel, selq, sh, o);
        if (defer) why = 7;                        // the nucleus reaches below the candidates
    }
    if (defer && tid == 0) defer_row<kOneRow>(A, sh, row, why);
}

}  // namespace born
