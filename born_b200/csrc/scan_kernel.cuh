// scan_kernel: the streaming pass of the sampler.
//
// One launch does penalties -> grammar mask -> row max / log-sum-exp -> candidate collection
// (top-k, min-p, nucleus) or whole-row mass blocks, and -- in the CTA that completes a row --
// the selection and the inverse-CDF draw (finish.cuh).  Every logit crosses HBM once.
//
// A CTA is 8 compute warps and one producer warp and streams a contiguous range of 16 KB
// tiles (scan_common.cuh): all tiles of all rows form one sequence, cut evenly over the CTAs,
// so a CTA may stream part of a row, a whole row, or several.  The part of a row inside one
// CTA is a segment.  The producer keeps four tiles in flight (five where the instantiation's
// shared memory has the room: scan_stages) with 1-D bulk copies (TMA, no multicast) that complete on `full` mbarriers; the compute warps hand a tile back with one
// arrival each on its `empty` mbarrier.  Every thread reads a fixed share of each tile (16
// values in four 16-byte vectors).  Inside a segment the warps meet only after its first tile
// (threshold bootstrap) and at its end (statistics, record or finish).
//
// Token histories.  At the start of a segment the compute threads build, in shared memory, the
// list of the row's distinct history tokens grouped by tile (hist_build).  In fp32 launches the
// producer warp then writes the penalised value over the logit in every tile that has landed
// and releases the tile on a second barrier (`ready`), so the compute warps never see an
// unpenalised logit; in bf16 launches (a bf16 tile cannot hold the value) the compute warps
// take the token out of the tile and feed its penalised value to the statistics and the
// candidates themselves (hist_apply).
//
// Full tiles of an aligned row after the segment's first run through a short steady-state loop
// (wait, one read of the thresholds, the straight-line tile body, the hand-back); everything
// that is decided once per segment stays outside it.
//
// Candidates.  A value reaches the slow path only when it is at or above the warp's
// threshold tau (one compare per 16 values).  tau is the maximum of
//   * the lane-maxima bound (top-k <= 256): every lane's running maximum belongs to a
//     different token, so the j-th largest of a warp's 32 lane maxima, j = ceil(k / 8),
//     minimised over the 8 warps, has at least k tokens at or above it;
//   * running maximum + delta (greedy: delta 0; min-p: T * (ln min_p - 0.05); top-p alone: a
//     window that the finish verifies against the exact row total);
//   * the CTA's exclusion level, raised when a candidate finds its warp's 256-entry buffer full
//     (the buffers are compacted against the current threshold when half full).
// The first two never exclude a token the row can keep.  The third (and the nucleus window)
// may; they are recorded as tau_excl, and a row whose kept set is not provably inside the
// complete part of its candidates takes the exact fallback instead (fallback.cuh).
//
// The greedy branch keeps the reference's tie rule -- the first maximum wins
// (born: internal/nn/cross_entropy.go:241-251); the row arithmetic keeps its structure
// (maximum, exp of the shifted logits, sum: internal/autodiff/ops/softmax.go:214-238).
#pragma once
#include <float.h>
#include "scan_common.cuh"
#include "finish.cuh"

namespace born {

struct ThreadStats {
    float mx;   // running maximum (NaN-propagating)
    float R;    // reference of the online log-sum-exp (z domain)
    float nRc;  // -R * c2
    float2 s;   // two partial sums of 2^((z - R) * c2)
    float pub;  // largest maximum this thread has published
};
__device__ __forceinline__ void stats_reset(ThreadStats& st, float c2) {
    st.mx = -INFINITY;
    st.R = -1e30f;
    st.nRc = 1e30f * c2;
    st.s = make_float2(0.0f, 0.0f);
    st.pub = -INFINITY;
}
template <bool kLse>
__device__ __forceinline__ void stats_one(ThreadStats& st, float z, float c2) {
    st.mx = max_nan(st.mx, z);
    if (kLse) {
        if (z > st.R && z < INFINITY) {
            const float f = ex2_approx(__fmul_rn(st.R - z, c2));
            st.s.x *= f;
            st.s.y *= f;
            st.R = z;
            st.nRc = -z * c2;
        }
        st.s.x += ex2_approx(fmaf(z, c2, st.nRc));
    }
}
// Online log-sum-exp of 16 values: the reference moves at most once (to their maximum mt),
// then the terms are formed two at a time with packed fp32x2 operations in two chains.
__device__ __forceinline__ void lse16(ThreadStats& st, const float (&v)[16], float mt, float c2) {
    if (mt > st.R && mt < INFINITY) {
        const float f = ex2_approx(__fmul_rn(st.R - mt, c2));
        st.s = __fmul2_rn(st.s, make_float2(f, f));
        st.R = mt;
        st.nRc = -mt * c2;
    }
    const float2 cc = make_float2(c2, c2), rr = make_float2(st.nRc, st.nRc);
    float2 s1 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        const float2 t0 = __ffma2_rn(make_float2(v[i], v[i + 1]), cc, rr);
        const float2 t1 = __ffma2_rn(make_float2(v[i + 2], v[i + 3]), cc, rr);
        st.s = __fadd2_rn(st.s, make_float2(ex2_approx(t0.x), ex2_approx(t0.y)));
        s1 = __fadd2_rn(s1, make_float2(ex2_approx(t1.x), ex2_approx(t1.y)));
    }
    st.s = __fadd2_rn(st.s, s1);
}

// One candidate from the lane that found it, into the warp's own buffer.  A candidate that finds
// the buffer full raises the CTA's exclusion level above itself: nothing at or below that level
// counts as collected any more, and every warp's threshold follows (current_tau).
__device__ __forceinline__ void push_cand(uint64_t* wbuf, uint32_t* wcount, uint32_t* excl, float z, int id) {
    const uint32_t pos = smem_atom_add(wcount, 1u);
    if (pos < (uint32_t)kWarpCand) wbuf[pos] = ((uint64_t)__float_as_uint(z) << 32) | (uint32_t)id;
    else smem_red_max(excl, key_above(z));
}

// A warp's buffer is half full: drop what lies below the threshold as it stands now.  Every
// part of the threshold only rises, and the finish uses nothing below its final value, so what
// goes is never missed -- while a buffer full of entries from the time the threshold was still
// low would turn away the candidates that count.  Called by the whole warp.
__device__ __forceinline__ void compact_cands(uint64_t* wbuf, uint32_t* wcount, float tau) {
    const int lane = threadIdx.x & 31;
    const uint32_t n = min(*reinterpret_cast<volatile uint32_t*>(wcount), (uint32_t)kWarpCand);
    uint32_t kept = 0;
    for (uint32_t base = 0; base < n; base += 32) {
        const uint32_t i = base + lane;
        const uint64_t e = i < n ? wbuf[i] : 0ull;
        const bool keep = i < n && __uint_as_float((uint32_t)(e >> 32)) >= tau;
        const uint32_t kb = __ballot_sync(0xffffffffu, keep);
        __syncwarp();  // the chunk is in registers before any of it is overwritten
        if (keep) wbuf[kept + __popc(kb & ((1u << lane) - 1u))] = e;
        kept += __popc(kb);
    }
    __syncwarp();
    if (lane == 0) *reinterpret_cast<volatile uint32_t*>(wcount) = kept;
    __syncwarp();
}

struct SegCtx {   // what the compute threads know about the segment they are in (block-uniform)
    RowPlan plan;
    int row, id0;       // virtual row; token id of the row's token 0 as written to candidates
    float tau_fix;      // lane-maxima bound / exclusion level (warp-uniform, only rises)
};

__device__ __forceinline__ float current_tau(const SegCtx& sg, const ScanShared& sh) {
    // (maxbits, excl_bits) sit side by side: one 8-byte read
    const unsigned long long both = *reinterpret_cast<const volatile unsigned long long*>(&sh.maxbits);
    float tau = fmaxf(sg.tau_fix, zkey_to_float((uint32_t)(both >> 32)));
    if (sg.plan.use_max) tau = fmaxf(tau, zkey_to_float((uint32_t)both) + sg.plan.delta);
    return tau;
}
__device__ __forceinline__ void publish_max(ThreadStats& st, ScanShared& sh) {
    if (st.mx > st.pub) {
        st.pub = st.mx;
        smem_red_max(&sh.maxbits, zkey(st.mx));
    }
}

// j-th largest of the warp's 32 lane maxima, j = ceil(k / 8): the warp's share of the
// lane-maxima bound.  Published for the other warps; returns the minimum over all warps.
__device__ __forceinline__ float lane_bound(ScanShared& sh, int k, float mx) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t key = zkey((mx == mx) ? mx : -INFINITY);
    const int j = (k + kScanWarps - 1) / kScanWarps;
    uint32_t kj;
    if (j == 1) {
        kj = __reduce_max_sync(0xffffffffu, key);
    } else {
#pragma unroll
        for (int kk = 2; kk <= 32; kk <<= 1) {
#pragma unroll
            for (int d = kk >> 1; d > 0; d >>= 1) {
                const uint32_t other = __shfl_xor_sync(0xffffffffu, key, d);
                const bool up = ((lane & kk) == 0), lower = ((lane & d) == 0);
                key = (up == lower) ? max(key, other) : min(key, other);
            }
        }
        kj = __shfl_sync(0xffffffffu, key, j - 1);
    }
    if (lane == 0) *reinterpret_cast<volatile float*>(&sh.wbound[warp]) = zkey_to_float(kj);
    __syncwarp();
    float m = *reinterpret_cast<const volatile float*>(&sh.wbound[0]);
#pragma unroll
    for (int i = 1; i < kScanWarps; ++i) m = fminf(m, *reinterpret_cast<const volatile float*>(&sh.wbound[i]));
    return m;
}

// ---- tiles ----------------------------------------------------------------------------------
// 16 values of a thread's share of the tile, batch h (fp32: one batch of four 16-byte vectors;
// bf16: two batches of two).  Two ways to deal the tile's 1024 vectors to the threads:
//   * interleaved (vector tid + 256*j): a partial tile still reaches every lane, which the
//     lane-maxima bound needs -- the candidate routes;
//   * warp slices (vector warp*128 + lane + 32*j): a warp owns 512 (fp32) or 1024 (bf16)
//     consecutive logits, i.e. whole mass blocks -- the whole-vocabulary routes.
// Either way a warp's 128-bit shared loads are conflict-free.
template <typename T, bool kMask, bool kWarpSlice>
__device__ __forceinline__ void load16(const T* tile, const uint32_t* smask, int h, float (&v)[16], int (&e0)[16 / VecOf<T>::n]) {
    constexpr int VEC = VecOf<T>::n, NV = 16 / VEC;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int vi = kWarpSlice ? warp * 128 + lane + 32 * (h * NV + j) : (int)threadIdx.x + kThreads * (h * NV + j);
        e0[j] = vi * VEC;
        if constexpr (VEC == 4) {
            const float4 q = reinterpret_cast<const float4*>(tile)[vi];
            v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
        } else {
            const uint4 q = reinterpret_cast<const uint4*>(tile)[vi];
            v[8 * j] = __uint_as_float(q.x << 16); v[8 * j + 1] = __uint_as_float(q.x & 0xFFFF0000u);
            v[8 * j + 2] = __uint_as_float(q.y << 16); v[8 * j + 3] = __uint_as_float(q.y & 0xFFFF0000u);
            v[8 * j + 4] = __uint_as_float(q.z << 16); v[8 * j + 5] = __uint_as_float(q.z & 0xFFFF0000u);
            v[8 * j + 6] = __uint_as_float(q.w << 16); v[8 * j + 7] = __uint_as_float(q.w & 0xFFFF0000u);
        }
        if constexpr (kMask) {
            const uint32_t bits = smask[e0[j] >> 5] >> (e0[j] & 31);
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[VEC * j + i] = ((bits >> i) & 1u) ? v[VEC * j + i] : -INFINITY;
        }
    }
}

// Element e of a tile as the candidate buffer wants it (the value is re-read from shared
// memory: a hit is rare, and this keeps the hot loop free of sixteen copies of the push).
template <typename T>
__device__ __forceinline__ float tile_elem(const T* tile, int e) {
    if constexpr (sizeof(T) == 4) return reinterpret_cast<const float*>(tile)[e];
    else return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(tile)[e]);
}
template <typename T>
__device__ __forceinline__ void push_hits(uint32_t hits, const T* tile, int h, int id_tile0, ThreadStats& st,
                                          uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int VEC = VecOf<T>::n, NV = 16 / VEC;
#pragma unroll 1
    while (hits) {
        const int i = __ffs(hits) - 1;
        hits &= hits - 1;
        const int e = ((int)threadIdx.x + kThreads * (h * NV + i / VEC)) * VEC + (i % VEC);
        push_cand(wbuf, wcount, excl, tile_elem<T>(tile, e), id_tile0 + e);
    }
}

// Which of a thread's 16 values are candidates (at or above tau, and not -inf): only the groups of
// four whose maximum m4[g] reaches tau are looked at, with one compare per value -- a threshold of
// -inf is replaced by the lowest finite value, which every value above -inf reaches and -inf does
// not.  The warp runs this whenever any of its lanes has a hit, which for top-k is most of the time.
__device__ __forceinline__ uint32_t hit_mask(const float (&v)[16], const float (&m4)[4], float tau) {
    const float tf = fmaxf(tau, -3.402823466e38f);
    uint32_t hits = 0;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (m4[g] >= tf) {
#pragma unroll
            for (int i = 0; i < 4; ++i) hits |= (v[4 * g + i] >= tf) ? (1u << (4 * g + i)) : 0u;
        }
    }
    return hits;
}

// A full tile of a 16-byte-aligned row: straight-line code, one compare per 16 values.
template <typename T, bool kMask, bool kLse>
__device__ __forceinline__ void fast_tile(const T* tile, const uint32_t* smask, int id_tile0, float tau, float c2,
                                          ThreadStats& st, uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int VEC = VecOf<T>::n, NV = 16 / VEC, NB = TileOf<T>::n / (kThreads * 16);
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        float v[16];
        int e0[NV];
        load16<T, kMask, false>(tile, smask, h, v, e0);
        float m4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) m4[i] = max_nan(max3_nan(v[4 * i], v[4 * i + 1], v[4 * i + 2]), v[4 * i + 3]);
        const float mt = max_nan(max3_nan(m4[0], m4[1], m4[2]), m4[3]);
        st.mx = max_nan(st.mx, mt);
        if constexpr (kLse) lse16(st, v, mt, c2);
        if (mt >= tau) {  // rare per lane
            push_hits<T>(hit_mask(v, m4, tau), tile, h, id_tile0, st, wbuf, wcount, excl);
        }
    }
    __syncwarp();
}

// Two full fp32 tiles at once: their loads, maxima and exponentials are independent, which gives
// the warp twice the work in flight per dependent step -- with 18 warps per SM that, not issue
// slots, is what the tile loop runs out of -- and the per-tile overhead of the loop once.
template <bool kMask, bool kLse>
__device__ __forceinline__ void fast_tile_pair(const float* tile_a, const uint32_t* smask_a, const float* tile_b,
                                               const uint32_t* smask_b, int id_tile0, float tau, float c2, ThreadStats& st,
                                               uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int TILE = TileOf<float>::n;
    float va[16], vb[16];
    int e0[4];
    load16<float, kMask, false>(tile_a, smask_a, 0, va, e0);
    load16<float, kMask, false>(tile_b, smask_b, 0, vb, e0);
    float ma[4], mb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        ma[i] = max_nan(max3_nan(va[4 * i], va[4 * i + 1], va[4 * i + 2]), va[4 * i + 3]);
        mb[i] = max_nan(max3_nan(vb[4 * i], vb[4 * i + 1], vb[4 * i + 2]), vb[4 * i + 3]);
    }
    const float mta = max_nan(max3_nan(ma[0], ma[1], ma[2]), ma[3]);
    const float mtb = max_nan(max3_nan(mb[0], mb[1], mb[2]), mb[3]);
    const float mt = max_nan(mta, mtb);
    st.mx = max_nan(st.mx, mt);
    if constexpr (kLse) {
        if (mt > st.R && mt < INFINITY) {
            const float f = ex2_approx(__fmul_rn(st.R - mt, c2));
            st.s = __fmul2_rn(st.s, make_float2(f, f));
            st.R = mt;
            st.nRc = -mt * c2;
        }
        const float2 cc = make_float2(c2, c2), rr = make_float2(st.nRc, st.nRc);
        float2 s1 = make_float2(0.0f, 0.0f), s2 = s1, s3 = s1;
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            const float2 a0 = __ffma2_rn(make_float2(va[i], va[i + 1]), cc, rr), a1 = __ffma2_rn(make_float2(va[i + 2], va[i + 3]), cc, rr);
            const float2 b0 = __ffma2_rn(make_float2(vb[i], vb[i + 1]), cc, rr), b1 = __ffma2_rn(make_float2(vb[i + 2], vb[i + 3]), cc, rr);
            st.s = __fadd2_rn(st.s, make_float2(ex2_approx(a0.x), ex2_approx(a0.y)));
            s1 = __fadd2_rn(s1, make_float2(ex2_approx(a1.x), ex2_approx(a1.y)));
            s2 = __fadd2_rn(s2, make_float2(ex2_approx(b0.x), ex2_approx(b0.y)));
            s3 = __fadd2_rn(s3, make_float2(ex2_approx(b1.x), ex2_approx(b1.y)));
        }
        st.s = __fadd2_rn(__fadd2_rn(st.s, s1), __fadd2_rn(s2, s3));
    }
    if (mta >= tau) push_hits<float>(hit_mask(va, ma, tau), tile_a, 0, id_tile0, st, wbuf, wcount, excl);  // rare per lane
    if (mtb >= tau) push_hits<float>(hit_mask(vb, mb, tau), tile_b, 0, id_tile0 + TILE, st, wbuf, wcount, excl);
    __syncwarp();
}

// The thread's maximum over its share of a full tile, nothing else: what the threshold bootstrap
// of a segment's first tile needs before the tile is processed like any other.
template <typename T, bool kMask>
__device__ __forceinline__ float tile_max(const T* tile, const uint32_t* smask) {
    constexpr int VEC = VecOf<T>::n, NV = 16 / VEC, NB = TileOf<T>::n / (kThreads * 16);
    float pm = -INFINITY;
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        float v[16];
        int e0[NV];
        load16<T, kMask, false>(tile, smask, h, v, e0);
        float m4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) m4[i] = max_nan(max3_nan(v[4 * i], v[4 * i + 1], v[4 * i + 2]), v[4 * i + 3]);
        pm = max_nan(pm, max_nan(max3_nan(m4[0], m4[1], m4[2]), m4[3]));
    }
    return pm;
}

// The last tile of an aligned row is partial: the copy brought n_el elements and left the rest
// of the stage as it was.  Every thread blanks its own elements from n_el on (-inf), after
// which the tile is a full one.  (The caller orders these writes before the stage's next copy.)
template <typename T>
__device__ __forceinline__ void pad_tile(T* tile, int n_el) {
    constexpr int VEC = VecOf<T>::n, ITER = TileOf<T>::n / (kThreads * VEC);
#pragma unroll
    for (int jj = 0; jj < ITER; ++jj) {
        const int e0 = ((int)threadIdx.x + kThreads * jj) * VEC;
        if (e0 + VEC <= n_el) continue;
        if (e0 >= n_el) {
            if constexpr (sizeof(T) == 4) reinterpret_cast<float4*>(tile)[e0 / VEC] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            else reinterpret_cast<uint4*>(tile)[e0 / VEC] = make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
        } else {
            for (int i = n_el - e0; i < VEC; ++i) {
                if constexpr (sizeof(T) == 4) reinterpret_cast<float*>(tile)[e0 + i] = -INFINITY;
                else reinterpret_cast<uint16_t*>(tile)[e0 + i] = 0xFF80u;
            }
        }
    }
}

// Candidates of a full tile whose statistics were taken before (the first tile of a segment,
// once its threshold exists): compact code, run once per segment.
template <typename T, bool kMask>
__device__ __forceinline__ void collect_tile(const T* tile, const uint32_t* smask, int id_tile0, float tau,
                                             ThreadStats& st, uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int VEC = VecOf<T>::n, ITER = TileOf<T>::n / (kThreads * VEC);
#pragma unroll 1
    for (int j = 0; j < ITER; ++j) {
        const int e0 = ((int)threadIdx.x + kThreads * j) * VEC;
        uint32_t bits = 0xFFFFFFFFu;
        if constexpr (kMask) bits = smask[e0 >> 5] >> (e0 & 31);
#pragma unroll 1
        for (int i = 0; i < VEC; ++i) {
            const float z = tile_elem<T>(tile, e0 + i);
            if (((bits >> i) & 1u) && z >= tau && z > -INFINITY) push_cand(wbuf, wcount, excl, z, id_tile0 + e0 + i);
        }
    }
    __syncwarp();
}

// Any tile: partial, of a row that does not start on a 16-byte boundary, or with mask words
// that do not line up with the vectors.  Element e of the tile counts when lo <= e < hi.
template <typename T, bool kMask, bool kLse>
__device__ __forceinline__ void slow_tile(const T* tile, const uint32_t* smask, int64_t mb_rel, int lo, int hi,
                                          int id_tile0, float tau, float c2, bool stats, bool collect,
                                          ThreadStats& st, uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int VEC = VecOf<T>::n, ITER = TileOf<T>::n / (kThreads * VEC);
#pragma unroll 1
    for (int j = 0; j < ITER; ++j) {
        const int vi = (int)threadIdx.x + kThreads * j;
#pragma unroll 1
        for (int i = 0; i < VEC; ++i) {
            const int e = vi * VEC + i;
            if (e < lo || e >= hi) continue;
            float z;
            if constexpr (sizeof(T) == 4) z = reinterpret_cast<const float*>(tile)[e];
            else z = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(tile)[e]);
            if constexpr (kMask) {
                const int64_t bi = mb_rel + e;  // bit index relative to the first loaded mask word
                if (!((smask[bi >> 5] >> (bi & 31)) & 1u)) z = -INFINITY;
            }
            if (stats) stats_one<kLse>(st, z, c2);
            if (collect && z >= tau && z > -INFINITY) push_cand(wbuf, wcount, excl, z, id_tile0 + e);
        }
    }
    __syncwarp();
}

// Whole-vocabulary routes: the warp's slice is one (fp32) or two (bf16) mass blocks.  Per block
// the maximum m_c and the exact mass M_c relative to it go to scratch; candidates (nucleus
// window) are collected as elsewhere.  Rows of these routes start on a 16-byte boundary.
template <typename T, bool kMask>
__device__ __forceinline__ void mass_tile(const T* tile, const uint32_t* smask, int hi, int tok_tile0, int id_tile0,
                                          float tau, float inv_T, bool collect, MassBlock* row_blocks, int nblk,
                                          ThreadStats& st, ScanShared& sh, uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int VEC = VecOf<T>::n, NV = 16 / VEC, NB = TileOf<T>::n / (kThreads * 16);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        float v[16];
        int e0[NV];
        load16<T, kMask, true>(tile, smask, h, v, e0);
        if (hi < TileOf<T>::n) {  // (a row's partial last tile: block-uniform)
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (e0[i / VEC] + (i % VEC) >= hi) v[i] = -INFINITY;
        }
        float m4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) m4[i] = max_nan(max3_nan(v[4 * i], v[4 * i + 1], v[4 * i + 2]), v[4 * i + 3]);
        const float mt = max_nan(max3_nan(m4[0], m4[1], m4[2]), m4[3]);
        st.mx = max_nan(st.mx, mt);
        const float mb = warp_max_nan(mt);
        unsigned long long q = 0;
        int fin = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) fin += (v[i] > -INFINITY) ? 1 : 0;
        fin = __reduce_add_sync(0xffffffffu, fin);
        const bool live = mb > -INFINITY && mb < INFINITY;  // false for NaN as well
        if (live) {
#pragma unroll
            for (int i = 0; i < 16; ++i) q += mass_of(scaled_shift(v[i], mb, inv_T));
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) q += shfl_xor_u64(q, d);
        }
        // block index: the warp's slice starts at element warp * (128 * VEC) + h * (64 * VEC) of the tile
        const int blk = (tok_tile0 + warp * 128 * VEC + h * (TileOf<T>::n / (kScanWarps * NB))) / kMassBlock;
        if (lane == 0 && blk < nblk) {
            MassBlock o;
            o.m = mb; o.pad = (uint32_t)fin; o.M = q;
            row_blocks[blk] = o;
        }
        if (collect) {
            publish_max(st, sh);
            if (mt >= tau) {
                uint32_t hits = hit_mask(v, m4, tau);
#pragma unroll 1
                while (hits) {
                    const int i = __ffs(hits) - 1;
                    hits &= hits - 1;
                    const int e = (warp * 128 + lane + 32 * (h * NV + i / VEC)) * VEC + (i % VEC);
                    push_cand(wbuf, wcount, excl, tile_elem<T>(tile, e), id_tile0 + e);
                }
            }
        }
    }
    __syncwarp();
}

// ---- producer ---------------------------------------------------------------------------------
struct TilePos {   // where global tile t lies
    int row, j;    // virtual row, tile within it
};
__device__ __forceinline__ TilePos tile_pos(long long t, int tpr) {
    TilePos p;
    // (a 64-bit division is a subroutine of a hundred instructions on the way to a CTA's first copy)
    if (t <= 0x7FFFFFFFll) p.row = (int)((uint32_t)t / (uint32_t)tpr);
    else p.row = (int)(t / tpr);
    p.j = (int)(t - (long long)p.row * tpr);
    return p;
}

template <typename T, bool kMask>
__device__ __forceinline__ void producer_issue(const ScanArgs& A, ScanShared& sh, uint8_t* smem, const ScanSmem& L,
                                               long long t, const TilePos& p, const RowGeom& q, int stage) {
    constexpr int TILE = TileOf<T>::n;
    const int n_el = min(TILE, q.lead + A.V - p.j * TILE);
    const int lo = max(0, q.lead - p.j * TILE);
    uint64_t* bar = reinterpret_cast<uint64_t*>(&sh.full_bar[stage]);
    uint32_t bytes_l = 0, bytes_m = 0;
    MaskTile mt;
    if (n_el > lo) {
        bytes_l = ((uint32_t)n_el * (uint32_t)sizeof(T) + 15u) & ~15u;
        if constexpr (kMask) {
            mt = mask_tile<T>(A, q, p.j, lo, n_el);
            bytes_m = (uint32_t)mt.nw * 4u;
        }
    }
    if (t == A.debug_skip_tile) {  // test hook: the barrier expects bytes that never come
        mbar_expect_tx(bar, 16u);
        return;
    }
    mbar_expect_tx(bar, bytes_l + bytes_m);
    if (bytes_l)
        bulk_load(smem + L.tiles + (size_t)stage * kTileBytes, q.abase + (size_t)p.j * kTileBytes, bytes_l, bar);
    if constexpr (kMask) {
        if (bytes_m)
            bulk_load(smem + L.masks + (size_t)stage * (mask_stage_words<T>() * 4),
                      A.mask + (int64_t)q.b * A.mask_stride + mt.w0a, bytes_m, bar);
    }
}

// Cursor over the CTA's tiles: (row, tile within the row) advanced without divisions.
template <typename T>
struct TileCursor {
    TilePos p;
    RowGeom q;
    __device__ __forceinline__ void start(const ScanArgs& A, long long t) {
        p = tile_pos(t, A.tpr);
        q = row_geom<T>(A, p.row);
    }
    // the CTA streams exactly row `row` (no divisions on the way to the first copy)
    __device__ __forceinline__ void start_row(const ScanArgs& A, int row) {
        p.row = row;
        p.j = 0;
        q = row_geom<T, true>(A, row);
    }
    // returns true when the next tile opens a new row
    __device__ __forceinline__ bool next(const ScanArgs& A, bool more) {
        if (++p.j < A.tpr) return false;
        p.j = 0;
        ++p.row;
        if (more) q = row_geom<T>(A, p.row);
        return true;
    }
};

// The producer warp: keeps the ring full.  Step n waits (bounded) for the stage of tile n to be
// handed back by the compute warps and issues its copy.
template <typename T, bool kMask, bool kOneRow, int kStages>
__device__ __forceinline__ void producer_loop(const ScanArgs& A, ScanShared& sh, uint8_t* smem, const ScanSmem& L,
                                              long long t0, long long t1) {
    const int lane = threadIdx.x & 31;
    const int n_tiles = (int)(t1 - t0);
    int n = 0, stage = 0;
    uint32_t round = 0;
    bool ok = true;
    TileCursor<T> ci;
    if constexpr (kOneRow) ci.start_row(A, (int)blockIdx.x);
    else ci.start(A, t0);
    for (; n < n_tiles; ++n) {
        if (n >= kStages &&
            !mbar_wait_limit(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage]), (round - 1u) & 1u, A.timeout_ns, &sh.fail)) {
            ok = false;
            break;
        }
        if (lane == 0) producer_issue<T, kMask>(A, sh, smem, L, t0 + n, ci.p, ci.q, stage);
        ci.next(A, n + 1 < n_tiles);
        if (++stage == kStages) { stage = 0; ++round; }
    }
    if (!ok) sh.fail = 1;
    // what the failure path of the compute threads needs to know (see the end of scan_kernel)
    if (lane == 0) {
        sh.issued = t0 + n;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&sh.prod_done) = 1;
    }
}

// The producer warp of an fp32 launch with token histories.  Besides keeping the ring full it
// applies the history penalties to every tile once it has landed -- the penalised value is
// written in place -- and only then hands the tile to the compute warps (`ready`), which so
// never see an unpenalised logit and spend nothing on it.  The list of a segment's history
// tokens is built by the compute threads (hist_build); `hist_seq` says for how many of the
// CTA's segments it has been.  The warp never blocks on one thing while the other could move:
// it alternates between "issue the next copy if its stage is free" and "patch and release the
// next tile if it has landed", and sleeps a few dozen nanoseconds when neither can.
template <typename T, bool kMask, bool kOneRow, int kStages>
__device__ __forceinline__ void producer_loop_patching(const ScanArgs& A, ScanShared& sh, uint8_t* smem, const ScanSmem& L,
                                                       long long t0, long long t1) {
    constexpr int TILE = TileOf<T>::n;
    const int lane = threadIdx.x & 31;
    const int n_tiles = (int)(t1 - t0);
    int n_i = 0, stage_i = 0;   // next tile to issue
    uint32_t round_i = 0;
    int n_p = 0, stage_p = 0;   // next tile to patch and release
    uint32_t round_p = 0;
    TileCursor<T> ci, cp;
    if constexpr (kOneRow) { ci.start_row(A, (int)blockIdx.x); cp = ci; }
    else { ci.start(A, t0); cp.start(A, t0); }
    int seg_p = 0;              // ordinal of the segment the release cursor is in
    bool seg_open = false;      // ... and whether its list has been taken over
    int n_list = 0, pos = 0;
    born_row_params rp = A.params;
    const unsigned long long* list = reinterpret_cast<const unsigned long long*>(smem + L.hist);
    unsigned long long idle_since = 0;
    bool ok = true;
    while (n_p < n_tiles) {
        bool moved = false;
        if (n_i < n_tiles &&
            (n_i < kStages || mbar_test(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage_i]), (round_i - 1u) & 1u))) {
            if (lane == 0) producer_issue<T, kMask>(A, sh, smem, L, t0 + n_i, ci.p, ci.q, stage_i);
            ++n_i;
            ci.next(A, n_i < n_tiles);
            if (++stage_i == kStages) { stage_i = 0; ++round_i; }
            moved = true;
        }
        if (n_p < n_i && mbar_test(reinterpret_cast<uint64_t*>(&sh.full_bar[stage_p]), round_p & 1u)) {
            if (!seg_open && *reinterpret_cast<const volatile int*>(&sh.hist_seq) > seg_p) {
                // (the compute threads' writes of the list are ordered before their write of hist_seq)
                __threadfence_block();
                n_list = *reinterpret_cast<const volatile int*>(&sh.hist_n);
                rp = sh.hist_rp;
                pos = 0;
                seg_open = true;
            }
            if (seg_open) {
                bool wrote = false;
                if (n_list > 0) {
                    float* tile = reinterpret_cast<float*>(smem + L.tiles + (size_t)stage_p * kTileBytes);
                    for (;;) {
                        const int idx = pos + lane;
                        const unsigned long long e = idx < n_list ? list[idx] : ~0ull;
                        const int off = (int)(uint32_t)e + cp.q.lead - cp.p.j * TILE;
                        const bool in = idx < n_list && off >= 0 && off < TILE;
                        const int c = __popc(__ballot_sync(0xffffffffu, in));
                        if (in && (e >> 32) != 0) {  // (0: a repeat of a token listed before)
                            tile[off] = penalise(rp, tile[off], (int)(e >> 32));
                            wrote = true;
                        }
                        pos += c;
                        if (c < 32) break;
                    }
                }
                if (wrote) fence_proxy_async();  // the stage is next written by a bulk copy
                __syncwarp();
                if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&sh.ready_bar[stage_p]));
                ++n_p;
                if (cp.next(A, n_p < n_tiles)) { ++seg_p; seg_open = false; }
                if (++stage_p == kStages) { stage_p = 0; ++round_p; }
                moved = true;
            }
        }
        if (moved) {
            idle_since = 0;
        } else {
            __nanosleep(40);
            if (*reinterpret_cast<const volatile int*>(&sh.fail)) { ok = false; break; }
            const unsigned long long now = global_timer_ns();
            if (idle_since == 0) idle_since = now;
            else if (now - idle_since > A.timeout_ns) { ok = false; break; }
        }
    }
    if (!ok) sh.fail = 1;
    if (lane == 0) {
        sh.issued = t0 + n_i;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&sh.prod_done) = 1;
    }
}

// ---- token history -----------------------------------------------------------------------------
// Penalties touch at most BORN_MAX_HISTORY tokens of a row.  At the start of a segment the
// compute threads turn the row's history into a list of its distinct tokens with their
// multiplicities, grouped by the tile they fall into (only the tiles of this segment), in shared
// memory: hist_build for segments of up to kHistNarrowTiles tiles, hist_build_wide beyond.  The
// global read of the ids is the only memory round trip; for a CTA's first row it leaves before
// the CTA's first copies.
//
// The list is applied tile by tile, in step with the stream: by the producer warp in fp32
// launches (producer_loop_patching), by the compute warps in bf16 launches (hist_apply: a warp
// applies the entries that fall into its own share of the tile -- the warp that reads an
// element is the only one that ever touches it, so a warp-level sync is all it takes).
constexpr int kHistPer = BORN_MAX_HISTORY / kThreads;  // history ids per compute thread
struct HistCursor {
    int n, pos;
};

__device__ __forceinline__ void hist_ids(const ScanArgs& A, int b, int (&ids)[kHistPer]) {
    // the ids do not wait for the length: both reads leave together, the length cuts afterwards
    const int cap = min(A.history_stride, (int)BORN_MAX_HISTORY);
    const int32_t* gh = A.history + (int64_t)b * A.history_stride;
#pragma unroll
    for (int r = 0; r < kHistPer; ++r) {
        const int p = (int)threadIdx.x + r * kThreads;
        ids[r] = p < cap ? __ldg(gh + p) : -1;
    }
    const int len = A.history_len ? __ldg(A.history_len + b) : cap;
#pragma unroll
    for (int r = 0; r < kHistPer; ++r)
        if ((int)threadIdx.x + r * kThreads >= len) ids[r] = -1;
}

// Segments of more than kHistNarrowTiles tiles (rows beyond some 260 000 fp32 logits): a hash table
// in the candidate area (empty at that point) removes the repeats; counters in the selection area
// -- per (tile, warp) up to 128 tiles, so that the warps do not meet on the same word -- drive a
// counting sort into the list.
template <int TILE>
__device__ __noinline__ int hist_build_wide(const ScanArgs& A, const int (&ids)[kHistPer], int g, int lead, int j_begin, int j_end,
                                          uint32_t* keys, uint32_t* cnt32, unsigned long long* list, uint32_t* wscr) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int span = j_end - j_begin;
    // the table: a power of two of at least twice the ids there can be
    const int cap = min(A.history_stride, (int)BORN_MAX_HISTORY);
    int lg = 6;
    while ((1 << lg) < 2 * cap) ++lg;
    const int slots = 1 << lg;
    uint32_t* mult = keys + slots;  // repeats, beside the keys
    const int P = span <= 128 ? kScanWarps : 1;
    const int nc = span * P;
    {
        uint4* k4 = reinterpret_cast<uint4*>(keys);
        uint4* m4 = reinterpret_cast<uint4*>(mult);
        for (int i = tid; i < slots / 4; i += kThreads) {
            k4[i] = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
            m4[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        for (int i = tid; i < nc / 2 + 1; i += kThreads) cnt32[i] = 0;
    }
    cta_sync();
    // (shared-memory atomics are what this build costs: one per id for the table, one per new
    // token to count it, one to place it)
    int ctr_of[kHistPer];  // the token's counter if this thread was the first to insert it, else -1
#pragma unroll
    for (int r = 0; r < kHistPer; ++r) {
        ctr_of[r] = -1;
        const int id = ids[r];
        if (id < 0) continue;
        int g2 = 0;
        uint32_t tok = (uint32_t)id;
        if (A.G > 1) { g2 = id / A.V; tok = (uint32_t)(id - g2 * A.V); }
        if (g2 != g || tok >= (uint32_t)A.V) continue;  // another vocabulary segment's token, or an id beyond the vocabulary
        const int tl = (int)((tok + (uint32_t)lead) / (uint32_t)TILE);
        if (tl < j_begin || tl >= j_end) continue;
        uint32_t slot = (tok * 2654435761u) >> (32 - lg);
        for (int probe = 0; probe < slots; ++probe) {
            const uint32_t old = atomicCAS(&keys[slot], 0xFFFFFFFFu, tok);
            if (old == 0xFFFFFFFFu) {  // the first of its kind: this thread will place it
                const int c = (tl - j_begin) * P + (P > 1 ? warp : 0);
                smem_red_add(&cnt32[c >> 1], 1u << (16 * (c & 1)));
                ctr_of[r] = c;
                break;
            }
            if (old == tok) {  // a repeat
                smem_red_add(&mult[slot], 1u);
                break;
            }
            slot = (slot + 1) & (slots - 1);
        }
    }
    cta_sync();
    // exclusive scan of the counters (a thread takes `per` consecutive ones)
    uint16_t* cnt16 = reinterpret_cast<uint16_t*>(cnt32);
    const int per = (nc + kThreads - 1) / kThreads;
    const int lo = min(tid * per, nc), hi = min(lo + per, nc);
    uint32_t loc = 0;
    for (int i = lo; i < hi; ++i) loc += cnt16[i];
    uint32_t incl = loc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) wscr[warp] = incl;
    cta_sync();
    uint32_t off = 0, n = 0;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w) {
        const uint32_t x = wscr[w];
        if (w < warp) off += x;
        n += x;
    }
    uint32_t run = off + incl - loc;
    for (int i = lo; i < hi; ++i) {
        const uint32_t c = cnt16[i];
        cnt16[i] = (uint16_t)run;  // becomes the counter's write cursor
        run += c;
    }
    cta_sync();
#pragma unroll
    for (int r = 0; r < kHistPer; ++r) {
        const int c = ctr_of[r];
        if (c < 0) continue;
        uint32_t tok = (uint32_t)ids[r];
        if (A.G > 1) tok -= (uint32_t)((ids[r] / A.V) * A.V);
        uint32_t slot = (tok * 2654435761u) >> (32 - lg);  // (found again: cheaper than carried along)
        while (keys[slot] != tok) slot = (slot + 1) & (slots - 1);
        const uint32_t old = smem_atom_add(&cnt32[c >> 1], 1u << (16 * (c & 1)));
        list[(old >> (16 * (c & 1))) & 0xFFFFu] = ((unsigned long long)(mult[slot] + 1u) << 32) | tok;
    }
    cta_sync();
    return (int)n;
}

// The same list for a segment of at most kHistNarrowTiles tiles -- every row below some 260 000
// fp32 logits.  The build sits in front of the segment's first tile, and shared-memory atomics
// cost about two cycles per lane and SM, so there are two per id and nothing else that
// serialises: a compare-and-swap into a hash table tells a token's first occurrence from its
// repeats (which only count themselves beside the key), and for a first occurrence the atomic on
// the (tile, warp) counter counts the token and returns its place among the warp's tokens of that
// tile.  After one barrier every warp works out the starts of all (tile, warp) runs for itself
// -- a lane per tile, eight counters each, a shuffle scan -- and stores its tokens with their
// multiplicities.  Table and counters are cleared by the segment set-up.
constexpr int kHistNarrowTiles = 64;
template <int TILE>
__device__ __forceinline__ int hist_build(const ScanArgs& A, const int (&ids)[kHistPer], int g, int lead, int j_begin, int j_end,
                                          uint32_t* keys, uint32_t* cnt32, unsigned long long* list, uint32_t* wscr) {
    const int span = j_end - j_begin;
    if (span > kHistNarrowTiles) return hist_build_wide<TILE>(A, ids, g, lead, j_begin, j_end, keys, cnt32, list, wscr);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t* mult = keys + kHashSlots;  // repeats, beside the keys
    int rel[kHistPer];
    uint32_t tok[kHistPer], rank[kHistPer];
#pragma unroll
    for (int r = 0; r < kHistPer; ++r) {
        rel[r] = -1;
        tok[r] = 0;
        rank[r] = 0;
        const int id = ids[r];
        if (id < 0) continue;
        int g2 = 0;
        uint32_t tk = (uint32_t)id;
        if (A.G > 1) { g2 = id / A.V; tk = (uint32_t)(id - g2 * A.V); }
        if (g2 != g || tk >= (uint32_t)A.V) continue;  // another vocabulary segment's token, or an id beyond the vocabulary
        const int tl = (int)((tk + (uint32_t)lead) / (uint32_t)TILE);
        if (tl < j_begin || tl >= j_end) continue;
        uint32_t slot = (tk * 2654435761u) >> (32 - 11);
        bool fresh = false;
        for (int probe = 0; probe < kHashSlots; ++probe) {
            const uint32_t old = atomicCAS(&keys[slot], 0xFFFFFFFFu, tk);
            if (old == 0xFFFFFFFFu) { fresh = true; break; }
            if (old == tk) { smem_red_add(&mult[slot], 1u); break; }  // a repeat
            slot = (slot + 1) & (kHashSlots - 1);
        }
        if (!fresh) continue;
        rel[r] = tl - j_begin;
        tok[r] = tk;
        const int c = rel[r] * kScanWarps + warp;
        rank[r] = (smem_atom_add(&cnt32[c >> 1], 1u << (16 * (c & 1))) >> (16 * (c & 1))) & 0xFFFFu;
    }
    cta_sync();
    // lane l: tiles l and l + 32 -- the tile's total, and what the warps below this one hold of it
    uint32_t tot[2] = {0, 0}, below[2] = {0, 0};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int t = lane + 32 * h;
        if (t < span) {
            const uint4 v = reinterpret_cast<const uint4*>(cnt32)[t];  // eight 16-bit counters
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < kScanWarps; ++i) {
                const uint32_t c = (w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
                tot[h] += c;
                if (i < warp) below[h] += c;
            }
        }
    }
    uint32_t incl0 = tot[0], incl1 = tot[1];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t u0 = __shfl_up_sync(0xffffffffu, incl0, d), u1 = __shfl_up_sync(0xffffffffu, incl1, d);
        if (lane >= d) { incl0 += u0; incl1 += u1; }
    }
    const uint32_t sum0 = __shfl_sync(0xffffffffu, incl0, 31);
    const uint32_t n = sum0 + __shfl_sync(0xffffffffu, incl1, 31);
    const uint32_t base0 = incl0 - tot[0], base1 = sum0 + incl1 - tot[1];
#pragma unroll
    for (int r = 0; r < kHistPer; ++r) {
        const int src = rel[r] >= 0 ? (rel[r] & 31) : 0;
        const uint32_t v0 = __shfl_sync(0xffffffffu, base0 + below[0], src), v1 = __shfl_sync(0xffffffffu, base1 + below[1], src);
        if (rel[r] >= 0) {
            uint32_t slot = (tok[r] * 2654435761u) >> (32 - 11);  // (found again: cheaper than carried along)
            while (keys[slot] != tok[r]) slot = (slot + 1) & (kHashSlots - 1);
            list[((rel[r] >> 5) ? v1 : v0) + rank[r]] = ((unsigned long long)(mult[slot] + 1u) << 32) | tok[r];
        }
    }
    cta_sync();
    return (int)n;
}

// The history tokens of tile j, by the warp.  Bits of `mode`: 2 statistics of the values taken
// out of a bf16 tile, 4 their candidates (all of them when tau is -inf).  Returns whether the
// warp wrote to the tile.
template <typename T, bool kMask, bool kLse>
__device__ __forceinline__ bool hist_apply(HistCursor& hc, const unsigned long long* list, const born_row_params& rp, T* tile,
                                           const uint32_t* smask, int64_t mb_rel, int j, int lead, int lo_el, int n_el,
                                           bool slices, int mode, int id_row0, float tau, float c2, ThreadStats& st,
                                           uint64_t* wbuf, uint32_t* wcount, uint32_t* excl) {
    constexpr int TILE = TileOf<T>::n, VEC = VecOf<T>::n;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool wrote = false;
    int pos = hc.pos;
    for (;;) {
        const int idx = pos + lane;
        const unsigned long long e = idx < hc.n ? list[idx] : ~0ull;
        const int tok = (int)(uint32_t)e;
        const int off = tok + lead - j * TILE;
        const bool in = idx < hc.n && off >= 0 && off < TILE;
        const int c = __popc(__ballot_sync(0xffffffffu, in));
        if (in && off >= lo_el && off < n_el && (e >> 32) != 0) {  // (0: a repeat of a token listed before)
            const int vec = off / VEC;
            const int owner = slices ? (vec >> 7) : ((vec & (kThreads - 1)) >> 5);
            if (owner == warp) {
                const int cnt = (int)(e >> 32);
                if constexpr (sizeof(T) == 4) {
                    float* pz = reinterpret_cast<float*>(tile) + off;
                    *pz = penalise(rp, *pz, cnt);
                } else {
                    uint16_t* pz = reinterpret_cast<uint16_t*>(tile) + off;
                    float zp = penalise(rp, bf16_bits_to_f32(*pz), cnt);
                    if constexpr (kMask) {
                        const int64_t bi = mb_rel + off;
                        if (!((smask[bi >> 5] >> (bi & 31)) & 1u)) zp = -INFINITY;
                    }
                    *pz = 0xFF80u;
                    if (mode & 2) stats_one<kLse>(st, zp, c2);
                    if ((mode & 4) && zp >= tau && zp > -INFINITY) push_cand(wbuf, wcount, excl, zp, id_row0 + tok);
                }
                wrote = true;
            }
        }
        pos += c;
        if (c < 32) break;
    }
    hc.pos = pos;
    __syncwarp();
    return __any_sync(0xffffffffu, wrote);
}

// Device-resident history: the CTA that finished caller row b appends the sampled token to the
// row's ring (the next call reads the ring as its history), marks the row finished when the
// token is a stop token, and blanks the outputs of a row that had finished before.  One thread,
// after a barrier that follows the row's output writes.
__device__ __forceinline__ void ring_append(const ScanArgs& A, int b) {
    if (A.ring_finished[b]) {
        A.out_token[b] = -1;
        A.out_status[b] = BORN_ROW_FINISHED;
        if (A.out_prob) A.out_prob[b] = 0.0f;
        if (A.out_kept_count) A.out_kept_count[b] = 0;
        return;
    }
    const int tok = A.out_token[b];
    if (A.out_status[b] != BORN_ROW_OK || tok < 0) return;
    const int total = A.ring_total[b];
    A.ring[(int64_t)b * A.ring_cap + total % A.ring_cap] = tok;
    A.ring_total[b] = total + 1;
    A.ring_len[b] = min(total + 1, A.ring_cap);
    for (int i = 0; i < A.n_stop; ++i)
        if (A.stop_ids[i] == tok) A.ring_finished[b] = 1;
}

// ---- the kernel -------------------------------------------------------------------------------
// kPair: a launch without token histories -- no history code in the instantiation, the segment's
// first and last tile are taken inside the steady-state loop, and (fp32) that loop may take two
// tiles at a time; a separate instantiation so that the other launches keep their register
// allocation.
// kShortHist: the launch's histories have at most kHistShort ids per row (the host checks the
// stride): the list takes half the room, which without a mask buys a fifth stage.
// kOneRow: a sampling launch whose grid gives every CTA exactly one whole row (the host checks
// grid == rows and the mode), so the segment records, the tickets and the k-best mode are left
// out of the instantiation -- code that is never run still costs registers and instruction cache.
template <typename T, bool kMask, bool kLse, bool kPair, int kRoute, bool kOneRow, bool kShortHist>
__global__ void __launch_bounds__(kScanThreads, 2) scan_kernel(const __grid_constant__ ScanArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ ScanShared sh;
    constexpr int TILE = TileOf<T>::n;
    constexpr int kHistCap = kShortHist ? kHistShort : (int)BORN_MAX_HISTORY;
    constexpr int kStages = scan_stages(kMask, !kPair, kHistCap);  // (launches with a history never take a kPair instantiation)
    const int tid = threadIdx.x;
    // What the instantiation knows about token histories: kPair instantiations serve the launches
    // without one; of the others, the fp32 ones always have one (the producer warp applies it), the
    // bf16 ones look at run time (a launch with a history pointer; the compute warps apply it).
    constexpr bool kFp32 = sizeof(T) == 4;
    const bool has_hist = kPair ? false : (kFp32 ? true : (A.history != nullptr));
    constexpr bool prod_patch = kFp32 && !kPair;
    const ScanSmem L = scan_smem_layout((int)sizeof(T), kMask, has_hist, kHistCap);
    const long long rows = (long long)A.B * A.G;
    const long long T_total = rows * A.tpr;
    const long long ncta = gridDim.x;
    // (one row per CTA: the tile range is the row's, known without the 64-bit divisions)
    long long t0, t1;
    if constexpr (kOneRow) {
        t0 = (long long)blockIdx.x * A.tpr;
        t1 = t0 + A.tpr;
    } else if (T_total * (ncta + 1) <= 0xFFFFFFFFll) {  // (the products fit 32 bits: the same quotients, cheaply)
        t0 = (long long)(((uint32_t)blockIdx.x * (uint32_t)T_total) / (uint32_t)ncta);
        t1 = (long long)((((uint32_t)blockIdx.x + 1u) * (uint32_t)T_total) / (uint32_t)ncta);
    } else {
        t0 = range_begin(blockIdx.x, T_total, ncta);
        t1 = range_begin(blockIdx.x + 1, T_total, ncta);
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(reinterpret_cast<uint64_t*>(&sh.full_bar[s]), 1);
            mbar_init(reinterpret_cast<uint64_t*>(&sh.empty_bar[s]), kScanWarps);
            mbar_init(reinterpret_cast<uint64_t*>(&sh.ready_bar[s]), 1);
        }
        sh.hist_seq = 0;
        mbar_fence_init();
        sh.fail = 0;
        sh.prod_done = 0;
        sh.issued = t0;
    }
    // The history ids of the CTA's first row go ahead of the bulk copies: behind them they
    // would wait in the memory system's queues.
    int ids[kHistPer];
#pragma unroll
    for (int r = 0; r < kHistPer; ++r) ids[r] = -1;
    if (has_hist && tid < kThreads && t0 < t1) hist_ids(A, kOneRow ? (int)blockIdx.x : (int)(t0 / A.tpr) / A.G, ids);
    __syncthreads();  // the only barrier all 288 threads share

    if (tid >= kThreads) {
        if constexpr (prod_patch) producer_loop_patching<T, kMask, kOneRow, kStages>(A, sh, smem, L, t0, t1);
        else producer_loop<T, kMask, kOneRow, kStages>(A, sh, smem, L, t0, t1);
        return;
    }

    // ------------------------------------------------------------------------ compute threads
    const int lane = tid & 31, warp = tid >> 5;
    uint64_t* wbuf = reinterpret_cast<uint64_t*>(smem + L.cand) + warp * kWarpCand;
    uint32_t* wcount = &sh.wcount[warp];
    uint32_t* excl = &sh.excl_bits;
    bool failed = false;
    int bad = 0;
    // fp32 launches with token histories: the producer warp patches the tiles and releases them
    unsigned long long* const wait_bar = prod_patch ? sh.ready_bar : sh.full_bar;
    int seg_ord = -1;
    long long t = t0;
    int stage = 0;         // ring stage of tile t
    uint32_t phase = 0;    // ... and the parity of its use
    while (t < t1) {
        // ---- segment set-up (block-synchronous)
        TilePos p0;
        if constexpr (kOneRow) { p0.row = (int)blockIdx.x; p0.j = 0; }
        else p0 = tile_pos(t, A.tpr);
        const long long seg_begin = t;
        const long long seg_end = min(t1, (long long)(p0.row + 1) * A.tpr);
        ++seg_ord;
        const RowGeom q = row_geom<T, kOneRow>(A, p0.row);
        const born_row_params rp = A.row_params ? A.row_params[q.b] : A.params;
        SegCtx sg;
        sg.plan = row_plan(rp);
        sg.row = p0.row;
        sg.id0 = A.idx_base + q.g * A.V;
        sg.tau_fix = (RouteOf<kRoute>::lane && sg.plan.no_bound) ? INFINITY : -INFINITY;
        const RowPlan& pl = sg.plan;
        cta_sync();
        if (tid == 0) {
            sh.maxbits = zkey(-INFINITY);
            sh.excl_bits = zkey(-INFINITY);
            sh.rec_count = 0;
            if constexpr (kOneRow) sh.defer = 0;
            sh.nl = 0;  // (the row's finish counts its candidates here)
        }
        // the row's uniform is wanted at the very end: fetch it now
        const float u_row = (A.uniforms != nullptr && (kOneRow || A.mode == kScanFull)) ? __ldg(A.uniforms + q.b) : 0.0f;
        if (tid < kScanWarps) { sh.wbound[tid] = -INFINITY; sh.wcount[tid] = 0; }
        if (has_hist) {
            // the history build's (tile, warp) counters (kHistNarrowTiles x 8 of 16 bits) and its hash
            // table in the candidate area (keys empty, repeat counts zero)
            reinterpret_cast<uint32_t*>(smem + L.sel)[tid] = 0;
            uint4* k4 = reinterpret_cast<uint4*>(smem + L.cand);
            k4[tid] = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
            k4[tid + kThreads] = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
            k4[tid + 2 * kThreads] = make_uint4(0u, 0u, 0u, 0u);
            k4[tid + 3 * kThreads] = make_uint4(0u, 0u, 0u, 0u);
        }
        cta_sync();
        ThreadStats st;
        stats_reset(st, pl.c2);
        MassBlock* row_blocks = A.blocks + (int64_t)p0.row * A.nblk;
        const bool collect = pl.collect && !(RouteOf<kRoute>::lane && pl.no_bound);
        int seen = 0;  // tiles of this segment done
        int j = (int)(t - (long long)p0.row * A.tpr);       // tile within the row
        int rem = q.lead + A.V - j * TILE;                  // elements of the row from this tile on
        const int j_end = (int)(seg_end - (long long)p0.row * A.tpr);
        HistCursor hc;
        hc.n = 0; hc.pos = 0;
        const unsigned long long* hlist = reinterpret_cast<const unsigned long long*>(smem + L.hist);
        if (has_hist) {
            if (seg_ord > 0) hist_ids(A, q.b, ids);  // (those of the CTA's first row were fetched before the first copy)
            if (penalties_on(rp))
                hc.n = hist_build<TILE>(A, ids, q.g, q.lead, j, j_end, reinterpret_cast<uint32_t*>(smem + L.cand),
                                        reinterpret_cast<uint32_t*>(smem + L.sel), reinterpret_cast<unsigned long long*>(smem + L.hist),
                                        reinterpret_cast<uint32_t*>(sh.red64));
        }
        if (prod_patch && tid == 0) {  // (hist_build ended on a barrier: the list is complete)
            sh.hist_n = hc.n;
            sh.hist_rp = rp;
            __threadfence_block();
            *reinterpret_cast<volatile int*>(&sh.hist_seq) = seg_ord + 1;
        }
        const bool hist_on = !kPair && sizeof(T) == 2 && hc.n > 0;  // (fp32: the producer warp applies the list)
        const bool lean = A.fast && !(RouteOf<kRoute>::mass && pl.need_mass);
        for (; t < seg_end; ++t, ++seen, ++j, rem -= TILE) {
            // ---- the tiles of an aligned row.  Everything that is decided per segment stays outside;
            // what is left per tile is the wait, one read of the thresholds, the straight-line tile
            // body and the hand-back (plus the threshold bootstrap on a segment's first tile and the
            // padding of a row's partial last one).
            // (kPair instantiations also take a segment's first tile and a row's partial last tile in this
            // loop; the others leave those two to the general body below -- measured: the extra branches
            // cost the history launches more than the general body costs them)
            if (lean && !failed && (kPair || seen > 0)) {
                while (t < seg_end && (kPair || rem >= TILE)) {
                    uint64_t* fb = reinterpret_cast<uint64_t*>(&wait_bar[stage]);
                    bool here = mbar_try(fb, phase);
                    if (!here) here = mbar_wait_limit(fb, phase, A.timeout_ns, &sh.fail);
                    if (!__all_sync(0xffffffffu, here)) {
                        failed = true;
                        sh.fail = 1;
                        break;
                    }
                    T* tile = reinterpret_cast<T*>(smem + L.tiles + stage * kTileBytes);
                    const uint32_t* smask = reinterpret_cast<const uint32_t*>(smem + L.masks + stage * (mask_stage_words<T>() * 4));
                    bool patched = false;
                    if (kPair && rem < TILE) {  // the row's last tile: blank what the copy did not bring
                        pad_tile<T>(tile, rem);
                        patched = true;
                    }
                    if (kPair && seen == 0) {
                        // The segment's first tile.  bf16 history tokens are offered whatever their value (no
                        // threshold exists yet, and they are gone from the tile when one does; the finish drops
                        // what lies below its cut).  Then the threshold is bootstrapped from the threads' maxima:
                        // the warp's maximum opens the running-maximum threshold; for top-k the warps meet once
                        // and take the lane-maxima bound.
                        if (hist_on)
                            patched |= hist_apply<T, kMask, kLse>(hc, hlist, rp, tile, smask, 0, j, 0, 0, min(rem, TILE), false, 6, sg.id0,
                                                                  collect ? -INFINITY : INFINITY, pl.c2, st, wbuf, wcount, excl);
                        st.mx = max_nan(st.mx, tile_max<T, kMask>(tile, smask));
                        if (pl.use_max) {
                            const float wm = warp_max_nan(st.mx);
                            if (lane == 0 && wm == wm) smem_red_max(&sh.maxbits, zkey(wm));
                            st.pub = fmaxf(st.pub, (wm == wm) ? wm : -INFINITY);
                            __syncwarp();
                        }
                        if ((RouteOf<kRoute>::lane && pl.lane_bound)) {
                            lane_bound(sh, pl.k, st.mx);
                            cta_sync();
                            sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
                        }
                    }
                    const float tau = collect ? current_tau(sg, sh) : INFINITY;
                    if (hist_on && (!kPair || seen > 0))
                        patched |= hist_apply<T, kMask, kLse>(hc, hlist, rp, tile, smask, 0, j, 0, 0, kPair ? min(rem, TILE) : TILE, false, 6, sg.id0, tau,
                                                              pl.c2, st, wbuf, wcount, excl);
                    if constexpr (kPair && sizeof(T) == 4) {
                        // fp32: when the tile after this one has landed as well, the two are taken together
                        bool pair = false;
                        if (t + 1 < seg_end && rem >= 2 * TILE) {
                            const int s2 = stage + 1 == kStages ? 0 : stage + 1;
                            const uint32_t p2 = stage + 1 == kStages ? phase ^ 1u : phase;
                            pair = __all_sync(0xffffffffu, mbar_test(reinterpret_cast<uint64_t*>(&wait_bar[s2]), p2));  // (a probe that never suspends)
                            if (pair) {
                                const float* tile2 = reinterpret_cast<const float*>(smem + L.tiles + s2 * kTileBytes);
                                const uint32_t* smask2 = reinterpret_cast<const uint32_t*>(smem + L.masks + s2 * (mask_stage_words<T>() * 4));
                                fast_tile_pair<kMask, kLse>(reinterpret_cast<const float*>(tile), smask, tile2, smask2, sg.id0 + j * TILE, tau,
                                                            pl.c2, st, wbuf, wcount, excl);
                            }
                        }
                        if (!pair) fast_tile<T, kMask, kLse>(tile, smask, sg.id0 + j * TILE, tau, pl.c2, st, wbuf, wcount, excl);
                        if (pl.use_max) publish_max(st, sh);
                        const int n_done = pair ? 2 : 1;
                        if ((RouteOf<kRoute>::lane && pl.lane_bound) && ((seen > 0 && ((seen + 1) & seen) == 0) || (pair && ((seen + 2) & (seen + 1)) == 0)))
                            sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
                        if (collect && *reinterpret_cast<volatile uint32_t*>(wcount) >= (uint32_t)(kWarpCand / 2))
                            compact_cands(wbuf, wcount, current_tau(sg, sh));
                        if (patched) fence_proxy_async();  // (a padded last tile) the stage is next written by a bulk copy
                        __syncwarp();
                        for (int d = 0; d < n_done; ++d) {
                            if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage]));
                            if (++stage == kStages) { stage = 0; phase ^= 1u; }
                        }
                        t += n_done; seen += n_done; j += n_done; rem -= n_done * TILE;
                    } else {
                        fast_tile<T, kMask, kLse>(tile, smask, sg.id0 + j * TILE, tau, pl.c2, st, wbuf, wcount, excl);
                        if (pl.use_max) publish_max(st, sh);
                        if ((RouteOf<kRoute>::lane && pl.lane_bound) && seen > 0 && ((seen + 1) & seen) == 0) sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
                        if (collect && *reinterpret_cast<volatile uint32_t*>(wcount) >= (uint32_t)(kWarpCand / 2))
                            compact_cands(wbuf, wcount, current_tau(sg, sh));
                        if (patched) fence_proxy_async();  // the stage is next written by a bulk copy
                        __syncwarp();
                        if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage]));
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                        ++t; ++seen; ++j; rem -= TILE;
                    }
                }
                if (t >= seg_end) break;
            }
            if (!failed) {
                const bool here = mbar_wait_limit(reinterpret_cast<uint64_t*>(&wait_bar[stage]), phase, A.timeout_ns, &sh.fail);
                if (!__all_sync(0xffffffffu, here)) {  // (the warp gives up as one: what follows votes and shuffles)
                    failed = true;
                    sh.fail = 1;
                }
            }
            T* tile = reinterpret_cast<T*>(smem + L.tiles + stage * kTileBytes);
            const uint32_t* smask = reinterpret_cast<const uint32_t*>(smem + L.masks + stage * (mask_stage_words<T>() * 4));
            const int n_el = min(TILE, rem);
            const int lo = max(0, q.lead - j * TILE);
            const int tok_tile0 = j * TILE - q.lead;          // token (within the virtual row) of element 0
            const int id_tile0 = sg.id0 + tok_tile0;
            bool full = A.fast && n_el == TILE;
            bool patched = false;
            if (A.fast && !full && n_el > 0 && !failed && !(RouteOf<kRoute>::mass && pl.need_mass)) {
                pad_tile<T>(tile, n_el);
                full = true;
                patched = true;
            }
            int64_t mb_rel = 0;
            if constexpr (kMask) {
                if (!full && n_el > lo) {
                    const MaskTile mt = mask_tile<T>(A, q, j, lo, n_el);
                    mb_rel = mt.mb0 - 32 * mt.w0a;
                }
            }
            const bool first = (seen == 0);
            if (hist_on && !failed) {
                // (a bf16 segment's first tile: no threshold exists yet, and the values are gone from the
                // tile when one does -- every finite one is offered; the finish drops what lies below its cut)
                const float tau_h = !collect ? INFINITY : (first ? -INFINITY : current_tau(sg, sh));
                patched |= hist_apply<T, kMask, kLse>(hc, hlist, rp, tile, smask, mb_rel, j, q.lead, lo, n_el, (RouteOf<kRoute>::mass && pl.need_mass), 6, sg.id0,
                                                      tau_h, pl.c2, st, wbuf, wcount, excl);
            }
            // A segment's first tile, when it is a full one: the threshold is bootstrapped from the
            // threads' maxima alone, then the tile is processed like any other.
            const bool quick_first = first && full && !(RouteOf<kRoute>::mass && pl.need_mass) && !failed;
            if (quick_first) st.mx = max_nan(st.mx, tile_max<T, kMask>(tile, smask));
            if (!failed && n_el > lo) {
                if ((RouteOf<kRoute>::mass && pl.need_mass)) {
                    // (rows of these routes are 16-byte aligned: the host sees to it)
                    const float tau = first ? INFINITY : current_tau(sg, sh);
                    mass_tile<T, kMask>(tile, smask, n_el, tok_tile0, id_tile0, tau, pl.inv_T, collect && !first, row_blocks, A.nblk,
                                        st, sh, wbuf, wcount, excl);
                } else if (quick_first) {
                    // (processed below, once the threshold exists)
                } else if (first) {
                    // statistics only: the threshold does not exist yet (tau = +inf collects nothing)
                    slow_tile<T, kMask, kLse>(tile, smask, mb_rel, lo, n_el, id_tile0, 0.0f, pl.c2, true, false, st, wbuf, wcount, excl);
                } else {
                    {
                    const float tau = collect ? current_tau(sg, sh) : INFINITY;
                    if (full) fast_tile<T, kMask, kLse>(tile, smask, id_tile0, tau, pl.c2, st, wbuf, wcount, excl);
                    else slow_tile<T, kMask, kLse>(tile, smask, mb_rel, lo, n_el, id_tile0, tau, pl.c2, true, collect, st, wbuf, wcount, excl);
                    if (pl.use_max) publish_max(st, sh);
                    }
                }
            }
            if (first) {
                // Threshold bootstrap: the warp's maximum opens the running-maximum threshold; for
                // top-k the warps meet once and take the lane-maxima bound.  Then the first tile's
                // candidates are collected under it (the tile is still held).
                if (pl.use_max) {
                    const float wm = warp_max_nan(st.mx);
                    if (lane == 0 && wm == wm) smem_red_max(&sh.maxbits, zkey(wm));
                    st.pub = fmaxf(st.pub, (wm == wm) ? wm : -INFINITY);
                    __syncwarp();
                }
                if ((RouteOf<kRoute>::lane && pl.lane_bound)) {
                    lane_bound(sh, pl.k, st.mx);
                    cta_sync();
                    sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
                }
                if (quick_first) {
                    const float tau = collect ? current_tau(sg, sh) : INFINITY;
                    fast_tile<T, kMask, kLse>(tile, smask, id_tile0, tau, pl.c2, st, wbuf, wcount, excl);
                    if (pl.use_max) publish_max(st, sh);
                } else if (!failed && collect && n_el > lo) {
                    const float tau = current_tau(sg, sh);
                    // collect only: the values are read again
                    if (full) collect_tile<T, kMask>(tile, smask, id_tile0, tau, st, wbuf, wcount, excl);
                    else slow_tile<T, kMask, kLse>(tile, smask, mb_rel, lo, n_el, id_tile0, tau, pl.c2, false, true, st, wbuf, wcount, excl);
                }
            } else if ((RouteOf<kRoute>::lane && pl.lane_bound) && ((seen + 1) & seen) == 0) {
                // tighten the bound when the number of tiles seen doubles (no barrier: values of
                // warps that lag are older, hence lower, hence still valid)
                sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
            }
            if (collect && !failed && *reinterpret_cast<volatile uint32_t*>(wcount) >= (uint32_t)(kWarpCand / 2))
                compact_cands(wbuf, wcount, current_tau(sg, sh));
            if (patched) fence_proxy_async();  // the stage is next written by a bulk copy
            __syncwarp();
            if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage]));  // tile back to the producer
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }

        // ---- segment record (block-synchronous)
        const float wm = warp_max_nan(st.mx);
        float ws = 0.0f;
        if (kLse && !(RouteOf<kRoute>::mass && pl.need_mass)) {
            const float ssum = st.s.x + st.s.y;
            ws = (ssum > 0.0f && wm == wm) ? ssum * ex2_approx(__fmul_rn(st.R - wm, pl.c2)) : 0.0f;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, d);
        }
        if ((RouteOf<kRoute>::lane && pl.lane_bound)) lane_bound(sh, pl.k, st.mx);
        if (lane == 0) { sh.wmax[warp] = wm; sh.wsum[warp] = ws; }
        cta_sync();
        float m_seg = sh.wmax[0];
#pragma unroll
        for (int w = 1; w < kScanWarps; ++w) m_seg = max_nan(m_seg, sh.wmax[w]);
        float s_seg = 0.0f;
        if (kLse && !(RouteOf<kRoute>::mass && pl.need_mass)) {
#pragma unroll
            for (int w = 0; w < kScanWarps; ++w) {
                const float x = sh.wsum[w];
                if (x > 0.0f) s_seg += x * ex2_approx(__fmul_rn(sh.wmax[w] - m_seg, pl.c2));
            }
        }
        float bound_k = -INFINITY;
        if ((RouteOf<kRoute>::lane && pl.lane_bound)) {
            bound_k = sh.wbound[0];
#pragma unroll
            for (int w = 1; w < kScanWarps; ++w) bound_k = fminf(bound_k, sh.wbound[w]);
        }
        // nothing below the segment's final valid bounds can be kept by the row
        float cut = bound_k;
        float excl_window = -INFINITY;
        if (pl.use_max && m_seg == m_seg) {
            if ((RouteOf<kRoute>::mass && pl.window)) excl_window = m_seg + pl.delta;
            cut = fmaxf(cut, m_seg + pl.delta);
        }
        // A row that this CTA streamed from its first tile to its last needs no record and no
        // ticket: it is finished straight from shared memory.
        const bool whole = kOneRow || seg_begin == (long long)p0.row * A.tpr && seg_end == (long long)(p0.row + 1) * A.tpr;
        RowSrc src;
        src.b = q.b; src.g = q.g; src.u = u_row; src.rp = rp; src.plan = pl;
        bool finish_here;
        if (whole) {
            if (cta_sync_or(*reinterpret_cast<const volatile int*>(&sh.fail))) { bad = 1; break; }
            src.direct = true;
            src.m = m_seg; src.ls = s_seg; src.bk = bound_k;
            src.taux = (RouteOf<kRoute>::lane && pl.no_bound) ? INFINITY : fmaxf(zkey_to_float(sh.excl_bits), excl_window);
            src.wbuf = reinterpret_cast<const uint64_t*>(smem + L.cand);
            src.wcount = sh.wcount;
            src.c_first = (int)blockIdx.x; src.nseg = 1;
            finish_here = true;
        } else {
            uint8_t* rec = A.records + (int64_t)(p0.row + (int)blockIdx.x) * A.rec_stride;
            uint64_t* ent = reinterpret_cast<uint64_t*>(rec + kRecordHdrBytes);
            if (!failed && collect) {
                const uint32_t nw = min(*wcount, (uint32_t)kWarpCand);
                float lost2 = -INFINITY;
                for (uint32_t base = 0; base < nw; base += 32) {
                    const uint32_t i2 = base + lane;
                    uint64_t e = 0;
                    bool ok = false;
                    float z = -INFINITY;
                    if (i2 < nw) {
                        e = wbuf[i2];
                        z = __uint_as_float((uint32_t)(e >> 32));
                        ok = z >= cut;
                    }
                    const uint32_t okb = __ballot_sync(0xffffffffu, ok);
                    uint32_t basepos = 0;
                    if (lane == 0 && okb) basepos = smem_atom_add(&sh.rec_count, (uint32_t)__popc(okb));
                    basepos = __shfl_sync(0xffffffffu, basepos, 0);
                    if (ok) {
                        const uint32_t pos = basepos + __popc(okb & ((1u << lane) - 1u));
                        if (pos < (uint32_t)A.rec_cap) ent[pos] = e;
                        else lost2 = fmaxf(lost2, z);
                    }
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) lost2 = fmaxf(lost2, __shfl_xor_sync(0xffffffffu, lost2, d));
                if (lane == 0 && lost2 > -INFINITY) smem_red_max(&sh.excl_bits, key_above(lost2));
            }
            cta_sync();
            if (tid == 0) {
                SegHdr h;
                h.m = m_seg;
                h.lse_sum = s_seg;
                float te = zkey_to_float(sh.excl_bits);
                te = fmaxf(te, excl_window);
                if ((RouteOf<kRoute>::lane && pl.no_bound)) te = INFINITY;
                h.tau_excl = te;
                h.bound_k = bound_k;
                h.count = min(sh.rec_count, (uint32_t)A.rec_cap);
                h.pad[0] = h.pad[1] = h.pad[2] = 0;
                *reinterpret_cast<SegHdr*>(rec) = h;
            }
            if (cta_sync_or(*reinterpret_cast<const volatile int*>(&sh.fail))) { bad = 1; break; }  // (the same answer in every thread)
            if (tid == 0) {
                // the barrier above has ordered every thread's record writes before this fence, which
                // makes them visible to the CTA that draws the last ticket
                __threadfence();
                const int c_first = cta_of_tile((long long)p0.row * A.tpr, T_total, ncta);
                const int c_last = cta_of_tile((long long)(p0.row + 1) * A.tpr - 1, T_total, ncta);
                const uint32_t tk = atomicAdd(&A.tickets[p0.row], 1u);
                sh.last = (tk == (uint32_t)(c_last - c_first));
                if (sh.last) A.tickets[p0.row] = 0;  // ready for the next launch
                sh.c_first = c_first;
                sh.c_last = c_last;
            }
            cta_sync();
            finish_here = sh.last != 0;
            if (finish_here) {
                __threadfence();
                src.direct = false;
                src.m = src.ls = src.taux = src.bk = 0.0f;
                src.wbuf = nullptr; src.wcount = nullptr;
                src.c_first = sh.c_first; src.nseg = sh.c_last - sh.c_first + 1;
            }
        }
        // (one call site: the finish is inlined, its arguments stay in registers)
        if (finish_here) {
            finish_row<T, kRoute, kOneRow>(A, sh, reinterpret_cast<uint64_t*>(smem + L.sel), reinterpret_cast<unsigned long long*>(smem + L.cand),
                          p0.row, src);
            if (A.ring != nullptr && (kOneRow || A.mode == kScanFull)) {
                cta_sync();  // the row's outputs are written (or the row is handed to the exact search)
                if (tid == 0 && (kOneRow ? sh.defer : A.deferred[p0.row]) == 0) ring_append(A, q.b);
            }
        }
        if constexpr (kOneRow) break;  // (the CTA's only row)
    }

    if (!bad) bad = cta_sync_or(*reinterpret_cast<const volatile int*>(&sh.fail));
    if (bad) {
        // A wait ran out.  Every row this CTA had a part in reports the failure.  A CTA must not
        // exit with bulk copies in flight into its shared memory: once the producer has stopped,
        // the copies that were issued and not consumed (all but the one the test hook withheld)
        // are given the same bounded wait.
        if (tid == 0) {
            atomicExch(A.dev_error, BORN_ERR_DEVICE_TIMEOUT);
            const unsigned long long w0 = global_timer_ns();
            while (!*reinterpret_cast<const volatile int*>(&sh.prod_done) && global_timer_ns() - w0 < 4 * A.timeout_ns) { }
            if (*reinterpret_cast<const volatile int*>(&sh.prod_done)) {
                const long long issued = sh.issued;
                for (long long tt = max(t0, issued - kStages); tt < issued; ++tt) {
                    if (tt == A.debug_skip_tile) continue;
                    const long long i = tt - t0;
                    mbar_wait_limit(reinterpret_cast<uint64_t*>(&sh.full_bar[i % kStages]), (uint32_t)(i / kStages) & 1u,
                                    A.timeout_ns, nullptr);
                }
            }
        }
        const int r0 = kOneRow ? (int)blockIdx.x : (int)(t0 / A.tpr), r1 = kOneRow ? r0 : (int)((t1 - 1) / A.tpr);
        for (int r = r0 + tid; r <= r1; r += kThreads) {
            if ((kOneRow || A.mode == kScanFull)) {
                A.out_status[r / A.G] = 100 + BORN_ERR_DEVICE_TIMEOUT;
                A.out_token[r / A.G] = -1;
            }
        }
        cta_sync();
        return;
    }

    // ---- rows whose kept set could not be proven complete: exact fallback, now that the ring is idle
    cta_sync();
    {
        const int r0 = kOneRow ? (int)blockIdx.x : (int)(t0 / A.tpr), r1 = kOneRow ? r0 : (int)((t1 - 1) / A.tpr);
        for (int r = r0; r <= r1; ++r) {
            const uint32_t owner = kOneRow ? sh.defer : __ldcg(&A.deferred[r]);
            if ((owner & 0xFFFFFFu) == (uint32_t)blockIdx.x + 1u) {
                cta_sync();
                if (tid == 0) {
                    if constexpr (!kOneRow) A.deferred[r] = 0;
                    atomicAdd(A.dev_error + 1, 1);
                    atomicAdd(A.dev_error + 8 + (owner >> 24), 1);
                }
                fallback_row<T>(A, sh, smem, r);
                cta_sync();
                if (A.ring != nullptr && (kOneRow || A.mode == kScanFull) && tid == 0) ring_append(A, r / A.G);
            }
        }
    }
}

}  // namespace born
