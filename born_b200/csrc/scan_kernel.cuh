// scan_kernel: the streaming pass of the sampler.
//
// One launch does penalties -> grammar mask -> row max / log-sum-exp -> candidate collection
// (top-k, min-p, nucleus) or whole-row mass blocks, and -- in the CTA that completes a row --
// the selection and the inverse-CDF draw (finish.cuh).  Every logit crosses HBM once.
//
// A CTA is 8 compute warps and one producer warp and streams a contiguous range of 16 KB
// tiles (scan_common.cuh).  The producer keeps kScanStages tiles in flight with 1-D bulk
// copies (TMA, no multicast) that complete on `full` mbarriers, applies the token-history
// penalties to each tile once it has landed (fp32: the penalised value is written in place;
// bf16: the token is taken out of the tile and its penalised value goes to the segment record
// directly) and releases it on a `ready` mbarrier.  It never blocks: it alternates between
// "issue the next copy if a stage is free" and "patch the next tile if it has landed".
// A compute warp owns a fixed 2 KB slice of every tile (512 fp32 / 1024 bf16 logits), waits
// for the tile, runs its slice and hands the tile back with one arrival on the `empty`
// mbarrier.  Inside a segment the warps never meet; they meet at segment boundaries only
// (threshold bootstrap after the first tile, record at the end).
//
// Candidates.  A value reaches the slow path only when it is at or above the warp's
// threshold tau (one compare per 16 values).  tau is the maximum of
//   * the lane-maxima bound (top-k <= 256): every lane's running maximum belongs to a
//     different token, so the j-th largest of a warp's 32 lane maxima, j = ceil(k / 8),
//     minimised over the 8 warps, has at least k tokens at or above it;
//   * running maximum + delta (greedy: delta 0; min-p: T * (ln min_p - 0.05); top-p alone: a
//     window that the finish verifies against the exact row total);
//   * the exclusion level of a warp whose 256-entry buffer overflowed.
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
    float lost; // largest candidate that found the warp's buffer full
};
__device__ __forceinline__ void stats_reset(ThreadStats& st, float c2) {
    st.mx = -INFINITY;
    st.R = -1e30f;
    st.nRc = 1e30f * c2;
    st.s = make_float2(0.0f, 0.0f);
    st.pub = -INFINITY;
    st.lost = -INFINITY;
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

// One candidate from the lane that found it, into the warp's own buffer.
__device__ __forceinline__ void push_cand(uint64_t* wbuf, uint32_t* wcount, ThreadStats& st, float z, int id) {
    const uint32_t pos = smem_atom_add(wcount, 1u);
    if (pos < (uint32_t)kWarpCand) wbuf[pos] = ((uint64_t)__float_as_uint(z) << 32) | (uint32_t)id;
    else st.lost = fmaxf(st.lost, z);
}

struct SegCtx {   // what the compute threads know about the segment they are in (block-uniform)
    RowPlan plan;
    int row, id0;       // virtual row; token id of the row's token 0 as written to candidates
    float tau_fix;      // lane-maxima bound / exclusion level (warp-uniform, only rises)
};

__device__ __forceinline__ float current_tau(const SegCtx& sg, const ScanShared& sh) {
    float tau = sg.tau_fix;
    if (sg.plan.use_max)
        tau = fmaxf(tau, zkey_to_float(*reinterpret_cast<const volatile uint32_t*>(&sh.maxbits)) + sg.plan.delta);
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

// A full tile of a 16-byte-aligned row: straight-line code, one compare per 16 values.
// kStats / kCollect select what the pass does (the first tile of a segment is taken twice).
template <typename T, bool kMask, bool kLse, bool kStats, bool kCollect>
__device__ __forceinline__ void fast_tile(const T* tile, const uint32_t* smask, int id_tile0, float tau, float c2,
                                          ThreadStats& st, uint64_t* wbuf, uint32_t* wcount) {
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
        if constexpr (kStats) {
            st.mx = max_nan(st.mx, mt);
            if constexpr (kLse) lse16(st, v, mt, c2);
        }
        if constexpr (kCollect) {
            if (mt >= tau) {  // rare per lane
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (v[i] >= tau && v[i] > -INFINITY) push_cand(wbuf, wcount, st, v[i], id_tile0 + e0[i / VEC] + (i % VEC));
            }
        }
    }
    __syncwarp();
}

// Any tile: partial, of a row that does not start on a 16-byte boundary, or with mask words
// that do not line up with the vectors.  Element e of the tile counts when lo <= e < hi.
template <typename T, bool kMask, bool kLse>
__device__ __forceinline__ void slow_tile(const T* tile, const uint32_t* smask, int64_t mb_rel, int lo, int hi,
                                          int id_tile0, float tau, float c2, bool stats, bool collect,
                                          ThreadStats& st, uint64_t* wbuf, uint32_t* wcount) {
    constexpr int VEC = VecOf<T>::n, ITER = TileOf<T>::n / (kThreads * VEC);
    for (int j = 0; j < ITER; ++j) {
        const int vi = (int)threadIdx.x + kThreads * j;
#pragma unroll
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
            if (collect && z >= tau && z > -INFINITY) push_cand(wbuf, wcount, st, z, id_tile0 + e);
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
                                          ThreadStats& st, ScanShared& sh, uint64_t* wbuf, uint32_t* wcount) {
    constexpr int VEC = VecOf<T>::n, NV = 16 / VEC, NB = TileOf<T>::n / (kThreads * 16);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int h = 0; h < NB; ++h) {
        float v[16];
        int e0[NV];
        load16<T, kMask, true>(tile, smask, h, v, e0);
#pragma unroll
        for (int i = 0; i < 16; ++i)
            if (e0[i / VEC] + (i % VEC) >= hi) v[i] = -INFINITY;
        float mt = v[0];
#pragma unroll
        for (int i = 1; i < 16; ++i) mt = max_nan(mt, v[i]);
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
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (v[i] >= tau && v[i] > -INFINITY) push_cand(wbuf, wcount, st, v[i], id_tile0 + e0[i / VEC] + (i % VEC));
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
    p.row = (int)(t / tpr);
    p.j = (int)(t - (long long)p.row * tpr);
    return p;
}

template <typename T, bool kMask>
__device__ __forceinline__ void producer_issue(const ScanArgs& A, ScanShared& sh, uint8_t* smem, const ScanSmem& L,
                                               long long t, int stage) {
    constexpr int TILE = TileOf<T>::n;
    const TilePos p = tile_pos(t, A.tpr);
    const RowGeom q = row_geom<T>(A, p.row);
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

// The distinct history tokens of caller row q.b (hist_prep_kernel left them in scratch with their
// multiplicities) that fall into tokens [tok_lo, tok_hi) of the virtual row, as
// (count << 32) | token-within-the-virtual-row.
__device__ __forceinline__ int producer_history(const ScanArgs& A, const RowGeom& q, unsigned long long* list,
                                                int tok_lo, int tok_hi) {
    const int lane = threadIdx.x & 31;
    const int n = min((int)__ldg(A.hist_counts + q.b), BORN_MAX_HISTORY);
    const unsigned long long* src = A.hist_lists + (int64_t)q.b * BORN_MAX_HISTORY;
    int out = 0;
    // all loads of a round are issued before any is used: one trip to L2 for up to 512 entries
    for (int base = 0; base < n; base += 512) {
        unsigned long long e[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const int i = base + 32 * k + lane;
            e[k] = (i < n) ? __ldg(src + i) : ~0ull;
        }
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (base + 32 * k >= n) break;  // (uniform)
            const long long tok = (long long)(uint32_t)e[k] - (long long)q.g * A.V;
            const bool in = e[k] != ~0ull && tok >= tok_lo && tok < tok_hi;
            const uint32_t inb = __ballot_sync(0xffffffffu, in);
            if (in) list[out + __popc(inb & ((1u << lane) - 1u))] = (e[k] & 0xFFFFFFFF00000000ull) | (uint32_t)tok;
            out += __popc(inb);
        }
    }
    __syncwarp();
    return out;
}

template <typename T, bool kMask, bool kLse>
__device__ __forceinline__ void producer_loop(const ScanArgs& A, ScanShared& sh, uint8_t* smem, const ScanSmem& L,
                                              long long t0, long long t1) {
    constexpr int TILE = TileOf<T>::n;
    const int lane = threadIdx.x & 31;
    const bool use_ready = A.history != nullptr;
    const int cta = blockIdx.x;
    unsigned long long* table = reinterpret_cast<unsigned long long*>(smem + L.hist);
    long long issue_t = t0, patch_t = t0;
    int cur_row = -1, nlist = 0, seg_ord = -1;
    RowGeom q = {};
    born_row_params rp = {};
    RowPlan plan = {};
    bool pen = false;
    // statistics of the penalised tokens that were taken out of bf16 tiles
    float p_mx = -INFINITY, p_R = -1e30f, p_s = 0.0f;
    uint32_t p_n = 0;
    // A software pipeline with blocking (bounded) waits: step n first patches tile n - lag, whose
    // copy was issued lag steps ago, and releases it to the compute warps; then it waits for the
    // stage of tile n to be handed back and issues its copy.  The tile the compute warps need
    // next is therefore patched while they still work on the one before.
    constexpr int lag = kScanStages - 1;
    const long long n_tiles = t1 - t0;
    bool ok = true;
    for (long long n = 0; ok && n < n_tiles + (use_ready ? lag : 0); ++n) {
        if (use_ready && n >= lag) {
            {
                const long long i = n - lag;
                const int stage = (int)(i % kScanStages);
                if (!mbar_wait_limit(reinterpret_cast<uint64_t*>(&sh.full_bar[stage]), (uint32_t)(i / kScanStages) & 1u, A.timeout_ns,
                                     &sh.fail)) {
                    ok = false;
                    break;
                }
                patch_t = t0 + i;
                const TilePos p = tile_pos(patch_t, A.tpr);
                if (p.row != cur_row) {  // first tile of a segment: its history list
                    cur_row = p.row;
                    ++seg_ord;
                    q = row_geom<T>(A, p.row);
                    rp = A.row_params ? A.row_params[q.b] : A.params;
                    plan = row_plan(rp);
                    pen = penalties_on(rp);
                    nlist = 0;
                    if (pen) {
                        const long long seg_t0 = max(t0, (long long)p.row * A.tpr), seg_t1 = min(t1, (long long)(p.row + 1) * A.tpr);
                        const long long e_lo = (seg_t0 - (long long)p.row * A.tpr) * TILE, e_hi = (seg_t1 - (long long)p.row * A.tpr) * TILE;
                        const int tok_lo = (int)max(0ll, e_lo - q.lead), tok_hi = (int)min((long long)A.V, e_hi - q.lead);
                        nlist = producer_history(A, q, table, tok_lo, tok_hi);
                    }
                    p_mx = -INFINITY; p_R = -1e30f; p_s = 0.0f; p_n = 0;
                }
                T* tile = reinterpret_cast<T*>(smem + L.tiles + (size_t)stage * kTileBytes);
                const int n_el = min(TILE, q.lead + A.V - p.j * TILE);
                const int lo = max(0, q.lead - p.j * TILE);
                bool wrote = false;
                if (nlist > 0 && n_el > lo) {
                    const uint32_t* smask = reinterpret_cast<const uint32_t*>(smem + L.masks + (size_t)stage * (mask_stage_words<T>() * 4));
                    MaskTile mt = {};
                    if constexpr (kMask) mt = mask_tile<T>(A, q, p.j, lo, n_el);
                    uint64_t* rec_ent = reinterpret_cast<uint64_t*>(A.records + (int64_t)(p.row + cta) * A.rec_stride + kRecordHdrBytes);
                    const int id0 = A.idx_base + q.g * A.V;
                    for (int base = 0; base < nlist; base += 32) {
                        const int i2 = base + lane;
                        bool side = false;
                        float zp = -INFINITY;
                        int tok = 0;
                        if (i2 < nlist) {
                            const unsigned long long e = table[i2];
                            tok = (int)(uint32_t)e;
                            const int cnt = (int)(e >> 32);
                            const int off = tok + q.lead - p.j * TILE;
                            if (off >= lo && off < n_el) {
                                float z;
                                if constexpr (sizeof(T) == 4) z = reinterpret_cast<float*>(tile)[off];
                                else z = bf16_bits_to_f32(reinterpret_cast<uint16_t*>(tile)[off]);
                                zp = penalise(rp, z, cnt);
                                if constexpr (sizeof(T) == 4) {
                                    reinterpret_cast<float*>(tile)[off] = zp;
                                } else {
                                    reinterpret_cast<uint16_t*>(tile)[off] = 0xFF80u;  // -inf: the token leaves the tile
                                    if constexpr (kMask) {
                                        const int64_t bi = mt.mb0 + off - 32 * mt.w0a;
                                        if (!((smask[bi >> 5] >> (bi & 31)) & 1u)) zp = -INFINITY;
                                    }
                                    side = true;
                                }
                                wrote = true;
                            }
                        }
                        if constexpr (sizeof(T) == 2) {
                            // the penalised value joins the segment's statistics and, if it can matter, its record
                            if (side) {
                                p_mx = max_nan(p_mx, zp);
                                if (kLse && zp > -INFINITY && zp < INFINITY) {
                                    if (zp > p_R) { p_s *= ex2_approx(__fmul_rn(p_R - zp, plan.c2)); p_R = zp; }
                                    p_s += ex2_approx(__fmul_rn(zp - p_R, plan.c2));
                                }
                            }
                            const bool keep = side && plan.collect && zp > -INFINITY;
                            const uint32_t kb = __ballot_sync(0xffffffffu, keep);
                            if (keep) {
                                const uint32_t pos = p_n + __popc(kb & ((1u << lane) - 1u));
                                if (pos < (uint32_t)A.rec_cap)
                                    rec_ent[pos] = ((uint64_t)__float_as_uint(zp) << 32) | (uint32_t)(id0 + tok);
                            }
                            p_n += __popc(kb);
                        }
                    }
                }
                if constexpr (sizeof(T) == 2) {
                    // last tile of the segment: leave the side statistics where the compute threads find them
                    const bool seg_end = (patch_t + 1 == t1) || (tile_pos(patch_t + 1, A.tpr).row != cur_row);
                    if (seg_end) {
                        const float wm = warp_max_nan(p_mx);
                        float ws = 0.0f;
                        if (kLse) {
                            ws = (p_s > 0.0f && wm == wm) ? p_s * ex2_approx(__fmul_rn(p_R - wm, plan.c2)) : 0.0f;
#pragma unroll
                            for (int d = 16; d > 0; d >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, d);
                        }
                        if (lane == 0) {
                            ScanShared::Side& sd = sh.side[seg_ord % (kScanStages + 1)];
                            sd.m = wm; sd.s = ws; sd.n = p_n;
                        }
                    }
                }
                if (wrote) fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&sh.ready_bar[stage]));
            }
        }
        if (n < n_tiles) {
            const int stage = (int)(n % kScanStages);
            if (n >= kScanStages &&
                !mbar_wait_limit(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage]), (uint32_t)((n / kScanStages) - 1) & 1u,
                                 A.timeout_ns, &sh.fail)) {
                ok = false;
                break;
            }
            if (lane == 0) producer_issue<T, kMask>(A, sh, smem, L, t0 + n, stage);
            issue_t = t0 + n + 1;
        }
    }
    if (!ok) sh.fail = 1;
    // what the failure path of the compute threads needs to know (see the end of scan_kernel)
    if (lane == 0) {
        sh.issued = issue_t;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&sh.prod_done) = 1;
    }
}

// ---- the kernel -------------------------------------------------------------------------------
template <typename T, bool kMask, bool kLse>
__global__ void __launch_bounds__(kScanThreads, 2) scan_kernel(const __grid_constant__ ScanArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ ScanShared sh;
    constexpr int TILE = TileOf<T>::n;
    const int tid = threadIdx.x;
    const ScanSmem L = scan_smem_layout((int)sizeof(T), kMask, A.history != nullptr);
    const long long rows = (long long)A.B * A.G;
    const long long T_total = rows * A.tpr;
    const long long ncta = gridDim.x;
    const long long t0 = range_begin(blockIdx.x, T_total, ncta), t1 = range_begin(blockIdx.x + 1, T_total, ncta);
    const bool use_ready = A.history != nullptr;

    if (tid == 0) {
        for (int s = 0; s < kScanStages; ++s) {
            mbar_init(reinterpret_cast<uint64_t*>(&sh.full_bar[s]), 1);
            mbar_init(reinterpret_cast<uint64_t*>(&sh.ready_bar[s]), 1);
            mbar_init(reinterpret_cast<uint64_t*>(&sh.empty_bar[s]), kScanWarps);
        }
        mbar_fence_init();
        sh.fail = 0;
        sh.prod_done = 0;
        sh.issued = t0;
    }
    __syncthreads();  // the only barrier all 288 threads share

    if (tid >= kThreads) {
        producer_loop<T, kMask, kLse>(A, sh, smem, L, t0, t1);
        return;
    }

    // ------------------------------------------------------------------------ compute threads
    PROF(0);
    const int lane = tid & 31, warp = tid >> 5;
    uint64_t* wbuf = reinterpret_cast<uint64_t*>(smem + L.cand) + warp * kWarpCand;
    uint32_t* wcount = &sh.wcount[warp];
#ifdef BORN_PROFILE
    long long pf_wait = 0, pf_proc = 0;
#endif
    bool failed = false;
    int bad = 0;
    int seg_ord = -1;
    long long t = t0;
    while (t < t1) {
        // ---- segment set-up (block-synchronous)
        const TilePos p0 = tile_pos(t, A.tpr);
        const long long seg_end = min(t1, (long long)(p0.row + 1) * A.tpr);
        ++seg_ord;
        const RowGeom q = row_geom<T>(A, p0.row);
        const born_row_params rp = A.row_params ? A.row_params[q.b] : A.params;
        SegCtx sg;
        sg.plan = row_plan(rp);
        sg.row = p0.row;
        sg.id0 = A.idx_base + q.g * A.V;
        sg.tau_fix = sg.plan.no_bound ? INFINITY : -INFINITY;
        const RowPlan& pl = sg.plan;
        cta_sync();
        if (tid == 0) {
            sh.maxbits = zkey(-INFINITY);
            sh.excl_bits = zkey(-INFINITY);
            sh.rec_count = 0;
        }
        if (tid < kScanWarps) { sh.wbound[tid] = -INFINITY; sh.wcount[tid] = 0; }
        cta_sync();
        ThreadStats st;
        stats_reset(st, pl.c2);
        MassBlock* row_blocks = A.blocks + (int64_t)p0.row * A.nblk;
        const bool collect = pl.collect && !pl.no_bound;
        int seen = 0;  // tiles of this segment done
        for (; t < seg_end; ++t, ++seen) {
            const long long i = t - t0;
            const int stage = (int)(i % kScanStages);
            const int j = (int)(t - (long long)p0.row * A.tpr);
#ifdef BORN_PROFILE
            const long long pw0 = clock64();
#endif
            if (!failed) {
                uint64_t* bar = reinterpret_cast<uint64_t*>(use_ready ? &sh.ready_bar[stage] : &sh.full_bar[stage]);
                if (!mbar_wait_limit(bar, (uint32_t)(i / kScanStages) & 1u, A.timeout_ns, &sh.fail)) {
                    failed = true;
                    sh.fail = 1;
                }
            }
#ifdef BORN_PROFILE
            const long long pw1 = clock64();
            pf_wait += pw1 - pw0;
            if (t == t0) PROF(1);
#endif
            const T* tile = reinterpret_cast<const T*>(smem + L.tiles + (size_t)stage * kTileBytes);
            const uint32_t* smask = reinterpret_cast<const uint32_t*>(smem + L.masks + (size_t)stage * (mask_stage_words<T>() * 4));
            const int n_el = min(TILE, q.lead + A.V - j * TILE);
            const int lo = max(0, q.lead - j * TILE);
            const int tok_tile0 = j * TILE - q.lead;          // token (within the virtual row) of element 0
            const int id_tile0 = sg.id0 + tok_tile0;
            const bool full = A.fast && n_el == TILE;
            int64_t mb_rel = 0;
            if constexpr (kMask) {
                if (!full && n_el > lo) {
                    const MaskTile mt = mask_tile<T>(A, q, j, lo, n_el);
                    mb_rel = mt.mb0 - 32 * mt.w0a;
                }
            }
            const bool first = (seen == 0);
            if (!failed && n_el > lo) {
                if (pl.need_mass) {
                    // (rows of these routes are 16-byte aligned: the host sees to it)
                    const float tau = first ? INFINITY : current_tau(sg, sh);
                    mass_tile<T, kMask>(tile, smask, n_el, tok_tile0, id_tile0, tau, pl.inv_T, collect && !first, row_blocks, A.nblk,
                                        st, sh, wbuf, wcount);
                } else if (first) {
                    if (full) fast_tile<T, kMask, kLse, true, false>(tile, smask, id_tile0, 0.0f, pl.c2, st, wbuf, wcount);
                    else slow_tile<T, kMask, kLse>(tile, smask, mb_rel, lo, n_el, id_tile0, 0.0f, pl.c2, true, false, st, wbuf, wcount);
                } else {
                    const float tau = collect ? current_tau(sg, sh) : INFINITY;
                    if (full) fast_tile<T, kMask, kLse, true, true>(tile, smask, id_tile0, tau, pl.c2, st, wbuf, wcount);
                    else slow_tile<T, kMask, kLse>(tile, smask, mb_rel, lo, n_el, id_tile0, tau, pl.c2, true, collect, st, wbuf, wcount);
                    if (pl.use_max) publish_max(st, sh);
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
                if (pl.lane_bound) {
                    lane_bound(sh, pl.k, st.mx);
                    cta_sync();
                    sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
                }
                if (!failed && collect && n_el > lo) {
                    const float tau = current_tau(sg, sh);
                    if (pl.need_mass) {
                        // collect only: the values are read again, no mass work
                        slow_tile<T, kMask, false>(tile, smask, mb_rel, lo, n_el, id_tile0, tau, pl.c2, false, true, st, wbuf, wcount);
                    } else if (full) {
                        fast_tile<T, kMask, kLse, false, true>(tile, smask, id_tile0, tau, pl.c2, st, wbuf, wcount);
                    } else {
                        slow_tile<T, kMask, kLse>(tile, smask, mb_rel, lo, n_el, id_tile0, tau, pl.c2, false, true, st, wbuf, wcount);
                    }
                }
            } else if (pl.lane_bound && ((seen + 1) & seen) == 0) {
                // tighten the bound when the number of tiles seen doubles (no barrier: values of
                // warps that lag are older, hence lower, hence still valid)
                sg.tau_fix = fmaxf(sg.tau_fix, lane_bound(sh, pl.k, st.mx));
            }
            // a lane that lost a candidate to a full buffer raises the warp's exclusion level
            if (collect && __any_sync(0xffffffffu, st.lost > -INFINITY)) {
                float lw = st.lost;
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) lw = fmaxf(lw, __shfl_xor_sync(0xffffffffu, lw, d));
                const uint32_t kx = key_above(lw);
                if (lane == 0) smem_red_max(&sh.excl_bits, kx);
                sg.tau_fix = fmaxf(sg.tau_fix, zkey_to_float(kx));
                st.lost = -INFINITY;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(reinterpret_cast<uint64_t*>(&sh.empty_bar[stage]));  // tile back to the producer
#ifdef BORN_PROFILE
            pf_proc += clock64() - pw1;
#endif
        }
        PROF(2 + 3 * min(seg_ord, 1));

        // ---- segment record (block-synchronous)
        const float wm = warp_max_nan(st.mx);
        float ws = 0.0f;
        if (kLse && !pl.need_mass) {
            const float ssum = st.s.x + st.s.y;
            ws = (ssum > 0.0f && wm == wm) ? ssum * ex2_approx(__fmul_rn(st.R - wm, pl.c2)) : 0.0f;
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, d);
        }
        if (pl.lane_bound) lane_bound(sh, pl.k, st.mx);
        if (lane == 0) { sh.wmax[warp] = wm; sh.wsum[warp] = ws; }
        uint32_t side_n = 0;
        float side_m = -INFINITY, side_s = 0.0f;
        if (sizeof(T) == 2 && use_ready) {
            const ScanShared::Side& sd = sh.side[seg_ord % (kScanStages + 1)];
            side_n = sd.n; side_m = sd.m; side_s = sd.s;
            if (tid == 0) sh.rec_count = min(side_n, (uint32_t)A.rec_cap);
            if (tid == 0 && side_n > (uint32_t)A.rec_cap) sh.excl_bits = zkey(INFINITY);  // cannot tell what was lost
        }
        cta_sync();
        float m_seg = max_nan(sh.wmax[0], side_m);
#pragma unroll
        for (int w = 1; w < kScanWarps; ++w) m_seg = max_nan(m_seg, sh.wmax[w]);
        float s_seg = 0.0f;
        if (kLse && !pl.need_mass) {
#pragma unroll
            for (int w = 0; w < kScanWarps; ++w) {
                const float x = sh.wsum[w];
                if (x > 0.0f) s_seg += x * ex2_approx(__fmul_rn(sh.wmax[w] - m_seg, pl.c2));
            }
            if (side_s > 0.0f) s_seg += side_s * ex2_approx(__fmul_rn(side_m - m_seg, pl.c2));
        }
        float bound_k = -INFINITY;
        if (pl.lane_bound) {
            bound_k = sh.wbound[0];
#pragma unroll
            for (int w = 1; w < kScanWarps; ++w) bound_k = fminf(bound_k, sh.wbound[w]);
        }
        // nothing below the segment's final valid bounds can be kept by the row
        float cut = bound_k;
        float excl_window = -INFINITY;
        if (pl.use_max && m_seg == m_seg) {
            if (pl.window) excl_window = m_seg + pl.delta;
            cut = fmaxf(cut, m_seg + pl.delta);
        }
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
            if (pl.no_bound) te = INFINITY;
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
        PROF(3 + 3 * min(seg_ord, 1));
        if (sh.last) {
            __threadfence();
            finish_row<T>(A, sh, smem + L.cand, p0.row, sh.c_first, sh.c_last);
        }
        PROF(4 + 3 * min(seg_ord, 1));
    }
    PROF(10);
#ifdef BORN_PROFILE
    PROF_ADD(8, pf_wait);
    PROF_ADD(9, pf_proc);
#endif

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
                for (long long tt = max(t0, issued - kScanStages); tt < issued; ++tt) {
                    if (tt == A.debug_skip_tile) continue;
                    const long long i = tt - t0;
                    mbar_wait_limit(reinterpret_cast<uint64_t*>(&sh.full_bar[i % kScanStages]), (uint32_t)(i / kScanStages) & 1u,
                                    A.timeout_ns, nullptr);
                }
            }
        }
        const int r0 = (int)(t0 / A.tpr), r1 = (int)((t1 - 1) / A.tpr);
        for (int r = r0 + tid; r <= r1; r += kThreads) {
            if (A.mode == kScanFull) {
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
        const int r0 = (int)(t0 / A.tpr), r1 = (int)((t1 - 1) / A.tpr);
        for (int r = r0; r <= r1; ++r) {
            const uint32_t owner = __ldcg(&A.deferred[r]);
            if (owner == (uint32_t)blockIdx.x + 1u) {
                cta_sync();
                if (tid == 0) { A.deferred[r] = 0; atomicAdd(A.dev_error + 1, 1); }
                fallback_row<T>(A, sh, smem, r);
                cta_sync();
            }
        }
    }
}

}  // namespace born
