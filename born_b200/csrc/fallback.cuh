// Exact fallback for rows whose kept set could not be proven to lie inside the complete part
// of their candidates: top-k above 256, a min-p survivor set or a nucleus beyond the 1024
// candidates the in-shared-memory selection takes, a candidate buffer that overflowed (rows of
// equal values), a kept-id list of a whole-vocabulary row.
//
// It is the sort-free threshold search over the whole row: the row is streamed again (from
// L2 / HBM, 4096 tokens at a time, penalties and mask applied in shared memory) once per
// radix digit of the 56-bit rank key (value, -index) -- 12 bits per pass, 4096 bins of exact
// integer counts and masses in shared memory, the crossing bin found by a block scan -- then
// once more for the inverse-CDF draw.  Slower than the one-pass route by design (a dozen
// passes over one row by one CTA), never approximate.  It runs in the CTA that finished the
// row, after that CTA has streamed its whole tile range, when its shared memory is idle.
#pragma once
#include "scan_common.cuh"
#include "finish.cuh"

namespace born {

constexpr int kFbChunk = 4096;   // tokens per chunk
constexpr int kFbBins = 4096;    // bins per radix pass (12 bits)

struct FbCtx {
    const ScanArgs* A;
    ScanShared* sh;
    float* chunk;                  // kFbChunk logits as the sampler sees them (the buffer in use)
    float* chunk2[2];              // the two buffers that take turns
    unsigned long long* hlist;     // distinct history tokens of the row: (count << 32) | token
    uint32_t* bcnt;                // kFbBins counts
    unsigned long long* bwt;       // kFbBins masses (also: the masses of one chunk for the draw)
    int nlist;
    int b, g, V, id0;
    born_row_params rp;
    float m, inv_T;
};

template <typename T>
__device__ __forceinline__ float fb_raw(const FbCtx& c, int tok) {
    const T* row = reinterpret_cast<const T*>(c.A->logits) + (int64_t)c.b * c.A->row_stride + (int64_t)c.g * c.V;
    if constexpr (sizeof(T) == 4) return __ldg(reinterpret_cast<const float*>(row) + tok);
    else return bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(row) + tok));
}
__device__ __forceinline__ bool fb_allowed(const FbCtx& c, int tok) {
    if (!c.A->mask) return true;
    const int64_t bi = (int64_t)c.g * c.V + tok;
    return ((__ldg(c.A->mask + (int64_t)c.b * c.A->mask_stride + (bi >> 5)) >> (bi & 31)) & 1u) != 0;
}

// Distinct history tokens of the row with their multiplicities (all pairs, once per row).
__device__ __forceinline__ void fb_history(FbCtx& c) {
    const ScanArgs& A = *c.A;
    const int tid = threadIdx.x;
    if (tid == 0) c.sh->nl = 0;
    cta_sync();
    if (A.history && penalties_on(c.rp)) {
        int len = A.history_len ? A.history_len[c.b] : A.history_stride;
        len = max(0, min(min(len, A.history_stride), BORN_MAX_HISTORY));
        const int32_t* gh = A.history + (int64_t)c.b * A.history_stride;
        for (int p = tid; p < len; p += kThreads) {
            const int idg = __ldg(gh + p);
            const long long tok = (long long)idg - (long long)c.g * c.V;
            if (tok < 0 || tok >= c.V) continue;
            int cnt = 0;
            bool first = true;
            for (int j = 0; j < len; ++j) {
                const bool eq = (__ldg(gh + j) == idg);
                cnt += eq ? 1 : 0;
                if (eq && j < p) first = false;
            }
            if (first) c.hlist[smem_atom_add(&c.sh->nl, 1u)] = ((unsigned long long)cnt << 32) | (uint32_t)tok;
        }
    }
    cta_sync();
    c.nlist = c.sh->nl;
}

// Chunk ci of the row, as the sampler sees it apart from the penalties: the thread's 16 elements
// (element tid + 256 * j), into registers.  The loads leave together; nothing waits for them here.
constexpr int kFbPer = kFbChunk / kThreads;
template <typename T>
__device__ __forceinline__ void fb_fetch(const FbCtx& c, int ci, float (&v)[kFbPer]) {
    const int c0 = ci * kFbChunk;
    bool ok[kFbPer];
#pragma unroll
    for (int j = 0; j < kFbPer; ++j) {
        const int tok = c0 + (int)threadIdx.x + kThreads * j;
        ok[j] = tok < c.V && fb_allowed(c, tok);
    }
#pragma unroll
    for (int j = 0; j < kFbPer; ++j) {
        const int tok = c0 + (int)threadIdx.x + kThreads * j;
        v[j] = tok < c.V ? fb_raw<T>(c, tok) : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < kFbPer; ++j)
        if (!ok[j]) v[j] = -INFINITY;
}
// ... from the registers into the buffer whose turn it is, with the history penalties on top.
template <typename T>
__device__ __forceinline__ void fb_store(FbCtx& c, int ci, const float (&v)[kFbPer]) {
    const int tid = threadIdx.x;
    const int c0 = ci * kFbChunk;
    c.chunk = c.chunk2[ci & 1];
#pragma unroll
    for (int j = 0; j < kFbPer; ++j) c.chunk[tid + kThreads * j] = v[j];
    cta_sync();  // (also: every thread is done with the chunk before last, whose buffer the next store takes)
    if (c.nlist > 0) {
        for (int i = tid; i < c.nlist; i += kThreads) {
            const unsigned long long e = c.hlist[i];
            const int tok = (int)(uint32_t)e;
            if (tok >= c0 && tok < c0 + kFbChunk && fb_allowed(c, tok)) c.chunk[tok - c0] = penalise(c.rp, fb_raw<T>(c, tok), (int)(e >> 32));
        }
        cta_sync();
    }
}
template <typename T>
__device__ __forceinline__ void fb_load(FbCtx& c, int ci) {
    float v[kFbPer];
    fb_fetch<T>(c, ci, v);
    fb_store<T>(c, ci, v);
}

// One pass over the row: f(token, z) for every token above -inf, by the thread that owns it.  The
// next chunk's loads are in flight while the current chunk is worked on.
template <typename T, typename F>
__device__ __forceinline__ void fb_pass(FbCtx& c, F f) {
    const int nchunks = (c.V + kFbChunk - 1) / kFbChunk;
    float v[kFbPer];
    fb_fetch<T>(c, 0, v);
    for (int ci = 0; ci < nchunks; ++ci) {
        fb_store<T>(c, ci, v);
        if (ci + 1 < nchunks) fb_fetch<T>(c, ci + 1, v);
        const float* ch = c.chunk;
        for (int e = threadIdx.x; e < kFbChunk; e += kThreads) {
            const float z = ch[e];
            if (z > -INFINITY) f(ci * kFbChunk + e, z);
        }
    }
    cta_sync();
}

__device__ __forceinline__ unsigned long long fb_mass(const FbCtx& c, float z) {
    const float x = scaled_shift(z, c.m, c.inv_T);
    return (x < -30.0f) ? 0ull : mass_of(x);
}

// Walking the tokens with rank key >= lowkey in rank order (key descending), the key at which the
// running weight (1 per token, or its mass) first exceeds `target`.  Returns 0 when the total
// weight does not exceed target (the caller keeps everything).
template <typename T, bool kWeighted>
__device__ __noinline__ unsigned long long fb_search(FbCtx& c, unsigned long long lowkey, unsigned long long target) {
    const int tid = threadIdx.x;
    ScanShared& sh = *c.sh;
    unsigned long long prefix = 0, pmask = 0;
    const int shifts[5] = {44, 32, 20, 8, 0};
    // Masses are summed per bin as three 14-bit limbs in 32-bit words: 32-bit shared-memory atomics
    // are native, 64-bit ones are compare-and-swap loops.  A limb sum stays below 2^32 for rows of
    // up to 2^17 tokens; longer rows use the 64-bit words.
    uint32_t* limb = reinterpret_cast<uint32_t*>(c.bwt);  // [3][kFbBins], over the mass and count areas
    const bool limbs = kWeighted && c.V <= (1 << 17);
    for (int lvl = 0; lvl < 5; ++lvl) {
        const int shift = shifts[lvl];
        const int nb = (lvl == 4) ? 256 : kFbBins;
        if (limbs) {
            for (int i = tid; i < 3 * kFbBins; i += kThreads) limb[i] = 0;
        } else {
            for (int i = tid; i < nb; i += kThreads) { c.bcnt[i] = 0; c.bwt[i] = 0; }
        }
        cta_sync();
        fb_pass<T>(c, [&](int tok, float z) {
            const unsigned long long ck = make_ck(z, c.id0 + tok);
            if (ck < lowkey || (ck & pmask) != prefix) return;
            const uint32_t d = (uint32_t)(ck >> shift) & (uint32_t)(nb - 1);
            if (kWeighted) {
                const unsigned long long w = fb_mass(c, z);
                if (!w) return;
                if (limbs) {
                    smem_red_add(&limb[d], (uint32_t)w & 0x3FFFu);
                    smem_red_add(&limb[kFbBins + d], (uint32_t)(w >> 14) & 0x3FFFu);
                    smem_red_add(&limb[2 * kFbBins + d], (uint32_t)(w >> 28));
                } else {
                    atomicAdd(&c.bwt[d], w);
                }
            } else {
                smem_red_add(&c.bcnt[d], 1u);
            }
        });
        if (limbs) {  // fold the limbs into the 64-bit words the scan below reads
            unsigned long long w[kFbBins / kThreads];
#pragma unroll
            for (int j = 0; j < kFbBins / kThreads; ++j) {
                const int bin = tid + kThreads * j;
                w[j] = (unsigned long long)limb[bin] + ((unsigned long long)limb[kFbBins + bin] << 14) +
                       ((unsigned long long)limb[2 * kFbBins + bin] << 28);
            }
            cta_sync();
#pragma unroll
            for (int j = 0; j < kFbBins / kThreads; ++j) c.bwt[tid + kThreads * j] = w[j];
            cta_sync();
        }
        // block scan over the bins in walk order (descending digit): thread t owns nb/256 of them
        const int per = nb / kThreads;
        unsigned long long loc = 0;
        for (int j = 0; j < per; ++j) {
            const int bin = nb - 1 - (tid * per + j);
            loc += kWeighted ? c.bwt[bin] : (unsigned long long)c.bcnt[bin];
        }
        unsigned long long incl = loc;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned long long up = shfl_up_u64(incl, d);
            if ((tid & 31) >= d) incl += up;
        }
        cta_sync();
        if ((tid & 31) == 31) sh.red64[tid >> 5] = incl;
        if (tid == 0) sh.found = -1;
        cta_sync();
        unsigned long long off = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kScanWarps; ++w) {
            const unsigned long long x = sh.red64[w];
            if (w < (tid >> 5)) off += x;
            total += x;
        }
        incl += off;
        if (total <= target) return 0ull;  // (uniform)
        if (incl > target && incl - loc <= target) {
            unsigned long long acc = incl - loc;
            for (int j = 0; j < per; ++j) {
                const int bin = nb - 1 - (tid * per + j);
                const unsigned long long w = kWeighted ? c.bwt[bin] : (unsigned long long)c.bcnt[bin];
                if (acc + w > target) { sh.found = bin; sh.before = acc; break; }
                acc += w;
            }
        }
        cta_sync();
        const unsigned long long digit = (unsigned long long)sh.found;
        target -= sh.before;
        prefix |= digit << shift;
        pmask |= (unsigned long long)(nb - 1) << shift;
        cta_sync();
    }
    return prefix;
}

// The (at most kSelCap) tokens with rank key >= lowkey, gathered and written in rank order.
template <typename T>
__device__ __forceinline__ int fb_gather(FbCtx& c, unsigned long long lowkey, uint64_t* sel) {
    if (threadIdx.x == 0) c.sh->nl = 0;
    cta_sync();
    fb_pass<T>(c, [&](int tok, float z) {
        const unsigned long long ck = make_ck(z, c.id0 + tok);
        if (ck >= lowkey) {
            const int pos = (int)smem_atom_add(&c.sh->nl, 1u);
            if (pos < kSelCap) sel[pos] = ck;
        }
    });
    return min(c.sh->nl, kSelCap);
}

template <typename T>
__device__ __noinline__ void fallback_row(const ScanArgs& A, ScanShared& sh, uint8_t* smem, int row) {
    const int tid = threadIdx.x;
    FbCtx c;
    c.A = &A;
    c.sh = &sh;
    // 88 KB of the CTA's dynamic shared memory (no variant of the kernel has less):
    // two chunk buffers | history list | mass bins | count bins
    c.chunk2[0] = reinterpret_cast<float*>(smem);
    c.chunk2[1] = reinterpret_cast<float*>(smem + kFbChunk * 4);
    c.chunk = c.chunk2[0];
    c.hlist = reinterpret_cast<unsigned long long*>(smem + 2 * kFbChunk * 4);
    c.bwt = reinterpret_cast<unsigned long long*>(smem + 2 * kFbChunk * 4 + BORN_MAX_HISTORY * 8);
    c.bcnt = reinterpret_cast<uint32_t*>(smem + 2 * kFbChunk * 4 + BORN_MAX_HISTORY * 8 + kFbBins * 8);
    static_assert(2 * kFbChunk * 4 + BORN_MAX_HISTORY * 8 + kFbBins * 12 <= kScanStages * kTileBytes + kScanWarps * kWarpCand * 8 + kSelCap * 8,
                  "the exact search lives in the streaming kernel's shared memory");
    uint64_t* sel = reinterpret_cast<uint64_t*>(c.bwt);  // gathers happen when no search is in flight
    c.b = row / A.G;
    c.g = row - c.b * A.G;
    c.V = A.V;
    c.id0 = A.idx_base + c.g * A.V;
    c.rp = A.row_params ? A.row_params[c.b] : A.params;
    const RowPlan pl = row_plan(c.rp);
    c.inv_T = pl.inv_T;
    fb_history(c);

    // row maximum (the row is known to be valid: the finish only defers rows with a finite maximum)
    float mx = -INFINITY;
    fb_pass<T>(c, [&](int, float z) { mx = fmaxf(mx, z); });
    c.m = block_max_nan(mx, sh.redf);

    RowOut o;
    o.token = A.out_token; o.prob = A.out_prob; o.lse = A.out_lse; o.status = A.out_status;
    o.kept_ids = A.out_kept_ids; o.kept_count = A.out_kept_count; o.kept_stride = A.kept_stride;
    o.row = c.b;
    const unsigned long long alive = 1ull << 24;  // smallest rank key of a token above -inf

    if (A.mode == kScanLocal) {
        // the k best of the virtual row, in rank order
        unsigned long long Ck = fb_search<T, false>(c, alive, (unsigned long long)(pl.k - 1));
        if (Ck == 0) Ck = alive;
        const int n = fb_gather<T>(c, Ck, sel);
        // statistics of the record come from the segment headers
        const int c_first = cta_of_tile((long long)row * A.tpr, (long long)A.B * A.G * A.tpr, gridDim.x);
        const int c_last = cta_of_tile((long long)(row + 1) * A.tpr - 1, (long long)A.B * A.G * A.tpr, gridDim.x);
        float ls = 0.0f;
        for (int s = tid; s <= c_last - c_first; s += kThreads) {
            const float4 h = __ldcg(reinterpret_cast<const float4*>(A.records + (int64_t)(row + c_first + s) * A.rec_stride));
            if (h.y > 0.0f) ls += h.y * ex2_approx(__fmul_rn(h.x - c.m, pl.c2));
        }
        ls = block_sum_f32(ls, sh.redf);
        write_packed(A, sh, sel, reinterpret_cast<unsigned long long*>(sel + kSelCap), n, pl.k, c.b, c.g, c.m, ls, -INFINITY, true);
        return;
    }

    if (pl.greedy) {
        uint64_t best = 0;
        fb_pass<T>(c, [&](int tok, float z) { best = max(best, make_ck(z, c.id0 + tok)); });
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) best = max(best, shfl_xor_u64(best, d));
        cta_sync();
        if ((tid & 31) == 0) sh.red64[tid >> 5] = best;
        cta_sync();
        if (tid == 0) {
            for (int w = 1; w < kScanWarps; ++w) best = max(best, (uint64_t)sh.red64[w]);
            const int tok = ck_idx(best);
            A.out_token[c.b] = tok;
            A.out_status[c.b] = BORN_ROW_OK;
            if (A.out_prob) A.out_prob[c.b] = 1.0f;
            if (A.out_kept_count) A.out_kept_count[c.b] = 1;
            if (A.out_kept_ids && A.kept_stride > 0) A.out_kept_ids[(int64_t)c.b * A.kept_stride] = tok;
        }
        return;
    }

    const float u = A.uniforms[c.b];
    unsigned long long lowkey = alive;
    if (pl.k > 0) {
        const unsigned long long Ck = fb_search<T, false>(c, lowkey, (unsigned long long)(pl.k - 1));
        if (Ck > lowkey) lowkey = Ck;
    }
    if (c.rp.min_p > 0.0f) {
        // the survivors are a prefix of the rank order (masses fall with the value): lowest surviving value
        const unsigned long long Qa = __double2ull_ru((double)c.rp.min_p * 1099511627776.0);
        uint32_t zmin = 0xFFFFFFFFu;
        fb_pass<T>(c, [&](int tok, float z) {
            if (make_ck(z, c.id0 + tok) >= lowkey && fb_mass(c, z) >= Qa) zmin = min(zmin, zkey(z));
        });
        zmin = __reduce_min_sync(0xffffffffu, zmin);
        cta_sync();
        if ((tid & 31) == 0) sh.red64[tid >> 5] = zmin;
        cta_sync();
        for (int w = 0; w < kScanWarps; ++w) zmin = min(zmin, (uint32_t)sh.red64[w]);
        const unsigned long long Cm = (unsigned long long)zmin << 24;
        if (Cm > lowkey) lowkey = Cm;
    }
    unsigned long long S_tot = 0;
    if (pl.need_mass) {
        const MassBlock* blocks = A.blocks + (int64_t)row * A.nblk;
        unsigned long long part = 0;
        for (int ci = tid; ci < A.nblk; ci += kThreads) part += block_share(load_block(blocks + ci), c.m, pl.inv_T);
        S_tot = block_sum_u64(part, sh.red64);
    }
    if (pl.need_mass && !pl.window) {
        // whole-row draw; only the kept-id list brought the row here
        if (A.out_kept_ids) {
            const int R = min(A.kept_stride, kSelCap);
            unsigned long long Cr = fb_search<T, false>(c, alive, (unsigned long long)(R - 1));
            if (Cr == 0) Cr = alive;
            const int n = fb_gather<T>(c, Cr, sel);
            for (int i = tid; i < n; i += kThreads) {
                int rank = 0;
                for (int j = 0; j < n; ++j) rank += (sel[j] > sel[i]) ? 1 : 0;
                if (rank < A.kept_stride) A.out_kept_ids[(int64_t)c.b * A.kept_stride + rank] = ck_idx(sel[i]);
            }
            cta_sync();
        }
        draw_whole_row<T>(A, sh, smem, o, c.rp, c.b, c.g, row, c.m, pl.inv_T, S_tot, u);
        return;
    }
    if (c.rp.top_p > 0.0f && c.rp.top_p < 1.0f) {
        unsigned long long S = S_tot;
        if (!pl.need_mass) {
            unsigned long long part = 0;
            fb_pass<T>(c, [&](int tok, float z) {
                if (make_ck(z, c.id0 + tok) >= lowkey) part += fb_mass(c, z);
            });
            S = block_sum_u64(part, sh.red64);
        }
        unsigned long long Tp = __double2ull_rz(__dmul_rn((double)c.rp.top_p, __ull2double_rn(S)));
        if (Tp < 1) Tp = 1;
        const unsigned long long Cp = fb_search<T, true>(c, lowkey, Tp - 1);
        if (Cp > lowkey) lowkey = Cp;
    }
    // the kept set is {rank key >= lowkey}: its mass, its size, then the draw in ascending token index
    unsigned long long part = 0;
    int cnt = 0;
    fb_pass<T>(c, [&](int tok, float z) {
        if (make_ck(z, c.id0 + tok) >= lowkey) { part += fb_mass(c, z); ++cnt; }
    });
    const unsigned long long S = block_sum_u64(part, sh.red64);
    const int n_kept = (int)block_sum_u64((uint64_t)cnt, sh.red64);
    if (S == 0) {
        row_fail(o, BORN_ROW_ALL_MASKED);
        return;
    }
    unsigned long long t = __double2ull_rz(__dmul_rn((double)u, __ull2double_rn(S)));
    if (t > S - 1) t = S - 1;
    {
        unsigned long long run = 0;
        const int nchunks = (c.V + kFbChunk - 1) / kFbChunk;
        unsigned long long* qm = c.bwt;  // masses of one chunk, in token order
        for (int ci = 0; ci < nchunks; ++ci) {
            fb_load<T>(c, ci);
            for (int e = tid; e < kFbChunk; e += kThreads) {
                const float z = c.chunk[e];
                qm[e] = (z > -INFINITY && make_ck(z, c.id0 + ci * kFbChunk + e) >= lowkey) ? fb_mass(c, z) : 0ull;
            }
            cta_sync();
            constexpr int PER = kFbChunk / kThreads;  // consecutive tokens per thread
            unsigned long long loc = 0;
            for (int j = 0; j < PER; ++j) loc += qm[tid * PER + j];
            unsigned long long incl = loc;
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
            if (run + total > t) {  // the token is in this chunk (uniform)
                if (run + incl > t && run + incl - loc <= t) {
                    unsigned long long acc = run + incl - loc;
                    for (int j = 0; j < PER; ++j) {
                        const unsigned long long q = qm[tid * PER + j];
                        if (acc + q > t) {
                            A.out_token[c.b] = c.id0 + ci * kFbChunk + tid * PER + j;
                            A.out_status[c.b] = BORN_ROW_OK;
                            if (A.out_prob) A.out_prob[c.b] = __double2float_rn(__ddiv_rn(__ull2double_rn(q), __ull2double_rn(S)));
                            break;
                        }
                        acc += q;
                    }
                }
                break;
            }
            run += total;
        }
        cta_sync();
    }
    if (A.out_kept_count && tid == 0) A.out_kept_count[c.b] = n_kept;
    if (A.out_kept_ids) {
        const int R = min(min(A.kept_stride, kSelCap), n_kept);
        unsigned long long Cr = fb_search<T, false>(c, lowkey, (unsigned long long)(R - 1));
        if (Cr < lowkey) Cr = lowkey;
        const int n = fb_gather<T>(c, Cr, sel);
        for (int i = tid; i < n; i += kThreads) {
            int rank = 0;
            for (int j = 0; j < n; ++j) rank += (sel[j] > sel[i]) ? 1 : 0;
            if (rank < A.kept_stride) A.out_kept_ids[(int64_t)c.b * A.kept_stride + rank] = ck_idx(sel[i]);
        }
        cta_sync();
    }
}

}  // namespace born
