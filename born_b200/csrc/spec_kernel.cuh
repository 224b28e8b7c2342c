// Speculative-decoding verification: accept/reject of K draft tokens per sequence and the
// resampling draw from the residual distribution max(0, p - q), in two launches.
//
// Launch 1 (spec_mass_kernel) treats every row of the call on its own -- (K+1) target rows
// and K draft rows per sequence -- and cuts it into contiguous ranges of tiles so that the GPU
// sees a few waves of CTAs whatever the batch.  A CTA streams its tiles through a ring of
// shared-memory stages filled by 1-D bulk copies (TMA, non-multicast) and leaves, per block of
// 1024 tokens, the block maximum and the exact fixed-point mass of the block relative to it
// (one warp per block: warp-shuffle max, deterministic exp, integer warp sum).
//
// Launch 2 (spec_draw_kernel) gives every sequence kSpecParts CTAs.  Each of them folds the
// block results into row maxima and row totals (one rescale per block), runs the accept tests
//     u * q(x) < p(x)   <=>   (u * wq_x) * S_p < wp_x * S_q
// and so knows the first rejecting position (or that the bonus token is due).  Only that
// position is drawn: the CTAs share its chunks of 4096 tokens, leave the chunk sums of the
// residual masses in scratch, and the last one to finish (atomic ticket, no spinning) picks
// the chunk the target falls into, scans inside it and writes the sequence's outputs.
//
// The row arithmetic keeps the reference's shape -- maximum, exp of the shifted logits, sum
// (born: internal/autodiff/ops/softmax.go:214-238) -- with integer masses in place of the
// float32 running sum so that the result does not depend on the order of accumulation.
#pragma once
#include "../../include/born_sampler.h"
#include "spec.cuh"

namespace born {

constexpr int kSpecThreads = 256;
constexpr int kSpecTile = 8192;  // floats per stage (32 KB)
constexpr int kSpecStages = 3;
constexpr int kSpecMassBlock = 1024;  // tokens per mass block, aligned to the row start
constexpr int kSpecMaxBlocks = 512;  // => vocab <= 524,288 on this path
constexpr int kSpecHalf = kSpecTile / 2;  // tokens per chunk in the paired (p, q) pass
constexpr int kSpecMaxChunks = kSpecMaxBlocks * kSpecMassBlock / kSpecHalf;
constexpr int kSpecParts = 8;  // CTAs per sequence in the draw launch
constexpr int kSpecMaxRows = 2 * BORN_MAX_DRAFT + 1;
constexpr int kRowBadToken = 5;
static_assert(kSpecThreads == kThreads, "the block helpers in spec.cuh are sized for kThreads");

struct BlockMass {  // result of one 1024-token block
    float m;               // block maximum (NaN if the block holds one)
    uint32_t pad;
    unsigned long long M;  // sum of the fixed-point masses relative to m
};
static_assert(sizeof(BlockMass) == 16, "BlockMass size");

// Scratch of one call: per-sequence tickets (zero between launches), chunk sums of the draw,
// block results of every row.
struct SpecScratchLayout {
    size_t tickets, csum, blocks, total;
};
inline SpecScratchLayout spec_scratch_layout(int B, int K, int V) {
    SpecScratchLayout L;
    const size_t nblk = (size_t)(V + kSpecMassBlock - 1) / kSpecMassBlock, nchb = (size_t)(V + kSpecHalf - 1) / kSpecHalf;
    size_t off = 0;
    L.tickets = off; off += ((size_t)B * 4 + 255) / 256 * 256;
    L.csum = off; off += ((size_t)B * nchb * 8 + 255) / 256 * 256;
    L.blocks = off; off += (size_t)B * (2 * K + 1) * nblk * sizeof(BlockMass);
    L.total = off;
    return L;
}

struct SpecKernelArgs {
    const float* target;
    const float* draft;
    const int32_t* draft_tok;
    const float* u_accept;
    const float* u_resample;
    int32_t* accept_len;
    int32_t* out_tok;
    int32_t* status;
    uint32_t* tickets;
    unsigned long long* csum;
    BlockMass* blocks;
    int* dev_error;
    int B, K, V, target_rows;
    float inv_T;
    int tma;
};

struct SpecPipe {  // ring of tiles; `it` counts every tile ever issued/consumed by this CTA
    float* tiles;
    unsigned long long* bars;
    int tma;
    uint32_t issued, consumed;
    __device__ float* tile(uint32_t it) const { return tiles + (size_t)(it % kSpecStages) * kSpecTile; }
    __device__ uint64_t* bar(uint32_t it) const { return reinterpret_cast<uint64_t*>(&bars[it % kSpecStages]); }
};

// thread 0: one or two bulk copies into the next tile
__device__ __forceinline__ void spec_issue(SpecPipe& P, const float* src0, int n0, const float* src1, int n1) {
    uint64_t* bar = P.bar(P.issued);
    float* dst = P.tile(P.issued);
    uint32_t b0 = ((uint32_t)n0 * 4u + 15u) & ~15u, b1 = src1 ? (((uint32_t)n1 * 4u + 15u) & ~15u) : 0u;
    mbar_expect_tx(bar, b0 + b1);
    bulk_load(dst, src0, b0, bar);
    if (src1) bulk_load(dst + kSpecHalf, src1, b1, bar);
    P.issued++;
}

// Consume side: wait for the next tile (or fill it with plain loads when rows are not 16-byte
// aligned).  A timeout sets *fail.
__device__ __forceinline__ float* spec_acquire(SpecPipe& P, const float* src0, int n0, const float* src1, int n1, int* fail) {
    float* t = P.tile(P.consumed);
    if (P.tma) {
        if (!mbar_wait(P.bar(P.consumed), (P.consumed / kSpecStages) & 1u)) *fail = 1;
    } else {
        for (int i = threadIdx.x; i < n0; i += kSpecThreads) t[i] = src0[i];
        if (src1) for (int i = threadIdx.x; i < n1; i += kSpecThreads) t[kSpecHalf + i] = src1[i];
        __syncthreads();
    }
    P.consumed++;
    return t;
}

// Exclusive block scan helper: returns the exclusive prefix of v over threads, total in *tot.
__device__ __forceinline__ uint64_t block_excl_scan_u64(uint64_t v, unsigned long long* buf, uint64_t* tot) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint64_t incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        uint64_t up = shfl_up_u64(incl, d);
        if (lane >= d) incl += up;
    }
    __syncthreads();
    if (lane == 31) buf[w] = incl;
    __syncthreads();
    uint64_t base = 0, total = 0;
#pragma unroll
    for (int i = 0; i < kSpecThreads / 32; ++i) {
        uint64_t x = buf[i];
        if (i < w) base += x;
        total += x;
    }
    *tot = total;
    return base + incl - v;
}

// Weight of token i in the draw: residual max(0, p - q) or the plain mass of p.
struct DrawCtx {
    int residual;  // 1: max(0, p_i - q_i); 0: mass of p_i
    float mp, mq, inv_T, invSp, invSq;
};
__device__ __forceinline__ uint64_t draw_weight(const DrawCtx& D, float zp, float zq) {
    if (D.residual) {
        float pi = __fmul_rn(exp_det<false>(scaled_shift(zp, D.mp, D.inv_T)), D.invSp);
        float qi = __fmul_rn(exp_det<false>(scaled_shift(zq, D.mq, D.inv_T)), D.invSq);
        float r = __fsub_rn(pi, qi);
        r = r > 0.0f ? r : 0.0f;
        return __float2ull_rn(__fmul_rn(r, 1099511627776.0f));
    }
    return mass_of<false>(scaled_shift(zp, D.mp, D.inv_T));
}

// ------------------------------------------------------------------ launch 1: block masses
struct MassShared {
    unsigned long long bars[kSpecStages];
    int fail;
};

__global__ void __launch_bounds__(kSpecThreads, 2) spec_mass_kernel(const SpecKernelArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ MassShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.y, V = A.V;
    const int ntarget = A.B * A.target_rows;
    const float* src_row = row < ntarget ? A.target + (int64_t)row * V : A.draft + (int64_t)(row - ntarget) * V;
    const int nch = (V + kSpecTile - 1) / kSpecTile;
    const int nblk = (V + kSpecMassBlock - 1) / kSpecMassBlock;
    const int per = (nch + (int)gridDim.x - 1) / (int)gridDim.x;
    const int t_lo = blockIdx.x * per, t_hi = min(nch, t_lo + per);
    if (t_lo >= t_hi) return;

    SpecPipe P;
    P.tiles = reinterpret_cast<float*>(smem);
    P.bars = sh.bars;
    P.tma = A.tma;
    P.issued = P.consumed = 0;
    if (tid == 0) {
        for (int s = 0; s < kSpecStages; ++s) mbar_init(reinterpret_cast<uint64_t*>(&sh.bars[s]), 1);
        mbar_fence_init();
        sh.fail = 0;
    }
    __syncthreads();
    auto issue = [&](int t) { spec_issue(P, src_row + (size_t)t * kSpecTile, min(kSpecTile, V - t * kSpecTile), nullptr, 0); };
    if (P.tma && tid == 0)
        for (int t = t_lo; t < min(t_lo + kSpecStages, t_hi); ++t) issue(t);

    for (int t = t_lo; t < t_hi; ++t) {
        const int nvalid = min(kSpecTile, V - t * kSpecTile);
        const float* tile = spec_acquire(P, src_row + (size_t)t * kSpecTile, nvalid, nullptr, 0, &sh.fail);
        const int base = warp * kSpecMassBlock;
        if (base < nvalid) {
            float v[32];
            float mc = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 q = *reinterpret_cast<const float4*>(tile + base + 4 * (lane + 32 * i));
                v[4 * i + 0] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
            }
            if (base + kSpecMassBlock > nvalid) {  // the row ends inside this block: nothing beyond it counts
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (base + 4 * (lane + 32 * (i >> 2)) + (i & 3) >= nvalid) v[i] = -INFINITY;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) mc = max_nan(mc, v[i]);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) mc = max_nan(mc, __shfl_xor_sync(0xffffffffu, mc, d));
            uint64_t Mc = 0;
#pragma unroll
            for (int i = 0; i < 32; ++i) Mc += mass_of<false>(scaled_shift(v[i], mc, A.inv_T));
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) Mc += shfl_xor_u64(Mc, d);
            if (lane == 0 && !sh.fail) {
                BlockMass r;
                r.m = mc; r.pad = 0; r.M = Mc;
                A.blocks[(size_t)row * nblk + t * (kSpecTile / kSpecMassBlock) + warp] = r;
            }
        }
        __syncthreads();
        if (sh.fail) break;
        if (P.tma && tid == 0 && t + kSpecStages < t_hi) {
            fence_proxy_async();
            issue(t + kSpecStages);
        }
    }
    if (sh.fail && tid == 0) {
        if (P.tma)
            for (uint32_t it = P.consumed; it < P.issued; ++it) mbar_wait(P.bar(it), (it / kSpecStages) & 1u);
        atomicExch(A.dev_error, 2);
    }
}

// ------------------------------------------------------------------ launch 2: accept and draw
struct DrawShared {
    unsigned long long bars[kSpecStages];
    unsigned long long red64[kSpecThreads / 32];
    unsigned long long scan[kSpecThreads / 32];
    unsigned long long rowS[kSpecMaxRows];   // row totals of the fixed-point masses
    unsigned long long csum[kSpecMaxChunks];
    unsigned long long pick_before;
    uint32_t rowkey[kSpecMaxRows];           // order-preserving key of the row maximum
    int rownan[kSpecMaxRows];
    int accept[BORN_MAX_DRAFT];
    int pstat[BORN_MAX_DRAFT + 1];
    int fail, last, pick_chunk, token;
};

__global__ void __launch_bounds__(kSpecThreads, 2) spec_draw_kernel(const SpecKernelArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ DrawShared sh;
    const int tid = threadIdx.x;
    const int part = blockIdx.x, nparts = gridDim.x, b = blockIdx.y;
    const int K = A.K, V = A.V, R = A.target_rows;
    const int nblk = (V + kSpecMassBlock - 1) / kSpecMassBlock;
    const int nrows = R + K;  // this sequence's rows: r < R target row r, else draft row r - R
    auto row_id = [&](int r) { return r < R ? b * R + r : A.B * R + b * K + (r - R); };

    SpecPipe P;
    P.tiles = reinterpret_cast<float*>(smem);
    P.bars = sh.bars;
    P.tma = A.tma;
    P.issued = P.consumed = 0;
    if (tid == 0) {
        for (int s = 0; s < kSpecStages; ++s) mbar_init(reinterpret_cast<uint64_t*>(&sh.bars[s]), 1);
        mbar_fence_init();
        sh.fail = 0;
        sh.last = 0;
        sh.token = -1;
    }
    if (tid < kSpecMaxRows) { sh.rowS[tid] = 0; sh.rowkey[tid] = zkey(-INFINITY); sh.rownan[tid] = 0; }
    __syncthreads();

    // ---- row maxima and totals from the block results (every CTA of the sequence on its own):
    // one warp per row, the blocks of the row dealt out to its lanes and held in registers, so
    // that the block results are fetched once, all loads in flight together, and the warp
    // reduces by shuffles.
    {
        constexpr int kPerLane = kSpecMaxBlocks / 32;  // 16 blocks per lane at most
        const int lane = tid & 31, warp = tid >> 5;
        for (int r = warp; r < nrows; r += kSpecThreads / 32) {
            const BlockMass* rb = A.blocks + (size_t)row_id(r) * nblk;
            float bm[kPerLane];
            unsigned long long bM[kPerLane];
#pragma unroll
            for (int q = 0; q < kPerLane; ++q) {
                const int blk = lane + 32 * q;
                bm[q] = -INFINITY;
                bM[q] = 0;
                if (blk < nblk) {
                    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(rb + blk));
                    bm[q] = __uint_as_float(raw.x);
                    bM[q] = ((unsigned long long)raw.w << 32) | raw.z;
                }
            }
            float m = -INFINITY;
#pragma unroll
            for (int q = 0; q < kPerLane; ++q) m = max_nan(m, bm[q]);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, d));
            unsigned long long S = 0;
            if (m == m && m > -INFINITY && m < INFINITY) {
#pragma unroll
                for (int q = 0; q < kPerLane; ++q) {
                    if (bm[q] == -INFINITY) continue;
                    const float ef = exp_det<false>(scaled_shift(bm[q], m, A.inv_T));
                    S += __double2ull_rn(__dmul_rn(__ull2double_rn(bM[q]), (double)ef));
                }
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) S += shfl_xor_u64(S, d);
            }
            if (lane == 0) {
                sh.rownan[r] = (m != m) ? 1 : 0;
                sh.rowkey[r] = (m != m) ? zkey(-INFINITY) : zkey(m);
                sh.rowS[r] = S;
            }
        }
    }
    __syncthreads();
    auto row_status = [&](int r) {
        const float m = zkey_to_float(sh.rowkey[r]);
        if (sh.rownan[r]) return (int)BORN_ROW_NAN;
        if (m == INFINITY) return (int)BORN_ROW_POS_INF;
        if (m == -INFINITY) return (int)BORN_ROW_ALL_MASKED;
        return (int)BORN_ROW_OK;
    };
    const bool dev_failed = *reinterpret_cast<volatile int*>(A.dev_error) != 0;  // launch 1 gave up on a copy
    if (tid < K) {
        const int j = tid;
        int st = row_status(j);
        if (st == BORN_ROW_OK) st = row_status(R + j);
        if (dev_failed) st = 100 + BORN_ERR_DEVICE_TIMEOUT;
        int acc = 0;
        if (st == BORN_ROW_OK) {
            const int x = A.draft_tok[(int64_t)b * K + j];
            if (x < 0 || x >= V) st = kRowBadToken;
            else {
                const float* rowp = A.target + ((int64_t)b * R + j) * (int64_t)V;
                const float* rowq = A.draft + ((int64_t)b * K + j) * (int64_t)V;
                const uint64_t wp = mass_of<false>(scaled_shift(rowp[x], zkey_to_float(sh.rowkey[j]), A.inv_T));
                const uint64_t wq = mass_of<false>(scaled_shift(rowq[x], zkey_to_float(sh.rowkey[R + j]), A.inv_T));
                const double u = (double)A.u_accept[(int64_t)b * K + j];
                const double lhs = __dmul_rn(__dmul_rn(u, __ull2double_rn(wq)), __ull2double_rn(sh.rowS[j]));
                const double rhs = __dmul_rn(__ull2double_rn(wp), __ull2double_rn(sh.rowS[R + j]));
                acc = lhs < rhs;
            }
        }
        sh.accept[j] = acc;
        sh.pstat[j] = st;
    }
    if (tid == K) sh.pstat[K] = (R > K) ? (dev_failed ? 100 + BORN_ERR_DEVICE_TIMEOUT : row_status(K)) : BORN_ROW_OK;
    __syncthreads();

    // ---- the outcome for the sequence (same in every thread of every CTA of the sequence)
    int len = K, seq_status = BORN_ROW_OK, jstar = -1;
    DrawCtx D;
    D.residual = 0; D.inv_T = A.inv_T; D.mp = 0.0f; D.mq = 0.0f; D.invSp = 0.0f; D.invSq = 0.0f;
    for (int i = 0; i < K; ++i) {
        if (sh.pstat[i] != BORN_ROW_OK) { seq_status = sh.pstat[i]; len = i; break; }
        if (!sh.accept[i]) { len = i; jstar = i; D.residual = 1; break; }
    }
    if (len == K && seq_status == BORN_ROW_OK && R > K) {
        if (sh.pstat[K] != BORN_ROW_OK) seq_status = sh.pstat[K];
        else jstar = K;
    }
    auto write_outputs = [&](int token) {  // one thread
        int32_t* out = A.out_tok + (int64_t)b * (K + 1);
        for (int i = 0; i <= K; ++i) out[i] = -1;
        for (int i = 0; i < len; ++i) out[i] = A.draft_tok[(int64_t)b * K + i];
        if (jstar >= 0) out[jstar] = token;
        A.accept_len[b] = len;
        A.status[b] = seq_status;
    };
    if (jstar < 0) {  // nothing to draw
        if (part == 0 && tid == 0) write_outputs(-1);
        return;
    }
    const float* rowp = A.target + ((int64_t)b * R + jstar) * (int64_t)V;
    const float* rowq = D.residual ? A.draft + ((int64_t)b * K + jstar) * (int64_t)V : nullptr;
    D.mp = zkey_to_float(sh.rowkey[jstar]);
    if (D.residual) {
        D.mq = zkey_to_float(sh.rowkey[R + jstar]);
        D.invSp = __double2float_rn(__ddiv_rn(1099511627776.0, __ull2double_rn(sh.rowS[jstar])));
        D.invSq = __double2float_rn(__ddiv_rn(1099511627776.0, __ull2double_rn(sh.rowS[R + jstar])));
    }

    // ---- chunk sums of the draw weights: this CTA's share of the chunks
    const int nchb = (V + kSpecHalf - 1) / kSpecHalf;
    auto issue_b = [&](int cc) {
        const int n = min(kSpecHalf, V - cc * kSpecHalf);
        spec_issue(P, rowp + (size_t)cc * kSpecHalf, n, D.residual ? rowq + (size_t)cc * kSpecHalf : nullptr, n);
    };
    // Weights of the 16 tokens a thread owns in a chunk: four strided groups of four when only
    // the sum matters (conflict-free shared loads), 16 consecutive tokens when the caller needs
    // them in index order.
    auto chunk_weights = [&](const float* tile, int nvalid, uint64_t* wts) -> uint64_t {
        uint64_t s = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = wts ? 16 * tid + 4 * i : 4 * (tid + kSpecThreads * i);
            float4 zp = *reinterpret_cast<const float4*>(tile + e);
            float4 zq = D.residual ? *reinterpret_cast<const float4*>(tile + kSpecHalf + e) : zp;
            const float ap[4] = {zp.x, zp.y, zp.z, zp.w}, aq[4] = {zq.x, zq.y, zq.z, zq.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint64_t wv = (e + k < nvalid) ? draw_weight(D, ap[k], aq[k]) : 0ull;
                if (wts) wts[4 * i + k] = wv;
                s += wv;
            }
        }
        return s;
    };
    // sums of chunks [lo, hi) into dst[cc] (thread 0 writes); tiles issued before have all been consumed
    auto sum_chunks = [&](int lo, int hi, unsigned long long* dst) {
        if (P.tma && tid == 0)
            for (int cc = lo; cc < min(lo + kSpecStages, hi); ++cc) issue_b(cc);
        for (int cc = lo; cc < hi; ++cc) {
            const int nvalid = min(kSpecHalf, V - cc * kSpecHalf);
            const float* tile = spec_acquire(P, rowp + (size_t)cc * kSpecHalf, nvalid,
                                             D.residual ? rowq + (size_t)cc * kSpecHalf : nullptr, nvalid, &sh.fail);
            uint64_t s = chunk_weights(tile, nvalid, nullptr);
            s = block_sum_u64(s, sh.red64);
            if (tid == 0) dst[cc] = s;
            __syncthreads();
            if (sh.fail) break;
            if (P.tma && tid == 0 && cc + kSpecStages < hi) {
                fence_proxy_async();
                issue_b(cc + kSpecStages);
            }
        }
    };
    unsigned long long* csum_g = A.csum + (size_t)b * nchb;
    const int per = (nchb + nparts - 1) / nparts;
    const int lo = min(nchb, part * per), hi = min(nchb, lo + per);
    sum_chunks(lo, hi, csum_g);
    if (sh.fail && tid == 0) atomicExch(A.dev_error, 2);

    // ---- ticket: the last CTA of the sequence picks the chunk and the token
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t tk = atomicAdd(&A.tickets[b], 1u);
        sh.last = (tk == (uint32_t)nparts - 1);
        if (sh.last) A.tickets[b] = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!sh.last) {
        if (sh.fail && tid == 0 && P.tma)
            for (uint32_t it = P.consumed; it < P.issued; ++it) mbar_wait(P.bar(it), (it / kSpecStages) & 1u);
        return;
    }
    __threadfence();
    int token = -1;
    bool failed = sh.fail || *reinterpret_cast<volatile int*>(A.dev_error) != 0;
    for (int attempt = 0; attempt < 2 && !failed; ++attempt) {
        if (attempt == 0) {
            for (int cc = tid; cc < nchb; cc += kSpecThreads) sh.csum[cc] = __ldcg(&csum_g[cc]);
        } else {
            sum_chunks(0, nchb, sh.csum);  // the residual vanished: the plain masses of p, all chunks
            if (sh.fail) { failed = true; break; }
        }
        __syncthreads();
        if (tid == 0) {
            uint64_t W = 0;
            for (int cc = 0; cc < nchb; ++cc) W += sh.csum[cc];
            sh.pick_chunk = -1;
            if (W > 0) {
                const float u = A.u_resample[(int64_t)b * (K + 1) + jstar];
                uint64_t t = __double2ull_rz(__dmul_rn((double)u, __ull2double_rn(W)));
                if (t > W - 1) t = W - 1;
                uint64_t cum = 0;
                int cc = 0;
                for (; cc < nchb - 1; ++cc) {
                    if (cum + sh.csum[cc] > t) break;
                    cum += sh.csum[cc];
                }
                sh.pick_chunk = cc;
                sh.pick_before = t - cum;
            }
        }
        __syncthreads();
        const int pc = sh.pick_chunk;
        if (pc < 0) {  // the residual vanished in fp32: draw from p instead
            if (D.residual) { D.residual = 0; continue; }
            break;
        }
        const int nvalid = min(kSpecHalf, V - pc * kSpecHalf);
        if (P.tma && tid == 0) { fence_proxy_async(); issue_b(pc); }
        const float* tile = spec_acquire(P, rowp + (size_t)pc * kSpecHalf, nvalid,
                                         D.residual ? rowq + (size_t)pc * kSpecHalf : nullptr, nvalid, &sh.fail);
        uint64_t wts[16];
        uint64_t s = chunk_weights(tile, nvalid, wts);
        uint64_t tot;
        uint64_t excl = block_excl_scan_u64(s, sh.scan, &tot);
        const uint64_t t = sh.pick_before;
        if (t >= excl && t < excl + s) {
            uint64_t cum = excl;
            int k = 15;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                if (cum + wts[i] > t) { k = i; break; }
                cum += wts[i];
            }
            sh.token = pc * kSpecHalf + 16 * tid + k;
        }
        __syncthreads();
        token = sh.token;
        if (sh.fail) failed = true;
        break;
    }
    if (tid == 0) {
        if (failed) {
            if (P.tma)
                for (uint32_t it = P.consumed; it < P.issued; ++it) mbar_wait(P.bar(it), (it / kSpecStages) & 1u);
            atomicExch(A.dev_error, 2);
            seq_status = 100 + BORN_ERR_DEVICE_TIMEOUT;
            len = min(len, jstar);
        }
        write_outputs(failed ? -1 : token);
    }
}

inline size_t spec_smem_bytes() { return (size_t)kSpecStages * kSpecTile * sizeof(float); }

// raises the dynamic shared-memory limit of both kernels; once per device, at handle creation
inline cudaError_t spec_attrs_all() {
    cudaError_t e = cudaFuncSetAttribute(spec_mass_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)spec_smem_bytes());
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(spec_draw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)spec_smem_bytes());
}

// returns 0 or a cudaError_t; `num_sms` sizes the first launch
inline int launch_spec(SpecKernelArgs A, int num_sms, cudaStream_t st) {
    if (A.V > kSpecMaxBlocks * kSpecMassBlock) return (int)cudaErrorInvalidValue;
    A.tma = ((uintptr_t)A.target % 16 == 0) && ((uintptr_t)A.draft % 16 == 0) && (((int64_t)A.V * 4) % 16 == 0);
    cudaError_t e;
    const int rows = A.B * (A.target_rows + A.K);
    const int nch = (A.V + kSpecTile - 1) / kSpecTile;
    // CTAs per row: enough for a few full waves of two CTAs per SM, with the last wave as full
    // as the choice allows, and at least two tiles each
    int parts = 1;
    {
        const int slots = 2 * num_sms;
        double best = 0.0;
        for (int p = 1; p <= 8 && 2 * p <= nch + 1; ++p) {
            const double waves = (double)rows * p / slots;
            const double fill = waves / (double)((long long)waves + ((double)(long long)waves < waves ? 1 : 0));
            const double score = (waves >= 2.0 ? 1.0 : waves / 2.0) * fill;
            if (score > best + 0.02) { best = score; parts = p; }
        }
    }
    spec_mass_kernel<<<dim3((unsigned)parts, (unsigned)rows, 1), kSpecThreads, spec_smem_bytes(), st>>>(A);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    const int nchb = (A.V + kSpecHalf - 1) / kSpecHalf;
    int dparts = kSpecParts < nchb ? kSpecParts : nchb;
    spec_draw_kernel<<<dim3((unsigned)dparts, (unsigned)A.B, 1), kSpecThreads, spec_smem_bytes(), st>>>(A);
    return (int)cudaGetLastError();
}

}  // namespace born
