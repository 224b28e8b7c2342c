// Speculative-decoding verification: accept/reject of K draft tokens per sequence and the
// resampling draw from the residual distribution max(0, p - q), in one launch.
//
// CTA (j, b) owns draft position j of sequence b.  It streams the target row p_j and the
// draft row q_j once through a ring of shared-memory tiles filled by 1-D bulk copies
// (TMA, non-multicast) and computes, per block of 1024 tokens, the block maximum and the
// exact fixed-point mass of the block relative to it (one warp per block: warp-shuffle
// max, deterministic exp, integer warp sum).  The row totals follow from the block
// results with one rescale per block, so the accept test
//     u * q(x) < p(x)   <=>   (u * wq_x) * S_p < wp_x * S_q
// needs a single pass over HBM.  A position that rejects draws its replacement token right
// away (a second pass over its two rows, normally served by L2): per-chunk sums of the
// residual masses, then a scan inside the one chunk the target falls into.  The extra CTA
// (K, b) draws the bonus token from the last target row.  The last CTA of a sequence to
// finish (atomic ticket, no spinning) picks the first rejection and writes the outputs.
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
constexpr int kMassBlock = 1024;  // tokens per mass block, aligned to the row start
constexpr int kSpecMaxBlocks = 512;  // => vocab <= 524,288 on this path
constexpr int kSpecHalf = kSpecTile / 2;  // tokens per chunk in the paired (p, q) pass
constexpr int kSpecMaxChunks = kSpecMaxBlocks * kMassBlock / kSpecHalf;
constexpr int kRowBadToken = 5;

struct SeqScratch {  // 256 bytes per sequence, zero between launches
    uint32_t ticket;
    int32_t pos_status[BORN_MAX_DRAFT + 1];
    int32_t accept[BORN_MAX_DRAFT];
    int32_t token[BORN_MAX_DRAFT + 1];
    int32_t pad[13];
};
static_assert(sizeof(SeqScratch) == 256, "SeqScratch size");

inline size_t spec_scratch_bytes(int max_batch) { return sizeof(SeqScratch) * (size_t)max_batch; }

struct SpecKernelArgs {
    const float* target;
    const float* draft;
    const int32_t* draft_tok;
    const float* u_accept;
    const float* u_resample;
    int32_t* accept_len;
    int32_t* out_tok;
    int32_t* status;
    uint8_t* scratch;
    int* dev_error;
    int B, K, V, target_rows;
    float inv_T;
    int tma;
};

struct SpecShared {
    unsigned long long bars[kSpecStages];
    unsigned long long red64[kSpecThreads / 32];
    unsigned long long scan[kSpecThreads / 32];
    float blk_m[2][kSpecMaxBlocks];
    unsigned long long blk_M[2][kSpecMaxBlocks];
    unsigned long long csum[kSpecMaxChunks];
    float redf[kSpecThreads / 32];
    int fail;
    int last;
    int pick_chunk;
    unsigned long long pick_before;
    int token;
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

// Weight of token i in the draw of this CTA: residual max(0, p - q) or the plain mass of p.
struct DrawCtx {
    int residual;  // 1: max(0, p_i - q_i); 0: mass of p_i
    float mp, mq, inv_T, invSp, invSq;
};
__device__ __forceinline__ uint64_t draw_weight(const DrawCtx& D, float zp, float zq) {
    if (D.residual) {
        float pi = __fmul_rn(exp_det(scaled_shift(zp, D.mp, D.inv_T)), D.invSp);
        float qi = __fmul_rn(exp_det(scaled_shift(zq, D.mq, D.inv_T)), D.invSq);
        float r = __fsub_rn(pi, qi);
        r = r > 0.0f ? r : 0.0f;
        return __float2ull_rn(__fmul_rn(r, 1099511627776.0f));
    }
    return mass_of(scaled_shift(zp, D.mp, D.inv_T));
}

__global__ void __launch_bounds__(kSpecThreads, 2) spec_verify_kernel(const SpecKernelArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ SpecShared sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int j = blockIdx.x, b = blockIdx.y;
    const int K = A.K, V = A.V;
    const bool bonus = (j == K);
    SeqScratch* seq = reinterpret_cast<SeqScratch*>(A.scratch) + b;

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
    }
    __syncthreads();

    const float* rowp = A.target + ((int64_t)b * A.target_rows + j) * (int64_t)V;
    const float* rowq = bonus ? nullptr : A.draft + ((int64_t)b * K + j) * (int64_t)V;
    const int nrows = bonus ? 1 : 2;
    const int nch = (V + kSpecTile - 1) / kSpecTile;
    const int nblk = (V + kMassBlock - 1) / kMassBlock;

    // tile `t` of pass A: row t / nch, chunk t % nch
    auto issue_a = [&](int t) {
        const int r = t / nch, cc = t % nch;
        const float* src = (r == 0 ? rowp : rowq) + (size_t)cc * kSpecTile;
        spec_issue(P, src, min(kSpecTile, V - cc * kSpecTile), nullptr, 0);
    };
    // Consume side: wait for tile `it` (or fill it with plain loads when rows are not
    // 16-byte aligned); returns false on a timeout.
    auto acquire = [&](const float* src0, int n0, const float* src1, int n1) -> float* {
        float* t = P.tile(P.consumed);
        if (P.tma) {
            if (!mbar_wait(P.bar(P.consumed), (P.consumed / kSpecStages) & 1u)) sh.fail = 1;
        } else {
            for (int i = tid; i < n0; i += kSpecThreads) t[i] = src0[i];
            if (src1) for (int i = tid; i < n1; i += kSpecThreads) t[kSpecHalf + i] = src1[i];
            __syncthreads();
        }
        P.consumed++;
        return t;
    };

    int status = BORN_ROW_OK;
    const int ntile_a = nrows * nch;
    if (P.tma && tid == 0)
        for (int t = 0; t < min(kSpecStages, ntile_a); ++t) issue_a(t);

    // ------------------------------------------------------------ pass A: block masses
    for (int t = 0; t < ntile_a; ++t) {
        const int r = t / nch, cc = t % nch;
        const int nvalid = min(kSpecTile, V - cc * kSpecTile);
        const float* src = (r == 0 ? rowp : rowq) + (size_t)cc * kSpecTile;
        const float* tile = acquire(src, nvalid, nullptr, 0);
        const int base = warp * kMassBlock;
        if (base < nvalid) {
            float v[32];
            float mc = -INFINITY;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = base + 4 * (lane + 32 * i);
                float4 q = *reinterpret_cast<const float4*>(tile + e);
                v[4 * i + 0] = (e + 0 < nvalid) ? q.x : -INFINITY;
                v[4 * i + 1] = (e + 1 < nvalid) ? q.y : -INFINITY;
                v[4 * i + 2] = (e + 2 < nvalid) ? q.z : -INFINITY;
                v[4 * i + 3] = (e + 3 < nvalid) ? q.w : -INFINITY;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) mc = max_nan(mc, v[i]);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) mc = max_nan(mc, __shfl_xor_sync(0xffffffffu, mc, d));
            uint64_t Mc = 0;
            if (!bonus) {  // the bonus row only needs its maximum here
#pragma unroll
                for (int i = 0; i < 32; ++i) Mc += mass_of(scaled_shift(v[i], mc, A.inv_T));
#pragma unroll
                for (int d = 16; d > 0; d >>= 1) Mc += shfl_xor_u64(Mc, d);
            }
            if (lane == 0) {
                const int blk = cc * (kSpecTile / kMassBlock) + warp;
                sh.blk_m[r][blk] = mc;
                sh.blk_M[r][blk] = Mc;
            }
        }
        __syncthreads();
        if (sh.fail) break;
        if (P.tma && tid == 0 && t + kSpecStages < ntile_a) {
            fence_proxy_async();
            issue_a(t + kSpecStages);
        }
    }

    // row maxima and totals
    float mrow[2] = {-INFINITY, -INFINITY};
    uint64_t Srow[2] = {0, 0};
    if (!sh.fail) {
        for (int r = 0; r < nrows; ++r) {
            float m = -INFINITY;
            for (int i = tid; i < nblk; i += kSpecThreads) m = max_nan(m, sh.blk_m[r][i]);
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, d));
            __syncthreads();
            if (lane == 0) sh.redf[warp] = m;
            __syncthreads();
            m = sh.redf[0];
            for (int w = 1; w < kSpecThreads / 32; ++w) m = max_nan(m, sh.redf[w]);
            mrow[r] = m;
            uint64_t part = 0;
            if (!bonus && m == m && m > -INFINITY && m < INFINITY) {
                for (int i = tid; i < nblk; i += kSpecThreads) {
                    const float mc = sh.blk_m[r][i];
                    if (mc == -INFINITY) continue;
                    const float ef = exp_det(scaled_shift(mc, m, A.inv_T));
                    part += __double2ull_rn(__dmul_rn(__ull2double_rn(sh.blk_M[r][i]), (double)ef));
                }
            }
            // block_sum_u64 is sized for kThreads == kSpecThreads
            Srow[r] = block_sum_u64(part, sh.red64);
            __syncthreads();
        }
        for (int r = 0; r < nrows && status == BORN_ROW_OK; ++r) {
            if (mrow[r] != mrow[r]) status = BORN_ROW_NAN;
            else if (mrow[r] == INFINITY) status = BORN_ROW_POS_INF;
            else if (mrow[r] == -INFINITY) status = BORN_ROW_ALL_MASKED;
        }
    }

    int accept = 0;
    int need_draw = 0;
    DrawCtx D;
    D.residual = 0; D.mp = mrow[0]; D.mq = mrow[1]; D.inv_T = A.inv_T; D.invSp = 0.0f; D.invSq = 0.0f;
    if (!sh.fail && status == BORN_ROW_OK) {
        if (bonus) {
            need_draw = 1;
        } else {
            const int x = A.draft_tok[(int64_t)b * K + j];
            if (x < 0 || x >= V) status = kRowBadToken;
            else {
                const uint64_t wp = mass_of(scaled_shift(rowp[x], mrow[0], A.inv_T));
                const uint64_t wq = mass_of(scaled_shift(rowq[x], mrow[1], A.inv_T));
                const double u = (double)A.u_accept[(int64_t)b * K + j];
                const double lhs = __dmul_rn(__dmul_rn(u, __ull2double_rn(wq)), __ull2double_rn(Srow[0]));
                const double rhs = __dmul_rn(__ull2double_rn(wp), __ull2double_rn(Srow[1]));
                accept = lhs < rhs;
                if (!accept) {
                    need_draw = 1;
                    D.residual = 1;
                    D.invSp = __double2float_rn(__ddiv_rn(1099511627776.0, __ull2double_rn(Srow[0])));
                    D.invSq = __double2float_rn(__ddiv_rn(1099511627776.0, __ull2double_rn(Srow[1])));
                }
            }
        }
    }

    // ------------------------------------------------ pass B: draw (rejecting positions, bonus)
    int token = -1;
    for (int attempt = 0; attempt < 2 && need_draw && !sh.fail; ++attempt) {
        const int nchb = (V + kSpecHalf - 1) / kSpecHalf;
        auto issue_b = [&](int cc) {
            const int n = min(kSpecHalf, V - cc * kSpecHalf);
            spec_issue(P, rowp + (size_t)cc * kSpecHalf, n, D.residual ? rowq + (size_t)cc * kSpecHalf : nullptr, n);
        };
        // Weights of the 16 tokens a thread owns in a chunk: four strided groups of four when
        // only the sum matters (conflict-free shared loads), 16 consecutive tokens when the
        // caller needs them in index order.
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
        // tiles issued so far have all been consumed (passes are separated by barriers)
        if (P.tma && tid == 0)
            for (int cc = 0; cc < min(kSpecStages, nchb); ++cc) issue_b(cc);
        for (int cc = 0; cc < nchb; ++cc) {
            const int nvalid = min(kSpecHalf, V - cc * kSpecHalf);
            const float* tile = acquire(rowp + (size_t)cc * kSpecHalf, nvalid,
                                        D.residual ? rowq + (size_t)cc * kSpecHalf : nullptr, nvalid);
            uint64_t s = chunk_weights(tile, nvalid, nullptr);
            s = block_sum_u64(s, sh.red64);
            if (tid == 0) sh.csum[cc] = s;
            __syncthreads();
            if (sh.fail) break;
            if (P.tma && tid == 0 && cc + kSpecStages < nchb) {
                fence_proxy_async();
                issue_b(cc + kSpecStages);
            }
        }
        if (sh.fail) break;
        if (tid == 0) {
            uint64_t W = 0;
            for (int cc = 0; cc < nchb; ++cc) W += sh.csum[cc];
            sh.pick_chunk = -1;
            if (W > 0) {
                const float u = A.u_resample[(int64_t)b * (K + 1) + j];
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
        {
            const int nvalid = min(kSpecHalf, V - pc * kSpecHalf);
            if (P.tma && tid == 0) { fence_proxy_async(); issue_b(pc); }
            const float* tile = acquire(rowp + (size_t)pc * kSpecHalf, nvalid,
                                        D.residual ? rowq + (size_t)pc * kSpecHalf : nullptr, nvalid);
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
        }
        break;
    }

    if (sh.fail) {
        if (tid == 0) {
            if (P.tma)
                for (uint32_t it = P.consumed; it < P.issued; ++it) mbar_wait(P.bar(it), (it / kSpecStages) & 1u);
            atomicExch(A.dev_error, 2);
        }
        status = 100 + BORN_ERR_DEVICE_TIMEOUT;
    }

    // ------------------------------------------------------------ publish, ticket, finish
    if (tid == 0) {
        seq->pos_status[j] = status;
        if (!bonus) seq->accept[j] = accept;
        seq->token[j] = token;
        __threadfence();
        const uint32_t nct = gridDim.x;
        const uint32_t tk = atomicAdd(&seq->ticket, 1u);
        if (tk == nct - 1) {
            __threadfence();
            volatile SeqScratch* vs = seq;
            int32_t* out = A.out_tok + (int64_t)b * (K + 1);
            for (int i = 0; i <= K; ++i) out[i] = -1;
            int len = K, st = BORN_ROW_OK;
            for (int i = 0; i < K; ++i) {
                const int ps = vs->pos_status[i];
                if (ps != BORN_ROW_OK) { st = ps; len = i; break; }
                if (!vs->accept[i]) { len = i; out[i] = vs->token[i]; break; }
                out[i] = A.draft_tok[(int64_t)b * K + i];
            }
            if (len == K && st == BORN_ROW_OK && A.target_rows > K) {
                const int ps = vs->pos_status[K];
                if (ps != BORN_ROW_OK) st = ps;
                else out[K] = vs->token[K];
            }
            A.accept_len[b] = len;
            A.status[b] = st;
            seq->ticket = 0;
        }
    }
}

inline size_t spec_smem_bytes() { return (size_t)kSpecStages * kSpecTile * sizeof(float); }

// returns 0 or a cudaError_t
inline int launch_spec(SpecKernelArgs A, cudaStream_t st) {
    if (A.V > kSpecMaxBlocks * kMassBlock) return (int)cudaErrorInvalidValue;
    A.tma = ((uintptr_t)A.target % 16 == 0) && ((uintptr_t)A.draft % 16 == 0) && (((int64_t)A.V * 4) % 16 == 0);
    cudaError_t e = cudaFuncSetAttribute(spec_verify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)spec_smem_bytes());
    if (e != cudaSuccess) return (int)e;
    dim3 grid((unsigned)(A.target_rows > A.K ? A.K + 1 : A.K), (unsigned)A.B, 1);
    spec_verify_kernel<<<grid, kSpecThreads, spec_smem_bytes(), st>>>(A);
    return (int)cudaGetLastError();
}

}  // namespace born
