// Sampling over the whole vocabulary, for rows no top-k or top-p narrows: temperature-only
// sampling, and min-p with any number of survivors.  Such a row has no small candidate set, so
// it is drawn in two launches instead of through the candidate buffer of sample_kernel:
//
// Launch 1 (fullrow_stat_kernel): CTAs over contiguous ranges of every row leave the range's
// maximum (NaN-propagating) and its share of the log-sum-exp.
// Launch 2 (fullrow_draw_kernel): every CTA folds those into the row maximum m, then forms the
// fixed-point masses q = rne(exp_det((z - m) * inv_T) * 2^40) of its chunks of 4096 tokens
// (tokens that the mask or min-p removes weigh nothing) and leaves the chunk sums in scratch;
// the last CTA of the row (atomic ticket, no spinning) picks the chunk the target
// t = min(floor(u * S), S - 1) falls into, scans inside it in token order and writes token,
// probability q / S, log-sum-exp and status.
//
// Integer masses make every sum exact, so the result does not depend on how the row was cut.
// The arithmetic is the reference's softmax shape -- maximum, exp of the shifted logits, sum
// (born: internal/autodiff/ops/softmax.go:214-238).
#pragma once
#include "../../include/born_sampler.h"
#include "spec.cuh"

namespace born {

constexpr int kFrThreads = 256;
constexpr int kFrChunk = 4096;     // tokens per chunk of the draw
constexpr int kFrMaxParts = 64;    // CTAs per row in either launch

struct FullRowArgs {
    const void* logits;
    const uint32_t* mask;
    const float* uniforms;
    int32_t* out_token;
    float* out_prob;
    float* out_lse;
    int32_t* out_status;
    int32_t* out_kept_count;
    float2* stat;               // [B, parts1]: range maximum, sum of 2^((z - max) * c2)
    unsigned long long* csum;   // [B, nchunks]
    uint32_t* ccount;           // [B, nchunks]
    uint32_t* tickets;          // [B], zero between launches
    unsigned long long* total_out;  // when set: launch 2 only leaves the row's total mass here (no draw, no outputs)
    int64_t row_stride, mask_stride;
    int B, V, parts1;
    float temperature, min_p;
    int vec_ok;                 // rows are 16-byte aligned: vector loads
};

template <typename T>
__device__ __forceinline__ float fr_load(const T* p) {
    if constexpr (sizeof(T) == 4) return __ldg(reinterpret_cast<const float*>(p));
    else return bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(p)));
}
// VecOf<T>::n consecutive logits starting at element e (a multiple of the vector length)
template <typename T>
__device__ __forceinline__ void fr_load_vec(const T* row, int e, int V, bool vec_ok, float* v) {
    constexpr int VEC = 16 / (int)sizeof(T);
    if (vec_ok && e + VEC <= V) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + e));
        if constexpr (VEC == 4) {
            v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y);
            v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
        } else {
            v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xFFFF0000u);
            v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xFFFF0000u);
            v[4] = __uint_as_float(raw.z << 16); v[5] = __uint_as_float(raw.z & 0xFFFF0000u);
            v[6] = __uint_as_float(raw.w << 16); v[7] = __uint_as_float(raw.w & 0xFFFF0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) v[i] = (e + i < V) ? fr_load(row + e + i) : -INFINITY;
    }
}
template <int VEC>
__device__ __forceinline__ void fr_apply_mask(const uint32_t* mrow, int e, float* v) {
    // e is a multiple of VEC (4 or 8), so the bits of one vector sit in one mask word
    const uint32_t bits = __ldg(mrow + (e >> 5)) >> (e & 31);
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = ((bits >> i) & 1u) ? v[i] : -INFINITY;
}

// ------------------------------------------------------------------ launch 1: range statistics
template <typename T, bool kHasMask>
__global__ void __launch_bounds__(kFrThreads) fullrow_stat_kernel(const FullRowArgs A) {
    constexpr int VEC = 16 / (int)sizeof(T);
    __shared__ float redm[kFrThreads / 32], reds[kFrThreads / 32];
    const int tid = threadIdx.x, row_i = blockIdx.y, part = blockIdx.x;
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)row_i * A.row_stride;
    const uint32_t* mrow = kHasMask ? A.mask + (int64_t)row_i * A.mask_stride : nullptr;
    const int nvec = (A.V + VEC - 1) / VEC;
    const int per = (nvec + A.parts1 - 1) / A.parts1;
    const int lo = part * per, hi = min(nvec, lo + per);
    const float c2 = 1.44269504f / A.temperature;
    float mx = -INFINITY, R = -1e30f, s = 0.0f;
    constexpr int UN = 4;  // vectors in flight per thread: the loop is bound by load latency otherwise
    for (int g0 = lo + tid; g0 < hi; g0 += kFrThreads * UN) {
        float v[UN][VEC];
#pragma unroll
        for (int k = 0; k < UN; ++k) {
            const int g = g0 + k * kFrThreads;
            if (g < hi) {
                fr_load_vec<T>(row, g * VEC, A.V, A.vec_ok != 0, v[k]);
                if constexpr (kHasMask) fr_apply_mask<VEC>(mrow, g * VEC, v[k]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[k][i] = -INFINITY;
            }
        }
        float m = v[0][0];
#pragma unroll
        for (int k = 0; k < UN; ++k)
#pragma unroll
            for (int i = 0; i < VEC; ++i) m = max_nan(m, v[k][i]);
        mx = max_nan(mx, m);
        if (m > R) {
            s *= ex2_approx(__fmul_rn(R - m, c2));
            R = m;
        }
        const float nRc = -R * c2;
#pragma unroll
        for (int k = 0; k < UN; ++k)
#pragma unroll
            for (int i = 0; i < VEC; ++i) s += ex2_approx(fmaf(v[k][i], c2, nRc));
    }
    // block reduce: maximum, then the sums rescaled to it
    float wm = mx;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) wm = max_nan(wm, __shfl_xor_sync(0xffffffffu, wm, d));
    float ws = (s > 0.0f && wm == wm) ? s * ex2_approx(__fmul_rn(R - wm, c2)) : 0.0f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, d);
    if ((tid & 31) == 0) { redm[tid >> 5] = wm; reds[tid >> 5] = ws; }
    __syncthreads();
    if (tid == 0) {
        float m = redm[0];
        for (int w = 1; w < kFrThreads / 32; ++w) m = max_nan(m, redm[w]);
        float tot = 0.0f;
        for (int w = 0; w < kFrThreads / 32; ++w)
            if (reds[w] > 0.0f) tot += reds[w] * ex2_approx(__fmul_rn(redm[w] - m, c2));
        A.stat[(size_t)row_i * A.parts1 + part] = make_float2(m, tot);
    }
}

// ------------------------------------------------------------------ launch 2: masses and draw
struct FrShared {
    unsigned long long red64[kFrThreads / 32];
    unsigned long long scan[kFrThreads / 32];
    unsigned long long pick_before, total;
    float m_row, lse_sum;
    int last, pick_chunk, token;
    uint32_t kept_total;
    unsigned long long q_tok;
};

template <typename T, bool kHasMask>
__global__ void __launch_bounds__(kFrThreads) fullrow_draw_kernel(const FullRowArgs A) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int PER = kFrChunk / kFrThreads;  // 16 tokens per thread and chunk
    __shared__ FrShared sh;
    const int tid = threadIdx.x, row_i = blockIdx.y, part = blockIdx.x, nparts = gridDim.x;
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)row_i * A.row_stride;
    const uint32_t* mrow = kHasMask ? A.mask + (int64_t)row_i * A.mask_stride : nullptr;
    const int V = A.V;
    const float inv_T = __fdiv_rn(1.0f, A.temperature);
    const float c2 = inv_T * 1.44269504f;
    const uint64_t Qa = A.min_p > 0.0f ? __double2ull_ru((double)A.min_p * 1099511627776.0) : 0ull;

    // row maximum and log-sum-exp from the range statistics (every CTA on its own)
    if (tid < 32) {
        float m = -INFINITY;
        for (int p = tid; p < A.parts1; p += 32) m = max_nan(m, __ldcg(&A.stat[(size_t)row_i * A.parts1 + p].x));
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) m = max_nan(m, __shfl_xor_sync(0xffffffffu, m, d));
        float s = 0.0f;
        for (int p = tid; p < A.parts1; p += 32) {
            const float2 st = __ldcg(&A.stat[(size_t)row_i * A.parts1 + p]);
            if (st.y > 0.0f) s += st.y * ex2_approx(__fmul_rn(st.x - m, c2));
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
        if (tid == 0) { sh.m_row = m; sh.lse_sum = s; sh.last = 0; sh.token = -1; sh.q_tok = 0; }
    }
    __syncthreads();
    const float m_row = sh.m_row;
    int status = BORN_ROW_OK;
    if (m_row != m_row) status = BORN_ROW_NAN;
    else if (m_row == INFINITY) status = BORN_ROW_POS_INF;
    else if (m_row == -INFINITY) status = BORN_ROW_ALL_MASKED;
    if (status != BORN_ROW_OK) {
        if (part == 0 && tid == 0 && !A.total_out) {
            A.out_token[row_i] = -1;
            A.out_status[row_i] = status;
            if (A.out_prob) A.out_prob[row_i] = 0.0f;
            if (A.out_lse) A.out_lse[row_i] = NAN;
            if (A.out_kept_count) A.out_kept_count[row_i] = 0;
        }
        return;
    }
    // mass of one token; `kept` says whether it belongs to the kept set at all
    auto weight = [&](float z, bool& kept) -> uint64_t {
        const float x = scaled_shift(z, m_row, inv_T);
        uint64_t q = (x < -30.0f) ? 0ull : mass_of(x);
        kept = (z > -INFINITY) && !(Qa && q < Qa);
        return kept ? q : 0ull;
    };
    const int nchunks = (V + kFrChunk - 1) / kFrChunk;
    const int per = (nchunks + nparts - 1) / nparts;
    const int c_lo = min(nchunks, part * per), c_hi = min(nchunks, c_lo + per);
    unsigned long long* csum = A.csum + (size_t)row_i * nchunks;
    uint32_t* ccount = A.ccount + (size_t)row_i * nchunks;
    for (int cc = c_lo; cc < c_hi; ++cc) {
        uint64_t s = 0;
        uint32_t nk = 0;
#pragma unroll
        for (int i = 0; i < PER / VEC; ++i) {
            const int e = cc * kFrChunk + (tid + kFrThreads * i) * VEC;  // coalesced vectors
            if (e >= V) continue;
            float v[VEC];
            fr_load_vec<T>(row, e, V, A.vec_ok != 0, v);
            if constexpr (kHasMask) fr_apply_mask<VEC>(mrow, e, v);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                bool kept;
                s += weight(v[k], kept);
                if (A.out_kept_count) nk += kept ? 1u : 0u;
            }
        }
        const uint64_t tot_s = block_sum_u64(s, sh.red64);
        const uint64_t tot_n = A.out_kept_count ? block_sum_u64((uint64_t)nk, sh.red64) : 0ull;  // only when asked for
        if (tid == 0) { csum[cc] = tot_s; ccount[cc] = (uint32_t)tot_n; }
    }
    // ticket: the last CTA of the row draws
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t tk = atomicAdd(&A.tickets[row_i], 1u);
        sh.last = (tk == (uint32_t)nparts - 1);
        if (sh.last) A.tickets[row_i] = 0;
    }
    __syncthreads();
    if (!sh.last) return;
    __threadfence();
    {
        uint64_t s = 0;
        uint32_t nk = 0;
        for (int cc = tid; cc < nchunks; cc += kFrThreads) { s += __ldcg(&csum[cc]); nk += __ldcg(&ccount[cc]); }
        const uint64_t S = block_sum_u64(s, sh.red64);
        const uint64_t NK = block_sum_u64((uint64_t)nk, sh.red64);
        if (A.total_out) {  // the caller only wants the total (top-p over the whole vocabulary)
            if (tid == 0) A.total_out[row_i] = S;
            return;
        }
        if (tid == 0) {
            sh.total = S;
            sh.kept_total = (uint32_t)NK;
            sh.pick_chunk = -1;
            if (S > 0) {
                const float u = A.uniforms ? A.uniforms[row_i] : 0.0f;
                uint64_t t = __double2ull_rz(__dmul_rn((double)u, __ull2double_rn(S)));
                if (t > S - 1) t = S - 1;
                uint64_t cum = 0;
                int cc = 0;
                for (; cc < nchunks - 1; ++cc) {
                    const uint64_t c = __ldcg(&csum[cc]);
                    if (cum + c > t) break;
                    cum += c;
                }
                sh.pick_chunk = cc;
                sh.pick_before = t - cum;
            }
        }
        __syncthreads();
    }
    const int pc = sh.pick_chunk;
    if (pc >= 0) {
        // the picked chunk again, this time 16 consecutive tokens per thread: scan in token order
        uint64_t w[PER];
        uint64_t s = 0;
#pragma unroll
        for (int i = 0; i < PER / VEC; ++i) {
            const int e = pc * kFrChunk + PER * tid + VEC * i;
            float v[VEC];
#pragma unroll
            for (int k = 0; k < VEC; ++k) v[k] = -INFINITY;
            if (e < V) {
                fr_load_vec<T>(row, e, V, A.vec_ok != 0, v);
                if constexpr (kHasMask) fr_apply_mask<VEC>(mrow, e, v);
            }
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                bool kept;
                w[VEC * i + k] = (e + k < V) ? weight(v[k], kept) : 0ull;
                s += w[VEC * i + k];
            }
        }
        // exclusive scan over the threads
        const int lane = tid & 31, wp = tid >> 5;
        uint64_t incl = s;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint64_t up = shfl_up_u64(incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) sh.scan[wp] = incl;
        __syncthreads();
        uint64_t base = 0;
        for (int i = 0; i < wp; ++i) base += sh.scan[i];
        const uint64_t excl = base + incl - s;
        const uint64_t t = sh.pick_before;
        if (t >= excl && t < excl + s) {
            uint64_t cum = excl, qsel = w[PER - 1];
            int k = PER - 1;
            bool found = false;
#pragma unroll
            for (int i = 0; i < PER; ++i) {  // (no dynamic index into w: it stays in registers)
                if (!found && cum + w[i] > t) { k = i; qsel = w[i]; found = true; }
                cum += w[i];
            }
            sh.token = pc * kFrChunk + PER * tid + k;
            sh.q_tok = qsel;
        }
        __syncthreads();
    }
    if (tid == 0) {
        const uint64_t S = sh.total;
        if (pc < 0 || sh.token < 0) {  // cannot happen while the row maximum is finite
            A.out_token[row_i] = -1;
            A.out_status[row_i] = BORN_ROW_ALL_MASKED;
            if (A.out_prob) A.out_prob[row_i] = 0.0f;
        } else {
            A.out_token[row_i] = sh.token;
            A.out_status[row_i] = BORN_ROW_OK;
            if (A.out_prob) A.out_prob[row_i] = __double2float_rn(__ddiv_rn(__ull2double_rn(sh.q_tok), __ull2double_rn(S)));
        }
        if (A.out_lse) A.out_lse[row_i] = m_row * inv_T + __log2f(sh.lse_sum) * 0.69314718f;
        if (A.out_kept_count) A.out_kept_count[row_i] = (int)sh.kept_total;
    }
}

struct FullRowScratchLayout {
    size_t tickets, stat, csum, ccount, totals, total;
};
inline FullRowScratchLayout fullrow_scratch_layout(int B, int V, int parts1) {
    FullRowScratchLayout L;
    const size_t nchunks = (size_t)(V + kFrChunk - 1) / kFrChunk;
    size_t off = 0;
    L.tickets = off; off += ((size_t)B * 4 + 255) / 256 * 256;
    L.stat = off; off += ((size_t)B * parts1 * 8 + 255) / 256 * 256;
    L.csum = off; off += ((size_t)B * nchunks * 8 + 255) / 256 * 256;
    L.ccount = off; off += ((size_t)B * nchunks * 4 + 255) / 256 * 256;
    L.totals = off; off += ((size_t)B * 8 + 255) / 256 * 256;
    L.total = off;
    return L;
}
inline int fullrow_parts(int B, int V, int num_sms) {
    const int nchunks = (V + kFrChunk - 1) / kFrChunk;
    int p = (8 * num_sms + B - 1) / B;  // about eight small CTAs per SM
    if (p > nchunks) p = nchunks;
    if (p > kFrMaxParts) p = kFrMaxParts;
    if (p < 1) p = 1;
    return p;
}

template <typename T, bool M>
inline int launch_fullrow_t(const FullRowArgs& A, int parts2, cudaStream_t st) {
    fullrow_stat_kernel<T, M><<<dim3((unsigned)A.parts1, (unsigned)A.B, 1), kFrThreads, 0, st>>>(A);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    fullrow_draw_kernel<T, M><<<dim3((unsigned)parts2, (unsigned)A.B, 1), kFrThreads, 0, st>>>(A);
    return (int)cudaGetLastError();
}
// returns 0 or a cudaError_t
inline int launch_fullrow(const FullRowArgs& A, int dtype, int parts2, cudaStream_t st) {
    const bool m = A.mask != nullptr;
    if (dtype == BORN_DTYPE_F32) return m ? launch_fullrow_t<float, true>(A, parts2, st) : launch_fullrow_t<float, false>(A, parts2, st);
    return m ? launch_fullrow_t<uint16_t, true>(A, parts2, st) : launch_fullrow_t<uint16_t, false>(A, parts2, st);
}

}  // namespace born

// ------------------------------------------------------------------ penalised copy of the rows
// The whole-vocabulary routes read a row more than once, so for rows with history penalties
// they work on an fp32 copy that already holds the penalised logits: a vector copy (bf16 is
// widened, exactly), then one small CTA per row that applies the penalties to the distinct
// history tokens -- the same operations in the same order as the one-pass kernel:
// repetition (z > 0 ? z / r : z * r), then z - (frequency * count + presence).
namespace born {

struct PenaliseArgs {
    const void* logits;        // [B, row_stride] fp32 or bf16
    float* out;                // [B, out_stride] fp32
    const int32_t* history;    // [B, history_stride]
    const int32_t* history_len;  // [B] or null
    int64_t row_stride, out_stride;
    int B, V, history_stride;
    float repetition, frequency, presence;
};

template <typename T>
__global__ void __launch_bounds__(kFrThreads) widen_copy_kernel(const PenaliseArgs A) {
    const int row_i = blockIdx.y;
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)row_i * A.row_stride;
    float* out = A.out + (int64_t)row_i * A.out_stride;
    for (int e = blockIdx.x * kFrThreads + threadIdx.x; e < A.V; e += gridDim.x * kFrThreads) out[e] = fr_load<T>(row + e);
}

template <typename T>
__global__ void __launch_bounds__(kFrThreads) penalise_patch_kernel(const PenaliseArgs A) {
    __shared__ int32_t ids[BORN_MAX_HISTORY];
    const int tid = threadIdx.x, row_i = blockIdx.x;
    int len = A.history_len ? A.history_len[row_i] : A.history_stride;
    len = max(0, min(min(len, A.history_stride), (int)BORN_MAX_HISTORY));
    const int32_t* h = A.history + (int64_t)row_i * A.history_stride;
    for (int i = tid; i < len; i += kFrThreads) ids[i] = h[i];
    __syncthreads();
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)row_i * A.row_stride;
    float* out = A.out + (int64_t)row_i * A.out_stride;
    for (int i = tid; i < len; i += kFrThreads) {
        const int id = ids[i];
        if (id < 0 || id >= A.V) continue;
        int cnt = 0;
        bool first = true;
        for (int j = 0; j < len; ++j) {
            const bool eq = (ids[j] == id);
            cnt += eq ? 1 : 0;
            if (eq && j < i) first = false;
        }
        if (!first) continue;  // once per distinct token
        float z = fr_load<T>(row + id);
        if (A.repetition != 1.0f && A.repetition != 0.0f) z = (z > 0.0f) ? __fdiv_rn(z, A.repetition) : __fmul_rn(z, A.repetition);
        if (A.frequency != 0.0f || A.presence != 0.0f) {
            float pen = __fmul_rn(A.frequency, (float)cnt);
            pen = __fadd_rn(pen, A.presence);
            z = __fsub_rn(z, pen);
        }
        out[id] = z;
    }
}

// returns 0 or a cudaError_t
inline int launch_penalised_copy(const PenaliseArgs& A, int dtype, int num_sms, cudaStream_t st) {
    int parts = (8 * num_sms + A.B - 1) / A.B;
    const int maxp = (A.V + kFrThreads * 4 - 1) / (kFrThreads * 4);
    if (parts > maxp) parts = maxp;
    if (parts < 1) parts = 1;
    const dim3 g((unsigned)parts, (unsigned)A.B, 1);
    if (dtype == BORN_DTYPE_F32) widen_copy_kernel<float><<<g, kFrThreads, 0, st>>>(A);
    else widen_copy_kernel<uint16_t><<<g, kFrThreads, 0, st>>>(A);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    if (dtype == BORN_DTYPE_F32) penalise_patch_kernel<float><<<A.B, kFrThreads, 0, st>>>(A);
    else penalise_patch_kernel<uint16_t><<<A.B, kFrThreads, 0, st>>>(A);
    return (int)cudaGetLastError();
}

}  // namespace born
