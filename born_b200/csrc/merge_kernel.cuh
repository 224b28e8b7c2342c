// merge_kernel: the second half of vocab-sharded sampling.  Every shard (a GPU of a
// tensor-parallel lm_head, or a vocabulary segment on one GPU) has left one packed record per
// row -- its k best tokens as rank keys with global token ids, its maximum and its share of
// the log-sum-exp.  One CTA per row folds the G records: row maximum, log-sum-exp, the union
// of the candidates, then top-p and the inverse-CDF draw on exact integer masses relative to
// the row maximum (finish.cuh), so the result does not depend on how the vocabulary was cut.
#pragma once
#include "finish.cuh"

namespace born {

struct MergeArgs {
    const uint8_t* gathered;  // record of (shard g, row b) at g*seg_stride + b*row_stride
    int64_t row_stride, seg_stride;
    int B, G;
    float temperature, top_p;
    const float* uniforms;
    int32_t* out_token;
    float* out_prob;
    float* out_lse;
    int32_t* out_status;
    int32_t* out_kept_ids;
    int32_t* out_kept_count;
    int kept_stride;
};

__global__ void __launch_bounds__(kThreads) merge_kernel(const __grid_constant__ MergeArgs A) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ ScanShared sh;
    const int tid = threadIdx.x, b = blockIdx.x;
    uint64_t* sel = reinterpret_cast<uint64_t*>(smem);
    unsigned long long* selq = reinterpret_cast<unsigned long long*>(sel + kSelCap);
    const float inv_T = __fdiv_rn(1.0f, A.temperature);
    const float c2 = inv_T * 1.44269504f;
    auto rec_of = [&](int g) { return A.gathered + (int64_t)g * A.seg_stride + (int64_t)b * A.row_stride; };
    // headers are read word by word: a record of an odd number of entries is only 8-byte aligned
    float m = -INFINITY;
    int inexact = 0;
    for (int g = 0; g < A.G; ++g) {
        const uint32_t* h = reinterpret_cast<const uint32_t*>(rec_of(g));
        m = max_nan(m, __uint_as_float(__ldcg(h)));
        inexact |= (int)(__ldcg(h + 3) & 2u);
    }
    float ls = 0.0f;
    if (tid == 0) sh.nl = 0;
    cta_sync();
    for (int g = 0; g < A.G; ++g) {
        const uint32_t* h = reinterpret_cast<const uint32_t*>(rec_of(g));
        const float mg = __uint_as_float(__ldcg(h)), sg = __uint_as_float(__ldcg(h + 1));
        if (sg > 0.0f) ls += sg * ex2_approx(__fmul_rn(mg - m, c2));
        const int cnt = (int)__ldcg(h + 2);
        const unsigned long long* ent = reinterpret_cast<const unsigned long long*>(rec_of(g) + kRecordHdrBytes);
        for (int i = tid; i < cnt; i += kThreads) {
            const unsigned long long e = __ldcg(ent + i);
            if (ck_alive(e)) {
                const int pos = (int)smem_atom_add(&sh.nl, 1u);
                if (pos < kSelCap) sel[pos] = e;
            }
        }
    }
    cta_sync();
    const int n = sh.nl;
    RowOut o;
    o.token = A.out_token; o.prob = A.out_prob; o.lse = A.out_lse; o.status = A.out_status;
    o.kept_ids = A.out_kept_ids; o.kept_count = A.out_kept_count; o.kept_stride = A.kept_stride;
    o.row = b;
    int status = BORN_ROW_OK;
    if (m != m) status = BORN_ROW_NAN;
    else if (m == INFINITY) status = BORN_ROW_POS_INF;
    else if (m == -INFINITY) status = BORN_ROW_ALL_MASKED;
    else if (inexact || n > kSelCap) status = BORN_ROW_OVERFLOW;
    if (A.out_lse && tid == 0) A.out_lse[b] = (status == BORN_ROW_OK || status == BORN_ROW_OVERFLOW) ? m * inv_T + __log2f(ls) * 0.69314718f : NAN;
    if (status != BORN_ROW_OK) {
        row_fail(o, status);
        return;
    }
    SelectIn in;
    in.n = n;
    in.k = 0;  // every shard has cut to its own k best already; the union is kept
    in.Qa = 0;
    in.top_p = A.top_p;
    in.S_ext = 0;
    in.complete = true;
    in.m_row = m; in.inv_T = inv_T; in.u = A.uniforms[b];
    if (n <= kThreads) select_small(in, sel, selq, sh, o);
    else select_and_draw(in, sel, selq, sh, o);
}

}  // namespace born
