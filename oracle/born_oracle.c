/*
 * born_oracle.c -- CPU oracle for the token-sampling / constrained-decoding path.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT.  Only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load this file's shared object.  The CUDA
 * library never calls into it and has no CPU fallback.
 *
 * Two groups of functions live here.
 *
 * (1) Restatements of the arithmetic the reference (born v0.1.1, pure Go) has on this
 *     path.  Each follows the cited Go function statement by statement:
 *       born_oracle_ref_logsoftmax  <- internal/nn/cross_entropy.go:126-153 (logSoftmax)
 *                                      internal/autodiff/ops/cross_entropy.go:306-331
 *       born_oracle_ref_softmax     <- internal/autodiff/ops/softmax.go:214-238 (softmaxFloat32)
 *                                      internal/autodiff/ops/cross_entropy.go:165-190
 *       born_oracle_ref_argmax      <- internal/nn/cross_entropy.go:241-251 (argmax, strict '>')
 *       born_oracle_ref_accuracy    <- internal/nn/cross_entropy.go:261-284 (Accuracy)
 *     These are pinned against the known-answer vectors of the reference's own tests
 *     (internal/autodiff/ops/ops_test.go:651-692,737-775;
 *      internal/nn/cross_entropy_test.go:42-57,124-142,146-178,181-210).
 *
 * (2) The sampler itself (penalties, grammar mask, temperature, top-k, min-p, top-p,
 *     inverse-CDF draw, speculative accept/reject).  The reference snapshot contains NO
 *     sampler, no tests and no golden vectors for these steps, so for them
 *     PARITY IS UNPINNED: this file is the written specification the CUDA kernels are
 *     checked against, cross-checked in the test-suite by an independent float64 numpy
 *     restatement.  Structure kept from the reference where it applies: max-shift before
 *     exp, row-major [batch, vocab] rows, int32 token indices, lowest index wins ties.
 *
 * Determinism contract (what makes token ids bit-exact between this file and the GPU):
 *   - every decision sum is an exact integer sum of fixed-point masses
 *       q_i = rne_u64( exp_det((z_i - m) * inv_T) * 2^40 ),
 *     so the order of accumulation cannot matter;
 *   - exp_det is a fixed sequence of IEEE fp32 operations (mul, add, fused multiply-add)
 *     written identically here and in the CUDA source; this file must be compiled with
 *     -ffp-contract=off so that only the explicit fmaf() calls are fused;
 *   - ranking is (value descending, token index ascending) on the penalised, masked,
 *     un-scaled logit.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BORN_ORACLE_VERSION 2

/* row status codes (same values as the CUDA library's BORN_ROW_*) */
enum {
    ROW_OK = 0,
    ROW_ALL_MASKED = 1,  /* no token with a logit above -inf */
    ROW_NAN = 2,         /* a NaN logit among the allowed tokens */
    ROW_POS_INF = 3,     /* a +inf logit among the allowed tokens */
    ROW_OVERFLOW = 4,    /* only produced by the GPU path (candidate buffer exceeded) */
    ROW_BAD_TOKEN = 5    /* speculative verify: draft token outside [0, vocab) */
};

enum { FLAG_GREEDY = 1u };

typedef struct {
    float temperature;        /* 0 => greedy */
    float top_p;              /* >= 1 or <= 0 => off */
    float min_p;              /* <= 0 => off */
    int32_t top_k;            /* <= 0 => off */
    float repetition_penalty; /* 1 (or 0) => off */
    float frequency_penalty;
    float presence_penalty;
    uint32_t flags;           /* bit 0: greedy */
} oracle_row_params;

/* ------------------------------------------------------------------------------------
 * (1) reference restatements
 * ---------------------------------------------------------------------------------- */

/* internal/nn/cross_entropy.go:126-153.  Returns log-sum-exp; writes z - lse to out
 * when out != NULL.  exp and log are evaluated in float64 and rounded to float32, the
 * running sum is float32 in index order, exactly as the Go code does. */
float born_oracle_ref_logsoftmax(const float* z, int n, float* out) {
    float maxz = z[0];
    for (int i = 1; i < n; i++)
        if (z[i] > maxz) maxz = z[i];
    float sum = 0.0f;
    for (int i = 0; i < n; i++) sum += (float)exp((double)(z[i] - maxz));
    float lse = maxz + (float)log((double)sum);
    if (out)
        for (int i = 0; i < n; i++) out[i] = z[i] - lse;
    return lse;
}

/* internal/autodiff/ops/softmax.go:214-238: three passes per row. */
void born_oracle_ref_softmax(const float* in, float* out, int batch, int classes) {
    for (int b = 0; b < batch; b++) {
        const float* x = in + (size_t)b * classes;
        float* y = out + (size_t)b * classes;
        float maxv = x[0];
        for (int j = 1; j < classes; j++)
            if (x[j] > maxv) maxv = x[j];
        float sum = 0.0f;
        for (int j = 0; j < classes; j++) {
            y[j] = (float)exp((double)(x[j] - maxv));
            sum += y[j];
        }
        for (int j = 0; j < classes; j++) y[j] /= sum;
    }
}

/* internal/nn/cross_entropy.go:241-251: strict '>' so the first maximum wins. */
int born_oracle_ref_argmax(const float* z, int n) {
    int idx = 0;
    float v = z[0];
    for (int i = 1; i < n; i++)
        if (z[i] > v) { v = z[i]; idx = i; }
    return idx;
}

/* internal/nn/cross_entropy.go:261-284 */
float born_oracle_ref_accuracy(const float* logits, const int32_t* targets, int batch, int classes) {
    int correct = 0;
    for (int b = 0; b < batch; b++)
        if (born_oracle_ref_argmax(logits + (size_t)b * classes, classes) == (int)targets[b]) correct++;
    return (float)correct / (float)batch;
}

/* ------------------------------------------------------------------------------------
 * (2) sampler specification
 * ---------------------------------------------------------------------------------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* Deterministic exp for x <= 0.  Valid on [-80, 0]; below that (and for NaN) returns 0.
 * Cody-Waite reduction by ln2 (two constants), degree-6 polynomial on [-ln2/2, ln2/2],
 * scaling by adding n to the exponent field.  Max relative error ~1.2e-7. */
float born_oracle_exp1(float x) {
    if (!(x >= -80.0f)) return 0.0f;
    const float magic = 12582912.0f; /* 1.5 * 2^23 */
    float t = x * 0x1.715476p+0f; /* log2(e) */
    float r = t + magic;
    float nf = r - magic;
    float f = fmaf(nf, -0x1.62e4p-1f, x);      /* ln2 high part */
    f = fmaf(nf, -0x1.7f7d1cp-20f, f);         /* ln2 low part */
    float p = 0x1.687bf6p-10f;
    p = fmaf(p, f, 0x1.123b9ep-7f);
    p = fmaf(p, f, 0x1.555b58p-5f);
    p = fmaf(p, f, 0x1.55548ep-3f);
    p = fmaf(p, f, 0x1.fffff8p-2f);
    p = fmaf(p, f, 1.0f);
    p = fmaf(p, f, 1.0f);
    uint32_t n = f2u(r) - 0x4B400000u; /* two's-complement n */
    return u2f(f2u(p) + (n << 23));
}

void born_oracle_exp(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = born_oracle_exp1(x[i]);
}

#define MASS_SCALE 1099511627776.0f /* 2^40 */

static inline uint64_t mass_of(float x) { /* x = (z - m) * inv_T */
    float w = born_oracle_exp1(x);
    return (uint64_t)llrintf(w * MASS_SCALE);
}

void born_oracle_mass(const float* x, uint64_t* q, int64_t n) {
    for (int64_t i = 0; i < n; i++) q[i] = mass_of(x[i]);
}

/* rank order: value descending, index ascending.  -0 == +0 as values. */
typedef struct { float z; int32_t idx; } cand_t;

static int cand_before(const cand_t* a, const cand_t* b) {
    if (a->z > b->z) return 1;
    if (a->z < b->z) return 0;
    return a->idx < b->idx;
}
static int cmp_rank(const void* pa, const void* pb) {
    const cand_t* a = (const cand_t*)pa; const cand_t* b = (const cand_t*)pb;
    if (cand_before(a, b)) return -1;
    if (cand_before(b, a)) return 1;
    return 0;
}
static int cmp_idx(const void* pa, const void* pb) {
    int32_t a = ((const cand_t*)pa)->idx, b = ((const cand_t*)pb)->idx;
    return (a > b) - (a < b);
}

/* min-heap on rank (root = worst kept) for top-k selection */
static void heap_sift_down(cand_t* h, int n, int i) {
    for (;;) {
        int l = 2 * i + 1, r = l + 1, w = i;
        if (l < n && cand_before(&h[w], &h[l])) w = l; /* h[l] ranks after h[w] => worse */
        if (r < n && cand_before(&h[w], &h[r])) w = r;
        if (w == i) return;
        cand_t t = h[i]; h[i] = h[w]; h[w] = t; i = w;
    }
}

/* first k of z[lo..hi) in rank order (finite-or-+inf entries only); returns count */
static int topk_range(const float* z, int lo, int hi, int k, cand_t* out) {
    int n = 0;
    for (int i = lo; i < hi; i++) {
        if (!(z[i] > -INFINITY)) continue; /* skips -inf (NaN rows are rejected earlier) */
        cand_t c = { z[i], i };
        if (n < k) {
            out[n++] = c;
            if (n == k)
                for (int j = k / 2 - 1; j >= 0; j--) heap_sift_down(out, n, j);
        } else if (cand_before(&c, &out[0])) {
            out[0] = c;
            heap_sift_down(out, n, 0);
        }
    }
    return n;
}

typedef struct {
    float* z;        /* V */
    int32_t* counts; /* V, kept zero between rows */
    cand_t* cand;    /* V */
    uint64_t* q;     /* V */
} row_ws;

static int ws_alloc(row_ws* w, int V) {
    w->z = (float*)malloc(sizeof(float) * (size_t)V);
    w->counts = (int32_t*)calloc((size_t)V, sizeof(int32_t));
    w->cand = (cand_t*)malloc(sizeof(cand_t) * (size_t)V);
    w->q = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)V);
    return w->z && w->counts && w->cand && w->q;
}
static void ws_free(row_ws* w) { free(w->z); free(w->counts); free(w->cand); free(w->q); }

/* Steps 1-4 of the row pipeline: upcast, penalties, mask.  Result in w->z. */
static void prepare_row(row_ws* w, int V, int dtype, const void* row, const uint32_t* mask,
                        const int32_t* hist, int hist_n, const oracle_row_params* p) {
    float* z = w->z;
    if (dtype == 0) memcpy(z, row, sizeof(float) * (size_t)V);
    else { const uint16_t* h = (const uint16_t*)row; for (int i = 0; i < V; i++) z[i] = bf16_to_f32(h[i]); }

    float rep = p->repetition_penalty;
    int rep_on = (rep != 1.0f && rep != 0.0f);
    int add_on = (p->frequency_penalty != 0.0f || p->presence_penalty != 0.0f);
    if (hist && hist_n > 0 && (rep_on || add_on)) {
        for (int j = 0; j < hist_n; j++) { int32_t t = hist[j]; if (t >= 0 && t < V) w->counts[t]++; }
        for (int j = 0; j < hist_n; j++) {
            int32_t t = hist[j];
            if (t < 0 || t >= V) continue;
            int32_t c = w->counts[t];
            if (c == 0) continue; /* already applied for this distinct token */
            w->counts[t] = 0;
            float v = z[t];
            if (rep_on) v = (v > 0.0f) ? v / rep : v * rep;
            if (add_on) {
                float pen = p->frequency_penalty * (float)c;
                pen = pen + p->presence_penalty;
                v = v - pen;
            }
            z[t] = v;
        }
    }
    if (mask)
        for (int i = 0; i < V; i++)
            if (!((mask[i >> 5] >> (i & 31)) & 1u)) z[i] = -INFINITY;
}

typedef struct {
    int B, V, dtype;
    const void* logits; int64_t row_stride;
    const uint32_t* mask; int64_t mask_stride;
    const int32_t* history; int hist_stride; const int32_t* hist_len;
    const oracle_row_params* rp; int rp_stride; /* 0 => one params struct for all rows */
    const float* u;
    int n_segments; /* >= 1: top-k is taken per contiguous vocab segment */
    int32_t* tok; float* prob; float* lse; int32_t* status;
    int32_t* kept_ids; int32_t* kept_count; int kept_stride;
    int32_t* near_cutoff;
} sample_job;

#define SAMPLE_MASS_BLOCK 512 /* tokens per mass block of the sampler, aligned to the row start */

/* Whole-row total of the sampler when neither top-k nor min-p narrows the row: per block of
 * 512 tokens the masses are taken relative to the block maximum m_c and summed exactly (M_c);
 * a block's share of the row is S_c = rne_u64((double)M_c * (double)exp_det((m_c - m) * inv_T)).
 * This is what a single streaming pass can form before the row maximum is known. */
static uint64_t block_mass(const float* z, int lo, int hi, float inv_T, float* mc_out) {
    float mc = -INFINITY;
    for (int i = lo; i < hi; i++) if (z[i] > mc) mc = z[i];
    *mc_out = mc;
    if (mc == -INFINITY) return 0;
    uint64_t Mc = 0;
    for (int i = lo; i < hi; i++) {
        float w = born_oracle_exp1((z[i] - mc) * inv_T);
        Mc += (uint64_t)llrintf(w * 1099511627776.0f);
    }
    return Mc;
}
static uint64_t block_share(uint64_t Mc, float mc, float m, float inv_T) {
    if (Mc == 0) return 0;
    float ef = born_oracle_exp1((mc - m) * inv_T);
    return (uint64_t)llrint((double)Mc * (double)ef);
}
static uint64_t sampler_row_total(const float* z, int V, float inv_T, float m) {
    uint64_t S = 0;
    for (int lo = 0; lo < V; lo += SAMPLE_MASS_BLOCK) {
        int hi = lo + SAMPLE_MASS_BLOCK; if (hi > V) hi = V;
        float mc; uint64_t Mc = block_mass(z, lo, hi, inv_T, &mc);
        S += block_share(Mc, mc, m, inv_T);
    }
    return S;
}

static void sample_row(const sample_job* J, row_ws* w, int b) {
    const int V = J->V;
    const oracle_row_params* p = J->rp + (size_t)b * J->rp_stride;
    const char* row = (const char*)J->logits + (size_t)b * (size_t)J->row_stride * (J->dtype == 0 ? 4 : 2);
    const uint32_t* mask = J->mask ? J->mask + (size_t)b * (size_t)J->mask_stride : NULL;
    const int32_t* hist = J->history ? J->history + (size_t)b * J->hist_stride : NULL;
    int hist_n = J->history ? (J->hist_len ? J->hist_len[b] : J->hist_stride) : 0;
    if (hist_n > J->hist_stride) hist_n = J->hist_stride;
    prepare_row(w, V, J->dtype, row, mask, hist, hist_n, p);
    const float* z = w->z;

    J->tok[b] = -1;
    if (J->prob) J->prob[b] = 0.0f;
    if (J->lse) J->lse[b] = NAN;
    if (J->kept_count) J->kept_count[b] = 0;
    if (J->near_cutoff) J->near_cutoff[b] = 0;

    /* row max and validity */
    float m = -INFINITY; int has_nan = 0;
    for (int i = 0; i < V; i++) { if (z[i] != z[i]) has_nan = 1; else if (z[i] > m) m = z[i]; }
    if (has_nan) { J->status[b] = ROW_NAN; return; }
    if (m == INFINITY) { J->status[b] = ROW_POS_INF; return; }
    if (m == -INFINITY) { J->status[b] = ROW_ALL_MASKED; return; }
    J->status[b] = ROW_OK;

    int greedy = (p->flags & FLAG_GREEDY) || p->temperature == 0.0f;
    float inv_T = greedy ? 1.0f : 1.0f / p->temperature;

    /* log-sum-exp of the scaled logits, the reference's way (float64 exp rounded to
     * float32, float32 running sum in index order): internal/nn/cross_entropy.go:138-145 */
    if (J->lse) {
        float sum = 0.0f;
        for (int i = 0; i < V; i++) sum += (float)exp((double)((z[i] - m) * inv_T));
        J->lse[b] = m * inv_T + (float)log((double)sum);
    }

    if (greedy) {
        /* first maximum: internal/nn/cross_entropy.go:241-251 */
        int idx = 0; float v = z[0];
        for (int i = 1; i < V; i++) if (z[i] > v) { v = z[i]; idx = i; }
        J->tok[b] = idx;
        if (J->prob) J->prob[b] = 1.0f;
        if (J->kept_ids && J->kept_stride > 0) J->kept_ids[(size_t)b * J->kept_stride] = idx;
        if (J->kept_count) J->kept_count[b] = 1;
        return;
    }

    /* Rows that neither top-k nor min-p narrows take their total from the mass blocks. */
    int whole = !(p->top_k > 0) && !(p->min_p > 0.0f);
    uint64_t S_tot = whole ? sampler_row_total(z, V, inv_T, m) : 0;
    int topp_on = (p->top_p > 0.0f && p->top_p < 1.0f);
    if (whole && !topp_on) {
        /* Temperature-only: the draw descends the blocks.  t = min(floor(u*S), S-1) picks the
         * block by the shares S_c in ascending order, then the token inside it by the block's own
         * masses with t'' = min(floor((t - before) * M_c / S_c), M_c - 1) in float64. */
        int nfin = 0;
        for (int i = 0; i < V; i++) if (z[i] > -INFINITY) nfin++;
        if (J->kept_count) J->kept_count[b] = nfin;
        if (J->kept_ids) {
            cand_t* K0 = w->cand; int n0 = 0;
            for (int i = 0; i < V; i++) if (z[i] > -INFINITY) { K0[n0].z = z[i]; K0[n0].idx = i; n0++; }
            qsort(K0, (size_t)n0, sizeof(cand_t), cmp_rank);
            for (int i = 0; i < n0 && i < J->kept_stride; i++) J->kept_ids[(size_t)b * J->kept_stride + i] = K0[i].idx;
        }
        if (S_tot == 0) { J->status[b] = ROW_ALL_MASKED; return; }
        uint64_t t = (uint64_t)((double)J->u[b] * (double)S_tot);
        if (t > S_tot - 1) t = S_tot - 1;
        uint64_t cum = 0;
        for (int lo = 0; lo < V; lo += SAMPLE_MASS_BLOCK) {
            int hi = lo + SAMPLE_MASS_BLOCK; if (hi > V) hi = V;
            float mc; uint64_t Mc = block_mass(z, lo, hi, inv_T, &mc);
            uint64_t Sc = block_share(Mc, mc, m, inv_T);
            if (cum + Sc > t) {
                uint64_t tb = t - cum;
                uint64_t tt = (uint64_t)(((double)tb * (double)Mc) / (double)Sc);
                if (tt > Mc - 1) tt = Mc - 1;
                uint64_t c2 = 0;
                for (int i = lo; i < hi; i++) {
                    uint64_t qi = mass_of((z[i] - mc) * inv_T);
                    c2 += qi;
                    if (c2 > tt) {
                        J->tok[b] = i;
                        if (J->prob) J->prob[b] = (float)(((double)qi / (double)Mc) * ((double)Sc / (double)S_tot));
                        return;
                    }
                }
            }
            cum += Sc;
        }
        return;
    }

    /* top-k (per segment when n_segments > 1) */
    cand_t* K = w->cand; int n = 0;
    int G = J->n_segments < 1 ? 1 : J->n_segments;
    if (p->top_k > 0) {
        int seg = V / G;
        for (int g = 0; g < G; g++) {
            int lo = g * seg, hi = (g == G - 1) ? V : lo + seg;
            n += topk_range(z, lo, hi, p->top_k, K + n);
        }
    } else {
        for (int i = 0; i < V; i++) if (z[i] > -INFINITY) { K[n].z = z[i]; K[n].idx = i; n++; }
    }

    /* masses; min-p */
    uint64_t* q = w->q;
    uint64_t Qa = 0;
    if (p->min_p > 0.0f) Qa = (uint64_t)ceil((double)p->min_p * 1099511627776.0);
    int n2 = 0;
    for (int i = 0; i < n; i++) {
        float x = (K[i].z - m) * inv_T;
        uint64_t qi = (x < -30.0f) ? 0 : mass_of(x); /* below -30 the mass rounds to 0 */
        if (Qa && J->near_cutoff) {
            /* float64 recomputation: is w / w_max within 1e-6 (relative) of min_p? */
            double wd = exp(((double)K[i].z - (double)m) * (double)inv_T), a = (double)p->min_p;
            if (fabs(wd - a) <= 1e-6 * a) J->near_cutoff[b] |= 1;
        }
        if (Qa && qi < Qa) continue;
        K[n2] = K[i]; n2++;
    }
    n = n2;

    /* rank order, then top-p prefix */
    qsort(K, (size_t)n, sizeof(cand_t), cmp_rank);
    uint64_t S = 0;
    for (int i = 0; i < n; i++) { q[i] = mass_of((K[i].z - m) * inv_T); S += q[i]; }
    if (topp_on) {
        /* the nucleus is taken against the block total when nothing else narrows the row */
        uint64_t Tp = (uint64_t)((double)p->top_p * (double)(whole ? S_tot : S));
        if (Tp < 1) Tp = 1;
        uint64_t cum = 0; int keep = n;
        for (int i = 0; i < n; i++) { cum += q[i]; if (cum >= Tp) { keep = i + 1; break; } }
        if (J->near_cutoff) {
            /* float64 recomputation: is the cumulative mass at the boundary within 1e-6 of P? */
            double Sd = 0; for (int i = 0; i < n; i++) Sd += exp(((double)K[i].z - (double)m) * (double)inv_T);
            double c = 0;
            for (int i = 0; i < n; i++) {
                c += exp(((double)K[i].z - (double)m) * (double)inv_T);
                if (i + 1 == keep || i + 2 == keep) { if (fabs(c / Sd - (double)p->top_p) <= 1e-6) J->near_cutoff[b] |= 2; }
            }
        }
        n = keep;
    }

    /* kept set out, in rank order */
    if (J->kept_count) J->kept_count[b] = n;
    if (J->kept_ids)
        for (int i = 0; i < n && i < J->kept_stride; i++) J->kept_ids[(size_t)b * J->kept_stride + i] = K[i].idx;

    /* draw: ascending token index */
    qsort(K, (size_t)n, sizeof(cand_t), cmp_idx);
    S = 0;
    for (int i = 0; i < n; i++) { q[i] = mass_of((K[i].z - m) * inv_T); S += q[i]; }
    uint64_t t = (uint64_t)((double)J->u[b] * (double)S);
    if (t > S - 1) t = S - 1;
    uint64_t cum = 0; int pick = n - 1;
    for (int i = 0; i < n; i++) { cum += q[i]; if (cum > t) { pick = i; break; } }
    J->tok[b] = K[pick].idx;
    if (J->prob) J->prob[b] = (float)((double)q[pick] / (double)S);
}

typedef struct { const sample_job* J; int lo, hi; int ok; } thread_arg;

static void* sample_thread(void* a) {
    thread_arg* T = (thread_arg*)a;
    row_ws w;
    T->ok = ws_alloc(&w, T->J->V);
    if (T->ok) for (int b = T->lo; b < T->hi; b++) sample_row(T->J, &w, b);
    ws_free(&w);
    return NULL;
}

static int run_threads(void* (*fn)(void*), thread_arg* args, int nthreads) {
    if (nthreads == 1) { fn(&args[0]); return args[0].ok ? 0 : -1; }
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nthreads);
    for (int i = 0; i < nthreads; i++) pthread_create(&th[i], NULL, fn, &args[i]);
    int ok = 1;
    for (int i = 0; i < nthreads; i++) { pthread_join(th[i], NULL); ok &= args[i].ok; }
    free(th);
    return ok ? 0 : -1;
}

/* The sampler.  rp_stride: 0 = one params struct for every row, 1 = per-row array.
 * nthreads splits rows over host threads (the reference itself is single-threaded). */
int born_oracle_sample(int B, int V, int dtype, const void* logits, int64_t row_stride,
                       const uint32_t* mask, int64_t mask_stride,
                       const int32_t* history, int hist_stride, const int32_t* hist_len,
                       const oracle_row_params* rp, int rp_stride, const float* u, int n_segments,
                       int32_t* tok, float* prob, float* lse, int32_t* status,
                       int32_t* kept_ids, int32_t* kept_count, int kept_stride,
                       int32_t* near_cutoff, int nthreads) {
    sample_job J = { B, V, dtype, logits, row_stride, mask, mask_stride, history, hist_stride, hist_len,
                     rp, rp_stride, u, n_segments, tok, prob, lse, status, kept_ids, kept_count, kept_stride,
                     near_cutoff };
    if (nthreads < 1) nthreads = 1;
    if (nthreads > B) nthreads = B > 0 ? B : 1;
    thread_arg* args = (thread_arg*)calloc((size_t)nthreads, sizeof(thread_arg));
    for (int i = 0; i < nthreads; i++) {
        args[i].J = &J;
        args[i].lo = (int)((int64_t)B * i / nthreads);
        args[i].hi = (int)((int64_t)B * (i + 1) / nthreads);
    }
    int rc = run_threads(sample_thread, args, nthreads);
    free(args);
    return rc;
}

/* ------------------------------------------------------------------------------------
 * speculative-decoding verification
 * ---------------------------------------------------------------------------------- */

#define MASS_BLOCK 1024 /* tokens per mass block, aligned to the row start */

/* Deterministic total mass of a full row: per block of 1024 tokens the masses are taken
 * relative to the block maximum m_c and summed exactly; blocks are then brought to the
 * row maximum with S = sum_c rne_u64( (double)M_c * (double)exp_det((m_c - m) * inv_T) ). */
static float row_max_nan(const float* z, int V) { /* NaN if any NaN, else the maximum */
    float m = -INFINITY;
    for (int i = 0; i < V; i++) { if (z[i] != z[i]) return NAN; if (z[i] > m) m = z[i]; }
    return m;
}
static int row_status(float m) {
    if (m != m) return ROW_NAN;
    if (m == INFINITY) return ROW_POS_INF;
    if (m == -INFINITY) return ROW_ALL_MASKED;
    return ROW_OK;
}
static uint64_t row_total_mass(const float* z, int V, float inv_T, float m) {
    int nb = (V + MASS_BLOCK - 1) / MASS_BLOCK;
    uint64_t S = 0;
    for (int c = 0; c < nb; c++) {
        int lo = c * MASS_BLOCK, hi = lo + MASS_BLOCK; if (hi > V) hi = V;
        float mc = -INFINITY;
        for (int i = lo; i < hi; i++) if (z[i] > mc) mc = z[i];
        if (mc == -INFINITY) continue;
        uint64_t Mc = 0;
        for (int i = lo; i < hi; i++) Mc += mass_of((z[i] - mc) * inv_T);
        float ef = born_oracle_exp1((mc - m) * inv_T);
        S += (uint64_t)llrint((double)Mc * (double)ef);
    }
    return S;
}

/* smallest i with sum_{j<=i} w_j > t, t = min(floor(u * W), W - 1); -1 when W == 0 */
static int draw_index(const uint64_t* w, int V, float u) {
    uint64_t W = 0;
    for (int i = 0; i < V; i++) W += w[i];
    if (W == 0) return -1;
    uint64_t t = (uint64_t)((double)u * (double)W);
    if (t > W - 1) t = W - 1;
    uint64_t cum = 0;
    for (int i = 0; i < V; i++) { cum += w[i]; if (cum > t) return i; }
    return V - 1;
}

typedef struct {
    int B, K, V, target_rows; /* target_rows = K or K+1 (bonus row present) */
    const float* target; const float* draft; const int32_t* draft_tok;
    const float* u_accept;   /* [B, K] */
    const float* u_resample; /* [B, K+1]; entry j used when position j rejects, entry K for the bonus */
    float temperature;
    int32_t* accept_len; int32_t* out_tok; /* [B, K+1], -1 padded */
    int32_t* status;
} spec_job;

static void spec_seq(const spec_job* J, uint64_t* wbuf, int b) {
    const int K = J->K, V = J->V;
    float inv_T = (J->temperature == 0.0f) ? 1.0f : 1.0f / J->temperature;
    int32_t* out = J->out_tok + (size_t)b * (K + 1);
    for (int j = 0; j <= K; j++) out[j] = -1;
    J->status[b] = ROW_OK;
    int j;
    for (j = 0; j < K; j++) {
        const float* zp = J->target + ((size_t)b * J->target_rows + j) * (size_t)V;
        const float* zq = J->draft + ((size_t)b * K + j) * (size_t)V;
        int32_t x = J->draft_tok[(size_t)b * K + j];
        float mp = row_max_nan(zp, V), mq = row_max_nan(zq, V);
        int ps = row_status(mp);
        if (ps == ROW_OK) ps = row_status(mq);
        if (ps == ROW_OK && (x < 0 || x >= V)) ps = ROW_BAD_TOKEN;
        if (ps != ROW_OK) { J->status[b] = ps; J->accept_len[b] = j; return; }
        uint64_t Sp = row_total_mass(zp, V, inv_T, mp);
        uint64_t Sq = row_total_mass(zq, V, inv_T, mq);
        uint64_t wp = mass_of((zp[x] - mp) * inv_T);
        uint64_t wq = mass_of((zq[x] - mq) * inv_T);
        double lhs = ((double)J->u_accept[(size_t)b * K + j] * (double)wq) * (double)Sp;
        double rhs = (double)wp * (double)Sq;
        if (lhs < rhs) { out[j] = x; continue; }
        /* reject: resample from max(0, p - q) */
        float invSp = (float)(1099511627776.0 / (double)Sp);
        float invSq = (float)(1099511627776.0 / (double)Sq);
        uint64_t W = 0;
        for (int i = 0; i < V; i++) {
            float pi = born_oracle_exp1((zp[i] - mp) * inv_T) * invSp;
            float qi = born_oracle_exp1((zq[i] - mq) * inv_T) * invSq;
            float r = pi - qi;
            r = r > 0.0f ? r : 0.0f;
            wbuf[i] = (uint64_t)llrintf(r * MASS_SCALE);
            W += wbuf[i];
        }
        if (W == 0) /* degenerate: residual vanished in fp32; draw from p instead */
            for (int i = 0; i < V; i++) wbuf[i] = mass_of((zp[i] - mp) * inv_T);
        out[j] = draw_index(wbuf, V, J->u_resample[(size_t)b * (K + 1) + j]);
        J->accept_len[b] = j;
        return;
    }
    J->accept_len[b] = K;
    if (J->target_rows > K) {
        const float* zp = J->target + ((size_t)b * J->target_rows + K) * (size_t)V;
        float mp = row_max_nan(zp, V);
        if (row_status(mp) != ROW_OK) { J->status[b] = row_status(mp); return; }
        for (int i = 0; i < V; i++) wbuf[i] = mass_of((zp[i] - mp) * inv_T);
        out[K] = draw_index(wbuf, V, J->u_resample[(size_t)b * (K + 1) + K]);
    }
}

typedef struct { const spec_job* J; int lo, hi; int ok; } spec_thread_arg;

static void* spec_thread(void* a) {
    spec_thread_arg* T = (spec_thread_arg*)a;
    uint64_t* wbuf = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)T->J->V);
    T->ok = wbuf != NULL;
    if (wbuf) for (int b = T->lo; b < T->hi; b++) spec_seq(T->J, wbuf, b);
    free(wbuf);
    return NULL;
}

/* Accept/reject K draft tokens per sequence against target logits; fp32 logits,
 * target [B, target_rows, V], draft [B, K, V].  accept iff u * q(x) < p(x). */
int born_oracle_spec_verify(int B, int K, int V, int target_rows, const float* target, const float* draft,
                            const int32_t* draft_tok, const float* u_accept, const float* u_resample,
                            float temperature, int32_t* accept_len, int32_t* out_tok, int32_t* status,
                            int nthreads) {
    spec_job J = { B, K, V, target_rows, target, draft, draft_tok, u_accept, u_resample, temperature,
                   accept_len, out_tok, status };
    if (nthreads < 1) nthreads = 1;
    if (nthreads > B) nthreads = B > 0 ? B : 1;
    spec_thread_arg* args = (spec_thread_arg*)calloc((size_t)nthreads, sizeof(spec_thread_arg));
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nthreads);
    for (int i = 0; i < nthreads; i++) {
        args[i].J = &J;
        args[i].lo = (int)((int64_t)B * i / nthreads);
        args[i].hi = (int)((int64_t)B * (i + 1) / nthreads);
        pthread_create(&th[i], NULL, spec_thread, &args[i]);
    }
    int ok = 1;
    for (int i = 0; i < nthreads; i++) { pthread_join(th[i], NULL); ok &= args[i].ok; }
    free(th); free(args);
    return ok ? 0 : -1;
}

/* Draft-token generator for the speculative-decoding workload: token j of sequence b is
 * drawn from softmax(draft[b, j] * inv_T) with uniform u[b, j] (full distribution,
 * ascending-index inverse CDF over fixed-point masses). */
int born_oracle_draft_tokens(int B, int K, int V, const float* draft, const float* u, float temperature,
                             int32_t* tok) {
    uint64_t* w = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)V);
    if (!w) return -1;
    float inv_T = (temperature == 0.0f) ? 1.0f : 1.0f / temperature;
    for (int r = 0; r < B * K; r++) {
        const float* z = draft + (size_t)r * (size_t)V;
        float m = -INFINITY;
        for (int i = 0; i < V; i++) if (z[i] > m) m = z[i];
        for (int i = 0; i < V; i++) w[i] = mass_of((z[i] - m) * inv_T);
        tok[r] = draw_index(w, V, u[r]);
    }
    free(w);
    return 0;
}

int born_oracle_version(void) { return BORN_ORACLE_VERSION; }
