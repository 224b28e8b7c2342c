// Arithmetic and block-level primitives shared by every kernel of libborn_sampler.so.
//
// Everything that feeds a *decision* (which tokens are kept, which token is drawn) is
// integer arithmetic on fixed-point masses, or a fixed sequence of individually rounded
// fp32 operations, so that results do not depend on the order in which threads run and
// can be restated bit-for-bit on a CPU.  The row arithmetic keeps the reference's
// structure (born: internal/autodiff/ops/softmax.go:214-238 -- subtract the row maximum,
// exponentiate, sum) but never materialises the softmax.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace born {

constexpr int kThreads = 256;        // threads per CTA in the row kernels
constexpr int kTileBytes = 16384;    // bytes of logits per pipeline stage (4096 fp32 / 8192 bf16)
constexpr int kStages = 5;           // bulk-copy stages in flight per CTA
constexpr int kMaxK = 1024;          // BORN_MAX_TOP_K / BORN_MAX_CANDIDATES
constexpr int kCandCap = 2048;       // candidate buffer entries (>= kMaxK + one half piece)
constexpr int kHistCap = 1024;       // history ids held per CTA
constexpr uint32_t kIdxMask = 0xFFFFFFu;
constexpr int kRecordHdrBytes = 32;

// ---- bit casts / keys -------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// Order-preserving map float -> uint32 (larger float => larger key); -0 is folded onto +0
// so that equal values have equal keys.  No float maps to key 0.
__device__ __forceinline__ uint32_t zkey(float z) {
    uint32_t b = __float_as_uint(z);
    if (b == 0x80000000u) b = 0u;
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}
__device__ __forceinline__ float zkey_to_float(uint32_t k) {
    uint32_t b = (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
    return __uint_as_float(b);
}
// 56-bit composite rank key: larger = ranks earlier (value descending, index ascending).
__device__ __forceinline__ uint64_t make_ck(float z, int idx) {
    return ((uint64_t)zkey(z) << 24) | (uint64_t)(kIdxMask - (uint32_t)idx);
}
__device__ __forceinline__ int ck_idx(uint64_t ck) { return (int)(kIdxMask - (uint32_t)(ck & kIdxMask)); }
__device__ __forceinline__ float ck_z(uint64_t ck) { return zkey_to_float((uint32_t)(ck >> 24)); }
__device__ __forceinline__ bool ck_alive(uint64_t ck) { return (ck >> 24) != 0; }

// ---- deterministic exp and fixed-point mass --------------------------------------------
// Same operation sequence as the CPU oracle: Cody-Waite reduction, degree-6 polynomial,
// exponent-field scaling.  x <= 0; returns 0 below -80 and for NaN.
// kSelect: no branch -- an argument below -80, or NaN, runs the arithmetic on -80 and selects 0 at the
// end; otherwise those arguments return early.  Same bits either way; which one is faster depends
// on the caller (measured: the select form takes 3 % off the whole-vocabulary rows of the streaming
// kernel and adds 2 % to the verify kernels, which therefore ask for the branch).
template <bool kSelect = true>
__device__ __forceinline__ float exp_det(float x) {
    const bool in_range = x >= -80.0f;
    if constexpr (kSelect) x = in_range ? x : -80.0f;
    else if (!in_range) return 0.0f;
    const float magic = 12582912.0f;
    float t = __fmul_rn(x, 0x1.715476p+0f);
    float r = __fadd_rn(t, magic);
    float nf = __fsub_rn(r, magic);
    float f = __fmaf_rn(nf, -0x1.62e4p-1f, x);
    f = __fmaf_rn(nf, -0x1.7f7d1cp-20f, f);
    float p = 0x1.687bf6p-10f;
    p = __fmaf_rn(p, f, 0x1.123b9ep-7f);
    p = __fmaf_rn(p, f, 0x1.555b58p-5f);
    p = __fmaf_rn(p, f, 0x1.55548ep-3f);
    p = __fmaf_rn(p, f, 0x1.fffff8p-2f);
    p = __fmaf_rn(p, f, 1.0f);
    p = __fmaf_rn(p, f, 1.0f);
    uint32_t n = __float_as_uint(r) - 0x4B400000u;
    const float e = __uint_as_float(__float_as_uint(p) + (n << 23));
    return (kSelect && !in_range) ? 0.0f : e;
}
// q = rne_u64(exp_det(x) * 2^40)
template <bool kSelect = true>
__device__ __forceinline__ uint64_t mass_of(float x) {
    return __float2ull_rn(__fmul_rn(exp_det<kSelect>(x), 1099511627776.0f));
}
// x = (z - m) * inv_T with two roundings
__device__ __forceinline__ float scaled_shift(float z, float m, float inv_T) {
    return __fmul_rn(__fsub_rn(z, m), inv_T);
}

__device__ __forceinline__ float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// ---- mbarrier + 1-D bulk copy (TMA) -----------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory atomics with the address space spelled out.  The pointers in this library
// travel through structs, where the compiler can no longer prove that they point to shared
// memory and would fall back to generic-address atomics.
__device__ __forceinline__ uint32_t smem_atom_add(void* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(p)), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void smem_red_add(void* p, uint32_t v) {
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void smem_red_max(void* p, uint32_t v) {
    asm volatile("red.shared.max.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void smem_red_min(void* p, uint32_t v) {
    asm volatile("red.shared.min.u32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Non-multicast bulk copy global -> this CTA's shared memory; both addresses 16-byte
// aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Bounded wait: gives up after about two seconds of wall-clock time (or kMbarSpinLimit
// probes, whichever comes first) and reports false; the caller records the failure and
// leaves the kernel in an orderly way.
constexpr uint32_t kMbarSpinLimit = 1u << 26;
constexpr unsigned long long kMbarTimeoutNs = 2000000000ull;
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < kMbarSpinLimit; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((it & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kMbarTimeoutNs) return false;
        }
    }
    return false;
}

// ---- barriers of the 256 compute threads ----------------------------------------------------
// The row kernels run 256 compute threads plus, in the streaming kernel, one producer warp
// that only issues bulk copies.  Everything the compute threads synchronise on uses named
// barrier 1 with a count of 256, so the producer warp never takes part.
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ int cta_sync_or(int pred) {
    int r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.s32 p, %1, 0;\n\t"
        "bar.red.or.pred q, 1, 256, p;\n\t"
        "selp.s32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(pred)
        : "memory");
    return r;
}
__device__ __forceinline__ int cta_sync_count(int pred) {
    int r;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.s32 p, %1, 0;\n\t"
        "bar.red.popc.u32 %0, 1, 256, p;\n\t}"
        : "=r"(r)
        : "r"(pred)
        : "memory");
    return r;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait that also gives up when *abort becomes non-zero (set by the compute threads
// when they leave early).
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, uint32_t parity, const volatile int* abort) {
    const uint32_t addr = smem_u32(bar);
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < kMbarSpinLimit; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return true;
        if (*abort) return false;
        if ((it & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kMbarTimeoutNs) return false;
        }
    }
    return false;
}

// Bounded wait that returns 1 when the phase completed, 2 as soon as *event is non-zero
// (checked between probes by the whole warp, so the answer is warp-uniform), 0 on a timeout.
__device__ __forceinline__ int mbar_wait_or_event(uint64_t* bar, uint32_t parity, const volatile int* event) {
    const uint32_t addr = smem_u32(bar);
    {   // the tile is usually there already: one probe, no votes
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (ok) return 1;
    }
    unsigned long long t0 = 0;
    for (uint32_t it = 0; it < kMbarSpinLimit; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(addr), "r"(parity)
            : "memory");
        if (__all_sync(0xffffffffu, ok != 0)) return 1;
        if (__any_sync(0xffffffffu, *event != 0)) return 2;
        if ((it & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (__any_sync(0xffffffffu, now - t0 > kMbarTimeoutNs)) return 0;
        }
    }
    return 0;
}

// ---- warp helpers ------------------------------------------------------------------------
__device__ __forceinline__ uint64_t shfl_u64(uint64_t v, int src) {
    uint32_t lo = __shfl_sync(0xffffffffu, (uint32_t)v, src);
    uint32_t hi = __shfl_sync(0xffffffffu, (uint32_t)(v >> 32), src);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ uint64_t shfl_up_u64(uint64_t v, int d) {
    uint32_t lo = __shfl_up_sync(0xffffffffu, (uint32_t)v, d);
    uint32_t hi = __shfl_up_sync(0xffffffffu, (uint32_t)(v >> 32), d);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ uint64_t shfl_xor_u64(uint64_t v, int m) {
    uint32_t lo = __shfl_xor_sync(0xffffffffu, (uint32_t)v, m);
    uint32_t hi = __shfl_xor_sync(0xffffffffu, (uint32_t)(v >> 32), m);
    return ((uint64_t)hi << 32) | lo;
}

// Scratch for the radix searches: 256 count bins and 256 weight bins (weights are split
// into two 20-bit halves so that plain 32-bit shared-memory atomics accumulate them exactly).
struct SearchScratch {
    uint32_t c[256];
    uint32_t wlo[256];
    uint32_t whi[256];
    uint32_t red_and[2 * (kThreads / 32)];
    uint32_t red_or[2 * (kThreads / 32)];
    uint32_t digit;
    uint32_t bin_count;
    unsigned long long before;  // weight ahead of the chosen bin in walk order
    unsigned long long found;
};

// Block-wide radix descent over n <= 4095 entries with unique integer keys of at most
// `kBits` bits.  Walking the entries in key order (descending when kDesc, else ascending)
// it returns the key of the entry at which the running weight first exceeds `target`
// (cum_before <= target < cum_before + weight); the caller guarantees target < total
// weight.  With kUnit every entry weighs 1 (rank selection: target = k - 1 finds the k-th
// entry); otherwise weights are fixed-point masses <= 2^40.  Weights are integers, so the
// bin sums accumulated with shared-memory atomics do not depend on thread order.
// The descent starts at the highest bit in which the keys differ, takes 8 bits per pass
// (256 shared-memory bins, the crossing bin located by a warp scan and ballot) and stops
// as soon as the crossing bin holds a single entry.  All kThreads threads must call.
template <bool kDesc, int kBits, bool kUnit, typename KeyFn, typename WeightFn>
__device__ uint64_t block_radix_search(int n, unsigned long long target, KeyFn key_of, WeightFn weight_of,
                                       SearchScratch& sc) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // bits in which the keys differ
    uint64_t k_and = ~0ull, k_or = 0ull;
    for (int i = tid; i < n; i += kThreads) {
        uint64_t k = key_of(i);
        k_and &= k;
        k_or |= k;
    }
    uint32_t a_lo = __reduce_and_sync(0xffffffffu, (uint32_t)k_and), a_hi = __reduce_and_sync(0xffffffffu, (uint32_t)(k_and >> 32));
    uint32_t o_lo = __reduce_or_sync(0xffffffffu, (uint32_t)k_or), o_hi = __reduce_or_sync(0xffffffffu, (uint32_t)(k_or >> 32));
    sc.c[tid] = 0;
    if (!kUnit) { sc.wlo[tid] = 0; sc.whi[tid] = 0; }
    if (lane == 0) {
        sc.red_and[2 * warp] = a_lo; sc.red_and[2 * warp + 1] = a_hi;
        sc.red_or[2 * warp] = o_lo; sc.red_or[2 * warp + 1] = o_hi;
    }
    cta_sync();
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) {
        a_lo &= sc.red_and[2 * w]; a_hi &= sc.red_and[2 * w + 1];
        o_lo |= sc.red_or[2 * w]; o_hi |= sc.red_or[2 * w + 1];
    }
    const uint64_t all_and = ((uint64_t)a_hi << 32) | a_lo, all_or = ((uint64_t)o_hi << 32) | o_lo;
    const uint64_t varying = all_and ^ all_or;
    if (varying == 0) return all_or;  // a single entry
    int shift = 63 - __clzll((long long)varying) - 7;
    if (shift < 0) shift = 0;
    uint64_t pmask = (shift + 8 >= 64) ? 0ull : (~0ull << (shift + 8));
    uint64_t prefix = all_or & pmask;
    for (;;) {
        for (int i = tid; i < n; i += kThreads) {
            uint64_t k = key_of(i);
            if ((k & pmask) == prefix) {
                uint32_t d = (uint32_t)(k >> shift) & 255u;
                smem_red_add(&sc.c[d], 1u);
                if (!kUnit) {
                    unsigned long long wt = weight_of(i);
                    if (wt) {
                        smem_red_add(&sc.wlo[d], (uint32_t)(wt & 0xFFFFFu));
                        smem_red_add(&sc.whi[d], (uint32_t)(wt >> 20));
                    }
                }
            }
        }
        cta_sync();
        if (tid < 32) {
            // lane l walks 8 bins; walk position o = 8*l + j maps to bin (kDesc ? 255 - o : o)
            unsigned long long loc[8];
            unsigned long long lane_sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int o = 8 * tid + j;
                int b = kDesc ? 255 - o : o;
                loc[j] = kUnit ? (unsigned long long)sc.c[b] : (((unsigned long long)sc.whi[b] << 20) + sc.wlo[b]);
                lane_sum += loc[j];
            }
            unsigned long long incl = lane_sum;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                unsigned long long up = shfl_up_u64(incl, d);
                if (tid >= d) incl += up;
            }
            unsigned long long excl = incl - lane_sum;
            uint32_t hit = __ballot_sync(0xffffffffu, incl > target);
            int hl = hit ? (__ffs(hit) - 1) : 31;
            if (tid == hl) {
                unsigned long long acc = excl;
                int jj = 7;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (acc + loc[j] > target) { jj = j; break; }
                    acc += loc[j];
                }
                int o = 8 * tid + jj;
                int b = kDesc ? 255 - o : o;
                sc.digit = (uint32_t)b;
                sc.before = acc;
                sc.bin_count = sc.c[b];
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {  // leave the bins clean for the next pass
                int b = 8 * tid + j;
                sc.c[b] = 0;
                if (!kUnit) { sc.wlo[b] = 0; sc.whi[b] = 0; }
            }
        }
        cta_sync();
        target -= sc.before;
        prefix |= (uint64_t)sc.digit << shift;
        pmask |= (uint64_t)255u << shift;
        if (shift == 0) return prefix;
        if (sc.bin_count == 1u) {
            for (int i = tid; i < n; i += kThreads) {
                uint64_t k = key_of(i);
                if ((k & pmask) == prefix) sc.found = k;
            }
            cta_sync();
            uint64_t r = sc.found;
            cta_sync();
            return r;
        }
        shift = shift >= 8 ? shift - 8 : 0;
    }
}

// Block-wide sum of per-thread u64 values; `buf` holds 8 words.  All threads get the sum.
__device__ __forceinline__ uint64_t block_sum_u64(uint64_t v, unsigned long long* buf) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += shfl_xor_u64(v, d);
    cta_sync();
    if ((threadIdx.x & 31) == 0) buf[threadIdx.x >> 5] = v;
    cta_sync();
    uint64_t s = 0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += buf[w];
    return s;
}

}  // namespace born
