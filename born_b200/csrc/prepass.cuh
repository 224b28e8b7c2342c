// Clean-copy prepass.  The whole-vocabulary routes of scan_kernel form their mass blocks on
// 512-token blocks aligned to the row start, inside the warps' fixed tile slices.  Rows that
// do not start on a 16-byte boundary, and bf16 rows with history penalties (a bf16 tile cannot
// hold a penalised fp32 value), are therefore first written to a 16-byte-aligned fp32 copy with
// the grammar mask and the penalties already applied -- the same operations in the same order
// as everywhere else: upcast, repetition (z > 0 ? z / r : z * r), z - (frequency * count +
// presence), then -inf where the mask bit is clear.
#pragma once
#include "scan_common.cuh"

namespace born {

struct CopyArgs {
    const void* logits;   // [B, row_stride]
    float* out;           // [B, out_stride]
    const uint32_t* mask;
    const int32_t* history;
    const int32_t* history_len;
    const born_row_params* row_params;
    born_row_params params;
    int64_t row_stride, out_stride, mask_stride;
    int B, V, history_stride;
};

template <typename T>
__device__ __forceinline__ float load_logit(const T* p) {
    if constexpr (sizeof(T) == 4) return __ldg(reinterpret_cast<const float*>(p));
    else return bf16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t*>(p)));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) clean_copy_kernel(const CopyArgs A) {
    const int b = blockIdx.y;
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)b * A.row_stride;
    float* out = A.out + (int64_t)b * A.out_stride;
    const uint32_t* mrow = A.mask ? A.mask + (int64_t)b * A.mask_stride : nullptr;
    for (int e = blockIdx.x * kThreads + threadIdx.x; e < A.V; e += gridDim.x * kThreads) {
        float z = load_logit<T>(row + e);
        if (mrow && !((__ldg(mrow + (e >> 5)) >> (e & 31)) & 1u)) z = -INFINITY;
        out[e] = z;
    }
}

// One CTA per row: the penalties of the distinct history tokens (multiplicities by all pairs).
template <typename T>
__global__ void __launch_bounds__(kThreads) clean_patch_kernel(const CopyArgs A) {
    __shared__ int32_t ids[BORN_MAX_HISTORY];
    const int tid = threadIdx.x, b = blockIdx.x;
    const born_row_params rp = A.row_params ? A.row_params[b] : A.params;
    if (!penalties_on(rp)) return;
    int len = A.history_len ? A.history_len[b] : A.history_stride;
    len = max(0, min(min(len, A.history_stride), (int)BORN_MAX_HISTORY));
    const int32_t* h = A.history + (int64_t)b * A.history_stride;
    for (int i = tid; i < len; i += kThreads) ids[i] = h[i];
    __syncthreads();
    const T* row = reinterpret_cast<const T*>(A.logits) + (int64_t)b * A.row_stride;
    float* out = A.out + (int64_t)b * A.out_stride;
    const uint32_t* mrow = A.mask ? A.mask + (int64_t)b * A.mask_stride : nullptr;
    for (int i = tid; i < len; i += kThreads) {
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
        float z = penalise(rp, load_logit<T>(row + id), cnt);
        if (mrow && !((__ldg(mrow + (id >> 5)) >> (id & 31)) & 1u)) z = -INFINITY;
        out[id] = z;
    }
}

// returns 0 or a cudaError_t; `launches` counts what was launched
inline int launch_clean_copy(const CopyArgs& A, int dtype, int num_sms, cudaStream_t st, int* launches) {
    int parts = (8 * num_sms + A.B - 1) / A.B;
    const int maxp = (A.V + kThreads * 4 - 1) / (kThreads * 4);
    if (parts > maxp) parts = maxp;
    if (parts < 1) parts = 1;
    const dim3 g((unsigned)parts, (unsigned)A.B, 1);
    if (dtype == BORN_DTYPE_F32) clean_copy_kernel<float><<<g, kThreads, 0, st>>>(A);
    else clean_copy_kernel<uint16_t><<<g, kThreads, 0, st>>>(A);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    *launches += 1;
    if (A.history) {
        if (dtype == BORN_DTYPE_F32) clean_patch_kernel<float><<<A.B, kThreads, 0, st>>>(A);
        else clean_patch_kernel<uint16_t><<<A.B, kThreads, 0, st>>>(A);
        *launches += 1;
    }
    return (int)cudaGetLastError();
}

}  // namespace born
