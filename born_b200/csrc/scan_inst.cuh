// Body of a translation unit that instantiates scan_kernel for one (element type, history form):
// included by the scan_*.cu units after they have defined
//   SCAN_INST_T      the element type (float or uint16_t)
//   SCAN_INST_PAIR   true: launches without a token history (fp32: paired tiles); false: with one
//   SCAN_INST_ONEROW true: sampling launches whose grid gives every CTA one whole row
//   SCAN_INST_SHORT  (optional) true: histories of at most kHistShort ids per row
//   SCAN_INST_ATTRS  / SCAN_INST_LAUNCH   the names of the two functions of scan_launch.cuh
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../../include/born_sampler.h"
#include "scan_kernel.cuh"
#include "fallback.cuh"
#include "scan_launch.cuh"

#ifndef SCAN_INST_SHORT
#define SCAN_INST_SHORT false
#endif

namespace born {
namespace {

template <bool M, bool Lse, int R>
cudaError_t attr_one() {
    return cudaFuncSetAttribute(scan_kernel<SCAN_INST_T, M, Lse, SCAN_INST_PAIR, R, SCAN_INST_ONEROW, SCAN_INST_SHORT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                scan_smem_layout((int)sizeof(SCAN_INST_T), M, !SCAN_INST_PAIR, SCAN_INST_SHORT ? kHistShort : (int)BORN_MAX_HISTORY).total);
}
// (the route classes 1 and 2 exist for launches without a mask that want the log-sum-exp -- the
// serving configurations; the others take the general instantiation: every instantiation costs
// a third of a minute of compile time)
template <bool M, bool Lse>
cudaError_t attr_all_routes() {
    cudaError_t e;
    if ((e = attr_one<M, Lse, 0>()) != cudaSuccess) return e;
    if constexpr (!M && Lse) {
        if ((e = attr_one<M, Lse, 1>()) != cudaSuccess) return e;
        if ((e = attr_one<M, Lse, 2>()) != cudaSuccess) return e;
    }
    return cudaSuccess;
}
template <bool M, bool Lse>
cudaError_t launch_route(const ScanArgs& A, int route, int grid, size_t smem, cudaStream_t st) {
    if constexpr (!M && Lse) {
        if (route == 1) { scan_kernel<SCAN_INST_T, M, Lse, SCAN_INST_PAIR, 1, SCAN_INST_ONEROW, SCAN_INST_SHORT><<<grid, kScanThreads, smem, st>>>(A); return cudaGetLastError(); }
        if (route == 2) { scan_kernel<SCAN_INST_T, M, Lse, SCAN_INST_PAIR, 2, SCAN_INST_ONEROW, SCAN_INST_SHORT><<<grid, kScanThreads, smem, st>>>(A); return cudaGetLastError(); }
    }
    scan_kernel<SCAN_INST_T, M, Lse, SCAN_INST_PAIR, 0, SCAN_INST_ONEROW, SCAN_INST_SHORT><<<grid, kScanThreads, smem, st>>>(A);
    return cudaGetLastError();
}

}  // namespace

cudaError_t SCAN_INST_ATTRS() {
    cudaError_t e;
    if ((e = attr_all_routes<false, false>()) != cudaSuccess) return e;
    if ((e = attr_all_routes<false, true>()) != cudaSuccess) return e;
    if ((e = attr_all_routes<true, false>()) != cudaSuccess) return e;
    return attr_all_routes<true, true>();
}

cudaError_t SCAN_INST_LAUNCH(const ScanArgs& A, bool mask, bool lse, int route, int grid, size_t smem, cudaStream_t st) {
    if (mask) return lse ? launch_route<true, true>(A, route, grid, smem, st) : launch_route<true, false>(A, route, grid, smem, st);
    return lse ? launch_route<false, true>(A, route, grid, smem, st) : launch_route<false, false>(A, route, grid, smem, st);
}

}  // namespace born
