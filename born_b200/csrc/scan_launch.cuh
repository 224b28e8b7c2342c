// Host-side entry points of the streaming kernel's instantiations.  The kernel is instantiated
// in three translation units that compile side by side -- fp32 launches without a token history
// (scan_f32_pair.cu), fp32 launches with one (scan_f32_hist.cu), bf16 launches (scan_bf16.cu) --
// each for mask x log-sum-exp and, without a mask and with the log-sum-exp, per route class
// (RouteOf in scan_common.cuh).  capi.cu only calls these.
#pragma once
#include <cuda_runtime.h>
#include "scan_common.cuh"

namespace born {

// raise the dynamic shared-memory limit of every instantiation of the unit (once per device)
cudaError_t scan_attrs_f32_pair();
cudaError_t scan_attrs_f32_hist();
cudaError_t scan_attrs_bf16();

// launch the instantiation for (mask, lse, route class); returns cudaGetLastError()
cudaError_t scan_launch_f32_pair(const ScanArgs& A, bool mask, bool lse, int route, int grid, size_t smem, cudaStream_t st);
cudaError_t scan_launch_f32_hist(const ScanArgs& A, bool mask, bool lse, int route, int grid, size_t smem, cudaStream_t st);
cudaError_t scan_launch_bf16(const ScanArgs& A, bool mask, bool lse, int route, int grid, size_t smem, cudaStream_t st);

}  // namespace born
