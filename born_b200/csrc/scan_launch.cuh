// Host-side entry points of the streaming kernel's instantiations.  The kernel is instantiated
// in nine translation units that compile side by side -- fp32 launches without a token history
// (scan_f32_pair*.cu) and with one (scan_f32_hist*.cu), bf16 launches without (scan_bf16_pair*.cu)
// and with one (scan_bf16*.cu), each once for any grid and mode and once (*_row.cu) for sampling launches whose grid gives
// every CTA exactly one whole row (for fp32 with a history: once more for histories of at most
// kHistShort ids per row, scan_f32_hist_short_row.cu) -- each for mask x log-sum-exp and, without a mask and with
// the log-sum-exp, per route class (RouteOf in scan_common.cuh).  capi.cu only calls these.
#pragma once
#include <cuda_runtime.h>
#include "scan_common.cuh"

namespace born {

// SCAN_UNIT(name) declares, for one translation unit,
//   scan_attrs_<name>():  raise the dynamic shared-memory limit of its instantiations (once per device)
//   scan_launch_<name>(): launch the instantiation for (mask, lse, route class); returns cudaGetLastError()
#define SCAN_UNIT(name)              \
    cudaError_t scan_attrs_##name(); \
    cudaError_t scan_launch_##name(const ScanArgs& A, bool mask, bool lse, int route, int grid, size_t smem, cudaStream_t st);
SCAN_UNIT(f32_pair)
SCAN_UNIT(f32_pair_row)
SCAN_UNIT(f32_hist)
SCAN_UNIT(f32_hist_row)
SCAN_UNIT(f32_hist_short_row)
SCAN_UNIT(bf16_pair)
SCAN_UNIT(bf16_pair_row)
SCAN_UNIT(bf16)
SCAN_UNIT(bf16_row)
#undef SCAN_UNIT

}  // namespace born
