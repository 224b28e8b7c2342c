// scan_kernel for fp32 launches with a token history (patched by the producer warp); any grid and mode.
#include <cstdint>
#define SCAN_INST_T float
#define SCAN_INST_PAIR false
#define SCAN_INST_ONEROW false
#define SCAN_INST_ATTRS scan_attrs_f32_hist
#define SCAN_INST_LAUNCH scan_launch_f32_hist
#include "scan_inst.cuh"
