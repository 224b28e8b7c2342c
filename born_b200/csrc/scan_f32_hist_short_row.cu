// scan_kernel for fp32 launches with a token history of at most kHistShort ids per row (five stages
// without a mask); one whole row per CTA, sampling mode.
#include <cstdint>
#define SCAN_INST_T float
#define SCAN_INST_PAIR false
#define SCAN_INST_ONEROW true
#define SCAN_INST_SHORT true
#define SCAN_INST_ATTRS scan_attrs_f32_hist_short_row
#define SCAN_INST_LAUNCH scan_launch_f32_hist_short_row
#include "scan_inst.cuh"
