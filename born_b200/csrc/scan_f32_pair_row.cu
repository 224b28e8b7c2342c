// scan_kernel for fp32 launches without a token history (paired tiles, no history code); one whole row per CTA, sampling mode.
#include <cstdint>
#define SCAN_INST_T float
#define SCAN_INST_PAIR true
#define SCAN_INST_ONEROW true
#define SCAN_INST_ATTRS scan_attrs_f32_pair_row
#define SCAN_INST_LAUNCH scan_launch_f32_pair_row
#include "scan_inst.cuh"
