// scan_kernel for bf16 launches with a token history (applied by the compute warps); one whole row per CTA, sampling mode.
#include <cstdint>
#define SCAN_INST_T uint16_t
#define SCAN_INST_PAIR false
#define SCAN_INST_ONEROW true
#define SCAN_INST_ATTRS scan_attrs_bf16_row
#define SCAN_INST_LAUNCH scan_launch_bf16_row
#include "scan_inst.cuh"
