// scan_kernel for bf16 launches with a token history (applied by the compute warps); any grid and mode.
#include <cstdint>
#define SCAN_INST_T uint16_t
#define SCAN_INST_PAIR false
#define SCAN_INST_ONEROW false
#define SCAN_INST_ATTRS scan_attrs_bf16
#define SCAN_INST_LAUNCH scan_launch_bf16
#include "scan_inst.cuh"
