// scan_kernel for bf16 launches without a token history (no history code); any grid and mode.
#include <cstdint>
#define SCAN_INST_T uint16_t
#define SCAN_INST_PAIR true
#define SCAN_INST_ONEROW false
#define SCAN_INST_ATTRS scan_attrs_bf16_pair
#define SCAN_INST_LAUNCH scan_launch_bf16_pair
#include "scan_inst.cuh"
