#define SLOTSCAN_TIN __nv_bfloat16
#define SLOTSCAN_SUFFIX bf16
#include "slotscan_addr_bwd_inst.cuh"
