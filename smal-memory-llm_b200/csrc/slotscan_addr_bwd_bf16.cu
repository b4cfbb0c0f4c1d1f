#define SLOTSCAN_TIN __nv_bfloat16
#define SLOTSCAN_SUFFIX bf16
#define SLOTSCAN_DEFINE_NEXT_WRITE   // the dtype-independent next-write launcher lives in this translation unit
#include "slotscan_addr_bwd_inst.cuh"
