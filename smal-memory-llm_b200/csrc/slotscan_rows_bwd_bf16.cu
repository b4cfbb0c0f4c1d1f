// Reverse row scan, bfloat16 token streams.
#define SLOTSCAN_TIN __nv_bfloat16
#define SLOTSCAN_SUFFIX bf16
#include "slotscan_rows_bwd_inst.cuh"
