// Reverse row scan, float32 token streams.
#define SLOTSCAN_TIN float
#define SLOTSCAN_SUFFIX f32
#include "slotscan_rows_bwd_inst.cuh"
