#define SLOTSCAN_TIN float
#define SLOTSCAN_SUFFIX f32
#include "slotscan_addr_bwd_inst.cuh"

namespace slotscan {
size_t addr_bwd_smem_bytes(int ncap, int DK) { return sizeof(float) * (size_t)addr_bwd_layout(ncap, DK).total; }
}  // namespace slotscan
