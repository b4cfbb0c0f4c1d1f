#define SLOTSCAN_TIN float
#define SLOTSCAN_SUFFIX f32
#include "slotscan_addr_fwd_inst.cuh"

namespace slotscan {
size_t addr_fwd_smem_bytes(int ncap, int DK, int in_bytes) {
    return sizeof(float) * (size_t)addr_fwd_layout(ncap, DK, ncap <= 64 ? 2 : 6, in_bytes).total;
}
}  // namespace slotscan
