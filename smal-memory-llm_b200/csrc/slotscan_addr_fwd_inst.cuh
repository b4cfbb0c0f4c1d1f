// Instantiation body of the forward address scan for one input dtype: included by slotscan_addr_fwd_{f32,bf16}.cu
// with SLOTSCAN_TIN and SLOTSCAN_SUFFIX defined.
#include <stdio.h>

#include "slotscan_addr_fwd.cuh"
#include "slotscan_launch.h"

namespace slotscan {

#define SS_CAT_(a, b) a##b
#define SS_CAT(a, b) SS_CAT_(a, b)
typedef SLOTSCAN_TIN Tin;

template <int DK, int RPL>
static cudaError_t launch_one(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                              const float* temp, const slotscan_log& L, const AddrFwdState& S0, int ncap, int second,
                              cudaStream_t st) {
    const size_t sm = sizeof(float) * (size_t)addr_fwd_layout(ncap, DK, RPL, (int)sizeof(Tin)).total;
    cudaError_t e = cudaSuccess;
#define AF_LAUNCH(OCCB_, CARRY_)                                                                                          \
    {                                                                                                                     \
        auto kern = addr_fwd_direct_kernel<DK, RPL, OCCB_, CARRY_, Tin>;                                                  \
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;                                                         \
        kern<<<p.B * p.H, AF_THREADS, sm, st>>>(p, (const Tin*)q, (const Tin*)k, gate, fr, temp, L.addr, L.oold, L.kiold, \
                                                L.ofin, L.tfirst, S0.K0, S0.o0, S0.nsq0, S0.nsqfin, ncap, second);        \
    }
    const bool carry = S0.K0 != nullptr;
    if (p.occ_bin) { if (carry) AF_LAUNCH(true, true) else AF_LAUNCH(true, false) }
    else { if (carry) AF_LAUNCH(false, true) else AF_LAUNCH(false, false) }
#undef AF_LAUNCH
    return cudaGetLastError();
}

template <int DK>
static cudaError_t launch_dk(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                             const float* temp, const slotscan_log& L, const AddrFwdState& S0, cudaStream_t st) {
    if (p.N <= AF_NCAP1) return launch_one<DK, 2>(p, q, k, gate, fr, temp, L, S0, p.N, 0, st);
    cudaError_t e = launch_one<DK, 2>(p, q, k, gate, fr, temp, L, S0, AF_NCAP1, 0, st);
    if (e != cudaSuccess) return e;
    return launch_one<DK, 6>(p, q, k, gate, fr, temp, L, S0, p.N, 1, st);       // N <= 192
}

cudaError_t SS_CAT(run_addr_fwd_, SLOTSCAN_SUFFIX)(const slotscan_params& p, const void* q, const void* k, const float* gate,
                                                  const float* fr, const float* temp, const slotscan_log& L,
                                                  const AddrFwdState& S0, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    SLOTSCAN_DISPATCH_D(p.DK, e = (launch_dk<DD>(p, q, k, gate, fr, temp, L, S0, st)));
    return e;
}

void SS_CAT(attrs_addr_fwd_, SLOTSCAN_SUFFIX)(slotscan_kernel_attr* out, int cap, int& n) {
    fill_attr(out, cap, n, "addr_fwd<128,rows<=64>", addr_fwd_direct_kernel<128, 2, true, false, Tin>);
    fill_attr(out, cap, n, "addr_fwd<128,rows<=192>", addr_fwd_direct_kernel<128, 6, true, false, Tin>);
}

}  // namespace slotscan

