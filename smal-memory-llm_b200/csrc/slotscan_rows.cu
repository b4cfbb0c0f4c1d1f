// Forward row replay (slotscan_rows.cuh) instantiated for every row width and dtype pair.
#include <stdio.h>

#include "slotscan_launch.h"
#include "slotscan_rows.cuh"

namespace slotscan {

template <int D, typename Tin, typename Tsn>
static cudaError_t replay_one(const slotscan_params& p, const void* x, const float* gate, const int* am, const int* tfirst,
                              const float* x0, void* xbuf, float* xold, float* xfin, float* kinv, uint8_t* valid,
                              cudaStream_t st) {
    constexpr int RPB = ROW_THREADS / (D / 8);
    dim3 grid(p.B * p.H, (p.N + RPB - 1) / RPB);
    if (kinv != nullptr)
        replay_rows_kernel<D, Tin, Tsn, true><<<grid, ROW_THREADS, 0, st>>>(p, (const Tin*)x, gate, am, tfirst, x0, (Tsn*)xbuf,
                                                                            xold, xfin, kinv, valid);
    else
        replay_rows_kernel<D, Tin, Tsn, false><<<grid, ROW_THREADS, 0, st>>>(p, (const Tin*)x, gate, am, tfirst, x0, (Tsn*)xbuf,
                                                                             xold, xfin, nullptr, nullptr);
    return cudaGetLastError();
}

#define ROWS_TYPES(CALL_F32_F32, CALL_F32_BF16, CALL_BF16_F32, CALL_BF16_BF16)            \
    if (p.in_dtype == SLOTSCAN_F32) {                                                     \
        if (p.snap_dtype == SLOTSCAN_F32) { CALL_F32_F32; } else { CALL_F32_BF16; }       \
    } else {                                                                              \
        if (p.snap_dtype == SLOTSCAN_F32) { CALL_BF16_F32; } else { CALL_BF16_BF16; }     \
    }

template <int D>
static cudaError_t replay_d(const slotscan_params& p, const void* x, const float* gate, const int* am, const int* tfirst,
                            const float* x0, void* xbuf, float* xold, float* xfin, float* kinv, uint8_t* valid,
                            cudaStream_t st) {
    typedef __nv_bfloat16 bf;
    ROWS_TYPES(return (replay_one<D, float, float>(p, x, gate, am, tfirst, x0, xbuf, xold, xfin, kinv, valid, st)),
               return (replay_one<D, float, bf>(p, x, gate, am, tfirst, x0, xbuf, xold, xfin, kinv, valid, st)),
               return (replay_one<D, bf, float>(p, x, gate, am, tfirst, x0, xbuf, xold, xfin, kinv, valid, st)),
               return (replay_one<D, bf, bf>(p, x, gate, am, tfirst, x0, xbuf, xold, xfin, kinv, valid, st)))
}

cudaError_t run_replay(const slotscan_params& p, int D, const void* x, const float* gate, const int* am, const int* tfirst,
                       const float* x0, void* xbuf, float* xold, float* xfin, float* kinv, uint8_t* valid, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    SLOTSCAN_DISPATCH_D(D, e = (replay_d<DD>(p, x, gate, am, tfirst, x0, xbuf, xold, xfin, kinv, valid, st)));
    return e;
}

void attrs_rows(slotscan_kernel_attr* out, int cap, int& n) {
    fill_attr(out, cap, n, "replay_rows<128,bf16,bf16>", replay_rows_kernel<128, __nv_bfloat16, __nv_bfloat16, false>);
    fill_attr(out, cap, n, "replay_rows<128,bf16,bf16,kinv>", replay_rows_kernel<128, __nv_bfloat16, __nv_bfloat16, true>);
    fill_attr(out, cap, n, "replay_rows<128,f32,f32>", replay_rows_kernel<128, float, float, false>);
}

}  // namespace slotscan
