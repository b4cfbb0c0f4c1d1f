// Instantiation body of the reverse row scan for one input dtype: included by slotscan_rows_bwd_{f32,bf16}.cu with
// SLOTSCAN_TIN and SLOTSCAN_SUFFIX defined.
#include <stdio.h>

#include "slotscan_launch.h"
#include "slotscan_rows_bwd.cuh"

namespace slotscan {

#define SS_CAT_(a, b) a##b
#define SS_CAT(a, b) SS_CAT_(a, b)
typedef SLOTSCAN_TIN Tin;

template <int D, typename Tsn>
static cudaError_t rows_bwd_one(const slotscan_params& p, int ntensors, const RowsBwdPtrs& a0, const RowsBwdPtrs& a1,
                                const float* gate, const int* am, const int* tfirst, cudaStream_t st) {
    constexpr int RPB = ROW_THREADS / (D / 8);
    // block index = (tile * B*H + (sequence, head)) * tensors + tensor: tile-major, so the low (working) tiles launch
    // first, keys and values side by side
    dim3 grid((unsigned)((size_t)p.B * p.H * ((p.N + RPB - 1) / RPB) * ntensors));
    constexpr size_t sm = RowsBwdLayout<D, Tin>::total;
    const RowsBwdArgs<Tin, Tsn> b0{(const Tin*)a0.x, a0.xold, a0.xfin, (const Tsn*)a0.dxbuf, (Tin*)a0.dx, a0.Dn, a0.dkinv};
    const RowsBwdArgs<Tin, Tsn> b1{(const Tin*)a1.x, a1.xold, a1.xfin, (const Tsn*)a1.dxbuf, (Tin*)a1.dx, a1.Dn, a1.dkinv};
    cudaError_t e;
    const bool dkinv = a0.dkinv != nullptr || a1.dkinv != nullptr;
    // the event-walk form: snapshot stride 8 or 16 (2 or 4 blocks per chunk) and D >= 64
    if constexpr (D >= 64) {
        constexpr size_t sm3 = RowsBwd3Layout<D, Tin>::total;
#define RB3_LAUNCH(GG_, DK_)                                                                 \
        {                                                                                    \
            auto kern = rows_bwd3_kernel<D, GG_, Tin, Tsn, DK_>;                             \
            if ((e = opt_in_smem(kern, sm3)) != cudaSuccess) return e;                       \
            kern<<<grid, ROW_THREADS, sm3, st>>>(p, b0, b1, gate, am, tfirst, ntensors);     \
            return cudaGetLastError();                                                       \
        }
        if (p.G == 8) { if (dkinv) RB3_LAUNCH(8, true) else RB3_LAUNCH(8, false) }
        if (p.G == 16) { if (dkinv) RB3_LAUNCH(16, true) else RB3_LAUNCH(16, false) }
#undef RB3_LAUNCH
    }
    if (dkinv) {
        auto kern = rows_bwd2_kernel<D, Tin, Tsn, true>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;
        kern<<<grid, ROW_THREADS, sm, st>>>(p, b0, b1, gate, am, tfirst, ntensors);
    } else {
        auto kern = rows_bwd2_kernel<D, Tin, Tsn, false>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;
        kern<<<grid, ROW_THREADS, sm, st>>>(p, b0, b1, gate, am, tfirst, ntensors);
    }
    return cudaGetLastError();
}

template <int D>
static cudaError_t rows_bwd_d(const slotscan_params& p, int nt, const RowsBwdPtrs& a0, const RowsBwdPtrs& a1,
                              const float* gate, const int* am, const int* tfirst, cudaStream_t st) {
    if (p.snap_dtype == SLOTSCAN_F32) return rows_bwd_one<D, float>(p, nt, a0, a1, gate, am, tfirst, st);
    return rows_bwd_one<D, __nv_bfloat16>(p, nt, a0, a1, gate, am, tfirst, st);
}

cudaError_t SS_CAT(run_rows_bwd_, SLOTSCAN_SUFFIX)(const slotscan_params& p, int D, int ntensors, const RowsBwdPtrs& a0,
                                                  const RowsBwdPtrs& a1, const float* gate, const int* am,
                                                  const int* tfirst, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    SLOTSCAN_DISPATCH_D(D, e = (rows_bwd_d<DD>(p, ntensors, a0, a1, gate, am, tfirst, st)));
    return e;
}

void SS_CAT(attrs_rows_bwd_, SLOTSCAN_SUFFIX)(slotscan_kernel_attr* out, int cap, int& n) {
    fill_attr(out, cap, n, "rows_bwd<128,snap=in>", rows_bwd3_kernel<128, 8, Tin, Tin, false>);
    fill_attr(out, cap, n, "rows_bwd_lockstep<128,snap=in>", rows_bwd2_kernel<128, Tin, Tin, false>);
}

// 1 when a bounded wait of this translation unit's kernels gave up since the last call (clears the flag)
int SS_CAT(rows_bwd_status_, SLOTSCAN_SUFFIX)() {
    int v = 0, z = 0;
    if (cudaMemcpyFromSymbol(&v, g_rows_bwd_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_rows_bwd_status, &z, sizeof(int));
    return v;
}

}  // namespace slotscan
