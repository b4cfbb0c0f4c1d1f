// Instantiation body of the address backward for one input dtype: included by slotscan_addr_bwd_{f32,bf16}.cu
// with SLOTSCAN_TIN and SLOTSCAN_SUFFIX defined.
#include <stdio.h>

#include "slotscan_addr_bwd.cuh"
#include "slotscan_addr_gather.cuh"
#include "slotscan_launch.h"

namespace slotscan {

#define SS_CAT_(a, b) a##b
#define SS_CAT(a, b) SS_CAT_(a, b)
typedef SLOTSCAN_TIN Tin;

template <int DK, int RPL, int MINB>
static cudaError_t launch_one(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                              const float* temp, const slotscan_log& L, const float* Dn, void* dq, float* dgate,
                              float* dfr, float* part, int ncap, int big, int skip_rows, int part_stride, cudaStream_t st) {
    const size_t sm = sizeof(float) * (size_t)addr_bwd_layout(ncap, DK).total;
    cudaError_t e;
    if (p.occ_bin) {
        auto kern = addr_bwd_chunked_kernel<DK, RPL, true, MINB, Tin>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;
        kern<<<p.B * p.H, AB_THREADS, sm, st>>>(p, (const Tin*)q, (const Tin*)k, gate, fr, temp, L.addr, L.kold, L.oold,
                                                L.kiold, L.kfin, L.ofin, L.tfirst, Dn, (Tin*)dq, dgate, dfr, part, ncap, big, skip_rows,
                                                part_stride);
    } else {
        auto kern = addr_bwd_chunked_kernel<DK, RPL, false, MINB, Tin>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;
        kern<<<p.B * p.H, AB_THREADS, sm, st>>>(p, (const Tin*)q, (const Tin*)k, gate, fr, temp, L.addr, L.kold, L.oold,
                                                L.kiold, L.kfin, L.ofin, L.tfirst, Dn, (Tin*)dq, dgate, dfr, part, ncap, big, skip_rows,
                                                part_stride);
    }
    return cudaGetLastError();
}

template <int DK>
static cudaError_t launch_gather(const slotscan_params& p, const void* q, const float* gate, const float* fr,
                                 const float* temp, const slotscan_log& L, const float* Dn, void* dq, float* dgate,
                                 float* dfr, float* part, int* vend, int part_stride, bool vend_ready, cudaStream_t st) {
    if constexpr (DK >= 32) {
        cudaError_t e = cudaSuccess;
        if (!vend_ready) {
            next_write_kernel<<<p.B * p.H, 32, 0, st>>>(p, L.addr, L.tfirst, vend);
            if ((e = cudaGetLastError()) != cudaSuccess) return e;
        }
        dim3 grid(p.B * p.H, (p.T + GC - 1) / GC);
        const size_t dyn = (size_t)GC * DK * sizeof(Tin) + 2 * (size_t)GC * GATHER_ROWS * sizeof(float);   // queries + D rows
        auto gk = addr_bwd_gather_kernel<DK, Tin>;
        if ((e = opt_in_smem(gk, dyn)) != cudaSuccess) return e;
        gk<<<grid, GA_THREADS, dyn, st>>>(p, (const Tin*)q, gate, fr, temp, L.addr, L.kold, L.oold,
                                                                      L.kiold, L.kfin, L.ofin, L.tfirst, vend, Dn, (Tin*)dq,
                                                                      dgate, dfr, part, part_stride);
        return cudaGetLastError();
    } else {
        return cudaSuccess;
    }
}

template <int DK>
static cudaError_t launch_dk(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                             const float* temp, const slotscan_log& L, const float* Dn, void* dq, float* dgate, float* dfr,
                             float* part, int* vend, int part_stride, bool vend_ready, cudaStream_t st) {
    // Sequences with at most GATHER_ROWS candidate rows go to the token-parallel gather kernel (occ_bin only: the
    // occupancy adjoint is not carried there); the rest, and every sequence of the other modes, to the chunked one.
    int skip = 0;
    if (p.occ_bin && DK >= 32) {
        cudaError_t e = launch_gather<DK>(p, q, gate, fr, temp, L, Dn, dq, dgate, dfr, part, vend, part_stride, vend_ready, st);
        if (e != cudaSuccess) return e;
        skip = GATHER_ROWS;
        if (p.N <= GATHER_ROWS) return cudaSuccess;
    }
    // Measured on B200 (B = 64, T = 1024, 6 heads, 192 x 128): splitting the chunked work between a 64-row variant
    // (three CTAs per SM) and the full one ran 1.6x SLOWER than the full variant alone, so only one is launched.
    if (p.N <= AF_NCAP1)
        return launch_one<DK, 2, 2>(p, q, k, gate, fr, temp, L, Dn, dq, dgate, dfr, part, p.N, 0, skip, part_stride, st);
    return launch_one<DK, 6, 2>(p, q, k, gate, fr, temp, L, Dn, dq, dgate, dfr, part, p.N, 0, skip, part_stride, st);   // N <= 192
}

cudaError_t SS_CAT(run_addr_bwd_, SLOTSCAN_SUFFIX)(const slotscan_params& p, const void* q, const void* k, const float* gate,
                                                  const float* fr, const float* temp, const slotscan_log& L,
                                                  const float* Dn, void* dq, float* dgate, float* dfr, float* part,
                                                  int* vend, int part_stride, bool vend_ready, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    SLOTSCAN_DISPATCH_D(p.DK, e = (launch_dk<DD>(p, q, k, gate, fr, temp, L, Dn, dq, dgate, dfr, part, vend, part_stride, vend_ready, st)));
    return e;
}

#ifdef SLOTSCAN_DEFINE_NEXT_WRITE
bool next_write_used(const slotscan_params& p) { return p.occ_bin && p.DK >= 32; }
cudaError_t run_next_write(const slotscan_params& p, const slotscan_log& L, int* vend, cudaStream_t st) {
    next_write_kernel<<<p.B * p.H, 32, 0, st>>>(p, L.addr, L.tfirst, vend);
    return cudaGetLastError();
}
#endif

// 1 when a bounded wait of this translation unit's kernels gave up since the last call (clears the flag)
int SS_CAT(gather_status_, SLOTSCAN_SUFFIX)() {
    int v = 0, z = 0;
    if (cudaMemcpyFromSymbol(&v, g_gather_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_gather_status, &z, sizeof(int));
    return v;
}

void SS_CAT(attrs_addr_bwd_, SLOTSCAN_SUFFIX)(slotscan_kernel_attr* out, int cap, int& n) {
    fill_attr(out, cap, n, "addr_bwd<128,rows<=64>", addr_bwd_chunked_kernel<128, 2, true, 2, Tin>);
    fill_attr(out, cap, n, "addr_bwd<128,rows<=192>", addr_bwd_chunked_kernel<128, 6, true, 2, Tin>);
    fill_attr(out, cap, n, "addr_bwd_gather<128>", addr_bwd_gather_kernel<128, Tin>);
}

}  // namespace slotscan
