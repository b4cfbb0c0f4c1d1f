// Forward row replay (slotscan_rows.cuh) instantiated for every row width and dtype pair.
#include <stdio.h>

#include "slotscan_launch.h"
#include "slotscan_rows.cuh"

namespace slotscan {

template <int D, typename Tin, typename Tsn>
static cudaError_t replay_one(const slotscan_params& p, int ntensors, const ReplayPtrs& r0, const ReplayPtrs& r1,
                              const float* gate, const int* am, const int* tfirst, int tile_lo, int tile_hi, cudaStream_t st) {
    constexpr int RPB = ROW_THREADS / (D / 8);
    const int ntiles = (p.N + RPB - 1) / RPB;
    if (tile_hi < 0 || tile_hi > ntiles) tile_hi = ntiles;
    if (tile_lo >= tile_hi) return cudaSuccess;
    dim3 grid(p.B * p.H, tile_hi - tile_lo, ntensors);
    const ReplayArgs<Tin, Tsn> a0{(const Tin*)r0.x, r0.x0, (Tsn*)r0.xbuf, r0.xold, r0.xfin, r0.kinv, r0.valid, r0.zero_from};
    const ReplayArgs<Tin, Tsn> a1{(const Tin*)r1.x, r1.x0, (Tsn*)r1.xbuf, r1.xold, r1.xfin, r1.kinv, r1.valid, r1.zero_from};
    constexpr int EPL = D >= 128 ? 16 : 8;                 // elements per lane: half-size CTAs for the widest rows
    constexpr int THREADS = ROW_THREADS * 8 / EPL;
    if (r0.kinv != nullptr || r1.kinv != nullptr)
        replay_rows_kernel<D, Tin, Tsn, true, EPL><<<grid, THREADS, 0, st>>>(p, a0, a1, gate, am, tfirst, tile_lo);
    else
        replay_rows_kernel<D, Tin, Tsn, false, EPL><<<grid, THREADS, 0, st>>>(p, a0, a1, gate, am, tfirst, tile_lo);
    return cudaGetLastError();
}

#define ROWS_TYPES(CALL_F32_F32, CALL_F32_BF16, CALL_BF16_F32, CALL_BF16_BF16)            \
    if (p.in_dtype == SLOTSCAN_F32) {                                                     \
        if (p.snap_dtype == SLOTSCAN_F32) { CALL_F32_F32; } else { CALL_F32_BF16; }       \
    } else {                                                                              \
        if (p.snap_dtype == SLOTSCAN_F32) { CALL_BF16_F32; } else { CALL_BF16_BF16; }     \
    }

template <int D>
static cudaError_t replay_d(const slotscan_params& p, int nt, const ReplayPtrs& r0, const ReplayPtrs& r1, const float* gate,
                            const int* am, const int* tfirst, int tlo, int thi, cudaStream_t st) {
    typedef __nv_bfloat16 bf;
    ROWS_TYPES(return (replay_one<D, float, float>(p, nt, r0, r1, gate, am, tfirst, tlo, thi, st)),
               return (replay_one<D, float, bf>(p, nt, r0, r1, gate, am, tfirst, tlo, thi, st)),
               return (replay_one<D, bf, float>(p, nt, r0, r1, gate, am, tfirst, tlo, thi, st)),
               return (replay_one<D, bf, bf>(p, nt, r0, r1, gate, am, tfirst, tlo, thi, st)))
}

// row tiles [tile_lo, tile_hi) of every (sequence, head); tile_hi < 0: up to the last one
cudaError_t run_replay(const slotscan_params& p, int D, int ntensors, const ReplayPtrs& r0, const ReplayPtrs& r1,
                       const float* gate, const int* am, const int* tfirst, int tile_lo, int tile_hi, cudaStream_t st) {
    cudaError_t e = cudaSuccess;
    SLOTSCAN_DISPATCH_D(D, e = (replay_d<DD>(p, ntensors, r0, r1, gate, am, tfirst, tile_lo, tile_hi, st)));
    return e;
}

int replay_status() {
    int v = 0, z = 0;
    if (cudaMemcpyFromSymbol(&v, g_replay_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_replay_status, &z, sizeof(int));
    return v;
}

// rows of a snapshot tile of the row kernels for width D
int replay_tile_rows(int D) { return ROW_THREADS / (D / 8); }

// Zero-fill of the rows [zk, N) of every key snapshot (with kinv = 1e6, valid = 0 when given) and [zv, N) of every
// value snapshot; zk / zv = N skips that tensor.
cudaError_t run_zero_rows(const slotscan_params& p, void* kbuf, int zk, void* vbuf, int zv, float* kinv, uint8_t* valid,
                          cudaStream_t st) {
    const long long nsnap = (long long)p.B * ((p.T + p.G - 1) / p.G) * p.H;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t esz = p.snap_dtype == SLOTSCAN_F32 ? 4 : 2;
    const ZeroTarget ta{zk < p.N ? (unsigned char*)kbuf : nullptr, (size_t)p.DK * esz, zk};
    const ZeroTarget tb{zv < p.N ? (unsigned char*)vbuf : nullptr, (size_t)p.DV * esz, zv};
    auto aligned = [&](const ZeroTarget& t) {
        return t.x == nullptr || ((t.row_bytes * (size_t)t.zero_from) % 16 == 0 && (t.row_bytes * (size_t)(p.N - t.zero_from)) % 16 == 0 &&
                                  (t.row_bytes * (size_t)p.N) % 16 == 0 && ((uintptr_t)t.x & 15) == 0);
    };
    if (ta.x == nullptr && tb.x == nullptr) return cudaSuccess;
    if (aligned(ta) && aligned(tb)) {
        const long long want = nsnap < (long long)sms ? nsnap : (long long)sms;         // one copy-issuing warp per SM
        zero_rows_bulk_kernel<<<(unsigned)want, ZB_THREADS, 0, st>>>(ta, tb, ta.x ? kinv : nullptr, valid, p.N, nsnap);
        return cudaGetLastError();
    }
    const long long want = nsnap < (long long)sms * 4 ? nsnap : (long long)sms * 4;     // a few small CTAs per SM: they share it with the scan
    for (int w = 0; w < 2; w++) {
        const ZeroTarget& t = w ? tb : ta;
        if (t.x == nullptr) continue;
        const int D = w ? p.DV : p.DK;
        float* ki = w ? nullptr : kinv;
        uint8_t* va = w ? nullptr : valid;
        if (p.snap_dtype == SLOTSCAN_F32)
            zero_rows_kernel<float><<<(unsigned)want, ZR_THREADS, 0, st>>>((float*)t.x, ki, va, p.N, D, t.zero_from, nsnap);
        else
            zero_rows_kernel<__nv_bfloat16><<<(unsigned)want, ZR_THREADS, 0, st>>>((__nv_bfloat16*)t.x, ki, va, p.N, D, t.zero_from, nsnap);
    }
    return cudaGetLastError();
}

void attrs_rows(slotscan_kernel_attr* out, int cap, int& n) {
    fill_attr(out, cap, n, "replay_rows<128,bf16,bf16>", replay_rows_kernel<128, __nv_bfloat16, __nv_bfloat16, false, 16>);
    fill_attr(out, cap, n, "replay_rows<128,bf16,bf16,kinv>", replay_rows_kernel<128, __nv_bfloat16, __nv_bfloat16, true, 16>);
    fill_attr(out, cap, n, "replay_rows<128,f32,f32>", replay_rows_kernel<128, float, float, false, 16>);
}

}  // namespace slotscan
