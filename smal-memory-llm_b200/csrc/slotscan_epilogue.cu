// Writer epilogue and storage quantiser: one streaming pass over the emitted snapshots.
//   [reference memlm_sh.py:464-475 (nsq, kinv, valid, cast to the model dtype), :221-234 (_fq, _quantize_mem)]
//
// Per snapshot row of D elements:  y = fq(x) (midrise, per group of `group` channels) or y = x;  the stored copy is
// cast to the output dtype;  for key rows  nsq = sum y^2 (fp32),  kinv = rsqrt(max(nsq, 1e-12)),  valid = nsq > 1e-12.
// The reference does this in four eager passes over 2 x 4.8 GB; here each element is read once and written once.
//
// Layout: LPR = D / 8 lanes per row, 8 consecutive elements per lane (one 16-byte load for bf16, two for f32), so a
// warp reads 32 / LPR whole rows back to back: fully coalesced.  A quantisation group of >= 8 channels spans
// group / 8 neighbouring lanes (absmax by shuffles); groups of 4 are two per lane.  Grid: a multiple of the SM
// count, grid-stride over rows.  HBM-bound: (e_in + e_out) * D bytes per row plus 5 bytes for kinv and valid.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "slotscan.h"
#include "slotscan_common.cuh"
#include "slotscan_launch.h"

namespace slotscan {

constexpr int EP_THREADS = 256;

__device__ __forceinline__ float round_to(float v, float) { return v; }
__device__ __forceinline__ float round_to(float v, __nv_bfloat16) { return __bfloat162float(__float2bfloat16_rn(v)); }

// fq of one group member, in the arithmetic of the reference: s = max(a / half, 1e-30),
// q = (clamp(floor(x / s), -half, half - 1) + 0.5) * s, zero for an all-zero group, returned in the straight-through
// form x + (q - x) evaluated in the input dtype (memlm_sh.py:229).
// The IEEE division x / s is what costs: it is replaced by x * (1 / s) wherever that provably has the same floor (the
// product is off by a few ulp of a quotient that is at most 128 in size, so any result further than 1e-3 from an
// integer floors alike), by the known answer for the group's own extreme (x = +-a gives exactly +-half), and kept for
// the rare rest.  s, 1 / s are per group.
struct FqScale { float a, half, s, rs; bool plain; };
__device__ __forceinline__ FqScale fq_scale(float a, float half) {
    FqScale g;
    g.a = a; g.half = half;
    g.s = fmaxf(__fdiv_rn(a, half), 1e-30f);
    g.rs = __frcp_rn(g.s);
    g.plain = a > 1e-20f;                    // s = a / half exactly: not clamped, not denormal
    return g;
}
// The same for the packed bf16 path: a * (1 / half) is the same float as a / half (half is a power of two), and 1 / s
// only has to place k within one of the quotient, so the approximate reciprocal will do; a group that is not `plain`
// goes through fq_one and gets the exact one.
__device__ __forceinline__ FqScale fq_scale_packed(float a, float half, float inv_half) {
    FqScale g;
    g.a = a; g.half = half;
    g.s = fmaxf(__fmul_rn(a, inv_half), 1e-30f);
    g.plain = a > 1e-20f;
    if (g.plain) asm("rcp.approx.f32 %0, %1;" : "=f"(g.rs) : "f"(g.s));     // (no .ftz: 1 / s may be subnormal for huge rows)
    else g.rs = __frcp_rn(g.s);
    return g;
}
template <typename Tin>
__device__ __forceinline__ float fq_one(float x, const FqScale& g) {
    float f;
    const float qt = x * g.rs, fl = floorf(qt), fr = qt - fl;
    if (g.plain && fabsf(x) == g.a) f = x > 0.f ? g.half : -g.half;
    else if (g.plain && fr > 1e-3f && fr < 0.999f) f = fl;
    else f = floorf(__fdiv_rn(x, g.s));
    f = fminf(fmaxf(f, -g.half), g.half - 1.f);
    const float q = (g.a > 0.f) ? __fmul_rn(__fadd_rn(f, 0.5f), g.s) : 0.f;
    const float qd = round_to(q, Tin());
    const float diff = round_to(__fsub_rn(qd, x), Tin());
    return round_to(__fadd_rn(x, diff), Tin());
}

// bf16 input, two elements at a time, in packed bf16 arithmetic wherever that is exact.  The group's extreme a is a
// bf16 value, so s = a / half (half a power of two) is a bf16 value too.  With k = rint(x * (1 / s)) (|k| <= 128, a
// bf16 value; one fused multiply-add against 1.5 * 2^23 rounds it)
//     floor(x / s) = k - [k * s > x],   and the sign of k * s - x survives the single rounding of a bf16 fma;
//     (f + 0.5) has at most 8 significant bits, and the bf16 product (f + 0.5) * s rounds the exact product once, as
//     the reference's float product (exact, 17 bits) followed by its cast does;
//     x + (q - x), each step rounded to bf16: a bf16 sum or difference of two bf16 values rounds once, and the float
//     detour of the reference rounds a value that is either exact in float or within 2^-16 of one operand, so both
//     land on the same bf16.
// No division and no near-integer case is left over.  The lower clamp never binds (x >= -a gives k * s >= x at
// k = -half).  Groups whose scale is clamped or denormal take fq_one.
template <bool KNOWN_PLAIN>
__device__ __forceinline__ unsigned fq_pair_bf16(const unsigned xw, const FqScale& g, const unsigned hm1) {   // hm1: half - 1 | half - 1
    const __nv_bfloat162 x2 = *reinterpret_cast<const __nv_bfloat162*>(&xw);
    const float2 x = __bfloat1622float2(x2);
    __nv_bfloat162 r2;
    if (!KNOWN_PLAIN && g.a == 0.f) return 0u;           // an all-zero group stays zero (x + (0 - x) = +0)
    if (KNOWN_PLAIN || g.plain) {
        const float MAGIC = 12582912.f;                  // 1.5 * 2^23: adding it rounds to an integer
        const float k0 = __fadd_rn(__fmaf_rn(x.x, g.rs, MAGIC), -MAGIC), k1 = __fadd_rn(__fmaf_rn(x.y, g.rs, MAGIC), -MAGIC);
        // k and s are bf16 values held in floats: their bf16 forms are the upper halves (byte permutes, no conversion)
        const unsigned kw = __byte_perm(__float_as_uint(k0), __float_as_uint(k1), 0x7632);
        const unsigned sw = __byte_perm(__float_as_uint(g.s), 0u, 0x3232), zw = 0u, hw = 0x3f003f00u;   // s | s, 0 | 0, 0.5 | 0.5
        const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(&kw), s2 = *reinterpret_cast<const __nv_bfloat162*>(&sw);
        const __nv_bfloat162 over = __hgt2(__hfma2(k2, s2, __hneg2(x2)), *reinterpret_cast<const __nv_bfloat162*>(&zw));   // 1.0 where k * s > x
        const __nv_bfloat162 f2 = __hmin2(__hsub2(k2, over), *reinterpret_cast<const __nv_bfloat162*>(&hm1));
        const __nv_bfloat162 qd = __hmul2(__hadd2(f2, *reinterpret_cast<const __nv_bfloat162*>(&hw)), s2);
        r2 = __hadd2(x2, __hsub2(qd, x2));
    } else {
        r2 = __floats2bfloat162_rn(fq_one<__nv_bfloat16>(x.x, g), fq_one<__nv_bfloat16>(x.y, g));
    }
    return *reinterpret_cast<const unsigned*>(&r2);
}
__device__ __forceinline__ float absmax_pair(const unsigned a, const unsigned b) {     // max |.| of four bf16 values
    const unsigned m = 0x7fff7fffu;
    const unsigned ua = a & m, ub = b & m;
    const __nv_bfloat162 h = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&ua), *reinterpret_cast<const __nv_bfloat162*>(&ub));
    const float2 f = __bfloat1622float2(h);
    return fmaxf(f.x, f.y);
}

// PACKED: the midrise quantiser on bf16 input (bits > 0), a kernel of its own so that its registers do not cost the
// plain pass its eight resident CTAs per SM.
template <int D, typename Tin, typename Tout, bool PACKED>
__global__ void __launch_bounds__(EP_THREADS, PACKED ? 6 : 1) writer_epilogue_kernel(const Tin* __restrict__ x, Tout* __restrict__ y,
                                                                     float* __restrict__ kinv,
                                                                     uint8_t* __restrict__ valid, const long long rows,
                                                                     const int bits, const int group) {
    constexpr int LPR = D / 8, RPB = EP_THREADS / LPR;
    const int r = threadIdx.x / LPR, c = threadIdx.x % LPR;
    const float half = bits > 0 ? (float)(1 << (bits - 1)) : 0.f;
    const float inv_half = bits > 0 ? 1.f / half : 0.f;
    const unsigned hm1 = __byte_perm(__float_as_uint(half - 1.f), 0u, 0x3232);     // half - 1 as a bf16 pair (exact)
    const long long stride = (long long)gridDim.x * RPB;
    uint4 ahead = make_uint4(0, 0, 0, 0);                // the next row of this lane, in flight while this one is worked on
    if constexpr (PACKED) {
        const long long first = (long long)blockIdx.x * RPB + r;
        if (first < rows) ahead = *reinterpret_cast<const uint4*>(x + first * D + c * 8);
    }
    for (long long row0 = (long long)blockIdx.x * RPB; row0 < rows; row0 += stride) {
        const long long row = row0 + r;
        const bool live = row < rows;                    // dead lanes keep running the shuffles on zeros
        float v[8];
        if constexpr (PACKED) {
            {                                             // midrise quantiser on packed bf16 pairs
                const uint4 u = ahead;
                ahead = row + stride < rows ? *reinterpret_cast<const uint4*>(x + (row + stride) * D + c * 8) : make_uint4(0, 0, 0, 0);
                unsigned w[4] = {u.x, u.y, u.z, u.w};
                float a0 = absmax_pair(w[0], w[1]), a1 = absmax_pair(w[2], w[3]);
                if (group >= 8) {
                    a0 = fmaxf(a0, a1);
                    for (int off = 1; off < group / 8; off <<= 1) a0 = fmaxf(a0, __shfl_xor_sync(FULL, a0, off));
                    a1 = a0;
                }
                const FqScale g0 = fq_scale_packed(a0, half, inv_half), g1 = group >= 8 ? g0 : fq_scale_packed(a1, half, inv_half);
                if (g0.plain && g1.plain) {                  // the usual case, straight-line
                    w[0] = fq_pair_bf16<true>(w[0], g0, hm1); w[1] = fq_pair_bf16<true>(w[1], g0, hm1);
                    w[2] = fq_pair_bf16<true>(w[2], g1, hm1); w[3] = fq_pair_bf16<true>(w[3], g1, hm1);
                } else {
                    w[0] = fq_pair_bf16<false>(w[0], g0, hm1); w[1] = fq_pair_bf16<false>(w[1], g0, hm1);
                    w[2] = fq_pair_bf16<false>(w[2], g1, hm1); w[3] = fq_pair_bf16<false>(w[3], g1, hm1);
                }
                if (y != nullptr && live) {
                    if constexpr (sizeof(Tout) == 2) *reinterpret_cast<uint4*>(y + row * D + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                if (kinv != nullptr || sizeof(Tout) == 4) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        v[2 * i] = __uint_as_float(w[i] << 16);
                        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
                    }
                    if constexpr (sizeof(Tout) == 4) {
                        if (y != nullptr && live) st8(y + row * D + c * 8, v);
                    }
                }
                if (kinv != nullptr) {
                    float nsq = 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) nsq = fmaf(v[j], v[j], nsq);
                    nsq = group_sum<LPR>(nsq);
                    if (live && c == 0) {
                        kinv[row] = rsqrtf(fmaxf(nsq, 1e-12f));
                        valid[row] = nsq > 1e-12f ? 1 : 0;
                    }
                }
                continue;
            }
        }
        if (live) ld8(v, x + row * D + c * 8);
        else {
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = 0.f;
        }
        if (bits == SLOTSCAN_BITS_E4M3) {                 // fp8-e4m3 storage, one scale per row
            float a = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) a = fmaxf(a, fabsf(v[j]));
            for (int off = 1; off < LPR; off <<= 1) a = fmaxf(a, __shfl_xor_sync(FULL, a, off));
            const float sc = fmaxf(__fdiv_rn(a, 448.f), 1e-30f);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(__fdiv_rn(v[j], sc), __NV_SATFINITE, __NV_E4M3);
                const float f = __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
                v[j] = a > 0.f ? __fmul_rn(f, sc) : 0.f;
            }
        } else if (bits) {
            if (group >= 8) {
                float a = 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) a = fmaxf(a, fabsf(v[j]));
                for (int off = 1; off < group / 8; off <<= 1) a = fmaxf(a, __shfl_xor_sync(FULL, a, off));
                const FqScale gs = fq_scale(a, half);
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] = fq_one<Tin>(v[j], gs);
            } else {                                     // group == 4: two groups inside the lane
#pragma unroll
                for (int g = 0; g < 2; g++) {
                    float a = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; j++) a = fmaxf(a, fabsf(v[4 * g + j]));
                    const FqScale gs = fq_scale(a, half);
#pragma unroll
                    for (int j = 0; j < 4; j++) v[4 * g + j] = fq_one<Tin>(v[4 * g + j], gs);
                }
            }
        }
        if (y != nullptr && live) st8(y + row * D + c * 8, v);
        if (kinv != nullptr) {
            float nsq = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) nsq = fmaf(v[j], v[j], nsq);
            nsq = group_sum<LPR>(nsq);
            if (live && c == 0) {
                kinv[row] = rsqrtf(fmaxf(nsq, 1e-12f));
                valid[row] = nsq > 1e-12f ? 1 : 0;
            }
        }
    }
}

template <int D, typename Tin, typename Tout>
static cudaError_t launch_ep(const void* x, void* y, float* kinv, uint8_t* valid, long long rows, int bits, int group,
                             cudaStream_t st) {
    constexpr int RPB = EP_THREADS / (D / 8);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long want = (rows + RPB - 1) / RPB;
    auto go = [&](auto kern) {
        int per_sm = 8;                                  // resident CTAs per SM: the grid is exactly one wave
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, EP_THREADS, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
        const long long cap = (long long)sms * per_sm;
        const int grid = (int)(want < cap ? (want > 0 ? want : 1) : cap);
        kern<<<grid, EP_THREADS, 0, st>>>((const Tin*)x, (Tout*)y, kinv, valid, rows, bits, group);
    };
    if (sizeof(Tin) == 2 && bits > 0) go(writer_epilogue_kernel<D, Tin, Tout, sizeof(Tin) == 2>);
    else go(writer_epilogue_kernel<D, Tin, Tout, false>);
    return cudaGetLastError();
}

template <typename Tin, typename Tout>
static cudaError_t launch_ep_d(int D, const void* x, void* y, float* kinv, uint8_t* valid, long long rows, int bits,
                               int group, cudaStream_t st) {
    cudaError_t e = cudaErrorInvalidValue;
    SLOTSCAN_DISPATCH_D(D, e = (launch_ep<DD, Tin, Tout>(x, y, kinv, valid, rows, bits, group, st)));
    return e;
}

}  // namespace slotscan

using namespace slotscan;

extern "C" int slotscan_epilogue_check(const slotscan_epilogue_params* p) {
    if (p == nullptr) return SLOTSCAN_E_NULL;
    if (p->rows < 0) return SLOTSCAN_E_SHAPE;
    const int D = p->D;
    if (!(D == 8 || D == 16 || D == 32 || D == 64 || D == 128)) return SLOTSCAN_E_SHAPE;
    if ((p->in_dtype != SLOTSCAN_F32 && p->in_dtype != SLOTSCAN_BF16) ||
        (p->out_dtype != SLOTSCAN_F32 && p->out_dtype != SLOTSCAN_BF16))
        return SLOTSCAN_E_DTYPE;
    if (p->bits != 0 && p->bits != SLOTSCAN_BITS_E4M3) {
        if (!(p->bits == 2 || p->bits == 3 || p->bits == 4 || p->bits == 8)) return SLOTSCAN_E_MODE;   /* memlm_sh.py:81 */
        const int g = p->group;
        if (g < 4 || g > D || (g & (g - 1)) != 0) return SLOTSCAN_E_MODE;   /* power of two that divides D (:82-83) */
    }
    return SLOTSCAN_OK;
}

extern "C" int slotscan_writer_epilogue(const slotscan_epilogue_params* p, const void* x, void* y, float* kinv,
                                        uint8_t* valid, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    const int rc = slotscan_epilogue_check(p);
    if (rc != SLOTSCAN_OK) return rc;
    if (x == nullptr || (kinv == nullptr) != (valid == nullptr) || (y == nullptr && kinv == nullptr)) return SLOTSCAN_E_NULL;
    if (((uintptr_t)x | (uintptr_t)y) & 15) return SLOTSCAN_E_ALIGN;
    if (p->rows == 0) return SLOTSCAN_OK;
    cudaError_t e;
    const bool ib = p->in_dtype == SLOTSCAN_BF16, ob = p->out_dtype == SLOTSCAN_BF16;
    if (ib && ob) e = launch_ep_d<__nv_bfloat16, __nv_bfloat16>(p->D, x, y, kinv, valid, p->rows, p->bits, p->group, stream);
    else if (ib) e = launch_ep_d<__nv_bfloat16, float>(p->D, x, y, kinv, valid, p->rows, p->bits, p->group, stream);
    else if (ob) e = launch_ep_d<float, __nv_bfloat16>(p->D, x, y, kinv, valid, p->rows, p->bits, p->group, stream);
    else e = launch_ep_d<float, float>(p->D, x, y, kinv, valid, p->rows, p->bits, p->group, stream);
    return (int)e;             /* 0, or the positive CUDA error code like the scan entry points */
}
