// Shared device helpers of the slot-scan kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "slotscan.h"

namespace slotscan {

constexpr unsigned FULL = 0xffffffffu;
constexpr int BIGI = 0x7fffffff;

// ---- typed vector loads / stores: token streams and snapshots are f32 or bf16, arithmetic is always f32 ----
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<unsigned*>(&a);
    u.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
}
__device__ __forceinline__ void ld8(float* d, const float* s) {
    const float4 a = ld4(s), b = ld4(s + 4);
    d[0] = a.x; d[1] = a.y; d[2] = a.z; d[3] = a.w; d[4] = b.x; d[5] = b.y; d[6] = b.z; d[7] = b.w;
}
__device__ __forceinline__ void ld8(float* d, const __nv_bfloat16* s) {
    const uint4 u = *reinterpret_cast<const uint4*>(s);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        d[2 * i] = f.x; d[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void st8(float* d, const float* s) {
    st4(d, make_float4(s[0], s[1], s[2], s[3]));
    st4(d + 4, make_float4(s[4], s[5], s[6], s[7]));
}
__device__ __forceinline__ void st8(__nv_bfloat16* d, const float* s) {
    unsigned w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(s[2 * i], s[2 * i + 1]);
        w[i] = *reinterpret_cast<unsigned*>(&h);
    }
    *reinterpret_cast<uint4*>(d) = make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(FULL, v, off);
    return v;
}
// sum over the LPR (power of two <= 32) adjacent lanes that share one row
template <int LPR>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(FULL, v, off);
    return v;
}
__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

// The one write rule of the scan, state <- (1-g) state + g x, spelled identically in every kernel so that a row
// replayed by another kernel is bit-identical to the row the address kernel held.
__device__ __forceinline__ float blend(float old, float x, float g, float omw) {
    return __fmaf_rn(g, x, __fmul_rn(omw, old));
}

// occupied candidate (z, i): larger z wins, equal z -> smaller index (argmax returns the FIRST maximum)
__device__ __forceinline__ void best(float& z, int& i, float z2, int i2) {
    if (z2 > z || (z2 == z && i2 < i)) { z = z2; i = i2; }
}

__device__ __forceinline__ unsigned ord_key(float f) {    // monotone float -> unsigned
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float gate_eff(float g, int hard_gate) { return hard_gate ? (g > 0.5f ? 1.f : 0.f) : g; }

}  // namespace slotscan
