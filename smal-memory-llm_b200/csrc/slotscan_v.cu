// Keyless slot scan: the address logits come from outside, the state holds values only.
//   [reference gqa25/slotkern_v.py: definition ref_scan_v :242-261, Triton kernels _vfwd :25, _vrecompute :75,
//    _vadjoint :120, adjoint stated in the module docstring :14-19]
//
//   z = wa_t - fr o over ALL N rows (no free-row mask),  a_s = softmax(z),  a = onehot(argmax z) if hard else a_s,
//   g_h = [g > 0.5] if hard_gate else g,  w = g_h a,  V <- (1 - w) V + w v_t,  o <- (1 - w) o + w;
//   the pre-write V goes out every G tokens.  Backward (straight-through for the hard address and the hard gate):
//   dw = <v - V, dV'> + (1 - o) do',  dv = sum_n w dV',  dg = a . dw,  dz = a_s (g_h dw - a_s . g_h dw),  dwa = dz,
//   dfr -= o . dz,  dV = (1 - w) dV' + dbuf,  do = (1 - w) do' - fr dz.
//
// One CTA per (sequence, head), values and occupancy resident in shared memory (the reference's shape is 48 x 16).
// The occupancies and the softmax run in double: with the penalty on o itself every rounding error of o comes back
// multiplied by fr at every later token.  The emitted buffers (values, and occupancies as a second output) are the
// backward's checkpoints: per block of G tokens it replays the forward into G state slots of scratch, then walks the
// block in reverse.  Like the general keyed scan this mode is built for completeness of the reference's call surface
// (no model of the reference run calls it) and is not tuned.
#include <math.h>
#include <stdio.h>

#include "slotscan_common.cuh"
#include "slotscan_launch.h"

namespace slotscan {

constexpr int KV_THREADS = 128, KV_WARPS = KV_THREADS / 32;

__device__ __forceinline__ float ldv(const float* p) { return *p; }
__device__ __forceinline__ float ldv(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stv(float* p, float x) { *p = x; }
__device__ __forceinline__ void stv(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }

// One warp: address of a token from its logits and the occupancies.  z[n] (double scratch) is overwritten.
// Returns the argmax (first maximum); asoft / afwd receive the softmax and the address the forward uses.
template <typename TO>
__device__ __forceinline__ int keyless_address(const float* wa_t, const TO* o, int N, double fr, int hard, double* z,
                                               float* asoft, float* afwd) {
    const int lane = threadIdx.x & 31;
    double bz = -INFINITY;
    int bi = BIGI;
    for (int n = lane; n < N; n += 32) {
        const double zz = (double)wa_t[n] - fr * (double)o[n];
        z[n] = zz;
        if (zz > bz) { bz = zz; bi = n; }
    }
    double zmax = bz;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) zmax = fmax(zmax, __shfl_xor_sync(FULL, zmax, off));
    int am = (int)__reduce_min_sync(FULL, (unsigned)((bi != BIGI && bz == zmax) ? bi : BIGI));
    am = min(am, N - 1);
    double se = 0.0;
    for (int n = lane; n < N; n += 32) { const double e = exp(z[n] - zmax); z[n] = e; se += e; }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) se += __shfl_xor_sync(FULL, se, off);
    for (int n = lane; n < N; n += 32) {
        const float a = (float)(z[n] / se);
        asoft[n] = a;
        afwd[n] = hard ? (n == am ? 1.f : 0.f) : a;
    }
    __syncwarp();
    return am;
}

__host__ __device__ inline size_t keyless_fwd_smem_floats(int N, int DV) { return (size_t)N * DV + 8 * (size_t)N + DV + 32; }
__host__ __device__ inline size_t keyless_bwd_smem_floats(int N, int DV) { return (size_t)N * DV + 10 * (size_t)N + DV + 64; }
__host__ __device__ inline size_t keyless_state_floats(int N, int DV) { return (size_t)N * (DV + 1); }

template <typename Tin>
__global__ void __launch_bounds__(KV_THREADS) keyless_fwd_kernel(const slotscan_v_params p, const Tin* __restrict__ v,
                                                                 const float* __restrict__ wa,
                                                                 const float* __restrict__ gate,
                                                                 const float* __restrict__ fr_p, float* __restrict__ buf,
                                                                 float* __restrict__ obuf, int* __restrict__ addr) {
    extern __shared__ __align__(16) float ksm[];
    const int N = p.N, T = p.T, H = p.H, DV = p.DV, G = p.G;
    const int NB = (T + G - 1) / G, NE = (N + 1) & ~1;
    double* z = reinterpret_cast<double*>(ksm);             // [N]
    double* o = z + NE;                                     // [N]
    float* V = ksm + 4 * (size_t)NE;
    float* a = V + (size_t)N * DV;
    float* as = a + N;
    float* wt = as + N;                                     // this token's logits
    float* vt = wt + N;
    float* s_f = vt + DV;                                   // [0] g_h
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, warp = tid >> 5;
    const double fr = (double)fr_p[0];
    for (int i = tid; i < N * DV; i += KV_THREADS) V[i] = 0.f;
    for (int i = tid; i < N; i += KV_THREADS) o[i] = 0.0;
    __syncthreads();
    for (int t = 0; t < T; t++) {
        const size_t ix = ((size_t)b * T + t) * H + h;
        if (t % G == 0) {
            const size_t so = ((size_t)b * NB + t / G) * H + h;
            for (int i = tid; i < N * DV; i += KV_THREADS) buf[so * N * DV + i] = V[i];
            for (int i = tid; i < N; i += KV_THREADS) obuf[so * N + i] = (float)o[i];
        }
        for (int n = tid; n < N; n += KV_THREADS) wt[n] = wa[ix * N + n];
        for (int d = tid; d < DV; d += KV_THREADS) vt[d] = ldv(v + ix * DV + d);
        __syncthreads();
        if (warp == 0) {
            const int am = keyless_address(wt, o, N, fr, p.hard, z, as, a);
            const float g = gate_eff(gate[ix], p.hard_gate);
            for (int n = (tid & 31); n < N; n += 32) {
                const double w = (double)g * (double)a[n];
                if (a[n] != 0.f) o[n] = (1.0 - w) * o[n] + w;
            }
            if (tid == 0) {
                s_f[0] = g;
                if (addr != nullptr) addr[ix] = am;
            }
        }
        __syncthreads();
        const float g = s_f[0];
        for (int n = tid >> 5; n < N; n += KV_THREADS / 32) {      // a warp per row, lanes over the columns
            const float an = a[n];
            if (an == 0.f) continue;
            const float w = g * an;
            float* Vr = V + (size_t)n * DV;
            for (int d = tid & 31; d < DV; d += 32) Vr[d] = (1.f - w) * Vr[d] + w * vt[d];
        }
        __syncthreads();
    }
}

template <typename Tin>
__global__ void __launch_bounds__(KV_THREADS) keyless_bwd_kernel(const slotscan_v_params p, const Tin* __restrict__ v,
                                                                 const float* __restrict__ wa,
                                                                 const float* __restrict__ gate,
                                                                 const float* __restrict__ fr_p,
                                                                 const float* __restrict__ buf,
                                                                 const float* __restrict__ obuf,
                                                                 const float* __restrict__ dbuf, float* __restrict__ seg,
                                                                 Tin* __restrict__ dv, float* __restrict__ dwa,
                                                                 float* __restrict__ dgate, float* __restrict__ part) {
    extern __shared__ __align__(16) float ksm[];
    const int N = p.N, T = p.T, H = p.H, DV = p.DV, G = p.G;
    const int NB = (T + G - 1) / G, NE = (N + 1) & ~1;
    double* z = reinterpret_cast<double*>(ksm);             // [N]
    float* dV = ksm + 2 * (size_t)NE;
    float* dO = dV + (size_t)N * DV;
    float* a = dO + N;
    float* as = a + N;
    float* wt = as + N;
    float* dw = wt + N;
    float* dz = dw + N;
    float* vt = dz + N;
    float* s_f = vt + DV;                                   // [0] g_h
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const double fr = (double)fr_p[0];
    const float frf = fr_p[0];
    const size_t SV = (size_t)N * DV, SS = keyless_state_floats(N, DV);
    float* myseg = seg + (size_t)bh * G * SS;               // slot j: state before token t0 + j (slot 0 unused: the snapshot)
    for (size_t i = tid; i < SV; i += KV_THREADS) dV[i] = 0.f;
    for (int i = tid; i < N; i += KV_THREADS) dO[i] = 0.f;
    float dfr_acc = 0.f;                                    // lane 0 of warp 0
    __syncthreads();
    for (int jb = NB - 1; jb >= 0; jb--) {
        const int t0 = jb * G, cn = min(G, T - t0);
        const size_t so = ((size_t)b * NB + jb) * H + h;
        auto stV = [&](int j) -> const float* { return j == 0 ? buf + so * SV : myseg + (size_t)j * SS; };
        auto stO = [&](int j) -> const float* { return j == 0 ? obuf + so * N : myseg + (size_t)j * SS + SV; };
        for (int j = 0; j + 1 < cn; j++) {                  // replay: slot j + 1 from slot j
            const size_t ix = ((size_t)b * T + t0 + j) * H + h;
            const float *Vp = stV(j), *op = stO(j);
            float* Vn = myseg + (size_t)(j + 1) * SS;
            float* on = Vn + SV;
            for (int n = tid; n < N; n += KV_THREADS) wt[n] = wa[ix * N + n];
            for (int d = tid; d < DV; d += KV_THREADS) vt[d] = ldv(v + ix * DV + d);
            __syncthreads();
            if (warp == 0) {
                keyless_address(wt, op, N, fr, p.hard, z, as, a);
                if (lane == 0) s_f[0] = gate_eff(gate[ix], p.hard_gate);
            }
            __syncthreads();
            const float g = s_f[0];
            for (int n = tid >> 5; n < N; n += KV_THREADS / 32) {  // a warp per row; the row's loads first (global memory)
                const bool hit = a[n] != 0.f;
                const float w = hit ? g * a[n] : 0.f;
                for (int d0 = 0; d0 < DV; d0 += 128) {         // 128 columns at a time, four loads per lane in flight
                    float vx[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) { const int d = d0 + (tid & 31) + 32 * c; vx[c] = d < DV ? Vp[(size_t)n * DV + d] : 0.f; }
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        const int d = d0 + (tid & 31) + 32 * c;
                        if (d < DV) Vn[(size_t)n * DV + d] = hit ? (1.f - w) * vx[c] + w * vt[d] : vx[c];
                    }
                }
            }
            for (int n = tid; n < N; n += KV_THREADS) {
                float x = op[n];
                if (a[n] != 0.f) { const float w = g * a[n]; x = (1.f - w) * x + w; }
                on[n] = x;
            }
            __syncthreads();
        }
        for (int j = cn - 1; j >= 0; j--) {                 // the block in reverse
            const size_t ix = ((size_t)b * T + t0 + j) * H + h;
            const float *Vp = stV(j), *op = stO(j);
            for (int n = tid; n < N; n += KV_THREADS) wt[n] = wa[ix * N + n];
            for (int d = tid; d < DV; d += KV_THREADS) vt[d] = ldv(v + ix * DV + d);
            __syncthreads();
            for (int n = warp; n < N; n += KV_WARPS) {      // dw_n = <v - V_n, dV_n> + (1 - o_n) dO_n
                float a1 = 0.f;
                for (int d = lane; d < DV; d += 32) a1 = fmaf(vt[d] - Vp[(size_t)n * DV + d], dV[(size_t)n * DV + d], a1);
                a1 = warp_sum(a1);
                if (lane == 0) dw[n] = a1 + (1.f - op[n]) * dO[n];
            }
            __syncthreads();
            if (warp == 0) {
                keyless_address(wt, op, N, fr, p.hard, z, as, a);
                const float g = gate_eff(gate[ix], p.hard_gate);
                float dg = 0.f, sa = 0.f;
                for (int n = lane; n < N; n += 32) { dg = fmaf(a[n], dw[n], dg); sa = fmaf(as[n], g * dw[n], sa); }
                dg = warp_sum(dg);
                sa = warp_sum(sa);
                float f1 = 0.f;
                for (int n = lane; n < N; n += 32) {
                    const float zz = as[n] * (g * dw[n] - sa);
                    dz[n] = zz;
                    dwa[ix * N + n] = zz;
                    f1 = fmaf(-op[n], zz, f1);
                }
                f1 = warp_sum(f1);
                if (lane == 0) { dgate[ix] = dg; dfr_acc += f1; s_f[0] = g; }
            }
            __syncthreads();
            const float g = s_f[0];
            for (int d = tid; d < DV; d += KV_THREADS) {    // dv_t = sum_n w_n dV_n (before dV moves to the pre-write side)
                float acc = 0.f;
                for (int n = 0; n < N; n++)
                    if (a[n] != 0.f) acc = fmaf(g * a[n], dV[(size_t)n * DV + d], acc);
                stv(dv + ix * DV + d, acc);
            }
            __syncthreads();
            const bool emit = (j == 0);
            for (int n = tid >> 5; n < N; n += KV_THREADS / 32) {
                const float om = 1.f - g * a[n];
                for (int d = tid & 31; d < DV; d += 32) {
                    const size_t i = (size_t)n * DV + d;
                    float x = om * dV[i];
                    if (emit && dbuf != nullptr) x += dbuf[so * SV + i];
                    dV[i] = x;
                }
            }
            for (int n = tid; n < N; n += KV_THREADS) dO[n] = (1.f - g * a[n]) * dO[n] - frf * dz[n];
            __syncthreads();
        }
    }
    if (tid == 0) part[bh] = dfr_acc;
}

__global__ void __launch_bounds__(256) keyless_finish_kernel(const float* __restrict__ part, int n, float* dfr) {
    __shared__ float s_a[256];
    float a = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) a += part[i];
    s_a[threadIdx.x] = a;
    __syncthreads();
    if (threadIdx.x == 0) {
        a = 0.f;
        for (int i = 0; i < 256; i++) a += s_a[i];          // fixed order: bitwise repeatable
        dfr[0] = a;
    }
}

}  // namespace slotscan

using namespace slotscan;

extern "C" int slotscan_v_check(const slotscan_v_params* p) {
    if (!p) return SLOTSCAN_E_NULL;
    if (p->B < 1 || p->T < 1 || p->H < 1 || p->N < 1 || p->G < 1 || p->DV < 1) return SLOTSCAN_E_SHAPE;
    if ((long long)p->B * p->H > 2147483647LL / 4) return SLOTSCAN_E_SHAPE;
    if (sizeof(float) * keyless_bwd_smem_floats(p->N, p->DV) > 227 * 1024) return SLOTSCAN_E_SHAPE;
    if (p->in_dtype != SLOTSCAN_F32 && p->in_dtype != SLOTSCAN_BF16) return SLOTSCAN_E_DTYPE;
    return SLOTSCAN_OK;
}

extern "C" int slotscan_v_fwd(const slotscan_v_params* p, const void* v, const float* wa, const float* gate,
                              const float* fr, float* buf, float* obuf, int32_t* addr, void* stream) {
    const int rc = slotscan_v_check(p);
    if (rc) return rc;
    if (!v || !wa || !gate || !fr || !buf || !obuf) return SLOTSCAN_E_NULL;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sm = sizeof(float) * keyless_fwd_smem_floats(p->N, p->DV);
    cudaError_t e;
    if (p->in_dtype == SLOTSCAN_F32) {
        auto kern = keyless_fwd_kernel<float>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<p->B * p->H, KV_THREADS, sm, st>>>(*p, (const float*)v, wa, gate, fr, buf, obuf, addr);
    } else {
        auto kern = keyless_fwd_kernel<__nv_bfloat16>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<p->B * p->H, KV_THREADS, sm, st>>>(*p, (const __nv_bfloat16*)v, wa, gate, fr, buf, obuf, addr);
    }
    return (int)cudaGetLastError();
}

extern "C" size_t slotscan_v_bwd_scratch_bytes(const slotscan_v_params* p) {
    if (slotscan_v_check(p)) return 0;
    size_t o = sizeof(float) * (size_t)p->B * p->H * p->G * keyless_state_floats(p->N, p->DV);
    o = (o + 255) & ~(size_t)255;
    return o + sizeof(float) * (size_t)p->B * p->H;
}

extern "C" int slotscan_v_bwd(const slotscan_v_params* p, const void* v, const float* wa, const float* gate,
                              const float* fr, const float* buf, const float* obuf, const float* dbuf, void* scratch,
                              size_t scratch_bytes, void* dv, float* dwa, float* dgate, float* dfr, void* stream) {
    const int rc = slotscan_v_check(p);
    if (rc) return rc;
    if (!v || !wa || !gate || !fr || !buf || !obuf || !scratch || !dv || !dwa || !dgate || !dfr) return SLOTSCAN_E_NULL;
    if (scratch_bytes < slotscan_v_bwd_scratch_bytes(p)) return SLOTSCAN_E_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sm = sizeof(float) * keyless_bwd_smem_floats(p->N, p->DV);
    const size_t seg_bytes = (sizeof(float) * (size_t)p->B * p->H * p->G * keyless_state_floats(p->N, p->DV) + 255) & ~(size_t)255;
    float* seg = (float*)scratch;
    float* part = (float*)((char*)scratch + seg_bytes);
    cudaError_t e;
    if (p->in_dtype == SLOTSCAN_F32) {
        auto kern = keyless_bwd_kernel<float>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<p->B * p->H, KV_THREADS, sm, st>>>(*p, (const float*)v, wa, gate, fr, buf, obuf, dbuf, seg, (float*)dv, dwa, dgate,
                                                  part);
    } else {
        auto kern = keyless_bwd_kernel<__nv_bfloat16>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<p->B * p->H, KV_THREADS, sm, st>>>(*p, (const __nv_bfloat16*)v, wa, gate, fr, buf, obuf, dbuf, seg,
                                                  (__nv_bfloat16*)dv, dwa, dgate, part);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
    keyless_finish_kernel<<<1, 256, 0, st>>>(part, p->B * p->H, dfr);
    return (int)cudaGetLastError();
}
