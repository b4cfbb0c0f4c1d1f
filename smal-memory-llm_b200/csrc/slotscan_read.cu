// Cosine read of the stride-G snapshots, forward.   [reference SharedMixer._read, gqa25/memlm_sh.py:379-397]
//
// Token t reads the snapshot of block t / G only.  Per (sequence, block, head) the G tokens x NQ queries of the block
// share one snapshot:  q is L2-normalised in fp32 (clamp 1e-6),  logit_n = <q, K_n> * kinv_n * sharp  over the VALID rows
// (sharp = the per-(token, head, query) multiplier exp(log_rsel) * exp(C tanh(.)) the caller forms, :383-393), softmax
// over the valid rows (an all-invalid snapshot reads exactly zero, :394), rd = att . V.
//
// One CTA of 4 warps per (sequence, block, head).  Warp 0 compacts the list of valid rows (rows are occupied in index
// order, so with the benchmark's scans ~12 of 192): all work and all memory traffic scale with the valid rows, not
// with N.  Each warp then takes 4 queries at a time: lane = columns (lane, lane + 32, ...), a key row is loaded once
// per warp for its 4 queries, logits are reduced by shuffles, the softmax runs with lane = row, and the value pass
// accumulates 4 queries x columns in registers.  Any dk, dv <= 128.  This first version uses the CUDA cores: with
// M = G * NQ = 16 queries per snapshot the contraction is far below what would need the tensor cores to stay
// HBM-bound when only the valid rows are read.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include "slotscan.h"
#include "slotscan_common.cuh"
#include "slotscan_launch.h"

namespace slotscan {

constexpr int RD_THREADS = 128, RD_WARPS = 4, RD_QPW = 4, RD_MAXC = 4;     // columns per lane: up to 128 / 32

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename Tq, typename Tsn>
__global__ void __launch_bounds__(RD_THREADS) read_fwd_kernel(const slotscan_read_params p, const Tq* __restrict__ qr,
                                                             const float* __restrict__ sharp,
                                                             const Tsn* __restrict__ kbuf, const Tsn* __restrict__ vbuf,
                                                             const float* __restrict__ kinv,
                                                             const uint8_t* __restrict__ valid, Tq* __restrict__ rd,
                                                             const int sparse_only) {
    extern __shared__ __align__(16) float rsm[];
    const int N = p.N, T = p.T, H = p.H, NQ = p.NQ, DK = p.DK, DV = p.DV, G = p.G;
    const int NB = (T + G - 1) / G;
    int* s_rows = reinterpret_cast<int*>(rsm);                 // [N] indices of the valid rows
    float* s_ki = rsm + N;                                     // [N] their kinv
    float* s_sc = rsm + ((2 * N + 3) & ~3);                    // [warps][N][4] logits, then attention weights (16-byte aligned)
    __shared__ int s_nv, s_hv;
    const int so = blockIdx.x;                                 // (b * NB + nb) * H + h
    const int h = so % H, nb = (so / H) % NB, b = so / (H * NB);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (warp == 0) {
        int nv = 0, hv = 0;
        for (int base = 0; base < N; base += 32) {
            const int n = base + lane;
            const bool v = n < N && valid[(size_t)so * N + n] != 0;
            const unsigned bal = __ballot_sync(FULL, v);
            if (v) {
                const int pos = nv + __popc(bal & ((1u << lane) - 1u));
                s_rows[pos] = n;
                s_ki[pos] = kinv[(size_t)so * N + n];
            }
            nv += __popc(bal);
            if (bal) hv = base + 32 - __clz(bal);              // highest valid row + 1
        }
        if (lane == 0) { s_nv = nv; s_hv = hv; }
    }
    __syncthreads();
    const int nv = s_nv;
    if (sparse_only && s_hv > RM_SPARSE_ROWS) return;          // the tensor-core kernel reads this snapshot
    const int t0 = nb * G, tc = min(G, T - t0), M = tc * NQ;   // queries that read this snapshot
    float* sc = s_sc + (size_t)warp * N * RD_QPW;
    const Tsn* Kb = kbuf + (size_t)so * N * DK;
    const Tsn* Vb = vbuf + (size_t)so * N * DV;

    for (int q0 = warp * RD_QPW; q0 < M; q0 += RD_WARPS * RD_QPW) {
        size_t qi[RD_QPW];
        float qv[RD_QPW][RD_MAXC], scale[RD_QPW];
#pragma unroll
        for (int u = 0; u < RD_QPW; u++) {
            const int m = min(q0 + u, M - 1);                  // a short last group repeats its last query
            qi[u] = (((size_t)b * T + t0 + m / NQ) * H + h) * NQ + m % NQ;
            float qq = 0.f;
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) {
                const int col = lane + 32 * c;
                qv[u][c] = col < DK ? ldf(qr + qi[u] * DK + col) : 0.f;
                qq = fmaf(qv[u][c], qv[u][c], qq);
            }
            qq = warp_sum(qq);
            scale[u] = sharp[qi[u]] / fmaxf(sqrtf(qq), 1e-6f);
        }
        // ---- logits over the valid rows ----
        for (int j = 0; j < nv; j++) {
            const Tsn* row = Kb + (size_t)s_rows[j] * DK;
            float kx[RD_MAXC];
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) kx[c] = (lane + 32 * c) < DK ? ldf(row + lane + 32 * c) : 0.f;
            float d[RD_QPW];
#pragma unroll
            for (int u = 0; u < RD_QPW; u++) {
                float a = 0.f;
#pragma unroll
                for (int c = 0; c < RD_MAXC; c++) a = fmaf(kx[c], qv[u][c], a);
                d[u] = warp_sum(a);
            }
            if (lane == 0) {
                const float ki = s_ki[j];
                *reinterpret_cast<float4*>(sc + 4 * j) =
                    make_float4(d[0] * ki * scale[0], d[1] * ki * scale[1], d[2] * ki * scale[2], d[3] * ki * scale[3]);
            }
        }
        __syncwarp();
        // ---- softmax over the valid rows, lane = row ----
#pragma unroll
        for (int u = 0; u < RD_QPW; u++) {
            float m = -INFINITY;
            for (int j = lane; j < nv; j += 32) m = fmaxf(m, sc[4 * j + u]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, off));
            float se = 0.f;
            for (int j = lane; j < nv; j += 32) {
                const float e = expf(sc[4 * j + u] - m);
                sc[4 * j + u] = e;
                se += e;
            }
            se = warp_sum(se);
            const float inv = 1.f / se;
            for (int j = lane; j < nv; j += 32) sc[4 * j + u] *= inv;
        }
        __syncwarp();
        // ---- rd = att . V ----
        float acc[RD_QPW][RD_MAXC];
#pragma unroll
        for (int u = 0; u < RD_QPW; u++)
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) acc[u][c] = 0.f;
        for (int j = 0; j < nv; j++) {
            const Tsn* row = Vb + (size_t)s_rows[j] * DV;
            const float4 a4 = *reinterpret_cast<const float4*>(sc + 4 * j);
            const float a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) {
                const float vx = (lane + 32 * c) < DV ? ldf(row + lane + 32 * c) : 0.f;
#pragma unroll
                for (int u = 0; u < RD_QPW; u++) acc[u][c] = fmaf(a[u], vx, acc[u][c]);
            }
        }
#pragma unroll
        for (int u = 0; u < RD_QPW; u++) {
            if (q0 + u < M) {
#pragma unroll
                for (int c = 0; c < RD_MAXC; c++)
                    if (lane + 32 * c < DV) stf(rd + qi[u] * DV + lane + 32 * c, acc[u][c]);   // nv == 0: exactly zero
            }
        }
        __syncwarp();
    }
}

template <typename Tq, typename Tsn>
static cudaError_t launch_read(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf,
                               const void* vbuf, const float* kinv, const uint8_t* valid, void* rd, cudaStream_t st,
                               int sparse_only = 0) {
    const int NB = (p.T + p.G - 1) / p.G;
    const size_t sm = sizeof(float) * ((size_t)((2 * p.N + 3) & ~3) + (size_t)p.N * RD_WARPS * RD_QPW);
    auto kern = read_fwd_kernel<Tq, Tsn>;
    if (sm > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return e;
    }
    kern<<<p.B * NB * p.H, RD_THREADS, sm, st>>>(p, (const Tq*)qr, sharp, (const Tsn*)kbuf, (const Tsn*)vbuf, kinv, valid,
                                                  (Tq*)rd, sparse_only);
    return cudaGetLastError();
}

}  // namespace slotscan

using namespace slotscan;

extern "C" int slotscan_read_check(const slotscan_read_params* p) {
    if (p == nullptr) return SLOTSCAN_E_NULL;
    if (p->B < 1 || p->T < 1 || p->H < 1 || p->NQ < 1 || p->G < 1) return SLOTSCAN_E_SHAPE;
    if (p->N < 1 || p->N > 2048) return SLOTSCAN_E_SHAPE;                   /* 72 N bytes of shared memory */
    if (p->DK < 1 || p->DK > 32 * RD_MAXC || p->DV < 1 || p->DV > 32 * RD_MAXC) return SLOTSCAN_E_SHAPE;
    if ((long long)p->B * ((p->T + p->G - 1) / p->G) * p->H > 2147483647LL) return SLOTSCAN_E_SHAPE;
    if ((p->q_dtype != SLOTSCAN_F32 && p->q_dtype != SLOTSCAN_BF16) ||
        (p->snap_dtype != SLOTSCAN_F32 && p->snap_dtype != SLOTSCAN_BF16))
        return SLOTSCAN_E_DTYPE;
    return SLOTSCAN_OK;
}

extern "C" int slotscan_read_fwd(const slotscan_read_params* p, const void* qr, const float* sharp, const void* kbuf,
                                 const void* vbuf, const float* kinv, const uint8_t* valid, void* rd, void* stream_) {
    const int rc = slotscan_read_check(p);
    if (rc != SLOTSCAN_OK) return rc;
    if (!qr || !sharp || !kbuf || !vbuf || !kinv || !valid || !rd) return SLOTSCAN_E_NULL;
    cudaStream_t st = (cudaStream_t)stream_;
    cudaError_t e;
    // bf16 with dk = dv in {64, 128}: snapshots with more than RM_SPARSE_ROWS rows in use go through the tensor-core
    // kernel, the others through the CUDA-core kernel; each kernel returns at once on the other's snapshots
    if (read_fwd_mma_try(*p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st, &e)) {
        if (e != cudaSuccess) return (int)e;
        return (int)launch_read<__nv_bfloat16, __nv_bfloat16>(*p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st, 1);
    }
    const bool qb = p->q_dtype == SLOTSCAN_BF16, sb = p->snap_dtype == SLOTSCAN_BF16;
    if (qb && sb) e = launch_read<__nv_bfloat16, __nv_bfloat16>(*p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    else if (qb) e = launch_read<__nv_bfloat16, float>(*p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    else if (sb) e = launch_read<float, __nv_bfloat16>(*p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    else e = launch_read<float, float>(*p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    return (int)e;
}

// ======================================================================================================
// Backward of the read.  [adjoint of memlm_sh.py:379-397; the reference gets it from autograd]
//
// Same CTA as the forward, two phases.  Phase A, per query (4 per warp at a time): recompute the attention over the
// valid rows, da_n = <drd, V_n>, dl_n = att_n (da_n - sum att da), then dsharp = sum dl_n base_n (base = logit / sharp),
// dq through the normalisation, and the per-(query, row) tables att and cf = dl * kinv * sharp in shared memory.
// Phase B, per valid row (rows dealt to warps): dV_n = sum_m att[m][n] drd_m, dK_n = sum_m cf[m][n] qinv_m q_m,
// dkinv_n = sum_m dl base sharp / kinv.  Every sum has a fixed order: results are bitwise repeatable.  kinv is an
// INPUT here (its own gradient dkinv goes back to the writer epilogue, which differentiates rsqrt(nsq)).
// Rows that are not valid get exact zeros.
namespace slotscan {

// zero n elements at p with the whole CTA: 16-byte stores when the block allows it
template <typename T>
__device__ __forceinline__ void zero_fill(T* p, size_t n, int tid) {
    const size_t bytes = n * sizeof(T);
    if (((reinterpret_cast<uintptr_t>(p) | bytes) & 15) == 0) {
        uint4* p4 = reinterpret_cast<uint4*>(p);
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (size_t i = tid; i < bytes / 16; i += RD_THREADS) p4[i] = z;
    } else {
        for (size_t i = tid; i < n; i += RD_THREADS) stf(p + i, 0.f);
    }
}

struct ReadBwdSmem { int rows, ki, qinv, sc, sd, dki, att, cf, total; };
__host__ __device__ inline ReadBwdSmem read_bwd_layout(int N, int M) {
    ReadBwdSmem L;
    const int N4 = (N + 3) & ~3, M4 = (M + 3) & ~3;
    L.rows = 0; L.ki = L.rows + N4; L.qinv = L.ki + N4;
    L.sc = L.qinv + M4;                          // [warps][N][4] base logits, then dl
    L.sd = L.sc + RD_WARPS * N4 * RD_QPW;        // [warps][N][4] da
    L.dki = L.sd + RD_WARPS * N4 * RD_QPW;       // [warps][N] per-warp partial dkinv
    L.att = L.dki + RD_WARPS * N4;               // [M][N]
    L.cf = L.att + M4 * N4;                      // [M][N]
    L.total = L.cf + M4 * N4;
    return L;
}

template <typename Tq, typename Tsn>
__global__ void __launch_bounds__(RD_THREADS) read_bwd_kernel(
    const slotscan_read_params p, const Tq* __restrict__ qr, const float* __restrict__ sharp, const Tsn* __restrict__ kbuf,
    const Tsn* __restrict__ vbuf, const float* __restrict__ kinv, const uint8_t* __restrict__ valid,
    const Tq* __restrict__ drd, Tq* __restrict__ dqr, float* __restrict__ dsharp, Tsn* __restrict__ dkbuf,
    Tsn* __restrict__ dvbuf, float* __restrict__ dkinv, const int sparse_only) {
    extern __shared__ __align__(16) float rsm[];
    const int N = p.N, T = p.T, H = p.H, NQ = p.NQ, DK = p.DK, DV = p.DV, G = p.G;
    const int NB = (T + G - 1) / G, N4 = (N + 3) & ~3;
    const ReadBwdSmem L = read_bwd_layout(N, G * NQ);
    int* s_rows = reinterpret_cast<int*>(rsm + L.rows);
    float* s_ki = rsm + L.ki;
    float* s_qinv = rsm + L.qinv;
    float* s_att = rsm + L.att;
    float* s_cf = rsm + L.cf;
    __shared__ int s_nv, s_hvb;
    const int so = blockIdx.x;
    const int h = so % H, nb = (so / H) % NB, b = so / (H * NB);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (warp == 0) {
        int nv = 0, hv = 0;
        for (int base = 0; base < N; base += 32) {
            const int n = base + lane;
            const bool v = n < N && valid[(size_t)so * N + n] != 0;
            const unsigned bal = __ballot_sync(FULL, v);
            if (v) {
                const int pos = nv + __popc(bal & ((1u << lane) - 1u));
                s_rows[pos] = n;
                s_ki[pos] = kinv[(size_t)so * N + n];
            }
            nv += __popc(bal);
            if (bal) hv = base + 32 - __clz(bal);              // highest valid row + 1
        }
        if (lane == 0) { s_nv = nv; s_hvb = hv; }
    }
    __syncthreads();
    const int nv = s_nv;
    if (sparse_only && s_hvb > RB_SPARSE_ROWS) return;            // the tensor-core kernel takes this snapshot (uniform per CTA)
    // zero the whole block of snapshot gradients first; the valid rows are overwritten after the barrier below
    zero_fill(dkbuf + (size_t)so * N * DK, (size_t)N * DK, tid);
    zero_fill(dvbuf + (size_t)so * N * DV, (size_t)N * DV, tid);
    for (int i = tid; i < N; i += RD_THREADS) dkinv[(size_t)so * N + i] = 0.f;
    __syncthreads();
    const int t0 = nb * G, tc = min(G, T - t0), M = tc * NQ;
    float* sc = rsm + L.sc + (size_t)warp * N4 * RD_QPW;
    float* sd = rsm + L.sd + (size_t)warp * N4 * RD_QPW;
    float* dkw = rsm + L.dki + (size_t)warp * N4;
    const Tsn* Kb = kbuf + (size_t)so * N * DK;
    const Tsn* Vb = vbuf + (size_t)so * N * DV;
    for (int j = lane; j < nv; j += 32) dkw[j] = 0.f;
    __syncwarp();

    // ---------------- phase A: per query ----------------
    for (int q0 = warp * RD_QPW; q0 < M; q0 += RD_WARPS * RD_QPW) {
        size_t qi[RD_QPW];
        float qv[RD_QPW][RD_MAXC], dr[RD_QPW][RD_MAXC], qinv[RD_QPW], sh[RD_QPW];
#pragma unroll
        for (int u = 0; u < RD_QPW; u++) {
            const int m = min(q0 + u, M - 1);
            qi[u] = (((size_t)b * T + t0 + m / NQ) * H + h) * NQ + m % NQ;
            float qq = 0.f;
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) {
                const int col = lane + 32 * c;
                qv[u][c] = col < DK ? ldf(qr + qi[u] * DK + col) : 0.f;
                dr[u][c] = col < DV ? ldf(drd + qi[u] * DV + col) : 0.f;
                qq = fmaf(qv[u][c], qv[u][c], qq);
            }
            qq = warp_sum(qq);
            qinv[u] = 1.f / fmaxf(sqrtf(qq), 1e-6f);
            sh[u] = sharp[qi[u]];
            if (lane == 0 && q0 + u < M) s_qinv[q0 + u] = qinv[u];
        }
        for (int j = 0; j < nv; j++) {
            const Tsn* krow = Kb + (size_t)s_rows[j] * DK;
            const Tsn* vrow = Vb + (size_t)s_rows[j] * DV;
            float kx[RD_MAXC], vx[RD_MAXC];
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) {
                kx[c] = (lane + 32 * c) < DK ? ldf(krow + lane + 32 * c) : 0.f;
                vx[c] = (lane + 32 * c) < DV ? ldf(vrow + lane + 32 * c) : 0.f;
            }
            float d[RD_QPW], da[RD_QPW];
#pragma unroll
            for (int u = 0; u < RD_QPW; u++) {
                float a = 0.f, e = 0.f;
#pragma unroll
                for (int c = 0; c < RD_MAXC; c++) { a = fmaf(kx[c], qv[u][c], a); e = fmaf(vx[c], dr[u][c], e); }
                d[u] = warp_sum(a);
                da[u] = warp_sum(e);
            }
            if (lane == 0) {
                const float ki = s_ki[j];
                *reinterpret_cast<float4*>(sc + 4 * j) =
                    make_float4(d[0] * ki * qinv[0], d[1] * ki * qinv[1], d[2] * ki * qinv[2], d[3] * ki * qinv[3]);
                *reinterpret_cast<float4*>(sd + 4 * j) = make_float4(da[0], da[1], da[2], da[3]);
            }
        }
        __syncwarp();
#pragma unroll
        for (int u = 0; u < RD_QPW; u++) {
            const bool live = q0 + u < M;                    // a repeated last query must not be counted twice
            float m = -INFINITY;
            for (int j = lane; j < nv; j += 32) m = fmaxf(m, sc[4 * j + u] * sh[u]);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL, m, off));
            float se = 0.f, sa = 0.f;
            for (int j = lane; j < nv; j += 32) {
                const float e = expf(sc[4 * j + u] * sh[u] - m);
                se += e;
                sa = fmaf(e, sd[4 * j + u], sa);
            }
            se = warp_sum(se);
            sa = warp_sum(sa) / se;                          // sum att * da
            float ds = 0.f;
            for (int j = lane; j < nv; j += 32) {
                const float base = sc[4 * j + u];
                const float att = expf(base * sh[u] - m) / se;
                const float dl = att * (sd[4 * j + u] - sa);
                ds = fmaf(dl, base, ds);
                const float cf = dl * s_ki[j] * sh[u];
                sc[4 * j + u] = cf;                          // for the dq pass below
                if (live) {
                    s_att[(size_t)(q0 + u) * N4 + j] = att;
                    s_cf[(size_t)(q0 + u) * N4 + j] = cf;
                    dkw[j] += dl * base * sh[u] / s_ki[j];   // d logit / d kinv = logit / kinv
                }
            }
            ds = warp_sum(ds);
            if (lane == 0 && live) dsharp[qi[u]] = ds;
        }
        __syncwarp();
        float acc[RD_QPW][RD_MAXC];
#pragma unroll
        for (int u = 0; u < RD_QPW; u++)
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) acc[u][c] = 0.f;
        for (int j = 0; j < nv; j++) {
            const Tsn* krow = Kb + (size_t)s_rows[j] * DK;
            const float4 c4 = *reinterpret_cast<const float4*>(sc + 4 * j);
            const float cfu[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) {
                const float kx = (lane + 32 * c) < DK ? ldf(krow + lane + 32 * c) : 0.f;
#pragma unroll
                for (int u = 0; u < RD_QPW; u++) acc[u][c] = fmaf(cfu[u], kx, acc[u][c]);
            }
        }
#pragma unroll
        for (int u = 0; u < RD_QPW; u++) {
            float pr = 0.f;
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) pr = fmaf(acc[u][c], qv[u][c] * qinv[u], pr);
            pr = warp_sum(pr);
            if (q0 + u < M) {
#pragma unroll
                for (int c = 0; c < RD_MAXC; c++) {
                    if (lane + 32 * c < DK) {
                        const float qn = qv[u][c] * qinv[u];
                        const float o = qinv[u] >= 1e6f ? qinv[u] * acc[u][c] : qinv[u] * (acc[u][c] - qn * pr);
                        stf(dqr + qi[u] * DK + lane + 32 * c, o);
                    }
                }
            }
        }
        __syncwarp();
    }
    __syncthreads();
    // ---------------- phase B: per valid row ----------------
    for (int j = warp; j < nv; j += RD_WARPS) {
        const int n = s_rows[j];
        float aK[RD_MAXC], aV[RD_MAXC];
#pragma unroll
        for (int c = 0; c < RD_MAXC; c++) aK[c] = aV[c] = 0.f;
        for (int m = 0; m < M; m++) {
            const size_t qm = (((size_t)b * T + t0 + m / NQ) * H + h) * NQ + m % NQ;
            const float at = s_att[(size_t)m * N4 + j], cq = s_cf[(size_t)m * N4 + j] * s_qinv[m];
#pragma unroll
            for (int c = 0; c < RD_MAXC; c++) {
                const int col = lane + 32 * c;
                if (col < DV) aV[c] = fmaf(at, ldf(drd + qm * DV + col), aV[c]);
                if (col < DK) aK[c] = fmaf(cq, ldf(qr + qm * DK + col), aK[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < RD_MAXC; c++) {
            const int col = lane + 32 * c;
            if (col < DK) stf(dkbuf + ((size_t)so * N + n) * DK + col, aK[c]);
            if (col < DV) stf(dvbuf + ((size_t)so * N + n) * DV + col, aV[c]);
        }
        if (lane == 0) {
            float s = 0.f;
            for (int w = 0; w < RD_WARPS; w++) s += rsm[L.dki + (size_t)w * N4 + j];
            dkinv[(size_t)so * N + n] = s;
        }
    }
}

template <typename Tq, typename Tsn>
static cudaError_t launch_read_bwd(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf,
                                   const void* vbuf, const float* kinv, const uint8_t* valid, const void* drd, void* dqr,
                                   float* dsharp, void* dkbuf, void* dvbuf, float* dkinv, int sparse_only, cudaStream_t st) {
    const int NB = (p.T + p.G - 1) / p.G;
    const size_t sm = sizeof(float) * (size_t)read_bwd_layout(p.N, p.G * p.NQ).total;
    auto kern = read_bwd_kernel<Tq, Tsn>;
    if (sm > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return e;
    }
    kern<<<p.B * NB * p.H, RD_THREADS, sm, st>>>(p, (const Tq*)qr, sharp, (const Tsn*)kbuf, (const Tsn*)vbuf, kinv, valid,
                                                  (const Tq*)drd, (Tq*)dqr, dsharp, (Tsn*)dkbuf, (Tsn*)dvbuf, dkinv, sparse_only);
    return cudaGetLastError();
}

}  // namespace slotscan

extern "C" int slotscan_read_bwd(const slotscan_read_params* p, const void* qr, const float* sharp, const void* kbuf,
                                 const void* vbuf, const float* kinv, const uint8_t* valid, const void* drd, void* dqr,
                                 float* dsharp, void* dkbuf, void* dvbuf, float* dkinv, void* stream_) {
    const int rc = slotscan_read_check(p);
    if (rc != SLOTSCAN_OK) return rc;
    if (!qr || !sharp || !kbuf || !vbuf || !kinv || !valid || !drd || !dqr || !dsharp || !dkbuf || !dvbuf || !dkinv)
        return SLOTSCAN_E_NULL;
    if (sizeof(float) * (size_t)read_bwd_layout(p->N, p->G * p->NQ).total > 200 * 1024) return SLOTSCAN_E_TOO_LARGE;
    cudaStream_t st = (cudaStream_t)stream_;
    cudaError_t e = cudaSuccess;
    const bool qb = p->q_dtype == SLOTSCAN_BF16, sb = p->snap_dtype == SLOTSCAN_BF16;
    // bf16 with dk = dv in {64, 128}: snapshots with more than RB_SPARSE_ROWS rows in use go through the tensor-core
    // kernel, the others through the CUDA-core one (each tests the row count itself and leaves the other's alone)
    int sparse_only = 0;
    if (read_bwd_mma_try(*p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, st, &e)) {
        if (e != cudaSuccess) return (int)e;
        sparse_only = 1;
    }
    if (qb && sb) e = launch_read_bwd<__nv_bfloat16, __nv_bfloat16>(*p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, sparse_only, st);
    else if (qb) e = launch_read_bwd<__nv_bfloat16, float>(*p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, 0, st);
    else if (sb) e = launch_read_bwd<float, __nv_bfloat16>(*p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, 0, st);
    else e = launch_read_bwd<float, float>(*p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, 0, st);
    return (int)e;
}
