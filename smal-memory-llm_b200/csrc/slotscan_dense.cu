// General slot scan: every mode of the reference's kv_scan_g that the specialised hard / detached kernels do not
// cover -- the soft address (every candidate row is written by every token), and the hard address whose gradient is
// attached to the stored keys.  [reference: forward gqa25/slotkern_kvt.py:43-119, step adjoint :157-171 and
// gqa25/slotkern_kvg.py:163-200 (stride-G replay backward); definition gqa25/slotkern_kv.py:66-123]
//
// One CTA per (sequence, head).  Forward: keys, values and occupancy resident in shared memory as float32
// (N x (dk + dv) + N floats: 197 KB at 192 x (128 + 128)), four phases per token -- token vectors in, scores (a warp
// per row), address (one warp: mask, argmax, softmax), write (all threads).  The pre-write state goes out every G
// tokens, occupancy included: these snapshots are the checkpoints of the backward.
// Backward: the state adjoints dK, dV, dO are what stays in shared memory; per block of G tokens the forward is
// replayed from the block's snapshot into G state slots of global scratch, then the block is walked in reverse with
// the full step adjoint (store path, softmax adjoint, query normalisation, and -- address attached -- the match
// gradient into the stored keys with the zero below the 1e-6 norm clamp, slotkern_kvg.py:183-188).
// Rows are occupied in index order and occupancy never decreases, so the candidates of a token are exactly rows
// 0 .. first-empty; everything above is zero and is not visited.
//
// These modes are not the training path of the reference run; they are built for completeness of the call signature
// and checked against the same oracle and golden vectors, not tuned.
#include <math.h>
#include <stdio.h>

#include "slotscan_common.cuh"
#include "slotscan_launch.h"

namespace slotscan {

constexpr int DN_THREADS = 256, DN_WARPS = DN_THREADS / 32;

__device__ __forceinline__ float ldtok(const float* p) { return *p; }
__device__ __forceinline__ float ldtok(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void sttok(float* p, float v) { *p = v; }
__device__ __forceinline__ void sttok(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// The address of one token from the scores s[0..lim] and occupancies o[0..lim] (rows 0..lim are the candidates: the
// occupied rows and the first empty one).  Writes afwd[n] (the address the forward uses) and asoft[n] (its softmax);
// warp-collective, every lane returns the same am.  occ_out[n] (may be NULL) receives the penalty factor of row n.
// The scores arrive in double and the softmax runs in double: a soft address feeds every rounding error of a score
// back into every row of the state, token after token, and float32 scores alone put the snapshots several 1e-5 away
// from the float64 definition after a few dozen tokens (the reference's own float32 path shows the same drift).
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(FULL, v, off);
    return v;
}
template <typename TO>
__device__ __forceinline__ int dense_address(double* s, const TO* o, int lim, float fr_t, float eps, int occ_bin,
                                             int hard, float* asoft, float* afwd, float* occ_out) {
    const int lane = threadIdx.x & 31;
    double bz = -INFINITY;
    int bi = BIGI;
    for (int n = lane; n <= lim; n += 32) {
        const TO oc = o[n];
        const double occ = occ_bin ? (oc >= (TO)eps ? 1.0 : 0.0) : (double)oc;
        const double z = s[n] - (double)fr_t * occ;
        if (occ_out != nullptr) occ_out[n] = (float)occ;
        s[n] = z;                                            // z replaces the score until the softmax below
        if (z > bz) { bz = z; bi = n; }                      // ascending n: the first maximum of this lane
    }
    // argmax with first-maximum semantics: the largest z, then the smallest index that holds it
    double zmax = bz;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) zmax = fmax(zmax, __shfl_xor_sync(FULL, zmax, off));
    int am = (int)__reduce_min_sync(FULL, (unsigned)((bi != BIGI && bz == zmax) ? bi : BIGI));
    am = min(am, lim);                                       // NaN scores: stay inside the rows
    double se = 0.0;
    for (int n = lane; n <= lim; n += 32) {
        const double e = exp(s[n] - zmax);
        s[n] = e;
        se += e;
    }
    se = warp_sum_d(se);
    for (int n = lane; n <= lim; n += 32) {
        const float a = (float)(s[n] / se);
        asoft[n] = a;
        afwd[n] = hard ? (n == am ? 1.f : 0.f) : a;
    }
    __syncwarp();
    return am;
}

// first row with o < eps among rows 0..N-1 (N if none); warp-collective
__device__ __forceinline__ int first_empty(const float* o, int N, float eps) {
    const int lane = threadIdx.x & 31;
    int m = BIGI;
    for (int n = lane; n < N; n += 32)
        if (o[n] < eps) { m = n; break; }
    m = (int)__reduce_min_sync(FULL, (unsigned)m);
    return m == BIGI ? N : m;
}

// scores of the candidate rows against q (a warp per row): s[n] = temp * <K_n / max(|K_n|, 1e-6), q / max(|q|, 1e-6)>,
// kinv[n] = 1 / max(|K_n|, 1e-6).  K may be shared or global memory.  Returns qinv (same in every thread).
__device__ __forceinline__ float dense_scores(const float* K, const float* qv, int DK, int lim, float temp, double* s,
                                              float* kinv, float* qnorm_out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double qq = 0.0;
    for (int d = lane; d < DK; d += 32) qq = fma((double)qv[d], (double)qv[d], qq);
    qq = warp_sum_d(qq);
    const double qnorm = sqrt(qq), qinv = 1.0 / fmax(qnorm, 1e-6);
    if (qnorm_out != nullptr) *qnorm_out = (float)qnorm;
    // 8 lanes per row, 4 rows per warp at a time: three shuffle stages per row group instead of five per row
    const int r4 = lane >> 3, l8 = lane & 7;
    for (int base = warp * 4; base <= lim; base += DN_WARPS * 4) {
        const int n = min(base + r4, lim);
        const float* Kn = K + (size_t)n * DK;
        // the row may sit in global memory (the backward's replayed states): every load of the slice is issued before
        // the first use, or each iteration would wait out a memory latency of its own
        float kx[16];
#pragma unroll
        for (int c = 0; c < 16; c++) { const int d = l8 + 8 * c; kx[c] = d < DK ? Kn[d] : 0.f; }
        double kk = 0.0, dt = 0.0;
#pragma unroll
        for (int c = 0; c < 16; c++) {
            const int d = l8 + 8 * c;
            if (d < DK) {
                const double kd = (double)kx[c];
                kk = fma(kd, kd, kk);
                dt = fma(kd, (double)qv[d], dt);
            }
        }
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) {
            kk += __shfl_xor_sync(FULL, kk, off);
            dt += __shfl_xor_sync(FULL, dt, off);
        }
        const double ki = 1.0 / fmax(sqrt(kk), 1e-6);
        if (l8 == 0 && base + r4 <= lim) { s[n] = (dt * ki * qinv) * (double)temp; kinv[n] = (float)ki; }
    }
    return (float)qinv;
}

// ======================================================================================================
template <typename Tin>
__global__ void __launch_bounds__(DN_THREADS) dense_fwd_kernel(
    const slotscan_params p, const int hard, const Tin* __restrict__ k, const Tin* __restrict__ q,
    const Tin* __restrict__ v, const float* __restrict__ gate, const float* __restrict__ fr,
    const float* __restrict__ temp_p, float* __restrict__ kbuf, float* __restrict__ vbuf, float* __restrict__ obuf,
    int* __restrict__ addr, float* __restrict__ kfin, float* __restrict__ vfin, float* __restrict__ ofin) {
    extern __shared__ __align__(16) float dsm_f[];
    const int N = p.N, T = p.T, H = p.H, DK = p.DK, DV = p.DV, G = p.G;
    const int NB = (T + G - 1) / G;
    double* s = reinterpret_cast<double*>(dsm_f);           // [N] scores, then z, then exp(z - zmax)
    double* o = s + ((N + 1) & ~1);                         // [N] occupancy, in double: with the penalty on o itself an
                                                            // error of o enters every later score multiplied by fr
    float* K = dsm_f + 4 * (size_t)((N + 1) & ~1);
    float* V = K + (size_t)N * DK;
    float* a = V + (size_t)N * DV;   // afwd
    float* as = a + N;           // asoft
    float* ki = as + N;
    float* qv = ki + N;
    float* kt = qv + DK;
    float* vt = kt + DK;
    int* s_i = reinterpret_cast<int*>(vt + DV);            // [0] fe, [1] lim of the current token
    float* s_f = reinterpret_cast<float*>(s_i + 4);         // [0] g_eff
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, warp = tid >> 5;
    const float temp = temp_p[0], eps = p.eps;

    for (int i = tid; i < N * DK; i += DN_THREADS) K[i] = 0.f;
    for (int i = tid; i < N * DV; i += DN_THREADS) V[i] = 0.f;
    for (int i = tid; i < N; i += DN_THREADS) o[i] = 0.0;
    if (tid == 0) s_i[0] = 0;
    __syncthreads();
    for (int t = 0; t < T; t++) {
        const size_t ix = ((size_t)b * T + t) * H + h;
        if (t % G == 0) {                                  // the pre-write state, every G tokens
            const size_t so = ((size_t)b * NB + t / G) * H + h;
            for (int i = tid; i < N * DK; i += DN_THREADS) kbuf[so * N * DK + i] = K[i];
            for (int i = tid; i < N * DV; i += DN_THREADS) vbuf[so * N * DV + i] = V[i];
            for (int i = tid; i < N; i += DN_THREADS) obuf[so * N + i] = (float)o[i];
        }
        for (int d = tid; d < DK; d += DN_THREADS) { qv[d] = ldtok(q + ix * DK + d); kt[d] = ldtok(k + ix * DK + d); }
        for (int d = tid; d < DV; d += DN_THREADS) vt[d] = ldtok(v + ix * DV + d);
        __syncthreads();
        const int lim = min(s_i[0], N - 1);                // candidates: rows 0 .. first empty row
        dense_scores(K, qv, DK, lim, temp, s, ki, nullptr);
        __syncthreads();
        if (warp == 0) {
            const float fr_t = p.fr_per_token ? fr[ix] : fr[0];
            const int am = dense_address(s, o, lim, fr_t, eps, p.occ_bin, hard, as, a, nullptr);
            const float g = gate_eff(gate[ix], p.hard_gate);
            for (int n = (tid & 31); n <= lim; n += 32) {
                const double w = (double)g * (double)a[n];
                if (a[n] != 0.f) o[n] = (1.0 - w) * o[n] + w;
            }
            __syncwarp();
            if (tid == 0) {
                int fe = s_i[0];
                if (fe < N && o[fe] >= (double)eps) fe++;  // only the first empty row can become occupied
                s_i[0] = fe;
                s_i[1] = lim;
                s_f[0] = g;
                if (addr != nullptr) addr[ix] = am;
            }
        }
        __syncthreads();
        {
            const float g = s_f[0];
            const int lane = tid & 31;
            for (int n = warp; n <= lim; n += DN_WARPS) {      // a warp per row, lanes over the columns
                const float an = a[n];
                if (an == 0.f) continue;
                const float w = g * an;
                float* Kr = K + (size_t)n * DK;
                float* Vr = V + (size_t)n * DV;
                for (int d = lane; d < DK; d += 32) Kr[d] = (1.f - w) * Kr[d] + w * kt[d];
                for (int d = lane; d < DV; d += 32) Vr[d] = (1.f - w) * Vr[d] + w * vt[d];
            }
        }
        __syncthreads();
    }
    if (kfin != nullptr) for (int i = tid; i < N * DK; i += DN_THREADS) kfin[(size_t)bh * N * DK + i] = K[i];
    if (vfin != nullptr) for (int i = tid; i < N * DV; i += DN_THREADS) vfin[(size_t)bh * N * DV + i] = V[i];
    if (ofin != nullptr) for (int i = tid; i < N; i += DN_THREADS) ofin[(size_t)bh * N + i] = (float)o[i];
}

__host__ __device__ inline size_t dense_fwd_smem_floats(int N, int DK, int DV) {
    return (size_t)N * (DK + DV) + 7 * (size_t)N + 4 + 2 * DK + DV + 32;
}

// ======================================================================================================
__host__ __device__ inline size_t dense_bwd_smem_floats(int N, int DK, int DV) {
    // s (double) 2N + 2, sf N, dK dV, dO as a ki occ dw dz 7N, qv kt dqn 3 DK, vt DV, s_f 32, s_i 8
    return (size_t)N * (DK + DV) + 10 * (size_t)N + 2 + 3 * DK + DV + 96;
}
__host__ __device__ inline size_t dense_state_floats(int N, int DK, int DV) { return (size_t)N * (DK + DV + 1); }

template <typename Tin>
__global__ void __launch_bounds__(DN_THREADS) dense_bwd_kernel(
    const slotscan_params p, const int hard, const int detach, const Tin* __restrict__ k, const Tin* __restrict__ q,
    const Tin* __restrict__ v, const float* __restrict__ gate, const float* __restrict__ fr,
    const float* __restrict__ temp_p, const float* __restrict__ kbuf, const float* __restrict__ vbuf,
    const float* __restrict__ obuf, const float* __restrict__ dkbuf, const float* __restrict__ dvbuf,
    float* __restrict__ seg, Tin* __restrict__ dk, Tin* __restrict__ dq, Tin* __restrict__ dv,
    float* __restrict__ dgate, float* __restrict__ dfr, float* __restrict__ part) {
    extern __shared__ __align__(16) float dsm_f[];
    const int N = p.N, T = p.T, H = p.H, DK = p.DK, DV = p.DV, G = p.G;
    const int NB = (T + G - 1) / G;
    double* s = reinterpret_cast<double*>(dsm_f);           // [N] scores, then z, then exp(z - zmax)
    float* sf = dsm_f + 2 * (size_t)((N + 1) & ~1);         // [N] the scores again as float32, for the adjoint
    float* dK = sf + N;
    float* dV = dK + (size_t)N * DK;
    float* dO = dV + (size_t)N * DV;
    float* as = dO + N;          // asoft
    float* a = as + N;           // afwd
    float* ki = a + N;
    float* occ = ki + N;
    float* dw = occ + N;
    float* dz = dw + N;
    float* qv = dz + N;
    float* kt = qv + DK;
    float* vt = kt + DK;
    float* dqn = vt + DV;
    float* s_f = dqn + DK;       // [0] g_eff [1] qinv [2] qnorm [3] fr_t, [8..15] partial <dqn, qn> per warp
    int* s_i = reinterpret_cast<int*>(s_f + 32);            // [0] lim
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float temp = temp_p[0], eps = p.eps;
    const size_t SK = (size_t)N * DK, SV = (size_t)N * DV, SS = dense_state_floats(N, DK, DV);
    float* myseg = seg + (size_t)bh * G * SS;               // slot j: state before token t0 + j  (slot 0 unused: the snapshot)

    for (size_t i = tid; i < SK; i += DN_THREADS) dK[i] = 0.f;
    for (size_t i = tid; i < SV; i += DN_THREADS) dV[i] = 0.f;
    for (int i = tid; i < N; i += DN_THREADS) dO[i] = 0.f;
    float dtemp_acc = 0.f, dfr_acc = 0.f;                   // lane 0 of warp 0
    __syncthreads();

    for (int jb = NB - 1; jb >= 0; jb--) {
        const int t0 = jb * G, cn = min(G, T - t0);
        const size_t so = ((size_t)b * NB + jb) * H + h;
        // state before token t0 + j
        auto stK = [&](int j) -> const float* { return j == 0 ? kbuf + so * SK : myseg + (size_t)j * SS; };
        auto stV = [&](int j) -> const float* { return j == 0 ? vbuf + so * SV : myseg + (size_t)j * SS + SK; };
        auto stO = [&](int j) -> const float* { return j == 0 ? obuf + so * N : myseg + (size_t)j * SS + SK + SV; };
        // ---- replay the block forward: slot j + 1 from slot j ----
        for (int j = 0; j + 1 < cn; j++) {
            const int t = t0 + j;
            const size_t ix = ((size_t)b * T + t) * H + h;
            const float *Kp = stK(j), *Vp = stV(j), *op = stO(j);
            float* Kn = myseg + (size_t)(j + 1) * SS;
            float* Vn = Kn + SK;
            float* on = Vn + SV;
            for (int d = tid; d < DK; d += DN_THREADS) { qv[d] = ldtok(q + ix * DK + d); kt[d] = ldtok(k + ix * DK + d); }
            for (int d = tid; d < DV; d += DN_THREADS) vt[d] = ldtok(v + ix * DV + d);
            if (warp == 0) {
                const int fe = first_empty(op, N, eps);
                if (lane == 0) s_i[0] = min(fe, N - 1);
            }
            __syncthreads();
            const int lim = s_i[0];
            dense_scores(Kp, qv, DK, lim, temp, s, ki, nullptr);
            __syncthreads();
            if (warp == 0) {
                const float fr_t = p.fr_per_token ? fr[ix] : fr[0];
                dense_address(s, op, lim, fr_t, eps, p.occ_bin, hard, as, a, nullptr);
                if (lane == 0) s_f[0] = gate_eff(gate[ix], p.hard_gate);
            }
            __syncthreads();
            const float g = s_f[0];
            for (int n = warp; n < N; n += DN_WARPS) {          // a warp per row, lanes over the columns
                const bool hit = n <= lim && a[n] != 0.f;
                const float w = hit ? g * a[n] : 0.f;
                const float *Kr = Kp + (size_t)n * DK, *Vr = Vp + (size_t)n * DV;
                float *Ko = Kn + (size_t)n * DK, *Vo = Vn + (size_t)n * DV;
                float kx[4], vx[4];
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int d = lane + 32 * c;
                    kx[c] = d < DK ? Kr[d] : 0.f;
                    vx[c] = d < DV ? Vr[d] : 0.f;
                }
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int d = lane + 32 * c;
                    if (d < DK) Ko[d] = hit ? (1.f - w) * kx[c] + w * kt[d] : kx[c];
                    if (d < DV) Vo[d] = hit ? (1.f - w) * vx[c] + w * vt[d] : vx[c];
                }
            }
            for (int n = tid; n < N; n += DN_THREADS) {
                float x = op[n];
                if (n <= lim && a[n] != 0.f) { const float w = g * a[n]; x = (1.f - w) * x + w; }
                on[n] = x;
            }
            __syncthreads();                                 // slot j + 1 complete (block-wide visibility of global writes)
        }
        // ---- walk the block in reverse ----
        for (int j = cn - 1; j >= 0; j--) {
            const int t = t0 + j;
            const size_t ix = ((size_t)b * T + t) * H + h;
            const float *Kp = stK(j), *Vp = stV(j), *op = stO(j);
            for (int d = tid; d < DK; d += DN_THREADS) { qv[d] = ldtok(q + ix * DK + d); kt[d] = ldtok(k + ix * DK + d); }
            for (int d = tid; d < DV; d += DN_THREADS) vt[d] = ldtok(v + ix * DV + d);
            if (warp == 0) {
                const int fe = first_empty(op, N, eps);
                if (lane == 0) s_i[0] = min(fe, N - 1);
            }
            __syncthreads();
            const int lim = s_i[0];
            float qnorm;
            const float qinv = dense_scores(Kp, qv, DK, lim, temp, s, ki, &qnorm);
            // dw_n = <k_t - K_n, dK_n> + <v_t - V_n, dV_n> + (1 - o_n) dO_n      (slotkern_kvg.py:165)
            for (int n = warp; n <= lim; n += DN_WARPS) {
                float kx[4], vx[4];                          // all loads of the row first (global memory: see dense_scores)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int d = lane + 32 * c;
                    kx[c] = d < DK ? Kp[(size_t)n * DK + d] : 0.f;
                    vx[c] = d < DV ? Vp[(size_t)n * DV + d] : 0.f;
                }
                float a1 = 0.f;
#pragma unroll
                for (int c = 0; c < 4; c++) { const int d = lane + 32 * c; if (d < DK) a1 = fmaf(kt[d] - kx[c], dK[(size_t)n * DK + d], a1); }
#pragma unroll
                for (int c = 0; c < 4; c++) { const int d = lane + 32 * c; if (d < DV) a1 = fmaf(vt[d] - vx[c], dV[(size_t)n * DV + d], a1); }
                a1 = warp_sum(a1);
                if (lane == 0) dw[n] = a1 + (1.f - op[n]) * dO[n];
            }
            __syncthreads();
            if (warp == 0) {
                const float fr_t = p.fr_per_token ? fr[ix] : fr[0];
                for (int n = lane; n <= lim; n += 32) sf[n] = (float)s[n];      // the address pass overwrites s
                dense_address(s, op, lim, fr_t, eps, p.occ_bin, hard, as, a, occ);
                const float g = gate_eff(gate[ix], p.hard_gate);
                float dg = 0.f, sa = 0.f;
                for (int n = lane; n <= lim; n += 32) { dg = fmaf(a[n], dw[n], dg); sa = fmaf(as[n], g * dw[n], sa); }
                dg = warp_sum(dg);
                sa = warp_sum(sa);
                float f1 = 0.f, f2 = 0.f;
                for (int n = lane; n <= lim; n += 32) {
                    const float z = as[n] * (g * dw[n] - sa);          // softmax adjoint (slotkern_kvg.py:170-179)
                    dz[n] = z;
                    f1 = fmaf(-occ[n], z, f1);
                    f2 = fmaf(z, sf[n], f2);
                }
                f1 = warp_sum(f1);
                f2 = warp_sum(f2);
                if (lane == 0) {
                    dgate[ix] = dg;
                    if (p.fr_per_token) dfr[ix] = f1; else dfr_acc += f1;
                    dtemp_acc += f2 / temp;
                    s_f[0] = g; s_f[1] = qinv; s_f[2] = qnorm; s_f[3] = fr_t;
                }
            }
            __syncthreads();
            const float g = s_f[0], fr_t = s_f[3];
            // token gradients through the store path, and the raw query gradient: one thread per output column
            float my_dqn = 0.f;
            if (tid < DK) {
                const int d = tid;
                float acc = 0.f, qacc = 0.f;
                for (int n0 = 0; n0 <= lim; n0 += 8) {          // eight rows of the (global) state in flight at a time
                    float kp[8];
#pragma unroll
                    for (int u = 0; u < 8; u++) kp[u] = (n0 + u <= lim) ? Kp[(size_t)(n0 + u) * DK + d] : 0.f;
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        const int n = n0 + u;
                        if (n <= lim) {
                            if (a[n] != 0.f) acc = fmaf(g * a[n], dK[(size_t)n * DK + d], acc);
                            if (dz[n] != 0.f) qacc = fmaf(dz[n] * temp, kp[u] * ki[n], qacc);
                        }
                    }
                }
                sttok(dk + ix * DK + d, acc);
                my_dqn = qacc;
                dqn[d] = qacc;
            }
            if (tid >= DN_THREADS - DV) {                    // the last DV threads take the value columns
                const int d = tid - (DN_THREADS - DV);
                float acc = 0.f;
                for (int n = 0; n <= lim; n++)
                    if (a[n] != 0.f) acc = fmaf(g * a[n], dV[(size_t)n * DV + d], acc);
                sttok(dv + ix * DV + d, acc);
            }
            {   // <dqn, qn> over the key columns, fixed order
                float pr = (tid < DK) ? my_dqn * (qv[tid] * qinv) : 0.f;
                pr = warp_sum(pr);
                if (lane == 0) s_f[8 + warp] = pr;
            }
            __syncthreads();
            if (tid < DK) {
                float prq = 0.f;
                for (int w = 0; w < DN_WARPS; w++) prq += s_f[8 + w];
                const float qn = qv[tid] * qinv;
                const float gq = (qnorm < 1e-6f) ? qinv * my_dqn : qinv * (my_dqn - qn * prq);
                sttok(dq + ix * DK + tid, gq);
            }
            // ---- carry the state adjoints to the pre-write side (slotkern_kvg.py:183-196) ----
            const bool emit = (j == 0);
            for (int n = warp; n <= lim; n += DN_WARPS) {        // a warp per row, lanes over the columns
                const float om = 1.f - g * a[n];
                const bool match = !detach && dz[n] != 0.f && ki[n] < 1e6f;   // the key-match gradient; zero under the norm clamp
                const float kin = ki[n], dzn = dz[n], sfn = sf[n];
                float kx[4], gk[4], gv[4];                   // global loads of the row first
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int d = lane + 32 * c;
                    kx[c] = (match && d < DK) ? Kp[(size_t)n * DK + d] : 0.f;
                    gk[c] = (emit && dkbuf != nullptr && d < DK) ? dkbuf[so * SK + (size_t)n * DK + d] : 0.f;
                    gv[c] = (emit && dvbuf != nullptr && d < DV) ? dvbuf[so * SV + (size_t)n * DV + d] : 0.f;
                }
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int d = lane + 32 * c;
                    if (d < DK) {
                        const size_t i = (size_t)n * DK + d;
                        float x = om * dK[i];
                        if (emit && dkbuf != nullptr) x += gk[c];
                        if (match) {
                            const float kh = kx[c] * kin;
                            x = fmaf(kin * dzn, temp * (qv[d] * qinv) - kh * sfn, x);
                        }
                        dK[i] = x;
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const int d = lane + 32 * c;
                    if (d < DV) {
                        const size_t i = (size_t)n * DV + d;
                        float x = om * dV[i];
                        if (emit && dvbuf != nullptr) x += gv[c];
                        dV[i] = x;
                    }
                }
            }
            for (int n = tid; n <= lim; n += DN_THREADS)
                dO[n] = (1.f - g * a[n]) * dO[n] - (p.occ_bin ? 0.f : fr_t * dz[n]);
            __syncthreads();
        }
    }
    if (tid == 0) {
        part[bh] = dtemp_acc;
        part[(size_t)p.B * H + bh] = dfr_acc;
    }
}

__global__ void __launch_bounds__(256) dense_finish_kernel(const float* __restrict__ part, int n, int fr_per_token,
                                                           float* dtemp, float* dfr) {
    __shared__ float s_a[256], s_c[256];
    float a = 0.f, c = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { a += part[i]; c += part[n + i]; }
    s_a[threadIdx.x] = a; s_c[threadIdx.x] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        a = 0.f; c = 0.f;
        for (int i = 0; i < 256; i++) { a += s_a[i]; c += s_c[i]; }      // fixed order: bitwise repeatable
        dtemp[0] = a;
        if (!fr_per_token) dfr[0] = c;
    }
}
template <typename Tin>
__global__ void dense_add_into_kernel(Tin* __restrict__ dst, const Tin* __restrict__ src, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        sttok(dst + i, ldtok(dst + i) + ldtok(src + i));
}

constexpr size_t DENSE_SMEM_CAP = 227 * 1024;

}  // namespace slotscan

using namespace slotscan;

extern "C" int slotscan_dense_check(const slotscan_dense_params* p) {
    if (!p) return SLOTSCAN_E_NULL;
    const slotscan_params& b = p->base;
    if (b.B < 1 || b.T < 1 || b.H < 1 || b.N < 1 || b.G < 1) return SLOTSCAN_E_SHAPE;
    if (b.DK < 1 || b.DK > 128 || b.DV < 1 || b.DV > 128) return SLOTSCAN_E_SHAPE;
    if ((long long)b.B * b.H > 2147483647LL / 4) return SLOTSCAN_E_SHAPE;
    if (sizeof(float) * dense_bwd_smem_floats(b.N, b.DK, b.DV) > DENSE_SMEM_CAP) return SLOTSCAN_E_SHAPE;
    if (b.in_dtype != SLOTSCAN_F32 && b.in_dtype != SLOTSCAN_BF16) return SLOTSCAN_E_DTYPE;
    if (b.snap_dtype != SLOTSCAN_F32) return SLOTSCAN_E_DTYPE;       /* the snapshots are the backward's checkpoints */
    return SLOTSCAN_OK;
}

extern "C" int slotscan_dense_fwd(const slotscan_dense_params* p, const void* k, const void* q, const void* v,
                                  const float* gate, const float* fr, const float* temp, float* kbuf, float* vbuf,
                                  float* obuf, int32_t* addr, float* kfin, float* vfin, float* ofin, void* stream) {
    const int rc = slotscan_dense_check(p);
    if (rc) return rc;
    if (!k || !v || !gate || !fr || !temp || !kbuf || !vbuf || !obuf) return SLOTSCAN_E_NULL;
    const slotscan_params& b = p->base;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sm = sizeof(float) * dense_fwd_smem_floats(b.N, b.DK, b.DV);
    cudaError_t e;
    if (b.in_dtype == SLOTSCAN_F32) {
        auto kern = dense_fwd_kernel<float>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<b.B * b.H, DN_THREADS, sm, st>>>(b, p->hard, (const float*)k, (const float*)(q ? q : k), (const float*)v, gate,
                                                fr, temp, kbuf, vbuf, obuf, addr, kfin, vfin, ofin);
    } else {
        typedef __nv_bfloat16 bf;
        auto kern = dense_fwd_kernel<bf>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<b.B * b.H, DN_THREADS, sm, st>>>(b, p->hard, (const bf*)k, (const bf*)(q ? q : k), (const bf*)v, gate, fr, temp,
                                                kbuf, vbuf, obuf, addr, kfin, vfin, ofin);
    }
    return (int)cudaGetLastError();
}

extern "C" size_t slotscan_dense_bwd_scratch_bytes(const slotscan_dense_params* p) {
    if (slotscan_dense_check(p)) return 0;
    const slotscan_params& b = p->base;
    size_t o = sizeof(float) * (size_t)b.B * b.H * b.G * dense_state_floats(b.N, b.DK, b.DV);
    o = (o + 255) & ~(size_t)255;
    return o + sizeof(float) * 2 * (size_t)b.B * b.H;
}

extern "C" int slotscan_dense_bwd(const slotscan_dense_params* p, const void* k, const void* q, const void* v,
                                  const float* gate, const float* fr, const float* temp, const float* kbuf,
                                  const float* vbuf, const float* obuf, const float* dkbuf, const float* dvbuf,
                                  void* scratch, size_t scratch_bytes, void* dk, void* dq, void* dv, float* dgate,
                                  float* dfr, float* dtemp, void* stream) {
    const int rc = slotscan_dense_check(p);
    if (rc) return rc;
    if (!k || !v || !gate || !fr || !temp || !kbuf || !vbuf || !obuf || !scratch || !dk || !dq || !dv || !dgate || !dfr ||
        !dtemp)
        return SLOTSCAN_E_NULL;
    if (scratch_bytes < slotscan_dense_bwd_scratch_bytes(p)) return SLOTSCAN_E_SHAPE;
    const slotscan_params& b = p->base;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t sm = sizeof(float) * dense_bwd_smem_floats(b.N, b.DK, b.DV);
    const size_t seg_bytes = (sizeof(float) * (size_t)b.B * b.H * b.G * dense_state_floats(b.N, b.DK, b.DV) + 255) & ~(size_t)255;
    float* seg = (float*)scratch;
    float* part = (float*)((char*)scratch + seg_bytes);
    cudaError_t e;
    if (b.in_dtype == SLOTSCAN_F32) {
        auto kern = dense_bwd_kernel<float>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<b.B * b.H, DN_THREADS, sm, st>>>(b, p->hard, p->detach_addr, (const float*)k, (const float*)(q ? q : k),
                                                (const float*)v, gate, fr, temp, kbuf, vbuf, obuf, dkbuf, dvbuf, seg,
                                                (float*)dk, (float*)dq, (float*)dv, dgate, dfr, part);
    } else {
        typedef __nv_bfloat16 bf;
        auto kern = dense_bwd_kernel<bf>;
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return (int)e;
        kern<<<b.B * b.H, DN_THREADS, sm, st>>>(b, p->hard, p->detach_addr, (const bf*)k, (const bf*)(q ? q : k), (const bf*)v,
                                                gate, fr, temp, kbuf, vbuf, obuf, dkbuf, dvbuf, seg, (bf*)dk, (bf*)dq, (bf*)dv,
                                                dgate, dfr, part);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
    dense_finish_kernel<<<1, 256, 0, st>>>(part, b.B * b.H, b.fr_per_token, dtemp, dfr);
    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
    if (q == nullptr) {           // the search query is the stored key: both gradient paths land in dk
        const size_t n = (size_t)b.B * b.T * b.H * b.DK;
        if (b.in_dtype == SLOTSCAN_F32) dense_add_into_kernel<float><<<592, 256, 0, st>>>((float*)dk, (const float*)dq, n);
        else dense_add_into_kernel<__nv_bfloat16><<<592, 256, 0, st>>>((__nv_bfloat16*)dk, (const __nv_bfloat16*)dq, n);
        e = cudaGetLastError();
    }
    return (int)e;
}
