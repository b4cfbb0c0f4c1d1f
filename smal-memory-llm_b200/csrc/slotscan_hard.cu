// Hard-address slot scan for sm_100a: forward and backward of the reference's training mode
// (hard argmax address, address gradient detached from the stored keys).
//
// Decomposition (the row a token writes is the only sequential decision):
//   addr_fwd_kernel    one CTA per (sequence, head), sequential in t: keys + occupancy resident in shared
//                      memory, cosine score against the rows touched so far, first-free-row rule, argmax.
//                      Emits only the address log.                       [reference addr_fwd, slotkern_cuda.py:72-174]
//   replay_rows_kernel row-parallel, no barriers in the token loop: replays each key / value row from the log,
//                      emits the stride-G snapshots, the undo log and the final state.   [val_fwd :178-206]
//   rows_bwd_kernel    row-parallel reverse scan: undoes rows from the log, carries dK / dV, emits dk / dv and the
//                      table D[t,n] = <x_t - X_n, dX_n>.                                    [rows_bwd :209-261]
//   addr_bwd_kernel    one CTA per (sequence, head), reverse in t: rebuilds the soft address from the restored
//                      keys, softmax adjoint -> dgate, dfr, dtemp, dq.                       [addr_bwd :264-443]
// Rows are taken in index order (only occupied rows and the lowest free row are candidates), so every row above
// the highest row touched so far is exactly zero: all four kernels skip those rows.
#include <math.h>
#include <stdio.h>

#include <mutex>
#include <vector>

#include "slotscan_common.cuh"
#include "slotscan_addr_fwd.cuh"
#include "slotscan_addr_bwd.cuh"

namespace slotscan {

constexpr int SEQ_THREADS = 256;              // sequential kernels: 8 warps per (sequence, head)
constexpr int SEQ_WARPS = SEQ_THREADS / 32;
constexpr int ROW_THREADS = 256;              // row-parallel kernels
constexpr int LOG_CHUNK = 2048;               // tokens of (address, gate) log staged in shared memory at a time

// ======================================================================================================
// addr_fwd: the sequential address scan.
// Shared memory: K[N][DK] f32 | o[N] | kinv[N].  One warp owns the rows n = warp, warp + 8, ...; lane l holds
// columns 4l..4l+3 of a row (DK <= 128).
template <typename Tin>
__global__ void __launch_bounds__(SEQ_THREADS) addr_fwd_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const Tin* __restrict__ k, const float* __restrict__ gate,
    const float* __restrict__ fr, const float* __restrict__ temp_p, int* __restrict__ am_out,
    float* __restrict__ oold, float* __restrict__ ofin, int* __restrict__ tfirst) {
    extern __shared__ __align__(16) float smem[];
    const int N = p.N, DK = p.DK, T = p.T, H = p.H;
    float* K = smem;
    float* o = K + (size_t)N * DK;
    float* kinv = o + N;
    __shared__ float x_bz[2][SEQ_WARPS], x_ez[2][SEQ_WARPS];
    __shared__ int x_bi[2][SEQ_WARPS], x_ei[2][SEQ_WARPS];

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = lane * 4;
    const bool act = col < DK;
    for (int i = tid; i < N * DK; i += SEQ_THREADS) K[i] = 0.f;
    for (int i = tid; i < N; i += SEQ_THREADS) {
        o[i] = 0.f;
        kinv[i] = 1e6f;                                  // 1 / max(|0|, 1e-6)
        tfirst[(size_t)bh * N + i] = (i == 0) ? 0 : T;
    }
    __syncthreads();
    const float temp = temp_p[0], eps = p.eps;
    float frv = p.fr_per_token ? 0.f : fr[0];
    int hw = -1;                                         // highest row touched so far
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 qa = zero4, ka = zero4;
    float ga, fa = 0.f;
    {
        const size_t ix = ((size_t)b * T) * H + h;
        if (act) { qa = ld4(q + ix * DK + col); ka = ld4(k + ix * DK + col); }
        ga = gate[ix];
        if (p.fr_per_token) fa = fr[ix];
    }
    int par = 0;
    for (int t = 0; t < T; t++) {
        const size_t ix = ((size_t)b * T + t) * H + h;
        const float4 qt = qa, kt = ka;
        const float g = gate_eff(ga, p.hard_gate);
        if (p.fr_per_token) frv = fa;
        if (t + 1 < T) {                                 // next token's loads fly during this step
            const size_t ix2 = ix + H;
            if (act) { qa = ld4(q + ix2 * DK + col); ka = ld4(k + ix2 * DK + col); }
            ga = gate[ix2];
            if (p.fr_per_token) fa = fr[ix2];
        }
        const float qq = warp_sum(dot4(qt, qt));
        const float qinv = 1.f / fmaxf(sqrtf(qq), 1e-6f);
        const float4 qn = make_float4(qt.x * qinv, qt.y * qinv, qt.z * qinv, qt.w * qinv);
        const int lim = min(hw + 1, N - 1);
        float bz = -INFINITY, ez = 0.f;
        int bi = BIGI, ei = BIGI;
        for (int n = warp; n <= lim; n += SEQ_WARPS) {
            const float4 Kn = act ? ld4(K + (size_t)n * DK + col) : zero4;
            const float ki = kinv[n];
            // normalise first, then dot (slotkern_kvt.py:86-97)
            const float dt = warp_sum((Kn.x * ki) * qn.x + (Kn.y * ki) * qn.y + (Kn.z * ki) * qn.z + (Kn.w * ki) * qn.w);
            const float s = temp * dt, oc = o[n];
            const float z = p.occ_bin ? (s - frv * (oc >= eps ? 1.f : 0.f)) : (s - frv * oc);
            if (oc < eps) { if (n < ei) { ei = n; ez = z; } }      // only the LOWEST free row competes
            else best(bz, bi, z, n);
        }
        if (lane == 0) { x_bz[par][warp] = bz; x_bi[par][warp] = bi; x_ei[par][warp] = ei; x_ez[par][warp] = ez; }
        __syncthreads();
        bz = -INFINITY; bi = BIGI; ei = BIGI; ez = 0.f;
#pragma unroll
        for (int w = 0; w < SEQ_WARPS; w++) {
            best(bz, bi, x_bz[par][w], x_bi[par][w]);
            if (x_ei[par][w] < ei) { ei = x_ei[par][w]; ez = x_ez[par][w]; }
        }
        par ^= 1;
        int am = bi;
        if (ei != BIGI && (bi == BIGI || ez > bz || (ez == bz && ei < bi))) am = ei;
        if (am > hw) {
            hw = am;
            if (tid == 0 && am + 1 < N) tfirst[(size_t)bh * N + am + 1] = t + 1;
        }
        if ((am % SEQ_WARPS) == warp) {                  // the owner warp writes the row; nobody else reads it
            const float omw = 1.f - g, oc = o[am];
            float4 Kn = act ? ld4(K + (size_t)am * DK + col) : zero4;
            Kn.x = blend(Kn.x, kt.x, g, omw); Kn.y = blend(Kn.y, kt.y, g, omw);
            Kn.z = blend(Kn.z, kt.z, g, omw); Kn.w = blend(Kn.w, kt.w, g, omw);
            if (act) st4(K + (size_t)am * DK + col, Kn);
            const float nsq = warp_sum(dot4(Kn, Kn));
            if (lane == 0) {
                am_out[ix] = am;
                oold[ix] = oc;
                kinv[am] = 1.f / fmaxf(sqrtf(nsq), 1e-6f);
                o[am] = __fmaf_rn(omw, oc, g);
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int i = tid; i < N; i += SEQ_THREADS) ofin[(size_t)bh * N + i] = o[i];
}

// ======================================================================================================
// replay_rows: one group of LPR = D/8 lanes per row, 8 elements per lane in registers; grid (B*H, row tiles).
// Runs once for the keys (x = k, D = DK) and once for the values (x = v, D = DV).
template <int D, typename Tin, typename Tsn>
__global__ void __launch_bounds__(ROW_THREADS) replay_rows_kernel(
    const slotscan_params p, const Tin* __restrict__ x, const float* __restrict__ gate, const int* __restrict__ am,
    Tsn* __restrict__ xbuf, float* __restrict__ xold, float* __restrict__ xfin) {
    constexpr int LPR = D / 8, RPB = ROW_THREADS / LPR;
    __shared__ int s_am[LOG_CHUNK];
    __shared__ float s_g[LOG_CHUNK];
    const int N = p.N, T = p.T, H = p.H, G = p.G;
    const int NB = (T + G - 1) / G;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, r = tid / LPR, c = tid % LPR, n = blockIdx.y * RPB + r;
    const bool live = n < N;
    float X[8];
#pragma unroll
    for (int j = 0; j < 8; j++) X[j] = 0.f;
    for (int t0 = 0; t0 < T; t0 += LOG_CHUNK) {
        const int tc = min(LOG_CHUNK, T - t0);
        __syncthreads();
        for (int i = tid; i < tc; i += ROW_THREADS) {
            const size_t ix = ((size_t)b * T + t0 + i) * H + h;
            s_am[i] = am[ix];
            s_g[i] = gate_eff(gate[ix], p.hard_gate);
        }
        __syncthreads();
        if (!live) continue;
        for (int i = 0; i < tc; i++) {
            const int t = t0 + i;
            if (t % G == 0)
                st8(xbuf + (((size_t)b * NB + t / G) * H + h) * N * D + (size_t)n * D + c * 8, X);
            if (s_am[i] == n) {
                const size_t ix = ((size_t)b * T + t) * H + h;
                const float g = s_g[i], omw = 1.f - g;
                float xv[8];
                ld8(xv, x + ix * D + c * 8);
                st8(xold + ix * D + c * 8, X);
#pragma unroll
                for (int j = 0; j < 8; j++) X[j] = blend(X[j], xv[j], g, omw);
            }
        }
    }
    if (live) st8(xfin + ((size_t)bh * N + n) * D + c * 8, X);
}

// ======================================================================================================
// rows_bwd: reverse scan per row.  dX_n <- (1-w) dX_n + dxbuf;  dx_t = g dX_am;  D[t,n] (+)= <x_t - X_n, dX_n>.
// A row stops at tfirst[n]: before that token it is neither written nor a candidate, so nothing reads its D.
template <int D, typename Tin, typename Tsn, bool ACCUM>
__global__ void __launch_bounds__(ROW_THREADS) rows_bwd_kernel(
    const slotscan_params p, const Tin* __restrict__ x, const float* __restrict__ gate, const int* __restrict__ am,
    const float* __restrict__ xold, const float* __restrict__ xfin, const int* __restrict__ tfirst,
    const Tsn* __restrict__ dxbuf, Tin* __restrict__ dx, float* __restrict__ Dn) {
    constexpr int LPR = D / 8, RPB = ROW_THREADS / LPR;
    __shared__ int s_am[LOG_CHUNK];
    __shared__ float s_g[LOG_CHUNK];
    const int N = p.N, T = p.T, H = p.H, G = p.G;
    const int NB = (T + G - 1) / G;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, r = tid / LPR, c = tid % LPR, n0 = blockIdx.y * RPB + r;
    const bool live = n0 < N;
    const int n = live ? n0 : 0;          // dead rows still run the shuffles; they read row 0 and write nothing
    const int tstop = live ? tfirst[(size_t)bh * N + n] : T;
    float X[8], dX[8];
    ld8(X, xfin + ((size_t)bh * N + n) * D + c * 8);
#pragma unroll
    for (int j = 0; j < 8; j++) dX[j] = 0.f;
    // chunks of the log, last chunk first
    const int nchunk = (T + LOG_CHUNK - 1) / LOG_CHUNK;
    for (int ck = nchunk - 1; ck >= 0; ck--) {
        const int t0 = ck * LOG_CHUNK, tc = min(LOG_CHUNK, T - t0);
        __syncthreads();
        for (int i = tid; i < tc; i += ROW_THREADS) {
            const size_t ix = ((size_t)b * T + t0 + i) * H + h;
            s_am[i] = am[ix];
            s_g[i] = gate_eff(gate[ix], p.hard_gate);
        }
        __syncthreads();
        // every lane of a warp must run the same number of shuffle steps: the warp's stop is its lowest row's
        const int wstop = __reduce_min_sync(FULL, tstop);
        for (int i = tc - 1; i >= 0; i--) {
            const int t = t0 + i;
            if (t < wstop) break;
            const size_t ix = ((size_t)b * T + t) * H + h;
            const bool on = t >= tstop;
            const bool hit = on && (s_am[i] == n);
            float xv[8];
            ld8(xv, x + ix * D + c * 8);
            if (hit) ld8(X, xold + ix * D + c * 8);
            float pacc = 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) pacc += (xv[j] - X[j]) * dX[j];
            pacc = group_sum<LPR>(pacc);
            if (on && c == 0) {
                float* dst = Dn + ((size_t)bh * T + t) * N + n;
                if (ACCUM) *dst += pacc; else *dst = pacc;
            }
            if (hit) {
                const float g = s_g[i], omw = 1.f - g;
                float a[8];
#pragma unroll
                for (int j = 0; j < 8; j++) { a[j] = g * dX[j]; dX[j] = omw * dX[j]; }
                st8(dx + ix * D + c * 8, a);
            }
            if (on && dxbuf != nullptr && t % G == 0) {
                float a[8];
                ld8(a, dxbuf + (((size_t)b * NB + t / G) * H + h) * N * D + (size_t)n * D + c * 8);
#pragma unroll
                for (int j = 0; j < 8; j++) dX[j] += a[j];
            }
        }
    }
}

// ======================================================================================================
// addr_bwd: reverse scan of the address.  Shared memory: K[N][DK] | o[N] | kinv[N] | dO[N] | sv[N] | zv[N] | dwv[N]
//           | tf[N] (int) | rq[2][SEQ_WARPS][DK].
template <typename Tin>
__global__ void __launch_bounds__(SEQ_THREADS) addr_bwd_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const float* __restrict__ gate, const float* __restrict__ fr,
    const float* __restrict__ temp_p, const int* __restrict__ am, const float* __restrict__ kold,
    const float* __restrict__ oold, const float* __restrict__ kfin, const float* __restrict__ ofin,
    const int* __restrict__ tfirst, const float* __restrict__ Din, Tin* __restrict__ dq, float* __restrict__ dg,
    float* __restrict__ dfr, float* __restrict__ part /* [2][B*H]: dtemp, scalar dfr */) {
    extern __shared__ __align__(16) float smem[];
    const int N = p.N, DK = p.DK, T = p.T, H = p.H;
    const int NP = (N + 3) & ~3;                         // keeps rq (read as float4) 16-byte aligned for any N
    float* K = smem;
    float* o = K + (size_t)N * DK;
    float* kinv = o + NP;
    float* dO = kinv + NP;
    float* sv = dO + NP;
    float* zv = sv + NP;
    float* dwv = zv + NP;
    int* tf = reinterpret_cast<int*>(dwv + NP);
    float* rq = reinterpret_cast<float*>(tf + NP);       // [2][SEQ_WARPS][DK]
    __shared__ float r_m[2][SEQ_WARPS], r_s[2][SEQ_WARPS], r_sd[2][SEQ_WARPS], r_ez[2][SEQ_WARPS], r_ed[2][SEQ_WARPS];
    __shared__ int r_e[2][SEQ_WARPS];
    __shared__ float r_fr[2][SEQ_WARPS], r_dt[SEQ_WARPS];

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int col = lane * 4;
    const bool act = col < DK;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i = tid; i < N * DK; i += SEQ_THREADS) K[i] = kfin[(size_t)bh * N * DK + i];
    for (int i = tid; i < N; i += SEQ_THREADS) {
        o[i] = ofin[(size_t)bh * N + i];
        dO[i] = 0.f;
        tf[i] = tfirst[(size_t)bh * N + i];
    }
    __syncthreads();
    for (int n = warp; n < N; n += SEQ_WARPS) {
        const float4 Kn = act ? ld4(K + (size_t)n * DK + col) : zero4;
        const float nsq = warp_sum(dot4(Kn, Kn));
        if (lane == 0) kinv[n] = 1.f / fmaxf(sqrtf(nsq), 1e-6f);
    }
    __syncthreads();
    const float temp = temp_p[0], eps = p.eps;
    float frv = p.fr_per_token ? 0.f : fr[0];
    float dtemp_acc = 0.f, dfr_acc = 0.f;
    int lim = N - 1;                                      // candidates at token t: rows n with tfirst[n] <= t
    int par = 0;
    for (int t = T - 1; t >= 0; t--) {
        const size_t ix = ((size_t)b * T + t) * H + h;
        const int a = am[ix];
        const float g = gate_eff(gate[ix], p.hard_gate);
        if (p.fr_per_token) frv = fr[ix];
        const float4 qt = act ? ld4(q + ix * DK + col) : zero4;
        while (lim > 0 && tf[lim] > t) lim--;
        if ((a % SEQ_WARPS) == warp) {                    // undo the write of token t
            const float4 Ko = act ? ld4(kold + ix * DK + col) : zero4;
            if (act) st4(K + (size_t)a * DK + col, Ko);
            const float nsq = warp_sum(dot4(Ko, Ko));
            if (lane == 0) { kinv[a] = 1.f / fmaxf(sqrtf(nsq), 1e-6f); o[a] = oold[ix]; }
            __syncwarp();
        }
        const float qq = warp_sum(dot4(qt, qt));
        const float qnorm = sqrtf(qq), qinv = 1.f / fmaxf(qnorm, 1e-6f);
        const float4 qn = make_float4(qt.x * qinv, qt.y * qinv, qt.z * qinv, qt.w * qinv);
        // pass 1: scores, dw, online softmax statistics over occupied rows; the lowest free row kept aside
        float M = -INFINITY, S = 0.f, SD = 0.f, ez = 0.f, ed = 0.f;
        int ei = BIGI;
        for (int n = warp; n <= lim; n += SEQ_WARPS) {
            const float4 Kn = act ? ld4(K + (size_t)n * DK + col) : zero4;
            const float ki = kinv[n];
            const float dt = warp_sum((Kn.x * ki) * qn.x + (Kn.y * ki) * qn.y + (Kn.z * ki) * qn.z + (Kn.w * ki) * qn.w);
            const float s = temp * dt, oc = o[n];
            const float occ = p.occ_bin ? (oc >= eps ? 1.f : 0.f) : oc;
            const float z = s - frv * occ;
            const float dw = Din[((size_t)bh * T + t) * N + n] + (1.f - oc) * dO[n];
            if (lane == 0) { sv[n] = s; zv[n] = z; dwv[n] = dw; }
            if (oc < eps) { if (n < ei) { ei = n; ez = z; ed = dw; } }
            else {
                const float m2 = fmaxf(M, z);
                const float sc = (M == -INFINITY) ? 0.f : __expf(M - m2);
                const float e = __expf(z - m2);
                S = S * sc + e; SD = SD * sc + e * dw; M = m2;
            }
        }
        if (lane == 0) { r_m[par][warp] = M; r_s[par][warp] = S; r_sd[par][warp] = SD;
                         r_e[par][warp] = ei; r_ez[par][warp] = ez; r_ed[par][warp] = ed; }
        __syncthreads();
        M = -INFINITY; S = 0.f; SD = 0.f; ei = BIGI; ez = 0.f; ed = 0.f;
#pragma unroll
        for (int w = 0; w < SEQ_WARPS; w++) {
            const float M2 = r_m[par][w], S2 = r_s[par][w], SD2 = r_sd[par][w];
            const float m = fmaxf(M, M2);
            if (m != -INFINITY) {
                const float s1 = (M == -INFINITY) ? 0.f : __expf(M - m), s2 = (M2 == -INFINITY) ? 0.f : __expf(M2 - m);
                S = S * s1 + S2 * s2; SD = SD * s1 + SD2 * s2; M = m;
            }
            if (r_e[par][w] < ei) { ei = r_e[par][w]; ez = r_ez[par][w]; ed = r_ed[par][w]; }
        }
        if (ei != BIGI) {                                 // the lowest free row competes too
            const float m = fmaxf(M, ez);
            const float s1 = (M == -INFINITY) ? 0.f : __expf(M - m), e = __expf(ez - m);
            S = S * s1 + e; SD = SD * s1 + e * ed; M = m;
        }
        const float sa = g * SD / S;                      // sum_n asoft_n (g dw_n)
        // pass 2: dz per row, scalar gradients, dqn = sum_n dz_n temp Kn_n
        float4 pq = zero4;
        float frp = 0.f;
        for (int n = warp; n <= lim; n += SEQ_WARPS) {
            const float oc = o[n];
            const bool ok = (oc >= eps) || (n == ei);
            const float dw = dwv[n];
            const float as = ok ? __expf(zv[n] - M) / S : 0.f;
            const float dz = ok ? as * (g * dw - sa) : 0.f;
            if (n == a && lane == 0) dg[ix] = dw;
            const float occ = p.occ_bin ? (oc >= eps ? 1.f : 0.f) : oc;
            if (lane == 0) { dtemp_acc += dz * sv[n] / temp; frp += -occ * dz; }
            const float4 Kn = act ? ld4(K + (size_t)n * DK + col) : zero4;
            const float cz = dz * temp * kinv[n];
            pq.x += cz * Kn.x; pq.y += cz * Kn.y; pq.z += cz * Kn.z; pq.w += cz * Kn.w;
            if (!p.occ_bin) { if (lane == 0) dO[n] = ((n == a) ? 1.f - g : 1.f) * dO[n] - frv * dz; }
            else if (n == a && lane == 0) dO[n] = (1.f - g) * dO[n];
        }
        __syncwarp();
        if (act) st4(rq + ((size_t)par * SEQ_WARPS + warp) * DK + col, pq);
        if (lane == 0) r_fr[par][warp] = frp;
        __syncthreads();
        if (warp == 0) {
            float4 dqn = zero4;
            float f = 0.f;
#pragma unroll
            for (int w = 0; w < SEQ_WARPS; w++) {
                if (act) {
                    const float4 v = ld4(rq + ((size_t)par * SEQ_WARPS + w) * DK + col);
                    dqn.x += v.x; dqn.y += v.y; dqn.z += v.z; dqn.w += v.w;
                }
                f += r_fr[par][w];
            }
            const float pr = warp_sum(dot4(dqn, qn));
            float4 out;
            if (qnorm < 1e-6f) out = make_float4(qinv * dqn.x, qinv * dqn.y, qinv * dqn.z, qinv * dqn.w);
            else out = make_float4(qinv * (dqn.x - qn.x * pr), qinv * (dqn.y - qn.y * pr),
                                   qinv * (dqn.z - qn.z * pr), qinv * (dqn.w - qn.w * pr));
            if (act) st4(dq + ix * DK + col, out);
            if (lane == 0) { if (p.fr_per_token) dfr[ix] = f; else dfr_acc += f; }
        }
        par ^= 1;
    }
    if (lane == 0) r_dt[warp] = dtemp_acc;
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int w = 0; w < SEQ_WARPS; w++) s += r_dt[w];
        part[bh] = s;
        part[(size_t)p.B * H + bh] = dfr_acc;
    }
}

// fixed-order sum of the per-sequence partials -> dtemp, scalar dfr; with q == NULL also dk += dq
__global__ void finish_scalars_kernel(const float* __restrict__ part, int BH, int fr_per_token, float* dtemp, float* dfr) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        float a = 0.f, c = 0.f;
        for (int i = 0; i < BH; i++) { a += part[i]; c += part[BH + i]; }
        dtemp[0] = a;
        if (!fr_per_token) dfr[0] = c;
    }
}
template <typename Tin>
__global__ void add_into_kernel(Tin* __restrict__ dst, const Tin* __restrict__ src, size_t n4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = ld4(dst + i * 4), c = ld4(src + i * 4);
        st4(dst + i * 4, make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w));
    }
}

// ------------------------------------------------------------------------------------------------------
// Optional per-kernel timing (slotscan_profile_*): CUDA events recorded on the launching stream around each launch.
struct ProfRec { int id; cudaEvent_t a, b; };
static bool g_prof_on = false;
static std::vector<ProfRec> g_prof;
static std::mutex g_prof_mu;
enum { K_ADDR_FWD = 0, K_REPLAY_K, K_REPLAY_V, K_ROWS_BWD_K, K_ROWS_BWD_V, K_ADDR_BWD, K_FINISH, K_NKERN };
static const char* const K_NAMES[K_NKERN] = {"addr_fwd", "replay_rows_k", "replay_rows_v", "rows_bwd_k", "rows_bwd_v",
                                             "addr_bwd", "finish"};
struct ProfScope {
    int id; cudaStream_t st; cudaEvent_t a = nullptr, b = nullptr; bool on;
    ProfScope(int id_, cudaStream_t st_) : id(id_), st(st_), on(g_prof_on) {
        if (on) { cudaEventCreate(&a); cudaEventCreate(&b); cudaEventRecord(a, st); }
    }
    ~ProfScope() {
        if (on) { cudaEventRecord(b, st); std::lock_guard<std::mutex> l(g_prof_mu); g_prof.push_back({id, a, b}); }
    }
};

static size_t addr_fwd_smem(const slotscan_params* p) { return sizeof(float) * ((size_t)p->N * p->DK + 2 * (size_t)p->N); }
static size_t addr_bwd_smem(const slotscan_params* p) {
    const size_t NP = ((size_t)p->N + 3) & ~(size_t)3;
    return sizeof(float) * ((size_t)p->N * p->DK + 7 * NP + 2 * (size_t)SEQ_WARPS * p->DK);
}
constexpr size_t SMEM_CAP = 227 * 1024;

template <typename F>
static cudaError_t opt_in_smem(F f, size_t bytes) {
    return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <int DK, typename Tin>
static cudaError_t launch_addr_fwd(const slotscan_params& p, const void* q, const void* k, const float* gate,
                                   const float* fr, const float* temp, const slotscan_log& L, cudaStream_t st) {
    const size_t sm = sizeof(float) * (size_t)addr_fwd_layout(p.N, DK, (int)sizeof(Tin)).total;
    cudaError_t e;
#define AF_LAUNCH(RPL_, OCCB_)                                                                                     \
    {                                                                                                              \
        auto kern = addr_fwd_chunked_kernel<DK, RPL_, OCCB_, Tin>;                                                 \
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;                                                  \
        kern<<<p.B * p.H, AF_THREADS, sm, st>>>(p, (const Tin*)q, (const Tin*)k, gate, fr, temp, L.addr, L.oold,   \
                                                L.kiold, L.ofin, L.tfirst);                                        \
    }
    if (p.N <= 192) {
        if (p.occ_bin) AF_LAUNCH(6, true) else AF_LAUNCH(6, false)
    } else {
        if (p.occ_bin) AF_LAUNCH(14, true) else AF_LAUNCH(14, false)
    }
#undef AF_LAUNCH
    return cudaGetLastError();
}

template <int DK, typename Tin>
static cudaError_t launch_addr_bwd(const slotscan_params& p, const void* q, const void* k, const float* gate,
                                   const float* fr, const float* temp, const slotscan_log& L, const float* Dn, void* dq,
                                   float* dgate, float* dfr, float* part, cudaStream_t st) {
    const size_t sm = sizeof(float) * (size_t)addr_bwd_layout(p.N, DK).total;
    cudaError_t e;
#define AB_LAUNCH(RPL_, OCCB_)                                                                                      \
    {                                                                                                               \
        auto kern = addr_bwd_chunked_kernel<DK, RPL_, OCCB_, Tin>;                                                  \
        if ((e = opt_in_smem(kern, sm)) != cudaSuccess) return e;                                                   \
        kern<<<p.B * p.H, AF_THREADS, sm, st>>>(p, (const Tin*)q, (const Tin*)k, gate, fr, temp, L.addr, L.kold,    \
                                                L.oold, L.kiold, L.kfin, L.ofin, L.tfirst, Dn, (Tin*)dq, dgate, dfr, \
                                                part);                                                              \
    }
    if (p.N <= 192) {
        if (p.occ_bin) AB_LAUNCH(6, true) else AB_LAUNCH(6, false)
    } else {
        if (p.occ_bin) AB_LAUNCH(14, true) else AB_LAUNCH(14, false)
    }
#undef AB_LAUNCH
    return cudaGetLastError();
}

template <int D, typename Tin, typename Tsn>
static cudaError_t launch_replay(const slotscan_params& p, const void* x, const float* gate, const int* am, void* xbuf,
                                 float* xold, float* xfin, cudaStream_t st) {
    constexpr int RPB = ROW_THREADS / (D / 8);
    dim3 grid(p.B * p.H, (p.N + RPB - 1) / RPB);
    replay_rows_kernel<D, Tin, Tsn><<<grid, ROW_THREADS, 0, st>>>(p, (const Tin*)x, gate, am, (Tsn*)xbuf, xold, xfin);
    return cudaGetLastError();
}
template <int D, typename Tin, typename Tsn>
static cudaError_t launch_rows_bwd(const slotscan_params& p, bool accum, const void* x, const float* gate, const int* am,
                                   const float* xold, const float* xfin, const int* tfirst, const void* dxbuf, void* dx,
                                   float* Dn, cudaStream_t st) {
    constexpr int RPB = ROW_THREADS / (D / 8);
    dim3 grid(p.B * p.H, (p.N + RPB - 1) / RPB);
    if (accum)
        rows_bwd_kernel<D, Tin, Tsn, true><<<grid, ROW_THREADS, 0, st>>>(p, (const Tin*)x, gate, am, xold, xfin, tfirst,
                                                                         (const Tsn*)dxbuf, (Tin*)dx, Dn);
    else
        rows_bwd_kernel<D, Tin, Tsn, false><<<grid, ROW_THREADS, 0, st>>>(p, (const Tin*)x, gate, am, xold, xfin, tfirst,
                                                                          (const Tsn*)dxbuf, (Tin*)dx, Dn);
    return cudaGetLastError();
}

#define DISPATCH_D(D_, CALL)                                   \
    switch (D_) {                                              \
        case 8: { constexpr int DD = 8; CALL; } break;         \
        case 16: { constexpr int DD = 16; CALL; } break;       \
        case 32: { constexpr int DD = 32; CALL; } break;       \
        case 64: { constexpr int DD = 64; CALL; } break;       \
        case 128: { constexpr int DD = 128; CALL; } break;     \
        default: { constexpr int DD = 0; (void)DD; return cudaErrorInvalidValue; }  \
    }

template <typename Tin, typename Tsn>
static cudaError_t fwd_typed(const slotscan_params& p, const void* k, const void* q, const void* v, const float* gate,
                             const float* fr, const float* temp, void* kbuf, void* vbuf, const slotscan_log& L,
                             cudaStream_t st) {
    cudaError_t e;
    {
        ProfScope ps(K_ADDR_FWD, st);
        DISPATCH_D(p.DK, e = (launch_addr_fwd<DD, Tin>(p, q ? q : k, k, gate, fr, temp, L, st)));
    }
    if (e != cudaSuccess) return e;
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    {
        ProfScope ps(K_REPLAY_K, st);
        DISPATCH_D(p.DK, e = (launch_replay<DD, Tin, Tsn>(p, k, gate, L.addr, kbuf, L.kold, L.kfin, st)));
    }
    if (e != cudaSuccess) return e;
    {
        ProfScope ps(K_REPLAY_V, st);
        DISPATCH_D(p.DV, e = (launch_replay<DD, Tin, Tsn>(p, v, gate, L.addr, vbuf, L.vold, L.vfin, st)));
    }
    return e;
}

template <typename Tin, typename Tsn>
static cudaError_t bwd_typed(const slotscan_params& p, const void* k, const void* q, const void* v, const float* gate,
                             const float* fr, const float* temp, const slotscan_log& L, const void* dkbuf,
                             const void* dvbuf, float* Dn, float* part, void* dk, void* dq, void* dv, float* dgate,
                             float* dfr, float* dtemp, cudaStream_t st) {
    cudaError_t e;
    {
        ProfScope ps(K_ROWS_BWD_K, st);
        DISPATCH_D(p.DK, e = (launch_rows_bwd<DD, Tin, Tsn>(p, false, k, gate, L.addr, L.kold, L.kfin, L.tfirst, dkbuf, dk, Dn, st)));
    }
    if (e != cudaSuccess) return e;
    {
        ProfScope ps(K_ROWS_BWD_V, st);
        DISPATCH_D(p.DV, e = (launch_rows_bwd<DD, Tin, Tsn>(p, true, v, gate, L.addr, L.vold, L.vfin, L.tfirst, dvbuf, dv, Dn, st)));
    }
    if (e != cudaSuccess) return e;
    {
        ProfScope ps(K_ADDR_BWD, st);
        DISPATCH_D(p.DK, e = (launch_addr_bwd<DD, Tin>(p, q ? q : k, k, gate, fr, temp, L, Dn, dq, dgate, dfr, part, st)));
    }
    if (e != cudaSuccess) return e;
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    ProfScope ps(K_FINISH, st);
    finish_scalars_kernel<<<1, 32, 0, st>>>(part, p.B * p.H, p.fr_per_token, dtemp, dfr);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (q == nullptr) {
        const size_t n4 = (size_t)p.B * p.T * p.H * p.DK / 4;
        add_into_kernel<Tin><<<592, 256, 0, st>>>((Tin*)dk, (const Tin*)dq, n4);
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace slotscan

using namespace slotscan;

static inline bool misaligned(const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

extern "C" int slotscan_abi_version(void) { return SLOTSCAN_ABI_VERSION; }

extern "C" int slotscan_check(const slotscan_params* p) {
    if (!p) return SLOTSCAN_E_NULL;
    if (p->B < 1 || p->T < 1 || p->H < 1 || p->N < 1 || p->G < 1) return SLOTSCAN_E_SHAPE;
    if (p->DK < 8 || p->DK > 128 || (p->DK & (p->DK - 1))) return SLOTSCAN_E_SHAPE;
    if (p->DV < 8 || p->DV > 128 || (p->DV & (p->DV - 1))) return SLOTSCAN_E_SHAPE;
    if (addr_bwd_smem(p) + 1024 > SMEM_CAP) return SLOTSCAN_E_SHAPE;
    if (sizeof(float) * (size_t)addr_fwd_layout(p->N, p->DK, 4).total + 1024 > SMEM_CAP || p->N > 448) return SLOTSCAN_E_SHAPE;
    if (sizeof(float) * (size_t)addr_bwd_layout(p->N, p->DK).total + 1024 > SMEM_CAP) return SLOTSCAN_E_SHAPE;
    if ((long long)p->B * p->H > 2147483647LL / 4) return SLOTSCAN_E_SHAPE;
    if (p->in_dtype != SLOTSCAN_F32 && p->in_dtype != SLOTSCAN_BF16) return SLOTSCAN_E_DTYPE;
    if (p->snap_dtype != SLOTSCAN_F32 && p->snap_dtype != SLOTSCAN_BF16) return SLOTSCAN_E_DTYPE;
    return SLOTSCAN_OK;
}

extern "C" int slotscan_hard_fwd(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                                 const float* fr, const float* temp, void* kbuf, void* vbuf, const slotscan_log* log,
                                 void* stream) {
    int rc = slotscan_check(p);
    if (rc) return rc;
    if (!k || !v || !gate || !fr || !temp || !kbuf || !vbuf || !log) return SLOTSCAN_E_NULL;
    if (!log->addr || !log->oold || !log->kold || !log->vold || !log->kfin || !log->vfin || !log->ofin || !log->tfirst ||
        !log->kiold)
        return SLOTSCAN_E_NULL;
    if (misaligned(k) || misaligned(q) || misaligned(v) || misaligned(kbuf) || misaligned(vbuf) || misaligned(log->kold) ||
        misaligned(log->vold) || misaligned(log->kfin) || misaligned(log->vfin))
        return SLOTSCAN_E_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (p->in_dtype == SLOTSCAN_F32)
        e = (p->snap_dtype == SLOTSCAN_F32) ? fwd_typed<float, float>(*p, k, q, v, gate, fr, temp, kbuf, vbuf, *log, st)
                                            : fwd_typed<float, __nv_bfloat16>(*p, k, q, v, gate, fr, temp, kbuf, vbuf, *log, st);
    else
        e = (p->snap_dtype == SLOTSCAN_F32)
                ? fwd_typed<__nv_bfloat16, float>(*p, k, q, v, gate, fr, temp, kbuf, vbuf, *log, st)
                : fwd_typed<__nv_bfloat16, __nv_bfloat16>(*p, k, q, v, gate, fr, temp, kbuf, vbuf, *log, st);
    return (int)e;
}

extern "C" size_t slotscan_hard_bwd_scratch_bytes(const slotscan_params* p) {
    if (slotscan_check(p)) return 0;
    const size_t BH = (size_t)p->B * p->H;
    size_t dn = sizeof(float) * BH * p->T * p->N;
    dn = (dn + 255) & ~(size_t)255;
    return dn + sizeof(float) * 2 * BH;
}

extern "C" int slotscan_hard_bwd(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                                 const float* fr, const float* temp, const slotscan_log* log, const void* dkbuf,
                                 const void* dvbuf, void* scratch, size_t scratch_bytes, void* dk, void* dq, void* dv,
                                 float* dgate, float* dfr, float* dtemp, void* stream) {
    int rc = slotscan_check(p);
    if (rc) return rc;
    if (!k || !v || !gate || !fr || !temp || !log || !scratch || !dk || !dq || !dv || !dgate || !dfr || !dtemp)
        return SLOTSCAN_E_NULL;
    if (!log->addr || !log->oold || !log->kold || !log->vold || !log->kfin || !log->vfin || !log->ofin || !log->tfirst ||
        !log->kiold)
        return SLOTSCAN_E_NULL;
    if (scratch_bytes < slotscan_hard_bwd_scratch_bytes(p)) return SLOTSCAN_E_SHAPE;
    if (misaligned(k) || misaligned(q) || misaligned(v) || misaligned(dkbuf) || misaligned(dvbuf) || misaligned(dk) ||
        misaligned(dq) || misaligned(dv) || misaligned(scratch) || misaligned(log->kold) || misaligned(log->vold) ||
        misaligned(log->kfin) || misaligned(log->vfin))
        return SLOTSCAN_E_ALIGN;
    const size_t BH = (size_t)p->B * p->H;
    size_t dn = sizeof(float) * BH * p->T * p->N;
    dn = (dn + 255) & ~(size_t)255;
    float* Dn = (float*)scratch;
    float* part = (float*)((char*)scratch + dn);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (p->in_dtype == SLOTSCAN_F32)
        e = (p->snap_dtype == SLOTSCAN_F32)
                ? bwd_typed<float, float>(*p, k, q, v, gate, fr, temp, *log, dkbuf, dvbuf, Dn, part, dk, dq, dv, dgate, dfr, dtemp, st)
                : bwd_typed<float, __nv_bfloat16>(*p, k, q, v, gate, fr, temp, *log, dkbuf, dvbuf, Dn, part, dk, dq, dv, dgate, dfr, dtemp, st);
    else
        e = (p->snap_dtype == SLOTSCAN_F32)
                ? bwd_typed<__nv_bfloat16, float>(*p, k, q, v, gate, fr, temp, *log, dkbuf, dvbuf, Dn, part, dk, dq, dv, dgate, dfr, dtemp, st)
                : bwd_typed<__nv_bfloat16, __nv_bfloat16>(*p, k, q, v, gate, fr, temp, *log, dkbuf, dvbuf, Dn, part, dk, dq, dv, dgate, dfr, dtemp, st);
    return (int)e;
}

template <typename F>
static void fill_attr(slotscan_kernel_attr* out, int cap, int& n, const char* name, F f) {
    if (n < cap) {
        cudaFuncAttributes a;
        if (cudaFuncGetAttributes(&a, f) == cudaSuccess) {
            snprintf(out[n].name, sizeof(out[n].name), "%s", name);
            out[n].regs = a.numRegs;
            out[n].local_bytes = (int)a.localSizeBytes;
            out[n].static_smem = (int)a.sharedSizeBytes;
            out[n].max_threads = a.maxThreadsPerBlock;
        }
    }
    n++;
}

extern "C" int slotscan_query_attrs(slotscan_kernel_attr* out, int cap) {
    int n = 0;
    fill_attr(out, cap, n, "addr_fwd<128,f32>", addr_fwd_chunked_kernel<128, 6, true, float>);
    fill_attr(out, cap, n, "addr_fwd<128,bf16>", addr_fwd_chunked_kernel<128, 6, true, __nv_bfloat16>);
    fill_attr(out, cap, n, "replay_rows<128,bf16,bf16>", replay_rows_kernel<128, __nv_bfloat16, __nv_bfloat16>);
    fill_attr(out, cap, n, "replay_rows<128,f32,f32>", replay_rows_kernel<128, float, float>);
    fill_attr(out, cap, n, "rows_bwd<128,bf16,bf16>", rows_bwd_kernel<128, __nv_bfloat16, __nv_bfloat16, false>);
    fill_attr(out, cap, n, "rows_bwd<128,f32,f32>", rows_bwd_kernel<128, float, float, false>);
    fill_attr(out, cap, n, "addr_bwd<128,f32>", addr_bwd_chunked_kernel<128, 6, true, float>);
    fill_attr(out, cap, n, "addr_bwd<128,bf16>", addr_bwd_chunked_kernel<128, 6, true, __nv_bfloat16>);
    return n;
}

extern "C" int slotscan_profile_enable(int on) {
    std::lock_guard<std::mutex> l(g_prof_mu);
    g_prof_on = on != 0;
    return 0;
}

extern "C" int slotscan_profile_read(slotscan_kernel_time* out, int cap) {
    std::lock_guard<std::mutex> l(g_prof_mu);
    float ms[K_NKERN] = {0};
    int cnt[K_NKERN] = {0};
    for (auto& r : g_prof) {
        float t = 0.f;
        if (cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess) {
            ms[r.id] += t;
            cnt[r.id]++;
        }
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    g_prof.clear();
    for (int i = 0; i < K_NKERN && i < cap; i++) {
        snprintf(out[i].name, sizeof(out[i].name), "%s", K_NAMES[i]);
        out[i].launches = cnt[i];
        out[i].total_ms = ms[i];
    }
    return K_NKERN;
}

// ------------------------------------------------------------------------------------------------------
// Backward without caller scratch.  Some hosts cannot hand this library a scratch buffer: a serving process that
// gave every byte of device memory to its own arena at start-up, a thin foreign-language binding that has no device
// allocator to call, a code path in which a synchronising cudaMalloc / cudaFree is not acceptable.  For them the
// table D[t,n] and the per-sequence partial sums live in a fixed array inside the library image.
//
// The array's name is only a host-side handle for the symbol; the device address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) unsigned char g_fixed_scratch[SLOTSCAN_NOALLOC_SCRATCH_BYTES];
constexpr int MAX_DEVICES = 64;
static void* g_fixed_scratch_addr[MAX_DEVICES] = {nullptr};
static std::mutex g_fixed_scratch_mu;

extern "C" size_t slotscan_hard_bwd_noalloc_capacity(void) { return (size_t)SLOTSCAN_NOALLOC_SCRATCH_BYTES; }

extern "C" int slotscan_hard_bwd_noalloc(const slotscan_params* p, const void* k, const void* q, const void* v,
                                         const float* gate, const float* fr, const float* temp, const slotscan_log* log,
                                         const void* dkbuf, const void* dvbuf, void* dk, void* dq, void* dv, float* dgate,
                                         float* dfr, float* dtemp, void* stream) {
    int rc = slotscan_check(p);
    if (rc) return rc;
    if (slotscan_hard_bwd_scratch_bytes(p) > (size_t)SLOTSCAN_NOALLOC_SCRATCH_BYTES) return SLOTSCAN_E_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return SLOTSCAN_E_SHAPE;
    void* scratch;
    {
        std::lock_guard<std::mutex> l(g_fixed_scratch_mu);
        if (g_fixed_scratch_addr[dev] == nullptr) {          // first call on this device: resolve the symbol
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_fixed_scratch);
            if (e != cudaSuccess) return (int)e;
            if (ptr == nullptr) return (int)cudaErrorInvalidSymbol;
            g_fixed_scratch_addr[dev] = ptr;
        }
        scratch = g_fixed_scratch_addr[dev];
    }
    // Nothing in the scratch has to start at zero: every D[t,n] and every partial sum that is read was written earlier
    // in the same call (the key pass stores D, the value pass adds to it, the address pass reads it).
    return slotscan_hard_bwd(p, k, q, v, gate, fr, temp, log, dkbuf, dvbuf, scratch, (size_t)SLOTSCAN_NOALLOC_SCRATCH_BYTES,
                             dk, dq, dv, dgate, dfr, dtemp, stream);
}

#ifdef SLOTSCAN_PHASE_TIMING
// development aid (not part of the ABI header): per-phase clock totals of the chunked kernels, summed over CTAs
extern "C" int slotscan_debug_phase_cycles(unsigned long long* out8, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out8, slotscan::g_phase_cycles, 16 * sizeof(unsigned long long));
    if (e == cudaSuccess && reset) {
        unsigned long long z[16] = {0};
        e = cudaMemcpyToSymbol(slotscan::g_phase_cycles, z, sizeof(z));
    }
    return (int)e;
}
#endif
