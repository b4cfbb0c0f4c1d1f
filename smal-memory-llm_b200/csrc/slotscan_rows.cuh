// Row-parallel kernels of the hard-address scan: once the address log exists, every key row and every value row
// evolves on its own (a row changes only at the tokens that addressed it).
//
//   replay_rows_kernel   forward: replays rows from the log, emits the stride-G snapshots, the undo log (the row
//                        before each write) and the final state.                 [reference val_fwd, slotkern_cuda.py:178-206]
// (The reverse row scan lives in slotscan_rows_bwd.cuh.)
//
// Layout: one group of LPR = D/8 lanes per row, 8 elements per lane in registers, RPB = 256 / LPR rows per CTA;
// grid (B*H, row tiles).  Tokens are taken in chunks of RC = 32: the chunk's gates, a per-row bit mask of the tokens
// that hit the row, and the chunk's token vectors are staged in shared memory once per CTA, so the walk over a chunk
// is a walk over EVENTS (next hit, next snapshot) and never waits on a global load.  A tile whose rows are never
// addressed (tfirst == T for all of them) only writes zeros (forward) or does nothing (reverse).
#pragma once
#include "slotscan_common.cuh"

namespace slotscan {

constexpr int ROW_THREADS = 256;
constexpr int RC = 32;                        // tokens per staged chunk (hit mask per row: one bit per token)

template <typename T>
__device__ __forceinline__ void copy8(T* dst, const T* src);
template <>
__device__ __forceinline__ void copy8<float>(float* dst, const float* src) {
    const float4 a = ld4(src), b = ld4(src + 4);
    st4(dst, a); st4(dst + 4, b);
}
template <>
__device__ __forceinline__ void copy8<__nv_bfloat16>(__nv_bfloat16* dst, const __nv_bfloat16* src) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
}

// true if any row of this CTA's tile is ever a candidate (row 0 always is)
__device__ __forceinline__ bool tile_active(const int* tfirst_bh, int n, bool live, int T, int* s_flag) {
    if (threadIdx.x == 0) *s_flag = 0;
    __syncthreads();
    if (live && tfirst_bh[n] < T) *s_flag = 1;
    __syncthreads();
    return *s_flag != 0;
}

// stage one chunk: gates, per-row hit masks and (optionally) token vectors; the caller syncs afterwards
template <int D, typename Tin>
__device__ __forceinline__ void stage_chunk(const slotscan_params& p, int b, int h, int t0, int tc, int row0,
                                            const float* __restrict__ gate, const int* __restrict__ am,
                                            const Tin* __restrict__ x, float* s_g, unsigned long long* s_mask, Tin* s_x) {
    constexpr int LPR = D / 8, RPB = ROW_THREADS / LPR;
    const int tid = threadIdx.x, T = p.T, H = p.H;
    for (int i = tid; i < RPB; i += ROW_THREADS) s_mask[i] = 0ull;
    __syncthreads();
    for (int i = tid; i < tc; i += ROW_THREADS) {
        const size_t ix = ((size_t)b * T + t0 + i) * H + h;
        s_g[i] = gate_eff(gate[ix], p.hard_gate);
        const int a = am[ix] - row0;
        if (a >= 0 && a < RPB) atomicOr(&s_mask[a], 1ull << i);
    }
    for (int it = tid; it < tc * LPR; it += ROW_THREADS) {
        const int j = it / LPR, cc = (it % LPR) * 8;
        copy8<Tin>(s_x + j * D + cc, x + (((size_t)b * T + t0 + j) * H + h) * D + cc);
    }
}

// ======================================================================================================
// kinv / valid of a row from its float32 state: rsqrt(max(|X|^2, 1e-12)) and [|X|^2 > 1e-12]  [memlm_sh.py:474-475]
// The rows of one warp walk their events independently, so the sum runs over the row's own LPR lanes only (`gmask`).
template <int LPR>
__device__ __forceinline__ float row_nsq(const float* X, unsigned gmask) {
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) a = fmaf(X[j], X[j], a);
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) a += __shfl_xor_sync(gmask, a, off);
    return a;
}
template <int LPR>
__device__ __forceinline__ unsigned row_group_mask() {
    const unsigned lane = threadIdx.x & 31u;
    return (LPR >= 32) ? FULL : (((1u << LPR) - 1u) << (LPR * (lane / LPR)));
}

// NORM: also emit kinv / valid of every snapshot row (keys only).  x0 (may be NULL): the rows the replay starts from.
template <int D, typename Tin, typename Tsn, bool NORM>
__global__ void __launch_bounds__(ROW_THREADS) replay_rows_kernel(
    const slotscan_params p, const Tin* __restrict__ x, const float* __restrict__ gate, const int* __restrict__ am,
    const int* __restrict__ tfirst, const float* __restrict__ x0, Tsn* __restrict__ xbuf, float* __restrict__ xold,
    float* __restrict__ xfin, float* __restrict__ kinv_out, uint8_t* __restrict__ valid_out) {
    constexpr int LPR = D / 8, RPB = ROW_THREADS / LPR;
    __shared__ float s_g[RC];
    __shared__ unsigned long long s_mask[RPB];
    __shared__ __align__(16) Tin s_x[RC * D];
    __shared__ int s_flag;
    const int N = p.N, T = p.T, H = p.H, G = p.G;
    const int NB = (T + G - 1) / G;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, r = tid / LPR, c = tid % LPR, row0 = blockIdx.y * RPB, n = row0 + r;
    const bool live = n < N;
    float X[8];
#pragma unroll
    for (int j = 0; j < 8; j++) X[j] = 0.f;
    const size_t snap_stride = (size_t)H * N * D;                   // between consecutive snapshots of one sequence
    Tsn* snap = xbuf + (((size_t)b * NB) * H + h) * N * D + (size_t)n * D + c * 8;
    // kinv / valid of snapshot j of this row live at norm_base + j * norm_stride (one lane per row writes them)
    const size_t norm_stride = (size_t)H * N;
    size_t norm_ix = (((size_t)b * NB) * H + h) * N + n;

    if (!tile_active(tfirst + (size_t)bh * N, n, live, T, &s_flag)) {
        if (live) {                                                  // never a candidate: the row stays zero
            for (int j = 0; j < NB; j++) st8(snap + j * snap_stride, X);
            st8(xfin + ((size_t)bh * N + n) * D + c * 8, X);
            if (NORM && c == 0) {
                for (int j = 0; j < NB; j++) { kinv_out[norm_ix + j * norm_stride] = 1e6f; valid_out[norm_ix + j * norm_stride] = 0; }
            }
        }
        return;
    }
    if (x0 != nullptr && live) ld8(X, x0 + ((size_t)bh * N + n) * D + c * 8);   // state carried in from the preceding chunk
    const unsigned gmask = row_group_mask<LPR>();
    int tsnap = 0;                                                   // next snapshot time (multiple of G)
    for (int t0 = 0; t0 < T; t0 += RC) {
        const int tc = min(RC, T - t0);
        __syncthreads();
        stage_chunk<D, Tin>(p, b, h, t0, tc, row0, gate, am, x, s_g, s_mask, s_x);
        __syncthreads();
        if (!live) continue;
        const unsigned long long m = s_mask[r];
        int i = 0;
        while (true) {
            const unsigned long long mm = m >> i;                    // i < tc <= 64 here
            const int ih = mm ? i + __ffsll((long long)mm) - 1 : tc; // next token that writes this row
            const int tlast = t0 + min(ih, tc - 1);
            if (NORM) {
                if (tsnap <= tlast) {                                // the state is the same for every snapshot of this stretch
                    const float nsq = row_nsq<LPR>(X, gmask);
                    if (c == 0) {
                        const float ki = rsqrtf(fmaxf(nsq, 1e-12f));
                        const uint8_t va = nsq > 1e-12f ? 1 : 0;
                        size_t o = norm_ix;
                        for (int ts = tsnap; ts <= tlast; ts += G) { kinv_out[o] = ki; valid_out[o] = va; o += norm_stride; }
                    }
                }
            }
            for (; tsnap <= tlast; tsnap += G) {                     // pre-write copies
                st8(snap, X);
                snap += snap_stride; norm_ix += norm_stride;
            }
            if (ih >= tc) break;
            const size_t ix = ((size_t)b * T + t0 + ih) * H + h;
            const float g = s_g[ih], omw = 1.f - g;
            float xv[8];
            ld8(xv, s_x + ih * D + c * 8);
            if (xold != nullptr) st8(xold + ix * D + c * 8, X);
#pragma unroll
            for (int j = 0; j < 8; j++) X[j] = blend(X[j], xv[j], g, omw);
            i = ih + 1;
            if (i >= tc) break;
        }
    }
    if (live) st8(xfin + ((size_t)bh * N + n) * D + c * 8, X);
}

// ======================================================================================================
// one tensor's worth of arguments: blockIdx.z picks the keys (0) or the values (1) when both run in one launch
template <typename Tin, typename Tsn>
struct RowsBwdArgs {
    const Tin* x;
    const float* xold;
    const float* xfin;
    const Tsn* dxbuf;
    Tin* dx;
    float* Dn;       // this tensor's own D table: the address backward adds the two
    const float* dkinv;   // (B,NB,H,N) gradient of the kinv output, or NULL: enters dX where the snapshot was taken
};

}  // namespace slotscan
