// Row-parallel kernels of the hard-address scan: once the address log exists, every key row and every value row
// evolves on its own (a row changes only at the tokens that addressed it).
//
//   replay_rows_kernel   forward: replays rows from the log, emits the stride-G snapshots, the undo log (the row
//                        before each write) and the final state.                 [reference val_fwd, slotkern_cuda.py:178-206]
//   rows_bwd_kernel      reverse: undoes rows from the undo log, carries dX <- (1-g) dX + dxbuf, emits dx_t = g dX_a and
//                        the table D[t,n] = <x_t - X_n, dX_n>.                    [reference rows_bwd, :209-261]
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
// rows_bwd: reverse scan per row.  dX_n <- (1-w) dX_n + dxbuf;  dx_t = g dX_am;  D[t,n] (+)= <x_t - X_n, dX_n>.
// A row stops at tfirst[n]: before that token it is neither written nor a candidate, so nothing reads its D.
// Dynamic shared memory: the chunk's token vectors (Tin), the undo rows of the tokens that hit this tile (f32),
// gates and hit masks.
template <int D, typename Tin>
__host__ __device__ constexpr size_t rows_bwd_smem_bytes() {
    return (size_t)RC * D * sizeof(Tin) + (size_t)RC * D * sizeof(float) + RC * sizeof(float) +
           (ROW_THREADS / (D / 8)) * sizeof(unsigned long long) + 16;
}

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

template <int D, typename Tin, typename Tsn>
__global__ void __launch_bounds__(ROW_THREADS) rows_bwd_kernel(
    const slotscan_params p, const RowsBwdArgs<Tin, Tsn> a0, const RowsBwdArgs<Tin, Tsn> a1,
    const float* __restrict__ gate, const int* __restrict__ am, const int* __restrict__ tfirst) {
    constexpr bool ACCUM = false;
    const RowsBwdArgs<Tin, Tsn>& A = blockIdx.z ? a1 : a0;
    const Tin* __restrict__ x = A.x;
    const float* __restrict__ xold = A.xold;
    const float* __restrict__ xfin = A.xfin;
    const Tsn* __restrict__ dxbuf = A.dxbuf;
    Tin* __restrict__ dx = A.dx;
    float* __restrict__ Dn = A.Dn;
    const float* __restrict__ dkinv = A.dkinv;
    constexpr int LPR = D / 8, RPB = ROW_THREADS / LPR;
    extern __shared__ __align__(16) unsigned char dsm[];
    float* s_xo = reinterpret_cast<float*>(dsm);                                   // [RC][D] undo rows
    Tin* s_x = reinterpret_cast<Tin*>(dsm + (size_t)RC * D * sizeof(float));       // [RC][D] token vectors
    unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(dsm + (size_t)RC * D * (sizeof(float) + sizeof(Tin)));
    float* s_g = reinterpret_cast<float*>(s_mask + RPB);
    __shared__ int s_flag, s_stop;
    const int N = p.N, T = p.T, H = p.H, G = p.G;
    const int NB = (T + G - 1) / G;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, r = tid / LPR, c = tid % LPR, row0 = blockIdx.y * RPB, n0 = row0 + r;
    const bool live = n0 < N;
    const int n = live ? n0 : 0;          // dead rows still run the shuffles; they read row 0 and write nothing
    if (!tile_active(tfirst + (size_t)bh * N, n, live, T, &s_flag)) return;
    const int tstop = live ? tfirst[(size_t)bh * N + n] : T;
    const int wstop = __reduce_min_sync(FULL, tstop);      // every lane of a warp runs the same shuffle steps
    if (tid == 0) s_stop = T;
    __syncthreads();
    if ((tid & 31) == 0) atomicMin(&s_stop, wstop);
    __syncthreads();
    const int cstop = s_stop;                               // the whole tile is done below this token
    float X[8], dX[8];
    ld8(X, xfin + ((size_t)bh * N + n) * D + c * 8);
#pragma unroll
    for (int j = 0; j < 8; j++) dX[j] = 0.f;
    const size_t snap_stride = (size_t)H * N * D;
    const Tsn* dsnap0 = (dxbuf == nullptr) ? nullptr : dxbuf + (((size_t)b * NB) * H + h) * N * D + (size_t)n * D + c * 8;
    // the snapshot gradient of block jb is added when the walk passes t = jb * G; it is fetched one block ahead
    int jb = NB - 1;
    float nxt[8], nxt_w = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) nxt[j] = 0.f;
    const float* dki0 = (dkinv == nullptr) ? nullptr : dkinv + (((size_t)b * NB) * H + h) * N + n;
    const size_t dki_stride = (size_t)H * N;
    // snapshot gradient of block JB into nxt (and the kinv gradient of that snapshot row into nxt_w)
#define RB_FETCH(JB)                                                                        \
    if ((JB) >= 0 && (JB) * G >= tstop) {                                                   \
        if (dsnap0 != nullptr) ld8(nxt, dsnap0 + (size_t)(JB) * snap_stride);               \
        if (dki0 != nullptr) nxt_w = dki0[(size_t)(JB) * dki_stride];                       \
    }
    // dX += the gradients that arrive at the snapshot taken at this token (X is the pre-write state here): the snapshot
    // gradient itself and, through kinv = rsqrt(max(|X|^2, 1e-12)), -kinv^3 dkinv X.  All lanes of the warp call.
#define RB_ADD_SNAPSHOT(ON)                                                                 \
    {                                                                                       \
        float w_ = 0.f;                                                                     \
        if (dki0 != nullptr) {                                                              \
            float nsq_ = 0.f;                                                               \
            _Pragma("unroll") for (int j = 0; j < 8; j++) nsq_ = fmaf(X[j], X[j], nsq_);    \
            nsq_ = group_sum<LPR>(nsq_);                                                    \
            const float ki_ = rsqrtf(fmaxf(nsq_, 1e-12f));                                  \
            w_ = nsq_ > 1e-12f ? -(ki_ * ki_ * ki_) * nxt_w : 0.f;                          \
        }                                                                                   \
        if (ON) {                                                                           \
            _Pragma("unroll") for (int j = 0; j < 8; j++) dX[j] += nxt[j] + w_ * X[j];      \
        }                                                                                   \
    }
    RB_FETCH(jb)

    const int nchunk = (T + RC - 1) / RC;
    for (int ck = nchunk - 1; ck >= 0; ck--) {
        const int t0 = ck * RC, tc = min(RC, T - t0);
        if (t0 + tc <= cstop) break;                                               // uniform over the CTA
        __syncthreads();
        stage_chunk<D, Tin>(p, b, h, t0, tc, row0, gate, am, x, s_g, s_mask, s_x);
        __syncthreads();
        // undo rows of the tokens that hit this tile
        for (int it = tid; it < tc * LPR; it += ROW_THREADS) {
            const int j = it / LPR, cc = (it % LPR) * 8;
            const int a = am[((size_t)b * T + t0 + j) * H + h] - row0;
            if (a >= 0 && a < RPB) copy8<float>(s_xo + j * D + cc, xold + (((size_t)b * T + t0 + j) * H + h) * D + cc);
        }
        __syncthreads();
        const unsigned long long m = live ? s_mask[r] : 0ull;
        // hit masks of the rows sharing this warp decide together whether the 4-token fast path may run
        unsigned long long mw = m;
#pragma unroll
        for (int off = 16; off >= LPR && off > 0; off >>= 1) mw |= __shfl_xor_sync(FULL, mw, off);
        for (int i = tc - 1; i >= 0; i--) {
            int t = t0 + i;
            if (t < wstop) break;
            if (LPR >= 4) {
                // Four consecutive tokens t, t-1, t-2, t-3 see the same (X, dX) when none of them writes a row of this
                // warp and no snapshot gradient lands after the first three: then the four dot products are reduced
                // together (5 shuffles instead of 16).
                while (i >= 3 && t - 3 >= wstop && ((mw >> (i - 3)) & 0xfull) == 0ull &&
                       (jb < 0 || jb * G <= t - 3 || jb * G > t)) {
                    float ps[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        float xv[8];
                        ld8(xv, s_x + (i - u) * D + c * 8);
                        float a = 0.f;
#pragma unroll
                        for (int j = 0; j < 8; j++) a += (xv[j] - X[j]) * dX[j];
                        ps[u] = a;
                    }
                    constexpr int O1 = LPR / 2, O2 = LPR / 4;
                    const bool up1 = (c & O1) != 0, up2 = (c & O2) != 0;
                    const float s0 = up1 ? ps[0] : ps[2], s1 = up1 ? ps[1] : ps[3];
                    const float r0 = __shfl_xor_sync(FULL, s0, O1), r1 = __shfl_xor_sync(FULL, s1, O1);
                    const float q0 = (up1 ? ps[2] : ps[0]) + r0, q1 = (up1 ? ps[3] : ps[1]) + r1;   // tokens 2u1, 2u1+1
                    const float r2 = __shfl_xor_sync(FULL, up2 ? q0 : q1, O2);
                    float w = (up2 ? q1 : q0) + r2;                                                // token 2 u1 + u2
#pragma unroll
                    for (int off = O2 / 2; off > 0; off >>= 1) w += __shfl_xor_sync(FULL, w, off);
                    const int u = (up1 ? 2 : 0) + (up2 ? 1 : 0);
                    const int tu = t - u;
                    if (live && tu >= tstop && (c & (O2 - 1)) == 0) {
                        float* dst = Dn + ((size_t)bh * T + tu) * N + n;
                        if (ACCUM) *dst += w; else *dst = w;
                    }
                    if (jb >= 0 && jb * G == t - 3) {                              // the group ended on a snapshot time
                        RB_ADD_SNAPSHOT(t - 3 >= tstop)
                        jb--;
                        RB_FETCH(jb)
                    }
                    i -= 4;
                    t -= 4;
                }
                if (i < 0 || t < wstop) break;
            }
            const bool on = t >= tstop;
            const bool hit = on && ((m >> i) & 1ull);
            float xv[8];
            ld8(xv, s_x + i * D + c * 8);
            if (hit) ld8(X, s_xo + i * D + c * 8);
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
                st8(dx + (((size_t)b * T + t) * H + h) * D + c * 8, a);
            }
            if (t == jb * G) {                                                     // pre-write state of block jb
                RB_ADD_SNAPSHOT(on)
                jb--;
                RB_FETCH(jb)
            }
        }
    }
#undef RB_FETCH
#undef RB_ADD_SNAPSHOT
}

}  // namespace slotscan
