// Reverse row scan of the hard-address backward.  [reference rows_bwd, slotkern_cuda.py:209-261]
//
//   dX_n <- (1 - w) dX_n + dxbuf;   dx_t = g dX_a;   D[t,n] = <x_t - X_n, dX_n>   for every candidate row n of token t
//
// Once the address log exists every row evolves on its own, so the grid is (sequence x head, tiles of RPB rows,
// tensor) and only tiles that hold a candidate row do anything.  One group of LPR = D/8 lanes per row, 8 columns per
// lane in registers.  Tokens come in chunks of RC = 32, newest first, through a two-stage shared-memory ring fed by
// bulk asynchronous copies (cp.async.bulk global -> shared, completion counted on an mbarrier): while the warps walk
// chunk c, the token vectors of chunk c-1 and the undo rows of the tokens of c-1 that hit THIS tile are already in
// flight, and the gates / addresses of chunk c-2 are being fetched (the addresses decide which undo rows to copy).
// Per token a lane does 2 shared loads + 8 FMAs: the token vectors are converted to float32 once per chunk, and
// D[t,n] = <x_t, dX_n> - <X_n, dX_n> with the second term kept per lane and refreshed only when X_n or dX_n changes
// (a hit, a snapshot time).  Four consecutive tokens that see the same (X, dX) reduce their four dot products
// together (5 shuffles instead of 16).
#pragma once
#include <type_traits>

#include "slotscan_async.cuh"
#include "slotscan_common.cuh"
#include "slotscan_rows.cuh"

namespace slotscan {

// Set when a bounded wait gave up; the kernel then returns without finishing (slotscan_device_status reads it).
static __device__ int g_rows_bwd_status = 0;

template <int D, typename Tin>
struct RowsBwdLayout {                         // byte offsets into dynamic shared memory
    static constexpr bool CONV = !std::is_same<Tin, float>::value;
    static constexpr int XRAW = RC * D * (int)sizeof(Tin), XO = RC * D * 4, STAGE = XRAW + XO;
    static constexpr int off_stage0 = 0, off_xf = 2 * STAGE, off_g = off_xf + (CONV ? RC * D * 4 : 0);
    static constexpr int off_am = off_g + 3 * RC * 4, off_bar = off_am + 3 * RC * 4, total = off_bar + 16;
};

template <int D, typename Tin, typename Tsn, bool DKINV>
__global__ void __launch_bounds__(ROW_THREADS, 3) rows_bwd2_kernel(
    const slotscan_params p, const RowsBwdArgs<Tin, Tsn> a0, const RowsBwdArgs<Tin, Tsn> a1,
    const float* __restrict__ gate, const int* __restrict__ am, const int* __restrict__ tfirst, const int ntens) {
    typedef RowsBwdLayout<D, Tin> LY;
    // Launch order = work order.  Rows are occupied in index order, so the low tiles carry the work and most high
    // tiles return at once; with tile-major block indices (tile, then sequence x head, then tensor) the tiles that
    // work are launched first, keys and values side by side, instead of queueing behind thousands of empty ones.
    const int BHn = p.B * p.H;
    const int tens = (int)(blockIdx.x % ntens), tb = (int)(blockIdx.x / ntens);
    const int tile = tb / BHn, bh = tb - tile * BHn;
    const RowsBwdArgs<Tin, Tsn>& A = tens ? a1 : a0;
    const Tin* __restrict__ x = A.x;
    const float* __restrict__ xold = A.xold;
    const float* __restrict__ xfin = A.xfin;
    const Tsn* __restrict__ dxbuf = A.dxbuf;
    Tin* __restrict__ dx = A.dx;
    float* __restrict__ Dn = A.Dn;
    constexpr int LPR = D / 8, RPB = ROW_THREADS / LPR, RPW = 32 / LPR;        // rows per CTA, rows per warp
    extern __shared__ __align__(128) unsigned char dsm[];
    float* s_g = reinterpret_cast<float*>(dsm + LY::off_g);                     // [3][RC] gates
    int* s_am = reinterpret_cast<int*>(dsm + LY::off_am);                       // [3][RC] addressed row - row0
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(dsm + LY::off_bar);           // [2]
    __shared__ int s_flag, s_stop;
    const int N = p.N, T = p.T, H = p.H, G = p.G;
    const int NB = (T + G - 1) / G;
    const int b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = tid / LPR, c = tid % LPR, row0 = tile * RPB, n0 = row0 + r;
    const bool live = n0 < N;
    const int n = live ? n0 : 0;          // dead rows still run the shuffles; they read row 0 and write nothing
    if (!tile_active(tfirst + (size_t)bh * N, n, live, T, &s_flag)) return;
    const int tstop = live ? tfirst[(size_t)bh * N + n] : T;
    const int wstop = __reduce_min_sync(FULL, tstop);      // every lane of a warp runs the same shuffle steps
    if (tid == 0) {
        s_stop = T;
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (lane == 0) atomicMin(&s_stop, wstop);
    __syncthreads();
    const int cstop = s_stop;                               // the whole tile is done below this token
    const int c_hi = (T + RC - 1) / RC - 1, c_lo = cstop / RC;   // chunks c_hi, c_hi - 1, ..., c_lo hold the work

    // gates and addresses of chunk ck into slot ck % 3 of the small ring (plain loads: they are gathers with stride H)
    auto load_scalars = [&](int ck) {
        if (tid < RC) {
            const int t = ck * RC + tid, slot = ck % 3;
            float g = 0.f;
            int a = -1;
            if (t < T) {
                const size_t ix = ((size_t)b * T + t) * H + h;
                g = gate_eff(gate[ix], p.hard_gate);
                a = am[ix] - row0;
                if (a >= RPB) a = -1;
            }
            s_g[slot * RC + tid] = g;
            s_am[slot * RC + tid] = a;
        }
    };
    // warp 0: the chunk's token vectors, and the undo rows of its tokens that hit this tile, into stage st
    auto issue_bulk = [&](int ck, int st) {
        const int t = ck * RC + lane;
        const bool in = t < T;
        const int a = s_am[(ck % 3) * RC + lane];
        const bool hit = in && a >= 0;
        const unsigned nin = __popc(__ballot_sync(FULL, in)), nhit = __popc(__ballot_sync(FULL, hit));
        if (lane == 0) mbar_arrive_expect_tx(&s_bar[st], nin * (unsigned)(D * sizeof(Tin)) + nhit * (unsigned)(D * 4));
        __syncwarp();
        if (in) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            unsigned char* base = dsm + st * LY::STAGE;
            bulk_g2s(base + lane * D * sizeof(Tin), x + ix * D, D * sizeof(Tin), &s_bar[st]);
            if (hit) bulk_g2s(base + LY::XRAW + lane * D * 4, xold + ix * D, D * 4, &s_bar[st]);
        }
    };

    float X[8], dX[8];
    ld8(X, xfin + ((size_t)bh * N + n) * D + c * 8);
#pragma unroll
    for (int j = 0; j < 8; j++) dX[j] = 0.f;
    float pxd = 0.f;                                        // this lane's part of <X, dX>
    const size_t snap_stride = (size_t)H * N * D;
    const Tsn* dsnap0 = (dxbuf == nullptr) ? nullptr : dxbuf + (((size_t)b * NB) * H + h) * N * D + (size_t)n * D + c * 8;
    // the snapshot gradient of block jb is added when the walk passes t = jb * G; it is fetched one block ahead
    int jb = NB - 1;
    float nxt[8], nxt_w = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) nxt[j] = 0.f;
    const float* dki0 = (!DKINV || A.dkinv == nullptr) ? nullptr : A.dkinv + (((size_t)b * NB) * H + h) * N + n;
    const size_t dki_stride = (size_t)H * N;
    // snapshot gradient of block JB into nxt (and the kinv gradient of that snapshot row into nxt_w)
#define RB_FETCH(JB)                                                                        \
    if ((JB) >= 0 && (JB) * G >= tstop) {                                                   \
        if (dsnap0 != nullptr) ld8(nxt, dsnap0 + (size_t)(JB) * snap_stride);               \
        if (DKINV && dki0 != nullptr) nxt_w = dki0[(size_t)(JB) * dki_stride];              \
    }
#define RB_PXD()                                                                            \
    {                                                                                       \
        pxd = 0.f;                                                                          \
        _Pragma("unroll") for (int j = 0; j < 8; j++) pxd = fmaf(X[j], dX[j], pxd);         \
    }
    // dX += the gradients that arrive at the snapshot taken at this token (X is the pre-write state here): the snapshot
    // gradient itself and, through kinv = rsqrt(max(|X|^2, 1e-12)), -kinv^3 dkinv X.  All lanes of the warp call.
#define RB_ADD_SNAPSHOT(ON)                                                                 \
    {                                                                                       \
        float w_ = 0.f;                                                                     \
        if (DKINV && dki0 != nullptr) {                                                     \
            float nsq_ = 0.f;                                                               \
            _Pragma("unroll") for (int j = 0; j < 8; j++) nsq_ = fmaf(X[j], X[j], nsq_);    \
            nsq_ = group_sum<LPR>(nsq_);                                                    \
            const float ki_ = rsqrtf(fmaxf(nsq_, 1e-12f));                                  \
            w_ = nsq_ > 1e-12f ? -(ki_ * ki_ * ki_) * nxt_w : 0.f;                          \
        }                                                                                   \
        if (ON) {                                                                           \
            _Pragma("unroll") for (int j = 0; j < 8; j++) dX[j] += nxt[j] + w_ * X[j];      \
            RB_PXD()                                                                        \
        }                                                                                   \
    }
    RB_FETCH(jb)

    // ---- prologue: scalars of the first two chunks, bulk copies of the first ----
    load_scalars(c_hi);
    if (c_hi - 1 >= c_lo) load_scalars(c_hi - 1);
    __syncthreads();
    if (warp == 0) issue_bulk(c_hi, 0);

    for (int k = 0; c_hi - k >= c_lo; k++) {
        const int ck = c_hi - k, st = k & 1, slot = ck % 3;
        const int t0 = ck * RC, tc = min(RC, T - t0);
        __syncthreads();                                    // every warp is done with chunk ck + 1 (stage st ^ 1, s_xf)
        if (warp == 0 && ck - 1 >= c_lo) issue_bulk(ck - 1, st ^ 1);
        if (ck - 2 >= c_lo) load_scalars(ck - 2);
        const bool landed = mbar_wait_bounded(&s_bar[st], (unsigned)(k >> 1) & 1u);
        const unsigned char* stage = dsm + st * LY::STAGE;
        const float* xs;
        if (LY::CONV) {                                     // token vectors to float32, once per chunk
            float* xf = reinterpret_cast<float*>(dsm + LY::off_xf);
            if (landed) {
                for (int it = tid; it < tc * LPR; it += ROW_THREADS) {
                    float f[8];
                    ld8(f, reinterpret_cast<const Tin*>(stage) + it * 8);
                    st8(xf + it * 8, f);
                }
            }
            xs = xf;
        } else {
            xs = reinterpret_cast<const float*>(stage);
        }
        const float* xo = reinterpret_cast<const float*>(stage + LY::XRAW);
        const float* sg = s_g + slot * RC;
        // hit masks: bit i set when token t0 + i writes this lane's row; mw = the rows sharing this warp
        unsigned m = 0u, mw = 0u;
        {
            const int aL = s_am[slot * RC + lane];
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) {
                const unsigned bm = __ballot_sync(FULL, aL == warp * RPW + rr);
                if (rr == lane / LPR) m = bm;
                mw |= bm;
            }
        }
        if (!__syncthreads_and(landed ? 1 : 0)) {           // a copy never landed: give up, all threads together
            if (tid == 0) atomicExch(&g_rows_bwd_status, 1);
            return;
        }
        for (int i = tc - 1; i >= 0; i--) {
            int t = t0 + i;
            if (t < wstop) break;
            if (LPR >= 4) {
                // Four consecutive tokens t, t-1, t-2, t-3 see the same (X, dX) when none of them writes a row of this
                // warp and no snapshot gradient lands after the first three: then the four dot products are reduced
                // together (5 shuffles instead of 16).
                while (i >= 3 && t - 3 >= wstop && ((mw >> (i - 3)) & 0xfu) == 0u &&
                       (jb < 0 || jb * G <= t - 3 || jb * G > t)) {
                    float ps[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        float xv[8];
                        ld8(xv, xs + (i - u) * D + c * 8);
                        float a = -pxd;
#pragma unroll
                        for (int j = 0; j < 8; j++) a = fmaf(xv[j], dX[j], a);
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
                    if (live && tu >= tstop && (c & (O2 - 1)) == 0) Dn[((size_t)bh * T + tu) * N + n] = w;
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
            const bool hit = on && ((m >> i) & 1u);
            float xv[8];
            ld8(xv, xs + i * D + c * 8);
            if (hit) {
                ld8(X, xo + i * D + c * 8);
                RB_PXD()
            }
            float pacc = -pxd;
#pragma unroll
            for (int j = 0; j < 8; j++) pacc = fmaf(xv[j], dX[j], pacc);
            pacc = group_sum<LPR>(pacc);
            if (on && c == 0) Dn[((size_t)bh * T + t) * N + n] = pacc;
            if (hit) {
                const float g = sg[i], omw = 1.f - g;
                float a[8];
#pragma unroll
                for (int j = 0; j < 8; j++) { a[j] = g * dX[j]; dX[j] = omw * dX[j]; }
                pxd *= omw;
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
#undef RB_PXD
#undef RB_ADD_SNAPSHOT
}


// ======================================================================================================
// Event-walk form of the reverse row scan, used when the snapshot stride is 8 or 16 and D >= 64.
//
// The lock-step walk above spends its time on bookkeeping: per token and row 8 FMAs per lane against a shuffle
// reduction, a hit test, a snapshot test.  But dX_n only changes at EVENTS -- a hit on row n scales it by (1 - g), a
// snapshot time adds that snapshot's gradient -- so inside one block of G tokens it is  dX_n(t) = c_n(t) S_n  with one
// vector S_n per (row, block) and a scalar c_n(t) (the product of (1 - g) over the hits since the block's top).  Hence
//     D[t,n] = c_n(t) <x_t, S_n> - <X_n(t), dX_n(t)>
// and each chunk of 32 tokens splits into
//   (E) an event walk per row (its own LPR lanes, rows of a warp independent of each other): restores X at hits, emits
//       dx_t = g dX, scales, adds the snapshot gradients at the block bottoms, and leaves in shared memory S per
//       (block, row), c and <X, dX> per (token, row);
//   (P) a token-parallel pass: lane = token, warp = row pair, 128-long dot products <x_t, S_n> straight out of shared
//       memory with no reduction and no dependency between tokens.
// Nothing waits on global memory inside a chunk: the token vectors of chunk c-1 are copied (bulk async, padded rows)
// while chunk c is processed, the undo rows of c-1 right after the walk of c has consumed those of c, gates and
// addresses two chunks ahead, and each lane holds the snapshot gradients of the next two blocks in registers as they
// came from memory (bf16: 4 registers per block).
// Shared memory (D = 128, bf16): S 32 KB, 2 x 8.5 KB token vectors, 16 KB undo rows, c and <X, dX> 4 KB: 70 KB,
// three CTAs per SM.
template <typename Tsn> struct SnapRaw;
template <> struct SnapRaw<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = ld4(p); b = ld4(p + 4); }
    __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void get(float* f) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};
template <> struct SnapRaw<__nv_bfloat16> {
    uint4 u;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { u = make_uint4(0u, 0u, 0u, 0u); }
    __device__ __forceinline__ void get(float* f) const {
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
};
// 8 consecutive elements of a staged token row as float32
__device__ __forceinline__ void row8(float* f, const float* p) { ld8(f, p); }
__device__ __forceinline__ void row8(float* f, const __nv_bfloat16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

template <int D, typename Tin>
struct RowsBwd3Layout {
    static constexpr int RPB = ROW_THREADS / (D / 8);
    static constexpr int XRS = D * (int)sizeof(Tin) + 16;                 // bytes per padded token row
    // [block][row][D] with 16 bytes between the blocks: in the token-parallel pass the lanes of a warp (tokens of up to
    // four blocks) read the same element of up to four blocks at once, and without the stagger those sit in the same banks
    static constexpr int SBS = RPB * D + 4;                               // floats per block
    static constexpr int off_S = 0, S_bytes = (RC / 8) * SBS * 4;
    static constexpr int off_x = off_S + S_bytes, x_bytes = RC * XRS;     // two stages
    static constexpr int off_xo = off_x + 2 * x_bytes, xo_bytes = RC * D * 4;
    static constexpr int off_c = off_xo + xo_bytes, c_bytes = RC * RPB * 4;   // [row][token]
    static constexpr int off_xdx = off_c + c_bytes;
    static constexpr int off_g = off_xdx + c_bytes, off_am = off_g + 2 * RC * 4, off_ts = off_am + 2 * RC * 4;
    static constexpr int off_bar = off_ts + RPB * 4, total = off_bar + 32;
};

template <int D, int GG, typename Tin, typename Tsn, bool DKINV>
__global__ void __launch_bounds__(ROW_THREADS, (sizeof(Tin) == 2 ? 3 : 2)) rows_bwd3_kernel(
    const slotscan_params p, const RowsBwdArgs<Tin, Tsn> a0, const RowsBwdArgs<Tin, Tsn> a1,
    const float* __restrict__ gate, const int* __restrict__ am, const int* __restrict__ tfirst, const int ntens) {
    typedef RowsBwd3Layout<D, Tin> LY;
    constexpr int LPR = D / 8, RPB = LY::RPB, RPW = 32 / LPR, NSEG = RC / GG, G = GG;
    static_assert(LPR >= 8 && (NSEG == 2 || NSEG == 4), "row groups of >= 8 lanes; an even number of blocks per chunk");
    const int BHn = p.B * p.H;
    const int tens = (int)(blockIdx.x % ntens), tb = (int)(blockIdx.x / ntens);
    const int tile = tb / BHn, bh = tb - tile * BHn;
    const RowsBwdArgs<Tin, Tsn>& A = tens ? a1 : a0;
    const Tin* __restrict__ x = A.x;
    const float* __restrict__ xold = A.xold;
    const float* __restrict__ xfin = A.xfin;
    const Tsn* __restrict__ dxbuf = A.dxbuf;
    Tin* __restrict__ dx = A.dx;
    float* __restrict__ Dn = A.Dn;
    extern __shared__ __align__(128) unsigned char dsm[];
    float* s_S = reinterpret_cast<float*>(dsm + LY::off_S);
    float* s_xo = reinterpret_cast<float*>(dsm + LY::off_xo);
    float* s_c = reinterpret_cast<float*>(dsm + LY::off_c);
    float* s_xdx = reinterpret_cast<float*>(dsm + LY::off_xdx);
    float* s_g = reinterpret_cast<float*>(dsm + LY::off_g);               // [2 slots][RC]
    int* s_am = reinterpret_cast<int*>(dsm + LY::off_am);                 // [2 slots][RC]
    int* s_ts = reinterpret_cast<int*>(dsm + LY::off_ts);                 // tstop of every row of the tile
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(dsm + LY::off_bar);     // [0], [1]: token-vector stages; [2]: undo rows
    __shared__ int s_flag, s_stop;
    const int N = p.N, T = p.T, H = p.H;
    const int NB = (T + G - 1) / G;
    const int b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // (Neighbouring rows share a warp.  Pairing row r with row r + 8 instead, so that a busy low row sits with an idle
    // high one, was measured: faster with few sequences per GPU, slower with three CTAs per SM, where it only spreads
    // the same instructions over more warps.)
    const int r = tid / LPR, c = lane % LPR, row0 = tile * RPB, n0 = row0 + r;
    const bool live = n0 < N;
    const int n = live ? n0 : 0;
    if (!tile_active(tfirst + (size_t)bh * N, n, live, T, &s_flag)) return;
    const int tstop = live ? tfirst[(size_t)bh * N + n] : T;
    if (c == 0) s_ts[r] = tstop;
    if (tid == 0) {
        s_stop = T;
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        mbar_init(&s_bar[2], 1);
        mbar_fence_init();
    }
    __syncthreads();
    if (c == 0) atomicMin(&s_stop, tstop);
    __syncthreads();
    const int cstop = s_stop;                               // the whole tile is done below this token
    const int c_hi = (T + RC - 1) / RC - 1, c_lo = cstop / RC;
    const unsigned gmask = row_group_mask<LPR>();

    float X[8], dX[8];
    ld8(X, xfin + ((size_t)bh * N + n) * D + c * 8);
#pragma unroll
    for (int j = 0; j < 8; j++) dX[j] = 0.f;
    const size_t snap_stride = (size_t)H * N * D;
    const Tsn* dsnap0 = (dxbuf == nullptr) ? nullptr : dxbuf + (((size_t)b * NB) * H + h) * N * D + (size_t)n * D + c * 8;
    const float* dki0 = (!DKINV || A.dkinv == nullptr) ? nullptr : A.dkinv + (((size_t)b * NB) * H + h) * N + n;
    const size_t dki_stride = (size_t)H * N;
    // The gradients that arrive at snapshot jb (taken before token jb * G), as they come from memory, two blocks ahead
    // of their use: slot jb & 1.  A chunk holds an even number of blocks, so the slot of block sg of a chunk is sg & 1.
    SnapRaw<Tsn> ring0, ring1;
    float ringw0 = 0.f, ringw1 = 0.f;
    ring0.zero(); ring1.zero();
    auto fetch = [&](int JB, SnapRaw<Tsn>& dst, float& dstw) {
        if (JB >= 0 && JB * G >= tstop && live) {
            if (dsnap0 != nullptr) dst.load(dsnap0 + (size_t)JB * snap_stride);
            if (DKINV && dki0 != nullptr) dstw = dki0[(size_t)JB * dki_stride];
        }
    };
    if ((NB - 1) & 1) { fetch(NB - 1, ring1, ringw1); fetch(NB - 2, ring0, ringw0); }
    else { fetch(NB - 1, ring0, ringw0); fetch(NB - 2, ring1, ringw1); }
    // sum over the row's own lanes (the rows of a warp walk their events independently)
    auto rsum = [&](float v) {
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1) v += __shfl_xor_sync(gmask, v, off);
        return v;
    };
    auto dotXdX = [&]() {
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) a = fmaf(X[j], dX[j], a);
        return rsum(a);
    };

    // The scalars of the chunks ahead are the duty of the last warp, after the barrier that releases the walk.
    const bool issuer = warp == ROW_THREADS / 32 - 1;
    // scalars of a chunk: fetched into registers two chunks ahead, stored one chunk ahead (issuing warp)
    float pre_g = 0.f;
    int pre_a = -1;
    auto load_scalars = [&](int ck) {
        pre_g = 0.f; pre_a = -1;
        if (issuer && ck >= c_lo) {
            const int t = ck * RC + lane;
            if (t < T) {
                const size_t ix = ((size_t)b * T + t) * H + h;
                pre_g = gate_eff(gate[ix], p.hard_gate);
                pre_a = am[ix] - row0;
                if (pre_a >= RPB) pre_a = -1;
            }
        }
    };
    // Every warp issues its share (RC / 8 tokens) of a chunk's copies: a warp's bulk copies leave one after the other,
    // some 75 cycles apiece, so 32 of them from one warp would hold that warp's rows up for a couple of thousand cycles.
    // One thread posts the byte count; copies that complete before it has done so make the count negative for a moment.
    constexpr int PER = RC / (ROW_THREADS / 32);
    // token vectors of chunk ck into stage st (padded rows, as they are in memory)
    auto issue_x = [&](int ck, int st) {
        const int i = warp * PER + lane, t = ck * RC + i;
        if (tid == 0) mbar_arrive_expect_tx(&s_bar[st], (unsigned)min(RC, T - ck * RC) * (unsigned)(D * sizeof(Tin)));
        if (lane < PER && t < T)
            bulk_g2s(dsm + LY::off_x + st * LY::x_bytes + i * LY::XRS, x + (((size_t)b * T + t) * H + h) * D, D * sizeof(Tin), &s_bar[st]);
    };
    // undo rows of the tokens of chunk ck that write a row of this tile (addresses in slot `slot`)
    auto issue_xo = [&](int ck, int slot) {
        if (warp == 0) {
            const bool hit = ck * RC + lane < T && s_am[slot * RC + lane] >= 0;
            const unsigned nhit = __popc(__ballot_sync(FULL, hit));
            if (lane == 0) mbar_arrive_expect_tx(&s_bar[2], nhit * (unsigned)(D * 4));
        }
        const int i = warp * PER + lane, t = ck * RC + i;
        if (lane < PER && t < T && s_am[slot * RC + i] >= 0)
            bulk_g2s(s_xo + i * D, xold + (((size_t)b * T + t) * H + h) * D, D * 4, &s_bar[2]);
    };

    // ---- prologue: chunk c_hi's scalars and copies; chunk c_hi - 1's scalars into registers ----
    load_scalars(c_hi);
    if (issuer) {
        s_g[lane] = pre_g;
        s_am[lane] = pre_a;
    }
    __syncthreads();
    issue_x(c_hi, 0);
    issue_xo(c_hi, 0);
    load_scalars(c_hi - 1);

    for (int k = 0; c_hi - k >= c_lo; k++) {
        const int ck = c_hi - k, st = k & 1;
        const int t0 = ck * RC, tc = min(RC, T - t0);
        const bool landed = mbar_wait_bounded(&s_bar[st], (unsigned)(k >> 1) & 1u) && mbar_wait_bounded(&s_bar[2], (unsigned)k & 1u);
        // one barrier: the previous chunk's token-parallel pass is over (its stage and scalar slot are free), and
        // this chunk's copies have landed for everybody -- or never will: then give up, all threads together
        if (!__syncthreads_and(landed ? 1 : 0)) {
            if (tid == 0) atomicExch(&g_rows_bwd_status, 1);
            return;
        }
        if (ck - 1 >= c_lo) issue_x(ck - 1, st ^ 1);        // next chunk: token vectors in flight
        if (issuer) {                                       // its scalars into the other slot; those of the chunk after it fetched
            if (ck - 1 >= c_lo) {
                s_g[(st ^ 1) * RC + lane] = pre_g;
                s_am[(st ^ 1) * RC + lane] = pre_a;
            }
            load_scalars(ck - 2);
        }
        // hit mask of this lane's row: bit i set when token t0 + i writes it
        unsigned m = 0u;
        {
            const int aL = s_am[st * RC + lane];
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) {
                const unsigned bm = __ballot_sync(FULL, aL == warp * RPW + rr);
                if (rr == lane / LPR) m = bm;
            }
        }
        // ---------------- (E) event walk of this lane's row over the chunk, newest token first ----------------
        if (live && t0 + tc > tstop) {
            const int nseg = (tc + G - 1) / G;              // chunk starts are multiples of G
            const float* sg_ = s_g + st * RC;
#pragma unroll
            for (int sg = NSEG - 1; sg >= 0; sg--) {
                if (sg < nseg) {
                    const int ilo = sg * G, ihi = min(tc, ilo + G) - 1;
                    // top of the block: dX is S, c = 1
                    {   // the row's two float4 halves of every lane go to [c] and [D/8 + c] of the row's float4 slots: lanes
                        // c and c + 4 of a quarter-warp would otherwise store to the same banks (the pass below reads it so)
                        float* Sw = s_S + (size_t)sg * LY::SBS + r * D;
                        st4(Sw + 4 * c, make_float4(dX[0], dX[1], dX[2], dX[3]));
                        st4(Sw + D / 2 + 4 * c, make_float4(dX[4], dX[5], dX[6], dX[7]));
                    }
                    float c_cur = 1.f;
                    float xdx_cur = dotXdX();
                    unsigned ms = (m >> ilo) & ((1u << G) - 1u);
                    int top = ihi;                          // tokens top, top-1, ... still to be recorded
                    while (true) {
                        const int ih = ms ? ilo + 31 - __clz(ms) : ilo - 1;   // next hit going down (or below the block)
                        for (int i = top - c; i > ih; i -= LPR) { s_c[r * RC + i] = c_cur; s_xdx[r * RC + i] = xdx_cur; }
                        if (ih < ilo) break;
                        ms &= ~(1u << (ih - ilo));
                        // token ih writes this row: its D sees the restored row, then the write's adjoint
                        ld8(X, s_xo + ih * D + c * 8);
                        const float xd = dotXdX();
                        const float g = sg_[ih], omw = 1.f - g;
                        if (c == 0) { s_c[r * RC + ih] = c_cur; s_xdx[r * RC + ih] = xd; }
                        float a[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) { a[j] = g * dX[j]; dX[j] = omw * dX[j]; }
                        st8(dx + (((size_t)b * T + t0 + ih) * H + h) * D + c * 8, a);
                        c_cur *= omw;
                        xdx_cur = xd * omw;
                        top = ih - 1;
                    }
                    // bottom of the block: token t0 + ilo is the time of snapshot jb; its gradients join dX for the
                    // tokens below, and the slot is refilled with the snapshot two blocks further down
                    const int jb = t0 / G + sg;
                    SnapRaw<Tsn>& slot = (sg & 1) ? ring1 : ring0;
                    float& slotw = (sg & 1) ? ringw1 : ringw0;
                    if (jb * G >= tstop) {
                        float nx[8];
                        slot.get(nx);
                        float w_ = 0.f;
                        if (DKINV && dki0 != nullptr) {
                            float nsq_ = 0.f;
#pragma unroll
                            for (int j = 0; j < 8; j++) nsq_ = fmaf(X[j], X[j], nsq_);
                            nsq_ = rsum(nsq_);
                            const float ki_ = rsqrtf(fmaxf(nsq_, 1e-12f));
                            w_ = nsq_ > 1e-12f ? -(ki_ * ki_ * ki_) * slotw : 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 8; j++) dX[j] += nx[j] + w_ * X[j];
                    }
                    fetch(jb - 2, slot, slotw);
                }
            }
        }
        __syncthreads();
        if (ck - 1 >= c_lo) issue_xo(ck - 1, st ^ 1);       // the undo rows of this chunk are consumed
        // ---------------- (P) token-parallel pass: lane = token, warp = rows warp, warp + 8, ... ----------------
        if (lane < tc) {
            const int t = t0 + lane, sg = lane / G;
            const Tin* xr = reinterpret_cast<const Tin*>(dsm + LY::off_x + st * LY::x_bytes + lane * LY::XRS);
            // one row: 128-long dot of the token vector with the row's S of this token's block
            auto one_row = [&](int rr) {
                const float* Sr = s_S + (size_t)sg * LY::SBS + rr * D;
                float a0_ = 0.f, a1_ = 0.f, a2_ = 0.f, a3_ = 0.f;
#pragma unroll 4
                for (int d = 0; d < D; d += 8) {
                    float xv[8];
                    row8(xv, xr + d);
                    const float4 s0 = ld4(Sr + d / 2), s1 = ld4(Sr + D / 2 + d / 2);      // elements d .. d+3 and d+4 .. d+7
                    a0_ = fmaf(xv[0], s0.x, a0_); a1_ = fmaf(xv[1], s0.y, a1_);
                    a2_ = fmaf(xv[2], s0.z, a2_); a3_ = fmaf(xv[3], s0.w, a3_);
                    a0_ = fmaf(xv[4], s1.x, a0_); a1_ = fmaf(xv[5], s1.y, a1_);
                    a2_ = fmaf(xv[6], s1.z, a2_); a3_ = fmaf(xv[7], s1.w, a3_);
                }
                const float dot = (a0_ + a1_) + (a2_ + a3_);
                Dn[((size_t)bh * T + t) * N + row0 + rr] = fmaf(s_c[rr * RC + lane], dot, -s_xdx[rr * RC + lane]);
            };
            constexpr int NW = ROW_THREADS / 32;
            for (int rr = warp; rr < RPB; rr += 2 * NW) {                  // rows rr and rr + NW of this warp
                const int rb = rr + NW;
                const bool okA = row0 + rr < N && t >= s_ts[rr], okB = rb < RPB && row0 + rb < N && t >= s_ts[rb];
                if (okA && okB) {                                          // both: the token vector is unpacked once
                    const float* SA = s_S + (size_t)sg * LY::SBS + rr * D;
                    const float* SB = s_S + (size_t)sg * LY::SBS + rb * D;
                    float a0_ = 0.f, a1_ = 0.f, a2_ = 0.f, a3_ = 0.f, b0_ = 0.f, b1_ = 0.f, b2_ = 0.f, b3_ = 0.f;
#pragma unroll 4
                    for (int d = 0; d < D; d += 8) {
                        float xv[8];
                        row8(xv, xr + d);
                        const float4 s0 = ld4(SA + d / 2), s1 = ld4(SA + D / 2 + d / 2);
                        const float4 u0 = ld4(SB + d / 2), u1 = ld4(SB + D / 2 + d / 2);
                        a0_ = fmaf(xv[0], s0.x, a0_); a1_ = fmaf(xv[1], s0.y, a1_);
                        a2_ = fmaf(xv[2], s0.z, a2_); a3_ = fmaf(xv[3], s0.w, a3_);
                        b0_ = fmaf(xv[0], u0.x, b0_); b1_ = fmaf(xv[1], u0.y, b1_);
                        b2_ = fmaf(xv[2], u0.z, b2_); b3_ = fmaf(xv[3], u0.w, b3_);
                        a0_ = fmaf(xv[4], s1.x, a0_); a1_ = fmaf(xv[5], s1.y, a1_);
                        a2_ = fmaf(xv[6], s1.z, a2_); a3_ = fmaf(xv[7], s1.w, a3_);
                        b0_ = fmaf(xv[4], u1.x, b0_); b1_ = fmaf(xv[5], u1.y, b1_);
                        b2_ = fmaf(xv[6], u1.z, b2_); b3_ = fmaf(xv[7], u1.w, b3_);
                    }
                    const float dotA = (a0_ + a1_) + (a2_ + a3_), dotB = (b0_ + b1_) + (b2_ + b3_);
                    Dn[((size_t)bh * T + t) * N + row0 + rr] = fmaf(s_c[rr * RC + lane], dotA, -s_xdx[rr * RC + lane]);
                    Dn[((size_t)bh * T + t) * N + row0 + rb] = fmaf(s_c[rb * RC + lane], dotB, -s_xdx[rb * RC + lane]);
                } else if (okA) {
                    one_row(rr);
                } else if (okB) {
                    one_row(rb);
                }
            }
        }
    }
}

}  // namespace slotscan
