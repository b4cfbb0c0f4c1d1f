// Forward address scan: which row does token t write?  [reference addr_fwd, slotkern_cuda.py:72-174]
//
// One CTA of 5 warps per (sequence, head), key rows resident in shared memory as f32 for the whole scan.
// Work split per token: LANE = ROW (row n = lane + 32 s for slot s); warps 1-4 each own a COLUMN QUARTER, warp 0
// resolves.  A column warp's lane reads its own row slice (row stride DK + 4 floats: the 8 lanes of a quarter-warp
// fall into 8 different bank groups) against the token's query and key slices (broadcast reads) and produces two
// partial dots, <K_n, q_t> and <K_n, k_t>.  Warp 0 adds the four partials, forms
// z_n = temp * qinv * kinv_n * <K_n, q_t> - fr * occ_n  over the candidate rows and takes the argmax with two warp
// reductions (max of an order-preserving key, then min index).  The row norm is never reduced again:
// |K_a'|^2 = (1-g)^2 |K_a|^2 + 2 g (1-g) <K_a, k_t> + g^2 |k_t|^2, accumulated in double.  The two halves run
// CONCURRENTLY, one token apart (see the schedule comment in the kernel): one barrier per token.  Only rows up to
// the highest row touched so far (+1) are visited: everything above is exactly zero.
//
// Against the reference this changes the order of operations (dot first, scale after; the reference normalises
// first), which moves a score by float32 round-off only; addresses are checked against the float64 oracle with a
// 1e-4 margin rule.
#pragma once
#include <type_traits>

#include "slotscan_common.cuh"

namespace slotscan {

constexpr int CH = 8;                       // tokens staged per chunk
constexpr int AF_CWARPS = 4;                // column warps: each owns a quarter of the key columns
constexpr int AF_THREADS = 32 * (AF_CWARPS + 1);   // + warp 0, the resolver
constexpr int AF_WARPS = AF_THREADS / 32;

// 8 elements of a token stream held in registers between the global load and the shared-memory store
template <typename T> struct Pre8;
template <> struct Pre8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = ld4(p); b = ld4(p + 4); }
    __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void store(float* d) const { st4(d, a); st4(d + 4, b); }
    __device__ __forceinline__ void store_raw(float* d) const { store(d); }
};
template <> struct Pre8<__nv_bfloat16> {
    uint4 u;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { u = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { u = make_uint4(0u, 0u, 0u, 0u); }
    __device__ __forceinline__ void store_raw(__nv_bfloat16* d) const { *reinterpret_cast<uint4*>(d) = u; }
    __device__ __forceinline__ void store(float* d) const {
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
        float f[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            f[2 * i] = t.x; f[2 * i + 1] = t.y;
        }
        st4(d, make_float4(f[0], f[1], f[2], f[3]));
        st4(d + 4, make_float4(f[4], f[5], f[6], f[7]));
    }
};

// tokens staged per chunk of the forward scan: the small variant has shared memory to spare for 16
__host__ __device__ constexpr int af_ch(int RPL) { return RPL <= 2 ? 16 : 8; }

struct AddrFwdSmem {       // offsets in floats into dynamic shared memory
    int K, part, tok, tokd, cross, log, cur, Qs, Ks, total;
    int kstride, stage;    // floats per key row; floats per staged chunk of one stream
};
// N here is the number of key rows held in shared memory (the kernel's `ncap`).  Everything per chunk exists twice:
// the scan runs through chunk boundaries, one chunk is consumed while the next is staged.
__host__ __device__ inline AddrFwdSmem addr_fwd_layout(int N, int DK, int RPL, int in_bytes) {
    AddrFwdSmem L;
    const int C = af_ch(RPL);
    if (RPL <= 2) in_bytes = 4;                   // the small variant stages the chunk as f32 (see Ts in the kernel)
    L.kstride = DK + 4;
    L.stage = C * DK * in_bytes / 4;
    L.K = 0;
    L.part = L.K + N * L.kstride;                 // [2 buffers][RPL][4 column warps][32 lanes] float2 partial dots
    L.tok = L.part + 2 * RPL * AF_CWARPS * 32 * 2;   // [2][C] float4: temp*qinv, fr, g, -
    L.tokd = L.tok + 2 * 4 * C;                   // [2][C][4] double: (1-g)^2, 2 g (1-g), g^2 |k|^2, pad
    L.cross = L.tokd + 2 * 8 * C;                 // [2][C][2]: <k_{t-1}, q_t>, <k_{t-1}, k_t>
    L.log = L.cross + 2 * 2 * C;                  // [2][3][C]: am, oold, kiold
    L.cur = L.log + 2 * 3 * C;                    // the next token's candidate limit, double-buffered by token parity
    L.Qs = L.cur + 4;                             // [2] chunks of queries, then [2] chunks of keys, in_bytes per element
    L.Ks = L.Qs + 2 * L.stage;
    L.total = L.Ks + 2 * L.stage;
    return L;
}

// Per-token constants of the staged chunk, one token per half-warp: temp / max(|q|, 1e-6), the three coefficients of
// the norm recurrence and the cross terms with the previous token's key (kprev).  All 32 lanes must call.
template <int DK, typename Ts>
__device__ __forceinline__ void af_token_consts(const Ts* __restrict__ qrow, const Ts* __restrict__ krow,
                                                const Ts* __restrict__ kprev, int l16, float temp, float* tok4,
                                                double* tokd4, float* cross2) {
    float qq = 0.f, kk = 0.f, pq = 0.f, pk = 0.f;
#pragma unroll
    for (int cc = l16 * 4; cc < DK; cc += 64) {
        const float4 q4 = ld4(qrow + cc), k4 = ld4(krow + cc), kp = ld4(kprev + cc);
        qq += dot4(q4, q4); kk += dot4(k4, k4); pq += dot4(kp, q4); pk += dot4(kp, k4);
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) {
        qq += __shfl_xor_sync(FULL, qq, off); kk += __shfl_xor_sync(FULL, kk, off);
        pq += __shfl_xor_sync(FULL, pq, off); pk += __shfl_xor_sync(FULL, pk, off);
    }
    if (l16 == 0) {
        tok4[0] = temp * fminf(rsqrtf(qq), 1e6f);                          // temp / max(|q|, 1e-6)
        const double gd = (double)tok4[2], od = 1.0 - gd;   // |K'|^2 = od^2 |K|^2 + 2 gd od <K,k> + gd^2 |k|^2
        tokd4[0] = od * od; tokd4[1] = 2.0 * gd * od; tokd4[2] = gd * gd * (double)kk;
        cross2[0] = pq; cross2[1] = pk;
    }
}

// RPL = row slots per lane (N <= 32 * RPL); CARRY: the scan starts from a state carried in from a preceding chunk
template <int DK, int RPL, bool OCCB, bool CARRY, typename Tin>
__global__ void __launch_bounds__(AF_THREADS, (RPL <= 2 ? 3 : 1)) addr_fwd_direct_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const Tin* __restrict__ k, const float* __restrict__ gate,
    const float* __restrict__ fr, const float* __restrict__ temp_p, int* __restrict__ am_out,
    float* __restrict__ oold_out, float* __restrict__ kiold_out, float* __restrict__ ofin, int* __restrict__ tfirst,
    const float* __restrict__ K0, const float* __restrict__ o0, const double* __restrict__ nsq0,
    double* __restrict__ nsqfin, const int ncap, const int second_pass) {
    // Two-pass protocol.  Most sequences touch few rows, and a CTA that holds only `ncap` rows is small enough for every
    // (sequence, head) of a large batch to be resident at once.  Pass 1 (ncap < N) runs every sequence; one that
    // needs row ncap gives up, marks itself by tfirst[bh][0] = -1 and leaves.  Pass 2 (ncap = N, second_pass = 1)
    // redoes exactly the marked sequences from the start and returns at once for the others.
    extern __shared__ __align__(16) float smem[];
    constexpr int C = af_ch(RPL);                         // tokens per staged chunk
    constexpr int RING = 2 * C;                           // token t lives in slot t % RING of every per-token array
    constexpr int CW = (DK >= 16) ? DK / 4 : 4;           // columns per warp
    constexpr int NF = CW / 4;                            // float4 per lane and row slice
    constexpr int LT = AF_THREADS - 32;                   // loader threads: warps 1..4
    constexpr int IPS = C * DK / 8;                       // 8-element items per stream and chunk
    constexpr int NIT = (2 * IPS + LT - 1) / LT;
    // Staging type of the chunk's queries and keys.  Every lane of a column warp reads the warp's whole q and k slice
    // per token, so unpacking bf16 there costs as many instructions as the dots themselves: the small variant converts
    // once per chunk instead.  The full-size variant keeps the input dtype to save shared memory.
    typedef typename std::conditional<(RPL <= 2), float, Tin>::type Ts;
    const int N = p.N, T = p.T, H = p.H;
    const AddrFwdSmem L = addr_fwd_layout(ncap, DK, RPL, (int)sizeof(Tin));
    const int KS = L.kstride;
    float* K = smem + L.K;
    float2* part = reinterpret_cast<float2*>(smem + L.part);
    float* s_tok = smem + L.tok;
    double* s_tokd = reinterpret_cast<double*>(smem + L.tokd);
    float* s_cross = smem + L.cross;
    int* s_am = reinterpret_cast<int*>(smem + L.log);
    float* s_oold = smem + L.log + RING;
    float* s_kiold = smem + L.log + 2 * RING;
    int* s_cur = reinterpret_cast<int*>(smem + L.cur);
    Ts* Qs = reinterpret_cast<Ts*>(smem + L.Qs);
    Ts* Ks = reinterpret_cast<Ts*>(smem + L.Ks);

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ltid = tid - 32;                            // loader thread index (warps 1..4)
    const int cw = warp - 1;                              // column warp index (warp 0 is the resolver)
    const int c0 = cw * CW;                               // first column of this warp
    const bool wact = warp >= 1 && c0 < DK;
    const float temp = temp_p[0], eps = p.eps;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    if (second_pass && tfirst[(size_t)bh * N] != -1) return;          // finished in the first pass (uniform per CTA)
    __syncthreads();
    for (int i = tid; i < ncap * KS; i += AF_THREADS) K[i] = 0.f;
    for (int i = tid; i < DK; i += AF_THREADS) Ks[(RING - 1) * DK + i] = (Ts)0.f;    // "the key before token 0"
    // State carried in from a preceding chunk (K0 / o0, optionally the squared key norms as that scan carried them).
    // hw0 = the highest row it has touched: rows above it are exactly zero, as in a scan from the empty memory.
    int hw0 = -1;
    double* s_nsq = reinterpret_cast<double*>(smem + L.part);         // N doubles, before `part` is first written
    if (CARRY) {
        for (int n = warp; n < N; n += AF_WARPS) {
            double a = 0.0;
            if (nsq0 != nullptr) {
                a = nsq0[(size_t)bh * N + n];
            } else {
                for (int c = lane; c < DK; c += 32) {
                    const double xk = (double)K0[((size_t)bh * N + n) * DK + c];
                    a = fma(xk, xk, a);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(FULL, a, off);
            }
            if (lane == 0) s_nsq[n] = a;
        }
        __syncthreads();
        for (int n = 0; n < N; n++)
            if (s_nsq[n] > 0.0 || o0[(size_t)bh * N + n] != 0.f) hw0 = n;             // same in every thread
        for (int i = tid; i < ncap * DK; i += AF_THREADS) {
            const int n = i / DK, c = i - n * DK;
            K[(size_t)n * KS + c] = K0[((size_t)bh * N + n) * DK + c];
        }
    }
    const int lim0 = CARRY ? min(hw0 + 1, N - 1) : 0;                 // candidate limit of token 0
    for (int i = tid; i < N; i += AF_THREADS) tfirst[(size_t)bh * N + i] = (i <= hw0 + 1) ? 0 : T;
    if (CARRY && lim0 >= ncap) {                                      // the carried-in state already needs more rows
        if (tid == 0) tfirst[(size_t)bh * N] = -1;
        return;
    }

    // ---- chunk loader (warps 1..4): 8-element items of q (first IPS) and k (next IPS); gate / fr on 2 C threads ----
    Pre8<Tin> pre[NIT];
    float pre_s = 0.f;
#define AF_ISSUE_LOADS(T0)                                                                                 \
    {                                                                                                      \
        _Pragma("unroll") for (int r_ = 0; r_ < NIT; r_++) {                                               \
            const int id_ = ltid + r_ * LT;                                                                \
            if (id_ < 2 * IPS) {                                                                           \
                const int s_ = id_ / IPS, rr_ = id_ % IPS, j_ = rr_ / (DK / 8), c_ = (rr_ % (DK / 8)) * 8; \
                if ((T0) + j_ < T) pre[r_].load((s_ ? k : q) + (((size_t)b * T + (T0) + j_) * H + h) * DK + c_); \
                else pre[r_].zero();                                                                       \
            }                                                                                              \
        }                                                                                                  \
        if (ltid < 2 * C) {                                                                                \
            const int tt_ = (T0) + (ltid & (C - 1));                                                       \
            const size_t ix_ = ((size_t)b * T + tt_) * H + h;                                              \
            if (ltid < C) pre_s = (tt_ < T) ? gate[ix_] : 0.f;   /* no arithmetic: the load stays in flight */ \
            else pre_s = (tt_ < T) ? (p.fr_per_token ? fr[ix_] : fr[0]) : 0.f;                             \
        }                                                                                                  \
    }
    // S0 = first ring slot of the chunk (0 or C)
#define AF_COMMIT_LOADS(S0)                                                                                \
    {                                                                                                      \
        _Pragma("unroll") for (int r_ = 0; r_ < NIT; r_++) {                                               \
            const int id_ = ltid + r_ * LT;                                                                \
            if (id_ < 2 * IPS) {                                                                           \
                const int s_ = id_ / IPS, rr_ = id_ % IPS;                                                 \
                Ts* d_ = (s_ ? Ks : Qs) + (S0) * DK + rr_ * 8;                                             \
                if constexpr (std::is_same<Ts, Tin>::value) pre[r_].store_raw(d_);                         \
                else pre[r_].store(d_);                                                                    \
            }                                                                                              \
        }                                                                                                  \
        if (ltid < C) s_tok[4 * ((S0) + ltid) + 2] = gate_eff(pre_s, p.hard_gate);                         \
        else if (ltid < 2 * C) s_tok[4 * ((S0) + ltid - C) + 1] = pre_s;                                   \
    }
    // per-token constants of 8 tokens of the chunk at ring slot S0: one token per half-warp of warps 1..4
#define AF_TOKEN_CONSTS(S0, ROUND)                                                                         \
    {                                                                                                      \
        const int sl_ = (S0) + (ROUND) * 8 + cw * 2 + (lane >> 4), sp_ = (sl_ + RING - 1) & (RING - 1);    \
        af_token_consts<DK, Ts>(Qs + sl_ * DK, Ks + sl_ * DK, Ks + sp_ * DK, lane & 15, temp, s_tok + 4 * sl_, \
                                s_tokd + 4 * sl_, s_cross + 2 * sl_);                                      \
    }

    // Schedule.  The scan never stops at a chunk boundary and has ONE barrier per token.  In the phase of token t
    //   warp 0        finishes the bookkeeping of token t-1 (norm, occupancy, free row: in the shadow of its loads),
    //                 then resolves token t from the partial dots of buffer t & 1;
    //   warps 1..4    apply the write of token t-1 to their column quarter of the rows, then compute the partial dots
    //                 of token t+1 into buffer (t+1) & 1.  Those rows lack exactly one write, token t's, and warp 0
    //                 repairs that one row when it reads the partials, by linearity:
    //                     <K_a', q_{t+1}> = (1-g_t) <K_a, q_{t+1}> + g_t <k_t, q_{t+1}>      (same with k_{t+1})
    //                 with the cross terms <k_t, q_{t+1}>, <k_t, k_{t+1}> computed once per chunk;
    //                 in phases 1..3 of a chunk they also stage the next chunk (loaded one chunk earlier into
    //                 registers), compute its per-token constants and write the previous chunk's log out.
#define AF_DOTS(NS, SL, BUF)                                                                                   \
    {                                                                                                          \
        float4 q4[NF], k4[NF];                                                                                 \
        _Pragma("unroll") for (int i = 0; i < NF; i++) {                                                       \
            q4[i] = ld4(Qs + (SL) * DK + c0 + 4 * i);                                                          \
            k4[i] = ld4(Ks + (SL) * DK + c0 + 4 * i);                                                          \
        }                                                                                                      \
        _Pragma("unroll") for (int s = 0; s < (NS); s++) {                                                     \
            const int n = min(lane + 32 * s, ncap - 1);                                                        \
            const float* Kr = K + (size_t)n * KS + c0;                                                         \
            float4 aS = zero4, aR = zero4;      /* 8 independent FMA chains; summed once at the end */          \
            _Pragma("unroll") for (int i = 0; i < NF; i++) {                                                   \
                const float4 K4 = ld4(Kr + 4 * i);                                                             \
                aS.x = fmaf(K4.x, q4[i].x, aS.x); aS.y = fmaf(K4.y, q4[i].y, aS.y);                            \
                aS.z = fmaf(K4.z, q4[i].z, aS.z); aS.w = fmaf(K4.w, q4[i].w, aS.w);                            \
                aR.x = fmaf(K4.x, k4[i].x, aR.x); aR.y = fmaf(K4.y, k4[i].y, aR.y);                            \
                aR.z = fmaf(K4.z, k4[i].z, aR.z); aR.w = fmaf(K4.w, k4[i].w, aR.w);                            \
            }                                                                                                  \
            part[(((BUF) * RPL + s) * AF_CWARPS + cw) * 32 + lane] =                                           \
                make_float2((aS.x + aS.y) + (aS.z + aS.w), (aR.x + aR.y) + (aR.z + aR.w));                     \
        }                                                                                                      \
    }
    // Few live rows (< 32 / F): a lane takes row lane % (32 / F) and the F-th part lane / (32 / F) of the warp's columns,
    // and F lanes add up by shuffles.  What bounds this kernel is the shared-memory return path (every LDS.128 delivers
    // 512 B to the warp, broadcast or not): F-fold fewer loads per token for the same rows.
#define AF_DOTS_SPLIT(F, SL, BUF)                                                                              \
    {                                                                                                          \
        constexpr int FF = (NF >= (F)) ? (F) : 1, R_ = 32 / FF, NFS = NF / FF;                                 \
        const int cb = c0 + (lane / R_) * (CW / FF);                                                           \
        float4 q4[NFS], k4[NFS];                                                                               \
        _Pragma("unroll") for (int i = 0; i < NFS; i++) {                                                      \
            q4[i] = ld4(Qs + (SL) * DK + cb + 4 * i);                                                          \
            k4[i] = ld4(Ks + (SL) * DK + cb + 4 * i);                                                          \
        }                                                                                                      \
        const float* Kr = K + (size_t)min(lane & (R_ - 1), ncap - 1) * KS + cb;                                \
        float4 aS = zero4, aR = zero4;                                                                         \
        _Pragma("unroll") for (int i = 0; i < NFS; i++) {                                                      \
            const float4 K4 = ld4(Kr + 4 * i);                                                                 \
            aS.x = fmaf(K4.x, q4[i].x, aS.x); aS.y = fmaf(K4.y, q4[i].y, aS.y);                                \
            aS.z = fmaf(K4.z, q4[i].z, aS.z); aS.w = fmaf(K4.w, q4[i].w, aS.w);                                \
            aR.x = fmaf(K4.x, k4[i].x, aR.x); aR.y = fmaf(K4.y, k4[i].y, aR.y);                                \
            aR.z = fmaf(K4.z, k4[i].z, aR.z); aR.w = fmaf(K4.w, k4[i].w, aR.w);                                \
        }                                                                                                      \
        float sS = (aS.x + aS.y) + (aS.z + aS.w), sR = (aR.x + aR.y) + (aR.z + aR.w);                          \
        _Pragma("unroll") for (int off = 16; off >= R_; off >>= 1) {                                           \
            sS += __shfl_xor_sync(FULL, sS, off);                                                              \
            sR += __shfl_xor_sync(FULL, sR, off);                                                              \
        }                                                                                                      \
        if (lane < R_) part[((BUF) * RPL * AF_CWARPS + cw) * 32 + lane] = make_float2(sS, sR);                 \
    }
    // compiled once per number of live rows: rows above the candidate limit are exactly zero and not visited
#define AF_DOTS_DISPATCH(LIMD, SL, BUF)                                  \
    if ((LIMD) < 8) AF_DOTS_SPLIT(4, SL, BUF)                            \
    else if ((LIMD) < 16) AF_DOTS_SPLIT(2, SL, BUF)                      \
    else if ((LIMD) < 32) AF_DOTS(1, SL, BUF)                            \
    else if ((LIMD) < 64) AF_DOTS((RPL < 2 ? RPL : 2), SL, BUF)          \
    else if ((LIMD) < 96) AF_DOTS((RPL < 3 ? RPL : 3), SL, BUF)          \
    else if ((LIMD) < 128) AF_DOTS((RPL < 4 ? RPL : 4), SL, BUF)         \
    else AF_DOTS(RPL, SL, BUF)
#define AF_WRITE_ROW(SL)                                                                                       \
    if (lane < NF) {                                                                                           \
        const int a_ = s_am[SL];                                                                               \
        const float g_ = s_tok[4 * (SL) + 2], omw_ = 1.f - g_;                                                 \
        const float4 kt_ = ld4(Ks + (SL) * DK + c0 + 4 * lane);                                                \
        float* Kr_ = K + (size_t)a_ * KS + c0 + 4 * lane;                                                      \
        float4 Kn_ = ld4(Kr_);                                                                                 \
        Kn_.x = blend(Kn_.x, kt_.x, g_, omw_); Kn_.y = blend(Kn_.y, kt_.y, g_, omw_);                          \
        Kn_.z = blend(Kn_.z, kt_.z, g_, omw_); Kn_.w = blend(Kn_.w, kt_.w, g_, omw_);                          \
        st4(Kr_, Kn_);                                                                                         \
    }                                                                                                          \
    __syncwarp();      /* a column warp only ever reads the columns it writes */
    // warp 0: the bookkeeping of the token resolved in the previous phase (am_prev, its constants in pc, the owner
    // lane's <K_am, k> in Rb_prev).  The owner lane is the one that holds row am_prev.
#define AF_FINISH_PREV(NS)                                                                                     \
    if (am_prev >= 0) {                                                                                        \
        const bool owner_ = (am_prev & 31) == lane;                                                            \
        const int ai_ = am_prev >> 5;                                                                          \
        float o_new = 0.f;                                                                                     \
        _Pragma("unroll") for (int s = 0; s < (NS); s++) {                                                     \
            if (owner_ && s == ai_) {                                                                          \
                const double nn = fmax(fma(pc.d0, nsq_r[s], fma(pc.d1, (double)Rb_prev, pc.d2)), 0.0);         \
                s_oold[pslot] = o_r[s]; s_kiold[pslot] = kinv_r[s];                                            \
                nsq_r[s] = nn;                                                                                 \
                kinv_r[s] = fminf(rsqrtf((float)nn), 1e6f);                                                    \
                o_r[s] = __fmaf_rn(1.f - pc.g, o_r[s], pc.g);                                                  \
                o_new = o_r[s];                                                                                \
            }                                                                                                  \
        }                                                                                                      \
        o_new = __shfl_sync(FULL, o_new, am_prev & 31);                                                        \
        if (am_prev == fe && o_new >= eps) {               /* the free row got taken: find the next one */     \
            int m = BIGI;                                                                                      \
            _Pragma("unroll") for (int s = RPL - 1; s >= 0; s--) {                                             \
                const int n = lane + 32 * s;                                                                   \
                if (n < N && o_r[s] < eps) m = n;                                                              \
            }                                                                                                  \
            m = (int)__reduce_min_sync(FULL, (unsigned)m);                                                     \
            fe = (m == BIGI) ? N : m;                                                                          \
        } else if (o_new < eps && am_prev < fe) {                                                              \
            fe = am_prev;                                                                                      \
        }                                                                                                      \
    }
#define AF_RESOLVE(NS, BUF)                                                                                    \
    {                                                                                                          \
        float2 pr[NS][AF_CWARPS];                                                                              \
        _Pragma("unroll") for (int s = 0; s < (NS); s++)                                                       \
            _Pragma("unroll") for (int w = 0; w < AF_CWARPS; w++)                                              \
                if (w * CW < DK) pr[s][w] = part[(((BUF) * RPL + s) * AF_CWARPS + w) * 32 + lane];             \
        AF_FINISH_PREV(NS)                                                                                     \
        float bz = -INFINITY;                                                                                  \
        int bi = BIGI;                                                                                         \
        Rb = 0.f;                                                                                              \
        _Pragma("unroll") for (int s = 0; s < (NS); s++) {                                                     \
            const int n = lane + 32 * s;                                                                       \
            float S = 0.f, R = 0.f;                                                                            \
            _Pragma("unroll") for (int w = 0; w < AF_CWARPS; w++)                                              \
                if (w * CW < DK) { S += pr[s][w].x; R += pr[s][w].y; }                                         \
            if (n == am_prev) {    /* the one row whose latest write the dots have not seen */                 \
                S = blend(S, cc.x0, pc.g, 1.f - pc.g);                                                         \
                R = blend(R, cc.x1, pc.g, 1.f - pc.g);                                                         \
            }                                                                                                  \
            const float oc = o_r[s];                                                                           \
            const float sc = cc.tq * (kinv_r[s] * S);                                                          \
            const float z = (OCCB ? (sc - cc.frv * (oc >= eps ? 1.f : 0.f)) : (sc - cc.frv * oc)) + 0.f;       \
            if (n <= lim && (oc >= eps || n == fe) && z > bz) { bz = z; bi = n; Rb = R; }   /* ascending n */  \
        }                                                                                                      \
        const unsigned key = (bi == BIGI) ? 0u : ord_key(bz);                                                  \
        const unsigned kmax = __reduce_max_sync(FULL, key);                                                    \
        am = (int)__reduce_min_sync(FULL, (unsigned)((key == kmax && bi != BIGI) ? bi : BIGI));                \
        am = min(am, lim);         /* no candidate compares greater (NaN scores): stay inside the rows */      \
        /* the owner lane's best row IS am (it holds the maximum), so its Rb is <K_am, k_t> */                 \
    }
    struct TokC { float tq, frv, g, x0, x1; double d0, d1, d2; };
#define AF_LOAD_CONSTS(DST, SL)                                                                                \
    {                                                                                                          \
        const float4 c4_ = ld4(s_tok + 4 * (SL));                                                              \
        const float2 x2_ = *reinterpret_cast<const float2*>(s_cross + 2 * (SL));                               \
        const double2 d2_ = *reinterpret_cast<const double2*>(s_tokd + 4 * (SL));                              \
        DST.tq = c4_.x; DST.frv = c4_.y; DST.g = c4_.z; DST.x0 = x2_.x; DST.x1 = x2_.y;                        \
        DST.d0 = d2_.x; DST.d1 = d2_.y; DST.d2 = s_tokd[4 * (SL) + 2];                                         \
    }

    // resolver state (warp 0), per owned row lane + 32 s: |K|^2 (double: the recurrence must not drift),
    // 1 / max(|K|, 1e-6) and the occupancy
    double nsq_r[RPL];
    float kinv_r[RPL], o_r[RPL];
#pragma unroll
    for (int s = 0; s < RPL; s++) { nsq_r[s] = 0.0; kinv_r[s] = 1e6f; o_r[s] = 0.f; }
    int hw = hw0, fe = 0, lim = lim0;                     // highest row touched; lowest free row (N if none)
    if (CARRY && warp == 0) {
        int m = BIGI;
#pragma unroll
        for (int s = RPL - 1; s >= 0; s--) {
            const int n = lane + 32 * s;
            if (n < N) {
                nsq_r[s] = s_nsq[n];
                kinv_r[s] = fminf(rsqrtf((float)nsq_r[s]), 1e6f);
                o_r[s] = o0[(size_t)bh * N + n];
                if (o_r[s] < eps) m = n;
            }
        }
        m = (int)__reduce_min_sync(FULL, (unsigned)m);
        fe = (m == BIGI) ? N : m;
    }
    int am_prev = -1, pslot = 0;                          // the token whose bookkeeping is still open
    float Rb_prev = 0.f;
    TokC cc = {}, pc = {}, nc = {};                       // constants of the current, previous and next token

    // ---- prologue: stage chunk 0, its constants, the plain dots of token 0 ----
    if (warp >= 1) {
        AF_ISSUE_LOADS(0);
        AF_COMMIT_LOADS(0);
    }
    __syncthreads();
    if (warp >= 1) {
        if (C < T) AF_ISSUE_LOADS(C);
#pragma unroll
        for (int r = 0; r < C / 8; r++) AF_TOKEN_CONSTS(0, r);
    }
    __syncthreads();
    if (wact) {
        if (CARRY) { AF_DOTS_DISPATCH(lim0, 0, 0) }
        else { AF_DOTS_SPLIT(4, 0, 0) }
    }
    if (warp == 0) AF_LOAD_CONSTS(cc, 0);
    __syncthreads();

    // The two roles run separate loops (their register states never mix) and meet at one named barrier per token.
#define AF_PHASE_BARRIER() asm volatile("bar.sync 1, %0;" ::"n"(AF_THREADS) : "memory")
    if (warp == 0) {
        for (int t = 0; t < T; t++) {
            const int sl = t & (RING - 1);
            if (t + 1 < T) AF_LOAD_CONSTS(nc, (t + 1) & (RING - 1));
            int am = 0;
            float Rb = 0.f;
            if (lim < 32) AF_RESOLVE(1, t & 1)
            else if (lim < 64) AF_RESOLVE((RPL < 2 ? RPL : 2), t & 1)
            else if (lim < 96) AF_RESOLVE((RPL < 3 ? RPL : 3), t & 1)
            else if (lim < 128) AF_RESOLVE((RPL < 4 ? RPL : 4), t & 1)
            else AF_RESOLVE(RPL, t & 1)
            if (am > hw) {
                hw = am;
                if (lane == 0 && am + 1 < N) tfirst[(size_t)bh * N + am + 1] = t + 1;
            }
            lim = min(hw + 1, N - 1);                      // the next token's candidate limit
            if (lane == 0) {
                s_am[sl] = am;
                s_cur[t & 1] = lim;
            }
            am_prev = am; Rb_prev = Rb; pslot = sl;
            pc = cc; cc = nc;
            AF_PHASE_BARRIER();
            if (lim >= ncap) {                             // the next token may address a row this CTA does not hold
                if (lane == 0) tfirst[(size_t)bh * N] = -1;
                return;                                    // the column warps read the same limit and leave too
            }
        }
        AF_FINISH_PREV(RPL)
#pragma unroll
        for (int s = 0; s < RPL; s++) {
            const int n = lane + 32 * s;
            if (n < N) {
                ofin[(size_t)bh * N + n] = o_r[s];
                if (nsqfin != nullptr) nsqfin[(size_t)bh * N + n] = nsq_r[s];
            }
        }
    } else {
        for (int t = 0; t < T; t++) {
            const int jj = t & (C - 1);
            if (wact) {
                if (t >= 1) { AF_WRITE_ROW((t - 1) & (RING - 1)) }
                if (t + 1 < T) {
                    const int limd = min(lim + 1, ncap - 1);      // token t can raise the candidate limit by one
                    AF_DOTS_DISPATCH(limd, (t + 1) & (RING - 1), (t + 1) & 1)
                }
            }
            // chunk duties, spread over the phases 1.. of the chunk
            const int tn = t - jj + C;                     // first token of the next chunk
            if (jj == 1) {
                if (t - jj >= C && ltid < C) {             // the previous chunk's log goes out
                    const int tp = t - jj - C + ltid, sp = tp & (RING - 1);
                    const size_t ix = ((size_t)b * T + tp) * H + h;
                    am_out[ix] = s_am[sp];
                    oold_out[ix] = s_oold[sp];
                    kiold_out[ix] = s_kiold[sp];
                }
                if (tn < T) {
                    AF_COMMIT_LOADS(tn & (RING - 1));
                    if (tn + C < T) AF_ISSUE_LOADS(tn + C);
                }
            } else if (jj >= 2 && jj < 2 + C / 8 && tn < T) {
                AF_TOKEN_CONSTS(tn & (RING - 1), jj - 2);
            }
            AF_PHASE_BARRIER();
            lim = s_cur[t & 1];
            if (lim >= ncap) return;
        }
    }
#undef AF_PHASE_BARRIER
    for (int n = 32 * RPL + tid; n < N; n += AF_THREADS) {                                // rows this pass never held
        ofin[(size_t)bh * N + n] = 0.f;
        if (nsqfin != nullptr) nsqfin[(size_t)bh * N + n] = 0.0;
    }
    __syncthreads();
    {   // the log entries not written out yet: the last chunk, and the one before it if the last stopped before phase 1
        const int cl = (T - 1) / C;
        const int f0 = (((T - 1) & (C - 1)) >= 1 ? cl : max(cl - 1, 0)) * C;
        for (int tp = f0 + tid; tp < T; tp += AF_THREADS) {
            const int sp = tp & (RING - 1);
            const size_t ix = ((size_t)b * T + tp) * H + h;
            am_out[ix] = s_am[sp];
            oold_out[ix] = s_oold[sp];
            kiold_out[ix] = s_kiold[sp];
        }
    }
#undef AF_DOTS
#undef AF_DOTS_DISPATCH
#undef AF_DOTS_SPLIT
#undef AF_WRITE_ROW
#undef AF_FINISH_PREV
#undef AF_RESOLVE
#undef AF_LOAD_CONSTS
#undef AF_TOKEN_CONSTS
#undef AF_ISSUE_LOADS
#undef AF_COMMIT_LOADS
}

}  // namespace slotscan
