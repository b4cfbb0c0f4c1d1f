// Forward address scan: which row does token t write?  [reference addr_fwd, slotkern_cuda.py:72-174]
//
// One CTA of 4 warps per (sequence, head), key rows resident in shared memory as f32 for the whole scan.
// Work split per token: LANE = ROW (row n = lane + 32 s for slot s), WARP = COLUMN QUARTER.  Each lane reads its own
// row slice (row stride DK + 4 floats: the 8 lanes of a quarter-warp fall into 8 different bank groups) against the
// token's query and key slices (broadcast reads) and produces two partial dots, <K_n, q_t> and <K_n, k_t>.  After one
// barrier warp 0 adds the four partials, forms  z_n = temp * qinv * kinv_n * <K_n, q_t> - fr * occ_n  over the
// candidate rows and takes the argmax with two warp reductions (max of an order-preserving key, then min index).
// The row norm is never reduced again: |K_a'|^2 = (1-g)^2 |K_a|^2 + 2 g (1-g) <K_a, k_t> + g^2 |k_t|^2, accumulated in
// double.  After a second barrier every warp blends its column quarter of the chosen row.  Only rows up to the
// highest row touched so far (+1) are visited: everything above is exactly zero.
//
// Against the reference this changes the order of operations (dot first, scale after; the reference normalises
// first), which moves a score by float32 round-off only; addresses are checked against the float64 oracle with a
// 1e-4 margin rule.
#pragma once
#include "slotscan_common.cuh"

namespace slotscan {

#ifdef SLOTSCAN_PHASE_TIMING
static __device__ unsigned long long g_phase_cycles[16];
#define STEP_T0() long long _st = clock64()
#define STEP_MARK(I) do { long long _n = clock64(); _acc[I] += _n - _st; _st = _n; } while (0)
#else
#define STEP_T0()
#define STEP_MARK(I)
#endif

constexpr int CH = 8;                       // tokens staged per chunk
constexpr int AF_THREADS = 128;
constexpr int AF_WARPS = AF_THREADS / 32;

__device__ __forceinline__ unsigned ord_key(float f) {    // monotone float -> unsigned
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

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

struct AddrFwdSmem {       // offsets in floats into dynamic shared memory
    int K, part, tok, tokd, log, cur, Qs, Ks, total;
    int kstride;
};
// N here is the number of key rows held in shared memory (the kernel's `ncap`)
__host__ __device__ inline AddrFwdSmem addr_fwd_layout(int N, int DK, int RPL, int in_bytes) {
    AddrFwdSmem L;
    L.kstride = DK + 4;
    L.K = 0;
    L.part = L.K + N * L.kstride;                 // [RPL][4 warps][32 lanes] float2 partial dots
    L.tok = L.part + RPL * AF_WARPS * 32 * 2;     // [CH] float4: temp*qinv, fr, g, |k|^2
    L.tokd = L.tok + 4 * CH;                      // [CH][4] double: (1-g)^2, 2 g (1-g), g^2 |k|^2, pad
    L.log = L.tokd + 8 * CH;                      // am, oold, kiold [CH each]
    L.cur = L.log + 3 * CH;                       // am, lim of the current token
    L.Qs = L.cur + 4;                             // the chunk's queries and keys in their input dtype
    L.Ks = L.Qs + CH * DK * in_bytes / 4;
    L.total = L.Ks + CH * DK * in_bytes / 4;
    return L;
}

// RPL = row slots per lane (N <= 32 * RPL)
template <int DK, int RPL, bool OCCB, typename Tin>
__global__ void __launch_bounds__(AF_THREADS) addr_fwd_direct_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const Tin* __restrict__ k, const float* __restrict__ gate,
    const float* __restrict__ fr, const float* __restrict__ temp_p, int* __restrict__ am_out,
    float* __restrict__ oold_out, float* __restrict__ kiold_out, float* __restrict__ ofin, int* __restrict__ tfirst,
    const int ncap, const int second_pass) {
    // Two-pass protocol.  Most sequences touch few rows, and a CTA that holds only `ncap` rows is small enough for every
    // (sequence, head) of a large batch to be resident at once.  Pass 1 (ncap < N) runs every sequence; one that
    // needs row ncap gives up, marks itself by tfirst[bh][0] = -1 and leaves.  Pass 2 (ncap = N, second_pass = 1)
    // redoes exactly the marked sequences from the start and returns at once for the others.
    extern __shared__ __align__(16) float smem[];
    constexpr int CW = (DK >= 16) ? DK / 4 : 4;           // columns per warp
    constexpr int NF = CW / 4;                            // float4 per lane and row slice
    constexpr int IPS = CH * DK / 8;                      // 8-element items per stream and chunk
    constexpr int NIT = (2 * IPS + AF_THREADS - 1) / AF_THREADS;
    const int N = p.N, T = p.T, H = p.H;
    const AddrFwdSmem L = addr_fwd_layout(ncap, DK, RPL, (int)sizeof(Tin));
    const int KS = L.kstride;
    float* K = smem + L.K;
    float2* part = reinterpret_cast<float2*>(smem + L.part);
    float* s_tok = smem + L.tok;
    double* s_tokd = reinterpret_cast<double*>(smem + L.tokd);
    int* s_am = reinterpret_cast<int*>(smem + L.log);
    float* s_oold = smem + L.log + CH;
    float* s_kiold = smem + L.log + 2 * CH;
    int* s_cur = reinterpret_cast<int*>(smem + L.cur);
    Tin* Qs = reinterpret_cast<Tin*>(smem + L.Qs);
    Tin* Ks = reinterpret_cast<Tin*>(smem + L.Ks);

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int c0 = warp * CW;                             // first column of this warp
    const bool wact = c0 < DK;
    const float temp = temp_p[0], eps = p.eps;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    if (second_pass && tfirst[(size_t)bh * N] != -1) return;          // finished in the first pass (uniform per CTA)
    __syncthreads();
    for (int i = tid; i < ncap * KS; i += AF_THREADS) K[i] = 0.f;
    for (int i = tid; i < N; i += AF_THREADS) tfirst[(size_t)bh * N + i] = (i == 0) ? 0 : T;

    // ---- chunk loader: 8-element items of q (first IPS) and k (next IPS), gate / fr on 16 threads ----
    Pre8<Tin> pre[NIT];
    float pre_s = 0.f;
#define AF_ISSUE_LOADS(T0)                                                                                 \
    {                                                                                                      \
        _Pragma("unroll") for (int r_ = 0; r_ < NIT; r_++) {                                               \
            const int id_ = tid + r_ * AF_THREADS;                                                         \
            if (id_ < 2 * IPS) {                                                                           \
                const int s_ = id_ / IPS, rr_ = id_ % IPS, j_ = rr_ / (DK / 8), c_ = (rr_ % (DK / 8)) * 8; \
                if ((T0) + j_ < T) pre[r_].load((s_ ? k : q) + (((size_t)b * T + (T0) + j_) * H + h) * DK + c_); \
                else pre[r_].zero();                                                                       \
            }                                                                                              \
        }                                                                                                  \
        if (tid < 2 * CH) {                                                                                \
            const int tt_ = (T0) + (tid & (CH - 1));                                                       \
            const size_t ix_ = ((size_t)b * T + tt_) * H + h;                                              \
            if (tid < CH) pre_s = (tt_ < T) ? gate[ix_] : 0.f;   /* no arithmetic: the load stays in flight */ \
            else pre_s = (tt_ < T) ? (p.fr_per_token ? fr[ix_] : fr[0]) : 0.f;                             \
        }                                                                                                  \
    }
#define AF_COMMIT_LOADS()                                                                                  \
    {                                                                                                      \
        _Pragma("unroll") for (int r_ = 0; r_ < NIT; r_++) {                                               \
            const int id_ = tid + r_ * AF_THREADS;                                                         \
            if (id_ < 2 * IPS) {                                                                           \
                const int s_ = id_ / IPS, rr_ = id_ % IPS;                                                 \
                pre[r_].store_raw((s_ ? Ks : Qs) + rr_ * 8);                                               \
            }                                                                                              \
        }                                                                                                  \
        if (tid < CH) s_tok[4 * tid + 2] = gate_eff(pre_s, p.hard_gate);                                   \
        else if (tid < 2 * CH) s_tok[4 * (tid - CH) + 1] = pre_s;                                          \
    }

    // resolver state (warp 0), per owned row lane + 32 s: |K|^2 (double: the recurrence must not drift),
    // 1 / max(|K|, 1e-6) and the occupancy
    double nsq_r[RPL];
    float kinv_r[RPL], o_r[RPL];
#pragma unroll
    for (int s = 0; s < RPL; s++) { nsq_r[s] = 0.0; kinv_r[s] = 1e6f; o_r[s] = 0.f; }
    int hw = -1, fe = 0, lim = 0;                         // highest row touched; lowest free row (N if none)

    AF_ISSUE_LOADS(0);
    AF_COMMIT_LOADS();
    __syncthreads();

#ifdef SLOTSCAN_PHASE_TIMING
    long long _acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
#endif
    STEP_T0();
    for (int t0 = 0; t0 < T; t0 += CH) {
        const int cn = min(CH, T - t0);
        if (t0 + CH < T) AF_ISSUE_LOADS(t0 + CH);         // next chunk's global loads fly through the whole chunk
        // per-token constants: warp w handles tokens w and w + 4
        for (int j = warp; j < CH; j += AF_WARPS) {
            float qq = 0.f, kk = 0.f;
            for (int cc = lane * 4; cc < DK; cc += 128) {
                const float4 q4 = ld4(Qs + j * DK + cc), k4 = ld4(Ks + j * DK + cc);
                qq += dot4(q4, q4); kk += dot4(k4, k4);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                qq += __shfl_xor_sync(FULL, qq, off);
                kk += __shfl_xor_sync(FULL, kk, off);
            }
            if (lane == 0) {
                s_tok[4 * j] = temp * fminf(rsqrtf(qq), 1e6f);                                        // 1 / max(|q|, 1e-6)
                const double gd = (double)s_tok[4 * j + 2], od = 1.0 - gd;     // |K'|^2 = od^2 |K|^2 + 2 gd od <K,k> + gd^2 |k|^2
                s_tokd[4 * j] = od * od; s_tokd[4 * j + 1] = 2.0 * gd * od; s_tokd[4 * j + 2] = gd * gd * (double)kk;
            }
        }
        __syncthreads();
        STEP_MARK(0);
        for (int j = 0; j < cn; j++) {
            const int t = t0 + j;
            // The step is compiled once per number of live row slots (rows above the highest touched one are exactly
            // zero and are not visited): the common case of few occupied rows runs a short instruction stream.
#define AF_DOTS(NS)                                                                                            \
    {                                                                                                          \
      if (wact) {                                                                                              \
        float4 q4[NF], k4[NF];                                                                                 \
        _Pragma("unroll") for (int i = 0; i < NF; i++) {                                                       \
            q4[i] = ld4(Qs + j * DK + c0 + 4 * i);                                                             \
            k4[i] = ld4(Ks + j * DK + c0 + 4 * i);                                                             \
        }                                                                                                      \
        _Pragma("unroll") for (int s = 0; s < (NS); s++) {                                                     \
            const int n = min(lane + 32 * s, N - 1);                                                           \
            const float* Kr = K + (size_t)n * KS + c0;                                                         \
            float4 aS = zero4, aR = zero4;      /* 8 independent FMA chains; summed once at the end */          \
            _Pragma("unroll") for (int i = 0; i < NF; i++) {                                                   \
                const float4 K4 = ld4(Kr + 4 * i);                                                             \
                aS.x = fmaf(K4.x, q4[i].x, aS.x); aS.y = fmaf(K4.y, q4[i].y, aS.y);                            \
                aS.z = fmaf(K4.z, q4[i].z, aS.z); aS.w = fmaf(K4.w, q4[i].w, aS.w);                            \
                aR.x = fmaf(K4.x, k4[i].x, aR.x); aR.y = fmaf(K4.y, k4[i].y, aR.y);                            \
                aR.z = fmaf(K4.z, k4[i].z, aR.z); aR.w = fmaf(K4.w, k4[i].w, aR.w);                            \
            }                                                                                                  \
            const float a0 = aS.x + aS.y, a1 = aS.z + aS.w, r0 = aR.x + aR.y, r1 = aR.z + aR.w;                \
            part[(s * AF_WARPS + warp) * 32 + lane] = make_float2(a0 + a1, r0 + r1);                           \
        }                                                                                                      \
      }                                                                                                        \
    }
            // lane = row, warp = column quarter
            if (lim < 32) AF_DOTS(1)
            else if (lim < 64) AF_DOTS(RPL < 2 ? RPL : 2)
            else if (lim < 96) AF_DOTS(RPL < 3 ? RPL : 3)
            else if (lim < 128) AF_DOTS(RPL < 4 ? RPL : 4)
            else if (lim < 192) AF_DOTS(RPL < 6 ? RPL : 6)
            else AF_DOTS(RPL)
#undef AF_DOTS
            STEP_MARK(1);
            __syncthreads();
            STEP_MARK(2);
            // ---------------- resolve (warp 0) ----------------
#define AF_RESOLVE(NS)                                                                                         \
    {                                                                                                          \
        float bz = -INFINITY, Rb = 0.f;                                                                        \
        int bi = BIGI;                                                                                         \
        _Pragma("unroll") for (int s = 0; s < (NS); s++) {                                                     \
            const int n = lane + 32 * s;                                                                       \
            float S = 0.f, R = 0.f;                                                                            \
            _Pragma("unroll") for (int w = 0; w < AF_WARPS; w++) {                                             \
                if (w * CW < DK) { const float2 pr = part[(s * AF_WARPS + w) * 32 + lane]; S += pr.x; R += pr.y; } \
            }                                                                                                  \
            const float oc = o_r[s];                                                                           \
            const float sc = tq * (kinv_r[s] * S);                                                             \
            const float z = (OCCB ? (sc - frv * (oc >= eps ? 1.f : 0.f)) : (sc - frv * oc)) + 0.f;             \
            if (n <= lim && (oc >= eps || n == fe) && z > bz) { bz = z; bi = n; Rb = R; }   /* ascending n */  \
        }                                                                                                      \
        const unsigned key = (bi == BIGI) ? 0u : ord_key(bz);                                                  \
        const unsigned kmax = __reduce_max_sync(FULL, key);                                                    \
        am = (int)__reduce_min_sync(FULL, (unsigned)((key == kmax && bi != BIGI) ? bi : BIGI));                \
        /* the owner lane's best row IS am (it holds the maximum), so Rb is <K_am, k_t> there */               \
        const bool owner = (am & 31) == lane;                                                                  \
        const int ai = am >> 5;                                                                                \
        _Pragma("unroll") for (int s = 0; s < (NS); s++) {                                                     \
            if (owner && s == ai) {                                                                            \
                const double nn = fmax(fma(s_tokd[4 * j], nsq_r[s], fma(s_tokd[4 * j + 1], (double)Rb, s_tokd[4 * j + 2])), 0.0); \
                s_am[j] = am; s_oold[j] = o_r[s]; s_kiold[j] = kinv_r[s];                                      \
                nsq_r[s] = nn;                                                                                 \
                kinv_r[s] = fminf(rsqrtf((float)nn), 1e6f);                                                    \
                o_r[s] = __fmaf_rn(omw, o_r[s], g);                                                            \
                o_new = o_r[s];                                                                                \
            }                                                                                                  \
        }                                                                                                      \
    }
            if (warp == 0) {
                const float4 c4 = ld4(s_tok + 4 * j);
                const float tq = c4.x, frv = c4.y, g = c4.z, omw = 1.f - g;
                int am = 0;
                float o_new = 0.f;
                if (lim < 32) AF_RESOLVE(1)
                else if (lim < 64) AF_RESOLVE(RPL < 2 ? RPL : 2)
                else if (lim < 96) AF_RESOLVE(RPL < 3 ? RPL : 3)
                else if (lim < 128) AF_RESOLVE(RPL < 4 ? RPL : 4)
                else if (lim < 192) AF_RESOLVE(RPL < 6 ? RPL : 6)
                else AF_RESOLVE(RPL)
#undef AF_RESOLVE
                o_new = __shfl_sync(FULL, o_new, am & 31);
                if (am > hw) {
                    hw = am;
                    if (lane == 0 && am + 1 < N) tfirst[(size_t)bh * N + am + 1] = t + 1;
                }
                if (am == fe && o_new >= eps) {            // the free row got taken: find the next one
                    int m = BIGI;
#pragma unroll
                    for (int s = RPL - 1; s >= 0; s--) {
                        const int n = lane + 32 * s;
                        if (n < N && o_r[s] < eps) m = n;
                    }
                    m = (int)__reduce_min_sync(FULL, (unsigned)m);
                    fe = (m == BIGI) ? N : m;
                } else if (o_new < eps && am < fe) {
                    fe = am;
                }
                if (lane == 0) { s_cur[0] = am; s_cur[1] = min(hw + 1, N - 1); }   // the next token's candidate limit
            }
            STEP_MARK(3);
            __syncthreads();
            STEP_MARK(4);
            // ---------------- the write: every warp blends its column quarter of the chosen row ----------------
            {
                const int am = s_cur[0];
                lim = s_cur[1];
                if (lim >= ncap) {                         // the next token may address a row this CTA does not hold
                    if (tid == 0) tfirst[(size_t)bh * N] = -1;
                    return;                                // uniform: every thread reads the same s_cur
                }
                if (wact && lane < NF) {
                    const float g = s_tok[4 * j + 2], omw = 1.f - g;
                    float* Kr = K + (size_t)am * KS + c0 + 4 * lane;
                    float4 Kn = ld4(Kr);
                    const float4 kt = ld4(Ks + j * DK + c0 + 4 * lane);
                    Kn.x = blend(Kn.x, kt.x, g, omw); Kn.y = blend(Kn.y, kt.y, g, omw);
                    Kn.z = blend(Kn.z, kt.z, g, omw); Kn.w = blend(Kn.w, kt.w, g, omw);
                    st4(Kr, Kn);
                }
                __syncwarp();                              // a warp only ever reads the columns it writes
            }
            STEP_MARK(5);
        }
        // ---------------- flush the chunk's log, land the next chunk ----------------
        __syncthreads();
        if (tid < cn) {
            const size_t ix = ((size_t)b * T + t0 + tid) * H + h;
            am_out[ix] = s_am[tid];
            oold_out[ix] = s_oold[tid];
            kiold_out[ix] = s_kiold[tid];
        }
        if (t0 + CH < T) AF_COMMIT_LOADS();
        __syncthreads();
        STEP_MARK(6);
    }
#ifdef SLOTSCAN_PHASE_TIMING
    if (tid == 0)
        for (int i = 0; i < 16; i++) atomicAdd(&g_phase_cycles[i], (unsigned long long)_acc[i]);
#endif
#undef AF_ISSUE_LOADS
#undef AF_COMMIT_LOADS
    if (warp == 0) {
#pragma unroll
        for (int s = 0; s < RPL; s++) {
            const int n = lane + 32 * s;
            if (n < N) ofin[(size_t)bh * N + n] = o_r[s];
        }
    }
    for (int n = 32 * RPL + tid; n < N; n += AF_THREADS) ofin[(size_t)bh * N + n] = 0.f;   // rows this pass never held
}

}  // namespace slotscan
