// Forward address scan, chunked: the sequential decision (which row does token t write?) is the only thing left in
// a token-by-token loop, and that loop runs in ONE warp on lane-local numbers prepared for it in bulk.
//
// Per chunk of CH = 8 tokens and per (sequence, head), one CTA of 8 warps does
//   1. score phase (all warps): St[j][n] = <K_n, q_j> and Rt[j][n] = <K_n, k_j> for every row touched so far against
//      the chunk's 8 write queries and 8 keys (key rows resident in shared memory as f32, each lane keeps its token
//      slice in registers, rows are broadcast reads), plus the 8x8 Gram tables Pm = <k_i, q_j>, Gm = <k_i, k_j>;
//   2. resolve phase (warp 0): each lane owns the rows lane, lane + 32, ... and holds their 8 scores of the chunk in
//      registers.  Per token  z_n = temp * qinv * kinv_n * S[n][j] - fr * occ_n  over the candidate rows, argmax by
//      a warp max-reduction and a ballot.  The write itself is NOT executed here: what the next token needs from it
//      follows from linearity of  K_a' = (1-g) K_a + g k_i  and stays inside the owner lane:
//          <K_a', q_j> = (1-g) S[a][j] + g Pm[i][j]          <K_a', k_j> = (1-g) R[a][j] + g Gm[i][j]
//          |K_a'|^2    = (1-g)^2 |K_a|^2 + 2 g (1-g) R[a][i] + g^2 Gm[i][i]       (accumulated in double)
//      so a step has no shared-memory row traffic and no cross-lane hand-off besides the reduction;
//   3. apply phase (all warps): the chunk's writes are executed on the key rows, one warp per written row.
// Against the reference (slotkern_cuda.py:72-174) this changes the order of operations (dot first, scale after;
// the reference normalises first), which moves a score by float32 round-off only; addresses are checked against
// the float64 oracle with a 1e-4 margin rule.
#pragma once
#include "slotscan_common.cuh"

namespace slotscan {

#ifdef SLOTSCAN_PHASE_TIMING
__device__ unsigned long long g_phase_cycles[16];
#define PHASE_T0() long long _pt = clock64()
#define PHASE_MARK(I) do { if (tid == 0) { long long _n = clock64(); _acc[I] += _n - _pt; _pt = _n; } } while (0)
#define STEP_MARK(I) do { long long _n = clock64(); _acc[I] += _n - _st; _st = _n; } while (0)
#else
#define PHASE_T0()
#define PHASE_MARK(I)
#define STEP_MARK(I)
#endif

constexpr int CH = 8;                       // tokens per chunk
constexpr int AF_THREADS = 256;
constexpr int AF_WARPS = AF_THREADS / 32;

__device__ __forceinline__ unsigned ord_key(float f) {    // monotone float -> unsigned
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct AddrFwdSmem {       // offsets in floats into dynamic shared memory
    int K, St, U, Pm, Gm, nsq, misc, Kc, total;    // Kc: the chunk's keys kept in their input dtype (last region)
    int qstride, sstride;
};
// U holds the chunk's queries while they are being copied into registers, then the table Rt for the rest of the chunk.
// St / Rt are token-major ([j][n]): the lanes of the resolver read consecutive rows of one token without conflicts.
__host__ __device__ inline AddrFwdSmem addr_fwd_layout(int N, int DK, int in_bytes) {
    AddrFwdSmem L;
    L.qstride = DK + 4;                     // padded: the 8 tokens of a quarter-warp hit 8 different bank groups
    L.sstride = (N + 3) & ~3;
    const int usz = (CH * L.qstride > CH * L.sstride) ? CH * L.qstride : CH * L.sstride;
    L.K = 0;
    L.St = L.K + N * DK;
    L.U = L.St + CH * L.sstride;
    L.Pm = L.U + usz;
    L.Gm = L.Pm + CH * CH;
    L.nsq = L.Gm + CH * CH;                 // per row: |K|^2 as double (2 floats)
    L.misc = L.nsq + 2 * L.sstride;         // qinv g fr (8 each) | am oold kiold (8 each) | tok[8][4] | hw
    L.Kc = L.misc + 6 * CH + 4 * CH + 8;
    L.total = L.Kc + CH * DK * in_bytes / 4;
    return L;
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

// RPL = rows per lane of the resolver warp (N <= 32 * RPL)
template <int DK, int RPL, bool OCCB, typename Tin>
__global__ void __launch_bounds__(AF_THREADS, 2) addr_fwd_chunked_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const Tin* __restrict__ k, const float* __restrict__ gate,
    const float* __restrict__ fr, const float* __restrict__ temp_p, int* __restrict__ am_out,
    float* __restrict__ oold_out, float* __restrict__ kiold_out, float* __restrict__ ofin, int* __restrict__ tfirst) {
    extern __shared__ __align__(16) float smem[];
    constexpr int NI = (DK + 15) / 16;                  // float4 slices per lane in the score phase
    constexpr int IPS = CH * DK / 8;                    // 8-element items per stream and chunk
    const int N = p.N, T = p.T, H = p.H;
    const AddrFwdSmem L = addr_fwd_layout(N, DK, (int)sizeof(Tin));
    float* K = smem + L.K;
    Tin* Kc = reinterpret_cast<Tin*>(smem + L.Kc);
    float* St = smem + L.St;
    float* Qc = smem + L.U;
    float* Rt = smem + L.U;
    float* Pm = smem + L.Pm;
    float* Gm = smem + L.Gm;
    double* s_nsq = reinterpret_cast<double*>(smem + L.nsq);       // |K_n|^2 (double: the recurrence must not drift)
    float* s_qinv = smem + L.misc;
    float* s_g = s_qinv + CH;
    float* s_fr = s_g + CH;
    int* s_am = reinterpret_cast<int*>(s_fr + CH);
    float* s_oold = reinterpret_cast<float*>(s_am + CH);
    float* s_kiold = s_oold + CH;
    float* s_tok = s_kiold + CH;
    int* s_hw = reinterpret_cast<int*>(s_tok + 4 * CH);

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pj = lane & 7, pp = lane >> 3;            // score phase: token and column part of this lane
    const float temp = temp_p[0], eps = p.eps;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int i = tid; i < N * DK; i += AF_THREADS) K[i] = 0.f;
    for (int i = tid; i < N; i += AF_THREADS) {
        tfirst[(size_t)bh * N + i] = (i == 0) ? 0 : T;
        s_nsq[i] = 0.0;
    }
    if (tid == 0) *s_hw = -1;

    // ---- chunk loader: each thread carries at most one 8-element item of q or k, plus gate / fr on 16 threads ----
    Pre8<Tin> pre;
    float pre_s = 0.f;
    const bool has_item = tid < 2 * IPS;
    const int it_s = has_item ? tid / IPS : 0, it_r = tid % IPS, it_j = it_r / (DK / 8), it_c = (it_r % (DK / 8)) * 8;
#define AF_ISSUE_LOADS(T0)                                                                                 \
    {                                                                                                      \
        const int t_ = (T0) + it_j;                                                                        \
        if (has_item) {                                                                                    \
            if (t_ < T) pre.load((it_s ? k : q) + (((size_t)b * T + t_) * H + h) * DK + it_c);             \
            else pre.zero();                                                                               \
        }                                                                                                  \
        if (tid < 2 * CH) {                                                                                \
            const int tt_ = (T0) + (tid & (CH - 1));                                                       \
            const size_t ix_ = ((size_t)b * T + tt_) * H + h;                                              \
            if (tid < CH) pre_s = (tt_ < T) ? gate[ix_] : 0.f;   /* no arithmetic here: the load must stay in flight */ \
            else pre_s = (tt_ < T) ? (p.fr_per_token ? fr[ix_] : fr[0]) : 0.f;                             \
        }                                                                                                  \
    }
#define AF_COMMIT_LOADS()                                                                                  \
    {                                                                                                      \
        if (has_item) {                                                                                    \
            if (it_s) pre.store_raw(Kc + it_j * DK + it_c); else pre.store(Qc + it_j * L.qstride + it_c);  \
        }                                                                                                  \
        if (tid < CH) s_g[tid] = gate_eff(pre_s, p.hard_gate);                                             \
        else if (tid < 2 * CH) s_fr[tid - CH] = pre_s;                                                     \
    }

    // resolver state (warp 0), per owned row lane + 32 i: 1 / max(|K|, 1e-6) and the occupancy
    float kinv_r[RPL], o_r[RPL];
#pragma unroll
    for (int i = 0; i < RPL; i++) { kinv_r[i] = 1e6f; o_r[i] = 0.f; }
    int hw = -1, fe = 0;                                  // highest row touched; lowest free row (N if none)

    AF_ISSUE_LOADS(0);
    AF_COMMIT_LOADS();
    __syncthreads();

#ifdef SLOTSCAN_PHASE_TIMING
    long long _acc[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    long long _st = 0;
#endif
    PHASE_T0();
    for (int t0 = 0; t0 < T; t0 += CH) {
        const int cn = min(CH, T - t0);
        if (t0 + CH < T) AF_ISSUE_LOADS(t0 + CH);         // next chunk's global loads fly through every phase
        // ---------------- score phase ----------------
        float4 Qr[NI], Kr[NI];
#pragma unroll
        for (int i = 0; i < NI; i++) {
            const int d0 = i * 16 + pp * 4;
            Qr[i] = (d0 < DK) ? ld4(Qc + pj * L.qstride + d0) : zero4;
            Kr[i] = (d0 < DK) ? ld4(Kc + pj * DK + d0) : zero4;
        }
        if (warp == 0) {
            float qq = 0.f;
#pragma unroll
            for (int i = 0; i < NI; i++) qq += dot4(Qr[i], Qr[i]);
            qq += __shfl_xor_sync(FULL, qq, 8);
            qq += __shfl_xor_sync(FULL, qq, 16);
            if (pp == 0) s_qinv[pj] = fminf(rsqrtf(qq), 1e6f);          // 1 / max(|q|, 1e-6)
        }
        __syncthreads();                                  // the queries are in registers: U becomes Rt
        PHASE_MARK(0);
        const int hw0 = *s_hw;
        const int rows = min(hw0 + CH, N - 1) + 1;        // rows that can be candidates before this chunk ends
        for (int n0 = warp; n0 < rows + CH; n0 += 2 * AF_WARPS) {      // two rows per pass: independent FMA chains
            const int n1 = n0 + AF_WARPS;
            const bool key0 = n0 >= rows, key1 = n1 >= rows, has1 = n1 < rows + CH;
            const int m0 = key0 ? n0 - rows : n0, m1 = has1 ? (key1 ? n1 - rows : n1) : m0;
            const bool k1 = has1 ? key1 : key0;
            float aq0 = 0.f, ak0 = 0.f, aq1 = 0.f, ak1 = 0.f;
#pragma unroll
            for (int i = 0; i < NI; i++) {
                const int d0 = i * 16 + pp * 4;
                if (d0 < DK) {
                    const float4 r0 = key0 ? ld4(Kc + m0 * DK + d0) : ld4(K + (size_t)m0 * DK + d0);
                    const float4 r1 = k1 ? ld4(Kc + m1 * DK + d0) : ld4(K + (size_t)m1 * DK + d0);
                    aq0 += dot4(r0, Qr[i]); ak0 += dot4(r0, Kr[i]);
                    aq1 += dot4(r1, Qr[i]); ak1 += dot4(r1, Kr[i]);
                }
            }
            aq0 += __shfl_xor_sync(FULL, aq0, 8);  ak0 += __shfl_xor_sync(FULL, ak0, 8);
            aq1 += __shfl_xor_sync(FULL, aq1, 8);  ak1 += __shfl_xor_sync(FULL, ak1, 8);
            aq0 += __shfl_xor_sync(FULL, aq0, 16); ak0 += __shfl_xor_sync(FULL, ak0, 16);
            aq1 += __shfl_xor_sync(FULL, aq1, 16); ak1 += __shfl_xor_sync(FULL, ak1, 16);
            if (pp == 0) {
                if (key0) { Pm[(n0 - rows) * CH + pj] = aq0; Gm[(n0 - rows) * CH + pj] = ak0; }
                else { St[pj * L.sstride + n0] = aq0; Rt[pj * L.sstride + n0] = ak0; }
                if (has1) {
                    if (key1) { Pm[(n1 - rows) * CH + pj] = aq1; Gm[(n1 - rows) * CH + pj] = ak1; }
                    else { St[pj * L.sstride + n1] = aq1; Rt[pj * L.sstride + n1] = ak1; }
                }
            }
        }
        __syncthreads();
        PHASE_MARK(1);
        // ---------------- resolve phase (warp 0) ----------------
        if (warp == 0) {
            if (lane < CH)         // per-token constants in one 16-byte word: temp * qinv, fr, g, |k|^2
                st4(s_tok + 4 * lane, make_float4(temp * s_qinv[lane], s_fr[lane], s_g[lane], Gm[lane * CH + lane]));
            __syncwarp();
            PHASE_MARK(2);
#ifdef SLOTSCAN_PHASE_TIMING
            _st = clock64();
#endif
            for (int j = 0; j < cn; j++) {
                const int t = t0 + j;
                const float4 c4 = ld4(s_tok + 4 * j);
                const float tq = c4.x, frv = c4.y, g = c4.z, omw = 1.f - g;
                const int lim = min(hw + 1, N - 1);
                const float* Sj = St + j * L.sstride;
                float bz = -INFINITY;
                int bi = BIGI;
#pragma unroll
                for (int i = 0; i < RPL; i++) {
                    if (32 * i <= lim) {                   // uniform: rows above the highest touched one are zero
                        const int n = lane + 32 * i;
                        const float oc = o_r[i];
                        const float s = tq * (kinv_r[i] * Sj[min(n, N - 1)]);
                        const float z = (OCCB ? (s - frv * (oc >= eps ? 1.f : 0.f)) : (s - frv * oc)) + 0.f;
                        if (n <= lim && (oc >= eps || n == fe) && z > bz) { bz = z; bi = n; }   // ascending n
                    }
                }
                STEP_MARK(8);
                const unsigned key = (bi == BIGI) ? 0u : ord_key(bz);
                const unsigned kmax = __reduce_max_sync(FULL, key);
                int am;
                if (lim < 32) am = __ffs(__ballot_sync(FULL, key == kmax && bi != BIGI)) - 1;   // one row per lane
                else am = (int)__reduce_min_sync(FULL, (unsigned)((key == kmax && bi != BIGI) ? bi : BIGI));
                STEP_MARK(9);
                // the write, booked by every lane alike from broadcast reads (no divergence, no hand-off):
                // |K_a'|^2 = (1-g)^2 |K_a|^2 + 2 g (1-g) <K_a, k_t> + g^2 |k_t|^2
                const double gd = (double)g, od = (double)omw;
                const double nn = fmax(od * od * s_nsq[am] + 2.0 * gd * od * (double)Rt[j * L.sstride + am] +
                                       gd * gd * (double)c4.w, 0.0);
                const bool owner = (am & 31) == lane;
                const int ai = am >> 5;
                float o_old = o_r[0], k_old = kinv_r[0];
#pragma unroll
                for (int i = 1; i < RPL; i++)
                    if (i == ai) { o_old = o_r[i]; k_old = kinv_r[i]; }
                o_old = __shfl_sync(FULL, o_old, am & 31);
                k_old = __shfl_sync(FULL, k_old, am & 31);
                const float k_new = fminf(rsqrtf((float)nn), 1e6f), o_new = __fmaf_rn(omw, o_old, g);
#pragma unroll
                for (int i = 0; i < RPL; i++)
                    if (owner && i == ai) { kinv_r[i] = k_new; o_r[i] = o_new; }
                STEP_MARK(10);
                // scores of the chunk's remaining tokens against the rewritten row, by linearity (one lane per token)
                if (lane > j && lane < cn) {
                    float* sp = St + lane * L.sstride + am;
                    float* rp = Rt + lane * L.sstride + am;
                    *sp = blend(*sp, Pm[j * CH + lane], g, omw);
                    *rp = blend(*rp, Gm[j * CH + lane], g, omw);
                }
                if (lane == 0) {
                    s_nsq[am] = nn;
                    s_am[j] = am; s_oold[j] = o_old; s_kiold[j] = k_old;
                    if (am > hw && am + 1 < N) tfirst[(size_t)bh * N + am + 1] = t + 1;
                }
                STEP_MARK(11);
                hw = max(hw, am);
                if (am == fe && o_new >= eps) {            // the free row got taken: find the next one
                    int m = BIGI;
#pragma unroll
                    for (int i = RPL - 1; i >= 0; i--) {
                        const int n = lane + 32 * i;
                        if (n < N && o_r[i] < eps) m = n;
                    }
                    m = (int)__reduce_min_sync(FULL, (unsigned)m);
                    fe = (m == BIGI) ? N : m;
                } else if (o_new < eps && am < fe) {
                    fe = am;
                }
                __syncwarp();
                STEP_MARK(12);
            }
            if (lane == 0) *s_hw = hw;
            PHASE_MARK(3);
        }
        __syncthreads();
        PHASE_MARK(4);
        // ---------------- apply phase: warp j executes token j's write unless a later token rewrites the same row;
        // the warp of the LAST hit replays every hit of its row in order ----------------
        if (warp < cn) {
            const int a = s_am[warp];
            bool last = true;
            for (int j2 = warp + 1; j2 < cn; j2++) last = last && (s_am[j2] != a);
            const int col = lane * 4;
            if (last && col < DK) {
                float4 Kn = ld4(K + (size_t)a * DK + col);
                for (int j = 0; j <= warp; j++) {
                    if (s_am[j] != a) continue;
                    const float g = s_g[j], omw = 1.f - g;
                    const float4 kt = ld4(Kc + j * DK + col);
                    Kn.x = blend(Kn.x, kt.x, g, omw); Kn.y = blend(Kn.y, kt.y, g, omw);
                    Kn.z = blend(Kn.z, kt.z, g, omw); Kn.w = blend(Kn.w, kt.w, g, omw);
                }
                st4(K + (size_t)a * DK + col, Kn);
            }
        }
        if (tid < cn) {
            const size_t ix = ((size_t)b * T + t0 + tid) * H + h;
            am_out[ix] = s_am[tid];
            oold_out[ix] = s_oold[tid];
            kiold_out[ix] = s_kiold[tid];
        }
        __syncthreads();
        PHASE_MARK(5);
        if (t0 + CH < T) AF_COMMIT_LOADS();
        __syncthreads();
        PHASE_MARK(6);
    }
#undef AF_ISSUE_LOADS
#undef AF_COMMIT_LOADS
#ifdef SLOTSCAN_PHASE_TIMING
    if (tid == 0)
        for (int i = 0; i < 16; i++) atomicAdd(&g_phase_cycles[i], (unsigned long long)_acc[i]);
#endif
    if (warp == 0) {
#pragma unroll
        for (int i = 0; i < RPL; i++) {
            const int n = lane + 32 * i;
            if (n < N) ofin[(size_t)bh * N + n] = o_r[i];
        }
    }
}

}  // namespace slotscan
