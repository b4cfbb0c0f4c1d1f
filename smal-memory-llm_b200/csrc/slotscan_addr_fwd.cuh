// Forward address scan, chunked: the sequential decision (which row does token t write?) is the only thing left in
// a token-by-token loop, and that loop runs in ONE warp on lane-local numbers prepared for it in bulk.
//
// Per chunk of CH = 8 tokens and per (sequence, head), one CTA of 8 warps does
//   1. score phase (all warps): St[j][n] = <K_n, q_j> and Rt[j][n] = <K_n, k_j> for every row touched so far against
//      the chunk's 8 write queries and 8 keys (key rows resident in shared memory as f32, each lane keeps its token
//      slice in registers, rows are broadcast reads), plus the 8x8 Gram tables Pm = <k_i, q_j>, Gm = <k_i, k_j>;
//   2. resolve phase (warp 0): per token  z_n = temp * qinv * kinv_n * St[j][n] - fr * occ_n  over the candidate
//      rows, argmax by two warp reductions.  The write itself is NOT executed here: what the next token needs from
//      it follows from linearity of  K_a' = (1-g) K_a + g k_i :
//          <K_a', q_j> = (1-g) St[j][a] + g Pm[i][j]          <K_a', k_j> = (1-g) Rt[j][a] + g Gm[i][j]
//          |K_a'|^2    = (1-g)^2 |K_a|^2 + 2 g (1-g) Rt[i][a] + g^2 Gm[i][i]
//      so a step is a few lane-local operations and two reductions, with no shared-memory row traffic;
//   3. apply phase (all warps): the chunk's writes are applied to the key rows in order, and the norm of every row
//      written is recomputed from the row itself, so the recurrence above never carries error past one chunk.
// Against the reference (slotkern_cuda.py:72-174) this changes the order of operations (dot first, scale after;
// the reference normalises first), which moves a score by float32 round-off only; addresses are checked against
// the float64 oracle with a 1e-4 margin rule.
#pragma once
#include "slotscan_common.cuh"

namespace slotscan {

constexpr int CH = 8;                       // tokens per chunk
constexpr int AF_THREADS = 256;
constexpr int AF_WARPS = AF_THREADS / 32;

__device__ __forceinline__ unsigned ord_key(float f) {    // monotone float -> unsigned
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct AddrFwdSmem {       // offsets in floats into dynamic shared memory
    int K, Kc, St, U, Pm, Gm, misc, total;
    int qstride, sstride;
};
// U holds the chunk's queries while they are being copied into registers, then the table Rt for the rest of the chunk.
__host__ __device__ inline AddrFwdSmem addr_fwd_layout(int N, int DK) {
    AddrFwdSmem L;
    L.qstride = DK + 4;                     // padded: the 8 tokens of a quarter-warp hit 8 different bank groups
    L.sstride = (N + 3) & ~3;
    const int usz = (CH * L.qstride > CH * L.sstride) ? CH * L.qstride : CH * L.sstride;
    L.K = 0;
    L.Kc = L.K + N * DK;
    L.St = L.Kc + CH * DK;
    L.U = L.St + CH * L.sstride;
    L.Pm = L.U + usz;
    L.Gm = L.Pm + CH * CH;
    L.misc = L.Gm + CH * CH;                // qinv g fr | am oold kiold nsqx (8 each) | hw
    L.total = L.misc + 7 * CH + 8;
    return L;
}

// RPL = rows per lane of the resolver warp (N <= 32 * RPL)
template <int DK, int RPL, typename Tin>
__global__ void __launch_bounds__(AF_THREADS, 2) addr_fwd_chunked_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const Tin* __restrict__ k, const float* __restrict__ gate,
    const float* __restrict__ fr, const float* __restrict__ temp_p, int* __restrict__ am_out,
    float* __restrict__ oold_out, float* __restrict__ kiold_out, float* __restrict__ ofin, int* __restrict__ tfirst) {
    extern __shared__ __align__(16) float smem[];
    constexpr int NI = (DK + 15) / 16;                  // float4 slices per lane in the score phase
    constexpr int IPS = CH * DK / 8;                    // 8-element items per stream and chunk
    const int N = p.N, T = p.T, H = p.H;
    const AddrFwdSmem L = addr_fwd_layout(N, DK);
    float* K = smem + L.K;
    float* Kc = smem + L.Kc;
    float* St = smem + L.St;
    float* Qc = smem + L.U;
    float* Rt = smem + L.U;
    float* Pm = smem + L.Pm;
    float* Gm = smem + L.Gm;
    float* s_qinv = smem + L.misc;
    float* s_g = s_qinv + CH;
    float* s_fr = s_g + CH;
    int* s_am = reinterpret_cast<int*>(s_fr + CH);
    float* s_oold = reinterpret_cast<float*>(s_am + CH);
    float* s_kiold = s_oold + CH;
    float* s_nsqx = s_kiold + CH;
    int* s_hw = reinterpret_cast<int*>(s_nsqx + CH);

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pj = lane & 7, pp = lane >> 3;            // score phase: token and column part of this lane
    const float temp = temp_p[0], eps = p.eps;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int i = tid; i < N * DK; i += AF_THREADS) K[i] = 0.f;
    for (int i = tid; i < N; i += AF_THREADS) tfirst[(size_t)bh * N + i] = (i == 0) ? 0 : T;
    if (tid == 0) *s_hw = -1;
    if (tid < CH) { s_nsqx[tid] = -1.f; s_am[tid] = 0; }

    // ---- chunk loader: each thread carries at most one 8-element item of q or k, plus gate / fr on 16 threads ----
    float pre[8];
    float pre_s = 0.f;
    const bool has_item = tid < 2 * IPS;
    const int it_s = has_item ? tid / IPS : 0, it_r = tid % IPS, it_j = it_r / (DK / 8), it_c = (it_r % (DK / 8)) * 8;
    auto issue_loads = [&](int t0) {
        const int t = t0 + it_j;
        if (has_item) {
            if (t < T) ld8(pre, (it_s ? k : q) + (((size_t)b * T + t) * H + h) * DK + it_c);
            else {
#pragma unroll
                for (int e = 0; e < 8; e++) pre[e] = 0.f;
            }
        }
        if (tid < 2 * CH) {
            const int tt = t0 + (tid & (CH - 1));
            const size_t ix = ((size_t)b * T + tt) * H + h;
            if (tid < CH) pre_s = (tt < T) ? gate_eff(gate[ix], p.hard_gate) : 0.f;
            else pre_s = (tt < T) ? (p.fr_per_token ? fr[ix] : fr[0]) : 0.f;
        }
    };
    auto commit_loads = [&]() {
        if (has_item) {
            float* dst = it_s ? (Kc + it_j * DK + it_c) : (Qc + it_j * L.qstride + it_c);
            st4(dst, make_float4(pre[0], pre[1], pre[2], pre[3]));
            st4(dst + 4, make_float4(pre[4], pre[5], pre[6], pre[7]));
        }
        if (tid < CH) s_g[tid] = pre_s;
        else if (tid < 2 * CH) s_fr[tid - CH] = pre_s;
    };

    // resolver state (warp 0): squared norm, its inverse root and the occupancy of the rows lane + 32 i, in registers
    float nsq_r[RPL], kinv_r[RPL], o_r[RPL];
#pragma unroll
    for (int i = 0; i < RPL; i++) { nsq_r[i] = 0.f; kinv_r[i] = 1e6f; o_r[i] = 0.f; }   // 1 / max(|0|, 1e-6)
    int hw = -1, fe = 0;                                  // highest row touched; lowest free row (N if none)

    issue_loads(0);
    commit_loads();
    __syncthreads();

    for (int t0 = 0; t0 < T; t0 += CH) {
        const int cn = min(CH, T - t0);
        if (t0 + CH < T) issue_loads(t0 + CH);            // next chunk's global loads fly through every phase
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
            if (pp == 0) s_qinv[pj] = 1.f / fmaxf(sqrtf(qq), 1e-6f);
        }
        __syncthreads();                                  // the queries are in registers: U becomes Rt
        {
            const int hw0 = *s_hw;
            const int rows = min(hw0 + CH, N - 1) + 1;    // rows that can be candidates before this chunk ends
            for (int n = warp; n < rows + CH; n += AF_WARPS) {
                const bool is_key = n >= rows;            // the chunk's own keys ride along as 8 extra rows
                const float* row = is_key ? (Kc + (n - rows) * DK) : (K + (size_t)n * DK);
                float aq = 0.f, ak = 0.f;
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    const int d0 = i * 16 + pp * 4;
                    if (d0 < DK) {
                        const float4 r4 = ld4(row + d0);
                        aq += dot4(r4, Qr[i]);
                        ak += dot4(r4, Kr[i]);
                    }
                }
                aq += __shfl_xor_sync(FULL, aq, 8);  ak += __shfl_xor_sync(FULL, ak, 8);
                aq += __shfl_xor_sync(FULL, aq, 16); ak += __shfl_xor_sync(FULL, ak, 16);
                if (pp == 0) {
                    if (is_key) { Pm[(n - rows) * CH + pj] = aq; Gm[(n - rows) * CH + pj] = ak; }
                    else { St[pj * L.sstride + n] = aq; Rt[pj * L.sstride + n] = ak; }
                }
            }
        }
        __syncthreads();
        // ---------------- resolve phase (warp 0) ----------------
        if (warp == 0) {
            // norms recomputed from the rows the previous chunk wrote replace the recurrence values
#pragma unroll
            for (int j = 0; j < CH; j++) {
                const float x = s_nsqx[j];
                const int a = s_am[j];
                if (x >= 0.f && (a & 31) == lane) {
#pragma unroll
                    for (int i = 0; i < RPL; i++)
                        if (i == (a >> 5)) { nsq_r[i] = x; kinv_r[i] = 1.f / fmaxf(sqrtf(x), 1e-6f); }
                }
            }
            __syncwarp();
            for (int j = 0; j < cn; j++) {
                const int t = t0 + j;
                const float tq = temp * s_qinv[j], frv = s_fr[j], g = s_g[j], omw = 1.f - g;
                const int lim = min(hw + 1, N - 1);
                float bz = -INFINITY;
                int bi = BIGI;
#pragma unroll
                for (int i = 0; i < RPL; i++) {
                    const int n = lane + 32 * i;
                    if (n <= lim) {
                        const float oc = o_r[i];
                        const float s = tq * (kinv_r[i] * St[j * L.sstride + n]);
                        const float z = (p.occ_bin ? (s - frv * (oc >= eps ? 1.f : 0.f)) : (s - frv * oc)) + 0.f;
                        if ((oc >= eps || n == fe) && z > bz) { bz = z; bi = n; }   // ascending n: first maximum kept
                    }
                }
                const unsigned key = (bi == BIGI) ? 0u : ord_key(bz);
                const unsigned kmax = __reduce_max_sync(FULL, key);
                const int am = (int)__reduce_min_sync(FULL, (unsigned)((key == kmax && bi != BIGI) ? bi : BIGI));
                const int ai = am >> 5;
                float o_new = 0.f;
                if ((am & 31) == lane) {                   // the owner lane books the write
                    const float R = Rt[j * L.sstride + am], kk = Gm[j * CH + j];
#pragma unroll
                    for (int i = 0; i < RPL; i++) {
                        if (i == ai) {
                            s_am[j] = am; s_oold[j] = o_r[i]; s_kiold[j] = kinv_r[i];
                            const float nn = fmaxf(omw * omw * nsq_r[i] + 2.f * g * omw * R + g * g * kk, 0.f);
                            nsq_r[i] = nn;
                            kinv_r[i] = 1.f / fmaxf(sqrtf(nn), 1e-6f);
                            o_r[i] = __fmaf_rn(omw, o_r[i], g);
                            o_new = o_r[i];
                        }
                    }
                }
                o_new = __shfl_sync(FULL, o_new, am & 31);
                // what the chunk's remaining tokens see of the rewritten row, by linearity
                if (lane > j && lane < cn) {
                    float* sp = St + lane * L.sstride + am;
                    float* rp = Rt + lane * L.sstride + am;
                    *sp = blend(*sp, Pm[j * CH + lane], g, omw);
                    *rp = blend(*rp, Gm[j * CH + lane], g, omw);
                }
                if (am > hw) {
                    hw = am;
                    if (lane == 0 && am + 1 < N) tfirst[(size_t)bh * N + am + 1] = t + 1;
                }
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
            }
            if (lane == 0) *s_hw = hw;
        }
        __syncthreads();
        // ---------------- apply phase: execute the chunk's writes on the key rows, flush the log ----------------
        {
            const int col = lane * 4;
            const bool act = col < DK;
            for (int j = 0; j < cn; j++) {
                const int a = s_am[j];
                if ((a & (AF_WARPS - 1)) != warp) continue;     // one warp per row keeps repeated hits in order
                const float g = s_g[j], omw = 1.f - g;
                float4 Kn = zero4;
                if (act) {
                    Kn = ld4(K + (size_t)a * DK + col);
                    const float4 kt = ld4(Kc + j * DK + col);
                    Kn.x = blend(Kn.x, kt.x, g, omw); Kn.y = blend(Kn.y, kt.y, g, omw);
                    Kn.z = blend(Kn.z, kt.z, g, omw); Kn.w = blend(Kn.w, kt.w, g, omw);
                    st4(K + (size_t)a * DK + col, Kn);
                }
                bool last = true;
                for (int j2 = j + 1; j2 < cn; j2++) last = last && (s_am[j2] != a);
                const float nsq = last ? warp_sum(dot4(Kn, Kn)) : -1.f;
                if (lane == 0) s_nsqx[j] = nsq;
                __syncwarp();
            }
            if (warp == AF_WARPS - 1 && lane >= cn && lane < CH) s_nsqx[lane] = -1.f;
            if (tid < cn) {
                const size_t ix = ((size_t)b * T + t0 + tid) * H + h;
                am_out[ix] = s_am[tid];
                oold_out[ix] = s_oold[tid];
                kiold_out[ix] = s_kiold[tid];
            }
        }
        __syncthreads();
        if (t0 + CH < T) commit_loads();
        __syncthreads();
    }
    if (warp == 0) {
#pragma unroll
        for (int i = 0; i < RPL; i++) {
            const int n = lane + 32 * i;
            if (n < N) ofin[(size_t)bh * N + n] = o_r[i];
        }
    }
}

}  // namespace slotscan
