// Forward address scan, chunked: the sequential decision (which row does token t write?) is the only thing left in
// a token-by-token loop, and that loop runs in ONE warp on numbers that were prepared for it in bulk.
//
// Per chunk of CH = 8 tokens and per (sequence, head), one CTA of 8 warps does
//   1. score phase (all warps): St[j][n] = <K_n, q_j> for every row touched so far against the chunk's 8 queries
//      (keys resident in shared memory as f32, each lane keeps its query slice in registers, rows are broadcast
//      reads), plus the 8x8 table Pm[i][j] = <k_i, q_j> of the chunk's own keys;
//   2. resolve phase (warp 0): per token  z_n = temp * qinv * kinv_n * St[j][n] - fr * occ_n  over the candidate
//      rows, argmax by two warp reductions, then the write: the row is blended in shared memory, its norm is
//      recomputed from the new row, and the scores of the REMAINING tokens of the chunk against that one row follow
//      from linearity:  <(1-g) K_a + g k_i, q_j> = (1-g) St[j][a] + g Pm[i][j].
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
    int K, Qc, Kc, St, Pm, misc, total;
    int qstride, sstride;
};
__host__ __device__ inline AddrFwdSmem addr_fwd_layout(int N, int DK) {
    AddrFwdSmem L;
    L.qstride = DK + 4;                     // padded: the 8 tokens of a quarter-warp hit 8 different bank groups
    L.sstride = (N + 3) & ~3;
    L.K = 0;
    L.Qc = L.K + N * DK;
    L.Kc = L.Qc + CH * L.qstride;
    L.St = L.Kc + CH * L.qstride;
    L.Pm = L.St + CH * L.sstride;
    L.misc = L.Pm + CH * CH;                // qinv[8] g[8] fr[8] | am[8] oold[8] kiold[8] | hw
    L.total = L.misc + 7 * CH;
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
    float* Qc = smem + L.Qc;
    float* Kc = smem + L.Kc;
    float* St = smem + L.St;
    float* Pm = smem + L.Pm;
    float* s_qinv = smem + L.misc;
    float* s_g = s_qinv + CH;
    float* s_fr = s_g + CH;
    int* s_am = reinterpret_cast<int*>(s_fr + CH);
    float* s_oold = reinterpret_cast<float*>(s_am + CH);
    float* s_kiold = s_oold + CH;
    int* s_hw = reinterpret_cast<int*>(s_kiold + CH);

    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pj = lane & 7, pp = lane >> 3;            // score phase: token and column part of this lane
    const float temp = temp_p[0], eps = p.eps;

    for (int i = tid; i < N * DK; i += AF_THREADS) K[i] = 0.f;
    for (int i = tid; i < N; i += AF_THREADS) tfirst[(size_t)bh * N + i] = (i == 0) ? 0 : T;
    if (tid == 0) *s_hw = -1;

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
            float* dst = (it_s ? Kc : Qc) + it_j * L.qstride + it_c;
            st4(dst, make_float4(pre[0], pre[1], pre[2], pre[3]));
            st4(dst + 4, make_float4(pre[4], pre[5], pre[6], pre[7]));
        }
        if (tid < CH) s_g[tid] = pre_s;
        else if (tid < 2 * CH) s_fr[tid - CH] = pre_s;
    };

    // resolver state (warp 0): norms and occupancy of the rows lane + 32 i, in registers
    float kinv_r[RPL], o_r[RPL];
#pragma unroll
    for (int i = 0; i < RPL; i++) { kinv_r[i] = 1e6f; o_r[i] = 0.f; }          // 1 / max(|0|, 1e-6)
    int hw = -1, fe = 0;                                  // highest row touched; lowest free row (N if none)

    issue_loads(0);
    commit_loads();
    __syncthreads();

    for (int t0 = 0; t0 < T; t0 += CH) {
        const int cn = min(CH, T - t0);
        if (t0 + CH < T) issue_loads(t0 + CH);            // next chunk's global loads fly through both phases
        // ---------------- score phase ----------------
        {
            float4 Qr[NI];
#pragma unroll
            for (int i = 0; i < NI; i++) {
                const int d0 = i * 16 + pp * 4;
                Qr[i] = (d0 < DK) ? ld4(Qc + pj * L.qstride + d0) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (warp == 0) {
                float qq = 0.f;
#pragma unroll
                for (int i = 0; i < NI; i++) qq += dot4(Qr[i], Qr[i]);
                qq += __shfl_xor_sync(FULL, qq, 8);
                qq += __shfl_xor_sync(FULL, qq, 16);
                if (pp == 0) s_qinv[pj] = 1.f / fmaxf(sqrtf(qq), 1e-6f);
            }
            const int hw0 = *s_hw;
            const int rows = min(hw0 + CH, N - 1) + 1;    // rows that can be candidates before this chunk ends
            for (int n = warp; n < rows + CH; n += AF_WARPS) {
                const bool is_key = n >= rows;            // the chunk's own keys ride along as 8 extra rows
                const float* row = is_key ? (Kc + (n - rows) * L.qstride) : (K + (size_t)n * DK);
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    const int d0 = i * 16 + pp * 4;
                    if (d0 < DK) acc += dot4(ld4(row + d0), Qr[i]);
                }
                acc += __shfl_xor_sync(FULL, acc, 8);
                acc += __shfl_xor_sync(FULL, acc, 16);
                if (pp == 0) {
                    if (is_key) Pm[(n - rows) * CH + pj] = acc;
                    else St[pj * L.sstride + n] = acc;
                }
            }
        }
        __syncthreads();
        // ---------------- resolve phase (warp 0) ----------------
        if (warp == 0) {
            const int col = lane * 4;
            const bool act = col < DK;
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
                // the write: blend the row where it lives, norm from the new row
                float4 Kr = make_float4(0.f, 0.f, 0.f, 0.f);
                if (act) {
                    Kr = ld4(K + (size_t)am * DK + col);
                    const float4 kt = ld4(Kc + j * L.qstride + col);
                    Kr.x = blend(Kr.x, kt.x, g, omw); Kr.y = blend(Kr.y, kt.y, g, omw);
                    Kr.z = blend(Kr.z, kt.z, g, omw); Kr.w = blend(Kr.w, kt.w, g, omw);
                    st4(K + (size_t)am * DK + col, Kr);
                }
                const float nsq = warp_sum(dot4(Kr, Kr));
                const float kinv_new = 1.f / fmaxf(sqrtf(nsq), 1e-6f);
                const int ai = am >> 5;
                const bool owner = (am & 31) == lane;
                float o_new = 0.f;
#pragma unroll
                for (int i = 0; i < RPL; i++) {
                    if (owner && i == ai) {
                        s_am[j] = am; s_oold[j] = o_r[i]; s_kiold[j] = kinv_r[i];
                        o_r[i] = __fmaf_rn(omw, o_r[i], g);
                        kinv_r[i] = kinv_new;
                        o_new = o_r[i];
                    }
                }
                o_new = __shfl_sync(FULL, o_new, am & 31);
                // scores of the chunk's remaining tokens against the rewritten row, by linearity
                if (lane > j && lane < cn) {
                    float* sp = St + lane * L.sstride + am;
                    *sp = blend(*sp, Pm[j * CH + lane], g, omw);
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
        // ---------------- flush the chunk's log, land the next chunk ----------------
        if (tid < cn) {
            const size_t ix = ((size_t)b * T + t0 + tid) * H + h;
            am_out[ix] = s_am[tid];
            oold_out[ix] = s_oold[tid];
            kiold_out[ix] = s_kiold[tid];
        }
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
