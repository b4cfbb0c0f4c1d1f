// Address backward for sequences that use FEW rows (at most GATHER_ROWS = 32): token-parallel, no resident state.
//
// The chunked address backward (slotscan_addr_bwd.cuh) walks a sequence's chunks one after another because it carries
// the key rows in shared memory.  But every version of every row already sits in memory: the undo log holds the row
// BEFORE each write, kold[t], and kfin holds the rows after the last one.  The key row n as token t sees it is
//     kold[t']  with t' = the first token >= t that writes row n,   or  kfin[n]  if no later token does,
// and its norm / occupancy are kiold[t'], oold[t'] (or those of the final state).  So with a table of "next write of
// row n at or after t" the tokens of a sequence are independent (occupancy penalty on [o >= eps]: no carried
// occupancy adjoint) and the work spreads over (sequence, head) x (32-token chunk) CTAs:
//   next_write_kernel    one warp per (sequence, head) walks the address log backwards once and stores, per chunk,
//                        the next write of each of the 32 rows at the chunk's END;
//   addr_bwd_gather_kernel  per CTA: every row version the chunk's tokens can see (<= 32 rows after the chunk + the 32
//                        undo rows of the chunk) comes into shared memory by bulk asynchronous copies; warp 0 expands
//                        the next-write table to a per-token table; then each warp takes 4 tokens: scores by 8 lanes
//                        per row (4 rows at a time, 3 shuffle stages), softmax adjoint with lane = row, dq accumulated
//                        with lane = 4 columns over the rows (no reduction).
// A sequence that ever made row 32 a candidate is left to the chunked kernel.  [reference addr_bwd, slotkern_cuda.py:264-443]
#pragma once
#include "slotscan_addr_fwd.cuh"
#include "slotscan_async.cuh"

namespace slotscan {

constexpr int GATHER_ROWS = 32;      // lanes = rows in the softmax part
constexpr int GC = 32;               // tokens per CTA
constexpr int GA_THREADS = 256;
constexpr int GA_WARPS = GA_THREADS / 32;

// true if the sequence never had more than GATHER_ROWS candidate rows
__device__ __forceinline__ bool gather_sequence(const int* tfirst_bh, int N, int T) {
    return N <= GATHER_ROWS || tfirst_bh[GATHER_ROWS] >= T;
}

// vend[bh][c][n]: first token >= (c+1)*GC that writes row n, or -1
static __global__ void __launch_bounds__(32) next_write_kernel(const slotscan_params p, const int* __restrict__ am,
                                                        const int* __restrict__ tfirst, int* __restrict__ vend) {
    const int N = p.N, T = p.T, H = p.H;
    const int bh = blockIdx.x, b = bh / H, h = bh % H, lane = threadIdx.x;
    if (!gather_sequence(tfirst + (size_t)bh * N, N, T)) return;
    const int nc = (T + GC - 1) / GC;
    __shared__ int s_first[GATHER_ROWS];            // first token of the chunk that writes row n (lane = token, then lane = row)
    int ver = -1;
    int a_next = ((nc - 1) * GC + lane < T) ? am[((size_t)b * T + (nc - 1) * GC + lane) * H + h] : -1;
    for (int c = nc - 1; c >= 0; c--) {
        vend[((size_t)bh * nc + c) * GATHER_ROWS + lane] = ver;
        const int a = a_next;
        if (c > 0) a_next = am[((size_t)b * T + (c - 1) * GC + lane) * H + h];     // the next chunk's addresses, in flight
        s_first[lane] = -1;
        __syncwarp();
        const unsigned same = __match_any_sync(FULL, a);                       // the tokens of the chunk with this address
        if (a >= 0 && a < GATHER_ROWS && lane == __ffs((int)same) - 1) s_first[a] = lane;
        __syncwarp();
        const int f = s_first[lane];
        if (f >= 0) ver = c * GC + f;
        __syncwarp();
    }
}

// Set when a bounded wait gave up (slotscan_device_status reads it through the translation unit's accessor).
static __device__ int g_gather_status = 0;

template <int DK, typename Tin>
__global__ void __launch_bounds__(GA_THREADS, 4) addr_bwd_gather_kernel(
    const slotscan_params p, const Tin* __restrict__ q, const float* __restrict__ gate, const float* __restrict__ fr,
    const float* __restrict__ temp_p, const int* __restrict__ am, const float* __restrict__ kold,
    const float* __restrict__ oold, const float* __restrict__ kiold, const float* __restrict__ kfin,
    const float* __restrict__ ofin, const int* __restrict__ tfirst, const int* __restrict__ vend,
    const float* __restrict__ Din, Tin* __restrict__ dq, float* __restrict__ dg, float* __restrict__ dfr,
    float* __restrict__ part, const int part_stride) {
    static_assert(DK >= 32, "8 lanes x float4 per row");
    constexpr int NF = DK / 32;                   // float4 per lane and row in the score pass (8 lanes per row)
    // Every key-row version a token of this chunk can see, staged once per CTA by bulk asynchronous copies:
    //   slot n        (n < 32)   row n as it is AFTER the chunk: the undo row of its next write, or the final row
    //   slot 32 + i              the undo row of token t0 + i: the row it writes, as it was before that write
    // Token i sees row n in slot 32 + (t' - t0) if some token t' >= t0 + i of this chunk writes n, else in slot n.
    // The per-token work then reads shared memory only (before: ~11 KB of gathered rows per token out of L2).
    __shared__ __align__(128) float s_rows[2 * GATHER_ROWS * DK];
    __shared__ float s_kiv[2 * GATHER_ROWS], s_ov[2 * GATHER_ROWS];    // 1 / |row| (clamped) and occupancy per slot
    __shared__ unsigned char s_slot[GC][GATHER_ROWS];   // slot that holds row n as token i sees it
    __shared__ int s_lim[GC];                     // highest candidate row of token i
    __shared__ int s_am[GC];
    __shared__ int s_tf[GATHER_ROWS], s_vend[GATHER_ROWS];
    __shared__ float s_S[GA_WARPS][GATHER_ROWS];
    __shared__ float s_red[2][GA_WARPS];
    __shared__ __align__(8) uint64_t s_bar;
    // The chunk's queries and the candidate rows' entries of both D tables come in with the same bulk copies (dynamic
    // shared memory: GC x DK queries, then 2 x GC x GATHER_ROWS floats): the per-token loop then never waits on global
    // memory (its loads of q and D were the kernel's first stall, 3.6 cycles per issue).
    extern __shared__ __align__(128) unsigned char ga_dyn[];
    Tin* s_q = reinterpret_cast<Tin*>(ga_dyn);
    float* s_D = reinterpret_cast<float*>(ga_dyn + (size_t)GC * DK * sizeof(Tin));      // [2 tables][GC][GATHER_ROWS]
    __shared__ float s_gt[GC], s_frt[GC];
    const int N = p.N, T = p.T, H = p.H;
    const int bh = blockIdx.x, c = blockIdx.y, b = bh / H, h = bh % H;    // chunks on grid.y: T / 32 <= 65535
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!gather_sequence(tfirst + (size_t)bh * N, N, T)) return;          // uniform per CTA
    const int nc = (T + GC - 1) / GC, t0 = c * GC, tc = min(GC, T - t0);
    const int NR = min(N, GATHER_ROWS);
    const float temp = temp_p[0], eps = p.eps;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);

    if (tid < GC) s_am[tid] = (tid < tc) ? am[((size_t)b * T + t0 + tid) * H + h] : -1;
    if (tid >= 32 && tid < 32 + GATHER_ROWS) {
        const int n = tid - 32;
        s_tf[n] = (n < N) ? tfirst[(size_t)bh * N + n] : T;
    }
    if (tid >= 64 && tid < 64 + GC) {             // norm and occupancy of the row each token of the chunk overwrote
        const int i = tid - 64;
        const size_t ix = ((size_t)b * T + t0 + i) * H + h;
        s_kiv[GATHER_ROWS + i] = (i < tc) ? kiold[ix] : 0.f;
        s_ov[GATHER_ROWS + i] = (i < tc) ? oold[ix] : 0.f;
        s_gt[i] = (i < tc) ? gate[ix] : 0.f;
        s_frt[i] = (i < tc) ? (p.fr_per_token ? fr[ix] : fr[0]) : 0.f;
    }
    if (tid == 0) {
        mbar_init(&s_bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    // The chunk's staging is up to 160 bulk copies; a warp issues its 32 one after the other, so the five groups go out
    // from five warps at once (warp 1 computes the candidate limits meanwhile).  One thread posts the byte count of all
    // of them; copies that complete before it has done so only make the count negative for a moment.
    const bool r_in = lane < NR, t_in = lane < tc;
    const unsigned drow = (unsigned)(NR * 4);                              // bytes of one token's candidate entries of a D table
    const bool d_ok = (drow & 15u) == 0u && ((size_t)N * 4 & 15u) == 0u;   // bulk copies want 16-byte pieces
    const size_t ixq = ((size_t)b * T + t0 + lane) * H + h;
    const size_t di = ((size_t)bh * T + t0 + lane) * N;
    if (warp == 2 && t_in) bulk_g2s(s_q + (size_t)lane * DK, q + ixq * DK, DK * sizeof(Tin), &s_bar);
    if ((warp == 3 || warp == 4) && t_in) {
        const int w = warp - 3;                                            // D table of the keys (0) / of the values (1)
        const float* src = Din + (size_t)w * p.B * H * T * N + di;
        if (d_ok) bulk_g2s(s_D + (w * GC + lane) * GATHER_ROWS, src, drow, &s_bar);
        else for (int n = 0; n < NR; n++) s_D[(w * GC + lane) * GATHER_ROWS + n] = src[n];
    }
    if (warp == 5 && t_in) bulk_g2s(s_rows + (GATHER_ROWS + lane) * DK, kold + ixq * DK, DK * 4, &s_bar);
    if (warp == 0) {
        const int ve = (lane < NR) ? vend[((size_t)bh * nc + c) * GATHER_ROWS + lane] : -1;
        if (lane == 0)
            mbar_arrive_expect_tx(&s_bar, (unsigned)(NR + tc) * (unsigned)(DK * 4) + (unsigned)tc * (unsigned)(DK * sizeof(Tin)) +
                                              (d_ok ? (unsigned)tc * 2u * drow : 0u));
        __syncwarp();
        if (r_in)
            bulk_g2s(s_rows + lane * DK, ve < 0 ? kfin + ((size_t)bh * N + lane) * DK : kold + (((size_t)b * T + ve) * H + h) * DK,
                     DK * 4, &s_bar);
        s_vend[lane] = ve;
        if (r_in) {
            if (ve >= 0) {
                const size_t vix = ((size_t)b * T + ve) * H + h;
                s_kiv[lane] = kiold[vix];
                s_ov[lane] = oold[vix];
            } else {
                s_ov[lane] = ofin[(size_t)bh * N + lane];                 // the norm follows once the row has landed
            }
        }
        int ver = ve;                                                      // per-token versions, walking the chunk backwards
        for (int i = GC - 1; i >= 0; i--) {
            if (s_am[i] == lane) ver = t0 + i;
            s_slot[i][lane] = (unsigned char)((ver >= t0 && ver < t0 + GC) ? GATHER_ROWS + (ver - t0) : lane);
        }
    }
    if (warp == 1) {                              // candidate limit of every token of the chunk (rows become candidates in order)
        const int t = t0 + min(lane, tc - 1);
        int lim = NR - 1;
        while (lim > 0 && s_tf[lim] > t) lim--;
        s_lim[lane] = lim;
    }
    {
        const bool landed = mbar_wait_bounded(&s_bar, 0u);
        if (!__syncthreads_and(landed ? 1 : 0)) {
            if (tid == 0) atomicExch(&g_gather_status, 1);
            return;
        }
    }
    for (int n = warp; n < NR; n += GA_WARPS) {   // norms of the rows that are final rows (never written again)
        if (s_vend[n] < 0) {
            const int col = lane * 4;
            const float4 Kn = (col < DK) ? ld4(s_rows + n * DK + col) : zero4;
            const float nsq = warp_sum(dot4(Kn, Kn));
            if (lane == 0) s_kiv[n] = fminf(rsqrtf(nsq), 1e6f);
        }
    }
    __syncthreads();
    float dtemp_acc = 0.f, dfr_acc = 0.f;
    for (int i = warp; i < tc; i += GA_WARPS) {
        const int t = t0 + i;
        const size_t ix = ((size_t)b * T + t) * H + h;
        const int lim = s_lim[i];
        // slot of row n as this token sees it
        auto slot_of = [&](int n) { return (int)s_slot[i][n]; };
        // ---- scores: 8 lanes per row (lane l of the 8 takes float4 chunks l, l + 8, ...: conflict-free), 4 rows per pass ----
        const int r = lane >> 3, l8 = lane & 7;
        float4 q4[NF];
        float qq = 0.f;
#pragma unroll
        for (int f = 0; f < NF; f++) { q4[f] = ld4(s_q + (size_t)i * DK + (l8 + 8 * f) * 4); qq += dot4(q4[f], q4[f]); }
        qq += __shfl_xor_sync(FULL, qq, 1); qq += __shfl_xor_sync(FULL, qq, 2); qq += __shfl_xor_sync(FULL, qq, 4);
        const float qinv = fminf(rsqrtf(qq), 1e6f);
        for (int base = 0; base <= lim; base += 4) {
            const int n = min(base + r, lim);
            const float* row = s_rows + slot_of(n) * DK;
            float a = 0.f;
#pragma unroll
            for (int f = 0; f < NF; f++) a += dot4(ld4(row + (l8 + 8 * f) * 4), q4[f]);
            a += __shfl_xor_sync(FULL, a, 1); a += __shfl_xor_sync(FULL, a, 2); a += __shfl_xor_sync(FULL, a, 4);
            if (l8 == 0 && base + r <= lim) s_S[warp][base + r] = a;
        }
        __syncwarp();
        // ---- softmax adjoint: lane = row ----
        const bool in = lane <= lim;
        const int sl = in ? slot_of(lane) : 0;
        const float ki = in ? s_kiv[sl] : 0.f;
        const float oc = in ? s_ov[sl] : 0.f;
        const float g = gate_eff(s_gt[i], p.hard_gate), frv = s_frt[i];
        const float s = in ? temp * qinv * (ki * s_S[warp][lane]) : 0.f;
        const float occ = oc >= eps ? 1.f : 0.f;
        const float z = s - frv * occ;
        const int ei = (int)__reduce_min_sync(FULL, (unsigned)((in && oc < eps) ? lane : BIGI));   // lowest free row
        const bool ok = in && (oc >= eps || lane == ei);
        const unsigned kk = __reduce_max_sync(FULL, ok ? ord_key(z) : 0u);
        const float zmax = __uint_as_float((kk & 0x80000000u) ? (kk & 0x7fffffffu) : ~kk);
        float dw = 0.f;
        if (in) dw = s_D[i * GATHER_ROWS + lane] + s_D[(GC + i) * GATHER_ROWS + lane];     // key part + value part
        const float e = ok ? __expf(z - zmax) : 0.f;
        float se = e, sd = e * dw;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            se += __shfl_xor_sync(FULL, se, off);
            sd += __shfl_xor_sync(FULL, sd, off);
        }
        const float sa = g * sd / se;
        const float dz = ok ? (e / se) * (g * dw - sa) : 0.f;
        if (lane == s_am[i]) dg[ix] = dw;
        float f1 = -occ * dz, f2 = dz * s;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            f1 += __shfl_xor_sync(FULL, f1, off);
            f2 += __shfl_xor_sync(FULL, f2, off);
        }
        if (lane == 0) {
            if (p.fr_per_token) dfr[ix] = f1; else dfr_acc += f1;
            dtemp_acc += f2 / temp;
        }
        __syncwarp();
        s_S[warp][lane] = dz * temp * ki;                                      // C_n
        __syncwarp();
        // ---- dq: lane = 4 columns, rows in sequence ----
        const int col = lane * 4;
        const bool act = col < DK;
        float4 acc = zero4;
        for (int n = 0; n <= lim; n++) {
            const float cn = s_S[warp][n];
            const float4 K4 = act ? ld4(s_rows + slot_of(n) * DK + col) : zero4;
            acc.x += cn * K4.x; acc.y += cn * K4.y; acc.z += cn * K4.z; acc.w += cn * K4.w;
        }
        const float4 qv = act ? ld4(s_q + (size_t)i * DK + col) : zero4;
        const float4 qn = make_float4(qv.x * qinv, qv.y * qinv, qv.z * qinv, qv.w * qinv);
        const float pr = warp_sum(dot4(acc, qn));
        if (act) {
            float4 out;
            if (qinv >= 1e6f) out = make_float4(qinv * acc.x, qinv * acc.y, qinv * acc.z, qinv * acc.w);   // |q| under the clamp
            else out = make_float4(qinv * (acc.x - qn.x * pr), qinv * (acc.y - qn.y * pr), qinv * (acc.z - qn.z * pr),
                                   qinv * (acc.w - qn.w * pr));
            st4(dq + ix * DK + col, out);
        }
        __syncwarp();
    }
    if (lane == 0) { s_red[0][warp] = dtemp_acc; s_red[1][warp] = dfr_acc; }
    __syncthreads();
    if (tid == 0) {
        float a = 0.f, d = 0.f;
        for (int w = 0; w < GA_WARPS; w++) { a += s_red[0][w]; d += s_red[1][w]; }
        part[(size_t)bh * part_stride + c] = a;                                          // dtemp partial
        part[((size_t)p.B * H + bh) * part_stride + c] = d;                              // scalar dfr partial
    }
}

}  // namespace slotscan
