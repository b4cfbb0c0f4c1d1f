// Row-parallel kernels of the hard-address scan: once the address log exists, every key row and every value row
// evolves on its own (a row changes only at the tokens that addressed it).
//
//   replay_rows_kernel   forward: replays rows from the log, emits the stride-G snapshots, the undo log (the row
//                        before each write) and the final state.                 [reference val_fwd, slotkern_cuda.py:178-206]
// (The reverse row scan lives in slotscan_rows_bwd.cuh.)
//
// Layout: one group of LPR = D/8 lanes per row, 8 elements per lane in registers, RPB = 256 / LPR rows per CTA;
// grid (B*H, row tiles, tensors).  Tokens are taken in chunks of RC = 32 through a two-stage shared-memory ring fed by
// bulk asynchronous copies: the walk over a chunk is a walk over EVENTS (next hit, next snapshot) and never waits on
// a global load.  A tile whose rows are never addressed (tfirst == T for all of them) only writes zeros, and not even
// those where the rows were zero-filled ahead of time.
#pragma once
#include "slotscan_async.cuh"
#include "slotscan_common.cuh"

namespace slotscan {

// Set when a bounded wait of the replay gave up (slotscan_device_status reads it through replay_status()).
static __device__ int g_replay_status = 0;

constexpr int ROW_THREADS = 256;
constexpr int RC = 32;                        // tokens per staged chunk (hit mask per row: one bit per token)

// true if any row of this CTA's tile is ever a candidate (row 0 always is)
__device__ __forceinline__ bool tile_active(const int* tfirst_bh, int n, bool live, int T, int* s_flag) {
    if (threadIdx.x == 0) *s_flag = 0;
    __syncthreads();
    if (live && tfirst_bh[n] < T) *s_flag = 1;
    __syncthreads();
    return *s_flag != 0;
}

// ======================================================================================================
// kinv / valid of a row from its float32 state: rsqrt(max(|X|^2, 1e-12)) and [|X|^2 > 1e-12]  [memlm_sh.py:474-475]
// The rows of one warp walk their events independently, so the sum runs over the row's own LPR lanes only (`gmask`).
template <int LPR, int EPL>
__device__ __forceinline__ float row_nsq(const float* X, unsigned gmask) {
    float a = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; j++) a = fmaf(X[j], X[j], a);
#pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) a += __shfl_xor_sync(gmask, a, off);
    return a;
}
template <int LPR>
__device__ __forceinline__ unsigned row_group_mask() {
    const unsigned lane = threadIdx.x & 31u;
    return (LPR >= 32) ? FULL : (((1u << LPR) - 1u) << (LPR * (lane / LPR)));
}

// One tensor of a replay launch: blockIdx.z picks the keys (0) or the values (1) when both run in one launch.
//   x0 (may be NULL): the rows the replay starts from; xold NULL: no undo log; kinv / valid (keys only, or NULL): per
//   emitted row, from the float32 state; zero_from: rows >= zero_from of every snapshot (and their kinv / valid) have
//   been zero-filled already by zero_rows_kernel, so a tile there that never becomes a candidate writes nothing
//   (N = no prefill).
template <typename Tin, typename Tsn>
struct ReplayArgs {
    const Tin* x;
    const float* x0;
    Tsn* xbuf;
    float* xold;
    float* xfin;
    float* kinv;
    uint8_t* valid;
    int zero_from;
};

// NORM: kinv / valid may be asked for (checked per tensor at run time).
// EPL: elements per lane, 8 or 16.  With 16 a lane holds two pieces of 8 columns half a row apart (every load and store
// of a row group stays one contiguous run of 16-byte pieces) and a CTA has half the threads: the busy tiles of a large
// batch (one CTA per sequence, head and tensor) then all fit on the machine at once instead of in two waves.
template <int D, typename Tin, typename Tsn, bool NORM, int EPL>
__global__ void __launch_bounds__(ROW_THREADS * 8 / EPL, EPL == 16 ? 6 : 1) replay_rows_kernel(
    const slotscan_params p, const ReplayArgs<Tin, Tsn> a0, const ReplayArgs<Tin, Tsn> a1,
    const float* __restrict__ gate, const int* __restrict__ am, const int* __restrict__ tfirst, const int tile0) {
    const ReplayArgs<Tin, Tsn>& A = blockIdx.z ? a1 : a0;
    const Tin* __restrict__ x = A.x;
    const float* __restrict__ x0 = A.x0;
    Tsn* __restrict__ xbuf = A.xbuf;
    float* __restrict__ xold = A.xold;
    float* __restrict__ xfin = A.xfin;
    float* __restrict__ kinv_out = A.kinv;
    uint8_t* __restrict__ valid_out = A.valid;
    const bool norm = NORM && kinv_out != nullptr;
    constexpr int NPC = EPL / 8, PS = D / NPC;                       // pieces of 8 columns per lane, columns between them
    constexpr int LPR = PS / 8, RPB = ROW_THREADS / (D / 8), RPW = 32 / LPR;
    static_assert(LPR >= 1 && RPB * LPR >= RC, "at least one lane per row and one thread per staged token");
    auto ldE = [](float* d, const auto* s) {
#pragma unroll
        for (int q = 0; q < NPC; q++) ld8(d + 8 * q, s + q * PS);
    };
    auto stE = [](auto* d, const float* s) {
#pragma unroll
        for (int q = 0; q < NPC; q++) st8(d + q * PS, s + 8 * q);
    };
    __shared__ float s_g[2][RC];                                     // gates of the chunk in work / the next one
    __shared__ int s_am[2][RC];                                      // addressed row - row0 (negative: not in this tile)
    __shared__ __align__(128) Tin s_x[2][RC * D];                    // token vectors, two stages (bulk async copies)
    __shared__ __align__(8) uint64_t s_bar[2];
    __shared__ int s_flag;
    const int N = p.N, T = p.T, H = p.H, G = p.G;
    const int NB = (T + G - 1) / G;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = tid / LPR, c = tid % LPR, row0 = ((int)blockIdx.y + tile0) * RPB, n = row0 + r;   // this launch covers the row tiles from tile0 on
    const bool live = n < N;
    float X[EPL];
#pragma unroll
    for (int j = 0; j < EPL; j++) X[j] = 0.f;
    const size_t snap_stride = (size_t)H * N * D;                   // between consecutive snapshots of one sequence
    Tsn* snap = xbuf + (((size_t)b * NB) * H + h) * N * D + (size_t)n * D + c * 8;
    // kinv / valid of snapshot j of this row live at norm_base + j * norm_stride (one lane per row writes them)
    const size_t norm_stride = (size_t)H * N;
    size_t norm_ix = (((size_t)b * NB) * H + h) * N + n;

    if (!tile_active(tfirst + (size_t)bh * N, n, live, T, &s_flag)) {
        if (live) {                                                  // never a candidate: the row stays zero
            stE(xfin + ((size_t)bh * N + n) * D + c * 8, X);
            if (row0 < A.zero_from) {                                // (tiles at or above zero_from were zero-filled ahead)
                for (int j = 0; j < NB; j++) stE(snap + j * snap_stride, X);
                if (norm && c == 0) {
                    for (int j = 0; j < NB; j++) { kinv_out[norm_ix + j * norm_stride] = 1e6f; valid_out[norm_ix + j * norm_stride] = 0; }
                }
            }
        }
        return;
    }
    if (x0 != nullptr && live) ldE(X, x0 + ((size_t)bh * N + n) * D + c * 8);   // state carried in from the preceding chunk
    const unsigned gmask = row_group_mask<LPR>();
    // Chunks of RC tokens through a two-stage ring: while the rows walk chunk k, the token vectors of chunk k + 1 are
    // being copied (bulk async, one mbarrier per stage) and the gates / addresses of chunk k + 2 are in flight.
    const int nchunk = (T + RC - 1) / RC;
    float pre_g = 0.f;
    int pre_a = -1;
    // The copies and scalars of the chunks ahead are the duty of the LAST warp (the highest rows of the tile: taken last,
    // fewest events), after the barrier that releases the other warps into their walk: issuing a chunk's 32 bulk copies
    // takes a couple of thousand cycles, which would otherwise sit on the path of the busiest rows.
    const bool issuer = warp == (int)(blockDim.x >> 5) - 1;
    auto load_scalars = [&](int ck) {
        pre_g = 0.f; pre_a = -1;
        const int t = ck * RC + lane;
        if (issuer && t < T) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            pre_g = gate_eff(gate[ix], p.hard_gate);
            pre_a = am[ix] - row0;
            if (pre_a >= RPB) pre_a = -1;
        }
    };
    auto issue_x = [&](int ck, int st) {                             // issuing warp
        const int t = ck * RC + lane;
        const bool in = t < T;
        const unsigned nin = __popc(__ballot_sync(FULL, in));
        if (lane == 0) mbar_arrive_expect_tx(&s_bar[st], nin * (unsigned)(D * sizeof(Tin)));
        __syncwarp();
        if (in) bulk_g2s(&s_x[st][lane * D], x + (((size_t)b * T + t) * H + h) * D, D * sizeof(Tin), &s_bar[st]);
    };
    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        mbar_fence_init();
    }
    load_scalars(0);
    __syncthreads();
    if (issuer) {
        s_g[0][lane] = pre_g;
        s_am[0][lane] = pre_a;
        __syncwarp();
        issue_x(0, 0);
    }
    load_scalars(1);
    int tsnap = 0;                                                   // next snapshot time (multiple of G)
    for (int k = 0; k < nchunk; k++) {
        const int t0 = k * RC, tc = min(RC, T - t0), st = k & 1;
        const bool landed = mbar_wait_bounded(&s_bar[st], (unsigned)(k >> 1) & 1u);
        // one barrier: every row is done with chunk k - 1 (stage st ^ 1 and its scalar slot are free) and chunk k has
        // landed for everybody -- or never will: then give up, all threads together
        if (!__syncthreads_and(landed ? 1 : 0)) {
            if (tid == 0) atomicExch(&g_replay_status, 1);
            return;
        }
        if (issuer) {
            if (k + 1 < nchunk) {
                s_g[st ^ 1][lane] = pre_g;
                s_am[st ^ 1][lane] = pre_a;
                __syncwarp();
                issue_x(k + 1, st ^ 1);
            }
            load_scalars(k + 2);
        }
        unsigned m = 0u;                                             // bit i: token t0 + i writes this lane's row
        {
            const int aL = s_am[st][lane];
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) {
                const unsigned bm = __ballot_sync(FULL, aL == warp * RPW + rr);
                if (rr == lane / LPR) m = bm;
            }
        }
        if (!live) continue;
        const Tin* sx = s_x[st];
        const float* sg = s_g[st];
        int i = 0;
        while (true) {
            const unsigned mm = m >> i;                              // i < tc <= 32 here
            const int ih = mm ? i + __ffs((int)mm) - 1 : tc;         // next token that writes this row
            const int tlast = t0 + min(ih, tc - 1);
            if (norm) {
                if (tsnap <= tlast) {                                // the state is the same for every snapshot of this stretch
                    const float nsq = row_nsq<LPR, EPL>(X, gmask);
                    if (c == 0) {
                        const float ki = rsqrtf(fmaxf(nsq, 1e-12f));
                        const uint8_t va = nsq > 1e-12f ? 1 : 0;
                        size_t o = norm_ix;
                        for (int ts = tsnap; ts <= tlast; ts += G) { kinv_out[o] = ki; valid_out[o] = va; o += norm_stride; }
                    }
                }
            }
            for (; tsnap <= tlast; tsnap += G) {                     // pre-write copies
                stE(snap, X);
                snap += snap_stride; norm_ix += norm_stride;
            }
            if (ih >= tc) break;
            const size_t ix = ((size_t)b * T + t0 + ih) * H + h;
            const float g = sg[ih], omw = 1.f - g;
            float xv[EPL];
            ldE(xv, sx + ih * D + c * 8);
            if (xold != nullptr) stE(xold + ix * D + c * 8, X);
#pragma unroll
            for (int j = 0; j < EPL; j++) X[j] = blend(X[j], xv[j], g, omw);
            i = ih + 1;
            if (i >= tc) break;
        }
    }
    if (live) stE(xfin + ((size_t)bh * N + n) * D + c * 8, X);
}

// ======================================================================================================
// Zero-fill of the rows [zero_from, N) of every snapshot (and their kinv = 1e6 / valid = 0), launched on a second
// stream while the sequential address scan runs: the scan needs almost no memory bandwidth, and its first pass holds
// only the first AF_NCAP1 rows, so every sequence that finishes in that pass leaves the rows above untouched -- they
// are zero in every snapshot.  Sequences that do need them (second pass) rewrite those tiles afterwards in the replay,
// which is ordered after this kernel.  Small CTAs (2 warps, few registers) so that they fit beside the scan's CTAs.
constexpr int ZR_THREADS = 64;
template <typename Tsn>
__global__ void __launch_bounds__(ZR_THREADS) zero_rows_kernel(Tsn* __restrict__ xbuf, float* __restrict__ kinv,
                                                              uint8_t* __restrict__ valid, const int N, const int D,
                                                              const int zero_from, const long long nsnap) {
    const size_t row_bytes = (size_t)D * sizeof(Tsn);
    const size_t chunk16 = (size_t)(N - zero_from) * row_bytes / 16;           // 16-byte pieces per snapshot
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (long long so = blockIdx.x; so < nsnap; so += gridDim.x) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(xbuf) + ((size_t)so * N + zero_from) * row_bytes);
        for (size_t i = threadIdx.x; i < chunk16; i += ZR_THREADS) dst[i] = z;
        if (kinv != nullptr) {
            for (int n = zero_from + threadIdx.x; n < N; n += ZR_THREADS) {
                kinv[(size_t)so * N + n] = 1e6f;
                valid[(size_t)so * N + n] = 0;
            }
        }
    }
}

// The same fill through the bulk-copy engine of the SM: one thread per CTA streams a zeroed shared-memory buffer to
// global memory with bulk asynchronous stores, one CTA per SM, both tensors in one launch.  Measured beside a
// resident kernel shaped like the scan (three CTAs of 73 KB per SM): the fill runs at the full write bandwidth
// (6.2 TB/s) when its CTAs are spread one per SM, and at half of it when they are launched after a scan whose CTAs
// load the SMs unevenly (384 CTAs on 148 SMs: the block scheduler then packs every fill CTA onto the 60 emptier SMs).
// So this kernel is submitted BEFORE the scan, with exactly one CTA per SM and little enough shared memory
// (ZB_BYTES) that three CTAs of the scan still fit beside it.
// Requires 16-byte aligned regions: (N - zero_from) * row_bytes, zero_from * row_bytes and N * row_bytes multiples of 16.
struct ZeroTarget {
    unsigned char* x;      // snapshot tensor (nsnap, N, row_bytes), or NULL
    size_t row_bytes;
    int zero_from;
};
constexpr int ZB_THREADS = 32;
constexpr int ZB_BYTES = 8192;
constexpr int ZB_DEPTH = 8;
static __global__ void __launch_bounds__(ZB_THREADS) zero_rows_bulk_kernel(const ZeroTarget ta, const ZeroTarget tb,
                                                                          float* __restrict__ kinv, uint8_t* __restrict__ valid,
                                                                          const int N, const long long nsnap) {
    __shared__ __align__(128) unsigned char s_zero[ZB_BYTES];
    for (int i = threadIdx.x; i < ZB_BYTES / 16; i += ZB_THREADS) reinterpret_cast<uint4*>(s_zero)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
    __syncwarp();
    for (long long so = blockIdx.x; so < nsnap; so += gridDim.x) {
        if (threadIdx.x == 0) {
#pragma unroll
            for (int w = 0; w < 2; w++) {
                const ZeroTarget& t = w ? tb : ta;
                if (t.x == nullptr) continue;
                const size_t region = (size_t)(N - t.zero_from) * t.row_bytes;
                unsigned char* dst = t.x + ((size_t)so * N + t.zero_from) * t.row_bytes;
                for (size_t off = 0; off < region; off += ZB_BYTES) {
                    const size_t nb = region - off < (size_t)ZB_BYTES ? region - off : (size_t)ZB_BYTES;
                    bulk_s2g(dst + off, s_zero, (unsigned)nb);
                    bulk_commit();
                    bulk_wait_read<ZB_DEPTH>();
                }
            }
        } else if (kinv != nullptr) {
            for (int n = ta.zero_from + (int)threadIdx.x - 1; n < N; n += ZB_THREADS - 1) {
                kinv[(size_t)so * N + n] = 1e6f;
                valid[(size_t)so * N + n] = 0;
            }
        }
    }
    if (threadIdx.x == 0) bulk_wait<0>();          // the buffer must outlive the copies that read it
    __syncwarp();
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
