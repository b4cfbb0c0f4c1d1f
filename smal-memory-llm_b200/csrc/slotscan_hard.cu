// Hard-address slot scan for sm_100a: host-side launchers and the C ABI of the reference's training mode
// (hard argmax address, address gradient detached from the stored keys).
//
// Decomposition (the row a token writes is the only sequential decision):
//   addr_fwd_direct_kernel (slotscan_addr_fwd.cuh)  one CTA per (sequence, head): keys resident in shared memory,
//                      scores per chunk of 8 tokens in bulk, one warp resolves the addresses.   [addr_fwd, slotkern_cuda.py:72-174]
//   replay_rows_kernel (slotscan_rows.cuh)  row-parallel: replays key / value rows from the log, emits the stride-G
//                      snapshots, the undo log and the final state.                              [val_fwd :178-206]
//   rows_bwd_kernel    (slotscan_rows.cuh)  row-parallel reverse scan: dK / dV recursion, dk / dv, the table D[t,n]. [rows_bwd :209-261]
//   addr_bwd_chunked_kernel (slotscan_addr_bwd.cuh)  softmax adjoint per chunk: dgate, dfr, dtemp, dq.   [addr_bwd :264-443]
// Rows are taken in index order (only occupied rows and the lowest free row are candidates), so every row above
// the highest row touched so far is exactly zero: all kernels skip those rows.
#include <math.h>
#include <stdio.h>

#include <mutex>
#include <vector>

#include "slotscan_common.cuh"
#include "slotscan_launch.h"

namespace slotscan {

// fixed-order sum of the partial sums (per sequence and token chunk) -> dtemp, scalar dfr: each thread adds a strided
// subset in index order, then the 256 subtotals are added in order, so the result is bitwise repeatable
__global__ void __launch_bounds__(256) finish_scalars_kernel(const float* __restrict__ part, int n, int fr_per_token,
                                                             float* dtemp, float* dfr) {
    __shared__ float s_a[256], s_c[256];
    float a = 0.f, c = 0.f;
    for (int i = threadIdx.x; i < n; i += 256) { a += part[i]; c += part[n + i]; }
    s_a[threadIdx.x] = a; s_c[threadIdx.x] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        a = 0.f; c = 0.f;
        for (int i = 0; i < 256; i++) { a += s_a[i]; c += s_c[i]; }
        dtemp[0] = a;
        if (!fr_per_token) dfr[0] = c;
    }
}
template <typename Tin>
__global__ void add_into_kernel(Tin* __restrict__ dst, const Tin* __restrict__ src, size_t n4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = ld4(dst + i * 4), c = ld4(src + i * 4);
        st4(dst + i * 4, make_float4(a.x + c.x, a.y + c.y, a.z + c.z, a.w + c.w));
    }
}

// ------------------------------------------------------------------------------------------------------
// Optional per-kernel timing (slotscan_profile_*): CUDA events recorded on the launching stream around each launch.
struct ProfRec { int id; cudaEvent_t a, b; };
static bool g_prof_on = false;
static std::vector<ProfRec> g_prof;
static std::mutex g_prof_mu;
enum { K_ADDR_FWD = 0, K_REPLAY_K, K_REPLAY_V, K_ROWS_BWD_K, K_ROWS_BWD_V, K_ADDR_BWD, K_FINISH, K_ZERO_FILL, K_NKERN };
static const char* const K_NAMES[K_NKERN] = {"addr_fwd", "replay_rows_k", "replay_rows_v", "rows_bwd_k", "rows_bwd_v",
                                             "addr_bwd", "finish", "zero_fill"};
struct ProfScope {
    int id; cudaStream_t st; cudaEvent_t a = nullptr, b = nullptr; bool on;
    ProfScope(int id_, cudaStream_t st_) : id(id_), st(st_), on(g_prof_on) {
        if (on) { cudaEventCreate(&a); cudaEventCreate(&b); cudaEventRecord(a, st); }
    }
    ~ProfScope() {
        if (on) { cudaEventRecord(b, st); std::lock_guard<std::mutex> l(g_prof_mu); g_prof.push_back({id, a, b}); }
    }
};

constexpr size_t SMEM_CAP = 227 * 1024;

// Extra streams so that the sequential address scan and the zero-fill of the snapshot rows its first pass cannot touch
// run side by side: one per (device, caller stream), created on first use and kept until the process exits, so that
// callers that work on several streams of a device at once (a pipeline over batch chunks) keep their scans independent
// of one another.  Beyond SIDE_STREAMS_MAX caller streams per device the extra streams are shared round-robin.
constexpr int MAX_DEVICES = 64;
constexpr int SIDE_STREAMS_MAX = 32;
struct SideStreams { cudaStream_t caller[SIDE_STREAMS_MAX]; cudaStream_t side[SIDE_STREAMS_MAX]; int n; };
static SideStreams g_side[MAX_DEVICES];
static std::mutex g_side_mu;
static cudaStream_t side_stream(cudaStream_t caller) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> l(g_side_mu);
    SideStreams& S = g_side[dev];
    for (int i = 0; i < S.n; i++)
        if (S.caller[i] == caller) return S.side[i];
    if (S.n == SIDE_STREAMS_MAX) return S.side[(size_t)((uintptr_t)caller >> 4) % SIDE_STREAMS_MAX];
    cudaStream_t s = nullptr;
    if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    S.caller[S.n] = caller;
    S.side[S.n] = s;
    S.n++;
    return s;
}

static cudaError_t fwd_run(const slotscan_params& p, const void* k, const void* q, const void* v, const float* gate,
                           const float* fr, const float* temp, void* kbuf, void* vbuf, const slotscan_log& L,
                           const slotscan_fwd_extra& ex, cudaStream_t st) {
    cudaError_t e;
    // While the address scan runs (sequential, almost no memory traffic; on a second stream, see below) every snapshot
    // row above the first row tile is zero-filled: rows are taken in index order, so a tile that never becomes a
    // candidate is zero in every snapshot, and with few rows in use that is most of the snapshot bytes.  The replay,
    // ordered after both, writes the first tile and rewrites every tile that did become a candidate (tile_active) on top
    // of the zeros; the others it leaves alone.  Not with a carried-in state (its rows may be anywhere).
    int zk = p.N, zv = p.N;
    cudaEvent_t joined = nullptr, fork = nullptr;
    cudaStream_t side = nullptr;
    if (p.N > min(replay_tile_rows(p.DK), replay_tile_rows(p.DV)) && ex.K0 == nullptr) {
        side = side_stream(st);
        if (side != nullptr && cudaEventCreateWithFlags(&fork, cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&joined, cudaEventDisableTiming) == cudaSuccess) {
            zk = min(replay_tile_rows(p.DK), p.N);
            zv = min(replay_tile_rows(p.DV), p.N);
            if ((e = cudaEventRecord(fork, st)) != cudaSuccess) { cudaEventDestroy(fork); cudaEventDestroy(joined); return e; }
        } else {
            if (fork != nullptr) cudaEventDestroy(fork);
            if (joined != nullptr) cudaEventDestroy(joined);
            fork = joined = nullptr;
        }
    }
    const AddrFwdState S0{ex.K0, ex.o0, ex.nsq0, ex.nsqfin};
    auto scan_on = [&](cudaStream_t s) {
        ProfScope ps(K_ADDR_FWD, s);
        return (p.in_dtype == SLOTSCAN_F32) ? run_addr_fwd_f32(p, q ? q : k, k, gate, fr, temp, L, S0, s)
                                            : run_addr_fwd_bf16(p, q ? q : k, k, gate, fr, temp, L, S0, s);
    };
    const ReplayPtrs rk{k, ex.K0, kbuf, ex.no_undo_log ? nullptr : L.kold, L.kfin, ex.kinv, ex.valid, zk};
    const ReplayPtrs rv{v, ex.V0, vbuf, ex.no_undo_log ? nullptr : L.vold, L.vfin, nullptr, nullptr, zv};
    if (joined != nullptr) {
        // The zero-fill goes on the caller's stream and the SCAN on the second stream, behind `fork`: the fill's CTAs (one
        // per SM) are then placed first, on an idle machine, evenly, and three CTAs of the scan still fit beside each.
        // The other way round the scan's 384 CTAs load the 148 SMs unevenly (3 on some, 2 on others) and the block
        // scheduler packs every fill CTA onto the emptier SMs: the fill then runs at half the write bandwidth.
        // The replay of the row tiles BELOW the fill (the busy ones) follows the scan on the second stream and does not
        // wait for the fill; the tiles above it are replayed after both.
        const bool merged = p.DK == p.DV;                    // keys and values in one launch: their busy tiles overlap
        const int tz = merged ? zk / replay_tile_rows(p.DK) : 0;    // first row tile that the fill covers
        cudaError_t e2;
        {
            ProfScope ps(K_ZERO_FILL, st);
            e2 = run_zero_rows(p, kbuf, zk, vbuf, zv, ex.kinv, ex.valid, st);
        }
        if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(side, fork, 0);
        if (e2 == cudaSuccess) e2 = scan_on(side);
        if (merged && tz > 0) {
            // tiles below the fill on the second stream, the tiles above it on the caller's (after scan and fill), side by
            // side; the caller's stream then waits for the second one
            if (e2 == cudaSuccess) e2 = cudaEventRecord(fork, side);              // `fork` has been waited for: reused as "scan done"
            if (e2 == cudaSuccess) {
                ProfScope ps(K_REPLAY_K, side);
                e2 = run_replay(p, p.DK, 2, rk, rv, gate, L.addr, L.tfirst, 0, tz, side);
            }
            if (e2 == cudaSuccess) e2 = cudaEventRecord(joined, side);
            if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(st, fork, 0);
            if (e2 == cudaSuccess) {
                ProfScope ps(K_REPLAY_V, st);
                e2 = run_replay(p, p.DK, 2, rk, rv, gate, L.addr, L.tfirst, tz, -1, st);
            }
            if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(st, joined, 0);
            cudaEventDestroy(fork);
            cudaEventDestroy(joined);
            return e2;
        }
        if (e2 == cudaSuccess) e2 = cudaEventRecord(joined, side);
        if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(st, joined, 0);          // the replay comes after both
        cudaEventDestroy(fork);
        cudaEventDestroy(joined);
        if (e2 != cudaSuccess) return e2;
        if (merged) {
            ProfScope ps(K_REPLAY_V, st);
            return run_replay(p, p.DK, 2, rk, rv, gate, L.addr, L.tfirst, tz, -1, st);
        }
    } else {
        e = scan_on(st);
        if (e != cudaSuccess) return e;
        if (p.DK == p.DV) {
            ProfScope ps(K_REPLAY_K, st);
            return run_replay(p, p.DK, 2, rk, rv, gate, L.addr, L.tfirst, 0, -1, st);
        }
    }
    {
        ProfScope ps(K_REPLAY_K, st);
        e = run_replay(p, p.DK, 1, rk, rk, gate, L.addr, L.tfirst, 0, -1, st);
    }
    if (e != cudaSuccess) return e;
    ProfScope ps(K_REPLAY_V, st);
    return run_replay(p, p.DV, 1, rv, rv, gate, L.addr, L.tfirst, 0, -1, st);
}

static cudaError_t bwd_run(const slotscan_params& p, const void* k, const void* q, const void* v, const float* gate,
                           const float* fr, const float* temp, const slotscan_log& L, const void* dkbuf, const void* dvbuf,
                           const float* dkinv, float* Dn, float* part, int* vend, void* dk, void* dq, void* dv,
                           float* dgate, float* dfr, float* dtemp, cudaStream_t st) {
    cudaError_t e;
    // partial sums of dtemp / scalar dfr: one slot per (sequence, 32-token chunk) + one per sequence; slots that no
    // kernel fills must read as zero
    const int part_stride = (p.T + GATHER_CHUNK - 1) / GATHER_CHUNK + 1;
    const size_t part_n = (size_t)p.B * p.H * part_stride;
    // The next-write table of the address backward needs the forward's log only: it runs on the second stream beside the
    // reverse row scan, and the address backward waits for it.
    bool vend_ready = false;
    cudaEvent_t joined = nullptr;
    if (next_write_used(p)) {
        cudaStream_t side = side_stream(st);
        cudaEvent_t fork = nullptr;
        if (side != nullptr && cudaEventCreateWithFlags(&fork, cudaEventDisableTiming) == cudaSuccess &&
            cudaEventCreateWithFlags(&joined, cudaEventDisableTiming) == cudaSuccess) {
            if (cudaEventRecord(fork, st) == cudaSuccess && cudaStreamWaitEvent(side, fork, 0) == cudaSuccess) {
                vend_ready = run_next_write(p, L, vend, side) == cudaSuccess && cudaEventRecord(joined, side) == cudaSuccess;
                // error path: nothing of this call stays in flight on the second stream; the table is then filled on the caller's
                if (!vend_ready) cudaStreamSynchronize(side);
            }
        }
        if (fork != nullptr) cudaEventDestroy(fork);
        if (!vend_ready && joined != nullptr) { cudaEventDestroy(joined); joined = nullptr; }
    }
    struct JoinedGuard { cudaEvent_t& e; ~JoinedGuard() { if (e != nullptr) cudaEventDestroy(e); } } joined_guard{joined};
    if ((e = cudaMemsetAsync(part, 0, 2 * part_n * sizeof(float), st)) != cudaSuccess) return e;
    // keys and values are independent given the log: one launch (blockIdx.z) when dk == dv, each into its own D table
    float* DnV = Dn + (size_t)p.B * p.H * p.T * p.N;
    const RowsBwdPtrs ak{k, L.kold, L.kfin, dkbuf, dk, Dn, dkinv};
    const RowsBwdPtrs av{v, L.vold, L.vfin, dvbuf, dv, DnV, nullptr};
    if (p.DK == p.DV) {
        ProfScope ps(K_ROWS_BWD_K, st);
        e = run_rows_bwd(p, p.DK, 2, ak, av, gate, L.addr, L.tfirst, st);
    } else {
        {
            ProfScope ps(K_ROWS_BWD_K, st);
            e = run_rows_bwd(p, p.DK, 1, ak, ak, gate, L.addr, L.tfirst, st);
        }
        if (e != cudaSuccess) return e;
        ProfScope ps(K_ROWS_BWD_V, st);
        e = run_rows_bwd(p, p.DV, 1, av, av, gate, L.addr, L.tfirst, st);
    }
    if (e != cudaSuccess) return e;
    if (vend_ready && (e = cudaStreamWaitEvent(st, joined, 0)) != cudaSuccess) return e;
    {
        ProfScope ps(K_ADDR_BWD, st);
        e = (p.in_dtype == SLOTSCAN_F32)
                ? run_addr_bwd_f32(p, q ? q : k, k, gate, fr, temp, L, Dn, dq, dgate, dfr, part, vend, part_stride, vend_ready, st)
                : run_addr_bwd_bf16(p, q ? q : k, k, gate, fr, temp, L, Dn, dq, dgate, dfr, part, vend, part_stride, vend_ready, st);
    }
    if (e != cudaSuccess) return e;
    ProfScope ps(K_FINISH, st);
    finish_scalars_kernel<<<1, 256, 0, st>>>(part, (int)part_n, p.fr_per_token, dtemp, dfr);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    if (q == nullptr) {       // the search query is the stored key: both gradient paths land in dk
        const size_t n4 = (size_t)p.B * p.T * p.H * p.DK / 4;
        if (p.in_dtype == SLOTSCAN_F32) add_into_kernel<float><<<592, 256, 0, st>>>((float*)dk, (const float*)dq, n4);
        else add_into_kernel<__nv_bfloat16><<<592, 256, 0, st>>>((__nv_bfloat16*)dk, (const __nv_bfloat16*)dq, n4);
        e = cudaGetLastError();
    }
    return e;
}

}  // namespace slotscan

using namespace slotscan;

static inline bool misaligned(const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

extern "C" int slotscan_abi_version(void) { return SLOTSCAN_ABI_VERSION; }

extern "C" int slotscan_check(const slotscan_params* p) {
    if (!p) return SLOTSCAN_E_NULL;
    if (p->B < 1 || p->T < 1 || p->H < 1 || p->N < 1 || p->G < 1) return SLOTSCAN_E_SHAPE;
    if (p->DK < 8 || p->DK > 128 || (p->DK & (p->DK - 1))) return SLOTSCAN_E_SHAPE;
    if (p->DV < 8 || p->DV > 128 || (p->DV & (p->DV - 1))) return SLOTSCAN_E_SHAPE;
    if (p->N > 192) return SLOTSCAN_E_SHAPE;
    if (addr_fwd_smem_bytes(p->N, p->DK, 4) + 1024 > SMEM_CAP || addr_bwd_smem_bytes(p->N, p->DK) + 1024 > SMEM_CAP)
        return SLOTSCAN_E_SHAPE;
    if ((long long)p->B * p->H > 2147483647LL / 4) return SLOTSCAN_E_SHAPE;
    /* the reverse row scan runs one block per (sequence, head, tile of 2048 / D rows, tensor) on grid.x */
    {
        const int dmax = p->DK > p->DV ? p->DK : p->DV;
        const long long tiles = ((long long)p->N * dmax + 2047) / 2048;
        if ((long long)p->B * p->H * tiles * 2 > 2147483647LL) return SLOTSCAN_E_SHAPE;
    }
    /* token chunks ride on grid.y (<= 65535) and the partial-sum table is indexed with ints */
    if (((long long)p->T + GATHER_CHUNK - 1) / GATHER_CHUNK > 65535) return SLOTSCAN_E_SHAPE;
    if ((long long)p->B * p->H * (((long long)p->T + GATHER_CHUNK - 1) / GATHER_CHUNK + 1) > 2147483647LL / 2) return SLOTSCAN_E_SHAPE;
    if (p->in_dtype != SLOTSCAN_F32 && p->in_dtype != SLOTSCAN_BF16) return SLOTSCAN_E_DTYPE;
    if (p->snap_dtype != SLOTSCAN_F32 && p->snap_dtype != SLOTSCAN_BF16) return SLOTSCAN_E_DTYPE;
    return SLOTSCAN_OK;
}

extern "C" int slotscan_hard_fwd_ex(const slotscan_params* p, const void* k, const void* q, const void* v,
                                    const float* gate, const float* fr, const float* temp, void* kbuf, void* vbuf,
                                    const slotscan_log* log, const slotscan_fwd_extra* ex_, void* stream) {
    int rc = slotscan_check(p);
    if (rc) return rc;
    slotscan_fwd_extra ex = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0};
    if (ex_) ex = *ex_;
    if (!k || !v || !gate || !fr || !temp || !kbuf || !vbuf || !log) return SLOTSCAN_E_NULL;
    if (!log->addr || !log->oold || !log->kfin || !log->vfin || !log->ofin || !log->tfirst || !log->kiold)
        return SLOTSCAN_E_NULL;
    if (!ex.no_undo_log && (!log->kold || !log->vold)) return SLOTSCAN_E_NULL;
    if ((ex.K0 != nullptr) != (ex.V0 != nullptr) || (ex.K0 != nullptr) != (ex.o0 != nullptr)) return SLOTSCAN_E_NULL;
    if (ex.nsq0 != nullptr && ex.K0 == nullptr) return SLOTSCAN_E_NULL;
    if ((ex.kinv != nullptr) != (ex.valid != nullptr)) return SLOTSCAN_E_NULL;
    if (misaligned(k) || misaligned(q) || misaligned(v) || misaligned(kbuf) || misaligned(vbuf) || misaligned(log->kold) ||
        misaligned(log->vold) || misaligned(log->kfin) || misaligned(log->vfin) || misaligned(ex.K0) || misaligned(ex.V0))
        return SLOTSCAN_E_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const cudaError_t e = fwd_run(*p, k, q, v, gate, fr, temp, kbuf, vbuf, *log, ex, st);
    return (int)e;
}

extern "C" int slotscan_hard_fwd(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                                 const float* fr, const float* temp, void* kbuf, void* vbuf, const slotscan_log* log,
                                 void* stream) {
    return slotscan_hard_fwd_ex(p, k, q, v, gate, fr, temp, kbuf, vbuf, log, nullptr, stream);
}

// scratch layout: [D table keys | D table values] [partial sums 2 x B*H x (chunks + 1) f32] [next-write table B*H x chunks x 32 i32]
static void bwd_scratch_layout(const slotscan_params* p, size_t* off_part, size_t* off_vend, size_t* total) {
    const size_t BH = (size_t)p->B * p->H, nc = ((size_t)p->T + GATHER_CHUNK - 1) / GATHER_CHUNK;
    size_t o = 2 * sizeof(float) * BH * p->T * p->N;       // one D table for the keys, one for the values
    o = (o + 255) & ~(size_t)255;
    *off_part = o;
    o += sizeof(float) * 2 * BH * (nc + 1);
    o = (o + 255) & ~(size_t)255;
    *off_vend = o;
    o += sizeof(int) * BH * nc * GATHER_ROWS_MAX;
    *total = o;
}

extern "C" size_t slotscan_hard_bwd_scratch_bytes(const slotscan_params* p) {
    if (slotscan_check(p)) return 0;
    size_t a, b, t;
    bwd_scratch_layout(p, &a, &b, &t);
    return t;
}

extern "C" int slotscan_hard_bwd(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                                 const float* fr, const float* temp, const slotscan_log* log, const void* dkbuf,
                                 const void* dvbuf, void* scratch, size_t scratch_bytes, void* dk, void* dq, void* dv,
                                 float* dgate, float* dfr, float* dtemp, void* stream) {
    return slotscan_hard_bwd_ex(p, k, q, v, gate, fr, temp, log, dkbuf, dvbuf, nullptr, scratch, scratch_bytes, dk, dq, dv,
                                dgate, dfr, dtemp, stream);
}

extern "C" int slotscan_hard_bwd_ex(const slotscan_params* p, const void* k, const void* q, const void* v,
                                    const float* gate, const float* fr, const float* temp, const slotscan_log* log,
                                    const void* dkbuf, const void* dvbuf, const float* dkinv, void* scratch,
                                    size_t scratch_bytes, void* dk, void* dq, void* dv, float* dgate, float* dfr,
                                    float* dtemp, void* stream) {
    int rc = slotscan_check(p);
    if (rc) return rc;
    if (!k || !v || !gate || !fr || !temp || !log || !scratch || !dk || !dq || !dv || !dgate || !dfr || !dtemp)
        return SLOTSCAN_E_NULL;
    if (!log->addr || !log->oold || !log->kold || !log->vold || !log->kfin || !log->vfin || !log->ofin || !log->tfirst ||
        !log->kiold)
        return SLOTSCAN_E_NULL;
    if (scratch_bytes < slotscan_hard_bwd_scratch_bytes(p)) return SLOTSCAN_E_SHAPE;
    if (misaligned(k) || misaligned(q) || misaligned(v) || misaligned(dkbuf) || misaligned(dvbuf) || misaligned(dk) ||
        misaligned(dq) || misaligned(dv) || misaligned(scratch) || misaligned(log->kold) || misaligned(log->vold) ||
        misaligned(log->kfin) || misaligned(log->vfin))
        return SLOTSCAN_E_ALIGN;
    size_t off_part, off_vend, total;
    bwd_scratch_layout(p, &off_part, &off_vend, &total);
    float* Dn = (float*)scratch;
    float* part = (float*)((char*)scratch + off_part);
    int* vend = (int*)((char*)scratch + off_vend);
    cudaStream_t st = (cudaStream_t)stream;
    const cudaError_t e = bwd_run(*p, k, q, v, gate, fr, temp, *log, dkbuf, dvbuf, dkinv, Dn, part, vend, dk, dq, dv, dgate,
                                  dfr, dtemp, st);
    return (int)e;
}

extern "C" int slotscan_query_attrs(slotscan_kernel_attr* out, int cap) {
    int n = 0;
    attrs_addr_fwd_f32(out, cap, n);
    attrs_addr_fwd_bf16(out, cap, n);
    attrs_rows(out, cap, n);
    attrs_rows_bwd_f32(out, cap, n);
    attrs_rows_bwd_bf16(out, cap, n);
    attrs_addr_bwd_f32(out, cap, n);
    attrs_addr_bwd_bf16(out, cap, n);
    return n;
}

extern "C" int slotscan_device_status(void) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    const int a = rows_bwd_status_f32(), b = rows_bwd_status_bf16(), c = read_mma_status();
    const int d = gather_status_f32(), e = gather_status_bf16(), f = replay_status();
    return (a < 0 || b < 0 || c < 0 || d < 0 || e < 0 || f < 0) ? -1 : (a | b | c | d | e | f);
}

extern "C" int slotscan_profile_enable(int on) {
    std::lock_guard<std::mutex> l(g_prof_mu);
    g_prof_on = on != 0;
    return 0;
}

extern "C" int slotscan_profile_read(slotscan_kernel_time* out, int cap) {
    std::lock_guard<std::mutex> l(g_prof_mu);
    float ms[K_NKERN] = {0};
    int cnt[K_NKERN] = {0};
    for (auto& r : g_prof) {
        float t = 0.f;
        if (cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&t, r.a, r.b) == cudaSuccess) {
            ms[r.id] += t;
            cnt[r.id]++;
        }
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    g_prof.clear();
    for (int i = 0; i < K_NKERN && i < cap; i++) {
        snprintf(out[i].name, sizeof(out[i].name), "%s", K_NAMES[i]);
        out[i].launches = cnt[i];
        out[i].total_ms = ms[i];
    }
    return K_NKERN;
}

// ------------------------------------------------------------------------------------------------------
// Backward without caller scratch.  Some hosts cannot hand this library a scratch buffer: a serving process that
// gave every byte of device memory to its own arena at start-up, a thin foreign-language binding that has no device
// allocator to call, a code path in which a synchronising cudaMalloc / cudaFree is not acceptable.  For them the
// table D[t,n] and the per-sequence partial sums live in a fixed array inside the library image.
//
// The array's name is only a host-side handle for the symbol; the device address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static __device__ __align__(256) unsigned char g_fixed_scratch[SLOTSCAN_NOALLOC_SCRATCH_BYTES];
static void* g_fixed_scratch_addr[MAX_DEVICES] = {nullptr};
static std::mutex g_fixed_scratch_mu;

extern "C" size_t slotscan_hard_bwd_noalloc_capacity(void) { return (size_t)SLOTSCAN_NOALLOC_SCRATCH_BYTES; }

extern "C" int slotscan_hard_bwd_noalloc(const slotscan_params* p, const void* k, const void* q, const void* v,
                                         const float* gate, const float* fr, const float* temp, const slotscan_log* log,
                                         const void* dkbuf, const void* dvbuf, void* dk, void* dq, void* dv, float* dgate,
                                         float* dfr, float* dtemp, void* stream) {
    int rc = slotscan_check(p);
    if (rc) return rc;
    if (slotscan_hard_bwd_scratch_bytes(p) > (size_t)SLOTSCAN_NOALLOC_SCRATCH_BYTES) return SLOTSCAN_E_TOO_LARGE;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return SLOTSCAN_E_SHAPE;
    // The array handed to the kernels is the CURRENT device's: the inputs (and so the stream) must live there too.
    if (k != nullptr) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, k) == cudaSuccess && at.type == cudaMemoryTypeDevice && at.device != dev)
            return SLOTSCAN_E_MODE;
    }
    void* scratch;
    {
        std::lock_guard<std::mutex> l(g_fixed_scratch_mu);
        if (g_fixed_scratch_addr[dev] == nullptr) {          // first call on this device: resolve the symbol
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_fixed_scratch);
            if (e != cudaSuccess) return (int)e;
            if (ptr == nullptr) return (int)cudaErrorInvalidSymbol;
            g_fixed_scratch_addr[dev] = ptr;
        }
        scratch = g_fixed_scratch_addr[dev];
    }
    // The array keeps the previous call's contents.  Every D[t,n] and next-write entry that is read was written earlier
    // in the same call; the partial-sum table, whose unused slots must read as zero, is cleared by the call itself
    // (cudaMemsetAsync on the caller's stream, inside slotscan_hard_bwd).
    return slotscan_hard_bwd(p, k, q, v, gate, fr, temp, log, dkbuf, dvbuf, scratch, (size_t)SLOTSCAN_NOALLOC_SCRATCH_BYTES,
                             dk, dq, dv, dgate, dfr, dtemp, stream);
}

