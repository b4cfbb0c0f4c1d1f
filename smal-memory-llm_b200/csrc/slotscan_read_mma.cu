// Cosine read of the stride-G snapshots on the tensor cores, forward, bf16 queries and snapshots.
//   [reference SharedMixer._read, gqa25/memlm_sh.py:379-397: bf16 (G*NQ x dk) @ (dk x N) logits, float32 softmax over the
//    valid rows, att.to(bf16) @ buf]
//
// The G tokens x NQ queries that share a snapshot form an M = 16 query tile -- exactly one mma.m16n8k16 row block -- so
// per (sequence, block, head) the read is  S = Q K^T (16 x N x dk),  softmax over the valid rows,  O = P V (16 x dv x N).
// At 16 flops per snapshot byte the kernel is bound by the snapshot traffic, not by the tensor pipe; what matters is to
// keep whole snapshot tiles in flight.  One CTA of 4 warps per snapshot:
//   * the key rows and the value rows up to the highest valid row come in by bulk asynchronous copies (one per row,
//     into rows padded by 16 bytes so that ldmatrix is conflict-free), each tensor on its own mbarrier: Q K^T starts
//     when the keys have landed while the values are still in flight; two CTAs per SM overlap one's loads with the
//     other's math;
//   * Q K^T: each warp takes every fourth 8-row tile of the snapshot, A fragments (the queries) stay in registers;
//     logits are scaled by kinv[n] * sharp[m] / |q_m| in float32, rows that are not valid are masked;
//   * softmax statistics by quad shuffles and one exchange between the warps; P goes to shared memory as bf16 (the
//     reference multiplies att.to(bf16) as well), normalisation by 1 / sum is applied to the float32 result;
//   * P V: each warp owns a quarter of the value columns, V fragments through ldmatrix.trans.
// Other dtypes and widths take the CUDA-core kernel of slotscan_read.cu.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "slotscan.h"
#include "slotscan_async.cuh"
#include "slotscan_common.cuh"
#include "slotscan_launch.h"

namespace slotscan {

typedef __nv_bfloat16 bf16;
constexpr int RM_THREADS = 128, RM_WARPS = 4;
constexpr int RM_MAXN = 192;                          // rows per snapshot this kernel holds (6 tiles of 8 rows per warp)
constexpr int RM_TPW = RM_MAXN / 8 / RM_WARPS;        // 8-row tiles per warp
// Snapshots whose highest valid row lies below this are left to the CUDA-core kernel of slotscan_read.cu (launched
// right after this one with the complementary test): with a handful of rows the tensor-core tile is mostly padding and
// the CTA's fixed chain of dependent loads dominates; measured crossover near 32 rows on B200.

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2(unsigned& r0, unsigned& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x2_trans(unsigned& r0, unsigned& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}
// D (16x8, f32) += A (16x16, bf16, row) * B (16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

static __device__ int g_read_status = 0;              // a bounded wait gave up (slotscan_device_status)

struct ReadMmaSmem { int K, V, PQ, kv, red, scale, misc, bar, total; int ldk, ldv, ldp; };
__host__ __device__ inline ReadMmaSmem read_mma_layout(int N, int DK, int DV) {      // byte offsets
    ReadMmaSmem L;
    const int NP = (N + 15) & ~15;
    L.ldk = DK + 8; L.ldv = DV + 8; L.ldp = (DK > NP ? DK : NP) + 8;                 // elements per padded row
    L.K = 0;
    L.V = L.K + NP * L.ldk * 2;
    L.PQ = L.V + NP * L.ldv * 2;
    L.kv = L.PQ + 16 * L.ldp * 2;                     // [NP] kinv of a valid row, -1 for the others
    L.red = L.kv + NP * 4;                            // [2][4 warps][16] row maxima, row sums
    L.scale = L.red + 2 * RM_WARPS * 16 * 4;          // [16] sharp / |q|
    L.misc = L.scale + 16 * 4;                        // [0] highest valid row + 1
    L.bar = L.misc + 16;
    L.total = L.bar + 16;
    return L;
}

template <int DK, int DV>
__global__ void __launch_bounds__(RM_THREADS, 2) read_fwd_mma_kernel(
    const slotscan_read_params p, const bf16* __restrict__ qr, const float* __restrict__ sharp,
    const bf16* __restrict__ kbuf, const bf16* __restrict__ vbuf, const float* __restrict__ kinv,
    const uint8_t* __restrict__ valid, bf16* __restrict__ rd) {
    extern __shared__ __align__(128) unsigned char rsm[];
    const int N = p.N, T = p.T, H = p.H, NQ = p.NQ, G = p.G;
    const int NB = (T + G - 1) / G;
    const ReadMmaSmem L = read_mma_layout(N, DK, DV);
    bf16* Ks = reinterpret_cast<bf16*>(rsm + L.K);
    bf16* Vs = reinterpret_cast<bf16*>(rsm + L.V);
    bf16* PQ = reinterpret_cast<bf16*>(rsm + L.PQ);
    float* s_kv = reinterpret_cast<float*>(rsm + L.kv);
    float* s_red = reinterpret_cast<float*>(rsm + L.red);
    float* s_scale = reinterpret_cast<float*>(rsm + L.scale);
    int* s_misc = reinterpret_cast<int*>(rsm + L.misc);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(rsm + L.bar);
    const int so = blockIdx.x;                                 // (b * NB + nb) * H + h
    const int h = so % H, nb = (so / H) % NB, b = so / (H * NB);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = nb * G, tc = min(G, T - t0), M = tc * NQ;   // queries that read this snapshot
    const bf16* Kb = kbuf + (size_t)so * N * DK;
    const bf16* Vb = vbuf + (size_t)so * N * DV;
    const int NPfull = (N + 15) & ~15;

    // ---- which rows count: kinv of the valid rows, -1 for the rest; nv = highest valid row + 1 ----
    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        mbar_fence_init();
        s_misc[0] = 0;
    }
    __syncthreads();
    {
        int hi = 0;
        for (int n = tid; n < NPfull; n += RM_THREADS) {
            const bool v = n < N && valid[(size_t)so * N + n] != 0;
            s_kv[n] = v ? kinv[(size_t)so * N + n] : -1.f;
            if (v) hi = n + 1;
        }
        hi = (int)__reduce_max_sync(FULL, (unsigned)hi);
        if (lane == 0 && hi > 0) atomicMax(&s_misc[0], hi);
    }
    __syncthreads();
    const int nv = s_misc[0];
    if (nv <= RM_SPARSE_ROWS) return;                          // few rows: the CUDA-core kernel, launched beside this one, reads it
    if (nv == 0) {                                             // the empty memory reads exactly zero
        for (int i = tid; i < M * DV; i += RM_THREADS) {
            const int m = i / DV, d = i - m * DV;
            const size_t qi = (((size_t)b * T + t0 + m / NQ) * H + h) * NQ + m % NQ;
            rd[qi * DV + d] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int NPv = (nv + 15) & ~15;                           // rows the MMAs visit
    // ---- snapshot rows 0 .. nv-1 in flight: keys on barrier 0, values on barrier 1; pad rows zeroed ----
    if (warp == 0) {
        if (lane == 0) {
            mbar_arrive_expect_tx(&s_bar[0], (unsigned)nv * DK * 2);
            mbar_arrive_expect_tx(&s_bar[1], (unsigned)nv * DV * 2);
        }
        __syncwarp();
        for (int n = lane; n < nv; n += 32) bulk_g2s(Ks + (size_t)n * L.ldk, Kb + (size_t)n * DK, DK * 2, &s_bar[0]);
        for (int n = lane; n < nv; n += 32) bulk_g2s(Vs + (size_t)n * L.ldv, Vb + (size_t)n * DV, DV * 2, &s_bar[1]);
    } else {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (int i = tid - 32; i < (NPv - nv) * (DK / 8); i += RM_THREADS - 32)
            *reinterpret_cast<uint4*>(Ks + (size_t)(nv + i / (DK / 8)) * L.ldk + (i % (DK / 8)) * 8) = z;
        for (int i = tid - 32; i < (NPv - nv) * (DV / 8); i += RM_THREADS - 32)
            *reinterpret_cast<uint4*>(Vs + (size_t)(nv + i / (DV / 8)) * L.ldv + (i % (DV / 8)) * 8) = z;
    }

    const int r0 = lane >> 2, cq = (lane & 3) * 2;             // this thread's rows r0, r0 + 8 and column pair in a C tile
    for (int m0 = 0; m0 < M; m0 += 16) {
        // ---- the 16 queries of this tile into shared memory (bf16 as given), their float32 scale ----
        for (int i = tid; i < 16 * (DK / 8); i += RM_THREADS) {
            const int mm = i / (DK / 8), c8 = (i % (DK / 8)) * 8, m = m0 + mm;
            uint4 u = make_uint4(0u, 0u, 0u, 0u);
            if (m < M) {
                const size_t qi = (((size_t)b * T + t0 + m / NQ) * H + h) * NQ + m % NQ;
                u = *reinterpret_cast<const uint4*>(qr + qi * DK + c8);
            }
            *reinterpret_cast<uint4*>(PQ + (size_t)mm * L.ldp + c8) = u;
        }
        __syncthreads();
        for (int mm = warp; mm < 16; mm += RM_WARPS) {         // |q| in float32, 4 rows per warp
            float qq = 0.f;
            for (int d = lane; d < DK; d += 32) { const float x = __bfloat162float(PQ[(size_t)mm * L.ldp + d]); qq = fmaf(x, x, qq); }
            qq = warp_sum(qq);
            const int m = m0 + mm;
            if (lane == 0) {
                float sc = 0.f;
                if (m < M) {
                    const size_t qi = (((size_t)b * T + t0 + m / NQ) * H + h) * NQ + m % NQ;
                    sc = sharp[qi] / fmaxf(sqrtf(qq), 1e-6f);
                }
                s_scale[mm] = sc;
            }
        }
        unsigned qa[DK / 16][4];                               // A fragments of the query tile
#pragma unroll
        for (int ks = 0; ks < DK / 16; ks++)
            ldsm_x4(qa[ks], PQ + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * L.ldp + ks * 16 + (lane >> 4) * 8);
        bool ok = true;
        if (m0 == 0) ok = mbar_wait_bounded(&s_bar[0], 0u);
        if (!__syncthreads_and(ok ? 1 : 0)) {                  // also orders: scales written, every warp holds its Q fragments
            if (tid == 0) atomicExch(&g_read_status, 1);
            return;
        }
        // ---- S = Q K^T over this warp's row tiles, scaled and masked ----
        float sc[RM_TPW][4];
        float mx0 = -INFINITY, mx1 = -INFINITY;
        const float sca = s_scale[r0], scb = s_scale[r0 + 8];
#pragma unroll
        for (int i = 0; i < RM_TPW; i++) {
            const int nt = warp + i * RM_WARPS;                // 8-row tile index
            sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = -INFINITY;
            if (nt * 8 < NPv) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int ks = 0; ks < DK / 16; ks++) {
                    unsigned b0, b1;
                    ldsm_x2(b0, b1, Ks + (size_t)(nt * 8 + (lane & 7)) * L.ldk + ks * 16 + ((lane >> 3) & 1) * 8);
                    mma_bf16(acc, qa[ks], b0, b1);
                }
                const float k0 = s_kv[nt * 8 + cq], k1 = s_kv[nt * 8 + cq + 1];
                sc[i][0] = k0 >= 0.f ? acc[0] * k0 * sca : -INFINITY;
                sc[i][1] = k1 >= 0.f ? acc[1] * k1 * sca : -INFINITY;
                sc[i][2] = k0 >= 0.f ? acc[2] * k0 * scb : -INFINITY;
                sc[i][3] = k1 >= 0.f ? acc[3] * k1 * scb : -INFINITY;
                mx0 = fmaxf(mx0, fmaxf(sc[i][0], sc[i][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[i][2], sc[i][3]));
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(FULL, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(FULL, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(FULL, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(FULL, mx1, 2));
        if ((lane & 3) == 0) { s_red[warp * 16 + r0] = mx0; s_red[warp * 16 + r0 + 8] = mx1; }
        __syncthreads();
        mx0 = fmaxf(fmaxf(s_red[r0], s_red[16 + r0]), fmaxf(s_red[32 + r0], s_red[48 + r0]));
        mx1 = fmaxf(fmaxf(s_red[r0 + 8], s_red[16 + r0 + 8]), fmaxf(s_red[32 + r0 + 8], s_red[48 + r0 + 8]));
        // ---- P = exp(S - max) as bf16 into shared memory (over the query tile, which every warp already holds) ----
        float su0 = 0.f, su1 = 0.f;
#pragma unroll
        for (int i = 0; i < RM_TPW; i++) {
            const int nt = warp + i * RM_WARPS;
            if (nt * 8 < NPv) {
                const float e0 = __expf(sc[i][0] - mx0), e1 = __expf(sc[i][1] - mx0);   // exp(-inf) = 0 for masked rows
                const float e2 = __expf(sc[i][2] - mx1), e3 = __expf(sc[i][3] - mx1);
                su0 += e0 + e1; su1 += e2 + e3;
                *reinterpret_cast<__nv_bfloat162*>(PQ + (size_t)r0 * L.ldp + nt * 8 + cq) = __floats2bfloat162_rn(e0, e1);
                *reinterpret_cast<__nv_bfloat162*>(PQ + (size_t)(r0 + 8) * L.ldp + nt * 8 + cq) = __floats2bfloat162_rn(e2, e3);
            }
        }
        su0 += __shfl_xor_sync(FULL, su0, 1); su0 += __shfl_xor_sync(FULL, su0, 2);
        su1 += __shfl_xor_sync(FULL, su1, 1); su1 += __shfl_xor_sync(FULL, su1, 2);
        float* s_sum = s_red + RM_WARPS * 16;
        if ((lane & 3) == 0) { s_sum[warp * 16 + r0] = su0; s_sum[warp * 16 + r0 + 8] = su1; }
        ok = true;
        if (m0 == 0) ok = mbar_wait_bounded(&s_bar[1], 0u);
        if (!__syncthreads_and(ok ? 1 : 0)) {
            if (tid == 0) atomicExch(&g_read_status, 1);
            return;
        }
        // ---- O = P V: this warp's quarter of the value columns ----
        constexpr int DT = DV / 8 / RM_WARPS;                  // 8-column tiles per warp
        float o[DT][4];
#pragma unroll
        for (int j = 0; j < DT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        for (int ks = 0; ks < NPv / 16; ks++) {
            unsigned pa[4];
            ldsm_x4(pa, PQ + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * L.ldp + ks * 16 + (lane >> 4) * 8);
#pragma unroll
            for (int j = 0; j < DT; j++) {
                unsigned b0, b1;
                ldsm_x2_trans(b0, b1, Vs + (size_t)(ks * 16 + (lane & 15)) * L.ldv + (warp * DT + j) * 8);
                mma_bf16(o[j], pa, b0, b1);
            }
        }
        const float inv0 = 1.f / ((s_sum[r0] + s_sum[16 + r0]) + (s_sum[32 + r0] + s_sum[48 + r0]));
        const float inv1 = 1.f / ((s_sum[r0 + 8] + s_sum[16 + r0 + 8]) + (s_sum[32 + r0 + 8] + s_sum[48 + r0 + 8]));
        const int ma = m0 + r0, mb = m0 + r0 + 8;
#pragma unroll
        for (int j = 0; j < DT; j++) {
            const int d = (warp * DT + j) * 8 + cq;
            if (ma < M) {
                const size_t qi = (((size_t)b * T + t0 + ma / NQ) * H + h) * NQ + ma % NQ;
                *reinterpret_cast<__nv_bfloat162*>(rd + qi * DV + d) = __floats2bfloat162_rn(o[j][0] * inv0, o[j][1] * inv0);
            }
            if (mb < M) {
                const size_t qi = (((size_t)b * T + t0 + mb / NQ) * H + h) * NQ + mb % NQ;
                *reinterpret_cast<__nv_bfloat162*>(rd + qi * DV + d) = __floats2bfloat162_rn(o[j][2] * inv1, o[j][3] * inv1);
            }
        }
        __syncthreads();                                       // PQ and the exchange arrays are reused by the next query tile
    }
}


// ======================================================================================================
// The same read as a PERSISTENT, warp-specialised kernel: one CTA per SM walks its share of the snapshots; one warp
// only issues copies and runs ahead of eight math warps, coupled to them by mbarriers alone ("tile landed" one way,
// "tile free" the other).  The kernel above pays, per snapshot, a serial chain "which rows count -> rows land ->
// Q K^T -> softmax -> P V" (about 20 us with two CTAs per SM: 17 % of DRAM peak); here only the math is on that chain
// and the copies of the next snapshots are in flight all the time: the key tile of snapshot i + 2 is requested as soon
// as Q K^T of snapshot i is done, its value tile when P V of snapshot i is done (a memory-bound kernel needs
// bandwidth x latency, about 90 KB per SM, in flight; one snapshot ahead was measured at 0.41 of the HBM peak).
//   * key / value tiles come in by TILED bulk tensor copies (a 3-D tensor map over (snapshot, row, column), box
//     64 columns x 64 / 128 / 192 rows, 128-byte swizzle): 2 copies per tensor and snapshot instead of one per row,
//     no row padding, and ldmatrix reads the swizzled tile without bank conflicts (16-byte chunk c of row r sits at
//     chunk c ^ (r & 7));
//   * the box height is the smallest that covers the highest valid row, read from the valid vector, which comes in
//     through a four-deep ring of small bulk copies together with kinv;
//   * the 16 query rows by plain bulk copies; sharp by ordinary loads one snapshot ahead.
// Needs G * NQ <= 16, N a multiple of 16 and dk = dv in {64, 128}; other shapes take the kernel above.
constexpr int RR_WARPS = 8;                            // math warps; warp RR_WARPS issues the copies
constexpr int RR_THREADS = (RR_WARPS + 1) * 32;
constexpr int RR_TPW = RM_MAXN / 8 / RR_WARPS;         // 8-row tiles per math warp
constexpr int RR_ROWS = RM_MAXN;                       // rows per sub-tile slot in shared memory
constexpr int RR_SUB = RR_ROWS * 128;                  // bytes of one 64-column sub-tile slot (a multiple of 1024)
constexpr int RR_META = 4;                             // kinv / valid vectors in flight
struct ReadMaps { CUtensorMap k[3], v[3]; };           // box heights min(N, 64), min(N, 128), N

struct ReadRingSmem { int stage, stage_bytes, q, q_bytes, pbuf, meta, kv, red, scale, sharp, nv, bar, total; int ldq, ldp; };
__host__ __device__ inline ReadRingSmem read_ring_layout(int DK) {
    ReadRingSmem L;
    const int nsub = DK / 64;
    L.ldq = DK + 8; L.ldp = RM_MAXN + 8;               // padded rows: conflict-free ldmatrix
    L.stage = 0;
    L.stage_bytes = 2 * nsub * RR_SUB;                 // keys then values
    L.q = 2 * L.stage_bytes;
    L.q_bytes = 16 * L.ldq * 2;                        // 16 query rows per stage
    L.pbuf = L.q + 2 * L.q_bytes;                      // P = exp(S - max) as bf16, 16 x N
    L.meta = L.pbuf + 16 * L.ldp * 2;                  // RR_META x (kinv [N] f32 | valid [N] u8), 1 KB each
    L.kv = L.meta + RR_META * 1024;                    // [2 stages][N] kinv of a valid row, -1 for the others
    L.red = L.kv + 2 * RM_MAXN * 4;
    L.scale = L.red + 2 * RR_WARPS * 16 * 4;
    L.sharp = L.scale + 16 * 4;                        // [2 stages][16]
    L.nv = L.sharp + 2 * 16 * 4;                       // [0..1] highest valid row + 1 per stage, [2] failure flag,
                                                       // [4..5] snapshot index per stage (-1: no more)
    L.bar = L.nv + 32;                                 // meta[RR_META], fullL[2], fullV[2], emptyK[2], emptyV[2]
    L.total = L.bar + (RR_META + 8) * 8;
    return L;
}

__device__ __forceinline__ void tensor_g2s_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {       // bytes to come; no arrival
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// barrier among the math warps only (the copy-issuing warp never joins it)
__device__ __forceinline__ void math_sync() { asm volatile("bar.sync 1, %0;" ::"n"(RR_WARPS * 32) : "memory"); }
// the same with an AND over the math threads' flags: every thread gets the same answer, so a wait that gave up in one
// thread ends the loop in all of them at the same place (a thread must never be left alone at a barrier)
__device__ __forceinline__ bool math_sync_and(bool ok) {
    int r;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.s32 q, %1, 0;\n"
        "bar.red.and.pred p, 1, %2, q;\n"
        "selp.s32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(r)
        : "r"((int)ok), "n"(RR_WARPS * 32)
        : "memory");
    return r != 0;
}

template <int DK>
__global__ void __launch_bounds__(RR_THREADS, 1) read_fwd_ring_kernel(
    const slotscan_read_params p, const __grid_constant__ ReadMaps maps, const bf16* __restrict__ qr,
    const float* __restrict__ sharp, const float* __restrict__ kinv, const uint8_t* __restrict__ valid,
    bf16* __restrict__ rd, const int nitems) {
    constexpr int DV = DK, NSUB = DK / 64;
    static_assert(DV / 8 % RR_WARPS == 0, "each math warp owns whole 8-column tiles of the values");
    extern __shared__ __align__(128) unsigned char rsm[];
    // the swizzled tiles want a 1024-byte boundary (the launch adds 1 KB of slack for this)
    unsigned char* const rsmb = rsm + ((1024u - (smem_u32(rsm) & 1023u)) & 1023u);
    const int N = p.N, T = p.T, H = p.H, NQ = p.NQ, G = p.G;
    const int NB = (T + G - 1) / G;
    const ReadRingSmem L = read_ring_layout(DK);
    float* s_kvst = reinterpret_cast<float*>(rsmb + L.kv);
    float* s_red = reinterpret_cast<float*>(rsmb + L.red);
    float* s_scale = reinterpret_cast<float*>(rsmb + L.scale);
    float* s_sharpst = reinterpret_cast<float*>(rsmb + L.sharp);
    volatile int* s_nv = reinterpret_cast<int*>(rsmb + L.nv);
    uint64_t* barM = reinterpret_cast<uint64_t*>(rsmb + L.bar);
    uint64_t* fullL = barM + RR_META;
    uint64_t* fullV = fullL + 2;
    uint64_t* emptyK = fullV + 2;
    uint64_t* emptyV = emptyK + 2;
    bf16* Pb = reinterpret_cast<bf16*>(rsmb + L.pbuf);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = blockIdx.x, stride = gridDim.x;
    const int h64 = min(N, 64), h128 = min(N, 128);
    const int nmine = first < nitems ? (nitems - first + stride - 1) / stride : 0;   // snapshots of this CTA

    auto q_stage = [&](int s) { return reinterpret_cast<bf16*>(rsmb + L.q + s * L.q_bytes); };
    // queries of snapshot `it`: (b, block, h) -> token t0 + m / NQ, query m % NQ
    auto q_index = [&](int it, int m) {
        const int hh = it % H, nb = (it / H) % NB, bb = it / (H * NB);
        return (((size_t)bb * T + nb * G + m / NQ) * H + hh) * NQ + m % NQ;
    };
    auto q_count = [&](int it) { const int nb = (it / H) % NB; return min(G, T - nb * G) * NQ; };

    if (tid == 0) {
        for (int i = 0; i < RR_META + 4; i++) mbar_init(&barM[i], 1);      // meta, fullL, fullV: one arrive (+ bytes)
        for (int i = 0; i < 4; i++) mbar_init(&emptyK[i], RR_WARPS);       // emptyK, emptyV: one arrive per math warp
        mbar_fence_init();
        s_nv[0] = s_nv[1] = s_nv[2] = 0;
    }
    for (int i = tid; i < 2 * L.q_bytes / 16; i += RR_THREADS)            // query rows beyond a short last block stay zero
        reinterpret_cast<uint4*>(rsmb + L.q)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
    __syncthreads();

    if (warp == RR_WARPS) {
        // ================= the copy-issuing warp =================
        auto issue_meta = [&](int k) {                                     // kinv / valid of this CTA's k-th snapshot
            if (lane == 0 && k < nmine) {
                const int it = first + k * stride, slot = k % RR_META;
                mbar_arrive_expect_tx(&barM[slot], (unsigned)(N * 5));
                bulk_g2s(rsmb + L.meta + slot * 1024, kinv + (size_t)it * N, N * 4, &barM[slot]);
                bulk_g2s(rsmb + L.meta + slot * 1024 + RM_MAXN * 4, valid + (size_t)it * N, N, &barM[slot]);
            }
        };
        for (int k = 0; k < RR_META; k++) issue_meta(k);
        int kd = 0;                                                        // snapshots handed to the math warps so far
        bool alive = true;
        for (int k = 0; k < nmine; k++) {
            const int it = first + k * stride, slot = k % RR_META;
            if (!__all_sync(FULL, mbar_wait_bounded(&barM[slot], (unsigned)((k / RR_META) & 1)))) { alive = false; break; }   // warp-uniform
            // kinv or -1 per row and the highest valid row, from the landed vectors; then the slot is free again
            const float* mk = reinterpret_cast<const float*>(rsmb + L.meta + slot * 1024);
            const unsigned char* mv = rsmb + L.meta + slot * 1024 + RM_MAXN * 4;
            float kvr[RM_MAXN / 32];
            int hi = 0;
#pragma unroll
            for (int j = 0; j < RM_MAXN / 32; j++) {
                const int n = lane + 32 * j;
                const bool v = n < N && mv[n] != 0;
                kvr[j] = v ? mk[n] : -1.f;
                if (v) hi = n + 1;
            }
            const int nv = (int)__reduce_max_sync(FULL, (unsigned)hi);
            fence_proxy_async_smem();
            __syncwarp();
            issue_meta(k + RR_META);
            if (nv <= RM_SPARSE_ROWS) continue;                            // left to the CUDA-core kernel: the math warps never see it
            const int M = q_count(it);
            const float sh = (lane < 16 && lane < M) ? sharp[q_index(it, lane)] : 0.f;   // needed only after the copies are out
            const int s = kd & 1;
            const unsigned epar = (unsigned)(((kd >> 1) & 1) ^ 1);         // the phase that snapshot kd - 2 completed
            // the key tile, the queries and the per-row vectors of stage s: free once Q K^T of snapshot kd - 2 is done
            if (kd >= 2 && !__all_sync(FULL, mbar_wait_bounded(&emptyK[s], epar))) { alive = false; break; }
            const int sel = nv <= h64 ? 0 : (nv <= h128 ? 1 : 2);
            const int rows = sel == 0 ? h64 : (sel == 1 ? h128 : N);
            unsigned char* st = rsmb + L.stage + s * L.stage_bytes;
            if (lane == 0) mbar_expect_tx(&fullL[s], (unsigned)(M * DK * 2 + rows * DK * 2));
            __syncwarp();
            if (lane < NSUB) tensor_g2s_3d(st + lane * RR_SUB, &maps.k[sel], lane * 64, 0, it, &fullL[s]);
            if (lane < M) bulk_g2s(q_stage(s) + (size_t)lane * L.ldq, qr + q_index(it, lane) * DK, DK * 2, &fullL[s]);
#pragma unroll
            for (int j = 0; j < RM_MAXN / 32; j++) s_kvst[s * RM_MAXN + lane + 32 * j] = kvr[j];
            if (lane < 16) s_sharpst[s * 16 + lane] = sh;
            if (lane == 0) { s_nv[s] = nv; s_nv[4 + s] = it; }
            __syncwarp();
            if (lane == 0) mbar_arrive(&fullL[s]);                         // the vectors are written; the phase ends when the bytes are in
            // the value tile: free once P V of snapshot kd - 2 is done
            if (kd >= 2 && !__all_sync(FULL, mbar_wait_bounded(&emptyV[s], epar))) { alive = false; break; }
            if (lane == 0) mbar_arrive_expect_tx(&fullV[s], (unsigned)(rows * DV * 2));
            __syncwarp();
            if (lane < NSUB) tensor_g2s_3d(st + (NSUB + lane) * RR_SUB, &maps.v[sel], lane * 64, 0, it, &fullV[s]);
            kd++;
        }
        if (alive) {                                                       // tell the math warps that nothing follows
            const int s = kd & 1;
            if (kd >= 2 && !__all_sync(FULL, mbar_wait_bounded(&emptyK[s], (unsigned)(((kd >> 1) & 1) ^ 1)))) alive = false;
            if (alive) {
                if (lane == 0) s_nv[4 + s] = -1;
                __syncwarp();
                if (lane == 0) mbar_arrive(&fullL[s]);
            }
        }
        if (!alive) s_nv[2] = 1;
    } else {
        // ================= the math warps =================
        const int r0 = lane >> 2, cq = (lane & 3) * 2;             // this thread's rows r0, r0 + 8 and column pair in a C tile
        bool failed = false;
        for (int kd = 0;; kd++) {                                  // the snapshots the copy-issuing warp hands over, in order
            const int s = kd & 1;
            const unsigned par = (unsigned)((kd >> 1) & 1);
            if (!math_sync_and(mbar_wait_bounded(&fullL[s], par))) { failed = true; break; }
            const int it = s_nv[4 + s];
            if (it < 0) break;
            const int nv = s_nv[s];
            const int M = q_count(it);
            const int NPv = (nv + 15) & ~15;
            const unsigned char* Kst = rsmb + L.stage + s * L.stage_bytes;
            const unsigned char* Vst = Kst + NSUB * RR_SUB;
            const bf16* Qs = q_stage(s);
            const float* s_kv = s_kvst + s * RM_MAXN;
            for (int mm = warp; mm < 16; mm += RR_WARPS) {         // |q| in float32, 2 rows per warp
                float qq = 0.f;
                for (int d = lane; d < DK; d += 32) { const float x = __bfloat162float(Qs[(size_t)mm * L.ldq + d]); qq = fmaf(x, x, qq); }
                qq = warp_sum(qq);
                if (lane == 0) s_scale[mm] = mm < M ? s_sharpst[s * 16 + mm] / fmaxf(sqrtf(qq), 1e-6f) : 0.f;
            }
            unsigned qa[DK / 16][4];                               // A fragments of the query tile
#pragma unroll
            for (int ks = 0; ks < DK / 16; ks++)
                ldsm_x4(qa[ks], Qs + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * L.ldq + ks * 16 + (lane >> 4) * 8);
            math_sync();                                           // scales written
            // ---- S = Q K^T over this warp's row tiles, scaled and masked ----
            float sc[RR_TPW][4];
            float mx0 = -INFINITY, mx1 = -INFINITY;
            const float sca = s_scale[r0], scb = s_scale[r0 + 8];
#pragma unroll
            for (int j = 0; j < RR_TPW; j++) {
                const int nt = warp + j * RR_WARPS;                // 8-row tile index
                sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = -INFINITY;
                if (nt * 8 < NPv) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    const int row = nt * 8 + (lane & 7);
#pragma unroll
                    for (int ks = 0; ks < DK / 16; ks++) {
                        const int cidx = ks * 2 + ((lane >> 3) & 1);
                        unsigned b0, b1;
                        ldsm_x2(b0, b1, Kst + (cidx >> 3) * RR_SUB + row * 128 + (((cidx & 7) ^ (row & 7)) << 4));
                        mma_bf16(acc, qa[ks], b0, b1);
                    }
                    const float k0 = s_kv[nt * 8 + cq], k1 = s_kv[nt * 8 + cq + 1];
                    sc[j][0] = k0 >= 0.f ? acc[0] * k0 * sca : -INFINITY;
                    sc[j][1] = k1 >= 0.f ? acc[1] * k1 * sca : -INFINITY;
                    sc[j][2] = k0 >= 0.f ? acc[2] * k0 * scb : -INFINITY;
                    sc[j][3] = k1 >= 0.f ? acc[3] * k1 * scb : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                    mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&emptyK[s]);                // this warp is done with the key tile, the queries, kinv
            mx0 = fmaxf(mx0, __shfl_xor_sync(FULL, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(FULL, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(FULL, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(FULL, mx1, 2));
            if ((lane & 3) == 0) { s_red[warp * 16 + r0] = mx0; s_red[warp * 16 + r0 + 8] = mx1; }
            math_sync();
            mx0 = s_red[r0]; mx1 = s_red[r0 + 8];
#pragma unroll
            for (int w = 1; w < RR_WARPS; w++) { mx0 = fmaxf(mx0, s_red[w * 16 + r0]); mx1 = fmaxf(mx1, s_red[w * 16 + r0 + 8]); }
            // ---- P = exp(S - max) as bf16 ----
            float su0 = 0.f, su1 = 0.f;
#pragma unroll
            for (int j = 0; j < RR_TPW; j++) {
                const int nt = warp + j * RR_WARPS;
                if (nt * 8 < NPv) {
                    const float e0 = __expf(sc[j][0] - mx0), e1 = __expf(sc[j][1] - mx0);   // exp(-inf) = 0 for masked rows
                    const float e2 = __expf(sc[j][2] - mx1), e3 = __expf(sc[j][3] - mx1);
                    su0 += e0 + e1; su1 += e2 + e3;
                    *reinterpret_cast<__nv_bfloat162*>(Pb + (size_t)r0 * L.ldp + nt * 8 + cq) = __floats2bfloat162_rn(e0, e1);
                    *reinterpret_cast<__nv_bfloat162*>(Pb + (size_t)(r0 + 8) * L.ldp + nt * 8 + cq) = __floats2bfloat162_rn(e2, e3);
                }
            }
            su0 += __shfl_xor_sync(FULL, su0, 1); su0 += __shfl_xor_sync(FULL, su0, 2);
            su1 += __shfl_xor_sync(FULL, su1, 1); su1 += __shfl_xor_sync(FULL, su1, 2);
            float* s_sum = s_red + RR_WARPS * 16;
            if ((lane & 3) == 0) { s_sum[warp * 16 + r0] = su0; s_sum[warp * 16 + r0 + 8] = su1; }
            if (!math_sync_and(mbar_wait_bounded(&fullV[s], par))) { failed = true; break; }   // also: P and the sums are written
            // ---- O = P V: this warp's share of the value columns ----
            constexpr int DT = DV / 8 / RR_WARPS;                  // 8-column tiles per warp
            float o[DT][4];
#pragma unroll
            for (int j = 0; j < DT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
#pragma unroll 2
            for (int ks = 0; ks < NPv / 16; ks++) {
                unsigned pa[4];
                ldsm_x4(pa, Pb + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * L.ldp + ks * 16 + (lane >> 4) * 8);
                const int row = ks * 16 + (lane & 15);
#pragma unroll
                for (int j = 0; j < DT; j++) {
                    const int cidx = warp * DT + j;
                    unsigned b0, b1;
                    ldsm_x2_trans(b0, b1, Vst + (cidx >> 3) * RR_SUB + row * 128 + (((cidx & 7) ^ (row & 7)) << 4));
                    mma_bf16(o[j], pa, b0, b1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&emptyV[s]);                // this warp is done with the value tile
            float t0s = 0.f, t1s = 0.f;
#pragma unroll
            for (int w = 0; w < RR_WARPS; w++) { t0s += s_sum[w * 16 + r0]; t1s += s_sum[w * 16 + r0 + 8]; }
            const float inv0 = 1.f / t0s, inv1 = 1.f / t1s;
            const size_t qi0 = q_index(it, r0), qi1 = q_index(it, r0 + 8);
#pragma unroll
            for (int j = 0; j < DT; j++) {
                const int d = (warp * DT + j) * 8 + cq;
                if (r0 < M) *reinterpret_cast<__nv_bfloat162*>(rd + qi0 * DV + d) = __floats2bfloat162_rn(o[j][0] * inv0, o[j][1] * inv0);
                if (r0 + 8 < M) *reinterpret_cast<__nv_bfloat162*>(rd + qi1 * DV + d) = __floats2bfloat162_rn(o[j][2] * inv1, o[j][3] * inv1);
            }
            // no barrier here: the next snapshot's first barrier comes before anything of this one is overwritten
        }
        if (failed) s_nv[2] = 1;
    }
    __syncthreads();
    if (s_nv[2] != 0) {                                            // a bounded wait gave up: report, and give the copies still
        if (tid == 0) atomicExch(&g_read_status, 1);               // in flight into this CTA's shared memory time to land
        for (int k = 0; k < 1000; k++) __nanosleep(1000);
    }
}

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return (TensorMapEncodeFn)f;
    }();
    return fn;
}

// (snapshot, row, column) bf16 tensor with a box of 64 columns x `rows` rows of one snapshot, 128-byte swizzle
static bool snapshot_map(CUtensorMap* m, const void* base, long long nsnap, int N, int D, int rows) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (enc == nullptr) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)nsnap};
    const cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)N * D * 2};
    const cuuint32_t box[3] = {64u, (cuuint32_t)rows, 1u};
    const cuuint32_t es[3] = {1u, 1u, 1u};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// false when the ring kernel does not apply (shape, or no tensor-map support in the driver): the caller falls back
template <int DK>
static bool launch_ring(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf, const void* vbuf,
                        const float* kinv, const uint8_t* valid, void* rd, cudaStream_t st, cudaError_t* err) {
    const int NB = (p.T + p.G - 1) / p.G;
    const long long nsnap = (long long)p.B * NB * p.H;
    if (p.N % 16 || p.G * p.NQ > 16 || nsnap > 2147483647LL || (((uintptr_t)kinv | (uintptr_t)valid) & 15)) return false;
    ReadMaps maps;
    const int hs[3] = {p.N < 64 ? p.N : 64, p.N < 128 ? p.N : 128, p.N};
    for (int i = 0; i < 3; i++)
        if (!snapshot_map(&maps.k[i], kbuf, nsnap, p.N, DK, hs[i]) || !snapshot_map(&maps.v[i], vbuf, nsnap, p.N, DK, hs[i])) return false;
    const size_t sm = (size_t)read_ring_layout(DK).total + 1024;      // + slack: the stages start on a 1024-byte boundary
    auto kern = read_fwd_ring_kernel<DK>;
    if ((*err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return true;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(nsnap < sms ? nsnap : sms);
    kern<<<grid, RR_THREADS, sm, st>>>(p, maps, (const bf16*)qr, sharp, kinv, valid, (bf16*)rd, (int)nsnap);
    *err = cudaGetLastError();
    return true;
}


// ======================================================================================================
// Backward of the read on the tensor cores, same pipeline as read_fwd_ring_kernel (persistent CTA, a copy-issuing warp
// ahead of eight math warps, tiled bulk tensor copies).  Per snapshot, with the M = 16 queries as one row block:
//     S = Q K^T, dA = dO V^T                 (16 x N each, the two share every fragment layout)
//     att = softmax(S * kinv_n * scale_m),  dl = att * (dA - sum_n att dA)
//     dsharp_m = sum_n dl * base,  dkinv_n = sum_m dl * (Q K^T) * scale_m
//     G = dl * kinv_n * scale_m  (bf16),  att (bf16)
//     dq'= G K   -> dq = dq' - qn <dq', qn>   (the query normalisation; dq' alone under the norm clamp)
//     dK = G^T Q,  dV = att^T dO             (N x dk each, one k-step of 16 per tile)
// [adjoint of gqa25/memlm_sh.py:379-397 as autograd takes it; G and att enter the MMAs in bf16 as the forward's P does]
// dK / dV tiles are written, as bf16, back into the shared-memory tiles their K / V came in (same swizzle) and leave by
// tiled bulk tensor STORES issued by the copy-issuing warp, whole snapshots at a time (rows above the highest valid
// row are written as zeros).  Snapshots with few rows in use are left to the CUDA-core kernel.
struct ReadBwdMaps { CUtensorMap k[3], v[3], dk, dv; };
struct ReadBwdSmem { int stage, stage_bytes, q, dO, pbuf, gbuf, meta, kv, redA, redB, scale, qinv, sharp, nv, bar, total; int ldq, ldp; };
__host__ __device__ inline ReadBwdSmem read_bwd_ring_layout(int DK) {
    ReadBwdSmem L;
    const int nsub = DK / 64;
    L.ldq = DK + 8; L.ldp = RM_MAXN + 8;
    L.stage = 0;
    L.stage_bytes = 2 * nsub * RR_SUB;
    L.q = 2 * L.stage_bytes;                           // 16 query rows (one buffer: its fragments go to registers early)
    L.dO = L.q + 16 * L.ldq * 2;                       // 16 rows of the upstream gradient
    L.pbuf = L.dO + 16 * L.ldq * 2;                    // att as bf16, 16 x N
    L.gbuf = L.pbuf + 16 * L.ldp * 2;                  // G as bf16, 16 x N
    L.meta = L.gbuf + 16 * L.ldp * 2;
    L.kv = L.meta + RR_META * 1024;
    L.redA = L.kv + 2 * RM_MAXN * 4;                   // [8 warps][16]: row maxima, later the dsharp partials
    L.redB = L.redA + RR_WARPS * 16 * 4;               // [2][8][16]: sum e, sum e dA; later the projection partials
    L.scale = L.redB + 2 * RR_WARPS * 16 * 4;
    L.qinv = L.scale + 16 * 4;
    L.sharp = L.qinv + 16 * 4;                         // [2 stages][16]
    L.nv = L.sharp + 2 * 16 * 4;                       // [0..1] rows, [2] failure flag, [4..5] snapshot index per stage
    L.bar = L.nv + 32;                                 // meta[RR_META], fullL[2], fullQ, emptyQ, staged[2]
    L.total = L.bar + (RR_META + 6) * 8;
    return L;
}

__device__ __forceinline__ void tensor_s2g_3d(const CUtensorMap* map, int x, int y, int z, const void* src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

template <int DK>
__global__ void __launch_bounds__(RR_THREADS, 1) read_bwd_ring_kernel(
    const slotscan_read_params p, const __grid_constant__ ReadBwdMaps maps, const bf16* __restrict__ qr,
    const float* __restrict__ sharp, const float* __restrict__ kinv, const uint8_t* __restrict__ valid,
    const bf16* __restrict__ drd, bf16* __restrict__ dqr, float* __restrict__ dsharp, float* __restrict__ dkinv,
    const int nitems) {
    constexpr int DV = DK, NSUB = DK / 64;
    constexpr int DT = DV / 8 / RR_WARPS;                      // 8-column tiles per math warp
    static_assert(DV / 8 % RR_WARPS == 0, "each math warp owns whole 8-column tiles");
    extern __shared__ __align__(128) unsigned char rsm[];
    unsigned char* const rsmb = rsm + ((1024u - (smem_u32(rsm) & 1023u)) & 1023u);
    const int N = p.N, T = p.T, H = p.H, NQ = p.NQ, G = p.G;
    const int NB = (T + G - 1) / G;
    const ReadBwdSmem L = read_bwd_ring_layout(DK);
    float* s_kvst = reinterpret_cast<float*>(rsmb + L.kv);
    float* s_redA = reinterpret_cast<float*>(rsmb + L.redA);
    float* s_redB = reinterpret_cast<float*>(rsmb + L.redB);
    float* s_scale = reinterpret_cast<float*>(rsmb + L.scale);
    float* s_qinv = reinterpret_cast<float*>(rsmb + L.qinv);
    float* s_sharpst = reinterpret_cast<float*>(rsmb + L.sharp);
    volatile int* s_nv = reinterpret_cast<int*>(rsmb + L.nv);
    uint64_t* barM = reinterpret_cast<uint64_t*>(rsmb + L.bar);
    uint64_t* fullL = barM + RR_META;
    uint64_t* fullQ = fullL + 2;
    uint64_t* emptyQ = fullQ + 1;
    uint64_t* staged = emptyQ + 1;
    bf16* Qs = reinterpret_cast<bf16*>(rsmb + L.q);
    bf16* Os = reinterpret_cast<bf16*>(rsmb + L.dO);
    bf16* Pb = reinterpret_cast<bf16*>(rsmb + L.pbuf);
    bf16* Gb = reinterpret_cast<bf16*>(rsmb + L.gbuf);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first = blockIdx.x, stride = gridDim.x;
    const int h64 = min(N, 64), h128 = min(N, 128);
    const int nmine = first < nitems ? (nitems - first + stride - 1) / stride : 0;

    auto q_index = [&](int it, int m) {
        const int hh = it % H, nb = (it / H) % NB, bb = it / (H * NB);
        return (((size_t)bb * T + nb * G + m / NQ) * H + hh) * NQ + m % NQ;
    };
    auto q_count = [&](int it) { const int nb = (it / H) % NB; return min(G, T - nb * G) * NQ; };

    if (tid == 0) {
        for (int i = 0; i < RR_META + 3; i++) mbar_init(&barM[i], 1);      // meta, fullL[2], fullQ
        mbar_init(emptyQ, 1);
        mbar_init(&staged[0], RR_WARPS);
        mbar_init(&staged[1], RR_WARPS);
        mbar_fence_init();
        s_nv[0] = s_nv[1] = s_nv[2] = 0;
    }
    for (int i = tid; i < 2 * 16 * L.ldq * 2 / 16; i += RR_THREADS)       // query / gradient rows beyond a short last block stay zero
        reinterpret_cast<uint4*>(rsmb + L.q)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
    __syncthreads();

    if (warp == RR_WARPS) {
        // ================= the copy-issuing warp =================
        auto issue_meta = [&](int k) {
            if (lane == 0 && k < nmine) {
                const int it = first + k * stride, slot = k % RR_META;
                mbar_arrive_expect_tx(&barM[slot], (unsigned)(N * 5));
                bulk_g2s(rsmb + L.meta + slot * 1024, kinv + (size_t)it * N, N * 4, &barM[slot]);
                bulk_g2s(rsmb + L.meta + slot * 1024 + RM_MAXN * 4, valid + (size_t)it * N, N, &barM[slot]);
            }
        };
        // snapshot gradients of the snapshot that used stage s leave shared memory; returns once they have been read
        auto store_stage = [&](int s, int it) {
            const unsigned char* st = rsmb + L.stage + s * L.stage_bytes;
            if (lane < NSUB) tensor_s2g_3d(&maps.dk, lane * 64, 0, it, st + lane * RR_SUB);
            else if (lane < 2 * NSUB) tensor_s2g_3d(&maps.dv, (lane - NSUB) * 64, 0, it, st + lane * RR_SUB);
            bulk_commit();
            bulk_wait_read<0>();
            __syncwarp();
        };
        for (int k = 0; k < RR_META; k++) issue_meta(k);
        int kd = 0, it_s0 = -1, it_s1 = -1;                              // snapshot whose gradients sit in stage 0 / 1
        bool alive = true;
        for (int k = 0; k < nmine; k++) {
            const int it = first + k * stride, slot = k % RR_META;
            if (!__all_sync(FULL, mbar_wait_bounded(&barM[slot], (unsigned)((k / RR_META) & 1)))) { alive = false; break; }
            const float* mk = reinterpret_cast<const float*>(rsmb + L.meta + slot * 1024);
            const unsigned char* mv = rsmb + L.meta + slot * 1024 + RM_MAXN * 4;
            float kvr[RM_MAXN / 32];
            int hi = 0;
#pragma unroll
            for (int j = 0; j < RM_MAXN / 32; j++) {
                const int n = lane + 32 * j;
                const bool v = n < N && mv[n] != 0;
                kvr[j] = v ? mk[n] : -1.f;
                if (v) hi = n + 1;
            }
            const int nv = (int)__reduce_max_sync(FULL, (unsigned)hi);
            fence_proxy_async_smem();
            __syncwarp();
            issue_meta(k + RR_META);
            if (nv <= RB_SPARSE_ROWS) continue;                            // left to the CUDA-core kernel
            const int M = q_count(it);
            const float sh = (lane < 16 && lane < M) ? sharp[q_index(it, lane)] : 0.f;
            // queries and upstream gradient: one buffer, free as soon as the math warps hold its fragments
            if (kd >= 1 && !__all_sync(FULL, mbar_wait_bounded(emptyQ, (unsigned)((kd - 1) & 1)))) { alive = false; break; }
            if (lane == 0) mbar_arrive_expect_tx(fullQ, (unsigned)(2 * M * DK * 2));
            __syncwarp();
            if (lane < M) {
                const size_t qi = q_index(it, lane);
                bulk_g2s(Qs + (size_t)lane * L.ldq, qr + qi * DK, DK * 2, fullQ);
                bulk_g2s(Os + (size_t)lane * L.ldq, drd + qi * DV, DV * 2, fullQ);
            }
            const int s = kd & 1;
            // stage s: the snapshot gradients of snapshot kd - 2 are staged in it; send them off, then it is free
            if (kd >= 2) {
                if (!__all_sync(FULL, mbar_wait_bounded(&staged[s], (unsigned)(((kd >> 1) & 1) ^ 1)))) { alive = false; break; }
                store_stage(s, s ? it_s1 : it_s0);
            }
            if (s) it_s1 = it; else it_s0 = it;
            const int sel = nv <= h64 ? 0 : (nv <= h128 ? 1 : 2);
            const int rows = sel == 0 ? h64 : (sel == 1 ? h128 : N);
            unsigned char* st = rsmb + L.stage + s * L.stage_bytes;
            if (lane == 0) mbar_expect_tx(&fullL[s], (unsigned)(rows * DK * 2 + rows * DV * 2));
            __syncwarp();
            if (lane < NSUB) tensor_g2s_3d(st + lane * RR_SUB, &maps.k[sel], lane * 64, 0, it, &fullL[s]);
            else if (lane < 2 * NSUB) tensor_g2s_3d(st + lane * RR_SUB, &maps.v[sel], (lane - NSUB) * 64, 0, it, &fullL[s]);
#pragma unroll
            for (int j = 0; j < RM_MAXN / 32; j++) s_kvst[s * RM_MAXN + lane + 32 * j] = kvr[j];
            if (lane < 16) s_sharpst[s * 16 + lane] = sh;
            if (lane == 0) { s_nv[s] = nv; s_nv[4 + s] = it; }
            __syncwarp();
            if (lane == 0) mbar_arrive(&fullL[s]);
            kd++;
        }
        if (alive) {
            // drain: the stage the terminator goes into (snapshot kd - 2), the terminator, then the last snapshot
            const int s = kd & 1;
            if (kd >= 2) {
                if (__all_sync(FULL, mbar_wait_bounded(&staged[s], (unsigned)(((kd >> 1) & 1) ^ 1)))) store_stage(s, s ? it_s1 : it_s0);
                else alive = false;
            }
            if (alive) {
                if (lane == 0) s_nv[4 + s] = -1;
                __syncwarp();
                if (lane == 0) mbar_arrive(&fullL[s]);
                if (kd >= 1) {
                    const int s1 = s ^ 1;                                  // snapshot kd - 1
                    if (__all_sync(FULL, mbar_wait_bounded(&staged[s1], (unsigned)((((kd - 1) >> 1) & 1))))) store_stage(s1, s1 ? it_s1 : it_s0);
                    else alive = false;
                }
            }
        }
        bulk_wait<0>();                                                    // the stores have been written, not only read
        if (!alive) s_nv[2] = 1;
    } else {
        // ================= the math warps =================
        const int r0 = lane >> 2, cq = (lane & 3) * 2;
        bool failed = false;
        int dirty0 = N, dirty1 = N;                                // rows of stage 0 / 1 below this may hold non-zero data
        for (int kd = 0;; kd++) {
            const int s = kd & 1;
            bool ok = mbar_wait_bounded(&fullL[s], (unsigned)((kd >> 1) & 1));
            int it = -1;
            if (ok) { it = s_nv[4 + s]; if (it >= 0) ok = mbar_wait_bounded(fullQ, (unsigned)(kd & 1)); }
            if (!math_sync_and(ok)) { failed = true; break; }
            it = s_nv[4 + s];
            if (it < 0) break;
            const int nv = s_nv[s];
            const int M = q_count(it);
            const int NPv = (nv + 15) & ~15;
            unsigned char* Kst = rsmb + L.stage + s * L.stage_bytes;
            unsigned char* Vst = Kst + NSUB * RR_SUB;
            const float* s_kv = s_kvst + s * RM_MAXN;
            for (int mm = warp; mm < 16; mm += RR_WARPS) {         // |q| in float32, 2 rows per warp
                float qq = 0.f;
                for (int d = lane; d < DK; d += 32) { const float x = __bfloat162float(Qs[(size_t)mm * L.ldq + d]); qq = fmaf(x, x, qq); }
                qq = warp_sum(qq);
                if (lane == 0) {
                    const float qi = 1.f / fmaxf(sqrtf(qq), 1e-6f);
                    s_qinv[mm] = mm < M ? qi : 0.f;
                    s_scale[mm] = mm < M ? s_sharpst[s * 16 + mm] * qi : 0.f;
                }
            }
            // every fragment of the queries and of the upstream gradient this warp will need, into registers
            unsigned qa[DK / 16][4], oa[DK / 16][4], qb[DT][2], ob[DT][2];
#pragma unroll
            for (int ks = 0; ks < DK / 16; ks++) {
                const size_t off = (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * L.ldq + ks * 16 + (lane >> 4) * 8;
                ldsm_x4(qa[ks], Qs + off);
                ldsm_x4(oa[ks], Os + off);
            }
#pragma unroll
            for (int j = 0; j < DT; j++) {                         // B operands (k = query, n = column) of dK = G^T Q, dV = att^T dO
                const size_t off = (size_t)(lane & 15) * L.ldq + (warp * DT + j) * 8;
                ldsm_x2_trans(qb[j][0], qb[j][1], Qs + off);
                ldsm_x2_trans(ob[j][0], ob[j][1], Os + off);
            }
            float qv[DT][4];                                       // this thread's query elements (rows r0, r0 + 8) for the projection
#pragma unroll
            for (int j = 0; j < DT; j++) {
                const int d = (warp * DT + j) * 8 + cq;
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(Qs + (size_t)r0 * L.ldq + d);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(Qs + (size_t)(r0 + 8) * L.ldq + d);
                qv[j][0] = __low2float(a); qv[j][1] = __high2float(a); qv[j][2] = __low2float(b); qv[j][3] = __high2float(b);
            }
            math_sync();                                           // scales written; nobody needs the query buffer any more
            if (tid == 0) mbar_arrive(emptyQ);
            const float sca = s_scale[r0], scb = s_scale[r0 + 8], qia = s_qinv[r0], qib = s_qinv[r0 + 8];
            // ---- S = Q K^T and dA = dO V^T over this warp's row tiles ----
            float ac[RR_TPW][4], da[RR_TPW][4], sc[RR_TPW][4];
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < RR_TPW; j++) {
                const int nt = warp + j * RR_WARPS;
#pragma unroll
                for (int e = 0; e < 4; e++) { ac[j][e] = 0.f; da[j][e] = 0.f; sc[j][e] = -INFINITY; }
                if (nt * 8 < NPv) {
                    const int row = nt * 8 + (lane & 7);
#pragma unroll
                    for (int ks = 0; ks < DK / 16; ks++) {
                        const int cidx = ks * 2 + ((lane >> 3) & 1);
                        const int off = (cidx >> 3) * RR_SUB + row * 128 + (((cidx & 7) ^ (row & 7)) << 4);
                        unsigned b0, b1;
                        ldsm_x2(b0, b1, Kst + off);
                        mma_bf16(ac[j], qa[ks], b0, b1);
                        ldsm_x2(b0, b1, Vst + off);
                        mma_bf16(da[j], oa[ks], b0, b1);
                    }
                    const float k0 = s_kv[nt * 8 + cq], k1 = s_kv[nt * 8 + cq + 1];
                    sc[j][0] = k0 >= 0.f ? ac[j][0] * k0 * sca : -INFINITY;
                    sc[j][1] = k1 >= 0.f ? ac[j][1] * k1 * sca : -INFINITY;
                    sc[j][2] = k0 >= 0.f ? ac[j][2] * k0 * scb : -INFINITY;
                    sc[j][3] = k1 >= 0.f ? ac[j][3] * k1 * scb : -INFINITY;
                    mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                    mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(FULL, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(FULL, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(FULL, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(FULL, mx1, 2));
            if ((lane & 3) == 0) { s_redA[warp * 16 + r0] = mx0; s_redA[warp * 16 + r0 + 8] = mx1; }
            math_sync();
            mx0 = s_redA[r0]; mx1 = s_redA[r0 + 8];
#pragma unroll
            for (int w = 1; w < RR_WARPS; w++) { mx0 = fmaxf(mx0, s_redA[w * 16 + r0]); mx1 = fmaxf(mx1, s_redA[w * 16 + r0 + 8]); }
            // ---- e = exp(S - max); sum e and sum e dA per query ----
            float su0 = 0.f, su1 = 0.f, sd0 = 0.f, sd1 = 0.f;
#pragma unroll
            for (int j = 0; j < RR_TPW; j++) {
                sc[j][0] = __expf(sc[j][0] - mx0); sc[j][1] = __expf(sc[j][1] - mx0);      // exp(-inf) = 0 for masked rows
                sc[j][2] = __expf(sc[j][2] - mx1); sc[j][3] = __expf(sc[j][3] - mx1);
                su0 += sc[j][0] + sc[j][1]; su1 += sc[j][2] + sc[j][3];
                sd0 += sc[j][0] * da[j][0] + sc[j][1] * da[j][1];
                sd1 += sc[j][2] * da[j][2] + sc[j][3] * da[j][3];
            }
#pragma unroll
            for (int off = 1; off < 4; off <<= 1) {
                su0 += __shfl_xor_sync(FULL, su0, off); su1 += __shfl_xor_sync(FULL, su1, off);
                sd0 += __shfl_xor_sync(FULL, sd0, off); sd1 += __shfl_xor_sync(FULL, sd1, off);
            }
            if ((lane & 3) == 0) {
                s_redB[warp * 16 + r0] = su0; s_redB[warp * 16 + r0 + 8] = su1;
                s_redB[(RR_WARPS + warp) * 16 + r0] = sd0; s_redB[(RR_WARPS + warp) * 16 + r0 + 8] = sd1;
            }
            math_sync();
            su0 = su1 = sd0 = sd1 = 0.f;
#pragma unroll
            for (int w = 0; w < RR_WARPS; w++) {
                su0 += s_redB[w * 16 + r0]; su1 += s_redB[w * 16 + r0 + 8];
                sd0 += s_redB[(RR_WARPS + w) * 16 + r0]; sd1 += s_redB[(RR_WARPS + w) * 16 + r0 + 8];
            }
            const float is0 = 1.f / su0, is1 = 1.f / su1;
            const float sa0 = sd0 * is0, sa1 = sd1 * is1;          // sum_n att dA
            // ---- dl, dsharp, dkinv; att and G as bf16 ----
            float ds0 = 0.f, ds1 = 0.f;
#pragma unroll
            for (int j = 0; j < RR_TPW; j++) {
                const int nt = warp + j * RR_WARPS;
                if (nt * 8 < NPv) {                                // warp-uniform
                    const int n0 = nt * 8 + cq;
                    const float k0 = fmaxf(s_kv[n0], 0.f), k1 = fmaxf(s_kv[n0 + 1], 0.f);   // masked rows: att = 0 anyway
                    const float ma = r0 < M ? is0 : 0.f, mb = r0 + 8 < M ? is1 : 0.f;         // rows beyond a short last block: nothing
                    const float a0 = sc[j][0] * ma, a1 = sc[j][1] * ma, a2 = sc[j][2] * mb, a3 = sc[j][3] * mb;
                    const float l0 = a0 * (da[j][0] - sa0), l1 = a1 * (da[j][1] - sa0);
                    const float l2 = a2 * (da[j][2] - sa1), l3 = a3 * (da[j][3] - sa1);
                    ds0 += (l0 * ac[j][0] * k0 + l1 * ac[j][1] * k1) * qia;               // dl * base, base = (q k) kinv / |q|
                    ds1 += (l2 * ac[j][2] * k0 + l3 * ac[j][3] * k1) * qib;
                    float c0 = l0 * ac[j][0] * sca + l2 * ac[j][2] * scb;                  // dkinv: column sums over the queries
                    float c1 = l1 * ac[j][1] * sca + l3 * ac[j][3] * scb;
#pragma unroll
                    for (int off = 4; off < 32; off <<= 1) { c0 += __shfl_xor_sync(FULL, c0, off); c1 += __shfl_xor_sync(FULL, c1, off); }
                    if (lane < 4) {
                        if (n0 < N) dkinv[(size_t)it * N + n0] = c0;
                        if (n0 + 1 < N) dkinv[(size_t)it * N + n0 + 1] = c1;
                    }
                    *reinterpret_cast<__nv_bfloat162*>(Pb + (size_t)r0 * L.ldp + n0) = __floats2bfloat162_rn(a0, a1);
                    *reinterpret_cast<__nv_bfloat162*>(Pb + (size_t)(r0 + 8) * L.ldp + n0) = __floats2bfloat162_rn(a2, a3);
                    *reinterpret_cast<__nv_bfloat162*>(Gb + (size_t)r0 * L.ldp + n0) = __floats2bfloat162_rn(l0 * k0 * sca, l1 * k1 * sca);
                    *reinterpret_cast<__nv_bfloat162*>(Gb + (size_t)(r0 + 8) * L.ldp + n0) = __floats2bfloat162_rn(l2 * k0 * scb, l3 * k1 * scb);
                }
            }
            ds0 += __shfl_xor_sync(FULL, ds0, 1); ds0 += __shfl_xor_sync(FULL, ds0, 2);
            ds1 += __shfl_xor_sync(FULL, ds1, 1); ds1 += __shfl_xor_sync(FULL, ds1, 2);
            if ((lane & 3) == 0) { s_redA[warp * 16 + r0] = ds0; s_redA[warp * 16 + r0 + 8] = ds1; }   // the maxima are no longer read
            for (int n = NPv + tid; n < N; n += RR_WARPS * 32) dkinv[(size_t)it * N + n] = 0.f;
            math_sync();                                           // att, G and the dsharp partials are written
            if (tid < 16 && tid < M) {
                float t = 0.f;
#pragma unroll
                for (int w = 0; w < RR_WARPS; w++) t += s_redA[w * 16 + tid];
                dsharp[q_index(it, tid)] = t;
            }
            // ---- dq' = G K over this warp's columns ----
            float o[DT][4];
#pragma unroll
            for (int j = 0; j < DT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
#pragma unroll 2
            for (int ks = 0; ks < NPv / 16; ks++) {
                unsigned ga[4];
                ldsm_x4(ga, Gb + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * L.ldp + ks * 16 + (lane >> 4) * 8);
                const int row = ks * 16 + (lane & 15);
#pragma unroll
                for (int j = 0; j < DT; j++) {
                    const int cidx = warp * DT + j;
                    unsigned b0, b1;
                    ldsm_x2_trans(b0, b1, Kst + (cidx >> 3) * RR_SUB + row * 128 + (((cidx & 7) ^ (row & 7)) << 4));
                    mma_bf16(o[j], ga, b0, b1);
                }
            }
            float pr0 = 0.f, pr1 = 0.f;                            // <dq', qn> over this thread's columns
#pragma unroll
            for (int j = 0; j < DT; j++) {
                pr0 += o[j][0] * qv[j][0] + o[j][1] * qv[j][1];
                pr1 += o[j][2] * qv[j][2] + o[j][3] * qv[j][3];
            }
            pr0 *= qia; pr1 *= qib;
            pr0 += __shfl_xor_sync(FULL, pr0, 1); pr0 += __shfl_xor_sync(FULL, pr0, 2);
            pr1 += __shfl_xor_sync(FULL, pr1, 1); pr1 += __shfl_xor_sync(FULL, pr1, 2);
            if ((lane & 3) == 0) { s_redB[warp * 16 + r0] = pr0; s_redB[warp * 16 + r0 + 8] = pr1; }     // the sums are no longer read
            math_sync();                                           // the key tile is free: dK can be staged in its place
            pr0 = pr1 = 0.f;
#pragma unroll
            for (int w = 0; w < RR_WARPS; w++) { pr0 += s_redB[w * 16 + r0]; pr1 += s_redB[w * 16 + r0 + 8]; }
            {
                const bool cl0 = qia >= 1e6f, cl1 = qib >= 1e6f;   // |q| under the clamp: no projection
                const size_t qi0 = q_index(it, r0), qi1 = q_index(it, r0 + 8);
#pragma unroll
                for (int j = 0; j < DT; j++) {
                    const int d = (warp * DT + j) * 8 + cq;
                    if (r0 < M) {
                        const float x = cl0 ? o[j][0] : o[j][0] - qv[j][0] * qia * pr0, y = cl0 ? o[j][1] : o[j][1] - qv[j][1] * qia * pr0;
                        *reinterpret_cast<__nv_bfloat162*>(dqr + qi0 * DK + d) = __floats2bfloat162_rn(x, y);
                    }
                    if (r0 + 8 < M) {
                        const float x = cl1 ? o[j][2] : o[j][2] - qv[j][2] * qib * pr1, y = cl1 ? o[j][3] : o[j][3] - qv[j][3] * qib * pr1;
                        *reinterpret_cast<__nv_bfloat162*>(dqr + qi1 * DK + d) = __floats2bfloat162_rn(x, y);
                    }
                }
            }
            // ---- dK = G^T Q and dV = att^T dO, 16 rows at a time, as bf16 into the tiles their K / V came in ----
            for (int n16 = 0; n16 < NPv / 16; n16++) {
                unsigned ga[4], pa[4];
                const size_t aoff = (size_t)((lane & 7) + ((lane >> 4) & 1) * 8) * L.ldp + n16 * 16 + ((lane >> 3) & 1) * 8;
                ldsm_x4_trans(ga, Gb + aoff);
                ldsm_x4_trans(pa, Pb + aoff);
#pragma unroll
                for (int j = 0; j < DT; j++) {
                    float ck[4] = {0.f, 0.f, 0.f, 0.f}, cv[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_bf16(ck, ga, qb[j][0], qb[j][1]);
                    mma_bf16(cv, pa, ob[j][0], ob[j][1]);
                    const int cidx = warp * DT + j;
                    const int ra = n16 * 16 + r0, rb = ra + 8;
                    const int offa = (cidx >> 3) * RR_SUB + ra * 128 + (((cidx & 7) ^ (ra & 7)) << 4) + cq * 2;
                    const int offb = (cidx >> 3) * RR_SUB + rb * 128 + (((cidx & 7) ^ (rb & 7)) << 4) + cq * 2;
                    *reinterpret_cast<__nv_bfloat162*>(Kst + offa) = __floats2bfloat162_rn(ck[0], ck[1]);
                    *reinterpret_cast<__nv_bfloat162*>(Kst + offb) = __floats2bfloat162_rn(ck[2], ck[3]);
                    *reinterpret_cast<__nv_bfloat162*>(Vst + offa) = __floats2bfloat162_rn(cv[0], cv[1]);
                    *reinterpret_cast<__nv_bfloat162*>(Vst + offb) = __floats2bfloat162_rn(cv[2], cv[3]);
                }
            }
            // Rows above the visited ones leave as zeros (the stores cover whole snapshots).  Only rows that can hold
            // something else are rewritten: what this snapshot's box brought in, or the previous gradients of this stage.
            const int hb = nv <= h64 ? h64 : (nv <= h128 ? h128 : N);
            const int dirty = max(hb, s ? dirty1 : dirty0);
            if (s) dirty1 = NPv; else dirty0 = NPv;
            for (int i = tid; i < (dirty - NPv) * 8 * NSUB; i += RR_WARPS * 32) {
                const int row = NPv + i / (8 * NSUB), c = i % (8 * NSUB);
                const int off = (c >> 3) * RR_SUB + row * 128 + ((c & 7) << 4);
                *reinterpret_cast<uint4*>(Kst + off) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(Vst + off) = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();                              // the bulk stores read these tiles through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&staged[s]);
        }
        if (failed) s_nv[2] = 1;
    }
    __syncthreads();
    if (s_nv[2] != 0) {
        if (tid == 0) atomicExch(&g_read_status, 1);
        for (int k = 0; k < 1000; k++) __nanosleep(1000);
    }
}

// false when the kernel does not apply (shape, alignment, or no tensor-map support in the driver)
template <int DK>
static bool launch_bwd_ring(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf, const void* vbuf,
                            const float* kinv, const uint8_t* valid, const void* drd, void* dqr, float* dsharp, void* dkbuf,
                            void* dvbuf, float* dkinv, cudaStream_t st, cudaError_t* err) {
    const int NB = (p.T + p.G - 1) / p.G;
    const long long nsnap = (long long)p.B * NB * p.H;
    if (p.N % 16 || p.G * p.NQ > 16 || nsnap > 2147483647LL || (((uintptr_t)kinv | (uintptr_t)valid) & 15)) return false;
    ReadBwdMaps maps;
    const int hs[3] = {p.N < 64 ? p.N : 64, p.N < 128 ? p.N : 128, p.N};
    for (int i = 0; i < 3; i++)
        if (!snapshot_map(&maps.k[i], kbuf, nsnap, p.N, DK, hs[i]) || !snapshot_map(&maps.v[i], vbuf, nsnap, p.N, DK, hs[i])) return false;
    if (!snapshot_map(&maps.dk, dkbuf, nsnap, p.N, DK, p.N) || !snapshot_map(&maps.dv, dvbuf, nsnap, p.N, DK, p.N)) return false;
    const size_t sm = (size_t)read_bwd_ring_layout(DK).total + 1024;
    auto kern = read_bwd_ring_kernel<DK>;
    if ((*err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)) != cudaSuccess) return true;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)(nsnap < sms ? nsnap : sms);
    kern<<<grid, RR_THREADS, sm, st>>>(p, maps, (const bf16*)qr, sharp, kinv, valid, (const bf16*)drd, (bf16*)dqr, dsharp, dkinv,
                                       (int)nsnap);
    *err = cudaGetLastError();
    return true;
}

template <int DK, int DV>
static cudaError_t launch_mma(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf,
                              const void* vbuf, const float* kinv, const uint8_t* valid, void* rd, cudaStream_t st) {
    const int NB = (p.T + p.G - 1) / p.G;
    const size_t sm = (size_t)read_mma_layout(p.N, DK, DV).total;
    auto kern = read_fwd_mma_kernel<DK, DV>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return e;
    kern<<<p.B * NB * p.H, RM_THREADS, sm, st>>>(p, (const bf16*)qr, sharp, (const bf16*)kbuf, (const bf16*)vbuf, kinv, valid,
                                                  (bf16*)rd);
    return cudaGetLastError();
}

// true (and *err set) when this kernel takes the call: bf16 queries and snapshots, dk = dv in {64, 128}, N <= 192,
// 16-byte aligned rows
bool read_fwd_mma_try(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf, const void* vbuf,
                      const float* kinv, const uint8_t* valid, void* rd, cudaStream_t st, cudaError_t* err) {
    if (p.q_dtype != SLOTSCAN_BF16 || p.snap_dtype != SLOTSCAN_BF16 || p.N > RM_MAXN || p.DK != p.DV) return false;
    if (((uintptr_t)qr | (uintptr_t)kbuf | (uintptr_t)vbuf | (uintptr_t)rd) & 15) return false;
    if (p.DK == 128) {
        if (!launch_ring<128>(p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st, err))
            *err = launch_mma<128, 128>(p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    } else if (p.DK == 64) {
        if (!launch_ring<64>(p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st, err))
            *err = launch_mma<64, 64>(p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    } else {
        return false;
    }
    return true;
}

// true (and *err set) when the tensor-core backward takes the snapshots with more than RB_SPARSE_ROWS rows in use; the
// caller then runs the CUDA-core kernel for the others
bool read_bwd_mma_try(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf, const void* vbuf,
                      const float* kinv, const uint8_t* valid, const void* drd, void* dqr, float* dsharp, void* dkbuf,
                      void* dvbuf, float* dkinv, cudaStream_t st, cudaError_t* err) {
    if (p.q_dtype != SLOTSCAN_BF16 || p.snap_dtype != SLOTSCAN_BF16 || p.N > RM_MAXN || p.DK != p.DV) return false;
    if (((uintptr_t)qr | (uintptr_t)kbuf | (uintptr_t)vbuf | (uintptr_t)drd | (uintptr_t)dqr | (uintptr_t)dkbuf | (uintptr_t)dvbuf) & 15)
        return false;
    if (p.DK == 128) return launch_bwd_ring<128>(p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, st, err);
    if (p.DK == 64) return launch_bwd_ring<64>(p, qr, sharp, kbuf, vbuf, kinv, valid, drd, dqr, dsharp, dkbuf, dvbuf, dkinv, st, err);
    return false;
}

int read_mma_status() {
    int v = 0, z = 0;
    if (cudaMemcpyFromSymbol(&v, g_read_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_read_status, &z, sizeof(int));
    return v;
}

}  // namespace slotscan
