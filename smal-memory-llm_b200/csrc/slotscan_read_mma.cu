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
    if (p.DK == 128) *err = launch_mma<128, 128>(p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    else if (p.DK == 64) *err = launch_mma<64, 64>(p, qr, sharp, kbuf, vbuf, kinv, valid, rd, st);
    else return false;
    return true;
}

int read_mma_status() {
    int v = 0, z = 0;
    if (cudaMemcpyFromSymbol(&v, g_read_status, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) cudaMemcpyToSymbol(g_read_status, &z, sizeof(int));
    return v;
}

}  // namespace slotscan
