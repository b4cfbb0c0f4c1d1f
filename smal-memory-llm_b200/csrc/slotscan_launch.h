// Internal launch interface between the translation units of libslotscan.so (not part of the C ABI).
// The kernels are templates over key width, live row slots and dtypes; each .cu instantiates one family so the
// library builds in parallel.
#pragma once
#include <cuda_runtime.h>
#include <stdio.h>

#include "slotscan.h"

namespace slotscan {

// rows a first-pass CTA of the address kernels holds in shared memory (sequences that need more rerun at full size)
constexpr int AF_NCAP1 = 64;

template <typename F>
static inline cudaError_t opt_in_smem(F f, size_t bytes) {
    return cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

// in_dtype / snap_dtype of p select the instantiation
// initial state of the address scan (all NULL: the empty memory) and where its carried squared key norms go
struct AddrFwdState { const float* K0; const float* o0; const double* nsq0; double* nsqfin; };
cudaError_t run_addr_fwd_f32(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                             const float* temp, const slotscan_log& L, const AddrFwdState& S0, cudaStream_t st);
cudaError_t run_addr_fwd_bf16(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                              const float* temp, const slotscan_log& L, const AddrFwdState& S0, cudaStream_t st);
// vend_ready: the next-write table (run_next_write) has been filled already, on a stream this one is ordered after
cudaError_t run_addr_bwd_f32(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                             const float* temp, const slotscan_log& L, const float* Dn, void* dq, float* dgate, float* dfr,
                             float* part, int* vend, int part_stride, bool vend_ready, cudaStream_t st);
cudaError_t run_addr_bwd_bf16(const slotscan_params& p, const void* q, const void* k, const float* gate, const float* fr,
                              const float* temp, const slotscan_log& L, const float* Dn, void* dq, float* dgate, float* dfr,
                              float* part, int* vend, int part_stride, bool vend_ready, cudaStream_t st);
// the next-write table of the token-parallel address backward: it depends on the forward's log only, so it can run
// beside the reverse row scan; true when the address backward of this shape uses it
bool next_write_used(const slotscan_params& p);
cudaError_t run_next_write(const slotscan_params& p, const slotscan_log& L, int* vend, cudaStream_t st);
// tokens per CTA of the token-parallel address backward: the partial-sum table has one slot per such chunk (+ 1)
constexpr int GATHER_CHUNK = 32;
constexpr int GATHER_ROWS_MAX = 32;
// One tensor (keys: D = DK, values: D = DV) of the forward row replay.  x0: the rows the replay starts from (NULL =
// zeros); xold NULL: no undo log; kinv / valid: per emitted row, from the float32 state (keys only, or NULL);
// zero_from: rows >= zero_from were zero-filled ahead by run_zero_rows (N = none).
struct ReplayPtrs { const void* x; const float* x0; void* xbuf; float* xold; float* xfin; float* kinv; uint8_t* valid; int zero_from; };
// ntensors = 2 runs keys and values in one launch (needs DK == DV), 1 runs r0 only
// row tiles [tile_lo, tile_hi) of replay_tile_rows(D) rows each; tile_hi < 0: up to the last one
cudaError_t run_replay(const slotscan_params& p, int D, int ntensors, const ReplayPtrs& r0, const ReplayPtrs& r1,
                       const float* gate, const int* am, const int* tfirst, int tile_lo, int tile_hi, cudaStream_t st);
int replay_tile_rows(int D);
int replay_status();
// zero-fill of rows [zk, N) of every key snapshot (+ kinv = 1e6, valid = 0 when given) and [zv, N) of every value snapshot
cudaError_t run_zero_rows(const slotscan_params& p, void* kbuf, int zk, void* vbuf, int zv, float* kinv, uint8_t* valid,
                          cudaStream_t st);
// reverse row scan; ntensors = 2 runs keys and values in one launch (needs DK == DV), 1 runs the first set only
// dkinv: upstream gradient of the kinv output (keys only, NULL otherwise)
struct RowsBwdPtrs { const void* x; const float* xold; const float* xfin; const void* dxbuf; void* dx; float* Dn; const float* dkinv; };
cudaError_t run_rows_bwd_f32(const slotscan_params& p, int D, int ntensors, const RowsBwdPtrs& a0, const RowsBwdPtrs& a1,
                             const float* gate, const int* am, const int* tfirst, cudaStream_t st);
cudaError_t run_rows_bwd_bf16(const slotscan_params& p, int D, int ntensors, const RowsBwdPtrs& a0, const RowsBwdPtrs& a1,
                              const float* gate, const int* am, const int* tfirst, cudaStream_t st);
static inline cudaError_t run_rows_bwd(const slotscan_params& p, int D, int ntensors, const RowsBwdPtrs& a0,
                                       const RowsBwdPtrs& a1, const float* gate, const int* am, const int* tfirst,
                                       cudaStream_t st) {
    return p.in_dtype == SLOTSCAN_F32 ? run_rows_bwd_f32(p, D, ntensors, a0, a1, gate, am, tfirst, st)
                                      : run_rows_bwd_bf16(p, D, ntensors, a0, a1, gate, am, tfirst, st);
}
// rows (highest valid row + 1) up to which a snapshot is read by the CUDA-core kernel even when the tensor-core one runs
constexpr int RM_SPARSE_ROWS = 32;
// The backward writes whole snapshots of gradients (zeros included), so it is bound by those writes whatever the row
// count: every snapshot with at least one valid row takes the tensor-core kernel, the empty ones the CUDA-core kernel.
constexpr int RB_SPARSE_ROWS = 0;
// tensor-core forward read (slotscan_read_mma.cu): returns false when the shape / dtypes are not its own
bool read_fwd_mma_try(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf, const void* vbuf,
                      const float* kinv, const uint8_t* valid, void* rd, cudaStream_t st, cudaError_t* err);
bool read_bwd_mma_try(const slotscan_read_params& p, const void* qr, const float* sharp, const void* kbuf, const void* vbuf,
                      const float* kinv, const uint8_t* valid, const void* drd, void* dqr, float* dsharp, void* dkbuf,
                      void* dvbuf, float* dkinv, cudaStream_t st, cudaError_t* err);
int read_mma_status();
int gather_status_f32();
int gather_status_bf16();
int rows_bwd_status_f32();
int rows_bwd_status_bf16();

size_t addr_fwd_smem_bytes(int ncap, int DK, int in_bytes);
size_t addr_bwd_smem_bytes(int ncap, int DK);
void attrs_addr_fwd_f32(slotscan_kernel_attr* out, int cap, int& n);
void attrs_addr_fwd_bf16(slotscan_kernel_attr* out, int cap, int& n);
void attrs_addr_bwd_f32(slotscan_kernel_attr* out, int cap, int& n);
void attrs_addr_bwd_bf16(slotscan_kernel_attr* out, int cap, int& n);
void attrs_rows(slotscan_kernel_attr* out, int cap, int& n);
void attrs_rows_bwd_f32(slotscan_kernel_attr* out, int cap, int& n);
void attrs_rows_bwd_bf16(slotscan_kernel_attr* out, int cap, int& n);

template <typename F>
static inline void fill_attr(slotscan_kernel_attr* out, int cap, int& n, const char* name, F f) {
    if (n < cap) {
        cudaFuncAttributes a;
        if (cudaFuncGetAttributes(&a, f) == cudaSuccess) {
            snprintf(out[n].name, sizeof(out[n].name), "%s", name);
            out[n].regs = a.numRegs;
            out[n].local_bytes = (int)a.localSizeBytes;
            out[n].static_smem = (int)a.sharedSizeBytes;
            out[n].max_threads = a.maxThreadsPerBlock;
        }
    }
    n++;
}

#define SLOTSCAN_DISPATCH_D(D_, CALL)                          \
    switch (D_) {                                              \
        case 8: { constexpr int DD = 8; CALL; } break;         \
        case 16: { constexpr int DD = 16; CALL; } break;       \
        case 32: { constexpr int DD = 32; CALL; } break;       \
        case 64: { constexpr int DD = 64; CALL; } break;       \
        case 128: { constexpr int DD = 128; CALL; } break;     \
        default: return cudaErrorInvalidValue;                 \
    }

}  // namespace slotscan
