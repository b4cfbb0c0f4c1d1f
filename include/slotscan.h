/* slotscan.h -- C ABI of libslotscan.so: the slot-scan hot path as hand-written CUDA for sm_100a.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless said otherwise, every call is
 * asynchronous on `stream` (a cudaStream_t passed as void*), allocates nothing and returns a status:
 *      0   ok
 *     <0   the arguments were rejected before any launch (SLOTSCAN_E_*)
 *     >0   a cudaError_t from a launch
 * The functions replace, one for one, the host side of the reference's runtime-compiled kernels
 * (gqa25/slotkern_cuda.py: _KVScanC.forward :484-511, _KVScanC.backward :514-533, kernel_attrs :467-479) and the
 * torch ops around them in gqa25/memlm_sh.py (:362-397 read, :464-475 writer epilogue, :221-234 quantiser).
 *
 * Layouts (all contiguous, identical to the reference):
 *   token streams   k, q (B,T,H,DK)   v (B,T,H,DV)   gate, fr (B,T,H)        token index ix = (b*T + t)*H + h
 *   snapshots       kbuf (B,NB,H,N,DK)  vbuf (B,NB,H,N,DV),  NB = ceil(T/G): the PRE-write state at t = 0, G, 2G, ...
 *   per-sequence    (B*H, N, D) finals, (B*H, N) occupancy
 */
#ifndef SLOTSCAN_H
#define SLOTSCAN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLOTSCAN_ABI_VERSION 2

enum { SLOTSCAN_F32 = 0, SLOTSCAN_BF16 = 1 };

enum {
    SLOTSCAN_OK = 0,
    SLOTSCAN_E_NULL = -1,       /* a required pointer is NULL */
    SLOTSCAN_E_SHAPE = -2,      /* a size is out of the supported range (see slotscan_check) */
    SLOTSCAN_E_DTYPE = -3,      /* unknown dtype code */
    SLOTSCAN_E_ALIGN = -4,      /* a pointer is not 16-byte aligned */
    SLOTSCAN_E_MODE = -5,       /* a mode this entry point does not implement */
    SLOTSCAN_E_TOO_LARGE = -6   /* beyond the fixed capacity of a no-allocation entry point */
};

/* Shape and mode of one scan call.  Mirrors the arguments of the reference's kv_scan_c
 * (gqa25/slotkern_cuda.py:536): N, G, hard_gate, eps, occ_bin; fr_per_token = (fr.dim() == 3) (:491). */
typedef struct {
    int32_t B, T, H, N, DK, DV, G;
    int32_t hard_gate;      /* forward uses [gate > 0.5]; gradient passes straight through */
    int32_t occ_bin;        /* free-row penalty on [o >= eps] instead of on o */
    int32_t fr_per_token;   /* fr is (B,T,H); otherwise one element */
    int32_t in_dtype;       /* SLOTSCAN_F32 / SLOTSCAN_BF16: k, q, v and their gradients */
    int32_t snap_dtype;     /* SLOTSCAN_F32 / SLOTSCAN_BF16: kbuf, vbuf, dkbuf, dvbuf */
    float eps;              /* occupancy threshold, 1e-4 in the reference */
} slotscan_params;

/* Argument check shared by every entry point: 0 or a SLOTSCAN_E_* code.  Supported: B,T,H,N,G >= 1;
 * DK, DV in {8,16,32,64,128}; N <= 192 (the key rows of one sequence, N*(DK+4) floats, stay resident in one CTA's shared memory). */
int slotscan_check(const slotscan_params* p);

/* Log of one forward call: what the backward (and a caller that streams chunks) needs.  All caller-allocated.
 *   addr   (B,T,H) int32   the row each token wrote                 [reference: `am`, slotkern_cuda.py:502]
 *   oold   (B,T,H) f32     that row's occupancy before the write    [`oold` :503]
 *   kiold  (B,T,H) f32     1 / max(|key row|, 1e-6) of that row before the write
 *   kold   (B,T,H,DK) f32, vold (B,T,H,DV) f32   the row before the write   [`kold`, `vold` :503]
 *   kfin   (B*H,N,DK) f32, vfin (B*H,N,DV) f32, ofin (B*H,N) f32    state after the last token  [:504]
 *   tfirst (B*H,N) int32   first token at which row n could be addressed (T if never): rows are taken in index
 *                          order, so everything above the highest row touched so far is exactly zero and is skipped. */
typedef struct {
    int32_t* addr;
    float* oold;
    float* kold;
    float* vold;
    float* kfin;
    float* vfin;
    float* ofin;
    int32_t* tfirst;
    float* kiold;
} slotscan_log;

/* Forward: hard (argmax) address, address reads the stored keys as constants.
 * Replaces _KVScanC.forward (gqa25/slotkern_cuda.py:484-511: addr_fwd :72-174 + val_fwd :178-206).
 * q may be NULL (search with k).  temp: 1 float on the device (exp(log_wsharp), memlm_sh.py:439).
 * Writes kbuf, vbuf (snap_dtype) and the log. */
int slotscan_hard_fwd(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                      const float* fr, const float* temp, void* kbuf, void* vbuf, const slotscan_log* log,
                      void* stream);

/* Extras of a forward call; every pointer may be NULL (a NULL `ex` is slotscan_hard_fwd).
 * [The reference carries no state across calls (gqa25/memlm_sh.py:676 asserts it) and forms kinv / valid in a separate
 * eager pass over the emitted keys (memlm_sh.py:474-475); its kernels hold the final state internally
 * (slotkern_cuda.py:504).]
 *   K0, V0, o0   (B*H,N,DK) (B*H,N,DV) (B*H,N) f32: the state the scan starts from -- kfin, vfin, ofin of the call that
 *                scanned the preceding tokens.  All three or none (none = the empty memory).  Snapshot 0 is then this
 *                state.  A long context is streamed chunk by chunk this way with memory constant in T.
 *   nsq0         (B*H,N) f64: squared key norms carried with the state (nsqfin of the preceding call).  NULL: they are
 *                summed again from K0, which may move a score by one float32 ulp against the unchunked scan.
 *   nsqfin       (B*H,N) f64 out: squared key norms of the final state as the scan carried them.
 *   kinv, valid  (B,NB,H,N) f32 / bytes out, both or neither: rsqrt(max(|K_n|^2, 1e-12)) and [|K_n|^2 > 1e-12] of every
 *                emitted key row, taken from the float32 state while the row is in registers (what memlm_sh.py:474-475
 *                computes from the float32 kbuf before casting it): no separate pass over the snapshots.
 *   no_undo_log  non-zero: the rows before each write (log->kold, log->vold, which may then be NULL) are not stored.
 *                For forward-only callers; the backward needs them.
 * The backward of a call that was given K0 / V0 / o0 produces no gradient for that carried-in state. */
typedef struct {
    const float* K0;
    const float* V0;
    const float* o0;
    const double* nsq0;
    double* nsqfin;
    float* kinv;
    uint8_t* valid;
    int32_t no_undo_log;
} slotscan_fwd_extra;
int slotscan_hard_fwd_ex(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                         const float* fr, const float* temp, void* kbuf, void* vbuf, const slotscan_log* log,
                         const slotscan_fwd_extra* ex, void* stream);

/* Bytes of scratch the backward needs (the per-token, per-row table D[t,n] plus per-sequence partial sums). */
size_t slotscan_hard_bwd_scratch_bytes(const slotscan_params* p);

/* Backward of slotscan_hard_fwd for upstream gradients dkbuf, dvbuf (snap_dtype; either may be NULL = zeros).
 * Replaces _KVScanC.backward (gqa25/slotkern_cuda.py:514-533: rows_bwd :209-261 + addr_bwd :264-443).
 * Outputs: dk, dv, dq (in_dtype; dq is always required: with q NULL it receives the search-path part, which is
 * then also added into dk),
 * dgate (B,T,H) f32, dfr (B,T,H) f32 or 1 float, dtemp 1 float.  The scalar sums are reduced in a fixed order:
 * results are bitwise repeatable (the reference uses float atomics, slotkern_cuda.py:440-441). */
int slotscan_hard_bwd(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                      const float* fr, const float* temp, const slotscan_log* log, const void* dkbuf,
                      const void* dvbuf, void* scratch, size_t scratch_bytes, void* dk, void* dq, void* dv,
                      float* dgate, float* dfr, float* dtemp, void* stream);

/* slotscan_hard_bwd with one more upstream gradient: dkinv (B,NB,H,N) f32, the gradient that reached the kinv output
 * of slotscan_hard_fwd_ex (NULL = none).  It enters the key rows where the snapshot was taken,
 * d kbuf[j,n] += -kinv^3 * dkinv[j,n] * K_n for valid rows, with K_n the float32 state -- the adjoint of
 * rsqrt(clamp_min(nsq, 1e-12)) that the reference gets from autograd (memlm_sh.py:474-475). */
int slotscan_hard_bwd_ex(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                         const float* fr, const float* temp, const slotscan_log* log, const void* dkbuf,
                         const void* dvbuf, const float* dkinv, void* scratch, size_t scratch_bytes, void* dk, void* dq,
                         void* dv, float* dgate, float* dfr, float* dtemp, void* stream);

/* The same backward for callers that cannot supply scratch memory.  [No counterpart in the reference: its host side
 * always allocates through torch.]  Meant for hosts whose device memory is already fully assigned (a server that
 * handed everything to its own arena, a binding with no device allocator) or that must not make a synchronising
 * allocation on this path.  The table D[t,n] and the partial sums live in ONE fixed array of
 * SLOTSCAN_NOALLOC_SCRATCH_BYTES inside the library (each GPU that loads the library holds that much until the process
 * exits).  Arguments and results are those of slotscan_hard_bwd without `scratch`; results are bit-identical to it.
 *   - Limit: slotscan_hard_bwd_scratch_bytes(p) must not exceed the capacity, i.e. roughly B*H*T*N <= 1 M table
 *     entries; beyond that the call returns SLOTSCAN_E_TOO_LARGE and launches nothing.
 *   - The call itself allocates no device memory and frees none.
 *   - On EVERY call the current device (cudaGetDevice) must be the one that owns `stream` and all the pointers: the
 *     array used is the current device's copy.  Inputs found on another device are refused with SLOTSCAN_E_MODE.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress, with that device
 *     current); make that first call outside any stream capture.
 *   - Every call on a device shares the one array, which still holds the previous call's table: nothing in it needs
 *     clearing, but two calls whose kernels overlap on the GPU (different streams, or threads) would overwrite each
 *     other's table.  Keep calls to this entry point ordered on one stream per device. */
#define SLOTSCAN_NOALLOC_SCRATCH_BYTES (8u << 20)
size_t slotscan_hard_bwd_noalloc_capacity(void);
int slotscan_hard_bwd_noalloc(const slotscan_params* p, const void* k, const void* q, const void* v, const float* gate,
                              const float* fr, const float* temp, const slotscan_log* log, const void* dkbuf,
                              const void* dvbuf, void* dk, void* dq, void* dv, float* dgate, float* dfr, float* dtemp,
                              void* stream);

/* The general scan: every mode of kv_scan_g (gqa25/slotkern_kvg.py:257) -- soft or hard address, address gradient
 * attached to the stored keys or detached, hard gate, either occupancy penalty, scalar or per-token fr, q or NULL.
 * [replaces the Triton kernels _kvfwd (gqa25/slotkern_kvt.py:43-119) and _kvbwd_g (gqa25/slotkern_kvg.py:41-205), which
 * the reference falls back to for everything but its hard + detached training mode (slotkern_cuda.py:540-542).]
 * The hard + detached mode has its own, much faster kernels (slotscan_hard_*); this entry point exists so that no
 * argument combination of the reference call is without a CUDA implementation.  One CTA per (sequence, head).
 *   base.snap_dtype must be SLOTSCAN_F32: kbuf, vbuf and obuf (B,NB,H,N) are float32 -- they are the checkpoints the
 *   backward replays from.  Any 1 <= DK, DV <= 128; N * (DK + DV + 8) floats must fit one CTA's shared memory
 *   (N <= 192 at 128 + 128).
 * slotscan_dense_fwd: addr (B,T,H) int32 = argmax of each token's address, kfin / vfin / ofin = the final state; each
 * of the four may be NULL.
 * slotscan_dense_bwd: needs the forward's kbuf, vbuf, obuf and scratch of slotscan_dense_bwd_scratch_bytes (G states
 * per (sequence, head)); dkbuf / dvbuf float32, either may be NULL.  Outputs as slotscan_hard_bwd. */
typedef struct {
    slotscan_params base;
    int32_t hard;           /* forward address: 1 = one-hot argmax, 0 = the softmax over the candidate rows */
    int32_t detach_addr;    /* 1 = the address reads the stored keys as constants: no gradient into them from the match */
} slotscan_dense_params;
int slotscan_dense_check(const slotscan_dense_params* p);
int slotscan_dense_fwd(const slotscan_dense_params* p, const void* k, const void* q, const void* v, const float* gate,
                       const float* fr, const float* temp, float* kbuf, float* vbuf, float* obuf, int32_t* addr,
                       float* kfin, float* vfin, float* ofin, void* stream);
size_t slotscan_dense_bwd_scratch_bytes(const slotscan_dense_params* p);
int slotscan_dense_bwd(const slotscan_dense_params* p, const void* k, const void* q, const void* v, const float* gate,
                       const float* fr, const float* temp, const float* kbuf, const float* vbuf, const float* obuf,
                       const float* dkbuf, const float* dvbuf, void* scratch, size_t scratch_bytes, void* dk, void* dq,
                       void* dv, float* dgate, float* dfr, float* dtemp, void* stream);

/* The keyless scan: address logits given from outside, value-only state.
 * [replaces the Triton kernels of gqa25/slotkern_v.py (_vfwd :25, _vrecompute :75, _vadjoint :120; entry slot_scan_v :232;
 * definition ref_scan_v :242-261).]  z = wa_t - fr o over all N rows, softmax or argmax (hard, straight-through), gate or
 * [gate > 0.5] (hard_gate, straight-through), V <- (1 - w) V + w v_t, o <- (1 - w) o + w.
 *   v (B,T,H,DV) in_dtype, wa (B,T,H,N) f32, gate (B,T,H) f32, fr 1 float (device)
 *   buf (B,NB,H,N,DV) f32: the pre-write values at t = 0, G, 2G, ...; obuf (B,NB,H,N) f32: the occupancies at the same
 *   times (the backward's checkpoints); addr (B,T,H) int32 or NULL.
 * Backward: dv (in_dtype), dwa (B,T,H,N), dgate (B,T,H), dfr 1 float, from dbuf (f32, or NULL = zeros); scratch of
 * slotscan_v_bwd_scratch_bytes.  N * DV + 10 N floats must fit one CTA's shared memory. */
typedef struct {
    int32_t B, T, H, N, DV, G;
    int32_t hard, hard_gate;
    int32_t in_dtype;       /* SLOTSCAN_F32 / SLOTSCAN_BF16: v and dv */
} slotscan_v_params;
int slotscan_v_check(const slotscan_v_params* p);
int slotscan_v_fwd(const slotscan_v_params* p, const void* v, const float* wa, const float* gate, const float* fr,
                   float* buf, float* obuf, int32_t* addr, void* stream);
size_t slotscan_v_bwd_scratch_bytes(const slotscan_v_params* p);
int slotscan_v_bwd(const slotscan_v_params* p, const void* v, const float* wa, const float* gate, const float* fr,
                   const float* buf, const float* obuf, const float* dbuf, void* scratch, size_t scratch_bytes, void* dv,
                   float* dwa, float* dgate, float* dfr, void* stream);

/* Writer epilogue and storage quantiser over emitted snapshot rows, one streaming pass.
 * [replaces memlm_sh.py:464-475 (nsq = sum kbuf^2 in fp32, kinv = rsqrt(max(nsq, 1e-12)), valid = nsq > 1e-12, cast of
 * the snapshots to the model dtype) and memlm_sh.py:221-234 (_fq, _quantize_mem).]
 *   x      rows x D elements (in_dtype): kbuf or vbuf as the scan emitted them, any leading shape flattened
 *   y      rows x D elements (out_dtype), or NULL when only kinv / valid are wanted
 *   kinv   rows fp32 and valid rows bytes (0 / 1): both or neither (NULL, NULL for value rows)
 *   bits   0: y = x.  2, 3, 4 or 8 (memlm_sh.py:81): y = _fq(x, bits, group), the midrise quantiser with one
 *          absmax scale per `group` channels, evaluated in the reference's arithmetic including its straight-through
 *          form x + (q - x); an all-zero group stays exactly zero.  group: a power of two, 4 <= group <= D.
 *          SLOTSCAN_BITS_E4M3 (-8): fp8-e4m3 storage with one scale per ROW, s = max(absmax / 448, 1e-30),
 *          y = e4m3(x / s) * s (round to nearest even, saturating), `group` ignored; an all-zero row stays zero.  The
 *          reference has no fp8 format (only a remark on storing the scale in fp8, memlm_sh.py:217-218): this mode
 *          follows a restatement, not reference code.
 *   kinv and valid are taken from the quantised row before the cast, as _quantize_mem does (:232-234).
 * Forward values only (the reference's gradient is the identity through _fq). */
#define SLOTSCAN_BITS_E4M3 (-8)
typedef struct {
    int64_t rows;
    int32_t D;              /* 8, 16, 32, 64 or 128 */
    int32_t in_dtype, out_dtype;
    int32_t bits, group;
} slotscan_epilogue_params;
int slotscan_epilogue_check(const slotscan_epilogue_params* p);
int slotscan_writer_epilogue(const slotscan_epilogue_params* p, const void* x, void* y, float* kinv, uint8_t* valid,
                             void* stream);

/* Cosine read of the stride-G snapshots, forward.  [replaces the core of SharedMixer._read, gqa25/memlm_sh.py:379-397:
 * fp32 L2-normalisation of the queries with clamp 1e-6 (:379), logits = (q . kbuf^T) * kinv * sharpness (:383-393),
 * masked softmax over the valid rows with an all-invalid snapshot reading exactly zero (:394), rd = att . buf (:395).]
 *   qr     (B, T, H, NQ, DK)  read queries as projected by the caller (q_dtype); normalised inside
 *   sharp  (B, T, H, NQ) fp32: the product exp(log_rsel) * exp(C tanh(read_s / C)) the caller forms (:383-393)
 *   kbuf   (B, NB, H, N, DK), vbuf (B, NB, H, N, DV)  snapshots (snap_dtype), NB = ceil(T / G)
 *   kinv   (B, NB, H, N) fp32, valid (B, NB, H, N) bytes: from slotscan_writer_epilogue
 *   rd     (B, T, H, NQ, DV) (q_dtype): token t reads snapshot t / G only
 * Any DK, DV <= 128, N <= 2048.
 * slotscan_read_bwd is the adjoint for an upstream gradient drd (shape and dtype of rd): dqr (like qr), dsharp (like
 * sharp), dkbuf / dvbuf (like kbuf / vbuf, exact zeros in the rows that are not valid) and dkinv (B, NB, H, N) fp32, the
 * gradient of the kinv INPUT (the writer epilogue differentiates kinv = rsqrt(nsq) itself; the reference gets the
 * same total from autograd).  Its shared-memory tables hold (G * NQ) x N entries: SLOTSCAN_E_TOO_LARGE beyond 200 KB. */
typedef struct {
    int32_t B, T, H, NQ, N, DK, DV, G;
    int32_t q_dtype, snap_dtype;
} slotscan_read_params;
int slotscan_read_check(const slotscan_read_params* p);
int slotscan_read_fwd(const slotscan_read_params* p, const void* qr, const float* sharp, const void* kbuf,
                      const void* vbuf, const float* kinv, const uint8_t* valid, void* rd, void* stream);
int slotscan_read_bwd(const slotscan_read_params* p, const void* qr, const float* sharp, const void* kbuf,
                      const void* vbuf, const float* kinv, const uint8_t* valid, const void* drd, void* dqr,
                      float* dsharp, void* dkbuf, void* dvbuf, float* dkinv, void* stream);

/* Registers / spilled bytes / static shared memory / max threads of each kernel, the analogue of kernel_attrs
 * (gqa25/slotkern_cuda.py:467-479).  Fills up to `cap` entries (HOST memory), returns how many kernels exist. */
typedef struct {
    char name[48];
    int32_t regs, local_bytes, static_smem, max_threads;
} slotscan_kernel_attr;
int slotscan_query_attrs(slotscan_kernel_attr* out, int cap);

/* Per-kernel device timing for benchmarks: while enabled, every launch made by this library is bracketed by CUDA
 * events on the stream it is launched on.  slotscan_profile_read waits for those events, fills per kernel the number
 * of launches and the summed device time since the last read (HOST memory, up to `cap` entries), clears the record
 * and returns the number of kernels.  The reference measures the same way from Python (kvu/prof_cuda.py:9-20). */
typedef struct {
    char name[48];
    int32_t launches;
    float total_ms;
} slotscan_kernel_time;
int slotscan_profile_enable(int on);
int slotscan_profile_read(slotscan_kernel_time* out, int cap);

/* Kernels of this library never wait without a limit: a wait on an asynchronous copy that does not complete within
 * about 0.2 s makes the kernel return early and raises a flag.  This call synchronises the current device and returns
 * 1 if that happened since the last call (the results of that launch are then incomplete), 0 if not, -1 on a CUDA error.
 * [No counterpart in the reference, whose kernels use no asynchronous copies.] */
int slotscan_device_status(void);

int slotscan_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SLOTSCAN_H */
