/* CPU ORACLE for the slot-scan path -- TEST INFRASTRUCTURE, not product code.
 *
 * Only tests/, __graft_entry__.smoke() and the cpu-baseline legs of bench.py may load this library; the product
 * (the CUDA extension and its Python host side) never imports, links or executes anything in this directory.
 *
 * What it restates, in plain C loops, float and double:
 *   slotscan_oracle_fwd_{f32,f64}        the reference recurrence  gqa25/slotkern_kv.py:66-123 (pin=False)
 *   slotscan_oracle_bwd_{f32,f64}        its adjoint               gqa25/slotkern_kvt.py:157-171, slotkern_kvg.py:163-200
 *   slotscan_oracle_epilogue_*           kinv / valid              gqa25/memlm_sh.py:474-475
 *   slotscan_oracle_read_{fwd,bwd}_*     cosine read               gqa25/memlm_sh.py:362-397
 *   slotscan_oracle_fq_*                 midrise quantiser         gqa25/memlm_sh.py:221-229
 *   slotscan_oracle_v_{fwd,bwd}_*        keyless scan + adjoint    gqa25/slotkern_v.py:242-261, :14-19
 *
 * Pinned by tests/test_oracle_golden.py against fixtures that tests/golden/make_golden.py produced by running the
 * reference's own torch code (forward in float64 and float32, gradients by torch autograd).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int B, T, H, N, DK, DV, G;
    int hard, hard_gate, occ_bin, detach_addr, fr_per_token;
    double eps, temp;
} slotscan_cfg;

#define REAL float
#define SUF _f32
#define SQRT sqrtf
#define EXP expf
#define FLOOR floorf
#include "slotscan_oracle_impl.h"
#undef REAL
#undef SUF
#undef SQRT
#undef EXP
#undef FLOOR

#define REAL double
#define SUF _f64
#define SQRT sqrt
#define EXP exp
#define FLOOR floor
#include "slotscan_oracle_impl.h"
#undef REAL
#undef SUF
#undef SQRT
#undef EXP
#undef FLOOR

#ifdef _OPENMP
#include <omp.h>
int slotscan_oracle_threads(void) { return omp_get_max_threads(); }
void slotscan_oracle_set_threads(int n) { omp_set_num_threads(n); }
#else
int slotscan_oracle_threads(void) { return 1; }
void slotscan_oracle_set_threads(int n) { (void)n; }
#endif
