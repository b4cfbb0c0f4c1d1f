/* CPU ORACLE (test infrastructure, not product code) -- body of the slot-scan restatement, included
 * once per arithmetic type by slotscan_oracle.c with REAL / SUF defined.
 *
 * Restates the key-matched slot scan of the reference project:
 *   forward recurrence            gqa25/slotkern_kv.py:66-123   (_ref_scan_kv_impl, always pin=False)
 *   first-free-row mask           gqa25/slotkern_kv.py:46-51
 *   step adjoint                  gqa25/slotkern_kvt.py:157-171, gqa25/slotkern_kvg.py:163-200
 *   cosine read                   gqa25/memlm_sh.py:362-397 (SharedMixer._read) with the writer epilogue :474-475
 *   midrise group quantiser       gqa25/memlm_sh.py:221-234 (_fq, _quantize_mem)
 * Everything is a plain loop over (sequence, head); OpenMP spreads those over the host cores.
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUF)

#define NEG_MASK ((REAL)-1e30)
#define CKPT 32 /* backward: full state kept every CKPT tokens, the segment in between is replayed */

/* scratch of one scan step: scores, candidates and the address actually used by the forward */
typedef struct {
    REAL *s, *z, *asoft, *afwd, *kinv, *occ, *qn;
    unsigned char* ok;
    REAL qnorm, qinv, g_eff, fr_t, margin;
    int am;
} FN(step_ws);

static void FN(ws_alloc)(FN(step_ws) * w, int N, int DK) {
    w->s = (REAL*)malloc(sizeof(REAL) * N);
    w->z = (REAL*)malloc(sizeof(REAL) * N);
    w->asoft = (REAL*)malloc(sizeof(REAL) * N);
    w->afwd = (REAL*)malloc(sizeof(REAL) * N);
    w->kinv = (REAL*)malloc(sizeof(REAL) * N);
    w->occ = (REAL*)malloc(sizeof(REAL) * N);
    w->qn = (REAL*)malloc(sizeof(REAL) * DK);
    w->ok = (unsigned char*)malloc(N);
}
static void FN(ws_free)(FN(step_ws) * w) {
    free(w->s); free(w->z); free(w->asoft); free(w->afwd); free(w->kinv); free(w->occ); free(w->qn); free(w->ok);
}

/* Address of one token against the pre-write state (K, o).  slotkern_kv.py:84-113. */
static void FN(step_address)(const slotscan_cfg* c, const REAL* K, const REAL* o, const REAL* qt, REAL gate_t,
                             REAL fr_t, FN(step_ws) * w) {
    const int N = c->N, DK = c->DK;
    const REAL eps = (REAL)c->eps, temp = (REAL)c->temp;
    REAL qq = 0;
    for (int d = 0; d < DK; d++) qq += qt[d] * qt[d];
    w->qnorm = SQRT(qq);
    w->qinv = (REAL)1 / (w->qnorm > (REAL)1e-6 ? w->qnorm : (REAL)1e-6);
    for (int d = 0; d < DK; d++) w->qn[d] = qt[d] * w->qinv;
    int first_empty = -1;
    for (int n = 0; n < N; n++)
        if (o[n] < eps) { first_empty = n; break; }
    REAL zmax = -INFINITY, z2 = -INFINITY;
    int am = 0;
    for (int n = 0; n < N; n++) {
        const REAL* Kn = K + (size_t)n * DK;
        REAL kk = 0;
        for (int d = 0; d < DK; d++) kk += Kn[d] * Kn[d];
        REAL kn = SQRT(kk);
        w->kinv[n] = (REAL)1 / (kn > (REAL)1e-6 ? kn : (REAL)1e-6);
        REAL dt = 0;
        for (int d = 0; d < DK; d++) dt += (Kn[d] * w->kinv[n]) * w->qn[d];   /* normalise first, then dot */
        w->s[n] = dt * temp;
        w->occ[n] = c->occ_bin ? (o[n] >= eps ? (REAL)1 : (REAL)0) : o[n];
        w->ok[n] = (o[n] >= eps) || (n == first_empty);
        REAL z = w->s[n] - fr_t * w->occ[n];
        if (!w->ok[n]) z = NEG_MASK;
        w->z[n] = z;
        if (z > zmax) { z2 = zmax; zmax = z; am = n; }        /* strict: the FIRST maximum wins */
        else if (z > z2) z2 = z;
    }
    w->am = am;
    w->margin = zmax - z2;
    REAL se = 0;
    for (int n = 0; n < N; n++) {   /* a masked row is exp(-1e30 - zmax) = 0 exactly; skip the slow libm underflow path */
        w->asoft[n] = w->ok[n] ? EXP(w->z[n] - zmax) : (REAL)0;
        se += w->asoft[n];
    }
    for (int n = 0; n < N; n++) w->asoft[n] /= se;
    if (c->hard) for (int n = 0; n < N; n++) w->afwd[n] = (n == am) ? (REAL)1 : (REAL)0;
    else for (int n = 0; n < N; n++) w->afwd[n] = w->asoft[n];
    w->g_eff = c->hard_gate ? (gate_t > (REAL)0.5 ? (REAL)1 : (REAL)0) : gate_t;
    w->fr_t = fr_t;
}

/* K,V,o <- (1-w) state + w * token.  slotkern_kv.py:114-120. */
static void FN(step_write)(const slotscan_cfg* c, REAL* K, REAL* V, REAL* o, const REAL* kt, const REAL* vt,
                           const FN(step_ws) * w) {
    const int N = c->N, DK = c->DK, DV = c->DV;
    for (int n = 0; n < N; n++) {
        const REAL wn = w->g_eff * w->afwd[n];
        if (w->afwd[n] == (REAL)0) continue;      /* exact no-op rows */
        const REAL om = (REAL)1 - wn;
        REAL* Kn = K + (size_t)n * DK;
        REAL* Vn = V + (size_t)n * DV;
        for (int d = 0; d < DK; d++) Kn[d] = om * Kn[d] + wn * kt[d];
        for (int d = 0; d < DV; d++) Vn[d] = om * Vn[d] + wn * vt[d];
        o[n] = om * o[n] + wn;
    }
}

/* Forward scan.  kbuf/vbuf: (B, NB, H, N, D) pre-write snapshots at t = 0, G, 2G, ...
 * addr (B,T,H) int32 / margin (B,T,H) / kfin,vfin (B,H,N,D) / ofin (B,H,N): optional (NULL to skip). */
int FN(slotscan_oracle_fwd)(const slotscan_cfg* c, const REAL* k, const REAL* q, const REAL* v, const REAL* gate,
                            const REAL* fr, REAL* kbuf, REAL* vbuf, int* addr, REAL* margin, REAL* kfin,
                            REAL* vfin, REAL* ofin) {
    const int B = c->B, T = c->T, H = c->H, N = c->N, DK = c->DK, DV = c->DV, G = c->G;
    const int NB = (T + G - 1) / G;
    if (!q) q = k;
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * H; bh++) {
        const int b = bh / H, h = bh % H;
        REAL* K = (REAL*)calloc((size_t)N * DK, sizeof(REAL));
        REAL* V = (REAL*)calloc((size_t)N * DV, sizeof(REAL));
        REAL* o = (REAL*)calloc(N, sizeof(REAL));
        FN(step_ws) w;
        FN(ws_alloc)(&w, N, DK);
        for (int t = 0; t < T; t++) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            if (t % G == 0) {
                const size_t so = ((size_t)b * NB + t / G) * H + h;
                if (kbuf) memcpy(kbuf + so * N * DK, K, sizeof(REAL) * N * DK);
                if (vbuf) memcpy(vbuf + so * N * DV, V, sizeof(REAL) * N * DV);
            }
            const REAL fr_t = c->fr_per_token ? fr[ix] : fr[0];
            FN(step_address)(c, K, o, q + ix * DK, gate[ix], fr_t, &w);
            if (addr) addr[ix] = w.am;
            if (margin) margin[ix] = w.margin;
            FN(step_write)(c, K, V, o, k + ix * DK, v + ix * DV, &w);
        }
        if (kfin) memcpy(kfin + (size_t)bh * N * DK, K, sizeof(REAL) * N * DK);
        if (vfin) memcpy(vfin + (size_t)bh * N * DV, V, sizeof(REAL) * N * DV);
        if (ofin) memcpy(ofin + (size_t)bh * N, o, sizeof(REAL) * N);
        FN(ws_free)(&w);
        free(K); free(V); free(o);
    }
    return 0;
}

/* Backward scan: gradients of sum(kbuf*dkbuf) + sum(vbuf*dvbuf) w.r.t. k, q, v, gate, fr, temp.
 * dq may be NULL when q is NULL (the search query is the stored key; both paths then add into dk).
 * dfr: (B,T,H) when fr_per_token else 1 element; dtemp: 1 element.  dkbuf/dvbuf may be NULL (zeros). */
int FN(slotscan_oracle_bwd)(const slotscan_cfg* c, const REAL* k, const REAL* q, const REAL* v, const REAL* gate,
                            const REAL* fr, const REAL* dkbuf, const REAL* dvbuf, REAL* dk, REAL* dq, REAL* dv,
                            REAL* dgate, REAL* dfr, REAL* dtemp) {
    const int B = c->B, T = c->T, H = c->H, N = c->N, DK = c->DK, DV = c->DV, G = c->G;
    const int NB = (T + G - 1) / G;
    const int q_is_k = (q == NULL);
    if (!q) q = k;
    const int NCK = (T + CKPT - 1) / CKPT;
    const size_t SK = (size_t)N * DK, SV = (size_t)N * DV;
    REAL* dfr_part = (REAL*)calloc((size_t)B * H, sizeof(REAL));
    REAL* dtemp_part = (REAL*)calloc((size_t)B * H, sizeof(REAL));
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * H; bh++) {
        const int b = bh / H, h = bh % H;
        /* checkpoints of the pre-write state at t = 0, CKPT, 2 CKPT, ... and the replayed segment */
        REAL* ckK = (REAL*)malloc(sizeof(REAL) * SK * NCK);
        REAL* ckV = (REAL*)malloc(sizeof(REAL) * SV * NCK);
        REAL* ckO = (REAL*)malloc(sizeof(REAL) * N * NCK);
        REAL* sgK = (REAL*)malloc(sizeof(REAL) * SK * CKPT);
        REAL* sgV = (REAL*)malloc(sizeof(REAL) * SV * CKPT);
        REAL* sgO = (REAL*)malloc(sizeof(REAL) * N * CKPT);
        REAL* K = (REAL*)calloc(SK, sizeof(REAL));
        REAL* V = (REAL*)calloc(SV, sizeof(REAL));
        REAL* o = (REAL*)calloc(N, sizeof(REAL));
        REAL* dK = (REAL*)calloc(SK, sizeof(REAL));
        REAL* dV = (REAL*)calloc(SV, sizeof(REAL));
        REAL* dO = (REAL*)calloc(N, sizeof(REAL));
        REAL* dw = (REAL*)malloc(sizeof(REAL) * N);
        REAL* dz = (REAL*)malloc(sizeof(REAL) * N);
        REAL* dqn = (REAL*)malloc(sizeof(REAL) * DK);
        FN(step_ws) w;
        FN(ws_alloc)(&w, N, DK);
        for (int t = 0; t < T; t++) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            if (t % CKPT == 0) {
                memcpy(ckK + SK * (t / CKPT), K, sizeof(REAL) * SK);
                memcpy(ckV + SV * (t / CKPT), V, sizeof(REAL) * SV);
                memcpy(ckO + (size_t)N * (t / CKPT), o, sizeof(REAL) * N);
            }
            FN(step_address)(c, K, o, q + ix * DK, gate[ix], c->fr_per_token ? fr[ix] : fr[0], &w);
            FN(step_write)(c, K, V, o, k + ix * DK, v + ix * DV, &w);
        }
        REAL dfr_acc = 0, dtemp_acc = 0;
        for (int ck = NCK - 1; ck >= 0; ck--) {
            const int t0 = ck * CKPT, t1 = (t0 + CKPT < T) ? t0 + CKPT : T;
            memcpy(K, ckK + SK * ck, sizeof(REAL) * SK);
            memcpy(V, ckV + SV * ck, sizeof(REAL) * SV);
            memcpy(o, ckO + (size_t)N * ck, sizeof(REAL) * N);
            for (int t = t0; t < t1; t++) {
                const size_t ix = ((size_t)b * T + t) * H + h;
                memcpy(sgK + SK * (t - t0), K, sizeof(REAL) * SK);
                memcpy(sgV + SV * (t - t0), V, sizeof(REAL) * SV);
                memcpy(sgO + (size_t)N * (t - t0), o, sizeof(REAL) * N);
                FN(step_address)(c, K, o, q + ix * DK, gate[ix], c->fr_per_token ? fr[ix] : fr[0], &w);
                FN(step_write)(c, K, V, o, k + ix * DK, v + ix * DV, &w);
            }
            for (int t = t1 - 1; t >= t0; t--) {
                const size_t ix = ((size_t)b * T + t) * H + h;
                const REAL* Kp = sgK + SK * (t - t0);
                const REAL* Vp = sgV + SV * (t - t0);
                const REAL* op = sgO + (size_t)N * (t - t0);
                const REAL *kt = k + ix * DK, *vt = v + ix * DV, *qt = q + ix * DK;
                const REAL temp = (REAL)c->temp;
                FN(step_address)(c, Kp, op, qt, gate[ix], c->fr_per_token ? fr[ix] : fr[0], &w);
                /* dw_n: slotkern_kvg.py:165 */
                REAL dg = 0, sa = 0;
                for (int n = 0; n < N; n++) {
                    REAL a1 = 0, a2 = 0;
                    for (int d = 0; d < DK; d++) a1 += (kt[d] - Kp[(size_t)n * DK + d]) * dK[(size_t)n * DK + d];
                    for (int d = 0; d < DV; d++) a2 += (vt[d] - Vp[(size_t)n * DV + d]) * dV[(size_t)n * DV + d];
                    dw[n] = a1 + a2 + ((REAL)1 - op[n]) * dO[n];
                    dg += w.afwd[n] * dw[n];
                    if (w.ok[n]) sa += w.asoft[n] * (w.g_eff * dw[n]);
                }
                /* token gradients through the store path: slotkern_kvg.py:167-169 */
                for (int d = 0; d < DK; d++) {
                    REAL acc = 0;
                    for (int n = 0; n < N; n++)
                        if (w.afwd[n] != (REAL)0) acc += (w.g_eff * w.afwd[n]) * dK[(size_t)n * DK + d];
                    dk[ix * DK + d] = acc;
                }
                for (int d = 0; d < DV; d++) {
                    REAL acc = 0;
                    for (int n = 0; n < N; n++)
                        if (w.afwd[n] != (REAL)0) acc += (w.g_eff * w.afwd[n]) * dV[(size_t)n * DV + d];
                    dv[ix * DV + d] = acc;
                }
                dgate[ix] = dg;
                /* softmax adjoint: slotkern_kvg.py:170-179 */
                REAL dfr_t = 0;
                for (int d = 0; d < DK; d++) dqn[d] = 0;
                for (int n = 0; n < N; n++) {
                    dz[n] = w.ok[n] ? w.asoft[n] * (w.g_eff * dw[n] - sa) : (REAL)0;
                    dfr_t -= w.occ[n] * dz[n];
                    dtemp_acc += dz[n] * w.s[n] / temp;
                    if (dz[n] != (REAL)0)
                        for (int d = 0; d < DK; d++) dqn[d] += dz[n] * temp * (Kp[(size_t)n * DK + d] * w.kinv[n]);
                }
                if (c->fr_per_token) dfr[ix] = dfr_t; else dfr_acc += dfr_t;
                /* query gradient through the normalisation: slotkern_kvg.py:189-190 */
                REAL prq = 0;
                for (int d = 0; d < DK; d++) prq += dqn[d] * w.qn[d];
                for (int d = 0; d < DK; d++) {
                    const REAL gq = (w.qnorm < (REAL)1e-6) ? w.qinv * dqn[d] : w.qinv * (dqn[d] - w.qn[d] * prq);
                    if (q_is_k) dk[ix * DK + d] += gq; else dq[ix * DK + d] = gq;
                }
                /* carry the state adjoints to the pre-write side: slotkern_kvg.py:183-196 */
                const int emit = (t % G == 0);
                const size_t so = ((size_t)b * NB + t / G) * H + h;
                for (int n = 0; n < N; n++) {
                    const REAL om = (REAL)1 - w.g_eff * w.afwd[n];
                    REAL* dKn = dK + (size_t)n * DK;
                    REAL* dVn = dV + (size_t)n * DV;
                    const REAL* Kn = Kp + (size_t)n * DK;
                    REAL knorm = (REAL)1 / w.kinv[n];   /* = max(|K_n|, 1e-6) */
                    REAL kk = 0;
                    for (int d = 0; d < DK; d++) kk += Kn[d] * Kn[d];
                    const int clamped = SQRT(kk) < (REAL)1e-6;
                    (void)knorm;
                    REAL prj = 0;
                    const int match = !c->detach_addr && !clamped && dz[n] != (REAL)0;
                    if (match)
                        for (int d = 0; d < DK; d++) prj += (dz[n] * temp * w.qn[d]) * (Kn[d] * w.kinv[n]);
                    for (int d = 0; d < DK; d++) {
                        REAL x = om * dKn[d];
                        if (emit && dkbuf) x += dkbuf[so * SK + (size_t)n * DK + d];
                        if (match) x += w.kinv[n] * (dz[n] * temp * w.qn[d] - (Kn[d] * w.kinv[n]) * prj);
                        dKn[d] = x;
                    }
                    for (int d = 0; d < DV; d++) {
                        REAL x = om * dVn[d];
                        if (emit && dvbuf) x += dvbuf[so * SV + (size_t)n * DV + d];
                        dVn[d] = x;
                    }
                    dO[n] = om * dO[n] - (c->occ_bin ? (REAL)0 : w.fr_t * dz[n]);
                }
            }
        }
        dfr_part[bh] = dfr_acc;
        dtemp_part[bh] = dtemp_acc;
        FN(ws_free)(&w);
        free(ckK); free(ckV); free(ckO); free(sgK); free(sgV); free(sgO);
        free(K); free(V); free(o); free(dK); free(dV); free(dO); free(dw); free(dz); free(dqn);
    }
    REAL sfr = 0, stp = 0;
    for (int i = 0; i < B * H; i++) { sfr += dfr_part[i]; stp += dtemp_part[i]; }   /* fixed order: repeatable */
    if (!c->fr_per_token) dfr[0] = sfr;
    dtemp[0] = stp;
    free(dfr_part); free(dtemp_part);
    return 0;
}

/* Writer epilogue, memlm_sh.py:474-475: kinv = rsqrt(max(|k|^2, 1e-12)), valid = |k|^2 > 1e-12 per snapshot row. */
int FN(slotscan_oracle_epilogue)(const REAL* kbuf, long rows, int DK, REAL* kinv, unsigned char* valid) {
#pragma omp parallel for
    for (long r = 0; r < rows; r++) {
        REAL nsq = 0;
        for (int d = 0; d < DK; d++) nsq += kbuf[r * DK + d] * kbuf[r * DK + d];
        kinv[r] = (REAL)1 / SQRT(nsq > (REAL)1e-12 ? nsq : (REAL)1e-12);
        valid[r] = nsq > (REAL)1e-12;
    }
    return 0;
}

/* Cosine read of the stride-G snapshots, memlm_sh.py:379-397.  qr (B,T,H,NQ,DK) raw read queries (normalised here
 * with the 1e-6 norm clamp), sharp (B,T,H,NQ) = the per-token logit multiplier (exp(log_rsel) * exp(s_tok)),
 * kbuf/vbuf (B,NB,H,N,D), kinv/valid (B,NB,H,N).  Token t reads snapshot t / G.  rd (B,T,H,NQ,DV).
 * An all-invalid snapshot reads exactly zero. */
int FN(slotscan_oracle_read_fwd)(int B, int T, int H, int NQ, int N, int DK, int DV, int G, const REAL* qr,
                                 const REAL* sharp, const REAL* kbuf, const REAL* vbuf, const REAL* kinv,
                                 const unsigned char* valid, REAL* rd, REAL* att_out) {
    const int NB = (T + G - 1) / G;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; b++)
        for (int t = 0; t < T; t++) {
            REAL* sc = (REAL*)malloc(sizeof(REAL) * N);
            for (int h = 0; h < H; h++) {
                const size_t so = ((size_t)b * NB + t / G) * H + h;
                const REAL *Kb = kbuf + so * N * DK, *Vb = vbuf + so * N * DV, *ki = kinv + so * N;
                const unsigned char* va = valid + so * N;
                for (int j = 0; j < NQ; j++) {
                    const size_t qi = (((size_t)b * T + t) * H + h) * NQ + j;
                    const REAL* qv = qr + qi * DK;
                    REAL qq = 0;
                    for (int d = 0; d < DK; d++) qq += qv[d] * qv[d];
                    REAL qn = SQRT(qq);
                    const REAL qinv = (REAL)1 / (qn > (REAL)1e-6 ? qn : (REAL)1e-6);
                    REAL m = -INFINITY;
                    int any = 0;
                    for (int n = 0; n < N; n++) {
                        if (!va[n]) { sc[n] = -INFINITY; continue; }
                        REAL dt = 0;
                        for (int d = 0; d < DK; d++) dt += (qv[d] * qinv) * Kb[(size_t)n * DK + d];
                        sc[n] = dt * ki[n] * sharp[qi];
                        if (sc[n] > m) m = sc[n];
                        any = 1;
                    }
                    REAL se = 0;
                    for (int n = 0; n < N; n++) { sc[n] = (any && va[n]) ? EXP(sc[n] - m) : (REAL)0; se += sc[n]; }
                    REAL* out = rd + qi * DV;
                    for (int d = 0; d < DV; d++) out[d] = 0;
                    for (int n = 0; n < N; n++) {
                        const REAL a = any ? sc[n] / se : (REAL)0;
                        if (att_out) att_out[qi * N + n] = a;
                        if (a != (REAL)0)
                            for (int d = 0; d < DV; d++) out[d] += a * Vb[(size_t)n * DV + d];
                    }
                }
            }
            free(sc);
        }
    return 0;
}

/* Adjoint of the read above for an upstream gradient drd (B,T,H,NQ,DV): dqr, dsharp per query, and the
 * snapshot gradients dkbuf, dvbuf (accumulated over the G tokens and NQ queries that share a snapshot).
 * kinv and valid are treated as constants of kbuf only if kinv_const != 0; otherwise kinv = rsqrt(max(|k|^2,1e-12))
 * is differentiated too (the reference differentiates it: kinv is computed from kbuf with autograd on). */
int FN(slotscan_oracle_read_bwd)(int B, int T, int H, int NQ, int N, int DK, int DV, int G, const REAL* qr,
                                 const REAL* sharp, const REAL* kbuf, const REAL* vbuf, const REAL* kinv,
                                 const unsigned char* valid, const REAL* drd, REAL* dqr, REAL* dsharp, REAL* dkbuf,
                                 REAL* dvbuf, int kinv_const) {
    const int NB = (T + G - 1) / G;
    memset(dkbuf, 0, sizeof(REAL) * (size_t)B * NB * H * N * DK);
    memset(dvbuf, 0, sizeof(REAL) * (size_t)B * NB * H * N * DV);
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int b = 0; b < B; b++)
        for (int jb = 0; jb < NB; jb++) {
            REAL* att = (REAL*)malloc(sizeof(REAL) * N);
            REAL* raw = (REAL*)malloc(sizeof(REAL) * N);
            REAL* datt = (REAL*)malloc(sizeof(REAL) * N);
            REAL* qn = (REAL*)malloc(sizeof(REAL) * DK);
            REAL* dqn = (REAL*)malloc(sizeof(REAL) * DK);
            for (int t = jb * G; t < T && t < (jb + 1) * G; t++)
                for (int h = 0; h < H; h++) {
                    const size_t so = ((size_t)b * NB + jb) * H + h;
                    const REAL *Kb = kbuf + so * N * DK, *Vb = vbuf + so * N * DV, *ki = kinv + so * N;
                    REAL *dKb = dkbuf + so * N * DK, *dVb = dvbuf + so * N * DV;
                    const unsigned char* va = valid + so * N;
                    for (int j = 0; j < NQ; j++) {
                        const size_t qi = (((size_t)b * T + t) * H + h) * NQ + j;
                        const REAL *qv = qr + qi * DK, *go = drd + qi * DV;
                        REAL qq = 0;
                        for (int d = 0; d < DK; d++) qq += qv[d] * qv[d];
                        const REAL qnorm = SQRT(qq);
                        const REAL qinv = (REAL)1 / (qnorm > (REAL)1e-6 ? qnorm : (REAL)1e-6);
                        for (int d = 0; d < DK; d++) { qn[d] = qv[d] * qinv; dqn[d] = 0; }
                        REAL m = -INFINITY;
                        int any = 0;
                        for (int n = 0; n < N; n++) {
                            raw[n] = 0;
                            if (!va[n]) continue;
                            REAL dt = 0;
                            for (int d = 0; d < DK; d++) dt += qn[d] * Kb[(size_t)n * DK + d];
                            raw[n] = dt;
                            const REAL scv = dt * ki[n] * sharp[qi];
                            if (scv > m) m = scv;
                            any = 1;
                        }
                        REAL se = 0;
                        for (int n = 0; n < N; n++) {
                            att[n] = (any && va[n]) ? EXP(raw[n] * ki[n] * sharp[qi] - m) : (REAL)0;
                            se += att[n];
                        }
                        REAL dot = 0;
                        for (int n = 0; n < N; n++) {
                            att[n] = any ? att[n] / se : (REAL)0;
                            REAL da = 0;
                            for (int d = 0; d < DV; d++) da += go[d] * Vb[(size_t)n * DV + d];
                            datt[n] = da;
                            dot += att[n] * da;
                            if (att[n] != (REAL)0)
                                for (int d = 0; d < DV; d++) dVb[(size_t)n * DV + d] += att[n] * go[d];
                        }
                        REAL dsh = 0;
                        for (int n = 0; n < N; n++) {
                            if (!va[n] || !any) continue;
                            const REAL dsc = att[n] * (datt[n] - dot);       /* softmax adjoint */
                            dsh += dsc * raw[n] * ki[n];
                            const REAL draw = dsc * ki[n] * sharp[qi];
                            for (int d = 0; d < DK; d++) {
                                dqn[d] += draw * Kb[(size_t)n * DK + d];
                                dKb[(size_t)n * DK + d] += draw * qn[d];
                            }
                            if (!kinv_const) {
                                /* d kinv / d k = -kinv^3 k  (only above the 1e-12 clamp, which valid implies) */
                                const REAL dki = dsc * raw[n] * sharp[qi];
                                const REAL c3 = -ki[n] * ki[n] * ki[n] * dki;
                                for (int d = 0; d < DK; d++) dKb[(size_t)n * DK + d] += c3 * Kb[(size_t)n * DK + d];
                            }
                        }
                        dsharp[qi] = dsh;
                        REAL pr = 0;
                        for (int d = 0; d < DK; d++) pr += dqn[d] * qn[d];
                        for (int d = 0; d < DK; d++)
                            dqr[qi * DK + d] = (qnorm < (REAL)1e-6) ? qinv * dqn[d] : qinv * (dqn[d] - qn[d] * pr);
                    }
                }
            free(att); free(raw); free(datt); free(qn); free(dqn);
        }
    return 0;
}

/* Midrise group quantiser, memlm_sh.py:221-229: per group of `group` channels, s = max(absmax / 2^(bits-1), 1e-30),
 * q = (clamp(floor(x / s), -half, half-1) + 0.5) * s, returned as x + (q - x); an all-zero group stays exactly zero. */
int FN(slotscan_oracle_fq)(const REAL* x, long n_groups, int group, int bits, REAL* y) {
    const REAL half = (REAL)(1 << (bits - 1));
#pragma omp parallel for
    for (long gi = 0; gi < n_groups; gi++) {
        const REAL* xg = x + gi * group;
        REAL* yg = y + gi * group;
        REAL a = 0;
        for (int i = 0; i < group; i++) { REAL v = xg[i] < 0 ? -xg[i] : xg[i]; if (v > a) a = v; }
        REAL s = a / half;
        if (s < (REAL)1e-30) s = (REAL)1e-30;
        for (int i = 0; i < group; i++) {
            REAL f = FLOOR(xg[i] / s);
            if (f < -half) f = -half;
            if (f > half - 1) f = half - 1;
            const REAL qv = (a > 0) ? (f + (REAL)0.5) * s : (REAL)0;
            /* the reference returns the straight-through form x + (q - x), memlm_sh.py:229: one more rounding */
            const volatile REAL diff = qv - xg[i];
            yg[i] = xg[i] + diff;
        }
    }
    return 0;
}

/* ---- keyless scan: address logits given from outside, value-only state ----
 * gqa25/slotkern_v.py:242-261 (ref_scan_v) and the adjoint stated in its module docstring (:14-19):
 *   z = wa_t - fr o over ALL N rows (no free-row mask),  a_s = softmax(z),  a = onehot(argmax z) if hard else a_s,
 *   g_h = [g > 0.5] if hard_gate else g,  w = g_h a,  V <- (1-w) V + w v_t,  o <- (1-w) o + w.
 * buf (B,NB,H,N,DV): pre-write V at t = 0, G, 2G, ...  fr: 1 element. */
static void FN(v_step)(int N, int hard, int hard_gate, const REAL* wa, const REAL* o, REAL fr, REAL gate_t, REAL* asoft,
                       REAL* afwd, REAL* g_eff) {
    REAL zmax = -INFINITY;
    int am = 0;
    for (int n = 0; n < N; n++) {
        const REAL z = wa[n] - fr * o[n];
        asoft[n] = z;
        if (z > zmax) { zmax = z; am = n; }                       /* first maximum */
    }
    REAL se = 0;
    for (int n = 0; n < N; n++) { asoft[n] = EXP(asoft[n] - zmax); se += asoft[n]; }
    for (int n = 0; n < N; n++) {
        asoft[n] /= se;
        afwd[n] = hard ? (n == am ? (REAL)1 : (REAL)0) : asoft[n];
    }
    *g_eff = hard_gate ? (gate_t > (REAL)0.5 ? (REAL)1 : (REAL)0) : gate_t;
}

int FN(slotscan_oracle_v_fwd)(int B, int T, int H, int N, int DV, int G, int hard, int hard_gate, const REAL* v,
                              const REAL* wa, const REAL* gate, const REAL* fr, REAL* buf, int* addr) {
    const int NB = (T + G - 1) / G;
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * H; bh++) {
        const int b = bh / H, h = bh % H;
        REAL* V = (REAL*)calloc((size_t)N * DV, sizeof(REAL));
        REAL* o = (REAL*)calloc(N, sizeof(REAL));
        REAL* as = (REAL*)malloc(sizeof(REAL) * N);
        REAL* af = (REAL*)malloc(sizeof(REAL) * N);
        for (int t = 0; t < T; t++) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            if (t % G == 0) memcpy(buf + (((size_t)b * NB + t / G) * H + h) * N * DV, V, sizeof(REAL) * N * DV);
            REAL g;
            FN(v_step)(N, hard, hard_gate, wa + ix * N, o, fr[0], gate[ix], as, af, &g);
            if (addr) { int am = 0; for (int n = 1; n < N; n++) if (af[n] > af[am]) am = n; addr[ix] = am; }
            for (int n = 0; n < N; n++) {
                const REAL w = g * af[n];
                if (af[n] == (REAL)0) continue;
                for (int d = 0; d < DV; d++) V[(size_t)n * DV + d] = ((REAL)1 - w) * V[(size_t)n * DV + d] + w * v[ix * DV + d];
                o[n] = ((REAL)1 - w) * o[n] + w;
            }
        }
        free(V); free(o); free(as); free(af);
    }
    return 0;
}

/* gradients of sum(buf * dbuf) w.r.t. v, wa, gate, fr (1 element) */
int FN(slotscan_oracle_v_bwd)(int B, int T, int H, int N, int DV, int G, int hard, int hard_gate, const REAL* v,
                              const REAL* wa, const REAL* gate, const REAL* fr, const REAL* dbuf, REAL* dv, REAL* dwa,
                              REAL* dgate, REAL* dfr) {
    const int NB = (T + G - 1) / G;
    REAL* part = (REAL*)calloc((size_t)B * H, sizeof(REAL));
#pragma omp parallel for schedule(dynamic)
    for (int bh = 0; bh < B * H; bh++) {
        const int b = bh / H, h = bh % H;
        const size_t SV = (size_t)N * DV;
        REAL* sV = (REAL*)malloc(sizeof(REAL) * SV * T);           /* every pre-write state: tests are small */
        REAL* sO = (REAL*)malloc(sizeof(REAL) * N * T);
        REAL* V = (REAL*)calloc(SV, sizeof(REAL));
        REAL* o = (REAL*)calloc(N, sizeof(REAL));
        REAL* as = (REAL*)malloc(sizeof(REAL) * N);
        REAL* af = (REAL*)malloc(sizeof(REAL) * N);
        REAL* dV = (REAL*)calloc(SV, sizeof(REAL));
        REAL* dO = (REAL*)calloc(N, sizeof(REAL));
        REAL* dw = (REAL*)malloc(sizeof(REAL) * N);
        for (int t = 0; t < T; t++) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            memcpy(sV + SV * t, V, sizeof(REAL) * SV);
            memcpy(sO + (size_t)N * t, o, sizeof(REAL) * N);
            REAL g;
            FN(v_step)(N, hard, hard_gate, wa + ix * N, o, fr[0], gate[ix], as, af, &g);
            for (int n = 0; n < N; n++) {
                const REAL w = g * af[n];
                if (af[n] == (REAL)0) continue;
                for (int d = 0; d < DV; d++) V[(size_t)n * DV + d] = ((REAL)1 - w) * V[(size_t)n * DV + d] + w * v[ix * DV + d];
                o[n] = ((REAL)1 - w) * o[n] + w;
            }
        }
        REAL acc_fr = 0;
        for (int t = T - 1; t >= 0; t--) {
            const size_t ix = ((size_t)b * T + t) * H + h;
            const REAL *Vp = sV + SV * t, *op = sO + (size_t)N * t;
            REAL g;
            FN(v_step)(N, hard, hard_gate, wa + ix * N, op, fr[0], gate[ix], as, af, &g);
            REAL dg = 0, sa = 0;
            for (int n = 0; n < N; n++) {
                REAL a1 = 0;
                for (int d = 0; d < DV; d++) a1 += (v[ix * DV + d] - Vp[(size_t)n * DV + d]) * dV[(size_t)n * DV + d];
                dw[n] = a1 + ((REAL)1 - op[n]) * dO[n];
                dg += af[n] * dw[n];
                sa += as[n] * (g * dw[n]);
            }
            for (int d = 0; d < DV; d++) {
                REAL a1 = 0;
                for (int n = 0; n < N; n++) a1 += (g * af[n]) * dV[(size_t)n * DV + d];
                dv[ix * DV + d] = a1;
            }
            dgate[ix] = dg;
            const int emit = (t % G == 0);
            const size_t so = ((size_t)b * NB + t / G) * H + h;
            for (int n = 0; n < N; n++) {
                const REAL dz = as[n] * (g * dw[n] - sa);
                dwa[ix * N + n] = dz;
                acc_fr -= op[n] * dz;
                const REAL om = (REAL)1 - g * af[n];
                for (int d = 0; d < DV; d++) {
                    REAL x = om * dV[(size_t)n * DV + d];
                    if (emit) x += dbuf[so * SV + (size_t)n * DV + d];
                    dV[(size_t)n * DV + d] = x;
                }
                dO[n] = om * dO[n] - fr[0] * dz;
            }
        }
        part[bh] = acc_fr;
        free(sV); free(sO); free(V); free(o); free(as); free(af); free(dV); free(dO); free(dw);
    }
    REAL sfr = 0;
    for (int i = 0; i < B * H; i++) sfr += part[i];
    dfr[0] = sfr;
    free(part);
    return 0;
}

#undef NEG_MASK
#undef CKPT
#undef FN
#undef CAT
#undef CAT_
