/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement (double precision, C99 complex)
 * of the reference's v2x2ssd scan.  Nothing in the shipped library may link or
 * call this file; it is the checker the CUDA path is compared against, and the
 * "port" CPU baseline that bench.py times.
 *
 * Parity status: PINNED.  tests/test_oracle_pins.py checks every function below
 * against fixtures under tests/golden/ that were produced by importing the
 * reference (slinoss/ops/v2x2ssd/reference.py and torch.autograd through it)
 * with tests/golden/make_golden.py.
 *
 * Conventions (slinoss/ops/v2x2ssd/reference.py:1-41):
 *   U (BH,T,P) real; M (BH,T,2) packed complex; K (BH,T,2,2) tap 0 = prev,
 *   tap 1 = curr, each (re,im); B,C (BH,T,2N) interleaved [re0,im0,re1,...];
 *   state (BH,P,2N) interleaved; Y (BH,T,P).
 *   A packed real gradient (d_re, d_im) is read as the complex d_re + i d_im.
 *
 * All arrays are double and contiguous.  Nullable pointers: init, Bprev, Uprev,
 * dfinal, and every gradient output.
 */
#include <complex.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef double complex cplx;

#define IDX_U(t, p) ((size_t)(t) * P + (p))

static inline cplx ld_c(const double *x) { return x[0] + I * x[1]; }
static inline void st_c(double *x, cplx v) {
  x[0] = creal(v);
  x[1] = cimag(v);
}
static inline void add_c(double *x, cplx v) {
  x[0] += creal(v);
  x[1] += cimag(v);
}

/* ------------------------------------------------------------------------- */
/* Sequential recurrence, one (batch,head).  reference.py:704-803 (v2x2ssm). */
/* z is the running state (P*N complex), updated in place for tokens [t0,t1). */
/* If Y != NULL the output rows are written.  traj (nullable) receives the    */
/* state AFTER each token: traj[(t-t0)*P*N + p*N + n].                        */
static void seq_forward_range(int t0, int t1, int P, int N, const double *U,
                              const double *M, const double *K,
                              const double *B, const double *C,
                              const double *bprev0, const double *uprev0,
                              cplx *z, double *Y, cplx *traj) {
  const int D = 2 * N;
  for (int t = t0; t < t1; ++t) {
    const cplx m = ld_c(M + 2 * (size_t)t);
    const cplx kp = ld_c(K + 4 * (size_t)t);
    const cplx kc = ld_c(K + 4 * (size_t)t + 2);
    const double *bp = (t == 0) ? bprev0 : B + (size_t)(t - 1) * D;
    const double *up = (t == 0) ? uprev0 : U + (size_t)(t - 1) * P;
    const double *bc = B + (size_t)t * D;
    const double *uc = U + (size_t)t * P;
    for (int p = 0; p < P; ++p) {
      const double upv = up ? up[p] : 0.0;
      const double ucv = uc[p];
      double acc = 0.0;
      for (int n = 0; n < N; ++n) {
        const cplx betap = bp ? kp * ld_c(bp + 2 * n) : 0.0;
        const cplx betac = kc * ld_c(bc + 2 * n);
        cplx v = m * z[(size_t)p * N + n] + upv * betap + ucv * betac;
        z[(size_t)p * N + n] = v;
        if (Y) acc += creal(conj(ld_c(C + (size_t)t * D + 2 * n)) * v);
      }
      if (Y) Y[(size_t)t * P + p] = acc;
    }
    if (traj)
      memcpy(traj + (size_t)(t - t0) * P * N, z, sizeof(cplx) * (size_t)P * N);
  }
}

void slx_oracle_v2x2ssm_fwd(int BH, int T, int P, int N, const double *U,
                            const double *M, const double *K, const double *B,
                            const double *C, const double *init,
                            const double *Bprev, const double *Uprev, double *Y,
                            double *final_state) {
  const int D = 2 * N;
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < BH; ++bh) {
    cplx *z = (cplx *)calloc((size_t)P * N, sizeof(cplx));
    if (init)
      for (int i = 0; i < P * N; ++i)
        z[i] = ld_c(init + (size_t)bh * P * D + 2 * (size_t)i);
    seq_forward_range(0, T, P, N, U + (size_t)bh * T * P, M + (size_t)bh * T * 2,
                      K + (size_t)bh * T * 4, B + (size_t)bh * T * D,
                      C + (size_t)bh * T * D,
                      Bprev ? Bprev + (size_t)bh * D : NULL,
                      Uprev ? Uprev + (size_t)bh * P : NULL, z,
                      Y + (size_t)bh * T * P, NULL);
    if (final_state)
      for (int i = 0; i < P * N; ++i)
        st_c(final_state + (size_t)bh * P * D + 2 * (size_t)i, z[i]);
    free(z);
  }
}

/* ------------------------------------------------------------------------- */
/* Gradients of the recurrence.  This restates what torch.autograd computes   */
/* through reference.py:1195 (v2x2ssd) / :704 (v2x2ssm): the adjoint state     */
/*   lambda_t = dY_t (x) c_t + conj(m_{t+1}) lambda_{t+1},  lambda_T = dfinal. */
/* States are re-materialised per checkpoint segment of `seg` tokens.          */
void slx_oracle_v2x2ssm_bwd(int BH, int T, int P, int N, const double *U,
                            const double *M, const double *K, const double *B,
                            const double *C, const double *init,
                            const double *Bprev, const double *Uprev,
                            const double *dY, const double *dfinal, double *dU,
                            double *dM, double *dK, double *dB, double *dC,
                            double *dinit, double *dBprev, double *dUprev) {
  const int D = 2 * N;
  const int seg = 64;
  const int nseg = (T + seg - 1) / seg;
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < BH; ++bh) {
    const double *Ub = U + (size_t)bh * T * P, *Mb = M + (size_t)bh * T * 2;
    const double *Kb = K + (size_t)bh * T * 4, *Bb = B + (size_t)bh * T * D;
    const double *Cb = C + (size_t)bh * T * D;
    const double *dYb = dY ? dY + (size_t)bh * T * P : NULL;
    const double *bp0 = Bprev ? Bprev + (size_t)bh * D : NULL;
    const double *up0 = Uprev ? Uprev + (size_t)bh * P : NULL;
    double *dUb = dU + (size_t)bh * T * P, *dMb = dM + (size_t)bh * T * 2;
    double *dKb = dK + (size_t)bh * T * 4, *dBb = dB + (size_t)bh * T * D;
    double *dCb = dC + (size_t)bh * T * D;
    const size_t PN = (size_t)P * N;

    memset(dUb, 0, sizeof(double) * (size_t)T * P);
    memset(dBb, 0, sizeof(double) * (size_t)T * D);
    double *dbp0 = (double *)calloc(D, sizeof(double));
    double *dup0 = (double *)calloc(P, sizeof(double));

    /* checkpoints: state BEFORE each segment */
    cplx *ckpt = (cplx *)calloc((size_t)(nseg + 1) * PN, sizeof(cplx));
    cplx *z = (cplx *)calloc(PN, sizeof(cplx));
    if (init)
      for (size_t i = 0; i < PN; ++i)
        z[i] = ld_c(init + (size_t)bh * P * D + 2 * i);
    for (int s = 0; s < nseg; ++s) {
      memcpy(ckpt + (size_t)s * PN, z, sizeof(cplx) * PN);
      int t0 = s * seg, t1 = t0 + seg < T ? t0 + seg : T;
      seq_forward_range(t0, t1, P, N, Ub, Mb, Kb, Bb, Cb, bp0, up0, z, NULL,
                        NULL);
    }
    cplx *traj = (cplx *)calloc((size_t)seg * PN, sizeof(cplx));
    cplx *lam = (cplx *)calloc(PN, sizeof(cplx));
    cplx *dbc = (cplx *)calloc(N, sizeof(cplx));
    cplx *dbp = (cplx *)calloc(N, sizeof(cplx));
    if (dfinal)
      for (size_t i = 0; i < PN; ++i)
        lam[i] = ld_c(dfinal + (size_t)bh * P * D + 2 * i);

    for (int s = nseg - 1; s >= 0; --s) {
      int t0 = s * seg, t1 = t0 + seg < T ? t0 + seg : T;
      memcpy(z, ckpt + (size_t)s * PN, sizeof(cplx) * PN);
      seq_forward_range(t0, t1, P, N, Ub, Mb, Kb, Bb, Cb, bp0, up0, z, NULL,
                        traj);
      for (int t = t1 - 1; t >= t0; --t) {
        const cplx *ht = traj + (size_t)(t - t0) * PN;
        const cplx *hm = (t == t0) ? ckpt + (size_t)s * PN
                                   : traj + (size_t)(t - 1 - t0) * PN;
        const cplx m = ld_c(Mb + 2 * (size_t)t);
        const cplx kp = ld_c(Kb + 4 * (size_t)t);
        const cplx kc = ld_c(Kb + 4 * (size_t)t + 2);
        const double *bcur = Bb + (size_t)t * D;
        const double *ucur = Ub + (size_t)t * P;
        const double *bpr = (t == 0) ? bp0 : Bb + (size_t)(t - 1) * D;
        const double *upr = (t == 0) ? up0 : Ub + (size_t)(t - 1) * P;
        double *dbpr = (t == 0) ? dbp0 : dBb + (size_t)(t - 1) * D;
        double *dupr = (t == 0) ? dup0 : dUb + (size_t)(t - 1) * P;
        /* lambda_t += dY_t (x) c_t ; dC_t = sum_p dY_t[p] h_t[p,:] */
        for (int n = 0; n < N; ++n) {
          cplx acc = 0.0;
          cplx c = ld_c(Cb + (size_t)t * D + 2 * n);
          for (int p = 0; p < P; ++p) {
            double g = dYb ? dYb[(size_t)t * P + p] : 0.0;
            lam[(size_t)p * N + n] += g * c;
            acc += g * ht[(size_t)p * N + n];
          }
          st_c(dCb + (size_t)t * D + 2 * n, acc);
        }
        cplx dm = 0.0;
        for (int n = 0; n < N; ++n) dbc[n] = dbp[n] = 0.0;
        for (int p = 0; p < P; ++p) {
          double uc = ucur[p], upv = upr ? upr[p] : 0.0;
          double du_c = 0.0, du_p = 0.0;
          for (int n = 0; n < N; ++n) {
            cplx l = lam[(size_t)p * N + n];
            dm += conj(hm[(size_t)p * N + n]) * l;
            dbc[n] += uc * l;
            dbp[n] += upv * l;
            du_c += creal(conj(kc * ld_c(bcur + 2 * n)) * l);
            if (bpr) du_p += creal(conj(kp * ld_c(bpr + 2 * n)) * l);
          }
          dUb[(size_t)t * P + p] += du_c;
          dupr[p] += du_p;
        }
        st_c(dMb + 2 * (size_t)t, dm);
        cplx dkc = 0.0, dkp = 0.0;
        for (int n = 0; n < N; ++n) {
          add_c(dBb + (size_t)t * D + 2 * n, conj(kc) * dbc[n]);
          add_c(dbpr + 2 * n, conj(kp) * dbp[n]);
          dkc += conj(ld_c(bcur + 2 * n)) * dbc[n];
          if (bpr) dkp += conj(ld_c(bpr + 2 * n)) * dbp[n];
        }
        st_c(dKb + 4 * (size_t)t, dkp);
        st_c(dKb + 4 * (size_t)t + 2, dkc);
        for (size_t i = 0; i < PN; ++i) lam[i] *= conj(m);
      }
    }
    if (dinit)
      for (size_t i = 0; i < PN; ++i)
        st_c(dinit + (size_t)bh * P * D + 2 * i, lam[i]);
    if (dBprev) memcpy(dBprev + (size_t)bh * D, dbp0, sizeof(double) * D);
    if (dUprev) memcpy(dUprev + (size_t)bh * P, dup0, sizeof(double) * P);
    free(dbp0); free(dup0); free(ckpt); free(z); free(traj); free(lam);
    free(dbc); free(dbp);
  }
}

/* ------------------------------------------------------------------------- */
/* Stage 1.  reference.py:937-1012 (chunk_increment) with the reverse scan of  */
/* reference.py:494-516 (_chunk_increment_core) and the padding of :612-667    */
/* (M=1, K=U=B=0 beyond T).  inc (BH,NC,P,2N), m_chunk (BH,NC,2).              */
void slx_oracle_chunk_increment(int BH, int T, int P, int N, int L,
                                const double *U, const double *M,
                                const double *K, const double *B,
                                const double *Bprev, const double *Uprev,
                                double *inc, double *m_chunk) {
  const int D = 2 * N;
  const int NC = (T + L - 1) / L;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int bh = 0; bh < BH; ++bh) {
    for (int c = 0; c < NC; ++c) {
      const double *Ub = U + (size_t)bh * T * P, *Mb = M + (size_t)bh * T * 2;
      const double *Kb = K + (size_t)bh * T * 4, *Bb = B + (size_t)bh * T * D;
      double *incb = inc + ((size_t)bh * NC + c) * P * D;
      memset(incb, 0, sizeof(double) * (size_t)P * D);
      cplx msuf = 1.0;
      for (int tl = L - 1; tl >= 0; --tl) {
        int t = c * L + tl;
        if (t >= T) continue; /* padded token: m=1, taps 0 */
        const cplx kp = ld_c(Kb + 4 * (size_t)t);
        const cplx kc = ld_c(Kb + 4 * (size_t)t + 2);
        const double *bpr = (t == 0) ? (Bprev ? Bprev + (size_t)bh * D : NULL)
                                     : Bb + (size_t)(t - 1) * D;
        const double *upr = (t == 0) ? (Uprev ? Uprev + (size_t)bh * P : NULL)
                                     : Ub + (size_t)(t - 1) * P;
        for (int p = 0; p < P; ++p) {
          double uc = Ub[(size_t)t * P + p];
          double upv = upr ? upr[p] : 0.0;
          for (int n = 0; n < N; ++n) {
            cplx v = uc * (msuf * (kc * ld_c(Bb + (size_t)t * D + 2 * n)));
            if (bpr) v += upv * (msuf * (kp * ld_c(bpr + 2 * n)));
            add_c(incb + (size_t)p * D + 2 * n, v);
          }
        }
        msuf *= ld_c(Mb + 2 * (size_t)t);
      }
      st_c(m_chunk + ((size_t)bh * NC + c) * 2, msuf);
    }
  }
}

/* Stage 2.  reference.py:1015-1056 (state_passing), :439-457.                */
void slx_oracle_state_passing(int BH, int NC, int P, int N, const double *inc,
                              const double *m_chunk, const double *init,
                              double *chunk_starts, double *final_state) {
  const int D = 2 * N;
  const size_t PN = (size_t)P * N;
#pragma omp parallel for schedule(dynamic)
  for (int bh = 0; bh < BH; ++bh) {
    cplx *z = (cplx *)calloc(PN, sizeof(cplx));
    if (init)
      for (size_t i = 0; i < PN; ++i)
        z[i] = ld_c(init + (size_t)bh * P * D + 2 * i);
    for (int c = 0; c < NC; ++c) {
      const cplx m = ld_c(m_chunk + ((size_t)bh * NC + c) * 2);
      const double *incb = inc + ((size_t)bh * NC + c) * P * D;
      double *st = chunk_starts + ((size_t)bh * NC + c) * P * D;
      for (size_t i = 0; i < PN; ++i) {
        st_c(st + 2 * i, z[i]);
        z[i] = m * z[i] + ld_c(incb + 2 * i);
      }
    }
    for (size_t i = 0; i < PN; ++i)
      st_c(final_state + (size_t)bh * P * D + 2 * i, z[i]);
    free(z);
  }
}

/* Stage 3.  reference.py:1059-1192 (chunk_scan) with the stable prefix split  */
/* of :466-491 (log-magnitude cumsum + unit-phase cumprod) and the segment     */
/* ratio formed directly as exp(lp_t - lp_s) (:1160-1166).                     */
/* Returns 1 if some |M| == 0 (the reference raises ValueError, :480-485).     */
int slx_oracle_chunk_scan(int BH, int T, int P, int N, int L, const double *U,
                          const double *M, const double *K, const double *B,
                          const double *C, const double *chunk_starts,
                          const double *Bprev, const double *Uprev, double *Y) {
  const int D = 2 * N;
  const int NC = (T + L - 1) / L;
  int bad = 0;
#pragma omp parallel for schedule(dynamic) collapse(2)
  for (int bh = 0; bh < BH; ++bh) {
    for (int c = 0; c < NC; ++c) {
      const double *Ub = U + (size_t)bh * T * P, *Mb = M + (size_t)bh * T * 2;
      const double *Kb = K + (size_t)bh * T * 4, *Bb = B + (size_t)bh * T * D;
      const double *Cb = C + (size_t)bh * T * D;
      const double *z0 = chunk_starts + ((size_t)bh * NC + c) * P * D;
      double *lp = (double *)calloc(L, sizeof(double));
      cplx *ph = (cplx *)calloc(L, sizeof(cplx));
      double lacc = 0.0;
      cplx pacc = 1.0;
      for (int tl = 0; tl < L; ++tl) {
        int t = c * L + tl;
        cplx m = (t < T) ? ld_c(Mb + 2 * (size_t)t) : 1.0;
        double mag = cabs(m);
        if (mag == 0.0) {
#pragma omp atomic write
          bad = 1;
          mag = 1.0;
        }
        lacc += log(mag);
        pacc *= m / mag;
        pacc /= cabs(pacc);
        lp[tl] = lacc;
        ph[tl] = pacc;
      }
      for (int tl = 0; tl < L; ++tl) {
        int t = c * L + tl;
        if (t >= T) break;
        double *y = Y + ((size_t)bh * T + t) * P;
        for (int p = 0; p < P; ++p) y[p] = 0.0;
        /* off-diagonal term: Re sum_n conj(c_t) prefix_t z0 */
        cplx pref = exp(lp[tl]) * ph[tl];
        for (int p = 0; p < P; ++p) {
          double acc = 0.0;
          for (int n = 0; n < N; ++n)
            acc += creal(conj(ld_c(Cb + (size_t)t * D + 2 * n)) * pref *
                         ld_c(z0 + (size_t)p * D + 2 * n));
          y[p] += acc;
        }
        for (int sl = 0; sl <= tl; ++sl) {
          int s = c * L + sl;
          cplx scale = exp(lp[tl] - lp[sl]) * ph[tl] * conj(ph[sl]);
          const cplx kp = ld_c(Kb + 4 * (size_t)s);
          const cplx kc = ld_c(Kb + 4 * (size_t)s + 2);
          const double *bpr = (s == 0) ? (Bprev ? Bprev + (size_t)bh * D : NULL)
                                       : Bb + (size_t)(s - 1) * D;
          const double *upr = (s == 0) ? (Uprev ? Uprev + (size_t)bh * P : NULL)
                                       : Ub + (size_t)(s - 1) * P;
          cplx sp = 0.0, sc = 0.0;
          for (int n = 0; n < N; ++n) {
            cplx cc = conj(ld_c(Cb + (size_t)t * D + 2 * n));
            if (bpr) sp += cc * (kp * ld_c(bpr + 2 * n));
            sc += cc * (kc * ld_c(Bb + (size_t)s * D + 2 * n));
          }
          double wp = creal(sp * scale), wc = creal(sc * scale);
          for (int p = 0; p < P; ++p) {
            if (upr) y[p] += wp * upr[p];
            y[p] += wc * Ub[(size_t)s * P + p];
          }
        }
      }
      free(lp);
      free(ph);
    }
  }
  return bad;
}

/* Staged forward = stage1 -> stage2 -> stage3.  reference.py:1195-1273.      */
int slx_oracle_v2x2ssd_fwd(int BH, int T, int P, int N, int L, const double *U,
                           const double *M, const double *K, const double *B,
                           const double *C, const double *init,
                           const double *Bprev, const double *Uprev, double *Y,
                           double *final_state, double *chunk_starts_out,
                           double *m_chunk_out) {
  const int D = 2 * N;
  const int NC = (T + L - 1) / L;
  size_t nstate = (size_t)BH * NC * P * D;
  double *inc = (double *)malloc(sizeof(double) * nstate);
  double *starts =
      chunk_starts_out ? chunk_starts_out : (double *)malloc(sizeof(double) * nstate);
  double *mch = m_chunk_out ? m_chunk_out
                            : (double *)malloc(sizeof(double) * (size_t)BH * NC * 2);
  slx_oracle_chunk_increment(BH, T, P, N, L, U, M, K, B, Bprev, Uprev, inc, mch);
  slx_oracle_state_passing(BH, NC, P, N, inc, mch, init, starts, final_state);
  int bad = slx_oracle_chunk_scan(BH, T, P, N, L, U, M, K, B, C, starts, Bprev,
                                  Uprev, Y);
  free(inc);
  if (!chunk_starts_out) free(starts);
  if (!m_chunk_out) free(mch);
  return bad;
}
