/* CPU oracle for KDA prefill, plain C.  TEST INFRASTRUCTURE ONLY: nothing in the product path links this file.
 *
 * Restates the token-by-token operator definition of the reference (kda/b200/reference.py:17-38):
 *   q, k <- x / max(||x||, 1e-6)                               reference.py:21-22
 *   a_t  <- lower_bound * sigmoid(exp(A_log) * (g_t + dt_bias)) reference.py:24
 *   beta <- sigmoid(beta)                                      reference.py:26
 *   S <- S * exp(a_t) (key rows);  S <- S + beta k (v - k^T S);  o = scale * q^T S    reference.py:33-36
 * The state is key-first [K][V] inside; kda_oracle_raw transposes value-first states on the way in and out
 * (reference.py:31,37).  Inputs arrive as fp32 copies of the caller's bf16 tensors (exact), the working precision is
 * REAL (double by default, -DKDA_ORACLE_FLOAT for float).  Sequence-head pairs are independent and run under OpenMP.
 * Pinned against tests/golden/ (outputs of the reference's reference.py) by tests/test_oracle.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifdef KDA_ORACLE_FLOAT
typedef float REAL;
#else
typedef double REAL;
#endif

#define KD 128

int kda_oracle_real_bytes(void) { return (int)sizeof(REAL); }

int kda_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the OpenMP thread count of later calls (n <= 0: every host CPU).  Launchers such as torch.distributed.run export
 * OMP_NUM_THREADS=1 to their children; a caller that wants all host cores for the CPU baseline has to say so. */
int kda_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n <= 0) n = omp_get_num_procs();
  omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* One (sequence, head): tokens t0..t1-1 of a packed [T][H][128] layout.  S is key-first [128][128], updated in place.
 * qn, kn: normalised; a: log-decay; b: beta in (0,1).  out may be NULL. */
static void recur_one(const REAL* qn, const REAL* kn, const float* v, const REAL* a, const REAL* b, REAL scale,
                      REAL* S, float* out, long t0, long t1, int H, int h) {
  REAL kS[KD], dec[KD];
  for (long t = t0; t < t1; t++) {
    const REAL* qt = qn + ((size_t)t * H + h) * KD;
    const REAL* kt = kn + ((size_t)t * H + h) * KD;
    const REAL* at = a + ((size_t)t * H + h) * KD;
    const float* vt = v + ((size_t)t * H + h) * KD;
    const REAL bt = b[(size_t)t * H + h];
    for (int i = 0; i < KD; i++) dec[i] = (REAL)exp((double)at[i]);
    for (int j = 0; j < KD; j++) kS[j] = 0;
    for (int i = 0; i < KD; i++) {                 /* reference.py:33-34 */
      REAL* Si = S + (size_t)i * KD;
      const REAL d = dec[i], ki = kt[i];
      for (int j = 0; j < KD; j++) { Si[j] *= d; kS[j] += ki * Si[j]; }
    }
    for (int j = 0; j < KD; j++) kS[j] = bt * ((REAL)vt[j] - kS[j]);
    for (int i = 0; i < KD; i++) {                 /* reference.py:35 */
      REAL* Si = S + (size_t)i * KD;
      const REAL ki = kt[i];
      for (int j = 0; j < KD; j++) Si[j] += ki * kS[j];
    }
    if (out) {                                     /* reference.py:36 */
      REAL o[KD];
      for (int j = 0; j < KD; j++) o[j] = 0;
      for (int i = 0; i < KD; i++) {
        const REAL* Si = S + (size_t)i * KD;
        const REAL qi = qt[i];
        for (int j = 0; j < KD; j++) o[j] += qi * Si[j];
      }
      float* ot = out + ((size_t)t * H + h) * KD;
      for (int j = 0; j < KD; j++) ot[j] = (float)(scale * o[j]);
    }
  }
}

/* Pre-activated front-end.  q,k,v,g [T][H][128] fp32, beta [T][H] fp32, state key-first [N][H][128][128] fp32
 * (init may be NULL = zeros), cu [N+1].  out [T][H][128] fp32, final [N][H][128][128] fp32 key-first. */
int kda_oracle_plain(const float* q, const float* k, const float* v, const float* g, const float* beta, double scale,
                     const float* init, const int64_t* cu, int N, int H, float* out, float* final_state) {
  const long T = cu[N];
  const size_t n_el = (size_t)T * H * KD;
  REAL* qn = (REAL*)malloc(n_el * sizeof(REAL));
  REAL* kn = (REAL*)malloc(n_el * sizeof(REAL));
  REAL* a = (REAL*)malloc(n_el * sizeof(REAL));
  REAL* b = (REAL*)malloc((size_t)T * H * sizeof(REAL));
  if (!qn || !kn || !a || !b) return -1;
  for (size_t i = 0; i < n_el; i++) { qn[i] = q[i]; kn[i] = k[i]; a[i] = g[i]; }
  for (size_t i = 0; i < (size_t)T * H; i++) b[i] = beta[i];
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int n = 0; n < N; n++)
    for (int h = 0; h < H; h++) {
      REAL* S = (REAL*)malloc(sizeof(REAL) * KD * KD);
      const size_t off = ((size_t)n * H + h) * KD * KD;
      for (int i = 0; i < KD * KD; i++) S[i] = init ? (REAL)init[off + i] : 0;
      recur_one(qn, kn, v, a, b, (REAL)scale, S, out, cu[n], cu[n + 1], H, h);
      if (final_state) for (int i = 0; i < KD * KD; i++) final_state[off + i] = (float)S[i];
      free(S);
    }
  free(qn); free(kn); free(a); free(b);
  return 0;
}

/* Raw-gate front-end.  q,k,v,g [T][H][128], beta [T][H]: fp32 copies of the bf16 inputs; A_log [H], dt_bias [H*128];
 * state VALUE-first [N][H][128 V][128 K] fp32.  out fp32 (the caller rounds to bf16). */
int kda_oracle_raw(const float* q, const float* k, const float* v, const float* g, const float* beta,
                   const float* A_log, const float* dt_bias, double scale, double lower_bound, const float* init,
                   const int64_t* cu, int N, int H, float* out, float* final_state) {
  const long T = cu[N];
  const size_t n_el = (size_t)T * H * KD;
  REAL* qn = (REAL*)malloc(n_el * sizeof(REAL));
  REAL* kn = (REAL*)malloc(n_el * sizeof(REAL));
  REAL* a = (REAL*)malloc(n_el * sizeof(REAL));
  REAL* b = (REAL*)malloc((size_t)T * H * sizeof(REAL));
  if (!qn || !kn || !a || !b) return -1;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < T * H; r++) {
    const int h = (int)(r % H);
    const float* qr = q + (size_t)r * KD;
    const float* kr = k + (size_t)r * KD;
    const float* gr = g + (size_t)r * KD;
    double sq = 0, sk = 0;
    for (int i = 0; i < KD; i++) { sq += (double)qr[i] * qr[i]; sk += (double)kr[i] * kr[i]; }
    const double nq = fmax(sqrt(sq), 1e-6), nk = fmax(sqrt(sk), 1e-6);       /* reference.py:21-22 */
    const double eA = exp((double)A_log[h]);
    for (int i = 0; i < KD; i++) {
      qn[(size_t)r * KD + i] = (REAL)(qr[i] / nq);
      kn[(size_t)r * KD + i] = (REAL)(kr[i] / nk);
      const double x = eA * ((double)gr[i] + (double)dt_bias[(size_t)h * KD + i]);
      a[(size_t)r * KD + i] = (REAL)(lower_bound / (1.0 + exp(-x)));         /* reference.py:24 */
    }
    b[r] = (REAL)(1.0 / (1.0 + exp(-(double)beta[r])));                      /* reference.py:26 */
  }
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int n = 0; n < N; n++)
    for (int h = 0; h < H; h++) {
      REAL* S = (REAL*)malloc(sizeof(REAL) * KD * KD);
      const size_t off = ((size_t)n * H + h) * KD * KD;
      for (int vi = 0; vi < KD; vi++)                                        /* reference.py:31 (transpose in) */
        for (int ki = 0; ki < KD; ki++) S[(size_t)ki * KD + vi] = init ? (REAL)init[off + (size_t)vi * KD + ki] : 0;
      recur_one(qn, kn, v, a, b, (REAL)scale, S, out, cu[n], cu[n + 1], H, h);
      if (final_state)
        for (int vi = 0; vi < KD; vi++)                                      /* reference.py:37 (transpose out) */
          for (int ki = 0; ki < KD; ki++) final_state[off + (size_t)vi * KD + ki] = (float)S[(size_t)ki * KD + vi];
      free(S);
    }
  free(qn); free(kn); free(a); free(b);
  return 0;
}
