/*
 * CPU oracle for the linear-recurrence path.  TEST INFRASTRUCTURE ONLY: the product
 * package never links, loads or calls this file; it exists so that the CUDA kernels
 * can be checked against a sequential restatement of the reference algorithm.
 *
 * Every routine restates, in plain C, the sequential-in-time / parallel-over-rows
 * loops of the reference project's CPU extension and the adjoint formulas of its
 * autograd rules.  Citations are paths inside the reference project.
 *
 * Convention shared by all routines (philtorch/csrc/host_recurN.cpp:254-255,
 * philtorch/lpv/recur.py:13-16): y[-1] := zi, y[t] = A[t] * y[t-1] + x[t]; the
 * coefficient with time index t multiplies the PREVIOUS state and A[0] multiplies zi.
 *
 * Pinning: checked against the reference extension itself (oracle/_ref) and against
 * the golden vectors in tests/golden/ that were produced by running the reference
 * (tests/golden/make_golden.py).
 *
 * Naming: <routine>_f32 / <routine>_f64.  Strides are implicit (row-major, dense).
 * `a_batched` / `A_batched` = 1 when the coefficient has a leading batch axis.
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define DEFINE_ALL(S, SUF)                                                                       \
  /* First-order LTI forward: philtorch/csrc/host_lti_recur.cpp:4-40 (out[t] += a*out[t-1]). */  \
  void CAT(oracle_lti_recur_, SUF)(int64_t B, int64_t T, const S *a, int a_batched,              \
                                   const S *zi, const S *x, S *y) {                              \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const S ab = a_batched ? a[b] : a[0];                                                      \
      S h = zi[b];                                                                               \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        h = x[b * T + t] + ab * h;                                                               \
        y[b * T + t] = h;                                                                        \
      }                                                                                          \
    }                                                                                            \
  }                                                                                              \
  /* First-order LTI adjoint: philtorch/lti/recur.py:25-59 and                                   \
     philtorch/__init__.py:115-148.  g[T-1] = gy[T-1], g[t] = a*g[t+1] + gy[t];                  \
     grad_x = g; grad_zi = a*g[0]; grad_a[b] = sum_t y[t-1]*g[t] (y[-1] = zi);                   \
     a shared: additionally summed over rows.  g_in (may be NULL) is an adjoint state            \
     entering from the right of the last sample: g[T-1] = gy[T-1] + g_in. */                     \
  void CAT(oracle_lti_recur_bwd_, SUF)(int64_t B, int64_t T, const S *a, int a_batched,          \
                                       const S *zi, const S *y, const S *gy, const S *g_in,      \
                                       S *grad_x, S *grad_a, S *grad_zi) {                       \
    if (!a_batched) grad_a[0] = 0;                                                               \
    for (int64_t b = 0; b < B; ++b) {                                                            \
      const S ab = a_batched ? a[b] : a[0];                                                      \
      S c = g_in ? g_in[b] : (S)0; /* c = a[t+1]*g[t+1] */                                       \
      S acc = 0;                                                                                 \
      for (int64_t t = T - 1; t >= 0; --t) {                                                     \
        const S g = gy[b * T + t] + c;                                                           \
        grad_x[b * T + t] = g;                                                                   \
        const S yp = (t == 0) ? zi[b] : y[b * T + t - 1];                                        \
        acc += yp * g;                                                                           \
        c = ab * g;                                                                              \
      }                                                                                          \
      grad_zi[b] = c;                                                                            \
      if (a_batched) grad_a[b] = acc; else grad_a[0] += acc;                                     \
    }                                                                                            \
  }                                                                                              \
  /* First-order LPV forward: philtorch/csrc/host_recurN.cpp:81-140 with N = 1 (the zero         \
     matrix padded in front at :254 means a[0] multiplies zi); same loop as                      \
     philtorch/lpv/recur.py:7-17.  a is (T,) when !a_batched, (B,T) otherwise. */                \
  void CAT(oracle_recur1_, SUF)(int64_t B, int64_t T, const S *a, int a_batched, const S *zi,    \
                                const S *x, S *y) {                                              \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const S *ab = a_batched ? a + b * T : a;                                                   \
      S h = zi[b];                                                                               \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        S sum = 0;                                                                               \
        sum += ab[t] * h;                                                                        \
        h = x[b * T + t] + sum;                                                                  \
        y[b * T + t] = h;                                                                        \
      }                                                                                          \
    }                                                                                            \
  }                                                                                              \
  /* First-order LPV adjoint: philtorch/lpv/ssm.py:64-99 with M = 1.                             \
     g[t] = a[t+1]*g[t+1] + gy[t]; grad_x = g; grad_zi = a[0]*g[0];                              \
     grad_a[b,t] = g[t]*y[t-1]; shared a: summed over rows (philtorch/__init__.py:62-65). */     \
  void CAT(oracle_recur1_bwd_, SUF)(int64_t B, int64_t T, const S *a, int a_batched,             \
                                    const S *zi, const S *y, const S *gy, const S *g_in,         \
                                    S *grad_x, S *grad_a, S *grad_zi) {                          \
    if (!a_batched) for (int64_t t = 0; t < T; ++t) grad_a[t] = 0;                               \
    /* rows are independent unless they share (and sum into) one coefficient gradient */         \
    _Pragma("omp parallel for if (a_batched)") for (int64_t b = 0; b < B; ++b) {                 \
      const S *ab = a_batched ? a + b * T : a;                                                   \
      S c = g_in ? g_in[b] : (S)0;                                                               \
      for (int64_t t = T - 1; t >= 0; --t) {                                                     \
        const S g = gy[b * T + t] + c;                                                           \
        grad_x[b * T + t] = g;                                                                   \
        const S yp = (t == 0) ? zi[b] : y[b * T + t - 1];                                        \
        if (a_batched) grad_a[b * T + t] = g * yp; else grad_a[t] += g * yp;                     \
        c = ab[t] * g;                                                                           \
      }                                                                                          \
      grad_zi[b] = c;                                                                            \
    }                                                                                            \
  }                                                                                              \
  /* 2x2 forward, LTI (A: (2,2) or (B,2,2)) and LPV (A: (T,2,2) or (B,T,2,2)):                   \
     philtorch/csrc/host_lti_recurN.cpp:4-61 and philtorch/csrc/host_recurN.cpp:81-140           \
     with N = 2: sum_i = A[i][0]*h0 + A[i][1]*h1 accumulated from 0, then added to x. */         \
  void CAT(oracle_recur2_, SUF)(int64_t B, int64_t T, const S *A, int A_batched, int A_timevar,  \
                                const S *zi, const S *x, S *y) {                                 \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const int64_t per_row = A_timevar ? T * 4 : 4;                                             \
      const S *Ab = A_batched ? A + b * per_row : A;                                             \
      S h0 = zi[b * 2], h1 = zi[b * 2 + 1];                                                      \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        const S *At = A_timevar ? Ab + t * 4 : Ab;                                               \
        S s0 = 0, s1 = 0;                                                                        \
        s0 += At[0] * h0; s0 += At[1] * h1;                                                      \
        s1 += At[2] * h0; s1 += At[3] * h1;                                                      \
        h0 = x[(b * T + t) * 2] + s0;                                                            \
        h1 = x[(b * T + t) * 2 + 1] + s1;                                                        \
        y[(b * T + t) * 2] = h0;                                                                 \
        y[(b * T + t) * 2 + 1] = h1;                                                             \
      }                                                                                          \
    }                                                                                            \
  }                                                                                              \
  /* 2x2 adjoint: philtorch/lti/ssm.py:67-96 (LTI) and philtorch/lpv/ssm.py:64-99 (LPV).         \
     g[t] = A[t+1]^T g[t+1] + gy[t]; grad_x = g; grad_zi = A[0]^T g[0];                          \
     grad_A[..][i][j] = g[t][i]*y[t-1][j], summed over t when A is time-invariant and            \
     over rows when A has no batch axis. */                                                      \
  void CAT(oracle_recur2_bwd_, SUF)(int64_t B, int64_t T, const S *A, int A_batched,             \
                                    int A_timevar, const S *zi, const S *y, const S *gy,         \
                                    const S *g_in, S *grad_x, S *grad_A, S *grad_zi) {           \
    const int64_t per_row = A_timevar ? T * 4 : 4;                                               \
    const int64_t nA = A_batched ? B * per_row : per_row;                                        \
    for (int64_t i = 0; i < nA; ++i) grad_A[i] = 0;                                              \
    for (int64_t b = 0; b < B; ++b) {                                                            \
      const S *Ab = A_batched ? A + b * per_row : A;                                             \
      S *gAb = A_batched ? grad_A + b * per_row : grad_A;                                        \
      S c0 = g_in ? g_in[b * 2] : (S)0, c1 = g_in ? g_in[b * 2 + 1] : (S)0;                      \
      for (int64_t t = T - 1; t >= 0; --t) {                                                     \
        const S *At = A_timevar ? Ab + t * 4 : Ab;                                               \
        S *gAt = A_timevar ? gAb + t * 4 : gAb;                                                  \
        const S g0 = gy[(b * T + t) * 2] + c0, g1 = gy[(b * T + t) * 2 + 1] + c1;                \
        grad_x[(b * T + t) * 2] = g0;                                                            \
        grad_x[(b * T + t) * 2 + 1] = g1;                                                        \
        const S y0 = (t == 0) ? zi[b * 2] : y[(b * T + t - 1) * 2];                              \
        const S y1 = (t == 0) ? zi[b * 2 + 1] : y[(b * T + t - 1) * 2 + 1];                      \
        gAt[0] += g0 * y0; gAt[1] += g0 * y1; gAt[2] += g1 * y0; gAt[3] += g1 * y1;              \
        c0 = At[0] * g0 + At[2] * g1;                                                            \
        c1 = At[1] * g0 + At[3] * g1;                                                            \
      }                                                                                          \
      grad_zi[b * 2] = c0;                                                                       \
      grad_zi[b * 2 + 1] = c1;                                                                   \
    }                                                                                            \
  }                                                                                              \
  /* One second-order section in transposed direct form II, scalar in / scalar out:              \
     philtorch/lti/filtering.py:304-317 builds A^T = [[-a1,1],[-a2,0]], B = [b1-b0*a1,           \
     b2-b0*a2], D = b0, out_idx = 0; philtorch/lti/ssm.py:466-504 runs h[t] = A^T h[t-1] +       \
     B*x[t], delays it by one sample and adds D*x.  b: (3,) or (B,3); a: (2,) or (B,2);          \
     zi: (B,2); zf (may be NULL): (B,2) final state. */                                          \
  void CAT(oracle_biquad_tdf2_, SUF)(int64_t B, int64_t T, const S *bc, const S *ac,             \
                                     int batched, const S *zi, const S *x, S *y, S *zf) {        \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const S *bb = batched ? bc + b * 3 : bc;                                                   \
      const S *aa = batched ? ac + b * 2 : ac;                                                   \
      const S B0 = bb[1] - bb[0] * aa[0], B1 = bb[2] - bb[0] * aa[1];                            \
      S h0 = zi ? zi[b * 2] : (S)0, h1 = zi ? zi[b * 2 + 1] : (S)0;                              \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        const S xt = x[b * T + t];                                                               \
        y[b * T + t] = h0 + bb[0] * xt;                                                          \
        S s0 = 0, s1 = 0;                                                                        \
        s0 += (-aa[0]) * h0; s0 += (S)1 * h1;                                                    \
        s1 += (-aa[1]) * h0; s1 += (S)0 * h1;                                                    \
        h0 = xt * B0 + s0;                                                                       \
        h1 = xt * B1 + s1;                                                                       \
      }                                                                                          \
      if (zf) { zf[b * 2] = h0; zf[b * 2 + 1] = h1; }                                            \
    }                                                                                            \
  }                                                                                              \
  /* Adjoint of that section: what autograd derives in the reference through the glue of         \
     philtorch/lti/filtering.py:304-317 and philtorch/lti/ssm.py:466-504 and the rule of         \
     LTIMatrixRecurrence (philtorch/lti/ssm.py:67-96), written out sequentially.  With           \
     M = [[-a1,1],[-a2,0]], Bv = [b1-b0*a1, b2-b0*a2] and l[t] the adjoint of the state h[t]:    \
       l[T-1] = gzf,  l[t] = M^T l[t+1] + [gy[t+1], 0];   grad_x[t] = b0*gy[t] + Bv.l[t];        \
       grad_b1 = sum l0[t]*x[t], grad_b2 = sum l1[t]*x[t],                                       \
       grad_b0 = sum gy[t]*x[t] - a1*grad_b1 - a2*grad_b2;                                       \
       grad_a1 = -sum l0[t]*(h0[t-1] + b0*x[t]), grad_a2 = -sum l1[t]*(h0[t-1] + b0*x[t])        \
       (through M: -l0[t]*h0[t-1], through Bv: -b0*l0[t]*x[t]);  grad_zi = M^T l[0] + [gy[0],0]. \
     h0[t-1] is recomputed by running the section forward first.  Sums are accumulated in        \
     double; shared coefficients: summed over the rows as well.  gzf, grad_zi may be NULL. */    \
  void CAT(oracle_biquad_tdf2_bwd_, SUF)(int64_t B, int64_t T, const S *bc, const S *ac,         \
                                         int batched, const S *zi, const S *x, const S *gy,      \
                                         const S *gzf, S *grad_x, S *grad_b, S *grad_a,          \
                                         S *grad_zi) {                                           \
    double *acc = (double *)calloc((size_t)B * 5, sizeof(double));                               \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const S *bb = batched ? bc + b * 3 : bc;                                                   \
      const S *aa = batched ? ac + b * 2 : ac;                                                   \
      const S B0 = bb[1] - bb[0] * aa[0], B1 = bb[2] - bb[0] * aa[1];                            \
      S *h0prev = (S *)malloc((size_t)T * sizeof(S)); /* h0[t-1] for every t */                  \
      S h0 = zi ? zi[b * 2] : (S)0, h1 = zi ? zi[b * 2 + 1] : (S)0;                              \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        const S xt = x[b * T + t];                                                               \
        h0prev[t] = h0;                                                                          \
        const S n0 = xt * B0 + ((-aa[0]) * h0 + h1);                                             \
        const S n1 = xt * B1 + (-aa[1]) * h0;                                                    \
        h0 = n0; h1 = n1;                                                                        \
      }                                                                                          \
      S l0 = gzf ? gzf[b * 2] : (S)0, l1 = gzf ? gzf[b * 2 + 1] : (S)0;                          \
      double sgx = 0, s0x = 0, s1x = 0, s0y = 0, s1y = 0;                                        \
      for (int64_t t = T - 1; t >= 0; --t) {                                                     \
        const S xt = x[b * T + t], gt = gy[b * T + t];                                           \
        grad_x[b * T + t] = bb[0] * gt + (B0 * l0 + B1 * l1);                                    \
        const S yt = h0prev[t] + bb[0] * xt;                                                     \
        sgx += (double)gt * xt; s0x += (double)l0 * xt; s1x += (double)l1 * xt;                  \
        s0y += (double)l0 * yt; s1y += (double)l1 * yt;                                          \
        const S m0 = (-aa[0]) * l0 + (-aa[1]) * l1 + gt; /* M^T l + [gy[t], 0] */                \
        const S m1 = l0;                                                                         \
        l0 = m0; l1 = m1;                                                                        \
      }                                                                                          \
      if (grad_zi) { grad_zi[b * 2] = l0; grad_zi[b * 2 + 1] = l1; }                             \
      acc[b * 5] = sgx - (double)aa[0] * s0x - (double)aa[1] * s1x;                              \
      acc[b * 5 + 1] = s0x; acc[b * 5 + 2] = s1x; acc[b * 5 + 3] = -s0y; acc[b * 5 + 4] = -s1y;  \
      free(h0prev);                                                                              \
    }                                                                                            \
    if (batched) {                                                                               \
      for (int64_t b = 0; b < B; ++b) {                                                          \
        for (int i = 0; i < 3; ++i) grad_b[b * 3 + i] = (S)acc[b * 5 + i];                       \
        for (int i = 0; i < 2; ++i) grad_a[b * 2 + i] = (S)acc[b * 5 + 3 + i];                   \
      }                                                                                          \
    } else {                                                                                     \
      double tot[5] = {0, 0, 0, 0, 0};                                                           \
      for (int64_t b = 0; b < B; ++b) for (int i = 0; i < 5; ++i) tot[i] += acc[b * 5 + i];      \
      for (int i = 0; i < 3; ++i) grad_b[i] = (S)tot[i];                                         \
      for (int i = 0; i < 2; ++i) grad_a[i] = (S)tot[3 + i];                                     \
    }                                                                                            \
    free(acc);                                                                                   \
  }

DEFINE_ALL(float, f32)
DEFINE_ALL(double, f64)

/*
 * Complex first-order recurrences (complex64 / complex128, C99 _Complex = interleaved {re, im}).
 * The reference dispatches its first-order ops over complex types as well
 * (philtorch/csrc/host_lti_recur.cpp:61-78, philtorch/csrc/host_recurN.cpp:259-281) and its
 * autograd rule conjugates the coefficient and the saved states
 * (philtorch/lti/recur.py:31-57: recursion on a.conj_physical(), grad_init = g[0]*conj(a),
 * grad_a = vecdot(y_prev, g) = sum conj(y[t-1])*g[t]).
 */
#include <complex.h>

#define DEFINE_CX(S, SUF, CONJ)                                                                  \
  void CAT(oracle_lti_recur_, SUF)(int64_t B, int64_t T, const S *a, int a_batched,              \
                                   const S *zi, const S *x, S *y) {                              \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const S ab = a_batched ? a[b] : a[0];                                                      \
      S h = zi[b];                                                                               \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        h = x[b * T + t] + ab * h;                                                               \
        y[b * T + t] = h;                                                                        \
      }                                                                                          \
    }                                                                                            \
  }                                                                                              \
  void CAT(oracle_lti_recur_bwd_, SUF)(int64_t B, int64_t T, const S *a, int a_batched,          \
                                       const S *zi, const S *y, const S *gy, const S *g_in,      \
                                       S *grad_x, S *grad_a, S *grad_zi) {                       \
    if (!a_batched) grad_a[0] = 0;                                                               \
    for (int64_t b = 0; b < B; ++b) {                                                            \
      const S ab = CONJ(a_batched ? a[b] : a[0]);                                                \
      S c = g_in ? g_in[b] : (S)0;                                                               \
      S acc = 0;                                                                                 \
      for (int64_t t = T - 1; t >= 0; --t) {                                                     \
        const S g = gy[b * T + t] + c;                                                           \
        grad_x[b * T + t] = g;                                                                   \
        const S yp = (t == 0) ? zi[b] : y[b * T + t - 1];                                        \
        acc += CONJ(yp) * g;                                                                     \
        c = ab * g;                                                                              \
      }                                                                                          \
      grad_zi[b] = c;                                                                            \
      if (a_batched) grad_a[b] = acc; else grad_a[0] += acc;                                     \
    }                                                                                            \
  }                                                                                              \
  void CAT(oracle_recur1_, SUF)(int64_t B, int64_t T, const S *a, int a_batched, const S *zi,    \
                                const S *x, S *y) {                                              \
    _Pragma("omp parallel for") for (int64_t b = 0; b < B; ++b) {                                \
      const S *ab = a_batched ? a + b * T : a;                                                   \
      S h = zi[b];                                                                               \
      for (int64_t t = 0; t < T; ++t) {                                                          \
        h = x[b * T + t] + ab[t] * h;                                                            \
        y[b * T + t] = h;                                                                        \
      }                                                                                          \
    }                                                                                            \
  }                                                                                              \
  void CAT(oracle_recur1_bwd_, SUF)(int64_t B, int64_t T, const S *a, int a_batched,             \
                                    const S *zi, const S *y, const S *gy, const S *g_in,         \
                                    S *grad_x, S *grad_a, S *grad_zi) {                          \
    if (!a_batched) for (int64_t t = 0; t < T; ++t) grad_a[t] = 0;                               \
    /* rows are independent unless they share (and sum into) one coefficient gradient */         \
    _Pragma("omp parallel for if (a_batched)") for (int64_t b = 0; b < B; ++b) {                 \
      const S *ab = a_batched ? a + b * T : a;                                                   \
      S c = g_in ? g_in[b] : (S)0;                                                               \
      for (int64_t t = T - 1; t >= 0; --t) {                                                     \
        const S g = gy[b * T + t] + c;                                                           \
        grad_x[b * T + t] = g;                                                                   \
        const S yp = (t == 0) ? zi[b] : y[b * T + t - 1];                                        \
        if (a_batched) grad_a[b * T + t] = g * CONJ(yp); else grad_a[t] += g * CONJ(yp);         \
        c = CONJ(ab[t]) * g;                                                                     \
      }                                                                                          \
      grad_zi[b] = c;                                                                            \
    }                                                                                            \
  }

DEFINE_CX(float _Complex, c64, conjf)
DEFINE_CX(double _Complex, c128, conj)
