// Scan-engine policies for ONE second-order section in transposed direct form II, scalar in and
// scalar out, with the state-space glue of the reference folded into the kernel:
//     y[t]  = h0[t-1] + b0 x[t]
//     h0[t] = -a1 h0[t-1] + h1[t-1] + (b1 - b0 a1) x[t]
//     h1[t] = -a2 h0[t-1]           + (b2 - b0 a2) x[t]
// (philtorch/lti/filtering.py:304-317 builds A^T = [[-a1,1],[-a2,0]], B = b[1:] - b0 a, D = b0 and
// philtorch/lti/ssm.py:466-504 materialises B x, runs the 2x2 recurrence, delays it by one sample
// and adds D x: five extra passes over (B,T,2) tensors that never leave the chip here.)
//
// Adjoint (lam[t] = dL/dh[t], M = A^T):
//     lam[t-1] = M^T lam[t] + e0 gy[t],   lam[T-1] = grad of the final state (0 if unused)
//     grad_x[t] = b0 gy[t] + B . lam[t]
//     grad_b0 = sum gy x - a1 sum x lam0 - a2 sum x lam1,  grad_b1 = sum x lam0,  grad_b2 = sum x lam1
//     grad_a1 = -sum y lam0,  grad_a2 = -sum y lam1        (y[t] = h0[t-1] + b0 x[t] absorbs both paths)
//     grad_zi = lam[-1]
// so the backward pass reads gy, x and y only: no state is stored or recomputed.
#pragma once
#include "second_order.cuh"

namespace ptb {

// The loops over a thread's 16-byte units are unrolled PTB_BQ_UNROLL times, not completely: the
// samples stay in shared memory and the hot code stays small enough for the instruction caches
// (a kernel unrolled over all its samples waits for instruction fetches instead of data).
#ifndef PTB_BQ_UNROLL
#define PTB_BQ_UNROLL 1
#endif
#define PTB_PRAGMA_(x) _Pragma(#x)
#define PTB_UNROLL_(n) PTB_PRAGMA_(unroll n)

// Derived constants of a row's section {b0, b1 - b0 a1, b2 - b0 a2, -a1, -a2}: computed once per tile
// by the DMA warp (row_constants) and read from the stage by every thread.
template <class S>
struct BqCoef {
  S b0, B0, B1, na1, na2;
  static __device__ __forceinline__ void derive(const S* b, int64_t bs, const S* a, int64_t as, int64_t row,
                                                S* out) {
    const S* pb = b + row * bs;
    const S* pa = a + row * as;
    const S b0 = __ldg(pb), b1 = __ldg(pb + 1), b2 = __ldg(pb + 2), a1 = __ldg(pa), a2 = __ldg(pa + 1);
    out[0] = b0; out[1] = b1 - b0 * a1; out[2] = b2 - b0 * a2; out[3] = -a1; out[4] = -a2;
  }
  __device__ __forceinline__ void load(const unsigned char* rowc) {
    const S* q = reinterpret_cast<const S*>(rowc);
    b0 = q[0]; B0 = q[1]; B1 = q[2]; na1 = q[3]; na2 = q[4];
  }
};

// M^n for a 2x2 matrix by binary powering (n a compile-time constant): the linear part of the map
// of a thread that owns n samples of a time-invariant section.
template <class S, int N>
__device__ __forceinline__ void mat2_power(const S* m, S* out) {
  S r[4] = {S(1), S(0), S(0), S(1)};
  S b[4] = {m[0], m[1], m[2], m[3]};
  bool first = true;
#pragma unroll
  for (int bit = 0; (1 << bit) <= N; ++bit) {
    if (N & (1 << bit)) {
      if (first) { r[0] = b[0]; r[1] = b[1]; r[2] = b[2]; r[3] = b[3]; first = false; }
      else {
        const S t0 = b[0] * r[0] + b[1] * r[2], t1 = b[0] * r[1] + b[1] * r[3];
        const S t2 = b[2] * r[0] + b[3] * r[2], t3 = b[2] * r[1] + b[3] * r[3];
        r[0] = t0; r[1] = t1; r[2] = t2; r[3] = t3;
      }
    }
    const S q0 = b[0] * b[0] + b[1] * b[2], q1 = b[0] * b[1] + b[1] * b[3];
    const S q2 = b[2] * b[0] + b[3] * b[2], q3 = b[2] * b[1] + b[3] * b[3];
    b[0] = q0; b[1] = q1; b[2] = q2; b[3] = q3;
  }
  out[0] = r[0]; out[1] = r[1]; out[2] = r[2]; out[3] = r[3];
}

template <class S>
struct BqFwdParams {
  const S* b; int64_t b_stride;   // 3 or 0
  const S* a; int64_t a_stride;   // 2 or 0
  const S* zi;                    // optional (B,2)
  const S* x;
  S* y;
  S* zf;                          // optional (B,2)
  int64_t T;
};

template <class S, int CH, int STAGES_, int MIN_CTAS_, int NT_>
struct BqFwd : MatAffine<S> {
  using Alg = MatAffine<S>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = BqFwdParams<S>;
  static constexpr int V = Vec16<S>::V;
  static constexpr int NT = NT_;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = false;
  static constexpr bool HAS_PARTIAL = false;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int X_OFF = 0;
  using Scalar = S;
  static constexpr int NROWC = 5;
  static constexpr int ROWC_OFF = TILE * (int)sizeof(S);
  static constexpr int STAGE_BYTES = ROWC_OFF + 128;
  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    BqCoef<S>::derive(p.b, p.b_stride, p.a, p.a_stride, row, out);
  }

  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    io.load(X_OFF, p.x + row * p.T + t0, bytes);
    io.store(X_OFF, p.y + row * p.T + t0, bytes);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s = Alg::zero_state();
    if (p.zi) { s.v[0] = __ldg(p.zi + row * 2); s.v[1] = __ldg(p.zi + row * 2 + 1); }
    return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.zf) { p.zf[row * 2] = s.v[0]; p.zf[row * 2 + 1] = s.v[1]; }
  }
  static __device__ __forceinline__ int load_x(const unsigned char* stage, int tpos, int nvalid, S* x) {
    const int p0 = tpos * SPT;
    int nv = nvalid - p0;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    const unsigned char* px = stage + X_OFF + (size_t)p0 * sizeof(S);
#pragma unroll
    for (int c = 0; c < CH; ++c) VecIO<S, V>::ld(px + 16 * c, &x[c * V]);
    return nv;
  }
  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t, int nvalid) {
    BqCoef<S> k;
    k.load(stage + ROWC_OFF);
    Map m = Alg::identity();
    if (nvalid - tpos * SPT >= SPT) {
      // full thread: offsets by the recurrence, linear part M^SPT by binary powering
      const unsigned char* px = stage + X_OFF + (size_t)tpos * SPT * sizeof(S);
      S s0 = S(0), s1 = S(0);
      PTB_UNROLL_(PTB_BQ_UNROLL)
      for (int c = 0; c < CH; ++c) {
        S xv[V];
        VecIO<S, V>::ld(px + 16 * c, xv);
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const S t = s1 + k.B0 * xv[q];   // off the chain through s0
          s1 = k.na2 * s0 + k.B1 * xv[q];
          s0 = k.na1 * s0 + t;
        }
      }
      const S M[4] = {k.na1, S(1), k.na2, S(0)};
      mat2_power<S, SPT>(M, m.v);
      m.v[4] = s0; m.v[5] = s1;
      return m;
    }
    S x[SPT];
    const int nv = load_x(stage, tpos, nvalid, x);
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      if (j < nv) {
        Map n;   // M = [na1 1; na2 0]
        n.v[0] = k.na1 * m.v[0] + m.v[2];
        n.v[1] = k.na1 * m.v[1] + m.v[3];
        n.v[2] = k.na2 * m.v[0];
        n.v[3] = k.na2 * m.v[1];
        n.v[4] = k.na1 * m.v[4] + m.v[5] + k.B0 * x[j];
        n.v[5] = k.na2 * m.v[4] + k.B1 * x[j];
        m = n;
      }
    }
    return m;
  }
  // FULL: every sample of the thread is valid, so the per-sample guards compile away
  template <bool FULL>
  static __device__ __forceinline__ void replay(const BqCoef<S>& k, S h0, S h1, int nv, S* x) {
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      if (FULL || j < nv) {
        const S xj = x[j];
        x[j] = h0 + k.b0 * xj;
        const S t = h1 + k.B0 * xj;   // off the chain through h0
        h1 = k.na2 * h0 + k.B1 * xj;
        h0 = k.na1 * h0 + t;
      }
    }
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t, int nvalid) {
    BqCoef<S> k;
    k.load(stage + ROWC_OFF);
    unsigned char* px = stage + X_OFF + (size_t)tpos * SPT * sizeof(S);
    if (nvalid - tpos * SPT >= SPT) {
      S h0 = in.v[0], h1 = in.v[1];
      PTB_UNROLL_(PTB_BQ_UNROLL)
      for (int c = 0; c < CH; ++c) {
        S xv[V];
        VecIO<S, V>::ld(px + 16 * c, xv);
#pragma unroll
        for (int q = 0; q < V; ++q) {
          const S xj = xv[q];
          xv[q] = h0 + k.b0 * xj;
          const S t = h1 + k.B0 * xj;   // off the chain through h0
          h1 = k.na2 * h0 + k.B1 * xj;
          h0 = k.na1 * h0 + t;
        }
        VecIO<S, V>::st(px + 16 * c, xv);
      }
    } else {
      S x[SPT];
      const int nv = load_x(stage, tpos, nvalid, x);
      replay<false>(k, in.v[0], in.v[1], nv, x);
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<S, V>::st(px + 16 * c, &x[c * V]);
    }
    Partial r; r.v[0] = S(0); return r;
  }
};

template <class S>
struct BqBwdParams {
  const S* b; int64_t b_stride;
  const S* a; int64_t a_stride;
  const S* x;
  const S* y;        // forward output; needed only when coefficient gradients are wanted
  const S* gy;
  const S* g_in;     // optional (B,2): gradient w.r.t. the final state
  S* grad_x;
  S* grad_zi;        // optional (B,2)
  int64_t T;
  int want_coef;
};

template <class S, int CH, int STAGES_, int MIN_CTAS_, int NT_>
struct BqBwd : MatAffine<S> {
  using Alg = MatAffine<S>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 5>;   // sum gy x, sum x lam0, sum x lam1, sum y lam0, sum y lam1
  using Params = BqBwdParams<S>;
  static constexpr int V = Vec16<S>::V;
  static constexpr int NT = NT_;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = true;
  static constexpr bool HAS_PARTIAL = true;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int SLOT = TILE * (int)sizeof(S);
  static constexpr int G_OFF = 0;          // gy in, grad_x out
  static constexpr int X_OFF = SLOT;       // x in
  static constexpr int Y_OFF = 2 * SLOT;   // y in
  using Scalar = S;
  static constexpr int NROWC = 5;
  static constexpr int ROWC_OFF = 3 * SLOT;
  static constexpr int STAGE_BYTES = ROWC_OFF + 128;
  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    BqCoef<S>::derive(p.b, p.b_stride, p.a, p.a_stride, row, out);
  }

  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    io.load(G_OFF, p.gy + row * p.T + t0, bytes);
    if (p.want_coef) {
      io.load(X_OFF, p.x + row * p.T + t0, bytes);
      io.load(Y_OFF, p.y + row * p.T + t0, bytes);
    }
    io.store(G_OFF, p.grad_x + row * p.T + t0, bytes);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s = Alg::zero_state();
    if (p.g_in) { s.v[0] = __ldg(p.g_in + row * 2); s.v[1] = __ldg(p.g_in + row * 2 + 1); }
    return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.grad_zi) { p.grad_zi[row * 2] = s.v[0]; p.grad_zi[row * 2 + 1] = s.v[1]; }
  }
  static __device__ __forceinline__ int load_slot(const unsigned char* stage, int off, int tpos, int nvalid, S* r) {
    const int p0 = tpos * SPT;
    int nv = nvalid - p0;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    const unsigned char* q = stage + off + (size_t)p0 * sizeof(S);
#pragma unroll
    for (int c = 0; c < CH; ++c) VecIO<S, V>::ld(q + 16 * c, &r[c * V]);
    return nv;
  }
  // map over lam (time descending): lam' = M^T lam + e0 gy,  M^T = [na1 na2; 1 0]
  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t, int nvalid) {
    BqCoef<S> k;
    k.load(stage + ROWC_OFF);
    Map m = Alg::identity();
    if (nvalid - tpos * SPT >= SPT) {
      const unsigned char* pg = stage + G_OFF + (size_t)tpos * SPT * sizeof(S);
      S s0 = S(0), s1 = S(0);
      PTB_UNROLL_(PTB_BQ_UNROLL)
      for (int c = CH - 1; c >= 0; --c) {
        S gv[V];
        VecIO<S, V>::ld(pg + 16 * c, gv);
#pragma unroll
        for (int q = V - 1; q >= 0; --q) {
          const S t = k.na2 * s1 + gv[q];   // off the chain through s0
          s1 = s0;
          s0 = k.na1 * s0 + t;
        }
      }
      const S Mt[4] = {k.na1, k.na2, S(1), S(0)};
      mat2_power<S, SPT>(Mt, m.v);
      m.v[4] = s0; m.v[5] = s1;
      return m;
    }
    S g[SPT];
    const int nv = load_slot(stage, G_OFF, tpos, nvalid, g);
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      if (j < nv) {
        Map n;
        n.v[0] = k.na1 * m.v[0] + k.na2 * m.v[2];
        n.v[1] = k.na1 * m.v[1] + k.na2 * m.v[3];
        n.v[2] = m.v[0];
        n.v[3] = m.v[1];
        n.v[4] = k.na1 * m.v[4] + k.na2 * m.v[5] + g[j];
        n.v[5] = m.v[4];
        m = n;
      }
    }
    return m;
  }
  template <bool FULL, bool COEF>
  static __device__ __forceinline__ Partial replay(const BqCoef<S>& k, S l0, S l1, int nv, S* g, const S* x,
                                                   const S* y) {
    Partial acc;
#pragma unroll
    for (int i = 0; i < 5; ++i) acc.v[i] = S(0);
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      if (FULL || j < nv) {
        const S gj = g[j];
        g[j] = k.b0 * gj + k.B0 * l0 + k.B1 * l1;
        if (COEF) {
          acc.v[0] += gj * x[j];
          acc.v[1] += x[j] * l0;
          acc.v[2] += x[j] * l1;
          acc.v[3] += y[j] * l0;
          acc.v[4] += y[j] * l1;
        }
        const S t = k.na2 * l1 + gj;   // off the chain through l0
        l1 = l0;
        l0 = k.na1 * l0 + t;
      }
    }
    return acc;
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t, int nvalid) {
    BqCoef<S> k;
    k.load(stage + ROWC_OFF);
    unsigned char* pg = stage + G_OFF + (size_t)tpos * SPT * sizeof(S);
    if (nvalid - tpos * SPT >= SPT) {
      const unsigned char* pxs = stage + X_OFF + (size_t)tpos * SPT * sizeof(S);
      const unsigned char* pys = stage + Y_OFF + (size_t)tpos * SPT * sizeof(S);
      S l0 = in.v[0], l1 = in.v[1];
      S a0 = S(0), a1 = S(0), a2 = S(0), a3 = S(0), a4 = S(0);
      if (p.want_coef) {
        PTB_UNROLL_(PTB_BQ_UNROLL)
        for (int c = CH - 1; c >= 0; --c) {
          S gv[V], xv[V], yv[V];
          VecIO<S, V>::ld(pg + 16 * c, gv);
          VecIO<S, V>::ld(pxs + 16 * c, xv);
          VecIO<S, V>::ld(pys + 16 * c, yv);
#pragma unroll
          for (int q = V - 1; q >= 0; --q) {
            const S gj = gv[q];
            gv[q] = k.b0 * gj + k.B0 * l0 + k.B1 * l1;
            a0 += gj * xv[q];
            a1 += xv[q] * l0;
            a2 += xv[q] * l1;
            a3 += yv[q] * l0;
            a4 += yv[q] * l1;
            const S t = k.na2 * l1 + gj;   // off the chain through l0
            l1 = l0;
            l0 = k.na1 * l0 + t;
          }
          VecIO<S, V>::st(pg + 16 * c, gv);
        }
      } else {
        PTB_UNROLL_(PTB_BQ_UNROLL)
        for (int c = CH - 1; c >= 0; --c) {
          S gv[V];
          VecIO<S, V>::ld(pg + 16 * c, gv);
#pragma unroll
          for (int q = V - 1; q >= 0; --q) {
            const S gj = gv[q];
            gv[q] = k.b0 * gj + k.B0 * l0 + k.B1 * l1;
            const S t = k.na2 * l1 + gj;
            l1 = l0;
            l0 = k.na1 * l0 + t;
          }
          VecIO<S, V>::st(pg + 16 * c, gv);
        }
      }
      Partial r;
      r.v[0] = a0; r.v[1] = a1; r.v[2] = a2; r.v[3] = a3; r.v[4] = a4;
      return r;
    }
    S g[SPT], x[SPT], y[SPT];
    const int nv = load_slot(stage, G_OFF, tpos, nvalid, g);
    Partial acc;
    if (p.want_coef) {
      load_slot(stage, X_OFF, tpos, nvalid, x);
      load_slot(stage, Y_OFF, tpos, nvalid, y);
      acc = nv == SPT ? replay<true, true>(k, in.v[0], in.v[1], nv, g, x, y)
                      : replay<false, true>(k, in.v[0], in.v[1], nv, g, x, y);
    } else {
      acc = nv == SPT ? replay<true, false>(k, in.v[0], in.v[1], nv, g, x, y)
                      : replay<false, false>(k, in.v[0], in.v[1], nv, g, x, y);
    }
#pragma unroll
    for (int c = 0; c < CH; ++c) VecIO<S, V>::st(pg + 16 * c, &g[c * V]);
    return acc;
  }
};

}  // namespace ptb
