// Scan-engine policy for the dense N x N recurrence, 2 < N <= NMAX,
//     h[t] = A[t] h[t-1] + x[t],   h[-1] = zi,   A row-major (N,N), x and h (N,)
// forward (REV = false) and the scan its adjoint needs (REV = true)
//     g[t] = gy[t] + c[t+1],  c[t] = A[t]^T g[t],  c[T] = g_in        (output g, final c[0])
// i.e. the reference's recurN / lti_recurN ops (philtorch/csrc/host_recurN.cpp:81-140,236-281,
// philtorch/csrc/host_lti_recurN.cpp:63-108; the reference has no GPU kernel for N > 2) and the
// scan inside its adjoint rules (philtorch/lpv/ssm.py:64-99, philtorch/lti/ssm.py:67-96).  The
// outer products g[t] (x) h[t-1] of grad_A are left to the caller: for time-invariant A they are a
// (N x T)(T x N) contraction per row, which belongs on the tensor cores of a library GEMM.
//
// N is a run-time value; matrices and vectors are held in registers padded with zeros to NMAX, so
// the arithmetic needs no predicates (padded rows and columns stay exactly zero).  A may vary per
// sample (a_t_stride = N*N, staged with the tile) or be constant along time (a_t_stride = 0,
// carried with the stage as row constants).  Maps are full affine maps (NMAX^2 + NMAX scalars):
// this policy is about coverage of larger state dimensions, not about the last 20 % of bandwidth.
#pragma once
#include "first_order.cuh"

namespace ptb {

template <class S, int NMAX>
struct MatNAffine {
  static constexpr int NN = NMAX * NMAX;
  using Map = Pod<S, NN + NMAX>;   // M row-major, then the offset vector
  using State = Pod<S, NMAX>;
  static __device__ __forceinline__ Map identity() {
    Map m;
#pragma unroll
    for (int i = 0; i < NMAX; ++i)
#pragma unroll
      for (int j = 0; j < NMAX; ++j) m.v[i * NMAX + j] = (i == j) ? S(1) : S(0);
#pragma unroll
    for (int i = 0; i < NMAX; ++i) m.v[NN + i] = S(0);
    return m;
  }
  static __device__ __forceinline__ State zero_state() {
    State s;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) s.v[i] = S(0);
    return s;
  }
  static __device__ __forceinline__ Map const_map(const State& s) {
    Map m;
#pragma unroll
    for (int i = 0; i < NN; ++i) m.v[i] = S(0);
#pragma unroll
    for (int i = 0; i < NMAX; ++i) m.v[NN + i] = s.v[i];
    return m;
  }
  // apply `f`, then `g`
  static __device__ __forceinline__ Map compose(const Map& f, const Map& g) {
    Map m;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) {
#pragma unroll
      for (int j = 0; j < NMAX; ++j) {
        S acc = S(0);
#pragma unroll
        for (int k = 0; k < NMAX; ++k) acc += g.v[i * NMAX + k] * f.v[k * NMAX + j];
        m.v[i * NMAX + j] = acc;
      }
      S acc = g.v[NN + i];
#pragma unroll
      for (int k = 0; k < NMAX; ++k) acc += g.v[i * NMAX + k] * f.v[NN + k];
      m.v[NN + i] = acc;
    }
    return m;
  }
  static __device__ __forceinline__ State apply(const Map& m, const State& s) {
    State r;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) {
      S acc = m.v[NN + i];
#pragma unroll
      for (int k = 0; k < NMAX; ++k) acc += m.v[i * NMAX + k] * s.v[k];
      r.v[i] = acc;
    }
    return r;
  }
  PTB_NO_CTX
};

template <class S>
struct MatNParams {
  const S* A; int64_t a_row_stride;   // elements between rows' matrices (0: shared by the rows)
  int64_t a_t_stride;                 // N*N (per sample) or 0 (constant along time)
  const S* zi;                        // forward: (B,N) initial state; adjoint: optional (B,N) c[T]
  const S* x;                         // forward: x; adjoint: gy            (B,T,N)
  S* y;                               // forward: h; adjoint: g             (B,T,N)
  S* zf;                              // optional (B,N): forward h[T-1]; adjoint c[0]
  int64_t T;
  int N;
};

template <class S, int NMAX, int NT_, int SPT_, int STAGES_, bool REV>
struct MatN : MatNAffine<S, NMAX> {
  using Alg = MatNAffine<S, NMAX>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = MatNParams<S>;
  using Scalar = S;
  static constexpr int NN = NMAX * NMAX;
  static constexpr int NT = NT_;
  static constexpr int SPT = SPT_;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = 1;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = REV;
  static constexpr bool HAS_PARTIAL = false;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int X_OFF = 0;                                     // x in, h out (TILE * N scalars used)
  static constexpr int A_OFF = TILE * NMAX * (int)sizeof(S);          // per-sample matrices (TILE * N*N scalars used)
  static constexpr int NROWC = NN;                                    // the row's matrix when it is constant along time
  static constexpr int ROWC_OFF = A_OFF + TILE * NN * (int)sizeof(S);
  static constexpr int STAGE_BYTES = ((ROWC_OFF + NN * (int)sizeof(S) + 127) / 128) * 128;

  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    if (p.a_t_stride != 0) return;   // per-sample matrices travel with the tile
    const S* a = p.A + row * p.a_row_stride;
    const int n2 = p.N * p.N;
#pragma unroll
    for (int i = 0; i < NN; ++i) out[i] = i < n2 ? ld_ro(a + i) : S(0);
  }
  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t vb = (uint32_t)nvalid * (uint32_t)p.N * (uint32_t)sizeof(S);
    io.load(X_OFF, p.x + (row * p.T + t0) * p.N, vb);
    if (p.a_t_stride != 0) io.load(A_OFF, p.A + row * p.a_row_stride + t0 * p.a_t_stride, vb * (uint32_t)p.N);
    io.store(X_OFF, p.y + (row * p.T + t0) * p.N, vb);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s = Alg::zero_state();
    if (p.zi) {
#pragma unroll
      for (int i = 0; i < NMAX; ++i)
        if (i < p.N) s.v[i] = ld_ro(p.zi + row * p.N + i);
    }
    return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.zf) {
#pragma unroll
      for (int i = 0; i < NMAX; ++i)
        if (i < p.N) p.zf[row * p.N + i] = s.v[i];
    }
  }
  // the matrix of local sample q (padded with zeros; transposed for the adjoint)
  static constexpr int VW = Vec16<S>::V;   // scalars per 16 bytes
  static __device__ __forceinline__ void load_mat(const Params& p, const unsigned char* stage, int q, S* a) {
    const S* src = p.a_t_stride != 0 ? reinterpret_cast<const S*>(stage + A_OFF) + (size_t)q * p.N * p.N
                                     : reinterpret_cast<const S*>(stage + ROWC_OFF);
    if (p.N == NMAX) {   // whole rows with 16-byte accesses: a quarter of the instructions, and of the bank conflicts
      S t[NN];
#pragma unroll
      for (int i = 0; i < NN; i += VW) VecIO<S, VW>::ld(reinterpret_cast<const unsigned char*>(src + i), t + i);
#pragma unroll
      for (int i = 0; i < NMAX; ++i)
#pragma unroll
        for (int j = 0; j < NMAX; ++j) a[i * NMAX + j] = REV ? t[j * NMAX + i] : t[i * NMAX + j];
      return;
    }
#pragma unroll
    for (int i = 0; i < NMAX; ++i)
#pragma unroll
      for (int j = 0; j < NMAX; ++j) {
        const int r = REV ? j : i, c = REV ? i : j;
        a[i * NMAX + j] = (i < p.N && j < p.N) ? src[r * p.N + c] : S(0);
      }
  }
  static __device__ __forceinline__ void load_vec(const Params& p, const unsigned char* stage, int q, S* v) {
    const S* src = reinterpret_cast<const S*>(stage + X_OFF) + (size_t)q * p.N;
    if (p.N == NMAX) {
#pragma unroll
      for (int i = 0; i < NMAX; i += VW) VecIO<S, VW>::ld(reinterpret_cast<const unsigned char*>(src + i), v + i);
      return;
    }
#pragma unroll
    for (int i = 0; i < NMAX; ++i) v[i] = i < p.N ? src[i] : S(0);
  }
  static __device__ __forceinline__ void store_vec(const Params& p, unsigned char* stage, int q, const S* v) {
    S* dst = reinterpret_cast<S*>(stage + X_OFF) + (size_t)q * p.N;
    if (p.N == NMAX) {
#pragma unroll
      for (int i = 0; i < NMAX; i += VW) VecIO<S, VW>::st(reinterpret_cast<unsigned char*>(dst + i), v + i);
      return;
    }
#pragma unroll
    for (int i = 0; i < NMAX; ++i)
      if (i < p.N) dst[i] = v[i];
  }
  static __device__ __forceinline__ void matvec(const S* a, const S* v, S* o) {
#pragma unroll
    for (int i = 0; i < NMAX; ++i) {
      S acc = S(0);
#pragma unroll
      for (int k = 0; k < NMAX; ++k) acc += a[i * NMAX + k] * v[k];
      o[i] = acc;
    }
  }

  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos, int64_t,
                                                  int64_t, int nvalid) {
    Map m = Alg::identity();
#pragma unroll 1
    for (int jj = 0; jj < SPT; ++jj) {
      const int j = REV ? SPT - 1 - jj : jj;
      const int q = tpos * SPT + j;
      if (q >= nvalid) continue;
      S a[NN], v[NMAX], t[NMAX];
      load_mat(p, stage, q, a);
      load_vec(p, stage, q, v);
      // forward: s <- A s + x;  adjoint: c <- A^T (c + gy)
      if (!REV) {
        matvec(a, &m.v[NN], t);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) m.v[NN + i] = t[i] + v[i];
      } else {
#pragma unroll
        for (int i = 0; i < NMAX; ++i) v[i] += m.v[NN + i];
        matvec(a, v, t);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) m.v[NN + i] = t[i];
      }
      S nm[NN];
#pragma unroll
      for (int i = 0; i < NMAX; ++i)
#pragma unroll
        for (int c = 0; c < NMAX; ++c) {
          S acc = S(0);
#pragma unroll
          for (int k = 0; k < NMAX; ++k) acc += a[i * NMAX + k] * m.v[k * NMAX + c];
          nm[i * NMAX + c] = acc;
        }
#pragma unroll
      for (int i = 0; i < NN; ++i) m.v[i] = nm[i];
    }
    return m;
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage, int tpos,
                                                   int64_t, int64_t, int nvalid) {
    S h[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; ++i) h[i] = in.v[i];
#pragma unroll 1
    for (int jj = 0; jj < SPT; ++jj) {
      const int j = REV ? SPT - 1 - jj : jj;
      const int q = tpos * SPT + j;
      if (q >= nvalid) continue;
      S a[NN], v[NMAX], t[NMAX];
      load_mat(p, stage, q, a);
      load_vec(p, stage, q, v);
      if (!REV) {
        matvec(a, h, t);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) h[i] = t[i] + v[i];
        store_vec(p, stage, q, h);
      } else {
#pragma unroll
        for (int i = 0; i < NMAX; ++i) v[i] += h[i];   // g = gy + c
        store_vec(p, stage, q, v);
        matvec(a, v, h);                               // c = A^T g
      }
    }
    Partial r; r.v[0] = S(0); return r;
  }
};

}  // namespace ptb
