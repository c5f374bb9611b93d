// Scan-engine policy for the dense N x N recurrence with a matrix that is CONSTANT along time,
//     h[t] = A h[t-1] + x[t],   h[-1] = zi          (forward)
//     g[t] = gy[t] + c[t+1],  c[t] = A^T g[t],  c[T] = g_in   (the scan of the adjoint; output g, final c[0])
// 2 < N <= NMAX: the reference's lti_recurN op (philtorch/csrc/host_lti_recurN.cpp:63-108, CPU only)
// and the scan inside its adjoint rule (philtorch/lti/ssm.py:67-96).
//
// The general policy of mat_n.cuh carries full affine maps and multiplies N x N matrices per sample
// and per scan step (N^3).  With a constant matrix the linear part of a span of n samples is A^n,
// the same for every span of that length in the row, so maps carry only the N-vector offset and
// their LENGTH (in thread units of SPT samples); the linear part is looked up as a product of the
// row's precomputed powers  Pw[i] = A^(SPT 2^i)  (one matrix-vector product per set bit of the
// length; in the scans lengths are powers of two).  Per sample that leaves two matrix-vector
// products (N^2), one per phase.  The powers are formed in double from the matrix as rounded to
// the working precision (repeated squaring doubles the relative error every step), once per call.
//
// Ragged ends: positions beyond T count as zero input, so every thread's map has full length.  What
// is wanted AT the ragged end -- the final state h[T-1] forward, the adjoint state entering at T
// backward -- is handled by the one thread that owns sample T-1; the adjoint's c[0] by the owner of
// sample 0.
#pragma once
#include "mat_n.cuh"
#include "sos_cascade.cuh"   // Ld4, LenCodec

namespace ptb {

template <int NMAX>
struct MatNLtiDims {
  static constexpr int NN = NMAX * NMAX;
  static constexpr int NPOW = 24;                      // Pw[0..NPOW): spans up to 2^24 thread units
  static constexpr int NPS = 9;                        // powers the compute warps need (spans <= one tile of <= 256 threads)
  static constexpr int ROWTAB = NN + NPOW * NN;        // A (padded; transposed for the adjoint), then the powers
  static constexpr int ROWC_SCALARS = NN + NPS * NN;   // leading part staged with every tile
};

template <class S>
struct MatNLtiCtx {
  const S* p;      // the row's powers (the matrix itself sits NN scalars before)
  bool shared;
};

template <class S, int NMAX>
struct MatNLtiAlg {
  using D = MatNLtiDims<NMAX>;
  static constexpr int NN = D::NN;
  using Map = Pod<S, NMAX + 1>;   // v[0..NMAX) offset, v[NMAX] = span length (thread units), bit-encoded
  using State = Pod<S, NMAX>;
  using Ctx = MatNLtiCtx<S>;

  static __device__ __forceinline__ uint32_t len(const Map& m) { return LenCodec<S>::dec(m.v[NMAX]); }
  static __device__ __forceinline__ Map identity() {
    Map m;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) m.v[i] = S(0);
    m.v[NMAX] = LenCodec<S>::enc(0);
    return m;
  }
  static __device__ __forceinline__ State zero_state() {
    State s;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) s.v[i] = S(0);
    return s;
  }
  // a map that ignores its input: only ever composed with inputs that are zero, so the length is irrelevant
  static __device__ __forceinline__ Map const_map(const State& s) {
    Map m;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) m.v[i] = s.v[i];
    m.v[NMAX] = LenCodec<S>::enc(0);
    return m;
  }
  // o = M v for the matrix at table offset `off` (scalars, relative to the powers).  Table matrices are
  // stored with their rows interleaved in pairs, element (r, q) at ((r / 2) * NMAX + q) * 2 + r % 2, so
  // one 16-byte load yields {M[2p][q], M[2p+1][q], M[2p][q+1], M[2p+1][q+1]}: in float32 the two rows of
  // a pair advance together with packed multiply-adds (fma.rn.f32x2: half the arithmetic instructions).
  static __device__ __forceinline__ void matvec(Ctx c, int off, const S* v, S* o) {
#pragma unroll
    for (int p = 0; p < NMAX / 2; ++p) {
      if constexpr (std::is_same<S, float>::value) {
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < NMAX; q += 2) {
          float m[4];
          if (c.shared) Ld4<float, true>::ld(c.p + off + (p * NMAX + q) * 2, m);
          else Ld4<float, false>::ld(c.p + off + (p * NMAX + q) * 2, m);
          acc = __ffma2_rn(make_float2(m[0], m[1]), make_float2(v[q], v[q]), acc);
          acc = __ffma2_rn(make_float2(m[2], m[3]), make_float2(v[q + 1], v[q + 1]), acc);
        }
        o[2 * p] = acc.x;
        o[2 * p + 1] = acc.y;
      } else {
        S a0 = S(0), a1 = S(0);
#pragma unroll
        for (int q = 0; q < NMAX; q += 2) {
          S m[4];
          if (c.shared) Ld4<S, true>::ld(c.p + off + (p * NMAX + q) * 2, m);
          else Ld4<S, false>::ld(c.p + off + (p * NMAX + q) * 2, m);
          a0 += m[0] * v[q] + m[2] * v[q + 1];
          a1 += m[1] * v[q] + m[3] * v[q + 1];
        }
        o[2 * p] = a0;
        o[2 * p + 1] = a1;
      }
    }
  }
  // v <- A^(n SPT) v
  static __device__ __forceinline__ void powapply(Ctx c, uint32_t n, S* v) {
#pragma unroll 1
    while (n) {
      const int i = __ffs(n) - 1;
      n &= n - 1;
      S o[NMAX];
      matvec(c, i * NN, v, o);
#pragma unroll
      for (int q = 0; q < NMAX; ++q) v[q] = o[q];
    }
  }
  // apply `first`, then `second`
  static __device__ __forceinline__ Map compose(Ctx c, const Map& first, const Map& second) {
    S t[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; ++i) t[i] = first.v[i];
    powapply(c, len(second), t);
    Map r;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) r.v[i] = t[i] + second.v[i];
    r.v[NMAX] = LenCodec<S>::enc(len(first) + len(second));
    return r;
  }
  static __device__ __forceinline__ State apply(Ctx c, const Map& m, const State& s) {
    S t[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; ++i) t[i] = s.v[i];
    powapply(c, len(m), t);
    State r;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) r.v[i] = t[i] + m.v[i];
    return r;
  }
  // inclusive scan over the lanes (level 0: threads of a warp, 1: warps of a tile); the lengths travel
  // with the maps, every step is one matrix-vector product with a power of two
  static __device__ __forceinline__ Map warp_scan(Ctx c, Map m, int lane, int) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const Map o = shfl_up_pod(m, d);
      if (lane >= d) m = compose(c, o, m);
    }
    return m;
  }
  // state entering a thread: the tile-incoming state carried over the warps before (wp) and the lanes
  // before (e)
  static __device__ __forceinline__ State thread_state(Ctx c, const Map& wp, const Map& e, const State& hin, int) {
    return apply(c, e, apply(c, wp, hin));
  }
};

// One block per matrix row of the call, NN threads: the (padded, for the adjoint transposed) matrix
// and its powers Pw[i] = A^(spt 2^i), in double, rounded to S.
template <class S, int NMAX, bool REV>
__global__ void matn_lti_setup_kernel(const S* __restrict__ A, int64_t a_row_stride, int N, S* __restrict__ tab, int spt) {
  using D = MatNLtiDims<NMAX>;
  constexpr int NN = D::NN;
  __shared__ double A0[NMAX][NMAX], U[NMAX][NMAX], V[NMAX][NMAX];
  const int tid = threadIdx.x;
  const int r = tid / NMAX, c = tid % NMAX;
  const S* a = A + (int64_t)blockIdx.x * a_row_stride;
  S* out = tab + (int64_t)blockIdx.x * D::ROWTAB;
  const int at = ((r >> 1) * NMAX + c) * 2 + (r & 1);   // rows interleaved in pairs, see MatNLtiAlg::matvec
  S val = S(0);
  if (r < N && c < N) val = REV ? a[c * N + r] : a[r * N + c];
  out[at] = val;
  A0[r][c] = (double)val;
  U[r][c] = (double)val;
  __syncthreads();
  for (int n = 1; n < spt; ++n) {   // U = A^spt
    double acc = 0.0;
    for (int q = 0; q < NMAX; ++q) acc += A0[r][q] * U[q][c];
    V[r][c] = acc;
    __syncthreads();
    U[r][c] = V[r][c];
    __syncthreads();
  }
  for (int i = 0; i < D::NPOW; ++i) {
    out[NN + (size_t)i * NN + at] = (S)U[r][c];
    double acc = 0.0;
    for (int q = 0; q < NMAX; ++q) acc += U[r][q] * U[q][c];
    V[r][c] = acc;
    __syncthreads();
    U[r][c] = V[r][c];
    __syncthreads();
  }
}

template <class S>
struct MatNLtiParams {
  const S* tab; int64_t tab_stride;   // table rows (scalars apart; 0 when the matrix is shared by the rows)
  const S* zi;                        // forward: (B,N) initial state; adjoint: optional (B,N) c[T]
  const S* x;                         // forward: x; adjoint: gy            (B,T,N)
  S* y;                               // forward: h; adjoint: g             (B,T,N)
  S* zf;                              // optional (B,N): forward h[T-1]; adjoint c[0]
  int64_t T;
  int N;
};

template <class S, int NMAX, int NT_, int SPT_, int STAGES_, bool REV>
struct MatNLti : MatNLtiAlg<S, NMAX> {
  static_assert(NT_ == 128 || NT_ == 256, "a tile is 2^7 or 2^8 thread units");
  static_assert(SPT_ % 2 == 1, "an odd number of samples per thread (shared-memory banks)");
  using Alg = MatNLtiAlg<S, NMAX>;
  using D = MatNLtiDims<NMAX>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = MatNLtiParams<S>;
  using Scalar = S;
  static constexpr int NN = D::NN;
  static constexpr int NT = NT_;
  static constexpr int SPT = SPT_;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = 1;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = REV;
  static constexpr bool HAS_PARTIAL = false;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int NROWC = 0;
  static constexpr int X_OFF = 0;                                     // x in, h out (TILE * N scalars used)
  static constexpr int ROWC_OFF = ((TILE * NMAX * (int)sizeof(S) + 127) / 128) * 128;
  static constexpr int ROWC_BYTES = D::ROWC_SCALARS * (int)sizeof(S);
  static constexpr int STAGE_BYTES = ((ROWC_OFF + ROWC_BYTES + 127) / 128) * 128;

  static __device__ __forceinline__ void row_constants(const Params&, int64_t, S*) {}
  static __device__ __forceinline__ typename Alg::Ctx ctx_stage(const unsigned char* stage) {
    return typename Alg::Ctx{reinterpret_cast<const S*>(stage + ROWC_OFF) + NN, true};
  }
  static __device__ __forceinline__ typename Alg::Ctx ctx_row(const Params& p, int64_t row) {
    return typename Alg::Ctx{p.tab + row * p.tab_stride + NN, false};
  }
  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid, IoPlan& io) {
    const uint32_t vb = (uint32_t)nvalid * (uint32_t)p.N * (uint32_t)sizeof(S);
    io.load(X_OFF, p.x + (row * p.T + t0) * p.N, vb);
    io.load(ROWC_OFF, p.tab + row * p.tab_stride, ROWC_BYTES);
    io.store(X_OFF, p.y + (row * p.T + t0) * p.N, vb);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s = Alg::zero_state();
    if (!REV && p.zi) {   // the adjoint's incoming state is injected by the owner of sample T-1
#pragma unroll
      for (int i = 0; i < NMAX; ++i)
        if (i < p.N) s.v[i] = ld_ro(p.zi + row * p.N + i);
    }
    return s;
  }
  static __device__ __forceinline__ void row_final(const Params&, int64_t, const State&) {}   // see finish

  // A thread's SPT samples are consecutive in the stage, so the lanes of a warp are SPT * N scalars
  // apart: SPT is odd, which keeps 16-byte accesses (N = NMAX) on different banks and 4-byte accesses
  // free of conflicts whenever N is odd as well.
  static constexpr int VW = Vec16<S>::V;   // scalars per 16 bytes
  static __device__ __forceinline__ void load_vec(const Params& p, const unsigned char* stage, int q, S* v) {
    if (p.N == NMAX) {
      const unsigned char* src = stage + X_OFF + (size_t)q * NMAX * sizeof(S);
#pragma unroll
      for (int i = 0; i < NMAX; i += VW) VecIO<S, VW>::ld(src + i * sizeof(S), v + i);
      return;
    }
    const S* src = reinterpret_cast<const S*>(stage + X_OFF) + (size_t)q * p.N;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) v[i] = i < p.N ? src[i] : S(0);
  }
  static __device__ __forceinline__ void store_vec(const Params& p, unsigned char* stage, int q, const S* v) {
    if (p.N == NMAX) {
      unsigned char* dst = stage + X_OFF + (size_t)q * NMAX * sizeof(S);
#pragma unroll
      for (int i = 0; i < NMAX; i += VW) VecIO<S, VW>::st(dst + i * sizeof(S), v + i);
      return;
    }
    S* dst = reinterpret_cast<S*>(stage + X_OFF) + (size_t)q * p.N;
#pragma unroll
    for (int i = 0; i < NMAX; ++i)
      if (i < p.N) dst[i] = v[i];
  }
  // o = A v (A^T for the adjoint: the table holds the transpose) with the matrix staged with the tile
  static __device__ __forceinline__ void step_matvec(const unsigned char* stage, const S* v, S* o) {
    const typename Alg::Ctx c{reinterpret_cast<const S*>(stage + ROWC_OFF) + NN, true};
    Alg::matvec(c, -NN, v, o);
  }
  static __device__ __forceinline__ void add_g_in(const Params& p, int64_t row, S* v) {
#pragma unroll
    for (int i = 0; i < NMAX; ++i)
      if (i < p.N) v[i] += ld_ro(p.zi + row * p.N + i);
  }

  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos, int64_t row,
                                                  int64_t t0, int nvalid) {
    S v[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; ++i) v[i] = S(0);
#pragma unroll 1
    for (int jj = 0; jj < SPT; ++jj) {
      const int j = REV ? SPT - 1 - jj : jj;
      const int q = tpos * SPT + j;
      S u[NMAX], t[NMAX];
      if (q < nvalid) load_vec(p, stage, q, u);
      else {
#pragma unroll
        for (int i = 0; i < NMAX; ++i) u[i] = S(0);
      }
      if (!REV) {             // s <- A s + x
        step_matvec(stage, v, t);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) v[i] = t[i] + u[i];
      } else {                // c <- A^T (c + gy), with c[T] entering above sample T-1
        if (p.zi && t0 + q == p.T - 1) add_g_in(p, row, u);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) u[i] += v[i];
        step_matvec(stage, u, v);
      }
    }
    Map m;
#pragma unroll
    for (int i = 0; i < NMAX; ++i) m.v[i] = v[i];
    m.v[NMAX] = LenCodec<S>::enc(1);
    return m;
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage, int tpos,
                                                   int64_t row, int64_t t0, int nvalid) {
    S h[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; ++i) h[i] = in.v[i];
#pragma unroll 1
    for (int jj = 0; jj < SPT; ++jj) {
      const int j = REV ? SPT - 1 - jj : jj;
      const int q = tpos * SPT + j;
      if (q >= nvalid) continue;   // beyond the end of the row: nothing to write, nothing later depends on it
      S u[NMAX], t[NMAX];
      load_vec(p, stage, q, u);
      if (!REV) {
        step_matvec(stage, h, t);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) h[i] = t[i] + u[i];
        store_vec(p, stage, q, h);
        if (p.zf && t0 + q == p.T - 1) {
#pragma unroll
          for (int i = 0; i < NMAX; ++i)
            if (i < p.N) p.zf[row * p.N + i] = h[i];
        }
      } else {
        if (p.zi && t0 + q == p.T - 1) add_g_in(p, row, u);
#pragma unroll
        for (int i = 0; i < NMAX; ++i) u[i] += h[i];   // g = gy + c
        store_vec(p, stage, q, u);
        step_matvec(stage, u, h);                      // c = A^T g
        if (p.zf && t0 + q == 0) {
#pragma unroll
          for (int i = 0; i < NMAX; ++i)
            if (i < p.N) p.zf[row * p.N + i] = h[i];
        }
      }
    }
    Partial r; r.v[0] = S(0); return r;
  }
};

// ---- gradient of a constant matrix: grad_A[r] = sum_t g[r,t] (x) h[r,t-1], h[r,-1] = zi[r] --------------
// (philtorch/lti/ssm.py:67-96 forms it as a matrix product of the time-reversed scan's output with the
// shifted states.)  One block per (row, time chunk): every thread accumulates the NMAX x NMAX outer
// products of its samples in registers, the block adds them up (warp shuffles, then shared memory, in
// a fixed order) and writes one partial matrix; the caller sums the partials of a row.  Reads g and h
// once, no shifted copy of h.
constexpr int kOuterNT = 256;

template <class S, int NMAX>
__global__ void __launch_bounds__(kOuterNT)
outer_prev_sum_kernel(const S* __restrict__ g, const S* __restrict__ h, const S* __restrict__ zi, S* __restrict__ partial,
                      int N, int64_t T, int chunks, int64_t chunk_len) {
  constexpr int NN = NMAX * NMAX;
  constexpr int VW = Vec16<S>::V;
  __shared__ S red[kOuterNT / 32][NN];
  const int64_t row = blockIdx.x / chunks;
  const int chunk = (int)(blockIdx.x % chunks);
  const int64_t c0 = (int64_t)chunk * chunk_len, c1 = (c0 + chunk_len < T) ? c0 + chunk_len : T;
  const S* gr = g + row * T * N;
  const S* hr = h + row * T * N;
  S acc[NN];
#pragma unroll
  for (int i = 0; i < NN; ++i) acc[i] = S(0);
  const bool vec = N == NMAX && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(h)) & 15u) == 0;
  auto fetch = [&](int64_t t, S* gv, S* hv) {
    if (t >= c1) {   // beyond the chunk: contributes nothing
#pragma unroll
      for (int i = 0; i < NMAX; ++i) { gv[i] = S(0); hv[i] = S(0); }
      return;
    }
    if (vec) {
#pragma unroll
      for (int i = 0; i < NMAX; i += VW) {
        VecIO<S, VW>::ld(reinterpret_cast<const unsigned char*>(gr + t * NMAX + i), gv + i);
        if (t > 0) VecIO<S, VW>::ld(reinterpret_cast<const unsigned char*>(hr + (t - 1) * NMAX + i), hv + i);
      }
      if (t == 0) {
#pragma unroll
        for (int i = 0; i < NMAX; ++i) hv[i] = zi[row * N + i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < NMAX; ++i) {
        gv[i] = i < N ? gr[t * N + i] : S(0);
        hv[i] = i < N ? (t > 0 ? hr[(t - 1) * N + i] : zi[row * N + i]) : S(0);
      }
    }
  };
  // two samples per trip: their loads are in flight together
  for (int64_t t = c0 + threadIdx.x; t < c1; t += 2 * kOuterNT) {
    S g0[NMAX], h0[NMAX], g1[NMAX], h1[NMAX];
    fetch(t, g0, h0);
    fetch(t + kOuterNT, g1, h1);
#pragma unroll
    for (int i = 0; i < NMAX; ++i)
#pragma unroll
      for (int j = 0; j < NMAX; ++j) acc[i * NMAX + j] += g0[i] * h0[j] + g1[i] * h1[j];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < NN; ++i) {
    S a = acc[i];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) a += __shfl_down_sync(0xffffffffu, a, d);
    if (lane == 0) red[warp][i] = a;
  }
  __syncthreads();
  if (threadIdx.x < NN) {
    S a = S(0);
    for (int w = 0; w < kOuterNT / 32; ++w) a += red[w][threadIdx.x];
    const int i = threadIdx.x / NMAX, j = threadIdx.x % NMAX;
    if (i < N && j < N) partial[((row * chunks + chunk) * N + i) * N + j] = a;
  }
}

}  // namespace ptb
