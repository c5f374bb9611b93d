// Scan-engine policies for a CASCADE of K second-order sections (transposed direct form II, scalar
// in, scalar out), all K sections in ONE pass over the signal per direction.
//
// The reference runs a cascade as K chained calls of lfilter(b_k, a_k, ., form="tdf2")
// (philtorch/lti/filtering.py:304-317 -> philtorch/lti/ssm.py:466-504), every one a full trip
// through memory.  Here the cascade is ONE linear time-invariant system with 2K states
//     s = [s^0; s^1; ...; s^{K-1}],   s[t] = Mc s[t-1] + (input terms)
// whose transition matrix Mc is block lower triangular (section k only sees sections < k).  A
// thread's map over its SPT samples is  s_out = Mc^SPT s_in + v : the linear part is the SAME for
// every thread of a row, so maps carry only the 2K-vector v and the LENGTH of their span (in
// thread units); the linear part of a span of n units is looked up as a product of the row's
// precomputed powers  Pw[i] = Mc^(SPT 2^i)  (one matrix per set bit of n; in the scans n is a power
// of two).  A tile is NT = 256 = 2^8 thread units, so the tile-level look-back uses Pw[8..].
//
// Forward: reads x once, writes y once.  Backward: reads gy, x and the K section outputs once,
// writes grad_x once: K+3 scalars per sample instead of 4K.
//
// Adjoint of section k (lam_k[t] = dL/ds^k[t], g_k = gradient w.r.t. the section's output):
//     gx_k[t]   = b0 g_k[t] + B . lam_k[t]              (= g_{k-1}[t], the next section's drive)
//     lam_k[t-1] = M_k^T lam_k[t] + e0 g_k[t]
// run for k = K-1 .. 0 in descending time: again a block-lower-triangular system when the states are
// ordered [lam_{K-1}; ...; lam_0].  Coefficient gradients from five sums per section, as for the
// single section (biquad.cuh).
//
// Ragged ends: positions beyond T are treated as zero input, so every thread's map has full length
// and all powers come from the table.  The state wanted at the ragged end (zf forward, the gradient
// entering through zf backward) is handled by the one thread that owns sample T-1.
#pragma once
#include "biquad.cuh"

namespace ptb {

template <int K>
struct SosDims {
  static constexpr int NS = 2 * K;                      // states of the cascade
  static constexpr int NBLK = K * (K + 1) / 2;          // 2x2 blocks of a block-lower-triangular matrix
  static constexpr int MATSZ = 4 * NBLK;                // scalars per packed matrix
  static constexpr int COEFN = ((5 * K + 3) / 4) * 4;   // derived coefficients {b0,B0,B1,-a1,-a2} x K, padded
  static constexpr int NPOW = 24;                       // Pw[0..NPOW): spans up to 2^24 thread units
  static constexpr int NPS = 10;                        // powers the compute warps need (spans <= one tile of <= 512 threads)
  static constexpr int ROWTAB = COEFN + NPOW * MATSZ;   // scalars per row of the table
  static constexpr int ROWC_SCALARS = COEFN + NPS * MATSZ;   // leading part staged with every tile
};

template <class S> struct LenCodec;
template <> struct LenCodec<float> {
  static __device__ __forceinline__ float enc(uint32_t n) { return __uint_as_float(n); }
  static __device__ __forceinline__ uint32_t dec(float f) { return __float_as_uint(f); }
};
template <> struct LenCodec<double> {
  static __device__ __forceinline__ double enc(uint32_t n) { return (double)n; }
  static __device__ __forceinline__ uint32_t dec(double f) { return (uint32_t)f; }
};

// Four consecutive table scalars.  The table is read from shared memory by the compute warps (the
// part staged with the tile) and from global memory by the look-back warp; SH is known at compile
// time at every call site, so each gets the load of its own address space (a generic load of
// shared memory would go through the long-latency path).
template <class S, bool SH> struct Ld4;
template <> struct Ld4<float, false> {
  static __device__ __forceinline__ void ld(const float* p, float* m) {
    const float4 q = __ldg(reinterpret_cast<const float4*>(p));
    m[0] = q.x; m[1] = q.y; m[2] = q.z; m[3] = q.w;
  }
};
template <> struct Ld4<double, false> {
  static __device__ __forceinline__ void ld(const double* p, double* m) {
    const double2 q = __ldg(reinterpret_cast<const double2*>(p)), r = __ldg(reinterpret_cast<const double2*>(p + 2));
    m[0] = q.x; m[1] = q.y; m[2] = r.x; m[3] = r.y;
  }
};
template <> struct Ld4<float, true> {
  static __device__ __forceinline__ void ld(const float* p, float* m) {
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(m[0]), "=f"(m[1]), "=f"(m[2]), "=f"(m[3])
                 : "r"(smem_u32(p)));
  }
};
template <> struct Ld4<double, true> {
  static __device__ __forceinline__ void ld(const double* p, double* m) {
    asm volatile("ld.shared.v2.f64 {%0,%1}, [%2];" : "=d"(m[0]), "=d"(m[1]) : "r"(smem_u32(p)));
    asm volatile("ld.shared.v2.f64 {%0,%1}, [%2];" : "=d"(m[2]), "=d"(m[3]) : "r"(smem_u32(p + 2)));
  }
};
// the row's table of powers and where it lives
template <class S>
struct SosCtx {
  const S* p;
  bool shared;
};

// Algebra of the maps  s -> Mc^(len SPT) s + v  of one row; Ctx = the row's table of powers.
template <class S, int K>
struct SosAlg {
  using D = SosDims<K>;
  static constexpr int NS = D::NS;
  using Map = Pod<S, NS + 1>;   // v[0..NS) offset, v[NS] = span length (thread units), bit-encoded
  using State = Pod<S, NS>;
  using Ctx = SosCtx<S>;

  static __device__ __forceinline__ uint32_t len(const Map& m) { return LenCodec<S>::dec(m.v[NS]); }
  static __device__ __forceinline__ Map identity() {
    Map m;
#pragma unroll
    for (int i = 0; i < NS; ++i) m.v[i] = S(0);
    m.v[NS] = LenCodec<S>::enc(0);
    return m;
  }
  static __device__ __forceinline__ State zero_state() {
    State s;
#pragma unroll
    for (int i = 0; i < NS; ++i) s.v[i] = S(0);
    return s;
  }
  // a map that ignores its input: only ever composed with inputs that are zero (nothing older is
  // used), so the length is irrelevant
  static __device__ __forceinline__ Map const_map(const State& s) {
    Map m;
#pragma unroll
    for (int i = 0; i < NS; ++i) m.v[i] = s.v[i];
    m.v[NS] = LenCodec<S>::enc(0);
    return m;
  }
  // o = M v for a packed block-lower-triangular M (blocks row-major over bj <= bi, 4 scalars each)
  static __device__ __forceinline__ void ld4(Ctx c, int off, S* m) {
    if (c.shared) Ld4<S, true>::ld(c.p + off, m);
    else Ld4<S, false>::ld(c.p + off, m);
  }
  static __device__ __forceinline__ void matvec(Ctx c, int moff, const S* v, S* o) {
#pragma unroll
    for (int bi = 0; bi < K; ++bi) {
      S o0 = S(0), o1 = S(0);
#pragma unroll
      for (int bj = 0; bj <= bi; ++bj) {
        S m[4];
        ld4(c, moff + 4 * (bi * (bi + 1) / 2 + bj), m);
        o0 += m[0] * v[2 * bj] + m[1] * v[2 * bj + 1];
        o1 += m[2] * v[2 * bj] + m[3] * v[2 * bj + 1];
      }
      o[2 * bi] = o0;
      o[2 * bi + 1] = o1;
    }
  }
  // v <- Mc^(n SPT) v
  static __device__ __forceinline__ void powapply(Ctx c, uint32_t n, S* v) {
#pragma unroll 1
    while (n) {
      const int i = __ffs(n) - 1;
      n &= n - 1;
      S o[NS];
      matvec(c, i * D::MATSZ, v, o);
#pragma unroll
      for (int q = 0; q < NS; ++q) v[q] = o[q];
    }
  }
  // apply `first`, then `second`
  static __device__ __forceinline__ Map compose(Ctx c, const Map& first, const Map& second) {
    S t[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) t[i] = first.v[i];
    powapply(c, len(second), t);
    Map r;
#pragma unroll
    for (int i = 0; i < NS; ++i) r.v[i] = t[i] + second.v[i];
    r.v[NS] = LenCodec<S>::enc(len(first) + len(second));
    return r;
  }
  static __device__ __forceinline__ State apply(Ctx c, const Map& m, const State& s) {
    S t[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) t[i] = s.v[i];
    powapply(c, len(m), t);
    State r;
#pragma unroll
    for (int i = 0; i < NS; ++i) r.v[i] = t[i] + m.v[i];
    return r;
  }
  // ---- scans over the lanes of a warp, section by section ------------------------------------------
  // With s(i) the state entering lane i, one lane advances the cascade by one unit:
  //     s_k(i+1) = D_k s_k(i) + sum_{j<k} C_kj s_j(i) + v_k(i)
  // (D_k, C_kj: diagonal / off-diagonal 2x2 blocks of the unit's power).  Section by section this is
  // a 2x2 time-invariant scan whose offsets are known once the sections before it are done:
  // 2 shuffles + 4 multiply-adds per step instead of a full block-triangular product.
  // u: index of the unit's power (0: one thread, 5: one warp).  On return sin = state entering the
  // lane and inc = state leaving it, when the state entering lane 0 is z (nullptr: zero).
  static __device__ __forceinline__ void lane_scan(Ctx c, int u, const S* v, const S* z, int lane, S* sin,
                                                   S* inc) {
    const int P0 = u * D::MATSZ;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      S w0 = v ? v[2 * k] : S(0), w1 = v ? v[2 * k + 1] : S(0);
#pragma unroll
      for (int j = 0; j < k; ++j) {
        S m[4];
        ld4(c, P0 + 4 * (k * (k + 1) / 2 + j), m);
        w0 += m[0] * sin[2 * j] + m[1] * sin[2 * j + 1];
        w1 += m[2] * sin[2 * j] + m[3] * sin[2 * j + 1];
      }
      if (z != nullptr && lane == 0) {
        S m[4];
        ld4(c, P0 + 4 * (k * (k + 1) / 2 + k), m);
        w0 += m[0] * z[2 * k] + m[1] * z[2 * k + 1];
        w1 += m[2] * z[2 * k] + m[3] * z[2 * k + 1];
      }
      S a0 = w0, a1 = w1;
#pragma unroll
      for (int d = 0; d < 5; ++d) {
        const S o0 = __shfl_up_sync(0xffffffffu, a0, 1 << d), o1 = __shfl_up_sync(0xffffffffu, a1, 1 << d);
        S m[4];
        ld4(c, (u + d) * D::MATSZ + 4 * (k * (k + 1) / 2 + k), m);
        if (lane >= (1 << d)) {
          a0 += m[0] * o0 + m[1] * o1;
          a1 += m[2] * o0 + m[3] * o1;
        }
      }
      inc[2 * k] = a0;
      inc[2 * k + 1] = a1;
      const S e0 = __shfl_up_sync(0xffffffffu, a0, 1), e1 = __shfl_up_sync(0xffffffffu, a1, 1);
      sin[2 * k] = lane == 0 ? (z ? z[2 * k] : S(0)) : e0;
      sin[2 * k + 1] = lane == 0 ? (z ? z[2 * k + 1] : S(0)) : e1;
    }
  }
  // inclusive scan of maps that all span one unit (level 0: a thread, level 1: a warp)
  static __device__ __forceinline__ Map warp_scan(Ctx c, const Map& m, int lane, int level) {
    S sin[NS];
    Map r;
    lane_scan(c, level ? 5 : 0, m.v, nullptr, lane, sin, r.v);
    r.v[NS] = LenCodec<S>::enc((uint32_t)(lane + 1) << (level ? 5 : 0));
    return r;
  }
  // state entering the thread `lane` of a warp: the state entering the warp carried along the
  // lanes, plus the thread's exclusive prefix inside the warp (from a zero state, phase 1)
  static __device__ __forceinline__ State thread_state(Ctx c, const Map& wp, const Map& e, const State& hin,
                                                       int lane) {
    S z[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) z[i] = hin.v[i];
    powapply(c, len(wp), z);
#pragma unroll
    for (int i = 0; i < NS; ++i) z[i] += wp.v[i];
    S sin[NS], inc[NS];
    lane_scan(c, 0, nullptr, z, lane, sin, inc);
    State r;
#pragma unroll
    for (int i = 0; i < NS; ++i) r.v[i] = sin[i] + e.v[i];
    return r;
  }
};

// One sample of the cascade with zero input, forward (ADJ = false: states [s^0..s^{K-1}]) or adjoint
// (ADJ = true: states [lam_{K-1}..lam_0]); the table of powers is built from these, so it matches
// the recurrences of the kernels by construction.  cf: {b0,B0,B1,-a1,-a2} per section.
template <int K, bool ADJ>
__device__ __forceinline__ void sos_zero_input_step(const double (*cf)[5], double* st) {
  double u = 0.0;
  if (!ADJ) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const double h0 = st[2 * k], h1 = st[2 * k + 1];
      const double y = h0 + cf[k][0] * u;
      st[2 * k] = cf[k][3] * h0 + h1 + cf[k][1] * u;
      st[2 * k + 1] = cf[k][4] * h0 + cf[k][2] * u;
      u = y;
    }
  } else {
#pragma unroll
    for (int k = K - 1; k >= 0; --k) {
      const int p = K - 1 - k;
      const double l0 = st[2 * p], l1 = st[2 * p + 1];
      const double gx = cf[k][0] * u + cf[k][1] * l0 + cf[k][2] * l1;
      st[2 * p] = cf[k][3] * l0 + cf[k][4] * l1 + u;
      st[2 * p + 1] = l0;
      u = gx;
    }
  }
}

// One block per row of coefficients, NS*NS threads: derived coefficients and Pw[i] = Mc^(spt 2^i),
// computed in double (repeated squaring doubles the relative error every step) and rounded to S.
template <class S, int K, bool ADJ>
__global__ void sos_setup_kernel(const S* __restrict__ b, int64_t b_sec, int64_t b_row, const S* __restrict__ a,
                                 int64_t a_sec, int64_t a_row, S* __restrict__ tab, int spt) {
  using D = SosDims<K>;
  constexpr int NS = D::NS;
  __shared__ double cf[K][5];
  __shared__ double U[NS][NS], V[NS][NS];
  const int tid = threadIdx.x;
  const int64_t row = blockIdx.x;
  S* out = tab + row * D::ROWTAB;
  if (tid < K) {
    const S* pb = b + tid * b_sec + row * b_row;
    const S* pa = a + tid * a_sec + row * a_row;
    // derived in S exactly as the single-section kernels derive them; the table is built from the
    // rounded values, so it describes the recurrence the kernels actually run
    S d[5];
    BqCoef<S>::derive(pb, 0, pa, 0, 0, d);
#pragma unroll
    for (int i = 0; i < 5; ++i) { out[5 * tid + i] = d[i]; cf[tid][i] = (double)d[i]; }
  }
  if (tid >= 5 * K && tid < D::COEFN) out[tid] = S(0);
  __syncthreads();
  if (tid < NS) {
    double st[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) st[i] = (i == tid) ? 1.0 : 0.0;
    for (int n = 0; n < spt; ++n) sos_zero_input_step<K, ADJ>(cf, st);
#pragma unroll
    for (int i = 0; i < NS; ++i) U[i][tid] = st[i];
  }
  __syncthreads();
  const int r = tid / NS, c = tid % NS;
  const bool in_mat = tid < NS * NS;
  for (int i = 0; i < D::NPOW; ++i) {
    if (in_mat && (r >> 1) >= (c >> 1)) {
      const int bi = r >> 1, bj = c >> 1;
      out[D::COEFN + (size_t)i * D::MATSZ + 4 * (bi * (bi + 1) / 2 + bj) + (r & 1) * 2 + (c & 1)] = (S)U[r][c];
    }
    double acc = 0.0;
    if (in_mat)
      for (int q = 0; q < NS; ++q) acc += U[r][q] * U[q][c];
    if (in_mat) V[r][c] = acc;
    __syncthreads();
    if (in_mat) U[r][c] = V[r][c];
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------ forward
// One pass: reads x, writes y (and the final states).  The outputs of the inner sections never
// leave the registers.  (When they are wanted, for coefficient gradients, the caller runs the
// sections one by one: K passes that are each bound by memory bandwidth already, see capi_sos.cu.)
template <class S>
struct SosFwdParams {
  const S* tab; int64_t tab_stride;   // table rows (scalars apart; 0 when the coefficients are shared)
  const S* zi;                        // optional (K,B,2)
  const S* x;
  S* y;
  S* zf;                              // optional (K,B,2)
  int64_t T, B;
};

template <class S, int K, int CH, int STAGES_, int NT_ = 256, int MIN_CTAS_ = 1>
struct SosFwd : SosAlg<S, K> {
  static_assert(NT_ == 128 || NT_ == 256 || NT_ == 512, "a tile is 2^7, 2^8 or 2^9 thread units");
  using Alg = SosAlg<S, K>;
  using D = SosDims<K>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = SosFwdParams<S>;
  using Scalar = S;
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
  static constexpr int NROWC = 0;
  static constexpr int X_OFF = 0;   // x in, y out
  static constexpr int ROWC_OFF = TILE * (int)sizeof(S);
  static constexpr int ROWC_BYTES = D::ROWC_SCALARS * (int)sizeof(S);
  static constexpr int STAGE_BYTES = ((ROWC_OFF + ROWC_BYTES + 127) / 128) * 128;
  static __device__ __forceinline__ void row_constants(const Params&, int64_t, S*) {}
  static __device__ __forceinline__ typename Alg::Ctx ctx_stage(const unsigned char* stage) {
    return typename Alg::Ctx{reinterpret_cast<const S*>(stage + ROWC_OFF) + D::COEFN, true};
  }
  static __device__ __forceinline__ typename Alg::Ctx ctx_row(const Params& p, int64_t row) {
    return typename Alg::Ctx{p.tab + row * p.tab_stride + D::COEFN, false};
  }
  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    io.load(X_OFF, p.x + row * p.T + t0, bytes);
    io.load(ROWC_OFF, p.tab + row * p.tab_stride, ROWC_BYTES);
    io.store(X_OFF, p.y + row * p.T + t0, bytes);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s = Alg::zero_state();
    if (p.zi) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        s.v[2 * k] = __ldg(p.zi + ((int64_t)k * p.B + row) * 2);
        s.v[2 * k + 1] = __ldg(p.zi + ((int64_t)k * p.B + row) * 2 + 1);
      }
    }
    return s;
  }
  static __device__ __forceinline__ void row_final(const Params&, int64_t, const State&) {}   // see finish

  // the thread's samples, zero beyond the end of the row
  static __device__ __forceinline__ int load_x(const unsigned char* stage, int tpos, int nvalid, S* x) {
    const int p0 = tpos * SPT;
    int nv = nvalid - p0;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    const unsigned char* px = stage + X_OFF + (size_t)p0 * sizeof(S);
#pragma unroll
    for (int c = 0; c < CH; ++c) VecIO<S, V>::ld(px + 16 * c, &x[c * V]);
    if (nv < SPT) {
#pragma unroll
      for (int j = 0; j < SPT; ++j)
        if (j >= nv) x[j] = S(0);
    }
    return nv;
  }
  // All K sections over the thread's samples, in place, as a skewed wavefront: at step st section g
  // works on the 16-byte unit st-g, so K independent recurrences are in flight per thread (one
  // section alone is a serial chain of dependent multiply-adds).  h: the 2K states.
  template <bool FULL>
  static __device__ __forceinline__ void sections(const S* cf, S* h, int nv, S* x) {
    BqCoef<S> c[K];
#pragma unroll
    for (int g = 0; g < K; ++g) c[g].load(reinterpret_cast<const unsigned char*>(cf + 5 * g));
#pragma unroll
    for (int st = 0; st < CH + K - 1; ++st) {
#pragma unroll
      for (int g = K - 1; g >= 0; --g) {
        const int u = st - g;
        if (u >= 0 && u < CH) {
          S h0 = h[2 * g], h1 = h[2 * g + 1];
#pragma unroll
          for (int jj = 0; jj < V; ++jj) {
            const int j = u * V + jj;
            if (FULL || j < nv) {
              const S xj = x[j];
              x[j] = h0 + c[g].b0 * xj;
              const S t = h1 + c[g].B0 * xj;        // off the chain through h0
              h1 = c[g].na2 * h0 + c[g].B1 * xj;
              h0 = c[g].na1 * h0 + t;
            }
          }
          h[2 * g] = h0;
          h[2 * g + 1] = h1;
        }
      }
    }
  }
  static __device__ __forceinline__ Map aggregate(const Params&, const unsigned char* stage, int tpos, int64_t,
                                                  int64_t, int nvalid) {
    S x[SPT];
    load_x(stage, tpos, nvalid, x);
    const S* cf = reinterpret_cast<const S*>(stage + ROWC_OFF);
    Map m;
#pragma unroll
    for (int i = 0; i < Alg::NS; ++i) m.v[i] = S(0);
    sections<true>(cf, m.v, SPT, x);   // rows count as zero beyond their end: every map spans a whole unit
    m.v[Alg::NS] = LenCodec<S>::enc(1);
    return m;
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t t0, int nvalid) {
    S x[SPT];
    const int nv = load_x(stage, tpos, nvalid, x);
    const S* cf = reinterpret_cast<const S*>(stage + ROWC_OFF);
    S h[Alg::NS];
#pragma unroll
    for (int i = 0; i < Alg::NS; ++i) h[i] = in.v[i];
    if (nv == SPT) sections<true>(cf, h, nv, x);
    else sections<false>(cf, h, nv, x);
    unsigned char* px = stage + X_OFF + (size_t)tpos * SPT * sizeof(S);
#pragma unroll
    for (int c = 0; c < CH; ++c) VecIO<S, V>::st(px + 16 * c, &x[c * V]);
    // the thread that owns the last sample of the row reports the final states
    if (p.zf != nullptr && nv > 0 && (t0 + (int64_t)tpos * SPT + nv == p.T)) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        p.zf[((int64_t)k * p.B + row) * 2] = h[2 * k];
        p.zf[((int64_t)k * p.B + row) * 2 + 1] = h[2 * k + 1];
      }
    }
    Partial r; r.v[0] = S(0); return r;
  }
};

// ------------------------------------------------------------------------------------ backward
template <class S>
struct SosBwdParams {
  const S* tab; int64_t tab_stride;   // ADJOINT table
  const S* gy;
  const S* x;
  const S* mid;      // (K-1,B,T) outputs of sections 0..K-2 (coefficient gradients only)
  const S* y;
  const S* g_in;     // optional (K,B,2): gradient w.r.t. the final states
  S* grad_x;
  S* grad_zi;        // optional (K,B,2)
  uint32_t* err;     // status word of the launch
  int64_t T, B;
  int bulk;
  int want_coef;
};

template <class S, int K, int CH, int STAGES_, int NT_ = 256, int MIN_CTAS_ = 1>
struct SosBwd : SosAlg<S, K> {
  static_assert(NT_ == 128 || NT_ == 256 || NT_ == 512, "a tile is 2^7, 2^8 or 2^9 thread units");
  using Alg = SosAlg<S, K>;
  using D = SosDims<K>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 5 * K>;   // per section: sum gy x, sum x lam0, sum x lam1, sum y lam0, sum y lam1
  using Params = SosBwdParams<S>;
  using Scalar = S;
  static constexpr int V = Vec16<S>::V;
  static constexpr int NT = NT_;
  static constexpr int NW = NT / 32;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = true;
  static constexpr bool HAS_PARTIAL = true;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int NROWC = 0;
  static constexpr int G_OFF = 0;   // gy in, grad_x out
  static constexpr int ROWC_OFF = TILE * (int)sizeof(S);
  static constexpr int ROWC_BYTES = D::ROWC_SCALARS * (int)sizeof(S);
  static constexpr int STAGE_BYTES = ((ROWC_OFF + ROWC_BYTES + 127) / 128) * 128;
  static constexpr int WSPAN = 32 * SPT;
  static constexpr int WBYTES = WSPAN * (int)sizeof(S);
  static constexpr int RING = 3;   // per warp: arrays Z_{k+1}, Z_k in use, Z_{k-1} on its way
  static constexpr int BAR_OFF = NW * RING * WBYTES;
  static constexpr int EXTRA_SMEM = BAR_OFF + NW * (K + 1) * 8;
  static __device__ __forceinline__ void row_constants(const Params&, int64_t, S*) {}
  static __device__ __forceinline__ typename Alg::Ctx ctx_stage(const unsigned char* stage) {
    return typename Alg::Ctx{reinterpret_cast<const S*>(stage + ROWC_OFF) + D::COEFN, true};
  }
  static __device__ __forceinline__ typename Alg::Ctx ctx_row(const Params& p, int64_t row) {
    return typename Alg::Ctx{p.tab + row * p.tab_stride + D::COEFN, false};
  }
  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    io.load(G_OFF, p.gy + row * p.T + t0, bytes);
    io.load(ROWC_OFF, p.tab + row * p.tab_stride, ROWC_BYTES);
    io.store(G_OFF, p.grad_x + row * p.T + t0, bytes);
  }
  // the gradient entering through the final states is injected by the thread that owns sample T-1
  static __device__ __forceinline__ State row_init(const Params&, int64_t) { return Alg::zero_state(); }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.grad_zi) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        p.grad_zi[((int64_t)k * p.B + row) * 2] = s.v[2 * (K - 1 - k)];
        p.grad_zi[((int64_t)k * p.B + row) * 2 + 1] = s.v[2 * (K - 1 - k) + 1];
      }
    }
  }
  // Z_0 = x, Z_m = output of section m-1 (Z_K = y): section k reads Z_k (input) and Z_{k+1} (output)
  static __device__ __forceinline__ const S* zrow(const Params& p, int m, int64_t row) {
    if (m == 0) return p.x + row * p.T;
    if (m == K) return p.y + row * p.T;
    return p.mid + ((int64_t)(m - 1) * p.B + row) * p.T;
  }
  static __device__ __forceinline__ uint64_t* bar_of(unsigned char* extra, int warp, int m) {
    return reinterpret_cast<uint64_t*>(extra + BAR_OFF) + warp * (K + 1) + m;
  }
  static __device__ __forceinline__ unsigned char* buf_of(unsigned char* extra, int warp, int m) {
    return extra + (size_t)(warp * RING + (m % RING)) * WBYTES;
  }
  static __device__ __forceinline__ void init_extra(unsigned char* extra) {
    uint64_t* bars = reinterpret_cast<uint64_t*>(extra + BAR_OFF);
    for (int i = 0; i < NW * (K + 1); ++i) mbar_init(&bars[i], 1);
  }
  static __device__ __forceinline__ void warp_span(int warp, int nvalid, int& wfirst, int& wvalid) {
    wfirst = (NT - 32 * (warp + 1)) * SPT;   // time runs against the thread index
    wvalid = nvalid - wfirst;
    wvalid = wvalid < 0 ? 0 : (wvalid > WSPAN ? WSPAN : wvalid);
  }
  // one lane: request the warp's part of array Z_m of the tile (every array once per tile)
  static __device__ __forceinline__ void request(const Params& p, unsigned char* extra, int warp, int m,
                                                 int64_t row, int64_t t0, int wfirst, int wvalid) {
    uint64_t* bar = bar_of(extra, warp, m);
    if (wvalid > 0) {
      const uint32_t bytes = (uint32_t)wvalid * sizeof(S);
      mbar_arrive_expect_tx(bar, bytes);
      bulk_g2s(buf_of(extra, warp, m), zrow(p, m, row) + t0 + wfirst, bytes, bar);
    } else {
      mbar_arrive(bar);
    }
  }
  static __device__ __forceinline__ void prefetch(const Params& p, unsigned char* extra, uint32_t, int warp,
                                                  int lane, int64_t row, int64_t t0, int nvalid) {
    if (!p.want_coef || !p.bulk) return;
    if (lane == 0) {
      int wfirst, wvalid;
      warp_span(warp, nvalid, wfirst, wvalid);
      fence_proxy_async_smem();
      request(p, extra, warp, K, row, t0, wfirst, wvalid);
      request(p, extra, warp, K - 1, row, t0, wfirst, wvalid);
    }
  }
  // All K sections (K-1 down to 0) in descending time as a skewed wavefront over the thread's
  // samples, in place in the stage (see SosFwd::wave for the structure).  l: states
  // [lam_{K-1}; ...; lam_0].  STORE: the gradient w.r.t. the cascade's input replaces g.
  // GUARD: samples >= nv are skipped (they are not run with zero drive: a state injected at the
  // end of the row must not move).
  template <bool GUARD, bool STORE>
  static __device__ __forceinline__ void wave(const S* cf, S* l, int nv, unsigned char* gs) {
    BqCoef<S> c[K];
#pragma unroll
    for (int q = 0; q < K; ++q) c[q].load(reinterpret_cast<const unsigned char*>(cf + 5 * (K - 1 - q)));
    S carry[K][V];
#pragma unroll
    for (int q = 0; q < K; ++q)
#pragma unroll
      for (int i = 0; i < V; ++i) carry[q][i] = S(0);
#pragma unroll 1
    for (int st = 0; st < CH + K - 1; ++st) {
#pragma unroll
      for (int q = K - 1; q >= 0; --q) {
        const int u = CH - 1 - (st - q);
        if (u >= 0 && u < CH) {
          S v[V];
          if (q == 0) {
            VecIO<S, V>::ld(gs + 16 * u, v);
          } else {
#pragma unroll
            for (int i = 0; i < V; ++i) v[i] = carry[q - 1][i];
          }
          S l0 = l[2 * q], l1 = l[2 * q + 1];
#pragma unroll
          for (int i = V - 1; i >= 0; --i) {
            if (!GUARD || u * V + i < nv) {
              const S gj = v[i];
              v[i] = c[q].b0 * gj + c[q].B0 * l0 + c[q].B1 * l1;
              const S t = c[q].na2 * l1 + gj;   // off the chain through l0
              l1 = l0;
              l0 = c[q].na1 * l0 + t;
            }
          }
          l[2 * q] = l0;
          l[2 * q + 1] = l1;
#pragma unroll
          for (int i = 0; i < V; ++i) carry[q][i] = v[i];
          if (STORE && q == K - 1) VecIO<S, V>::st(gs + 16 * u, v);
        }
      }
    }
  }
  // one section over the thread's samples in descending time, in place in the stage, with the five
  // sums (independent chains: this loop has instruction-level parallelism of its own).  xs, ys:
  // the section's input and output in the warp's buffers.
  template <bool GUARD>
  static __device__ __forceinline__ void section_sums(const BqCoef<S>& k, S& l0, S& l1, int nv, unsigned char* gs,
                                                      const unsigned char* xs, const unsigned char* ys, S* acc) {
    S a0 = S(0), a1 = S(0), a2 = S(0), a3 = S(0), a4 = S(0);
#pragma unroll 1
    for (int u = CH - 1; u >= 0; --u) {
      S gv[V], xv[V], yv[V];
      VecIO<S, V>::ld(gs + 16 * u, gv);
      VecIO<S, V>::ld(xs + 16 * u, xv);
      VecIO<S, V>::ld(ys + 16 * u, yv);
#pragma unroll
      for (int i = V - 1; i >= 0; --i) {
        if (!GUARD || u * V + i < nv) {
          const S gj = gv[i];
          gv[i] = k.b0 * gj + k.B0 * l0 + k.B1 * l1;
          a0 += gj * xv[i];
          a1 += xv[i] * l0;
          a2 += xv[i] * l1;
          a3 += yv[i] * l0;
          a4 += yv[i] * l1;
          const S t = k.na2 * l1 + gj;   // off the chain through l0
          l1 = l0;
          l0 = k.na1 * l0 + t;
        }
      }
      VecIO<S, V>::st(gs + 16 * u, gv);
    }
    acc[0] = a0; acc[1] = a1; acc[2] = a2; acc[3] = a3; acc[4] = a4;
  }
  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t t0, int nvalid) {
    int nv = nvalid - tpos * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    const S* cf = reinterpret_cast<const S*>(stage + ROWC_OFF);
    const bool owner = p.g_in != nullptr && nv > 0 && (t0 + (int64_t)tpos * SPT + nv == p.T);
    Map m;
#pragma unroll
    for (int i = 0; i < Alg::NS; ++i) m.v[i] = S(0);
    if (owner) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        m.v[2 * (K - 1 - k)] = __ldg(p.g_in + ((int64_t)k * p.B + row) * 2);
        m.v[2 * (K - 1 - k) + 1] = __ldg(p.g_in + ((int64_t)k * p.B + row) * 2 + 1);
      }
    }
    unsigned char* gs = const_cast<unsigned char*>(stage) + G_OFF + (size_t)tpos * SPT * sizeof(S);
    if (nvalid == TILE) {
      // the common case, unrolled with the samples in registers (fewest instructions)
      S g[SPT];
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<S, V>::ld(gs + 16 * c, &g[c * V]);
      sections_reg(cf, m.v, g);
    } else {
      wave<true, false>(cf, m.v, nv, gs);
    }
    m.v[Alg::NS] = LenCodec<S>::enc(1);
    return m;
  }
  // wave<false, false> with the samples in registers and every loop unrolled
  static __device__ __forceinline__ void sections_reg(const S* cf, S* l, S* g) {
    BqCoef<S> c[K];
#pragma unroll
    for (int q = 0; q < K; ++q) c[q].load(reinterpret_cast<const unsigned char*>(cf + 5 * (K - 1 - q)));
#pragma unroll
    for (int st = 0; st < CH + K - 1; ++st) {
#pragma unroll
      for (int q = K - 1; q >= 0; --q) {
        const int u = CH - 1 - (st - q);
        if (u >= 0 && u < CH) {
          S l0 = l[2 * q], l1 = l[2 * q + 1];
#pragma unroll
          for (int i = V - 1; i >= 0; --i) {
            const S gj = g[u * V + i];
            g[u * V + i] = c[q].b0 * gj + c[q].B0 * l0 + c[q].B1 * l1;
            const S t = c[q].na2 * l1 + gj;
            l1 = l0;
            l0 = c[q].na1 * l0 + t;
          }
          l[2 * q] = l0;
          l[2 * q + 1] = l1;
        }
      }
    }
  }
  static __device__ __forceinline__ Partial finish_x(const Params& p, const State& in, unsigned char* stage,
                                                     unsigned char* extra, uint32_t seq, int warp, int lane,
                                                     int64_t row, int64_t t0, int nvalid, uint64_t wait_ns) {
    const int tpos = NT - 1 - (warp * 32 + lane);
    int nv = nvalid - tpos * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    const S* cf = reinterpret_cast<const S*>(stage + ROWC_OFF);
    const bool owner = p.g_in != nullptr && nv > 0 && (t0 + (int64_t)tpos * SPT + nv == p.T);
    int wfirst, wvalid;
    warp_span(warp, nvalid, wfirst, wvalid);
    const size_t toff = (size_t)(31 - lane) * SPT * sizeof(S);   // this thread's samples inside a warp buffer
    const uint32_t par = seq & 1u;
    unsigned char* gs = stage + G_OFF + (size_t)tpos * SPT * sizeof(S);
    Partial acc;
#pragma unroll
    for (int i = 0; i < 5 * K; ++i) acc.v[i] = S(0);
    S l[Alg::NS];
#pragma unroll
    for (int i = 0; i < Alg::NS; ++i) l[i] = in.v[i];
    if (owner) {
#pragma unroll
      for (int k = 0; k < K; ++k) {
        l[2 * (K - 1 - k)] += __ldg(p.g_in + ((int64_t)k * p.B + row) * 2);
        l[2 * (K - 1 - k) + 1] += __ldg(p.g_in + ((int64_t)k * p.B + row) * 2 + 1);
      }
    }
    if (!p.want_coef) {
      if (nvalid == TILE) wave<false, true>(cf, l, SPT, gs);
      else wave<true, true>(cf, l, nv, gs);
    } else {
#pragma unroll 1
      for (int k = K - 1; k >= 0; --k) {
        const int q = K - 1 - k;
        BqCoef<S> c;
        c.load(reinterpret_cast<const unsigned char*>(cf + 5 * k));
        if (p.bulk) {
          if (k >= 1) {
            // Z_{k-1} goes where Z_{k+2} was: every lane is through with section k+1
            __syncwarp();
            if (lane == 0) {
              fence_proxy_async_smem();
              request(p, extra, warp, k - 1, row, t0, wfirst, wvalid);
            }
          }
          bool ok = true;
          if (k == K - 1) ok = mbar_wait_bounded(bar_of(extra, warp, k + 1), par, wait_ns);
          ok = mbar_wait_bounded(bar_of(extra, warp, k), par, wait_ns) && ok;
          if (!ok && lane == 0) atomicOr(p.err, kErrLoadTimeout);
        } else {
          __syncwarp();
          for (int m = (k == K - 1 ? k + 1 : k); m >= k; --m) {
            const S* src = zrow(p, m, row) + t0 + wfirst;
            S* dst = reinterpret_cast<S*>(buf_of(extra, warp, m));
            for (int w = lane; w < wvalid; w += 32) dst[w] = __ldg(src + w);
          }
          __syncwarp();
        }
        const unsigned char* xs = buf_of(extra, warp, k) + toff;
        const unsigned char* ys = buf_of(extra, warp, k + 1) + toff;
        // states and sums of section k, selected without dynamic register indexing
        S l0 = S(0), l1 = S(0);
#pragma unroll
        for (int i = 0; i < K; ++i)
          if (i == q) { l0 = l[2 * i]; l1 = l[2 * i + 1]; }
        S sums[5];
        if (nvalid == TILE) section_sums<false>(c, l0, l1, SPT, gs, xs, ys, sums);
        else section_sums<true>(c, l0, l1, nv, gs, xs, ys, sums);
#pragma unroll
        for (int i = 0; i < K; ++i)
          if (i == k) {
#pragma unroll
            for (int j = 0; j < 5; ++j) acc.v[5 * i + j] = sums[j];
          }
      }
    }
    __syncwarp();   // the warp's buffers are free for the next tile's requests
    return acc;
  }
};

}  // namespace ptb
