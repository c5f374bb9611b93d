// Scan-engine policies for the 2x2 recurrence
//     h[t] = A[t] h[t-1] + x[t],   h[-1] = zi,   A row-major [a00 a01 a10 a11]
// and its adjoint
//     g[t] = gy[t] + c[t+1],  c[t] = A[t]^T g[t],  c[T] = g_in
//     grad_x = g,  grad_A[t] = g[t] (x) h[t-1],  grad_zi = c[0].
// LPV = true : A per sample, (B,T,2,2) or (T,2,2) (row stride 0)
// LPV = false: A per row, (B,2,2) or (2,2); grad_A is a sum over time, emitted as one partial
//              per tile and reduced afterwards.
// XS  = true : the input is a scalar sequence (B,T) feeding state 0 only (the reference pads it
//              with zeros to (B,T,2), philtorch/lpv/ssm.py:197-201); grad_x is then (B,T).
//
// Shared-memory access pattern: a thread owns NS consecutive samples, NS odd.  fp32: A is one
// 16-byte unit per sample (stride NS units, odd => conflict free), 2-vectors are 8-byte units
// (stride NS, odd).  fp64: A is two 16-byte units per sample, so the stride is even and threads
// i and i+4 of a quarter warp would collide; threads with bit 2 of their position set therefore
// read (and write) the two halves in the opposite order.
#pragma once
#include "first_order.cuh"

namespace ptb {

template <class S>
struct MatAffine {
  using Map = Pod<S, 6>;     // {p00 p01 p10 p11 s0 s1}
  using State = Pod<S, 2>;
  static __device__ __forceinline__ Map identity() {
    Map m; m.v[0] = S(1); m.v[1] = S(0); m.v[2] = S(0); m.v[3] = S(1); m.v[4] = S(0); m.v[5] = S(0); return m;
  }
  static __device__ __forceinline__ State zero_state() { State s; s.v[0] = S(0); s.v[1] = S(0); return s; }
  static __device__ __forceinline__ Map const_map(const State& s) {
    Map m; m.v[0] = S(0); m.v[1] = S(0); m.v[2] = S(0); m.v[3] = S(0); m.v[4] = s.v[0]; m.v[5] = s.v[1]; return m;
  }
  // apply `first`, then `second`
  static __device__ __forceinline__ Map compose(const Map& f, const Map& g) {
    Map m;
    m.v[0] = g.v[0] * f.v[0] + g.v[1] * f.v[2];
    m.v[1] = g.v[0] * f.v[1] + g.v[1] * f.v[3];
    m.v[2] = g.v[2] * f.v[0] + g.v[3] * f.v[2];
    m.v[3] = g.v[2] * f.v[1] + g.v[3] * f.v[3];
    m.v[4] = g.v[0] * f.v[4] + g.v[1] * f.v[5] + g.v[4];
    m.v[5] = g.v[2] * f.v[4] + g.v[3] * f.v[5] + g.v[5];
    return m;
  }
  static __device__ __forceinline__ State apply(const Map& m, const State& s) {
    State r;
    r.v[0] = m.v[0] * s.v[0] + m.v[1] * s.v[1] + m.v[4];
    r.v[1] = m.v[2] * s.v[0] + m.v[3] * s.v[1] + m.v[5];
    return r;
  }
  PTB_NO_CTX
};

// ---- per-sample shared-memory accessors ---------------------------------------------------------
template <class S> struct SoIO;
template <> struct SoIO<float> {
  static __device__ __forceinline__ void ld_mat(const unsigned char* base, int p, int, float* a) {
    const float4 q = *reinterpret_cast<const float4*>(base + (size_t)p * 16);
    a[0] = q.x; a[1] = q.y; a[2] = q.z; a[3] = q.w;
  }
  static __device__ __forceinline__ void st_mat(unsigned char* base, int p, int, const float* a) {
    *reinterpret_cast<float4*>(base + (size_t)p * 16) = make_float4(a[0], a[1], a[2], a[3]);
  }
  static __device__ __forceinline__ void ld_vec(const unsigned char* base, int p, float* v) {
    const float2 q = *reinterpret_cast<const float2*>(base + (size_t)p * 8);
    v[0] = q.x; v[1] = q.y;
  }
  static __device__ __forceinline__ void st_vec(unsigned char* base, int p, const float* v) {
    *reinterpret_cast<float2*>(base + (size_t)p * 8) = make_float2(v[0], v[1]);
  }
};
template <> struct SoIO<double> {
  static __device__ __forceinline__ void ld_mat(const unsigned char* base, int p, int swap, double* a) {
    const unsigned char* q = base + (size_t)p * 32;
    const double2 u = *reinterpret_cast<const double2*>(q + (swap ? 16 : 0));
    const double2 w = *reinterpret_cast<const double2*>(q + (swap ? 0 : 16));
    a[0] = swap ? w.x : u.x; a[1] = swap ? w.y : u.y; a[2] = swap ? u.x : w.x; a[3] = swap ? u.y : w.y;
  }
  static __device__ __forceinline__ void st_mat(unsigned char* base, int p, int swap, const double* a) {
    unsigned char* q = base + (size_t)p * 32;
    const double2 lo = make_double2(a[0], a[1]), hi = make_double2(a[2], a[3]);
    *reinterpret_cast<double2*>(q + (swap ? 16 : 0)) = swap ? hi : lo;
    *reinterpret_cast<double2*>(q + (swap ? 0 : 16)) = swap ? lo : hi;
  }
  static __device__ __forceinline__ void ld_vec(const unsigned char* base, int p, double* v) {
    const double2 q = *reinterpret_cast<const double2*>(base + (size_t)p * 16);
    v[0] = q.x; v[1] = q.y;
  }
  static __device__ __forceinline__ void st_vec(unsigned char* base, int p, const double* v) {
    *reinterpret_cast<double2*>(base + (size_t)p * 16) = make_double2(v[0], v[1]);
  }
};

constexpr int align128(int v) { return (v + 127) / 128 * 128; }

// ------------------------------------------------------------------------------------ forward
template <class S>
struct SoFwdParams {
  const S* A; int64_t a_row_stride;   // LPV: 4T or 0; LTI: 4 or 0
  const S* zi; int64_t zi_stride;     // 2, or 0 when shared
  const S* x;                         // (B,T,2), or (B,T) when XS
  S* y;                               // (B,T,2)
  S* zf;                              // optional (B,2)
  int64_t T;
};

template <class S, int NS, int STAGES_, int MIN_CTAS_, int NT_, bool LPV, bool XS>
struct SoFwd : MatAffine<S> {
  using Alg = MatAffine<S>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = SoFwdParams<S>;
  static constexpr int NT = NT_;
  static constexpr int SPT = NS;
  static constexpr int TILE = NT * NS;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = false;
  static constexpr bool HAS_PARTIAL = false;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int SZ = (int)sizeof(S);
  static constexpr int Y_OFF = 0;                                       // y out (x in when !XS)
  static constexpr int XS_OFF = align128(TILE * 2 * SZ);                // scalar x in (XS only)
  static constexpr int A_OFF = XS_OFF + (XS ? align128(TILE * SZ) : 0); // A in (LPV only)
  using Scalar = S;
  static constexpr int NROWC = LPV ? 0 : 4;                             // time-invariant: the row's matrix
  static constexpr int ROWC_OFF = A_OFF;
  static constexpr int STAGE_BYTES = A_OFF + (LPV ? align128(TILE * 4 * SZ) : 128);
  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    const S* q = p.A + row * p.a_row_stride;
    out[0] = __ldg(q); out[1] = __ldg(q + 1); out[2] = __ldg(q + 2); out[3] = __ldg(q + 3);
  }

  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    if (XS) io.load(XS_OFF, p.x + row * p.T + t0, (uint32_t)nvalid * SZ);
    else io.load(Y_OFF, p.x + (row * p.T + t0) * 2, (uint32_t)nvalid * 2 * SZ);
    if (LPV) io.load(A_OFF, p.A + row * p.a_row_stride + t0 * 4, (uint32_t)nvalid * 4 * SZ);
    io.store(Y_OFF, p.y + (row * p.T + t0) * 2, (uint32_t)nvalid * 2 * SZ);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s; s.v[0] = __ldg(p.zi + row * p.zi_stride); s.v[1] = __ldg(p.zi + row * p.zi_stride + 1); return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.zf) { p.zf[row * 2] = s.v[0]; p.zf[row * 2 + 1] = s.v[1]; }
  }

  // operands of sample j of this thread; masked samples are the identity map
  // (FULL: the whole thread is inside the row, the per-sample test compiles away)
  template <bool FULL>
  static __device__ __forceinline__ void sample(const Params& p, const unsigned char* stage, int pos, int nvalid,
                                                int swap, const S* arow, S* a, S* x) {
    if (FULL || pos < nvalid) {
      if (LPV) SoIO<S>::ld_mat(stage + A_OFF, pos, swap, a);
      else { a[0] = arow[0]; a[1] = arow[1]; a[2] = arow[2]; a[3] = arow[3]; }
      if (XS) { x[0] = *reinterpret_cast<const S*>(stage + XS_OFF + (size_t)pos * SZ); x[1] = S(0); }
      else SoIO<S>::ld_vec(stage + Y_OFF, pos, x);
    } else {
      a[0] = S(1); a[1] = S(0); a[2] = S(0); a[3] = S(1); x[0] = S(0); x[1] = S(0);
    }
  }
  static __device__ __forceinline__ void row_matrix(const unsigned char* stage, S* arow) {
    if (!LPV) {
      const S* q = reinterpret_cast<const S*>(stage + ROWC_OFF);
      arow[0] = q[0]; arow[1] = q[1]; arow[2] = q[2]; arow[3] = q[3];
    }
  }

  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t, int nvalid) {
    return (tpos + 1) * NS <= nvalid ? aggregate_t<true>(p, stage, tpos, row, nvalid)
                                     : aggregate_t<false>(p, stage, tpos, row, nvalid);
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t, int nvalid) {
    return (tpos + 1) * NS <= nvalid ? finish_t<true>(p, in, stage, tpos, row, nvalid)
                                     : finish_t<false>(p, in, stage, tpos, row, nvalid);
  }
  template <bool FULL>
  static __device__ __forceinline__ Map aggregate_t(const Params& p, const unsigned char* stage, int tpos,
                                                    int64_t row, int nvalid) {
    S arow[4];
    row_matrix(stage, arow);
    const int swap = (tpos >> 2) & 1;
    Map m = Alg::identity();
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      S a[4], x[2];
      sample<FULL>(p, stage, tpos * NS + j, nvalid, swap, arow, a, x);
      Map n;
      n.v[0] = a[0] * m.v[0] + a[1] * m.v[2];
      n.v[1] = a[0] * m.v[1] + a[1] * m.v[3];
      n.v[2] = a[2] * m.v[0] + a[3] * m.v[2];
      n.v[3] = a[2] * m.v[1] + a[3] * m.v[3];
      n.v[4] = a[0] * m.v[4] + a[1] * m.v[5] + x[0];
      n.v[5] = a[2] * m.v[4] + a[3] * m.v[5] + x[1];
      m = n;
    }
    return m;
  }
  template <bool FULL>
  static __device__ __forceinline__ Partial finish_t(const Params& p, const State& in, unsigned char* stage,
                                                     int tpos, int64_t row, int nvalid) {
    S arow[4];
    row_matrix(stage, arow);
    const int swap = (tpos >> 2) & 1;
    S h0 = in.v[0], h1 = in.v[1];
    S out[NS][2];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
      S a[4], x[2];
      sample<FULL>(p, stage, tpos * NS + j, nvalid, swap, arow, a, x);
      const S n0 = a[0] * h0 + a[1] * h1 + x[0];
      const S n1 = a[2] * h0 + a[3] * h1 + x[1];
      h0 = n0; h1 = n1;
      out[j][0] = h0; out[j][1] = h1;
    }
    // all of this thread's reads of the y/x slot precede its writes (same region when !XS)
#pragma unroll
    for (int j = 0; j < NS; ++j) SoIO<S>::st_vec(stage + Y_OFF, tpos * NS + j, out[j]);
    Partial r; r.v[0] = S(0); return r;
  }
};

// ------------------------------------------------------------------------------------ adjoint
template <class S>
struct SoBwdParams {
  const S* A; int64_t a_row_stride;
  const S* zi; int64_t zi_stride;
  const S* y;        // forward states (B,T,2), needed only when grad_A is wanted
  const S* gy;       // (B,T,2)
  const S* g_in;     // optional (B,2)
  S* grad_x;         // (B,T,2), or (B,T) when XS
  S* grad_A;         // LPV: (B,T,2,2); LTI: unused here
  S* grad_zi;        // optional (B,2)
  int64_t T;
  int want_gA;
  int gA_shared;     // LPV: grad_A is ONE (T,2,2) array that every row ADDS its tiles into (bulk path only)
};

template <class S, int NS, int STAGES_, int MIN_CTAS_, int NT_, bool LPV, bool XS>
struct SoBwd : MatAffine<S> {
  using Alg = MatAffine<S>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 4>;
  using Params = SoBwdParams<S>;
  static constexpr int NT = NT_;
  static constexpr int SPT = NS;
  static constexpr int TILE = NT * NS;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = true;
  static constexpr bool HAS_PARTIAL = !LPV;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int SZ = (int)sizeof(S);
  static constexpr int G_OFF = 0;                                            // gy in, grad_x out (!XS)
  static constexpr int Y_OFF = align128(TILE * 2 * SZ);                      // y in (read-only)
  static constexpr int HALO_OFF = Y_OFF + align128(TILE * 2 * SZ);           // 16 bytes ending with y[t0-1]
  static constexpr int GX_OFF = HALO_OFF + 128;                              // scalar grad_x out (XS only)
  static constexpr int A_OFF = GX_OFF + (XS ? align128(TILE * SZ) : 0);      // A in, grad_A out (LPV only)
  using Scalar = S;
  static constexpr int NROWC = LPV ? 0 : 4;
  static constexpr int ROWC_OFF = A_OFF;
  static constexpr int STAGE_BYTES = A_OFF + (LPV ? align128(TILE * 4 * SZ) : 128);
  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    const S* q = p.A + row * p.a_row_stride;
    out[0] = __ldg(q); out[1] = __ldg(q + 1); out[2] = __ldg(q + 2); out[3] = __ldg(q + 3);
  }

  static __device__ __forceinline__ void plan(const Params& p, bool bulk, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    io.load(G_OFF, p.gy + (row * p.T + t0) * 2, (uint32_t)nvalid * 2 * SZ);
    if (LPV) io.load(A_OFF, p.A + row * p.a_row_stride + t0 * 4, (uint32_t)nvalid * 4 * SZ);
    if (p.want_gA) {
      io.load(Y_OFF, p.y + (row * p.T + t0) * 2, (uint32_t)nvalid * 2 * SZ);
      if (t0 > 0) {
        if (bulk) io.load(HALO_OFF, reinterpret_cast<const char*>(p.y + (row * p.T + t0) * 2) - 16, 16);
        else io.load(HALO_OFF + 16 - 2 * SZ, p.y + (row * p.T + t0 - 1) * 2, 2 * SZ);
      }
    }
    if (XS) io.store(GX_OFF, p.grad_x + row * p.T + t0, (uint32_t)nvalid * SZ);
    else io.store(G_OFF, p.grad_x + (row * p.T + t0) * 2, (uint32_t)nvalid * 2 * SZ);
    if (LPV && p.want_gA)
      io.store(A_OFF, p.grad_A + ((p.gA_shared ? 0 : row * p.T) + t0) * 4, (uint32_t)nvalid * 4 * SZ,
               p.gA_shared ? SZ : 0);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s = Alg::zero_state();
    if (p.g_in) { s.v[0] = __ldg(p.g_in + row * 2); s.v[1] = __ldg(p.g_in + row * 2 + 1); }
    return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.grad_zi) { p.grad_zi[row * 2] = s.v[0]; p.grad_zi[row * 2 + 1] = s.v[1]; }
  }
  static __device__ __forceinline__ void row_matrix(const unsigned char* stage, S* arow) {
    if (!LPV) {
      const S* q = reinterpret_cast<const S*>(stage + ROWC_OFF);
      arow[0] = q[0]; arow[1] = q[1]; arow[2] = q[2]; arow[3] = q[3];
    }
  }
  template <bool FULL>
  static __device__ __forceinline__ void sample(const unsigned char* stage, int pos, int nvalid, int swap,
                                                const S* arow, S* a, S* g) {
    if (FULL || pos < nvalid) {
      if (LPV) SoIO<S>::ld_mat(stage + A_OFF, pos, swap, a);
      else { a[0] = arow[0]; a[1] = arow[1]; a[2] = arow[2]; a[3] = arow[3]; }
      SoIO<S>::ld_vec(stage + G_OFF, pos, g);
    } else {
      a[0] = S(1); a[1] = S(0); a[2] = S(0); a[3] = S(1); g[0] = S(0); g[1] = S(0);
    }
  }

  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t, int nvalid) {
    return (tpos + 1) * NS <= nvalid ? aggregate_t<true>(p, stage, tpos, row, nvalid)
                                     : aggregate_t<false>(p, stage, tpos, row, nvalid);
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t t0, int nvalid) {
    return (tpos + 1) * NS <= nvalid ? finish_t<true>(p, in, stage, tpos, row, t0, nvalid)
                                     : finish_t<false>(p, in, stage, tpos, row, t0, nvalid);
  }
  // map over c (time descending): c_out = A_j^T (gy_j + c_in)
  template <bool FULL>
  static __device__ __forceinline__ Map aggregate_t(const Params& p, const unsigned char* stage, int tpos,
                                                    int64_t row, int nvalid) {
    S arow[4];
    row_matrix(stage, arow);
    const int swap = (tpos >> 2) & 1;
    Map m = Alg::identity();
#pragma unroll
    for (int j = NS - 1; j >= 0; --j) {
      S a[4], g[2];
      sample<FULL>(stage, tpos * NS + j, nvalid, swap, arow, a, g);
      const S u0 = m.v[4] + g[0], u1 = m.v[5] + g[1];
      Map n;   // A^T = [a0 a2; a1 a3]
      n.v[0] = a[0] * m.v[0] + a[2] * m.v[2];
      n.v[1] = a[0] * m.v[1] + a[2] * m.v[3];
      n.v[2] = a[1] * m.v[0] + a[3] * m.v[2];
      n.v[3] = a[1] * m.v[1] + a[3] * m.v[3];
      n.v[4] = a[0] * u0 + a[2] * u1;
      n.v[5] = a[1] * u0 + a[3] * u1;
      m = n;
    }
    return m;
  }
  template <bool FULL>
  static __device__ __forceinline__ Partial finish_t(const Params& p, const State& in, unsigned char* stage,
                                                     int tpos, int64_t row, int64_t t0, int nvalid) {
    S arow[4];
    row_matrix(stage, arow);
    const int swap = (tpos >> 2) & 1;
    const int p0 = tpos * NS;
    S yv[NS][2];
    S yprev[2] = {S(0), S(0)};
    if (p.want_gA) {
#pragma unroll
      for (int j = 0; j < NS; ++j) {
        if (FULL || p0 + j < nvalid) SoIO<S>::ld_vec(stage + Y_OFF, p0 + j, yv[j]);
        else { yv[j][0] = S(0); yv[j][1] = S(0); }
      }
      if (tpos > 0) SoIO<S>::ld_vec(stage + Y_OFF, p0 - 1, yprev);
      else if (t0 > 0) {
        yprev[0] = *reinterpret_cast<const S*>(stage + HALO_OFF + 16 - 2 * SZ);
        yprev[1] = *reinterpret_cast<const S*>(stage + HALO_OFF + 16 - SZ);
      } else {
        yprev[0] = __ldg(p.zi + row * p.zi_stride);
        yprev[1] = __ldg(p.zi + row * p.zi_stride + 1);
      }
    }
    S c0 = in.v[0], c1 = in.v[1];
    Partial acc;
    acc.v[0] = acc.v[1] = acc.v[2] = acc.v[3] = S(0);
#pragma unroll
    for (int j = NS - 1; j >= 0; --j) {
      S a[4], g[2];
      sample<FULL>(stage, p0 + j, nvalid, swap, arow, a, g);
      const S g0 = g[0] + c0, g1 = g[1] + c1;
      if (XS) {
        *reinterpret_cast<S*>(stage + GX_OFF + (size_t)(p0 + j) * SZ) = g0;
      } else {
        const S gv[2] = {g0, g1};
        SoIO<S>::st_vec(stage + G_OFF, p0 + j, gv);   // own region, already read
      }
      if (p.want_gA) {
        const S y0 = j > 0 ? yv[j - 1][0] : yprev[0];
        const S y1 = j > 0 ? yv[j - 1][1] : yprev[1];
        if (LPV) {
          const S ga[4] = {g0 * y0, g0 * y1, g1 * y0, g1 * y1};
          SoIO<S>::st_mat(stage + A_OFF, p0 + j, swap, ga);   // over this thread's own coefficients
        } else if (FULL || p0 + j < nvalid) {
          acc.v[0] += g0 * y0; acc.v[1] += g0 * y1; acc.v[2] += g1 * y0; acc.v[3] += g1 * y1;
        }
      }
      c0 = a[0] * g0 + a[2] * g1;
      c1 = a[1] * g0 + a[3] * g1;
    }
    return acc;
  }
};

}  // namespace ptb
