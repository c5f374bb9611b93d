// Scan-engine policies for the scalar first-order recurrence
//     y[t] = a[t] * y[t-1] + x[t],   y[-1] = zi
// and its adjoint
//     g[t] = gy[t] + c[t+1],  c[t] = a[t] * g[t],  c[T] = g_in (0 unless the row continues to the right)
//     grad_x = g,  grad_a[t] = g[t] * y[t-1],  grad_zi = c[0].
// For complex scalars (Cx<float>, Cx<double>) the adjoint uses conj(a) and conj(y[t-1]).
// LPV = true : a is per sample, (B,T) or (T,) (row stride 0)
// LPV = false: a is per row, (B,) or a single value (row stride 0); grad_a is a sum over time,
//              emitted as one partial per tile and reduced by reduce_partials_kernel.
#pragma once
#include "scan_engine.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace ptb {

// the real type a scalar is made of (complex sums add component-wise)
template <class S> struct RealOfScalar { using type = S; };
template <class R> struct RealOfScalar<Cx<R>> { using type = R; };

template <class S, int N_>
struct Pod {
  static constexpr int N = N_;
  S v[N_];
};

template <class S> struct Vec16;
template <> struct Vec16<float> { using type = float4; static constexpr int V = 4; };
template <> struct Vec16<double> { using type = double2; static constexpr int V = 2; };

template <> struct Vec16<Cx<float>> { using type = float4; static constexpr int V = 2; };
template <> struct Vec16<Cx<double>> { using type = double2; static constexpr int V = 1; };

// ---- storage types narrower than the arithmetic type -------------------------------------------
// float16 / bfloat16 tensors are staged and stored as they are (2 bytes per sample in HBM and in
// shared memory) while the recurrence runs in float32 registers: one rounding per result instead of
// one per step, and 2 instead of 4 bytes per sample of traffic.
template <> struct Vec16<__half> { using type = uint4; static constexpr int V = 8; };
template <> struct Vec16<__nv_bfloat16> { using type = uint4; static constexpr int V = 8; };

template <class S, class G> struct Cvt {
  static __device__ __forceinline__ S in(const G& v) { return v; }
  static __device__ __forceinline__ G out(const S& v) { return v; }
};
template <> struct Cvt<float, __half> {
  static __device__ __forceinline__ float in(const __half& v) { return __half2float(v); }
  static __device__ __forceinline__ __half out(const float& v) { return __float2half_rn(v); }
};
template <> struct Cvt<float, __nv_bfloat16> {
  static __device__ __forceinline__ float in(const __nv_bfloat16& v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 out(const float& v) { return __float2bfloat16_rn(v); }
};

template <class S, int V> struct VecIO;
template <> struct VecIO<__half, 8> {
  static __device__ __forceinline__ void ld(const unsigned char* p, float* r) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); r[2 * i] = f.x; r[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void st(unsigned char* p, const float* r) {
    uint4 q;
    __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(r[2 * i], r[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = q;
  }
};
template <> struct VecIO<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void ld(const unsigned char* p, float* r) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); r[2 * i] = f.x; r[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ void st(unsigned char* p, const float* r) {
    uint4 q;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = q;
  }
};
template <> struct VecIO<Cx<float>, 2> {
  static __device__ __forceinline__ void ld(const unsigned char* p, Cx<float>* r) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    r[0] = Cx<float>(q.x, q.y); r[1] = Cx<float>(q.z, q.w);
  }
  static __device__ __forceinline__ void st(unsigned char* p, const Cx<float>* r) {
    *reinterpret_cast<float4*>(p) = make_float4(r[0].re, r[0].im, r[1].re, r[1].im);
  }
};
template <> struct VecIO<Cx<double>, 1> {
  static __device__ __forceinline__ void ld(const unsigned char* p, Cx<double>* r) {
    const double2 q = *reinterpret_cast<const double2*>(p);
    r[0] = Cx<double>(q.x, q.y);
  }
  static __device__ __forceinline__ void st(unsigned char* p, const Cx<double>* r) {
    *reinterpret_cast<double2*>(p) = make_double2(r[0].re, r[0].im);
  }
};
template <> struct VecIO<float, 4> {
  static __device__ __forceinline__ void ld(const unsigned char* p, float* r) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    r[0] = q.x; r[1] = q.y; r[2] = q.z; r[3] = q.w;
  }
  static __device__ __forceinline__ void st(unsigned char* p, const float* r) {
    *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
  }
};
template <> struct VecIO<double, 2> {
  static __device__ __forceinline__ void ld(const unsigned char* p, double* r) {
    const double2 q = *reinterpret_cast<const double2*>(p);
    r[0] = q.x; r[1] = q.y;
  }
  static __device__ __forceinline__ void st(unsigned char* p, const double* r) {
    *reinterpret_cast<double2*>(p) = make_double2(r[0], r[1]);
  }
};

// Algebra of scalar affine maps m(h) = P*h + s, stored as v = {P, s}.
template <class S>
struct ScalarAffine {
  using Map = Pod<S, 2>;
  using State = Pod<S, 1>;
  static __device__ __forceinline__ Map identity() { Map m; m.v[0] = S(1); m.v[1] = S(0); return m; }
  static __device__ __forceinline__ State zero_state() { State s; s.v[0] = S(0); return s; }
  static __device__ __forceinline__ Map const_map(const State& s) { Map m; m.v[0] = S(0); m.v[1] = s.v[0]; return m; }
  // apply `first`, then `second`
  static __device__ __forceinline__ Map compose(const Map& first, const Map& second) {
    Map m;
    m.v[0] = second.v[0] * first.v[0];
    m.v[1] = second.v[0] * first.v[1] + second.v[1];
    return m;
  }
  static __device__ __forceinline__ State apply(const Map& m, const State& s) {
    State r; r.v[0] = m.v[0] * s.v[0] + m.v[1]; return r;
  }
  PTB_NO_CTX
};

// ------------------------------------------------------------------------------------ forward
// S: arithmetic type; G: type of the arrays in memory (S itself, or a 2-byte float with S = float)
template <class G>
struct FoFwdParams {
  const G* a; int64_t a_row_stride;   // LPV: T or 0; LTI: 1 or 0
  const G* zi; int64_t zi_stride;     // 1, or 0 when one value is shared by all rows
  const G* x;
  G* y;
  G* zf;                              // optional (B,) final state
  int64_t T;
};

template <class S, int CH, int STAGES_, int MIN_CTAS_, int LBW_, bool LPV, class G = S>
struct FoFwd : ScalarAffine<S> {
  using Alg = ScalarAffine<S>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = FoFwdParams<G>;
  using Scalar = S;
  using C = Cvt<S, G>;
  static constexpr int V = Vec16<G>::V;
  static constexpr int NT = 256;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = LBW_;
  static constexpr bool REVERSE = false;
  static constexpr bool HAS_PARTIAL = false;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int SLOT = TILE * (int)sizeof(G);
  static constexpr int X_OFF = 0;
  static constexpr int A_OFF = SLOT;
  static constexpr int NROWC = LPV ? 0 : 1;                 // time-invariant: the row's coefficient
  static constexpr int ROWC_OFF = LPV ? 2 * SLOT : SLOT;
  static constexpr int STAGE_BYTES = ROWC_OFF + (LPV ? 0 : 128);
  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    out[0] = C::in(ld_ro(p.a + row * p.a_row_stride));
  }

  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(G);
    io.load(X_OFF, p.x + row * p.T + t0, bytes);
    if (LPV) io.load(A_OFF, p.a + row * p.a_row_stride + t0, bytes);
    io.store(X_OFF, p.y + row * p.T + t0, bytes);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s; s.v[0] = C::in(ld_ro(p.zi + row * p.zi_stride)); return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.zf) p.zf[row] = C::out(s.v[0]);
  }

  struct Regs {
    S x[SPT];
    S a[LPV ? SPT : 1];
    int nv;
    // time-invariant: the row's coefficient, 1 for masked samples (only tail threads have any)
    __device__ __forceinline__ S coef(int j) const { return LPV ? a[j] : ((nv == SPT || j < nv) ? a[0] : S(1)); }
    __device__ __forceinline__ void load(const Params& p, const unsigned char* stage, int tpos, int64_t row,
                                         int nvalid) {
      const int p0 = tpos * SPT;
      nv = nvalid - p0;
      nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
      const unsigned char* px = stage + X_OFF + (size_t)p0 * sizeof(G);
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<G, V>::ld(px + 16 * c, &x[c * V]);
      if (LPV) {
        const unsigned char* pa = stage + A_OFF + (size_t)p0 * sizeof(G);
#pragma unroll
        for (int c = 0; c < CH; ++c) VecIO<G, V>::ld(pa + 16 * c, &a[c * V]);
      } else {
        a[0] = *reinterpret_cast<const S*>(stage + ROWC_OFF);
      }
      if (nv < SPT) {
#pragma unroll
        for (int j = 0; j < SPT; ++j)
          if (j >= nv) { x[j] = S(0); if (LPV) a[j] = S(1); }
      }
    }
  };

  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t, int nvalid) {
    Regs r;
    r.load(p, stage, tpos, row, nvalid);
    S P = S(1), s = S(0);
#pragma unroll
    for (int j = 0; j < SPT; ++j) { const S aj = r.coef(j); s = aj * s + r.x[j]; P *= aj; }
    Map m; m.v[0] = P; m.v[1] = s; return m;
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t, int nvalid) {
    Regs r;
    r.load(p, stage, tpos, row, nvalid);
    S h = in.v[0];
#pragma unroll
    for (int j = 0; j < SPT; ++j) { h = r.coef(j) * h + r.x[j]; r.x[j] = h; }
    unsigned char* px = stage + X_OFF + (size_t)tpos * SPT * sizeof(G);
#pragma unroll
    for (int c = 0; c < CH; ++c) VecIO<G, V>::st(px + 16 * c, &r.x[c * V]);
    Partial out; out.v[0] = S(0); return out;
  }
};

// ------------------------------------------------------------------------------------ adjoint
template <class G, class S = G>
struct FoBwdParams {
  const G* a; int64_t a_row_stride;
  const G* zi; int64_t zi_stride;
  const G* y;        // forward output, needed only when grad_a is wanted
  const G* gy;       // upstream gradient
  const G* g_in;     // optional (B,): adjoint state entering from the right of the last sample
  G* grad_x;
  G* grad_a;         // LPV: (B,T) per-sample; LTI: unused here (partials go to the workspace)
  int64_t ga_row_stride;   // LPV: T, or 0 when the rows share one (T,) gradient array: tiles are then ADDED into it
                           // by bulk reduce copies (bulk path only; the array must start at zero)
  G* grad_zi;        // optional (B,)
  int64_t T;
  int want_ga;
  S fuse_scale;      // FUSE: the kernel writes fuse_scale * (g + y - gy) instead of g (y = any second signal)
  // time-invariant, small launches: the grid's last warp adds the per-tile sums up itself (no second launch)
  G* ga_out = nullptr;     // (B,) if ga_batched else (1,)
  int ga_batched = 0;
  int fuse_reduce = 0;
};

// FUSE (time-invariant use): the result of the reverse-time recurrence is combined with its own
// input and one more signal on the way out, out[t] = fuse_scale * (g[t] + y[t] - gy[t]): the
// symmetric two-pass filters (causal pass y, then this pass) need no separate combining pass.
template <class S, int CH, int STAGES_, int MIN_CTAS_, int LBW_, bool LPV, bool FUSE = false, class G = S>
struct FoBwd : ScalarAffine<S> {
  using Alg = ScalarAffine<S>;
  using typename Alg::Map;
  using typename Alg::State;
  using Partial = Pod<S, 1>;
  using Params = FoBwdParams<G, S>;
  using Scalar = S;
  using C = Cvt<S, G>;
  static constexpr int V = Vec16<G>::V;
  static constexpr int NT = 256;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = LBW_;
  static constexpr bool REVERSE = true;
  static constexpr bool HAS_PARTIAL = !LPV;
  static constexpr bool FINAL_REDUCE = !LPV && std::is_arithmetic<S>::value;   // real scalars only
  static __device__ __forceinline__ bool wants_final_reduce(const Params& p) { return p.fuse_reduce != 0; }
  // One warp: grad_a = sum over the tiles of a row (rows too when the coefficient is shared) of the
  // per-tile sums, in double, every lane in a fixed order.  partial: [B][nchunks] scalars.
  static __device__ void final_reduce(const Params& p, const void* partial, uint32_t B, uint32_t nchunks, int lane) {
    if constexpr (FINAL_REDUCE) {
      const volatile S* part = static_cast<const volatile S*>(partial);
      if (p.ga_batched) {
        for (uint32_t row = lane; row < B; row += 32) {
          double acc = 0.0;
          for (uint32_t c = 0; c < nchunks; ++c) acc += (double)part[(size_t)row * nchunks + c];
          p.ga_out[row] = C::out((S)acc);
        }
      } else {
        double acc = 0.0;
        const size_t total = (size_t)B * nchunks;
        for (size_t i = lane; i < total; i += 32) acc += (double)part[i];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
        if (lane == 0) p.ga_out[0] = C::out((S)acc);
      }
    }
  }
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int SLOT = TILE * (int)sizeof(G);
  static constexpr int G_OFF = 0;                       // gy in, grad_x out
  static constexpr int Y_OFF = SLOT;                    // y in (read-only)
  static constexpr int HALO_OFF = 2 * SLOT;             // 16 bytes ending with y[t0-1]
  static constexpr int A_OFF = 2 * SLOT + 128;          // a in, grad_a out (LPV)
  static constexpr int NROWC = LPV ? 0 : 1;
  static constexpr int ROWC_OFF = HALO_OFF + 64;         // second half of the halo line
  static constexpr int STAGE_BYTES = (LPV ? 3 * SLOT : 2 * SLOT) + 128;
  static __device__ __forceinline__ void row_constants(const Params& p, int64_t row, S* out) {
    out[0] = C::in(ld_ro(p.a + row * p.a_row_stride));
  }

  static __device__ __forceinline__ void plan(const Params& p, bool bulk, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(G);
    // every slot is planned unconditionally, with zero bytes when it is not wanted (the engine skips
    // those): the number of copies then does not depend on run-time data and the plan stays in registers
    io.load(G_OFF, p.gy + row * p.T + t0, bytes);
    if (LPV) io.load(A_OFF, p.a + row * p.a_row_stride + t0, bytes);
    const bool want_y = FUSE || p.want_ga;
    io.load(Y_OFF, p.y + row * p.T + t0, want_y ? bytes : 0u);
    const bool halo = p.want_ga && t0 > 0;
    if (bulk) io.load(HALO_OFF, p.y + row * p.T + t0 - V, halo ? 16u : 0u);
    else io.load(HALO_OFF + 16 - (int)sizeof(G), p.y + row * p.T + t0 - 1, halo ? (uint32_t)sizeof(G) : 0u);
    // grad_x is optional (coefficient gradients only): a store of zero bytes is skipped by the engine.  The
    // slot itself stays unconditional: a plan whose number of stores depends on run-time data keeps the
    // compiler from holding it in registers (measured: +2 % on the adjoint kernel).
    io.store(G_OFF, p.grad_x + row * p.T + t0, p.grad_x ? bytes : 0u);
    if (LPV)
      io.store(A_OFF, p.grad_a + row * p.ga_row_stride + t0, p.want_ga ? bytes : 0u,
               p.ga_row_stride == 0 ? (int)sizeof(typename RealOfScalar<S>::type) : 0);
  }
  static __device__ __forceinline__ State row_init(const Params& p, int64_t row) {
    State s; s.v[0] = p.g_in ? C::in(ld_ro(p.g_in + row)) : S(0); return s;
  }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    if (p.grad_zi) p.grad_zi[row] = C::out(s.v[0]);
  }

  struct Regs {
    S g[SPT];
    S a[LPV ? SPT : 1];
    int nv;
    // time-invariant: the row's coefficient, 1 for masked samples (only tail threads have any)
    __device__ __forceinline__ S coef(int j) const { return LPV ? a[j] : ((nv == SPT || j < nv) ? a[0] : S(1)); }
    __device__ __forceinline__ void load(const Params& p, const unsigned char* stage, int tpos, int64_t row,
                                         int nvalid) {
      const int p0 = tpos * SPT;
      nv = nvalid - p0;
      nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
      const unsigned char* pg = stage + G_OFF + (size_t)p0 * sizeof(G);
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<G, V>::ld(pg + 16 * c, &g[c * V]);
      if (LPV) {
        const unsigned char* pa = stage + A_OFF + (size_t)p0 * sizeof(G);
#pragma unroll
        for (int c = 0; c < CH; ++c) VecIO<G, V>::ld(pa + 16 * c, &a[c * V]);
#pragma unroll
        for (int j = 0; j < SPT; ++j) a[j] = cj(a[j]);   // the adjoint runs on conj(a) (no-op for reals)
      } else {
        a[0] = cj(*reinterpret_cast<const S*>(stage + ROWC_OFF));   // row constants are staged in S
      }
      if (nv < SPT) {
#pragma unroll
        for (int j = 0; j < SPT; ++j)
          if (j >= nv) { g[j] = S(0); if (LPV) a[j] = S(1); }
      }
    }
  };

  // map over c (time descending): c_out = a_j * (gy_j + c_in)
  static __device__ __forceinline__ Map aggregate(const Params& p, const unsigned char* stage, int tpos,
                                                  int64_t row, int64_t, int nvalid) {
    Regs r;
    r.load(p, stage, tpos, row, nvalid);
    S P = S(1), s = S(0);
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) { const S aj = r.coef(j); s = aj * (s + r.g[j]); P *= aj; }
    Map m; m.v[0] = P; m.v[1] = s; return m;
  }
  static __device__ __forceinline__ Partial finish(const Params& p, const State& in, unsigned char* stage,
                                                   int tpos, int64_t row, int64_t t0, int nvalid) {
    Regs r;
    r.load(p, stage, tpos, row, nvalid);
    S y[SPT];
    S yprev = S(0);
    const int p0 = tpos * SPT;
    unsigned char* py = stage + Y_OFF + (size_t)p0 * sizeof(G);
    if (FUSE && !p.want_ga) {
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<G, V>::ld(py + 16 * c, &y[c * V]);
    }
    if (p.want_ga) {
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<G, V>::ld(py + 16 * c, &y[c * V]);
      if (tpos > 0) yprev = C::in(*reinterpret_cast<const G*>(py - sizeof(G)));
      else if (t0 > 0) yprev = C::in(*reinterpret_cast<const G*>(stage + HALO_OFF + 16 - sizeof(G)));
      else yprev = C::in(ld_ro(p.zi + row * p.zi_stride));
    }
    S c = in.v[0];
    S acc = S(0);
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      const S gyj = r.g[j];
      const S gj = gyj + c;
      r.g[j] = FUSE ? p.fuse_scale * (gj + y[j] - gyj) : gj;
      c = r.coef(j) * gj;
      if (p.want_ga) {
        const S yp = cj(j > 0 ? y[j - 1] : yprev);
        if (LPV) y[j] = gj * yp;
        else if (j < r.nv) acc += gj * yp;
      }
    }
    unsigned char* pg = stage + G_OFF + (size_t)p0 * sizeof(G);
#pragma unroll
    for (int c2 = 0; c2 < CH; ++c2) VecIO<G, V>::st(pg + 16 * c2, &r.g[c2 * V]);
    if (LPV && p.want_ga) {
      // grad_a goes over this thread's own coefficients: the y slot stays read-only, because the
      // neighbouring thread reads its previous sample from it at an unsynchronised time
      unsigned char* pa = stage + A_OFF + (size_t)p0 * sizeof(G);
#pragma unroll
      for (int c2 = 0; c2 < CH; ++c2) VecIO<G, V>::st(pa + 16 * c2, &y[c2 * V]);
    }
    Partial out; out.v[0] = acc; return out;
  }
};

}  // namespace ptb

namespace ptb {

// ------------------------------------------------------------------------------------ carry pass
// Total affine map of every row, (product of a, end state from a zero start), without writing
// the sequence: the first pass of a scan whose time axis is split across devices.  The carried
// "state" is itself a map S = (P, s); a tile acts on it by composition, S -> m o S.  Operators on
// maps are kept as three numbers (alpha, beta, gamma): S -> (alpha S.P + beta, alpha S.s + gamma),
// which also represents the constant operators the look-back needs.
// REVERSE_ = false: maps of the forward recurrence, offsets x.
// REVERSE_ = true : maps of the adjoint recurrence over c, offsets a*gy, time descending.
// WRITE_   = true : (forward only) additionally writes the sequence y started from a ZERO state,
//                   i.e. the local scan of a time shard and its total map in one pass.
template <class S>
struct FoCarryParams {
  const S* a; int64_t a_row_stride;
  const S* x;        // x (forward) or gy (adjoint)
  S* y;              // WRITE_ only: (B,T) zero-start outputs
  S* carry;          // (B,2): {product of a over the row, end state from a zero start}
  int64_t T;
};

template <class S, int CH, int STAGES_, int MIN_CTAS_, bool REVERSE_, bool WRITE_ = false>
struct FoCarry {
  static_assert(!(REVERSE_ && WRITE_), "the writing variant is forward only");
  using Map = Pod<S, 3>;
  using State = Pod<S, 2>;
  using Partial = Pod<S, 1>;
  using Params = FoCarryParams<S>;
  static constexpr int V = Vec16<S>::V;
  static constexpr int NT = 256;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int STAGES = STAGES_;
  static constexpr int MIN_CTAS = MIN_CTAS_;
  static constexpr int LBW = 1;
  static constexpr bool REVERSE = REVERSE_;
  static constexpr bool HAS_PARTIAL = false;
  static constexpr int SLOT_WORDS = Words<Map>::W;
  static constexpr int SLOT = TILE * (int)sizeof(S);
  static constexpr int X_OFF = 0;
  static constexpr int A_OFF = SLOT;
  static constexpr int STAGE_BYTES = 2 * SLOT;
  using Scalar = S;
  static constexpr int NROWC = 0;
  static constexpr int ROWC_OFF = 0;
  static __device__ __forceinline__ void row_constants(const Params&, int64_t, S*) {}

  static __device__ __forceinline__ Map identity() { Map m; m.v[0] = S(1); m.v[1] = S(0); m.v[2] = S(0); return m; }
  static __device__ __forceinline__ State zero_state() { State s; s.v[0] = S(1); s.v[1] = S(0); return s; }
  static __device__ __forceinline__ Map const_map(const State& s) {
    Map m; m.v[0] = S(0); m.v[1] = s.v[0]; m.v[2] = s.v[1]; return m;
  }
  static __device__ __forceinline__ Map compose(const Map& f, const Map& g) {   // f first, then g
    Map m;
    m.v[0] = g.v[0] * f.v[0];
    m.v[1] = g.v[0] * f.v[1] + g.v[1];
    m.v[2] = g.v[0] * f.v[2] + g.v[2];
    return m;
  }
  static __device__ __forceinline__ State apply(const Map& m, const State& s) {
    State r; r.v[0] = m.v[0] * s.v[0] + m.v[1]; r.v[1] = m.v[0] * s.v[1] + m.v[2]; return r;
  }
  PTB_NO_CTX
  static __device__ __forceinline__ void plan(const Params& p, bool, int64_t row, int64_t t0, int nvalid,
                                              IoPlan& io) {
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    io.load(X_OFF, p.x + row * p.T + t0, bytes);
    io.load(A_OFF, p.a + row * p.a_row_stride + t0, bytes);
    if (WRITE_) io.store(X_OFF, p.y + row * p.T + t0, bytes);
  }
  static __device__ __forceinline__ State row_init(const Params&, int64_t) { return zero_state(); }
  static __device__ __forceinline__ void row_final(const Params& p, int64_t row, const State& s) {
    p.carry[row * 2] = s.v[0];
    p.carry[row * 2 + 1] = s.v[1];
  }
  static __device__ __forceinline__ Map aggregate(const Params&, const unsigned char* stage, int tpos, int64_t,
                                                  int64_t, int nvalid) {
    const int p0 = tpos * SPT;
    int nv = nvalid - p0;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    S x[SPT], a[SPT];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      VecIO<S, V>::ld(stage + X_OFF + (size_t)p0 * sizeof(S) + 16 * c, &x[c * V]);
      VecIO<S, V>::ld(stage + A_OFF + (size_t)p0 * sizeof(S) + 16 * c, &a[c * V]);
    }
    S P = S(1), s = S(0);
    if (!REVERSE) {
#pragma unroll
      for (int j = 0; j < SPT; ++j)
        if (j < nv) { s = a[j] * s + x[j]; P *= a[j]; }
    } else {
#pragma unroll
      for (int j = SPT - 1; j >= 0; --j)
        if (j < nv) { s = a[j] * (s + x[j]); P *= a[j]; }
    }
    Map m; m.v[0] = P; m.v[1] = S(0); m.v[2] = s; return m;   // S -> (P S.P, P S.s + s)
  }
  static __device__ __forceinline__ Partial finish(const Params&, const State& in, unsigned char* stage, int tpos,
                                                   int64_t, int64_t, int nvalid) {
    if (WRITE_) {
      const int p0 = tpos * SPT;
      int nv = nvalid - p0;
      nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
      S x[SPT], a[SPT];
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        VecIO<S, V>::ld(stage + X_OFF + (size_t)p0 * sizeof(S) + 16 * c, &x[c * V]);
        VecIO<S, V>::ld(stage + A_OFF + (size_t)p0 * sizeof(S) + 16 * c, &a[c * V]);
      }
      S h = in.v[1];   // the state reached from a zero start
#pragma unroll
      for (int j = 0; j < SPT; ++j)
        if (j < nv) { h = a[j] * h + x[j]; x[j] = h; }
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<S, V>::st(stage + X_OFF + (size_t)p0 * sizeof(S) + 16 * c, &x[c * V]);
    }
    Partial r; r.v[0] = S(0); return r;
  }
};

}  // namespace ptb
