// Fix-up kernels of the time-varying 2x2 recurrence  h[t] = A[t] h[t-1] + x[t]  whose rows are cut
// into S segments along time (the matrix-valued counterpart of shard_fixup.cuh; one device).
//
// Every segment is first scanned from a ZERO incoming state by the small-CTA kernel of
// so_small.cuh, which also writes the product of every tile's matrices; a fold turns those into
// the segment's total matrix P (the ordered product of its A[t]), and the segment's end state from
// zero, e, is the kernel's final state.  The true state entering segment j is the fold
//     s <- P_i s + e_i   over the segments i < j   (s = zi before the first),
// and by linearity the true output is  y[t] += k[t],  k[t] = A[t] k[t-1],  k[-1] = s.
// For contracting systems k underflows to EXACTLY (0, 0) after a few thousand samples and stays
// there, so the walk goes block by block from the segment's start and stops at the first block that
// k enters as exactly zero; nothing is approximated, and if the products never vanish the walk
// covers the whole segment.
//
// Adjoint (g[t] = gy[t] + c[t+1], c[t] = A[t]^T g[t]): segments are scanned with nothing entering
// from the right; the adjoint state entering segment j from its right is the fold
//     c <- P_i^T c + (c leaving segment i on its left)   over the segments i > j, from the last down,
// and   g[t] += d[t],  d[L-1] = c,  d[t-1] = A[t]^T d[t];   grad_x += d,  grad_A[t] += d[t] (x) h[t-1].
//
// One CTA per (row, segment); a step takes kFix2NT * kFix2SPT samples with an ordered block scan of
// 2x2 matrix products (warp shuffles + one shared-memory exchange).
#pragma once
#include "ptx.cuh"
#include "first_order.cuh"

#include <cstdint>

namespace ptb {

constexpr int kFix2NT = 256;
constexpr int kFix2SPT = 4;
constexpr int kFix2Block = kFix2NT * kFix2SPT;

template <class S> struct Mat2 { S a, b, c, d; };   // [[a, b], [c, d]]
template <class S> struct Vec2 { S x, y; };

template <class S>
__device__ __forceinline__ Mat2<S> mat2_identity() { return Mat2<S>{S(1), S(0), S(0), S(1)}; }
template <class S>
__device__ __forceinline__ Mat2<S> mat2_mul(const Mat2<S>& l, const Mat2<S>& r) {   // l r
  return Mat2<S>{l.a * r.a + l.b * r.c, l.a * r.b + l.b * r.d, l.c * r.a + l.d * r.c, l.c * r.b + l.d * r.d};
}
template <class S>
__device__ __forceinline__ Vec2<S> mat2_apply(const Mat2<S>& m, const Vec2<S>& v) {
  return Vec2<S>{m.a * v.x + m.b * v.y, m.c * v.x + m.d * v.y};
}
template <class S>
__device__ __forceinline__ Mat2<S> mat2_transpose(const Mat2<S>& m) { return Mat2<S>{m.a, m.c, m.b, m.d}; }
template <class S>
__device__ __forceinline__ Mat2<S> mat2_shfl_up(const Mat2<S>& m, int d) {
  return Mat2<S>{__shfl_up_sync(0xffffffffu, m.a, d), __shfl_up_sync(0xffffffffu, m.b, d),
                 __shfl_up_sync(0xffffffffu, m.c, d), __shfl_up_sync(0xffffffffu, m.d, d)};
}
template <class S>
__device__ __forceinline__ Mat2<S> mat2_load(const S* p) {   // four consecutive scalars, 16-byte aligned rows
  return Mat2<S>{ld_ro(p), ld_ro(p + 1), ld_ro(p + 2), ld_ro(p + 3)};
}

template <class S>
struct Fixup2Params {
  // geometry: R = B * nseg kernel rows of L samples; kernel row r = b * nseg + j
  int64_t B, nseg, L;
  const S* A;          // (R, L, 2, 2)
  const S* P;          // (R, 4): ordered product of the segment's matrices
  const S* e;          // (R, 2): forward: end state from zero; adjoint: c leaving the segment on its left
  // forward
  const S* zi;         // (B, 2)
  S* y;                // (R, L, 2) corrected in place
  S* states;           // (R, 2) out (forward) / in (adjoint): state entering every segment
  // adjoint
  int x_scalar;        // grad_x is (R, L): only component 0 of d is added
  S* grad_x;           // (R, L, 2) or (R, L), corrected in place
  S* grad_A;           // (R, L, 2, 2) corrected in place, or nullptr
  S* grad_zi;          // (B, 2) out, or nullptr
};

// Ordered exclusive product over the CTA: thread i receives  v_{i-1} ... v_1 v_0  (identity for thread 0);
// `total` receives the product over all threads (the same in every thread).
template <class S>
__device__ __forceinline__ Mat2<S> block_excl_matprod(const Mat2<S>& v, Mat2<S>* sm_warp, Mat2<S>& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Mat2<S> inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const Mat2<S> o = mat2_shfl_up(inc, d);
    if (lane >= d) inc = mat2_mul(inc, o);
  }
  Mat2<S> exc = mat2_shfl_up(inc, 1);
  if (lane == 0) exc = mat2_identity<S>();
  __syncthreads();                       // the previous step's readers are done with sm_warp
  if (lane == 31) sm_warp[warp] = inc;
  __syncthreads();
  Mat2<S> wpre = mat2_identity<S>(), tot = mat2_identity<S>();
#pragma unroll
  for (int w = 0; w < kFix2NT / 32; ++w) {
    const Mat2<S> t = sm_warp[w];
    if (w < warp) wpre = mat2_mul(t, wpre);
    tot = mat2_mul(t, tot);
  }
  total = tot;
  return mat2_mul(exc, wpre);
}

// maps {P (4), e (2)} of `n` segments staged in shared memory by all threads, folded by thread 0
template <class S, bool ADJ>
__device__ __forceinline__ Vec2<S> fold2(const Fixup2Params<S>& p, int64_t b, int64_t j, Vec2<S> start, S* sm_maps,
                                         Vec2<S>* sm_out) {
  Vec2<S> s = start;
  const int64_t n = ADJ ? p.nseg - 1 - j : j;
  for (int64_t base = 0; base < n; base += kFix2NT) {
    const int64_t k = base + threadIdx.x;   // k-th map of the walk (forward: segment k; adjoint: from the last down)
    __syncthreads();
    if (k < n) {
      const int64_t r = b * p.nseg + (ADJ ? p.nseg - 1 - k : k);
      Mat2<S> m = mat2_load(p.P + r * 4);
      if (ADJ) m = mat2_transpose(m);
      S* d = sm_maps + 6 * threadIdx.x;
      d[0] = m.a; d[1] = m.b; d[2] = m.c; d[3] = m.d;
      d[4] = ld_ro(p.e + r * 2); d[5] = ld_ro(p.e + r * 2 + 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int cnt = (int)((n - base) < kFix2NT ? (n - base) : kFix2NT);
      for (int i = 0; i < cnt; ++i) {
        const S* d = sm_maps + 6 * i;
        const Vec2<S> t{d[0] * s.x + d[1] * s.y + d[4], d[2] * s.x + d[3] * s.y + d[5]};
        s = t;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *sm_out = s;
  __syncthreads();
  return *sm_out;
}

template <class S>
__global__ void __launch_bounds__(kFix2NT) fixup2_fwd_kernel(const Fixup2Params<S> p) {
  __shared__ S sm_maps[6 * kFix2NT];
  __shared__ Mat2<S> sm_warp[kFix2NT / 32];
  __shared__ Vec2<S> sm_state;
  const int64_t R = p.B * p.nseg;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const int64_t b = r / p.nseg, j = r - b * p.nseg;
    Vec2<S> z{S(0), S(0)};
    if (threadIdx.x == 0) { z.x = p.zi[b * 2]; z.y = p.zi[b * 2 + 1]; }
    const Vec2<S> s = fold2<S, false>(p, b, j, z, sm_maps, &sm_state);
    if (threadIdx.x == 0) { p.states[r * 2] = s.x; p.states[r * 2 + 1] = s.y; }
    const S* A = p.A + r * p.L * 4;
    S* y = p.y + r * p.L * 2;
    Vec2<S> carry = s;   // k just before the block
    for (int64_t t0 = 0; t0 < p.L && (carry.x != S(0) || carry.y != S(0)); t0 += kFix2Block) {
      const int64_t t = t0 + (int64_t)threadIdx.x * kFix2SPT;
      Mat2<S> a[kFix2SPT];
      Mat2<S> run = mat2_identity<S>();
#pragma unroll
      for (int i = 0; i < kFix2SPT; ++i) {
        a[i] = mat2_identity<S>();
        if (t + i < p.L) { a[i] = mat2_load(A + (t + i) * 4); run = mat2_mul(a[i], run); }
      }
      Mat2<S> total;
      const Mat2<S> exc = block_excl_matprod(run, sm_warp, total);
      Vec2<S> k = mat2_apply(exc, carry);
#pragma unroll
      for (int i = 0; i < kFix2SPT; ++i) {
        if (t + i < p.L) {
          k = mat2_apply(a[i], k);
          y[(t + i) * 2] += k.x;
          y[(t + i) * 2 + 1] += k.y;
        }
      }
      carry = mat2_apply(total, carry);
    }
  }
}

template <class S>
__global__ void __launch_bounds__(kFix2NT) fixup2_bwd_kernel(const Fixup2Params<S> p) {
  __shared__ S sm_maps[6 * kFix2NT];
  __shared__ Mat2<S> sm_warp[kFix2NT / 32];
  __shared__ Vec2<S> sm_state;
  const int64_t R = p.B * p.nseg;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const int64_t b = r / p.nseg, j = r - b * p.nseg;
    const Vec2<S> c0 = fold2<S, true>(p, b, j, Vec2<S>{S(0), S(0)}, sm_maps, &sm_state);
    if (j == 0 && p.grad_zi && threadIdx.x == 0) {   // the adjoint state leaving the row on its left
      const Mat2<S> pt = mat2_transpose(mat2_load(p.P + r * 4));
      const Vec2<S> g = mat2_apply(pt, c0);
      p.grad_zi[b * 2] = g.x + p.e[r * 2];
      p.grad_zi[b * 2 + 1] = g.y + p.e[r * 2 + 1];
    }
    const S* A = p.A + r * p.L * 4;
    const S* y = p.y + r * p.L * 2;
    S* gA = p.grad_A ? p.grad_A + r * p.L * 4 : nullptr;
    const Vec2<S> hprev0{p.states[r * 2], p.states[r * 2 + 1]};
    Vec2<S> carry = c0;   // d of the block's last sample
    for (int64_t hi = p.L; hi > 0 && (carry.x != S(0) || carry.y != S(0)); hi -= kFix2Block) {
      // k-th sample of the descending walk: t = hi - 1 - k; d[t - 1] = A[t]^T d[t]
      const int64_t k0 = (int64_t)threadIdx.x * kFix2SPT;
      Mat2<S> at[kFix2SPT];
      Mat2<S> run = mat2_identity<S>();
#pragma unroll
      for (int i = 0; i < kFix2SPT; ++i) {
        const int64_t t = hi - 1 - (k0 + i);
        at[i] = mat2_identity<S>();
        if (t >= 0) { at[i] = mat2_transpose(mat2_load(A + t * 4)); run = mat2_mul(at[i], run); }
      }
      Mat2<S> total;
      const Mat2<S> exc = block_excl_matprod(run, sm_warp, total);
      Vec2<S> d = mat2_apply(exc, carry);
#pragma unroll
      for (int i = 0; i < kFix2SPT; ++i) {
        const int64_t t = hi - 1 - (k0 + i);
        if (t >= 0) {
          if (p.x_scalar) {
            p.grad_x[r * p.L + t] += d.x;
          } else {
            p.grad_x[(r * p.L + t) * 2] += d.x;
            p.grad_x[(r * p.L + t) * 2 + 1] += d.y;
          }
          if (gA) {
            Vec2<S> hp = hprev0;
            if (t > 0) { hp.x = ld_ro(y + (t - 1) * 2); hp.y = ld_ro(y + (t - 1) * 2 + 1); }
            gA[t * 4] += d.x * hp.x;
            gA[t * 4 + 1] += d.x * hp.y;
            gA[t * 4 + 2] += d.y * hp.x;
            gA[t * 4 + 3] += d.y * hp.y;
          }
          d = mat2_apply(at[i], d);
        }
      }
      carry = mat2_apply(total, carry);
    }
  }
}

// P of every kernel row: the ordered product of its tiles' matrix products (one thread per row).
template <class S>
__global__ void fold_tile_products_kernel(const S* __restrict__ tile_prod, int64_t R, int64_t nchunks,
                                          S* __restrict__ P) {
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  Mat2<S> acc = mat2_identity<S>();
  for (int64_t c = 0; c < nchunks; ++c) acc = mat2_mul(mat2_load(tile_prod + (r * nchunks + c) * 4), acc);
  P[r * 4] = acc.a; P[r * 4 + 1] = acc.b; P[r * 4 + 2] = acc.c; P[r * 4 + 3] = acc.d;
}

}  // namespace ptb
