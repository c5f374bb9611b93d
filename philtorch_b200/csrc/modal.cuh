// Output map of a state-space model evaluated in its eigenbasis (philtorch/lti/ssm.py:805-830,
// diag_state_space): the M complex modes w[r, m, t] of row r are mixed into one output
//     y[r, t] = sum_m coef[r, m] * w[r, m, t - 1],   w[r, m, -1] = w0[r, m]
// (the state BEFORE sample t), keeping only the real part when the system is real.  The
// reference forms V w for all states, shifts them with a concatenation and applies C as a
// complex batched matrix product; here the mode sum, the one-sample shift and the real part are
// one pass that reads each mode sample once (8 M bytes per output sample in complex64).
//
// Adjoint: grad_w[r, m, t] = conj(coef[r, m]) * gy[r, t + 1]  (0 for the last sample),
//          grad_w0[r, m]   = conj(coef[r, m]) * gy[r, 0],
//          grad_coef[r, m] = sum_t conj(w[r, m, t - 1]) * gy[r, t]   (per-block partial sums).
#pragma once
#include "complex.cuh"
#include <stdint.h>

namespace ptb {

constexpr int kModalThreads = 256;
constexpr int kModalSpan = 4;    // output samples per thread (blockDim apart): independent loads in flight
constexpr int kModalTile = kModalThreads * kModalSpan;

template <class R>
__global__ void __launch_bounds__(kModalThreads)
modal_mix_fwd_kernel(const Cx<R>* __restrict__ w, const Cx<R>* __restrict__ w0, const Cx<R>* __restrict__ coef,
                     int coef_batched, int real_out, void* __restrict__ y, int64_t M, int64_t N, int64_t blocks_per_row) {
  // w0 == nullptr: no delay, y[r, t] = sum_m coef[r, m] * w[r, m, t] (the transposed input map)
  const int64_t r = blockIdx.x / blocks_per_row;
  const int64_t t0 = (blockIdx.x % blocks_per_row) * kModalTile + threadIdx.x;
  const Cx<R>* c = coef + (coef_batched ? r * M : 0);
  const int64_t back = w0 ? 1 : 0;
  Cx<R> acc[kModalSpan];
#pragma unroll
  for (int k = 0; k < kModalSpan; ++k) acc[k] = Cx<R>(R(0));
  for (int64_t m = 0; m < M; ++m) {
    const Cx<R> cm = c[m];
    const Cx<R>* wm = w + (r * M + m) * N - back;
    Cx<R> v[kModalSpan];
#pragma unroll
    for (int k = 0; k < kModalSpan; ++k) {
      const int64_t t = t0 + k * kModalThreads;
      v[k] = Cx<R>(R(0));
      if (t < N) v[k] = (back && t == 0) ? w0[r * M + m] : wm[t];
    }
#pragma unroll
    for (int k = 0; k < kModalSpan; ++k) acc[k] += cm * v[k];
  }
#pragma unroll
  for (int k = 0; k < kModalSpan; ++k) {
    const int64_t t = t0 + k * kModalThreads;
    if (t < N) {
      if (real_out) static_cast<R*>(y)[r * N + t] = acc[k].re;
      else static_cast<Cx<R>*>(y)[r * N + t] = acc[k];
    }
  }
}

// u[r, m, t] = gain[r, m] * x[r, t] for a REAL signal x: the input map of the eigenbasis for a
// scalar input (philtorch/lti/ssm.py:783-788), written mode by mode without a complex copy of x.
template <class R>
__global__ void __launch_bounds__(kModalThreads)
modal_drive_fwd_kernel(const R* __restrict__ x, const Cx<R>* __restrict__ gain, int gain_batched,
                       Cx<R>* __restrict__ u, int64_t M, int64_t N, int64_t blocks_per_row) {
  const int64_t r = blockIdx.x / blocks_per_row;
  const int64_t t0 = (blockIdx.x % blocks_per_row) * kModalTile + threadIdx.x;
  const Cx<R>* g = gain + (gain_batched ? r * M : 0);
  R v[kModalSpan];
#pragma unroll
  for (int k = 0; k < kModalSpan; ++k) {
    const int64_t t = t0 + k * kModalThreads;
    v[k] = t < N ? x[r * N + t] : R(0);
  }
  for (int64_t m = 0; m < M; ++m) {
    const Cx<R> gm = g[m];
    Cx<R>* um = u + (r * M + m) * N;
#pragma unroll
    for (int k = 0; k < kModalSpan; ++k) {
      const int64_t t = t0 + k * kModalThreads;
      if (t < N) um[t] = Cx<R>(gm.re * v[k], gm.im * v[k]);
    }
  }
}

template <class R>
__global__ void __launch_bounds__(kModalThreads)
modal_mix_bwd_kernel(const Cx<R>* __restrict__ w, const Cx<R>* __restrict__ w0, const Cx<R>* __restrict__ coef,
                     int coef_batched, int real_out, const void* __restrict__ gy, Cx<R>* __restrict__ grad_w,
                     Cx<R>* __restrict__ grad_w0, Cx<R>* __restrict__ partial, int64_t M, int64_t N,
                     int64_t blocks_per_row) {
  const int64_t r = blockIdx.x / blocks_per_row;
  const int64_t blk = blockIdx.x % blocks_per_row;
  const int64_t t0 = blk * kModalTile + threadIdx.x;
  auto upstream = [&](int64_t i) -> Cx<R> {
    if (real_out) return Cx<R>(static_cast<const R*>(gy)[r * N + i]);
    return static_cast<const Cx<R>*>(gy)[r * N + i];
  };
  const Cx<R>* c = coef + (coef_batched ? r * M : 0);
  Cx<R> g_here[kModalSpan], g_next[kModalSpan];
#pragma unroll
  for (int k = 0; k < kModalSpan; ++k) {
    const int64_t t = t0 + k * kModalThreads;
    g_here[k] = Cx<R>(R(0));
    g_next[k] = Cx<R>(R(0));
    if (t < N) {
      g_here[k] = upstream(t);
      if (t + 1 < N) g_next[k] = upstream(t + 1);
    }
  }
  __shared__ Cx<R> warp_sums[kModalThreads / 32];
  for (int64_t m = 0; m < M; ++m) {
    const Cx<R> cm = cj(c[m]);
    Cx<R> p(R(0));
#pragma unroll
    for (int k = 0; k < kModalSpan; ++k) {
      const int64_t t = t0 + k * kModalThreads;
      if (t < N) {
        grad_w[(r * M + m) * N + t] = cm * g_next[k];
        if (t == 0) grad_w0[r * M + m] = cm * g_here[k];
        if (partial) p += cj(t == 0 ? w0[r * M + m] : w[(r * M + m) * N + t - 1]) * g_here[k];
      }
    }
    if (partial) {
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) p += shfl_down_s(p, s);
      if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = p;
      __syncthreads();
      if (threadIdx.x == 0) {
        Cx<R> tot(R(0));
        for (int k = 0; k < kModalThreads / 32; ++k) tot += warp_sums[k];
        partial[(r * blocks_per_row + blk) * M + m] = tot;
      }
      __syncthreads();
    }
  }
}

}  // namespace ptb
