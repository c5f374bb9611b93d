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

template <class R>
__global__ void __launch_bounds__(kModalThreads)
modal_mix_fwd_kernel(const Cx<R>* __restrict__ w, const Cx<R>* __restrict__ w0, const Cx<R>* __restrict__ coef,
                     int coef_batched, int real_out, void* __restrict__ y, int64_t M, int64_t N, int64_t blocks_per_row) {
  const int64_t r = blockIdx.x / blocks_per_row;
  const int64_t t = (blockIdx.x % blocks_per_row) * kModalThreads + threadIdx.x;
  if (t >= N) return;
  const Cx<R>* c = coef + (coef_batched ? r * M : 0);
  Cx<R> acc(R(0));
  for (int64_t m = 0; m < M; ++m) {
    const Cx<R> v = t == 0 ? w0[r * M + m] : w[(r * M + m) * N + t - 1];
    acc += c[m] * v;
  }
  if (real_out) static_cast<R*>(y)[r * N + t] = acc.re;
  else static_cast<Cx<R>*>(y)[r * N + t] = acc;
}

template <class R>
__global__ void __launch_bounds__(kModalThreads)
modal_mix_bwd_kernel(const Cx<R>* __restrict__ w, const Cx<R>* __restrict__ w0, const Cx<R>* __restrict__ coef,
                     int coef_batched, int real_out, const void* __restrict__ gy, Cx<R>* __restrict__ grad_w,
                     Cx<R>* __restrict__ grad_w0, Cx<R>* __restrict__ partial, int64_t M, int64_t N,
                     int64_t blocks_per_row) {
  const int64_t r = blockIdx.x / blocks_per_row;
  const int64_t blk = blockIdx.x % blocks_per_row;
  const int64_t t = blk * kModalThreads + threadIdx.x;
  const bool live = t < N;
  auto upstream = [&](int64_t i) -> Cx<R> {
    if (real_out) return Cx<R>(static_cast<const R*>(gy)[r * N + i]);
    return static_cast<const Cx<R>*>(gy)[r * N + i];
  };
  const Cx<R>* c = coef + (coef_batched ? r * M : 0);
  Cx<R> g_here(R(0)), g_next(R(0));
  if (live) {
    g_here = upstream(t);
    if (t + 1 < N) g_next = upstream(t + 1);
  }
  __shared__ Cx<R> warp_sums[kModalThreads / 32];
  for (int64_t m = 0; m < M; ++m) {
    if (live) {
      grad_w[(r * M + m) * N + t] = cj(c[m]) * g_next;
      if (t == 0) grad_w0[r * M + m] = cj(c[m]) * g_here;
    }
    if (partial) {
      Cx<R> p(R(0));
      if (live) p = cj(t == 0 ? w0[r * M + m] : w[(r * M + m) * N + t - 1]) * g_here;
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
