// Feedback comb filter  y[t] = x[t] - a * y[t - D]  (philtorch/lti/filtering.py:15-71) without
// folding the signal: the D phases t = k D + d of a row are independent first-order recurrences,
// so a LANE owns one phase (row b, phase d).  Neighbouring lanes own neighbouring phases, so
// every step of a warp reads and writes 32 consecutive samples: the accesses are coalesced on
// the signal's own layout and each sample moves once (8 B forward, 12 B backward in fp32).
// A block is kCombWarps warps on the SAME 32 phases: the time axis is cut into super-steps of
// kCombWarps * kCombSteps steps, warp w taking the w-th run of kCombSteps steps.  Each warp scans
// its run from a zero state out of registers, the warps exchange the runs' end values through
// shared memory, and every warp adds the decayed incoming state  coef^(k+1) * h_in  to its run
// before storing it (the recurrence is time-invariant, so powers of one coefficient suffice).
// That multiplies the threads -- and the loads -- in flight per phase by kCombWarps without
// moving a byte more; the kernels are bound by exactly that (a one-thread-per-phase version ran
// at 0.66 of the copy bandwidth with 64000 phases).
// The host uses these kernels from a few thousand (row, phase) pairs on, the folded first-order
// scan otherwise.
//
// Adjoint:  g[t] = gy[t] - a * g[t + D]  (g = 0 beyond the end),  grad_x = g,
//           grad_a = - sum_t g[t] * y[t - D]   (y[t - D] = the initial state for t < D),
//           gradient of the initial state of phase d:  - a * g[d].
// Per-block partial sums of grad_a go to partial[row][block]; the host adds them up.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ptb {

constexpr int kCombWarps = 4;
constexpr int kCombThreads = 32 * kCombWarps;
constexpr int kCombSteps = 16;      // steps a warp holds in registers per super-step

// zi_mode: 0 none, 1 (D,) shared by the rows, 2 (B, D).  zi[..., k] is the output k + 1 samples
// before the start, so phase d starts from zi[..., D - 1 - d].
template <class S>
__device__ __forceinline__ S comb_initial(const S* zi, int zi_mode, int64_t row, int64_t D, int64_t d) {
  if (zi_mode == 0) return S(0);
  return zi[(zi_mode == 2 ? row * D : 0) + (D - 1 - d)];
}

template <class S>
__device__ __forceinline__ S comb_power(S c, int n) {
  S p = S(1);
  for (int i = 0; i < n; ++i) p *= c;
  return p;
}

// blocks_per_row = ceil(D / 32): a block is one group of 32 phases
template <class S>
__global__ void __launch_bounds__(kCombThreads)
comb_fwd_kernel(const S* __restrict__ x, const S* __restrict__ a, int a_stride, const S* __restrict__ zi,
                int zi_mode, S* __restrict__ y, int64_t N, int64_t D, int blocks_per_row) {
  __shared__ S ends[2][kCombWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x / blocks_per_row;
  const int64_t d = (int64_t)(blockIdx.x % blocks_per_row) * 32 + lane;
  const bool live = d < D && d < N;
  const S coef = -a[row * a_stride];
  const S coef_run = comb_power(coef, kCombSteps);
  const S* xr = x + row * N + d;
  S* yr = y + row * N + d;
  const int64_t steps = live ? (N - d + D - 1) / D : 0;
  const int64_t most = (N + D - 1) / D;                       // steps of the longest phase: uniform loop bound
  S carry = live ? comb_initial(zi, zi_mode, row, D, d) : S(0);   // state entering the super-step
  int buf = 0;
  for (int64_t k0 = 0; k0 < most; k0 += kCombWarps * kCombSteps, buf ^= 1) {
    const int64_t k = k0 + warp * kCombSteps;
    S v[kCombSteps];
#pragma unroll
    for (int u = 0; u < kCombSteps; ++u) v[u] = (k + u < steps) ? xr[(k + u) * D] : S(0);
    S h = S(0);
#pragma unroll
    for (int u = 0; u < kCombSteps; ++u) { h = coef * h + v[u]; v[u] = h; }
    ends[buf][warp][lane] = h;
    __syncthreads();
    S h_in = carry;
#pragma unroll
    for (int j = 0; j < kCombWarps; ++j) {
      const S e = ends[buf][j][lane];
      if (j < warp) h_in = coef_run * h_in + e;
      carry = coef_run * carry + e;
    }
    S p = coef;
#pragma unroll
    for (int u = 0; u < kCombSteps; ++u) {
      if (k + u < steps) yr[(k + u) * D] = v[u] + p * h_in;
      p *= coef;
    }
  }
}

template <class S>
__global__ void __launch_bounds__(kCombThreads)
comb_bwd_kernel(const S* __restrict__ gy, const S* __restrict__ y, const S* __restrict__ a, int a_stride,
                const S* __restrict__ zi, int zi_mode, S* __restrict__ grad_x, S* __restrict__ partial,
                S* __restrict__ grad_state, int64_t N, int64_t D, int blocks_per_row) {
  __shared__ S ends[2][kCombWarps][32];
  __shared__ S warp_sums[kCombWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x / blocks_per_row;
  const int64_t d = (int64_t)(blockIdx.x % blocks_per_row) * 32 + lane;
  const bool live = d < D && d < N;
  const S coef = -a[row * a_stride];
  const S coef_run = comb_power(coef, kCombSteps);
  const S* gr = gy + row * N + d;
  const S* yr = y + row * N + d;
  S* xr = grad_x + row * N + d;
  const int64_t steps = live ? (N - d + D - 1) / D : 0;
  const int64_t most = (N + D - 1) / D;
  const int64_t span = kCombWarps * kCombSteps;
  const int64_t rounds = (most + span - 1) / span;
  // time runs backwards: super-step r covers steps [r span, (r+1) span); warp w takes the w-th run
  // from the TOP of it, its own steps descending.  g[k] = gy[k] + coef * g[k+1].
  S carry = S(0);                                            // g of the step just above the super-step
  S acc = S(0);
  int buf = 0;
  for (int64_t r = rounds - 1; r >= 0; --r, buf ^= 1) {
    const int64_t top = r * span + span - 1 - warp * kCombSteps;    // highest step of this warp's run
    S v[kCombSteps], p[kCombSteps];
#pragma unroll
    for (int u = 0; u < kCombSteps; ++u) {
      const int64_t k = top - u;
      const bool in = k < steps;                                   // k >= 0 always
      v[u] = in ? gr[k * D] : S(0);
      p[u] = S(0);
      if (partial && in) p[u] = k > 0 ? yr[(k - 1) * D] : comb_initial(zi, zi_mode, row, D, d);
    }
    S h = S(0);
#pragma unroll
    for (int u = 0; u < kCombSteps; ++u) { h = coef * h + v[u]; v[u] = h; }
    ends[buf][warp][lane] = h;
    __syncthreads();
    S h_in = carry;
#pragma unroll
    for (int j = 0; j < kCombWarps; ++j) {
      const S e = ends[buf][j][lane];
      if (j < warp) h_in = coef_run * h_in + e;
      carry = coef_run * carry + e;
    }
    S q = coef;
#pragma unroll
    for (int u = 0; u < kCombSteps; ++u) {
      const int64_t k = top - u;
      const S g = v[u] + q * h_in;
      q *= coef;
      if (k < steps) {
        xr[k * D] = g;
        acc += g * p[u];
      }
    }
  }
  if (grad_state && d < D && warp == 0) grad_state[row * D + (D - 1 - d)] = live ? coef * carry : S(0);
  if (partial) {                                       // grad_a = - sum g[t] y[t - D]: block sum
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, s);
    __syncthreads();
    if (lane == 0) warp_sums[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      S t = S(0);
      for (int w = 0; w < kCombWarps; ++w) t += warp_sums[w];
      partial[blockIdx.x] = -t;
    }
  }
}

}  // namespace ptb
