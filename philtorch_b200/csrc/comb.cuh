// Feedback comb filter  y[t] = x[t] - a * y[t - D]  (philtorch/lti/filtering.py:15-71) without
// folding the signal: the D phases t = k D + d of a row are independent first-order recurrences,
// so one THREAD owns one phase (row b, phase d) and walks it in time.  Neighbouring threads own
// neighbouring phases, so every step of a warp reads and writes 32 consecutive samples: the
// accesses are coalesced on the signal's own layout and each sample moves once (8 B forward,
// 12 B + 4 B backward in fp32).  The loads do not depend on the recurrence, so U steps are
// fetched ahead of the serial multiply-adds to keep enough bytes in flight.
// The parallelism is B * D threads: the host uses this kernel when that is a few thousand or
// more, and the folded first-order scan otherwise.
//
// Adjoint:  g[t] = gy[t] - a * g[t + D]  (g = 0 beyond the end),  grad_x = g,
//           grad_a = - sum_t g[t] * y[t - D]   (y[t - D] = the initial state for t < D),
//           gradient of the initial state of phase d:  - a * g[d].
// Per-block partial sums of grad_a go to partial[row][block]; the host adds them up.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ptb {

constexpr int kCombThreads = 128;
constexpr int kCombAhead = 32;      // forward: loads in flight per thread
constexpr int kCombAheadBwd = 16;   // adjoint: per array (gy and y)

// zi_mode: 0 none, 1 (D,) shared by the rows, 2 (B, D).  zi[..., k] is the output k + 1 samples
// before the start, so phase d starts from zi[..., D - 1 - d].
template <class S>
__device__ __forceinline__ S comb_initial(const S* zi, int zi_mode, int64_t row, int64_t D, int64_t d) {
  if (zi_mode == 0) return S(0);
  return zi[(zi_mode == 2 ? row * D : 0) + (D - 1 - d)];
}

template <class S>
__global__ void __launch_bounds__(kCombThreads)
comb_fwd_kernel(const S* __restrict__ x, const S* __restrict__ a, int a_stride, const S* __restrict__ zi,
                int zi_mode, S* __restrict__ y, int64_t N, int64_t D, int blocks_per_row) {
  const int64_t row = blockIdx.x / blocks_per_row;
  const int64_t d = (int64_t)(blockIdx.x % blocks_per_row) * kCombThreads + threadIdx.x;
  if (d >= D || d >= N) return;
  const S coef = -a[row * a_stride];
  const S* xr = x + row * N + d;
  S* yr = y + row * N + d;
  const int64_t steps = (N - d + D - 1) / D;
  S h = comb_initial(zi, zi_mode, row, D, d);
  int64_t k = 0;
  for (; k + kCombAhead <= steps; k += kCombAhead) {
    S v[kCombAhead];
#pragma unroll
    for (int u = 0; u < kCombAhead; ++u) v[u] = xr[(k + u) * D];
#pragma unroll
    for (int u = 0; u < kCombAhead; ++u) { h = coef * h + v[u]; yr[(k + u) * D] = h; }
  }
  for (; k < steps; ++k) { h = coef * h + xr[k * D]; yr[k * D] = h; }
}

template <class S>
__global__ void __launch_bounds__(kCombThreads)
comb_bwd_kernel(const S* __restrict__ gy, const S* __restrict__ y, const S* __restrict__ a, int a_stride,
                const S* __restrict__ zi, int zi_mode, S* __restrict__ grad_x, S* __restrict__ partial,
                S* __restrict__ grad_state, int64_t N, int64_t D, int blocks_per_row) {
  const int64_t row = blockIdx.x / blocks_per_row;
  const int64_t d = (int64_t)(blockIdx.x % blocks_per_row) * kCombThreads + threadIdx.x;
  S acc = S(0);
  if (d < D && d < N) {
    const S coef = -a[row * a_stride];
    const S* gr = gy + row * N + d;
    const S* yr = y + row * N + d;
    S* xr = grad_x + row * N + d;
    const int64_t steps = (N - d + D - 1) / D;
    S c = S(0);                        // coef * g[t + D]
    int64_t k = steps - 1;
    for (; k - kCombAheadBwd >= 0; k -= kCombAheadBwd) {      // steps k .. k - kCombAheadBwd + 1, all with k - u >= 1
      S v[kCombAheadBwd], p[kCombAheadBwd];
#pragma unroll
      for (int u = 0; u < kCombAheadBwd; ++u) { v[u] = gr[(k - u) * D]; p[u] = partial ? yr[(k - u - 1) * D] : S(0); }
#pragma unroll
      for (int u = 0; u < kCombAheadBwd; ++u) {
        const S g = v[u] + c;
        xr[(k - u) * D] = g;
        acc += g * p[u];
        c = coef * g;
      }
    }
    for (; k >= 0; --k) {
      const S g = gr[k * D] + c;
      xr[k * D] = g;
      if (partial) acc += g * (k > 0 ? yr[(k - 1) * D] : comb_initial(zi, zi_mode, row, D, d));
      c = coef * g;
    }
    if (grad_state) grad_state[row * D + (D - 1 - d)] = c;
  } else if (d < D && grad_state) {
    grad_state[row * D + (D - 1 - d)] = S(0);          // a phase beyond a signal shorter than the delay
  }
  if (partial) {                                       // grad_a = - sum g[t] y[t - D]: block sum
    __shared__ S warp_sums[kCombThreads / 32];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, s);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      S t = S(0);
      for (int w = 0; w < kCombThreads / 32; ++w) t += warp_sums[w];
      partial[blockIdx.x] = -t;
    }
  }
}

}  // namespace ptb
