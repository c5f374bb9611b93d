// A bank of M complex first-order modes driven by one real signal and mixed into one real output,
// fused: the whole of a real-output state-space model evaluated in its eigenbasis
// (philtorch/lti/ssm.py:590-850, diag_state_space with a scalar input and a scalar output)
//     w_m[t] = lam_m w_m[t-1] + gain_m x[t],   w_m[-1] = w0_m
//     y[t]   = Re( sum_m coef_m w_m[t-1] ) + d x[t]
// reads x and writes y; the (rows, M, N) complex mode signals that the reference materialises (and
// the earlier five passes over them here) never exist.
//
// Time-invariant and diagonal, so the linear part of any span of n samples is lam^n: maps between
// tiles carry only the M complex offsets.  Three launches per direction, no waiting between CTAs:
//   A  one CTA per (row, tile): the tile's aggregate  S_m = sum_t lam^(end-t) gain x[t]   (reads x)
//   B  one thread per (row, mode): sequential fold over the row's tiles in double, turning the
//      aggregates into the state entering every tile (in place)
//   C  one CTA per (row, tile): intra-tile scan from that state, outputs                  (reads x, writes y)
// i.e. 12 bytes per sample for an algorithmic 8.  Samples beyond the end of a row count as zero
// input, so every tile spans the same power lam^TILE.
//
// Adjoint (gy real; r_m[t] = gradient w.r.t. w_m[t-1]):
//     r_m[t] = conj(lam_m) r_m[t+1] + conj(coef_m) gy[t],   r_m[N] = gradient of the final state
//     grad_x[t]   = Re( sum_m conj(gain_m) r_m[t+1] ) + d gy[t]
//     grad_gain_m = sum_t r_m[t+1] x[t]            grad_lam_m = sum_t r_m[t+1] conj(w_m[t-1])
//     grad_coef_m = sum_t gy[t] conj(w_m[t-1])     grad_d = sum_t gy[t] x[t]     grad_w0_m = r_m[0]
// the same three steps in reversed time on gy; step C also recomputes the tile's forward states
// from the checkpoints that the forward fold left (the states entering every tile), so the mode
// signals are not stored for the backward pass either.  Sums are emitted per tile.
#pragma once
#include "complex.cuh"

#include <cstdint>

namespace ptb {

constexpr int kBankNT = 128;   // threads per CTA; few threads with many samples each keep the scans cheap per sample
constexpr int kBankNW = kBankNT / 32;

template <class R, int MMAX>
struct BankCfg {
  static constexpr int SPT = 64 / MMAX;          // 16 samples per thread for up to 4 modes, 8 for up to 8
  static constexpr int TILE = kBankNT * SPT;
  static constexpr int NPOW = 6;                 // lam^(SPT 2^d), d = 0..5 (d = 5: one warp)
};

template <class R>
struct BankParams {
  int64_t rows, M, N, ntiles;
  const R* x;              // (rows, N)   forward: input; adjoint: also needed for the sums
  const R* gy;             // (rows, N)   adjoint only
  const Cx<R>* lam;        // (rows, M)
  const Cx<R>* gain;       // (rows, M)
  const Cx<R>* coef;       // (rows, M)
  const R* d;              // (rows,) or nullptr
  const Cx<R>* w0;         // (rows, M)   forward: initial modes (state entering the row); adjoint: nullptr
  const Cx<R>* g_wf;       // (rows, M)   adjoint: gradient of the final modes r[N], or nullptr.  It enters at
                           //             sample N, not at the zero-padded end of the last tile: the thread that
                           //             owns sample N-1 adds it before stepping over that sample
  Cx<R>* chk;              // (rows, ntiles, M) aggregates -> states entering every tile (this direction)
  const Cx<R>* fwd_chk;    // adjoint: the forward direction's checkpoints
  R* y;                    // (rows, N)   forward: y; adjoint: grad_x
  Cx<R>* wf;               // (rows, M)   forward: final modes; adjoint: grad_w0
  R* partial;              // adjoint: (rows, ntiles, 6 M + 1) sums; a run's sums are stored with its last tile, zeros elsewhere
  int64_t run;             // consecutive tiles of a row handled by one CTA (the per-row set-up is paid once)
  int need;                // adjoint: sums wanted: 1 grad_gain, 2 grad_lam, 4 grad_coef (skipped ones are zero)
};

// lam^(SPT 2^d) for d < NPOW and lam^TILE, per mode, formed in double (squaring doubles the
// relative error) and rounded once.  pw: shared [NPOW + 1][MMAX].
template <class R, int MMAX, bool ADJ>
__device__ __forceinline__ void bank_powers(const BankParams<R>& p, int64_t row, Cx<R>* pw) {
  using C = BankCfg<R, MMAX>;
  const int m = threadIdx.x;
  if (m < MMAX) {
    Cx<double> b(0.0, 0.0);
    if (m < p.M) {
      const Cx<R> l = p.lam[row * p.M + m];
      b = Cx<double>((double)l.re, ADJ ? -(double)l.im : (double)l.im);
    }
    for (int s = 1; s < C::SPT; s <<= 1) b = b * b;          // lam^SPT (SPT is a power of two)
#pragma unroll
    for (int d = 0; d < C::NPOW; ++d) {
      pw[d * MMAX + m] = Cx<R>((R)b.re, (R)b.im);
      b = b * b;
    }
    // b = lam^(SPT 64); the tile is SPT * kBankNT samples
    for (int n = 64; n < kBankNT; n <<= 1) b = b * b;
    pw[C::NPOW * MMAX + m] = Cx<R>((R)b.re, (R)b.im);
  }
}

// The thread's SPT consecutive samples of a row-major real array, zero beyond the row.  Rows whose
// start is 16-byte aligned (vec = true) use 128-bit accesses for the units that lie inside the row.
template <class R, int SPT>
__device__ __forceinline__ void bank_load(const R* __restrict__ src, int64_t row_len, int64_t t0, int pos, bool vec,
                                          R* v) {
  constexpr int VW = 16 / (int)sizeof(R);
  const int64_t tb = t0 + (int64_t)pos * SPT;
  if (vec && tb + SPT <= row_len) {
#pragma unroll
    for (int u = 0; u < SPT / VW; ++u) {
      if constexpr (sizeof(R) == 4) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(src + tb) + u);
        v[4 * u] = q.x; v[4 * u + 1] = q.y; v[4 * u + 2] = q.z; v[4 * u + 3] = q.w;
      } else {
        const double2 q = __ldg(reinterpret_cast<const double2*>(src + tb) + u);
        v[2 * u] = q.x; v[2 * u + 1] = q.y;
      }
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < SPT; ++j) v[j] = tb + j < row_len ? __ldg(src + tb + j) : R(0);
}
template <class R, int SPT>
__device__ __forceinline__ void bank_store(R* __restrict__ dst, int64_t row_len, int64_t tb, bool vec, const R* v) {
  constexpr int VW = 16 / (int)sizeof(R);
  if (vec && tb + SPT <= row_len) {
#pragma unroll
    for (int u = 0; u < SPT / VW; ++u) {
      if constexpr (sizeof(R) == 4)
        reinterpret_cast<float4*>(dst + tb)[u] = make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
      else
        reinterpret_cast<double2*>(dst + tb)[u] = make_double2(v[2 * u], v[2 * u + 1]);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < SPT; ++j)
    if (tb + j < row_len) dst[tb + j] = v[j];
}
// rows start on 16-byte boundaries: aligned base and a row length that keeps every row aligned
template <class R>
__device__ __forceinline__ bool bank_vec_ok(const void* a, const void* b, const void* c, int64_t N) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c);
  return (bits & 15u) == 0 && (N * (int64_t)sizeof(R)) % 16 == 0;
}

// real x complex products written out (a complex product with a zero imaginary part costs twice as much)
template <class R>
__device__ __forceinline__ void cfma_r(Cx<R>& acc, const Cx<R>& a, R x) { acc.re += a.re * x; acc.im += a.im * x; }
// float32: both components in one packed multiply-add (fma.rn.f32x2; same rounding as two scalar ones)
__device__ __forceinline__ void cfma_r(Cx<float>& acc, const Cx<float>& a, float x) {
  const float2 r = __ffma2_rn(make_float2(a.re, a.im), make_float2(x, x), make_float2(acc.re, acc.im));
  acc.re = r.x;
  acc.im = r.y;
}

// Per-CTA tables for a thread's SPT samples (l = lam forward, conj(lam) adjoint; g = gain forward,
// conj(coef) adjoint):  lp[m][k] = l^k, k = 0..SPT;  wt[m][j] = weight of local sample j in the
// thread's aggregate, so that the aggregate is a plain real-times-complex dot product:
//   forward  s = sum_j l^(SPT-1-j) g x_j        adjoint (descending time)  s = sum_j l^j g gy_j
template <class R, int MMAX, int SPT, bool ADJ>
__device__ __forceinline__ void bank_tables(const BankParams<R>& p, int64_t row, Cx<R>* lp, Cx<R>* wt) {
  const int tid = threadIdx.x;
  if (tid < MMAX * (SPT + 1)) {
    const int m = tid / (SPT + 1), k = tid % (SPT + 1);
    Cx<R> l(R(0));
    if (m < p.M) { l = p.lam[row * p.M + m]; if (ADJ) l = cj(l); }
    Cx<R> r(R(1));
    for (int i = 0; i < k; ++i) r = r * l;
    lp[m * (SPT + 1) + k] = r;
  }
  __syncthreads();
  if (tid < MMAX * SPT) {
    const int m = tid / SPT, j = tid % SPT;
    Cx<R> g(R(0));
    if (m < p.M) g = ADJ ? cj(p.coef[row * p.M + m]) : p.gain[row * p.M + m];
    wt[m * SPT + j] = lp[m * (SPT + 1) + (ADJ ? j : SPT - 1 - j)] * g;
  }
}

// Inclusive scan over the threads of the CTA of per-thread offsets s (M complex each) under the
// common per-thread power: on return `exc` holds the offset accumulated by the threads before this
// one (from a zero state), and sm_w the warps' totals.  Thread order = threadIdx order.
template <class R, int MMAX>
__device__ __forceinline__ void bank_scan(const Cx<R>* s, const Cx<R>* pw, Cx<R>* sm_w, Cx<R>* exc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    Cx<R> a = s[m];
#pragma unroll
    for (int d = 0; d < 5; ++d) {
      const Cx<R> o = shfl_up_s(a, 1 << d);
      if (lane >= (1 << d)) a = a + pw[d * MMAX + m] * o;
    }
    Cx<R> e = shfl_up_s(a, 1);
    if (lane == 0) e = Cx<R>(R(0));
    exc[m] = e;
    if (lane == 31) sm_w[warp * MMAX + m] = a;
  }
}

// lam^(SPT * lane) from the binary digits of the lane
template <class R, int MMAX>
__device__ __forceinline__ Cx<R> bank_lane_power(const Cx<R>* pw, int m, int lane) {
  Cx<R> r(R(1));
#pragma unroll
  for (int d = 0; d < 5; ++d)
    if (lane & (1 << d)) r = r * pw[d * MMAX + m];
  return r;
}

// lanep[m][lane] = lam^(SPT * lane), once per CTA: what a thread multiplies the state entering its warp by
template <class R, int MMAX>
__device__ __forceinline__ void bank_lane_table(const Cx<R>* pw, Cx<R>* lanep) {
  for (int i = threadIdx.x; i < MMAX * 32; i += kBankNT) lanep[i] = bank_lane_power<R, MMAX>(pw, i >> 5, i & 31);
}

// ---- step A: tile aggregates (forward: x with gain; adjoint: gy with conj(coef), reversed time) ----
template <class R, int MMAX, bool ADJ>
__global__ void __launch_bounds__(kBankNT) bank_aggregate_kernel(const BankParams<R> p) {
  using C = BankCfg<R, MMAX>;
  constexpr int SPT = C::SPT;
  __shared__ Cx<R> pw[(C::NPOW + 1) * MMAX];
  __shared__ Cx<R> sm_w[kBankNW * MMAX];
  __shared__ Cx<R> lp[MMAX * (SPT + 1)];
  __shared__ Cx<R> wt[MMAX * SPT];
  __shared__ Cx<R> lanep[MMAX * 32];
  const int64_t runs = (p.ntiles + p.run - 1) / p.run;
  const int64_t row = blockIdx.x / runs, tile0 = (blockIdx.x % runs) * p.run;
  // thread order along the scan: forward = ascending time, adjoint = descending time
  const int pos = ADJ ? (kBankNT - 1 - threadIdx.x) : threadIdx.x;
  const R* src = ADJ ? p.gy : p.x;
  const bool vec = bank_vec_ok<R>(src, src, src, p.N);
  bank_powers<R, MMAX, ADJ>(p, row, pw);
  bank_tables<R, MMAX, SPT, ADJ>(p, row, lp, wt);   // (a barrier inside: pw is complete after it)
  bank_lane_table<R, MMAX>(pw, lanep);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t tile = tile0; tile < tile0 + p.run && tile < p.ntiles; ++tile) {
    const int64_t t0 = tile * C::TILE;
    R v[SPT];
    bank_load<R, SPT>(src + row * p.N, p.N, t0, pos, vec, v);
    Cx<R> s[MMAX];
    const int64_t tb = t0 + (int64_t)pos * SPT;
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      Cx<R> a(R(0));
#pragma unroll
      for (int j = 0; j < SPT; ++j) cfma_r(a, wt[m * SPT + j], v[j]);
      if (ADJ && p.g_wf && m < p.M && p.N - 1 >= tb && p.N - 1 < tb + SPT)   // r[N] enters above sample N-1
        a = a + lp[m * (SPT + 1) + (int)(p.N - tb)] * p.g_wf[row * p.M + m];
      s[m] = a;
    }
    // only the totals are wanted: every thread's offset times the power that carries it to the end of
    // its warp, then a plain sum over the lanes (a scan would cost twice the shuffles)
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      Cx<R> a = lanep[m * 32 + 31 - lane] * s[m];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) a = a + shfl_down_s(a, d);
      if (lane == 0) sm_w[warp * MMAX + m] = a;
    }
    __syncthreads();
    if (threadIdx.x < MMAX && threadIdx.x < p.M) {
      const int m = threadIdx.x;
      const Cx<R> p32 = pw[5 * MMAX + m];
      Cx<R> a(R(0));
      for (int w = 0; w < kBankNW; ++w) a = p32 * a + sm_w[w * MMAX + m];
      p.chk[(row * p.ntiles + tile) * p.M + m] = a;
    }
    __syncthreads();   // sm_w is rewritten by the next tile
  }
}

// ---- step B: aggregates -> states entering every tile, in place (double arithmetic) ----------------
// One warp per (row, mode): 32 consecutive tiles per step, scanned with the powers b^(2^d) of
// b = lam^TILE; the carry moves on by b^32.
template <class R, bool ADJ>
__global__ void bank_fold_kernel(const BankParams<R> p, int tile_len) {
  const int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (idx >= p.rows * p.M) return;
  const int64_t row = idx / p.M, m = idx % p.M;
  const Cx<R> l = p.lam[idx];
  Cx<double> b((double)l.re, ADJ ? -(double)l.im : (double)l.im);
  for (int s = 1; s < tile_len; s <<= 1) b = b * b;   // lam^TILE
  Cx<double> pd[5];
  Cx<double> blane(1.0, 0.0);                          // b^lane
#pragma unroll
  for (int d = 0; d < 5; ++d) {
    pd[d] = b;
    if (lane & (1 << d)) blane = blane * b;
    b = b * b;
  }
  const Cx<double> b32 = b;
  Cx<double> st(0.0, 0.0);
  if (!ADJ && p.w0) { const Cx<R> z = p.w0[idx]; st = Cx<double>((double)z.re, (double)z.im); }
  Cx<R>* c = p.chk + row * p.ntiles * p.M + m;
  // the aggregates of the next 32 tiles are fetched while this step's scan runs
  Cx<R> ahead(R(0));
  if (lane < p.ntiles) ahead = c[(ADJ ? p.ntiles - 1 - lane : lane) * p.M];
  for (int64_t k0 = 0; k0 < p.ntiles; k0 += 32) {
    const int64_t k = k0 + lane;
    const int64_t tile = ADJ ? p.ntiles - 1 - k : k;       // the adjoint walks the tiles from the last one
    Cx<double> a((double)ahead.re, (double)ahead.im);
    ahead = Cx<R>(R(0));
    if (k + 32 < p.ntiles) ahead = c[(ADJ ? p.ntiles - 1 - (k + 32) : k + 32) * p.M];
#pragma unroll
    for (int d = 0; d < 5; ++d) {
      const Cx<double> o = shfl_up_s(a, 1 << d);
      if (lane >= (1 << d)) a = a + pd[d] * o;
    }
    Cx<double> e = shfl_up_s(a, 1);
    if (lane == 0) e = Cx<double>(0.0, 0.0);
    const Cx<double> sin = blane * st + e;                 // the state entering tile k
    if (k < p.ntiles) c[tile * p.M] = Cx<R>((R)sin.re, (R)sin.im);
    const int64_t rem = p.ntiles - k0;
    const Cx<double> full = b32 * st + shfl_s(a, 31);      // after 32 tiles
    st = rem < 32 ? shfl_s(sin, (int)rem) : full;          // after the row's last tile when the step is ragged
  }
  // the state after the whole (zero-padded) row; only the adjoint uses it: r[0] = grad_w0
  if (ADJ && p.wf && lane == 0) p.wf[idx] = Cx<R>((R)st.re, (R)st.im);
}

// State entering this thread, given the state entering the tile (z_tile), the scan's exclusive
// offsets and the warps' totals.
template <class R, int MMAX>
__device__ __forceinline__ void bank_thread_state(const Cx<R>* z_tile, const Cx<R>* exc, const Cx<R>* pw,
                                                  const Cx<R>* sm_w, const Cx<R>* lanep, Cx<R>* h) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    const Cx<R> p32 = pw[5 * MMAX + m];
    Cx<R> z = z_tile[m];
    for (int w = 0; w < warp; ++w) z = p32 * z + sm_w[w * MMAX + m];
    h[m] = lanep[m * 32 + lane] * z + exc[m];
  }
}

// ---- step C forward ---------------------------------------------------------------------------------
// Inside a thread the outputs are a short real convolution plus the decaying incoming state:
//   y_j = d x_j + sum_{i<j} K[j-1-i] x_i + Re( sum_m (coef_m lam_m^j) h_m ),   K[n] = Re sum_m coef_m lam_m^n gain_m
// (SPT (SPT-1) / 2 + 2 M SPT real multiply-adds instead of 8 M SPT for stepping the M complex modes).
template <class R, int MMAX>
__global__ void __launch_bounds__(kBankNT, 4) bank_forward_kernel(const BankParams<R> p) {
  using C = BankCfg<R, MMAX>;
  constexpr int SPT = C::SPT;
  __shared__ Cx<R> pw[(C::NPOW + 1) * MMAX];
  __shared__ Cx<R> sm_w[kBankNW * MMAX];
  __shared__ Cx<R> lp[MMAX * (SPT + 1)];
  __shared__ Cx<R> wt[MMAX * SPT];
  __shared__ Cx<R> cl[MMAX * SPT];   // conj(coef_m lam_m^j): Re(coef lam^j h) = cl.re h.re + cl.im h.im, one packed multiply-add
  __shared__ Cx<R> zt[MMAX];         // the modes entering the tile
  __shared__ R kern[SPT];
  __shared__ Cx<R> lanep[MMAX * 32];
  const int64_t runs = (p.ntiles + p.run - 1) / p.run;
  const int64_t row = blockIdx.x / runs, tile0 = (blockIdx.x % runs) * p.run;
  const bool vec = bank_vec_ok<R>(p.x, p.y, p.y, p.N);
  bank_powers<R, MMAX, false>(p, row, pw);
  bank_tables<R, MMAX, SPT, false>(p, row, lp, wt);   // (a barrier inside: pw is complete after it)
  bank_lane_table<R, MMAX>(pw, lanep);
  if (threadIdx.x < MMAX * SPT) {
    const int m = threadIdx.x / SPT, j = threadIdx.x % SPT;
    cl[threadIdx.x] = m < p.M ? cj(p.coef[row * p.M + m] * lp[m * (SPT + 1) + j]) : Cx<R>(R(0));
  }
  __syncthreads();
  if (threadIdx.x < SPT) {   // K[n] = Re sum_m (coef lam^n) gain
    R a = R(0);
    for (int m = 0; m < p.M; ++m) {
      const Cx<R> c = cl[m * SPT + threadIdx.x], g = p.gain[row * p.M + m];
      a += c.re * g.re + c.im * g.im;
    }
    kern[threadIdx.x] = a;
  }
  const R dd = p.d ? __ldg(p.d + row) : R(0);
  for (int64_t tile = tile0; tile < tile0 + p.run && tile < p.ntiles; ++tile) {
    const int64_t t0 = tile * C::TILE;
    R v[SPT];
    bank_load<R, SPT>(p.x + row * p.N, p.N, t0, threadIdx.x, vec, v);
    if (threadIdx.x < MMAX)
      zt[threadIdx.x] = threadIdx.x < p.M ? p.chk[(row * p.ntiles + tile) * p.M + threadIdx.x] : Cx<R>(R(0));
    Cx<R> s[MMAX];
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      Cx<R> a(R(0));
#pragma unroll
      for (int j = 0; j < SPT; ++j) cfma_r(a, wt[m * SPT + j], v[j]);
      s[m] = a;
    }
    Cx<R> exc[MMAX], h[MMAX];
    bank_scan<R, MMAX>(s, pw, sm_w, exc);
    __syncthreads();   // also publishes kern (first tile) and zt
    bank_thread_state<R, MMAX>(zt, exc, pw, sm_w, lanep, h);
    const int64_t tb = t0 + (int64_t)threadIdx.x * SPT;
    R out[SPT];
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      R acc = dd * v[j];
#pragma unroll
      for (int i = 0; i < j; ++i) acc += kern[j - 1 - i] * v[i];
      if constexpr (std::is_same<R, float>::value) {
        float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
        for (int m = 0; m < MMAX; ++m) {
          const Cx<R> c = cl[m * SPT + j];
          acc2 = __ffma2_rn(make_float2(c.re, c.im), make_float2(h[m].re, h[m].im), acc2);
        }
        acc += acc2.x + acc2.y;
      } else {
#pragma unroll
        for (int m = 0; m < MMAX; ++m) {
          const Cx<R> c = cl[m * SPT + j];
          acc += c.re * h[m].re + c.im * h[m].im;
        }
      }
      out[j] = acc;
    }
    bank_store<R, SPT>(p.y + row * p.N, p.N, tb, vec, out);
    if (p.wf && p.N - 1 >= tb && p.N - 1 < tb + SPT) {   // the modes after the row's last sample
      const int last = (int)(p.N - 1 - tb);
      for (int m = 0; m < p.M; ++m) {
        const Cx<R> l = p.lam[row * p.M + m], g = p.gain[row * p.M + m];
        Cx<R> w = h[0];
#pragma unroll
        for (int q = 1; q < MMAX; ++q)
          if (q == m) w = h[q];
        for (int j = 0; j <= last; ++j) { w = l * w; cfma_r(w, g, v[j]); }
        p.wf[row * p.M + m] = w;
      }
    }
    __syncthreads();   // sm_w and zt are rewritten by the next tile
  }
}

// ---- step C adjoint ---------------------------------------------------------------------------------
// Neither the forward nor the adjoint modes are stepped sample by sample.  Inside a thread (S = SPT
// samples x_j, gy_j; h = w[tb-1], the forward modes entering the thread; rin = r[tb+S], the adjoint
// modes entering it from the right; l = lam, a = conj(lam)):
//   W_j = w[tb+j-1] = l^j h + gain sum_{k<j} l^(j-1-k) x_k
//   R_j = r[tb+j+1] = a^(S-1-j) rin + conj(coef) sum_{i>j} a^(i-j-1) gy_i
// With the REAL cross-correlation of the thread's samples, C[n] = sum_j x_j gy_(j+n) (the same for every
// mode), and per mode four real-times-complex dot products and two sums over C,
//   SX = sum_j a^(S-1-j) x_j     U = sum_k (S-1-k) a^(S-2-k) x_k     SG = sum_j a^j gy_j     V = sum_i i a^(i-1) gy_i
//   Q  = sum_{n>=1} a^(n-1) C[n]                                    Q2 = sum_{n>=2} (n-1) a^(n-2) C[n]
// the thread's outputs and sums are
//   grad_x_j  = d gy_j + sum_{i>j} K[i-j-1] gy_i + Re sum_m conj(gain l^(S-1-j)) rin      (K as in the forward kernel)
//   grad_gain = sum_j R_j x_j        = rin SX + conj(coef) Q
//   grad_coef = sum_j gy_j conj(W_j) = conj(h) SG + conj(gain) Q
//   grad_lam  = sum_j R_j conj(W_j)  = S a^(S-1) rin conj(h) + rin conj(gain) U + conj(coef) conj(h) V + conj(coef gain) Q2
//   grad_d    = C[0]
// and the aggregates the two scans over the threads start from are gain conj(SX) and conj(coef) SG.
// (Stepping both sets of modes and keeping the forward ones in 64 KB of shared memory took about four
// times the instructions.)  The gradient of the final modes enters at sample N-1: the one thread that
// owns it adds the terms of dR_j = a^(jN-j) g_wf, j <= jN = N-1-tb, from the same tables.
template <class R, int MMAX>
__global__ void __launch_bounds__(kBankNT, sizeof(R) == 4 ? 3 : 1) bank_backward_kernel(const BankParams<R> p) {
  using C = BankCfg<R, MMAX>;
  constexpr int SPT = C::SPT;
  constexpr int LS = SPT + 1;   // stride of the power tables
  constexpr int NSUM = 6 * MMAX + 1;
  __shared__ Cx<R> pw[(C::NPOW + 1) * MMAX];
  __shared__ Cx<R> pwa[(C::NPOW + 1) * MMAX];
  __shared__ Cx<R> sm_w[kBankNW * MMAX];
  __shared__ Cx<R> sm_c[6 * MMAX];   // lam, gain, coef, forward / adjoint state entering the tile, r[N]
  __shared__ R sm_red[kBankNW * NSUM];
  __shared__ Cx<R> lp[MMAX * LS], lpa[MMAX * LS];   // l^k, a^k, k = 0..SPT
  __shared__ Cx<R> wt[MMAX * SPT], wta[MMAX * SPT];
  __shared__ Cx<R> dta[MMAX * LS];                  // k a^(k-1)
  __shared__ Cx<R> gl[MMAX * SPT];                  // gain l^k
  __shared__ R kern[SPT];                           // K[n] = Re sum_m coef l^n gain
  __shared__ Cx<R> lanep[MMAX * 32], lanepa[MMAX * 32];   // l^(SPT lane), a^(SPT lane)
  const int64_t runs = (p.ntiles + p.run - 1) / p.run;
  const int64_t row = blockIdx.x / runs, tile0 = (blockIdx.x % runs) * p.run;
  bank_powers<R, MMAX, false>(p, row, pw);
  bank_powers<R, MMAX, true>(p, row, pwa);
  bank_tables<R, MMAX, SPT, false>(p, row, lp, wt);    // (barriers inside: pw and pwa are complete after them)
  bank_tables<R, MMAX, SPT, true>(p, row, lpa, wta);
  bank_lane_table<R, MMAX>(pw, lanep);
  bank_lane_table<R, MMAX>(pwa, lanepa);
  if (threadIdx.x < MMAX) {
    const int m = threadIdx.x;
    const bool on = m < p.M;
    sm_c[m] = on ? p.lam[row * p.M + m] : Cx<R>(R(0));
    sm_c[MMAX + m] = on ? p.gain[row * p.M + m] : Cx<R>(R(0));
    sm_c[2 * MMAX + m] = on ? p.coef[row * p.M + m] : Cx<R>(R(0));
    sm_c[5 * MMAX + m] = (on && p.g_wf) ? p.g_wf[row * p.M + m] : Cx<R>(R(0));
  }
  if (threadIdx.x < MMAX * LS) {
    const int k = threadIdx.x % LS;
    const Cx<R> prev = k > 0 ? lpa[threadIdx.x - 1] : Cx<R>(R(0));
    dta[threadIdx.x] = Cx<R>((R)k * prev.re, (R)k * prev.im);
  }
  if (threadIdx.x < MMAX * SPT) {
    const int m = threadIdx.x / SPT, k = threadIdx.x % SPT;
    gl[threadIdx.x] = m < p.M ? p.gain[row * p.M + m] * lp[m * LS + k] : Cx<R>(R(0));
  }
  __syncthreads();
  if (threadIdx.x < SPT) {
    R a = R(0);
    for (int m = 0; m < p.M; ++m) {
      const Cx<R> c = p.coef[row * p.M + m], g = gl[m * SPT + threadIdx.x];
      a += c.re * g.re - c.im * g.im;
    }
    kern[threadIdx.x] = a;
  }
  const bool vec = bank_vec_ok<R>(p.x, p.gy, p.y, p.N);
  const R dd = p.d ? __ldg(p.d + row) : R(0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  Cx<R> g_gain[MMAX], g_lam[MMAX], g_coef[MMAX];
#pragma unroll
  for (int m = 0; m < MMAX; ++m) { g_gain[m] = Cx<R>(R(0)); g_lam[m] = Cx<R>(R(0)); g_coef[m] = Cx<R>(R(0)); }
  R g_d = R(0);
  for (int64_t tile = tile0; tile < tile0 + p.run && tile < p.ntiles; ++tile) {
  if (threadIdx.x < MMAX) {
    const int m = threadIdx.x;
    const bool on = m < p.M;
    sm_c[3 * MMAX + m] = on ? p.fwd_chk[(row * p.ntiles + tile) * p.M + m] : Cx<R>(R(0));
    sm_c[4 * MMAX + m] = on ? p.chk[(row * p.ntiles + tile) * p.M + m] : Cx<R>(R(0));
  }
  __syncthreads();
  const int64_t t0 = tile * C::TILE;
  const int64_t tb = t0 + (int64_t)threadIdx.x * SPT;
  R xv[SPT], gv[SPT];
  bank_load<R, SPT>(p.x + row * p.N, p.N, t0, threadIdx.x, vec, xv);
  bank_load<R, SPT>(p.gy + row * p.N, p.N, t0, threadIdx.x, vec, gv);
  const bool own = p.N - 1 >= tb && p.N - 1 < tb + SPT;   // this thread holds the row's last sample
  const int jn = own ? (int)(p.N - 1 - tb) : 0;

  // (1) forward modes entering this thread, from the tile's checkpoint
  Cx<R> sx[MMAX], sg[MMAX], s[MMAX], exc[MMAX], h[MMAX];
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    Cx<R> a(R(0)), b(R(0));
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      cfma_r(a, lpa[m * LS + SPT - 1 - j], xv[j]);
      cfma_r(b, lpa[m * LS + j], gv[j]);
    }
    sx[m] = a;
    sg[m] = b;
    s[m] = sm_c[MMAX + m] * cj(a);
  }
  bank_scan<R, MMAX>(s, pw, sm_w, exc);
  __syncthreads();
  bank_thread_state<R, MMAX>(sm_c + 3 * MMAX, exc, pw, sm_w, lanep, h);
  __syncthreads();   // sm_w is reused by the adjoint scan

  // (2) adjoint modes: the scan runs over the threads in DESCENDING time, i.e. the thread that
  // holds the tile's last samples comes first: exchange roles through a mirrored thread index
  // (thread i plays scan position NT-1-i by shuffling with mirrored lanes and warps).
  Cx<R> rin[MMAX];
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    Cx<R> a = cj(sm_c[2 * MMAX + m]) * sg[m];
    if (own) a = a + lpa[m * LS + jn + 1] * sm_c[5 * MMAX + m];   // r[N] enters above sample N-1
    // mirrored inclusive scan: lane L takes contributions of lanes L+1.. (later in time) first
#pragma unroll
    for (int d = 0; d < 5; ++d) {
      const Cx<R> o = shfl_down_s(a, 1 << d);
      if (lane + (1 << d) < 32) a = a + pwa[d * MMAX + m] * o;
    }
    Cx<R> e = shfl_down_s(a, 1);
    if (lane == 31) e = Cx<R>(R(0));
    rin[m] = e;                                   // offset accumulated by the later threads of the warp
    if (lane == 0) sm_w[warp * MMAX + m] = a;     // the warp's total
  }
  __syncthreads();
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    const Cx<R> p32 = pwa[5 * MMAX + m];
    Cx<R> z = sm_c[4 * MMAX + m];                 // adjoint state entering the tile from the right
    for (int w = kBankNW - 1; w > warp; --w) z = p32 * z + sm_w[w * MMAX + m];
    rin[m] = lanepa[m * 32 + 31 - lane] * z + rin[m];   // r[t+1] of the thread's last sample
  }

  // (3) grad_x: a short real convolution of gy plus the decaying incoming adjoint modes
  R gxv[SPT];
#pragma unroll
  for (int j = 0; j < SPT; ++j) {
    R acc = dd * gv[j];
#pragma unroll
    for (int i = j + 1; i < SPT; ++i) acc += kern[i - j - 1] * gv[i];
    if constexpr (std::is_same<R, float>::value) {
      float2 acc2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int m = 0; m < MMAX; ++m) {
        const Cx<R> g = gl[m * SPT + SPT - 1 - j];
        acc2 = __ffma2_rn(make_float2(g.re, g.im), make_float2(rin[m].re, rin[m].im), acc2);
      }
      acc += acc2.x + acc2.y;
    } else {
#pragma unroll
      for (int m = 0; m < MMAX; ++m) {
        const Cx<R> g = gl[m * SPT + SPT - 1 - j];
        acc += g.re * rin[m].re + g.im * rin[m].im;
      }
    }
    gxv[j] = acc;
  }

  // (4) the thread's sums, accumulated over the tiles of the run
  if (p.need) {
    R cr[SPT];   // C[n]
#pragma unroll
    for (int n = 0; n < SPT; ++n) {
      R a = R(0);
#pragma unroll
      for (int j = 0; j + n < SPT; ++j) a += xv[j] * gv[j + n];
      cr[n] = a;
    }
    g_d += cr[0];
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      Cx<R> u(R(0)), v(R(0)), q(R(0)), q2(R(0));
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        cfma_r(u, dta[m * LS + SPT - 1 - j], xv[j]);
        cfma_r(v, dta[m * LS + j], gv[j]);
      }
#pragma unroll
      for (int n = 1; n < SPT; ++n) {
        cfma_r(q, lpa[m * LS + n - 1], cr[n]);
        if (n >= 2) cfma_r(q2, dta[m * LS + n - 1], cr[n]);
      }
      const Cx<R> gb = cj(sm_c[MMAX + m]), cb = cj(sm_c[2 * MMAX + m]), hb = cj(h[m]), r = rin[m];
      const Cx<R> ap = lpa[m * LS + SPT - 1];
      g_gain[m] = g_gain[m] + (r * sx[m] + cb * q);
      g_coef[m] = g_coef[m] + (hb * sg[m] + gb * q);
      const Cx<R> rh = r * hb;
      g_lam[m] = g_lam[m] + (Cx<R>((R)SPT * ap.re, (R)SPT * ap.im) * rh + (r * gb) * u + (cb * hb) * v + (cb * gb) * q2);
    }
  }
  if (own && p.g_wf) {   // one thread per row: the terms of r[N], which enters at sample jn
#pragma unroll
    for (int m = 0; m < MMAX; ++m) {
      const Cx<R> G = sm_c[5 * MMAX + m];
      Cx<R> ax(R(0)), ad(R(0));   // sum_{j<=jn} a^(jn-j) x_j,  sum_{k<jn} (jn-k) a^(jn-k-1) x_k
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        if (j <= jn) {
          const Cx<R> g = gl[m * SPT + jn - j];
          gxv[j] += g.re * G.re + g.im * G.im;
          cfma_r(ax, lpa[m * LS + jn - j], xv[j]);
          cfma_r(ad, dta[m * LS + jn - j], xv[j]);
        }
      }
      const Cx<R> an = lpa[m * LS + jn];
      g_gain[m] = g_gain[m] + G * ax;
      g_lam[m] = g_lam[m] + G * (Cx<R>((R)(jn + 1) * an.re, (R)(jn + 1) * an.im) * cj(h[m]) + cj(sm_c[MMAX + m]) * ad);
    }
  }
  bank_store<R, SPT>(p.y + row * p.N, p.N, tb, vec, gxv);

  // (5) sums of the run, stored with its last tile (the slots of its other tiles hold zeros): warp
  // shuffles, then the warps' results through shared memory
  const bool last_of_run = tile + 1 == tile0 + p.run || tile + 1 == p.ntiles;
  if (!last_of_run) {
    if (threadIdx.x < 6 * p.M + 1) p.partial[(row * p.ntiles + tile) * (6 * p.M + 1) + threadIdx.x] = R(0);
    __syncthreads();   // the shared scratch is rewritten by the next tile
    continue;
  }
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    if (!(p.need & 1)) g_gain[m] = Cx<R>(R(0));
    if (!(p.need & 2)) g_lam[m] = Cx<R>(R(0));
    if (!(p.need & 4)) g_coef[m] = Cx<R>(R(0));
  }
  R sums[NSUM];
#pragma unroll
  for (int m = 0; m < MMAX; ++m) {
    sums[6 * m + 0] = g_gain[m].re; sums[6 * m + 1] = g_gain[m].im;
    sums[6 * m + 2] = g_lam[m].re;  sums[6 * m + 3] = g_lam[m].im;
    sums[6 * m + 4] = g_coef[m].re; sums[6 * m + 5] = g_coef[m].im;
  }
  sums[NSUM - 1] = g_d;
#pragma unroll
  for (int i = 0; i < NSUM; ++i) {
    R a = sums[i];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) a += __shfl_down_sync(0xffffffffu, a, d);
    if (lane == 0) sm_red[warp * NSUM + i] = a;
  }
  __syncthreads();
  if (threadIdx.x < NSUM) {
    R a = R(0);
    for (int w = 0; w < kBankNW; ++w) a += sm_red[w * NSUM + threadIdx.x];
    // output layout per tile: [gain (2M) | lam (2M) | coef (2M) | d], modes beyond M dropped
    const int i = threadIdx.x;
    R* out = p.partial + (row * p.ntiles + tile) * (6 * p.M + 1);
    if (i == NSUM - 1) out[6 * p.M] = a;
    else {
      const int m = i / 6, k = i % 6;
      if (m < p.M) out[(k / 2) * 2 * p.M + 2 * m + (k & 1)] = a;
    }
  }
  __syncthreads();   // the shared scratch is rewritten by the next tile
  }   // tiles of the run
}

}  // namespace ptb
