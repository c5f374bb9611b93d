// Fix-up kernels of the first-order per-sample-coefficient recurrence whose rows are cut into
// pieces along time: S segments per row inside one device and, optionally, W time shards on W
// devices (rank r owns the samples [r T/W, (r+1) T/W) of every row).
//
// Every piece is first scanned from a ZERO incoming state (scan kernels, one pass over the data),
// which also yields the piece's total affine map (P = product of a, e = end state from zero).
// The true incoming state of a piece is the fold of the maps of all pieces before it,
//     s <- P_k s + e_k,
// and by linearity the piece's true output is
//     y[t] += (prod_{u<=t} a[u]) * s.
// The correction z[t] = a[t] z[t-1], z[-1] = s, normally underflows to EXACTLY zero after a few
// thousand samples (|a| < 1), and once zero it stays zero: each row is corrected block by block
// from its start and the walk stops at the first block whose incoming z is exactly 0.0.  Nothing
// is approximated by stopping there; if the products never vanish the walk covers the whole piece.
//
// The adjoint mirrors this from the right: pieces are scanned with nothing entering from the
// right, the adjoint state c entering piece k is the fold of the maps of the pieces to its right,
// and   grad_x[t] += d[t],  grad_a[t] += d[t] * y[t-1],  d[t] = c * prod_{t<u<L} a[u].
//
// One CTA per (row, segment).  The fold (at most W-1 + S-1 maps) is done by one thread from shared
// memory in the sequential order; the walk takes NT*SPT samples per step with a multiplicative
// block scan (warp shuffles + one shared-memory exchange).
#pragma once
#include "ptx.cuh"
#include "complex.cuh"

#include <cstdint>

namespace ptb {

constexpr int kFixNT = 256;     // threads per CTA
constexpr int kFixSPT = 4;      // consecutive samples per thread and step
constexpr int kFixBlock = kFixNT * kFixSPT;

template <class S>
struct FixupParams {
  // geometry: R = B * nseg kernel rows of L samples; kernel row r = b * nseg + j
  int64_t B, nseg, L;
  const S* a; int64_t a_row_stride;   // L (per kernel row) or 0 (one (L,) array shared by the rows; nseg == 1)
  const S* seg_maps;                  // (R, 2): {P, e} of every piece (forward) / {P, adjoint end state} (adjoint)
  const S* rank_maps;                 // (W, B, 2) total maps of the time shards, or nullptr (one shard)
  int rank, world;
  // forward
  const S* zi;                        // (B,) state entering the whole sequence
  S* y;                               // (R, L) corrected in place
  S* states;                          // (R,) out (forward) / in (adjoint): state entering every piece
  // adjoint
  S* grad_x;                          // (R, L) corrected in place
  S* grad_a;                          // (R, L) or, with shared coefficients, (L,) (atomic adds); nullptr: not wanted
  S* grad_zi;                         // (B,) out, or nullptr: adjoint state leaving the shard on its left
};

template <class S>
__device__ __forceinline__ S shfl_up_val(S v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }

// Multiplicative exclusive scan of one value per thread over the CTA.  Returns this thread's
// exclusive prefix; `total` receives the product over all threads (identical in every thread).
template <class S>
__device__ __forceinline__ S block_excl_prod(S v, S* sm_warp, S& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  S inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const S o = shfl_up_val(inc, d);
    if (lane >= d) inc *= o;
  }
  S exc = shfl_up_val(inc, 1);
  if (lane == 0) exc = S(1);
  __syncthreads();                       // previous step's readers are done with sm_warp
  if (lane == 31) sm_warp[warp] = inc;
  __syncthreads();
  S wpre = S(1), tot = S(1);
#pragma unroll
  for (int w = 0; w < kFixNT / 32; ++w) {
    const S t = sm_warp[w];
    if (w < warp) wpre *= t;
    tot *= t;
  }
  total = tot;
  return wpre * exc;
}

// State entering kernel row (b, j): fold of the shards before `rank`, then of the segments before j.
// Called by all threads; returns the same value in all of them.
template <class S>
__device__ __forceinline__ S fold_forward(const FixupParams<S>& p, int64_t b, int64_t j, S* sm_maps, S* sm_out) {
  // stage the maps in shared memory (batches of kFixNT), fold sequentially by thread 0
  S s = S(0);
  if (threadIdx.x == 0) s = p.zi[b];
  const int64_t n_rank = p.rank_maps ? p.rank : 0;
  const int64_t n = n_rank + j;
  for (int64_t base = 0; base < n; base += kFixNT) {
    const int64_t k = base + threadIdx.x;
    __syncthreads();
    if (k < n) {
      const S* m = k < n_rank ? p.rank_maps + (k * p.B + b) * 2 : p.seg_maps + (b * p.nseg + (k - n_rank)) * 2;
      sm_maps[2 * threadIdx.x] = m[0];
      sm_maps[2 * threadIdx.x + 1] = m[1];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int cnt = (int)((n - base) < kFixNT ? (n - base) : kFixNT);
      for (int i = 0; i < cnt; ++i) s = sm_maps[2 * i] * s + sm_maps[2 * i + 1];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *sm_out = s;
  __syncthreads();
  return *sm_out;
}

// Adjoint state entering kernel row (b, j) from its right: fold of the shards after `rank`
// (from the last one down), then of the segments after j (from the last one down).
template <class S>
__device__ __forceinline__ S fold_backward(const FixupParams<S>& p, int64_t b, int64_t j, S* sm_maps, S* sm_out) {
  S c = S(0);
  const int64_t n_rank = p.rank_maps ? (p.world - 1 - p.rank) : 0;
  const int64_t n_seg = p.nseg - 1 - j;
  const int64_t n = n_rank + n_seg;
  for (int64_t base = 0; base < n; base += kFixNT) {
    const int64_t k = base + threadIdx.x;   // k-th map of the walk from the far right
    __syncthreads();
    if (k < n) {
      const S* m = k < n_rank ? p.rank_maps + ((p.world - 1 - k) * p.B + b) * 2
                              : p.seg_maps + (b * p.nseg + (p.nseg - 1 - (k - n_rank))) * 2;
      sm_maps[2 * threadIdx.x] = m[0];
      sm_maps[2 * threadIdx.x + 1] = m[1];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const int cnt = (int)((n - base) < kFixNT ? (n - base) : kFixNT);
      for (int i = 0; i < cnt; ++i) c = sm_maps[2 * i] * c + sm_maps[2 * i + 1];
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *sm_out = c;
  __syncthreads();
  return *sm_out;
}

template <class S>
__global__ void __launch_bounds__(kFixNT) fixup_fwd_kernel(const FixupParams<S> p) {
  __shared__ S sm_maps[2 * kFixNT];
  __shared__ S sm_warp[kFixNT / 32];
  __shared__ S sm_state;
  const int64_t R = p.B * p.nseg;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const int64_t b = r / p.nseg, j = r - b * p.nseg;
    const S s = fold_forward(p, b, j, sm_maps, &sm_state);
    if (threadIdx.x == 0) p.states[r] = s;
    const S* a = p.a + r * p.a_row_stride;
    S* y = p.y + r * p.L;
    S carry = s;   // z just before the block
    for (int64_t t0 = 0; t0 < p.L && carry != S(0); t0 += kFixBlock) {
      const int64_t t = t0 + (int64_t)threadIdx.x * kFixSPT;
      S pr[kFixSPT];
      S run = S(1);
#pragma unroll
      for (int i = 0; i < kFixSPT; ++i) {
        if (t + i < p.L) run *= ld_ro(a + t + i);
        pr[i] = run;
      }
      S total;
      const S exc = block_excl_prod(run, sm_warp, total);
      const S zin = carry * exc;
#pragma unroll
      for (int i = 0; i < kFixSPT; ++i)
        if (t + i < p.L) y[t + i] += zin * pr[i];
      carry *= total;
    }
  }
}

template <class S>
__global__ void __launch_bounds__(kFixNT) fixup_bwd_kernel(const FixupParams<S> p) {
  __shared__ S sm_maps[2 * kFixNT];
  __shared__ S sm_warp[kFixNT / 32];
  __shared__ S sm_state;
  const int64_t R = p.B * p.nseg;
  for (int64_t r = blockIdx.x; r < R; r += gridDim.x) {
    const int64_t b = r / p.nseg, j = r - b * p.nseg;
    const S c0 = fold_backward(p, b, j, sm_maps, &sm_state);
    if (j == 0 && p.grad_zi && threadIdx.x == 0) {
      const S* m = p.seg_maps + (b * p.nseg) * 2;   // the adjoint state leaving the first segment on its left
      p.grad_zi[b] = m[0] * c0 + m[1];
    }
    const S* a = p.a + r * p.a_row_stride;
    const S* y = p.y + r * p.L;
    S* gx = p.grad_x + r * p.L;
    S* ga = p.grad_a ? p.grad_a + r * p.a_row_stride : nullptr;
    const bool shared_a = p.a_row_stride == 0;
    const S yprev0 = p.states[r];
    S carry = c0;   // d of the block's last sample
    for (int64_t hi = p.L; hi > 0 && carry != S(0); hi -= kFixBlock) {
      // k-th sample of the descending walk: t = hi - 1 - k; d[t] = carry * prod_{m<k} a[hi-1-m]
      const int64_t k0 = (int64_t)threadIdx.x * kFixSPT;
      S ex[kFixSPT];
      S run = S(1);
#pragma unroll
      for (int i = 0; i < kFixSPT; ++i) {
        const int64_t t = hi - 1 - (k0 + i);
        ex[i] = run;
        if (t >= 0) run *= ld_ro(a + t);
      }
      S total;
      const S exc = block_excl_prod(run, sm_warp, total);
      const S din = carry * exc;
#pragma unroll
      for (int i = 0; i < kFixSPT; ++i) {
        const int64_t t = hi - 1 - (k0 + i);
        if (t >= 0) {
          const S d = din * ex[i];
          gx[t] += d;
          if (ga) {
            const S yp = t > 0 ? ld_ro(y + t - 1) : yprev0;
            if (shared_a) atomicAdd(ga + t, d * yp);
            else ga[t] += d * yp;
          }
        }
      }
      carry *= total;
    }
  }
}

// Total map of every row's S pieces: forward (reverse = 0) s -> P_{S-1}(...P_0 s + e_0...) + e_{S-1};
// adjoint (reverse = 1) the same fold from the last piece down.  One thread per row.
template <class S>
__global__ void fold_maps_kernel(const S* __restrict__ maps, int64_t B, int64_t nseg, int reverse, S* __restrict__ out) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  S P = S(1), e = S(0);
  for (int64_t i = 0; i < nseg; ++i) {
    const int64_t k = reverse ? nseg - 1 - i : i;
    const S Pk = maps[(b * nseg + k) * 2], ek = maps[(b * nseg + k) * 2 + 1];
    e = Pk * e + ek;
    P *= Pk;
  }
  out[b * 2] = P;
  out[b * 2 + 1] = e;
}

}  // namespace ptb
