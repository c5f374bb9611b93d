// Feedback comb filter  y[t] = x[t] - a * y[t - D]  on slabs staged by tiled TMA copies.
//
// A row of the signal is a (steps x D) matrix in memory: step k holds the samples k D .. k D + D - 1
// and the recurrence runs down the columns (phases).  The lane-per-phase kernels of comb.cuh read
// it in 128-byte pieces that lie 4 D bytes apart, which the memory system serves at about two
// thirds of its rate.  Here the signal is described to the TMA unit as a 3-D tensor
// (phase, step, row) and a CTA owns a band of W neighbouring phases of one row: it walks down the
// steps in slabs of KS steps, every slab ONE tiled copy (cp.async.bulk.tensor.3d, box W x KS x 1,
// 16-64 KB) into a ring of shared-memory stages; one thread per phase runs the KS steps of its
// column in shared memory in place, and the slab leaves with one tiled store.  Loads of the next
// stages - 1 slabs are in flight meanwhile.  What counts is the size of a copy: with one 1-D bulk
// copy per step row (256 B - 1 KB) the TMA unit's per-copy cost bounds a row of the signal at
// ~85 GB/s whatever the band width; with tiled copies a CTA's rate still grows with the slab
// height up to 32-64 KB (delay 1000, T = 2^22, 64 rows, fwd+bwd: 1.05 ms at 16 / 8 steps per slab,
// 0.92 ms at 32 / 16, 0.90 ms at 64 / 32; the lane-per-phase kernels: 1.28 ms).
// Phases beyond D in the last band and steps beyond the last full one read as zeros and are
// clipped on the way out by the tensor's bounds.
//
// Needs D and N to be multiples of 16 bytes worth of samples and 16-byte aligned arrays (tensor
// strides); the host falls back to comb.cuh otherwise.  The N mod D samples after the last full
// step are handled with plain loads and stores.
//
// Adjoint (g[t] = gy[t] - a g[t + D], grad_x = g, grad_a = -sum g[t] y[t - D]): the same walk from
// the last step up, with a second slab holding y one step earlier (a box that starts one step
// before the slab; its row -1 reads as zeros and is replaced by the initial state); block sums of
// grad_a go to partial[row][band], the gradient of the initial state of phase d is -a g[d].
#pragma once
#include "comb.cuh"
#include "scan_engine.cuh"

#include <cuda.h>   // CUtensorMap (types only: the encoder is fetched through the runtime)

namespace ptb {

// tiled TMA copies of a (W x KS x 1) box at element coordinates (x, y, z); x * sizeof(element) must be
// a multiple of 16 bytes.  No multicast.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}

constexpr int kCombMaxStages = 16;
constexpr int kCombSlabHeader = 256;   // mbarriers and the warps' sums, ahead of the stage ring

template <class S, int W_, int KS_>
struct CombSlabCfg {
  static constexpr int W = W_, KS = KS_;
  static constexpr int SLAB = KS * W;   // scalars
  static constexpr int bytes(int stages, bool adjoint) {
    return kCombSlabHeader + (adjoint ? 2 : 1) * stages * SLAB * (int)sizeof(S);
  }
};

template <class S>
struct CombSlabParams {
  const S* a; int a_stride;
  const S* zi; int zi_mode;
  int64_t N, D;
  int bands;              // ceil(D / W)
  int stages;             // depth of the shared-memory ring (3 .. kCombMaxStages): stages - 1 slabs are in flight
  uint32_t* status;       // may be nullptr
  uint64_t wait_ns;
  // forward
  const S* x; S* y;
  // adjoint
  const S* gy; const S* yfwd; S* grad_x; S* partial; int partial_stride; S* grad_state;
};

// every thread waits for the stage itself; a wait that ran out raises the CTA's abort word, which all
// threads read after the iteration's barrier (the iteration then worked on stale data: flagged invalid)
__device__ __forceinline__ void comb_stage_wait(uint64_t* bar, uint32_t parity, uint64_t wait_ns, uint32_t* status,
                                                volatile uint32_t* abort_word) {
  if (!mbar_wait_bounded(bar, parity, wait_ns)) {
    if (status) atomicOr(status, kErrLoadTimeout);
    *abort_word = 1u;
  }
}

template <class S, class C>
__global__ void __launch_bounds__(C::W)
comb_slab_fwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                     const CombSlabParams<S> p) {
  constexpr int W = C::W, KS = C::KS;
  constexpr uint32_t kBoxBytes = (uint32_t)C::SLAB * sizeof(S);   // a box counts in full, clipped or not
  const int STAGES = p.stages;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  S* slab = reinterpret_cast<S*>(smem + kCombSlabHeader);
  const int tid = threadIdx.x;
  const int row = (int)(blockIdx.x / p.bands);
  const int d0 = (int)(blockIdx.x % p.bands) * W;
  const int wv = (int)((p.D - d0) < W ? (p.D - d0) : W);
  const int64_t K = p.N / p.D, tail = p.N - K * p.D;
  const int64_t nchunks = (K + KS - 1) / KS;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem + 8 * kCombMaxStages + 64);
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    *abort_word = 0u;
    fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int64_t c) {   // one thread: slab c
    const int s = (int)(c % STAGES);
    mbar_arrive_expect_tx(&full[s], kBoxBytes);
    tma_load_3d(slab + (size_t)s * C::SLAB, &map_x, d0, (int)(c * KS), row, &full[s]);
  };
  if (tid == 0)
    for (int64_t c = 0; c < STAGES - 1 && c < nchunks; ++c) issue(c);
  const bool live = tid < wv;
  const S coef = -p.a[(int64_t)row * p.a_stride];
  S h = live ? comb_initial(p.zi, p.zi_mode, (int64_t)row, p.D, (int64_t)d0 + tid) : S(0);
  int64_t c = 0;
  bool failed = false;
  for (; c < nchunks; ++c) {
    const int s = (int)(c % STAGES);
    comb_stage_wait(&full[s], (uint32_t)((c / STAGES) & 1), p.wait_ns, p.status, abort_word);
    const int64_t k0 = c * KS;
    const int nk = (int)((K - k0) < KS ? (K - k0) : KS);
    S* col = slab + (size_t)s * C::SLAB + tid;
    if (live) {
      if (nk == KS) {
#pragma unroll
        for (int k = 0; k < KS; ++k) { h = coef * h + col[k * W]; col[k * W] = h; }
      } else {
        for (int k = 0; k < nk; ++k) { h = coef * h + col[k * W]; col[k * W] = h; }
      }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (*abort_word) { failed = true; break; }
    if (tid == 0) {
      tma_store_3d(&map_y, slab + (size_t)s * C::SLAB, d0, (int)k0, row);   // steps beyond K are clipped
      bulk_commit();
      if (c + STAGES - 1 < nchunks) {
        // the stage stored one iteration ago is refilled once that store has read it
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        issue(c + STAGES - 1);
      }
    }
  }
  if (failed && tid == 0)   // copies still in flight into this CTA's shared memory: give them a moment before leaving
    for (int64_t j = c; j < nchunks && j < c + STAGES - 1; ++j)
      mbar_wait_bounded(&full[j % STAGES], (uint32_t)((j / STAGES) & 1), kWaitNsAfterError);
  if (live && d0 + tid < tail) {
    const int64_t at = (int64_t)row * p.N + K * p.D + d0 + tid;
    p.y[at] = coef * h + p.x[at];
  }
  if (tid == 0) bulk_wait_all();
}

template <class S, class C>
__global__ void __launch_bounds__(C::W)
comb_slab_bwd_kernel(const __grid_constant__ CUtensorMap map_gy, const __grid_constant__ CUtensorMap map_y,
                     const __grid_constant__ CUtensorMap map_gx, const CombSlabParams<S> p) {
  constexpr int W = C::W, KS = C::KS;
  constexpr uint32_t kBoxBytes = (uint32_t)C::SLAB * sizeof(S);
  const int STAGES = p.stages;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  S* warp_sums = reinterpret_cast<S*>(smem + 8 * kCombMaxStages);
  S* slab_g = reinterpret_cast<S*>(smem + kCombSlabHeader);    // [STAGES][KS][W]  gy in, grad_x out
  S* slab_y = slab_g + (size_t)STAGES * C::SLAB;               // [STAGES][KS][W]  y one step earlier
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = (int)(blockIdx.x / p.bands);
  const int band = (int)(blockIdx.x % p.bands);
  const int d0 = band * W;
  const int wv = (int)((p.D - d0) < W ? (p.D - d0) : W);
  const int64_t K = p.N / p.D, tail = p.N - K * p.D;
  const int64_t nchunks = (K + KS - 1) / KS;
  const bool want_a = p.partial != nullptr;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem + 8 * kCombMaxStages + 64);
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    *abort_word = 0u;
    fence_mbar_init();
  }
  __syncthreads();
  // iteration i handles slab c = nchunks - 1 - i in stage i % STAGES
  auto issue = [&](int64_t i) {   // one thread
    const int s = (int)(i % STAGES);
    const int k0 = (int)((nchunks - 1 - i) * KS);
    mbar_arrive_expect_tx(&full[s], want_a ? 2 * kBoxBytes : kBoxBytes);
    tma_load_3d(slab_g + (size_t)s * C::SLAB, &map_gy, d0, k0, row, &full[s]);
    // y of the steps k0 - 1 .. k0 + KS - 2 (a load may start at step -1: that row reads as zeros)
    if (want_a) tma_load_3d(slab_y + (size_t)s * C::SLAB, &map_y, d0, k0 - 1, row, &full[s]);
  };
  if (tid == 0)
    for (int64_t i = 0; i < STAGES - 1 && i < nchunks; ++i) issue(i);
  const bool live = tid < wv;
  const S coef = -p.a[(int64_t)row * p.a_stride];
  const S init = (live && want_a) ? comb_initial(p.zi, p.zi_mode, (int64_t)row, p.D, (int64_t)d0 + tid) : S(0);
  S h = S(0), acc = S(0);
  if (live && d0 + tid < tail) {   // the samples after the last full step come first
    const int64_t at = (int64_t)row * p.N + K * p.D + d0 + tid;
    h = p.gy[at];
    p.grad_x[at] = h;
    if (want_a) acc = h * (K > 0 ? p.yfwd[at - p.D] : init);
  }
  int64_t i = 0;
  bool failed = false;
  for (; i < nchunks; ++i) {
    const int s = (int)(i % STAGES);
    comb_stage_wait(&full[s], (uint32_t)((i / STAGES) & 1), p.wait_ns, p.status, abort_word);
    const int64_t k0 = (nchunks - 1 - i) * KS;
    const int nk = (int)((K - k0) < KS ? (K - k0) : KS);
    S* cg = slab_g + (size_t)s * C::SLAB + tid;
    const S* cy = slab_y + (size_t)s * C::SLAB + tid;
    if (live) {
      if (nk == KS && k0 > 0) {
#pragma unroll
        for (int k = KS - 1; k >= 0; --k) {
          h = coef * h + cg[k * W];
          cg[k * W] = h;
          if (want_a) acc += h * cy[k * W];
        }
      } else {
        for (int k = nk - 1; k >= 0; --k) {
          h = coef * h + cg[k * W];
          cg[k * W] = h;
          if (want_a) acc += h * (k0 + k > 0 ? cy[k * W] : init);
        }
      }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (*abort_word) { failed = true; break; }
    if (tid == 0) {
      tma_store_3d(&map_gx, slab_g + (size_t)s * C::SLAB, d0, (int)k0, row);
      bulk_commit();
      if (i + STAGES - 1 < nchunks) {
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        issue(i + STAGES - 1);
      }
    }
  }
  if (failed && tid == 0)
    for (int64_t j = i; j < nchunks && j < i + STAGES - 1; ++j)
      mbar_wait_bounded(&full[j % STAGES], (uint32_t)((j / STAGES) & 1), kWaitNsAfterError);
  if (p.grad_state && live)
    p.grad_state[(int64_t)row * p.D + (p.D - 1 - (d0 + tid))] = (d0 + tid < p.N) ? coef * h : S(0);
  if (want_a) {   // grad_a = - sum g[t] y[t - D]: block sum
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
    if (lane == 0) warp_sums[warp] = acc;
    __syncthreads();
    if (tid == 0) {
      S t = S(0);
      for (int w = 0; w < W / 32; ++w) t += warp_sums[w];
      p.partial[(int64_t)row * p.partial_stride + band] = -t;
    }
  }
  if (tid == 0) bulk_wait_all();
}

}  // namespace ptb
