// Host-side launch helpers shared by the translation units of the C ABI: workspace layout, the
// launch of scan_kernel<P> (per-device occupancy cache, persistent grid) and the reduction of
// per-tile partial sums.
#pragma once
#include "../../include/philtorch_b200.h"

#include "scan_engine.cuh"

#include <algorithm>
#include <mutex>

namespace ptb {

constexpr int kMinTile = 512;        // every policy's TILE is at least this (workspace bound)
constexpr int kTileRecordBytes = 160;   // look-back record + Partial, generous upper bound
constexpr int kHeaderBytes = 256;
constexpr int kMaxDevices = 64;

inline thread_local int g_last_cuda_error = 0;
// guards the lazily filled per-device launch caches (occupancy, function attributes, symbol addresses)
inline std::mutex& init_mutex() {
  static std::mutex m;
  return m;
}
inline uint64_t g_wait_ns = kDefaultWaitNs;   // bound of every device-side wait (ptb_set_wait_limit_ms)

#define PTB_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t e_ = (expr);                             \
    if (e_ != cudaSuccess) {                             \
      g_last_cuda_error = (int)e_;                       \
      return PTB_ERR_CUDA;                               \
    }                                                    \
  } while (0)

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct WsLayout {
  int64_t slots_off, part_off, total;
};
static WsLayout ws_layout(int64_t ntiles, int slot_words, int part_bytes) {
  WsLayout l;
  l.slots_off = kHeaderBytes;
  l.part_off = l.slots_off + align_up((int64_t)slot_words * 8 * ntiles, 256);
  l.total = l.part_off + align_up((int64_t)part_bytes * ntiles, 256);
  return l;
}

template <class P>
struct KernelCache {
  bool ready[kMaxDevices] = {};
  int ctas_per_sm[kMaxDevices] = {};
  int sms[kMaxDevices] = {};
};

template <class P, bool kGenericWorkspaceBound = true>
static int launch_scan(const typename P::Params& prm, int64_t B, int64_t T, bool bulk, void* workspace,
                       int64_t workspace_bytes, uint32_t* status, cudaStream_t st, void** partial_out,
                       int64_t* nchunks_out, bool skip_first_chunk = false) {
  // ptb_workspace_bytes(B, T) must cover every policy launched with the generic bound
  static_assert(!kGenericWorkspaceBound || P::TILE >= kMinTile, "workspace bound assumes TILE >= kMinTile");
  static_assert(!kGenericWorkspaceBound || P::SLOT_WORDS * 8 + sizeof(typename P::Partial) <= kTileRecordBytes,
                "per-tile record too large");
  static_assert(P::STAGE_BYTES % 128 == 0, "stages must stay 128-byte aligned");
  static_assert(EngineSmem<P>::kTotal <= 227 * 1024, "stage ring exceeds the shared memory of an SM");
  const int64_t nchunks = (T + P::TILE - 1) / P::TILE;
  const int64_t ntiles = B * nchunks;
  if (ntiles >= 0xFFFFFFFEll || B >= 0xFFFFFFFFll) return PTB_ERR_TOO_LARGE;
  const WsLayout l = ws_layout(ntiles, P::SLOT_WORDS, sizeof(typename P::Partial));
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < l.total)
    return PTB_ERR_WORKSPACE;
  char* w = static_cast<char*>(workspace);
  PTB_CUDA(cudaMemsetAsync(w, 0, (size_t)l.part_off, st));   // header + look-back records
  // self-test only: start the ticket counter at 1, so the first tile is never processed and its
  // successor's look-back waits for a record that nothing writes
  if (skip_first_chunk) PTB_CUDA(cudaMemsetAsync(w, 1, 1, st));
  Workspace ws;
  ws.ticket = reinterpret_cast<uint32_t*>(w);
  ws.error = status ? status : reinterpret_cast<uint32_t*>(w + 4);
  ws.slots = reinterpret_cast<uint64_t*>(w + l.slots_off);
  ws.partial = w + l.part_off;
  ws.done = reinterpret_cast<uint32_t*>(w + 8);
  if (partial_out) *partial_out = ws.partial;
  if (nchunks_out) *nchunks_out = nchunks;

  static KernelCache<P> cache;
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  constexpr int smem = EngineSmem<P>::kTotal;
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!cache.ready[dev]) {
      PTB_CUDA(cudaFuncSetAttribute(scan_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      int occ = 0;
      PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, scan_kernel<P>, P::NT + 32 * (P::LBW + 1), smem));
      int sms = 0;
      PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      cache.ctas_per_sm[dev] = std::max(occ, 1);
      cache.sms[dev] = sms;
      cache.ready[dev] = true;
    }
  }
  const int64_t resident = (int64_t)cache.sms[dev] * cache.ctas_per_sm[dev];
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, resident);
  // tiles of one row that are in flight together: the depth the look-back usually has to cover
  const int64_t depth = resident * P::STAGES / B;
  const int lb_first = depth > 6 ? 32 : 8;
  scan_kernel<P><<<grid, P::NT + 32 * (P::LBW + 1), smem, st>>>(prm, ws, (uint32_t)B, T, (uint32_t)nchunks, (uint32_t)ntiles,
                                                bulk ? 1 : 0, lb_first, g_wait_ns);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

// Sums per-tile partials part[row][chunk][N] per row (batched) or over all rows, in double, and
// hands the N sums to an epilogue that writes the result.
template <class S, int N>
struct StoreSums {
  S* out;
  __device__ void operator()(int64_t row, const double* acc) const {
    for (int i = 0; i < N; ++i) out[row * N + i] = (S)acc[i];
  }
};
// sums {gy x, x lam0, x lam1, y lam0, y lam1} -> grad_b (3), grad_a (2) of a TDF-II section
template <class S>
struct BiquadCoefGrads {
  const S* a; int64_t a_stride;
  S* grad_b; S* grad_a;
  __device__ void operator()(int64_t row, const double* acc) const {
    const double a1 = (double)a[row * a_stride], a2 = (double)a[row * a_stride + 1];
    if (grad_b) {
      grad_b[row * 3 + 0] = (S)(acc[0] - a1 * acc[1] - a2 * acc[2]);
      grad_b[row * 3 + 1] = (S)acc[1];
      grad_b[row * 3 + 2] = (S)acc[2];
    }
    if (grad_a) {
      grad_a[row * 2 + 0] = (S)(-acc[3]);
      grad_a[row * 2 + 1] = (S)(-acc[4]);
    }
  }
};

template <class S, int N, class Epi>
__global__ void reduce_partials_kernel(const S* __restrict__ part, int64_t B, int64_t nchunks, int batched,
                                       Epi epi) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  double acc[N];
#pragma unroll
  for (int i = 0; i < N; ++i) acc[i] = 0.0;
  if (batched) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= B) return;
    for (int64_t c = lane; c < nchunks; c += 32)
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += (double)part[(row * nchunks + c) * N + i];
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], d);
    if (lane == 0) epi(row, acc);
  } else {
    __shared__ double sm[32][N];
    const int64_t total = B * nchunks;
    for (int64_t c = threadIdx.x; c < total; c += blockDim.x)
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += (double)part[c * N + i];
#pragma unroll
    for (int i = 0; i < N; ++i) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], d);
      if (lane == 0) sm[warp][i] = acc[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      double t[N];
      for (int i = 0; i < N; ++i) {
        t[i] = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t[i] += sm[w][i];
      }
      epi(0, t);
    }
  }
}

template <class S, int N, class Epi>
static int launch_reduce(const void* part, int64_t B, int64_t nchunks, int batched, Epi epi, cudaStream_t st) {
  if (batched) {
    const int wpb = 4;
    reduce_partials_kernel<S, N, Epi><<<(unsigned)((B + wpb - 1) / wpb), wpb * 32, 0, st>>>(
        static_cast<const S*>(part), B, nchunks, 1, epi);
  } else {
    reduce_partials_kernel<S, N, Epi><<<1, 1024, 0, st>>>(static_cast<const S*>(part), B, nchunks, 0, epi);
  }
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

}  // namespace ptb
