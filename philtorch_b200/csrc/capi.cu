// C ABI of the linear-recurrence kernels: argument checks, workspace layout, launches.
// See include/philtorch_b200.h for the contract of every entry point.
#include "../../include/philtorch_b200.h"

#include "first_order.cuh"

#include <algorithm>

namespace ptb {

constexpr int kMinTile = 512;        // every policy's TILE is at least this (workspace bound)
constexpr int kTileRecordBytes = 160;   // look-back record + Partial, generous upper bound
constexpr int kHeaderBytes = 256;
constexpr int kMaxDevices = 64;

static thread_local int g_last_cuda_error = 0;

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

template <class P>
static int launch_scan(const typename P::Params& prm, int64_t B, int64_t T, bool bulk, void* workspace,
                       int64_t workspace_bytes, uint32_t* status, cudaStream_t st, void** partial_out,
                       int64_t* nchunks_out) {
  static_assert(P::TILE >= kMinTile, "workspace bound assumes TILE >= kMinTile");
  static_assert(P::SLOT_WORDS * 8 + sizeof(typename P::Partial) <= kTileRecordBytes,
                "per-tile record too large");
  static_assert(P::STAGE_BYTES % 128 == 0, "stages must stay 128-byte aligned");
  const int64_t nchunks = (T + P::TILE - 1) / P::TILE;
  const int64_t ntiles = B * nchunks;
  if (ntiles >= 0xFFFFFFFEll || B >= 0xFFFFFFFFll) return PTB_ERR_TOO_LARGE;
  const WsLayout l = ws_layout(ntiles, P::SLOT_WORDS, sizeof(typename P::Partial));
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_bytes < l.total)
    return PTB_ERR_WORKSPACE;
  char* w = static_cast<char*>(workspace);
  PTB_CUDA(cudaMemsetAsync(w, 0, (size_t)l.part_off, st));   // header + look-back records
  Workspace ws;
  ws.ticket = reinterpret_cast<uint32_t*>(w);
  ws.error = status ? status : reinterpret_cast<uint32_t*>(w + 4);
  ws.slots = reinterpret_cast<uint64_t*>(w + l.slots_off);
  ws.partial = w + l.part_off;
  if (partial_out) *partial_out = ws.partial;
  if (nchunks_out) *nchunks_out = nchunks;

  static KernelCache<P> cache;
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  constexpr int smem = EngineSmem<P>::kTotal;
  if (!cache.ready[dev]) {
    PTB_CUDA(cudaFuncSetAttribute(scan_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    int occ = 0;
    PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, scan_kernel<P>, P::NT + 32 * (P::STAGES + 1), smem));
    int sms = 0;
    PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cache.ctas_per_sm[dev] = std::max(occ, 1);
    cache.sms[dev] = sms;
    cache.ready[dev] = true;
  }
  const int64_t resident = (int64_t)cache.sms[dev] * cache.ctas_per_sm[dev];
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, resident);
  scan_kernel<P><<<grid, P::NT + 32 * (P::STAGES + 1), smem, st>>>(prm, ws, (uint32_t)B, T, (uint32_t)nchunks, (uint32_t)ntiles,
                                                bulk ? 1 : 0);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

// Sums per-tile partials: part[row][chunk][N] -> out[row][N] (batched) or out[N] (all rows).
template <class S, int N>
__global__ void reduce_partials_kernel(const S* __restrict__ part, S* __restrict__ out, int64_t B,
                                       int64_t nchunks, int batched) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  if (batched) {
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= B) return;
    double acc[N];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.0;
    for (int64_t c = lane; c < nchunks; c += 32)
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] += (double)part[(row * nchunks + c) * N + i];
#pragma unroll
    for (int i = 0; i < N; ++i) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], d);
      if (lane == 0) out[row * N + i] = (S)acc[i];
    }
  } else {
    __shared__ double sm[32][N];
    double acc[N];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.0;
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
    if (threadIdx.x < N) {
      double t = 0.0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sm[w][threadIdx.x];
      out[threadIdx.x] = (S)t;
    }
  }
}

template <class S, int N>
static int launch_reduce(const void* part, void* out, int64_t B, int64_t nchunks, int batched, cudaStream_t st) {
  if (batched) {
    const int wpb = 4;
    reduce_partials_kernel<S, N><<<(unsigned)((B + wpb - 1) / wpb), wpb * 32, 0, st>>>(
        static_cast<const S*>(part), static_cast<S*>(out), B, nchunks, 1);
  } else {
    reduce_partials_kernel<S, N><<<1, 1024, 0, st>>>(static_cast<const S*>(part), static_cast<S*>(out), B,
                                                    nchunks, 0);
  }
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

// ---------------------------------------------------------------------------- first order
// Tile geometry: 3 x 16 bytes per thread and array (odd => bank-conflict-free strided access).
// (16-byte units per thread and array, stages, CTAs per SM); overridable for tuning experiments
#ifndef PTB_FO_FWD_CH
#define PTB_FO_FWD_CH 3
#define PTB_FO_FWD_STAGES 3
#define PTB_FO_FWD_CTAS 3
#endif
#ifndef PTB_FO_BWD_CH
#define PTB_FO_BWD_CH 3
#define PTB_FO_BWD_STAGES 3
#define PTB_FO_BWD_CTAS 2
#endif
template <class S, bool LPV> using FoFwdP = FoFwd<S, PTB_FO_FWD_CH, PTB_FO_FWD_STAGES, PTB_FO_FWD_CTAS, LPV>;
template <class S, bool LPV> using FoBwdP = FoBwd<S, PTB_FO_BWD_CH, PTB_FO_BWD_STAGES, PTB_FO_BWD_CTAS, LPV>;

template <class S, bool LPV>
static int fo_fwd(int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
                  const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = FoFwdP<S, LPV>;
  typename P::Params p;
  p.a = static_cast<const S*>(a);
  p.a_row_stride = a_batched ? (LPV ? T : 1) : 0;
  p.zi = static_cast<const S*>(zi);
  p.zi_stride = zi_batched ? 1 : 0;
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  const bool bulk = aligned16(x) && aligned16(y) && (!LPV || aligned16(a)) && (T * sizeof(S)) % 16 == 0;
  return launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

template <class S, bool LPV>
static int fo_bwd(int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
                  const void* y, const void* gy, const void* g_in, void* grad_x, void* grad_a, void* grad_zi,
                  void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = FoBwdP<S, LPV>;
  typename P::Params p;
  p.a = static_cast<const S*>(a);
  p.a_row_stride = a_batched ? (LPV ? T : 1) : 0;
  p.zi = static_cast<const S*>(zi);
  p.zi_stride = zi_batched ? 1 : 0;
  p.y = static_cast<const S*>(y);
  p.gy = static_cast<const S*>(gy);
  p.g_in = static_cast<const S*>(g_in);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_a = LPV ? static_cast<S*>(grad_a) : nullptr;
  p.grad_zi = static_cast<S*>(grad_zi);
  p.T = T;
  p.want_ga = grad_a != nullptr;
  const bool bulk = aligned16(gy) && aligned16(grad_x) && (!LPV || aligned16(a)) &&
                    (!p.want_ga || (aligned16(y) && (!LPV || aligned16(grad_a)))) &&
                    (T * sizeof(S)) % 16 == 0;
  void* partial = nullptr;
  int64_t nchunks = 0;
  int rc = launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, &partial, &nchunks);
  if (rc != PTB_OK) return rc;
  if (!LPV && grad_a) rc = launch_reduce<S, 1>(partial, grad_a, B, nchunks, a_batched, st);
  return rc;
}

}  // namespace ptb

using namespace ptb;

extern "C" {

const char* ptb_version(void) { return "philtorch_b200 0.1 (sm_100a)"; }

const char* ptb_error_string(int code) {
  switch (code) {
    case PTB_OK: return "ok";
    case PTB_ERR_ARG: return "invalid argument (null pointer, negative size or unknown dtype)";
    case PTB_ERR_WORKSPACE: return "workspace missing, not 256-byte aligned or smaller than ptb_workspace_bytes";
    case PTB_ERR_CUDA: return "CUDA runtime call failed";
    case PTB_ERR_TOO_LARGE: return "problem needs more than 2^32-2 tiles";
    default: return "unknown error";
  }
}

int ptb_last_cuda_error(void) { return g_last_cuda_error; }

int64_t ptb_workspace_bytes(int64_t B, int64_t T) {
  if (B <= 0 || T <= 0) return kHeaderBytes;
  const int64_t ntiles = B * ((T + kMinTile - 1) / kMinTile);
  return kHeaderBytes + 2 * 256 + (int64_t)kTileRecordBytes * ntiles;
}

int ptb_read_status(const uint32_t* status, ptb_stream_t stream, uint32_t* host_out) {
  if (!status || !host_out) return PTB_ERR_ARG;
  PTB_CUDA(cudaMemcpyAsync(host_out, status, sizeof(uint32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  PTB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  return PTB_OK;
}

#define PTB_DISPATCH(dtype, CALL)              \
  switch (dtype) {                             \
    case PTB_F32: { using S = float; return CALL; }   \
    case PTB_F64: { using S = double; return CALL; }  \
    default: return PTB_ERR_ARG;               \
  }

int ptb_lti_recur_fwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* x, void* y, void* zf, void* workspace,
                      int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !zi || !x || !y) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_fwd<S, false>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace,
                                        workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lpv_recur_fwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* x, void* y, void* zf, void* workspace,
                      int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !zi || !x || !y) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_fwd<S, true>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace,
                                       workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lti_recur_bwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* y, const void* gy, const void* g_in, void* grad_x,
                      void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !gy || !grad_x || (grad_a && (!y || !zi))) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_bwd<S, false>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a,
                                        grad_zi, workspace, workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lpv_recur_bwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* y, const void* gy, const void* g_in, void* grad_x,
                      void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !gy || !grad_x || (grad_a && (!y || !zi))) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_bwd<S, true>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a,
                                       grad_zi, workspace, workspace_bytes, status, (cudaStream_t)stream)));
}

}  // extern "C"
