// C ABI of the linear-recurrence kernels: argument checks, workspace layout, launches.
// See include/philtorch_b200.h for the contract of every entry point.
#include "launch.cuh"

#include "biquad.cuh"
#include "first_order_host.cuh"
#include "so_small.cuh"

namespace ptb {
// single section through the chained kernels, defined with the cascade (capi_sos.cu); -1: not applicable
int biquad_chain_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                     const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b, void* grad_a,
                     void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st);
// single section on the decoupled kernels with a per-row table of matrix powers (capi_sos.cu); -1: not applicable
int biquad_table_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* zi,
                     const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st);
int biquad_table_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                     const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b, void* grad_a,
                     void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st);
// complex first-order recurrences (capi_cx.cu)
int cx_fo_fwd(int dtype, int lpv, int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
              const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st);
int cx_fo_bwd(int dtype, int lpv, int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
              const void* y, const void* gy, const void* g_in, void* grad_x, void* grad_a, void* grad_zi, void* ws,
              int64_t wsb, uint32_t* status, cudaStream_t st, int ga_shared = 0);
}  // namespace ptb

namespace ptb {

template <class S, bool REV, bool WRITE = false>
static int fo_carry(int64_t B, int64_t T, const void* a, int a_batched, const void* x, void* y, void* carry,
                    void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = FoCarry<S, PTB_FO_FWD_CH, PTB_FO_FWD_STAGES, PTB_FO_FWD_CTAS, REV, WRITE>;
  typename P::Params p;
  p.a = static_cast<const S*>(a);
  p.a_row_stride = a_batched ? T : 0;
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.carry = static_cast<S*>(carry);
  p.T = T;
  const bool bulk = aligned16(x) && aligned16(a) && (!WRITE || aligned16(y)) && (T * sizeof(S)) % 16 == 0;
  return launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

// ---------------------------------------------------------------------------- 2x2
// samples per thread (odd), stages, CTAs per SM
template <class S> struct SoCfg;
// samples per thread (odd) and stages, per precision; one CTA per SM
#ifndef PTB_SO_F32_FWD_NS
#define PTB_SO_F32_FWD_NS 15
#define PTB_SO_F32_FWD_STAGES 2
#endif
#ifndef PTB_SO_F32_BWD_NS
#define PTB_SO_F32_BWD_NS 11
#define PTB_SO_F32_BWD_STAGES 2
#endif
#ifndef PTB_SO_F64_FWD_NS
#define PTB_SO_F64_FWD_NS 7
#define PTB_SO_F64_FWD_STAGES 2
#endif
#ifndef PTB_SO_F64_BWD_NS
#define PTB_SO_F64_BWD_NS 5
#define PTB_SO_F64_BWD_STAGES 2
#endif
#ifndef PTB_SO_CTAS
#define PTB_SO_CTAS 1
#endif
#ifndef PTB_SO_NT
#define PTB_SO_NT 256   // compute threads per CTA
#endif
template <> struct SoCfg<float> {
  static constexpr int FWD_NS = PTB_SO_F32_FWD_NS, FWD_ST = PTB_SO_F32_FWD_STAGES;
  static constexpr int BWD_NS = PTB_SO_F32_BWD_NS, BWD_ST = PTB_SO_F32_BWD_STAGES;
};
template <> struct SoCfg<double> {
  static constexpr int FWD_NS = PTB_SO_F64_FWD_NS, FWD_ST = PTB_SO_F64_FWD_STAGES;
  static constexpr int BWD_NS = PTB_SO_F64_BWD_NS, BWD_ST = PTB_SO_F64_BWD_STAGES;
};
template <class S, bool LPV, bool XS>
using SoFwdP = SoFwd<S, SoCfg<S>::FWD_NS, SoCfg<S>::FWD_ST, PTB_SO_CTAS, PTB_SO_NT, LPV, XS>;
template <class S, bool LPV, bool XS>
using SoBwdP = SoBwd<S, SoCfg<S>::BWD_NS, SoCfg<S>::BWD_ST, PTB_SO_CTAS, PTB_SO_NT, LPV, XS>;

// 2x2 LPV forward in small CTAs (so_small.cuh): from this many rows on
#ifndef PTB_SO_SMALL_MIN_ROWS
#define PTB_SO_SMALL_MIN_ROWS 48
#endif
template <class S> struct SoSmallSel;
#ifndef PTB_SO_SMALL_NT
#define PTB_SO_SMALL_NT 128
#define PTB_SO_SMALL_MINB 4
#define PTB_SO_SMALL_MINB64 3
#endif
#ifndef PTB_SO_SMALL_SPT64
#define PTB_SO_SMALL_SPT64 9
#endif
template <> struct SoSmallSel<float> { using C = LpvBqCfg<float, 15, PTB_SO_SMALL_NT, PTB_SO_SMALL_MINB>; };
template <> struct SoSmallSel<double> { using C = LpvBqCfg<double, PTB_SO_SMALL_SPT64, PTB_SO_SMALL_NT, PTB_SO_SMALL_MINB64>; };

template <class S, bool XS>
static int so_small_fwd(int64_t B, int64_t T, const void* A, int A_batched, const void* zi, const void* x, void* y,
                        void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st, void* tile_prod = nullptr) {
  using C = typename SoSmallSel<S>::C;
  using L = SoSmallFwdSmem<C, XS>;
  static_assert(C::TILE >= kMinTile && C::SLOT_WORDS * 8 <= kTileRecordBytes, "generic workspace bound");
  const int64_t nchunks = (T + C::TILE - 1) / C::TILE;
  const int64_t ntiles = B * nchunks;
  if (ntiles >= 0xFFFFFFFEll || B >= 0xFFFFFFFFll) return PTB_ERR_TOO_LARGE;
  const WsLayout l = ws_layout(ntiles, C::SLOT_WORDS, 0);
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < l.total) return PTB_ERR_WORKSPACE;
  char* w = static_cast<char*>(ws);
  PTB_CUDA(cudaMemsetAsync(w, 0, (size_t)l.part_off, st));
  Workspace wk;
  wk.ticket = reinterpret_cast<uint32_t*>(w);
  wk.error = status ? status : reinterpret_cast<uint32_t*>(w + 4);
  wk.slots = reinterpret_cast<uint64_t*>(w + l.slots_off);
  wk.partial = nullptr;
  SoSmallFwdParams<S> p;
  p.A = static_cast<const S*>(A);
  p.a_row = A_batched ? 4 * T : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  p.tile_prod = static_cast<S*>(tile_prod);
  const bool bulk = aligned16(x) && aligned16(y) && aligned16(A) && (T * (XS ? 1 : 2) * sizeof(S)) % 16 == 0;
  static bool attr_set[kMaxDevices] = {};
  static int grid_max[kMaxDevices] = {};
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!attr_set[dev]) {
      PTB_CUDA(cudaFuncSetAttribute(so_small_fwd_kernel<S, C, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      int sms = 0, occ = 1;
      PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, so_small_fwd_kernel<S, C, XS>, C::NT, L::kTotal));
      grid_max[dev] = sms * std::max(occ, 1);
      attr_set[dev] = true;
    }
  }
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, grid_max[dev]);
  so_small_fwd_kernel<S, C, XS><<<grid, C::NT, L::kTotal, st>>>(p, wk, (uint32_t)B, (uint32_t)nchunks, (uint32_t)ntiles,
                                                                bulk ? 1 : 0, g_wait_ns);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

static int g_so_small_min_rows = PTB_SO_SMALL_MIN_ROWS;
static int g_bq_policy = 0;   // ptb_biquad_set_policy: 0 table-of-powers kernels, 1 generic 2x2 policy (tests)

#ifndef PTB_SO_SMALL_BWD_MINB
#define PTB_SO_SMALL_BWD_NT 128
#define PTB_SO_SMALL_BWD_SPT 11
#define PTB_SO_SMALL_BWD_MINB 4
#define PTB_SO_SMALL_BWD_SPT64 5
#define PTB_SO_SMALL_BWD_MINB64 4
#endif
template <class S> struct SoSmallBwdSel;
template <> struct SoSmallBwdSel<float> { using C = LpvBqCfg<float, PTB_SO_SMALL_BWD_SPT, PTB_SO_SMALL_BWD_NT, PTB_SO_SMALL_BWD_MINB>; };
template <> struct SoSmallBwdSel<double> { using C = LpvBqCfg<double, PTB_SO_SMALL_BWD_SPT64, PTB_SO_SMALL_BWD_NT, PTB_SO_SMALL_BWD_MINB64>; };

template <class S, bool XS>
static int so_small_bwd(int64_t B, int64_t T, const void* A, int A_batched, const void* zi, const void* y,
                        const void* gy, const void* g_in, void* grad_x, void* grad_A, void* grad_zi, void* ws,
                        int64_t wsb, uint32_t* status, cudaStream_t st, bool gA_shared = false) {
  using C = typename SoSmallBwdSel<S>::C;
  using L = SoSmallBwdSmem<C, XS>;
  static_assert(C::TILE >= kMinTile && C::SLOT_WORDS * 8 <= kTileRecordBytes, "generic workspace bound");
  static_assert(L::kTotal * C::MINB <= 227 * 1024, "shared memory of an SM");
  const int64_t nchunks = (T + C::TILE - 1) / C::TILE;
  const int64_t ntiles = B * nchunks;
  if (ntiles >= 0xFFFFFFFEll || B >= 0xFFFFFFFFll) return PTB_ERR_TOO_LARGE;
  const WsLayout l = ws_layout(ntiles, C::SLOT_WORDS, 0);
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < l.total) return PTB_ERR_WORKSPACE;
  char* w = static_cast<char*>(ws);
  PTB_CUDA(cudaMemsetAsync(w, 0, (size_t)l.part_off, st));
  Workspace wk;
  wk.ticket = reinterpret_cast<uint32_t*>(w);
  wk.error = status ? status : reinterpret_cast<uint32_t*>(w + 4);
  wk.slots = reinterpret_cast<uint64_t*>(w + l.slots_off);
  wk.partial = nullptr;
  SoSmallBwdParams<S> p;
  p.A = static_cast<const S*>(A);
  p.a_row = A_batched ? 4 * T : 0;
  p.zi = static_cast<const S*>(zi);
  p.y = static_cast<const S*>(y);
  p.gy = static_cast<const S*>(gy);
  p.g_in = static_cast<const S*>(g_in);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_A = static_cast<S*>(grad_A);
  p.grad_zi = static_cast<S*>(grad_zi);
  p.T = T;
  p.gA_shared = gA_shared ? 1 : 0;
  const bool bulk = aligned16(gy) && aligned16(grad_x) && aligned16(A) &&
                    (!grad_A || (aligned16(y) && aligned16(grad_A))) && (T * (XS ? 1 : 2) * sizeof(S)) % 16 == 0;
  if (gA_shared && !bulk) return PTB_ERR_ARG;
  static bool attr_set[kMaxDevices] = {};
  static int grid_max[kMaxDevices] = {};
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!attr_set[dev]) {
      PTB_CUDA(cudaFuncSetAttribute(so_small_bwd_kernel<S, C, XS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      int sms = 0, occ = 1;
      PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, so_small_bwd_kernel<S, C, XS>, C::NT, L::kTotal));
      grid_max[dev] = sms * std::max(occ, 1);
      attr_set[dev] = true;
    }
  }
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, grid_max[dev]);
  so_small_bwd_kernel<S, C, XS><<<grid, C::NT, L::kTotal, st>>>(p, wk, (uint32_t)B, (uint32_t)nchunks, (uint32_t)ntiles,
                                                                bulk ? 1 : 0, g_wait_ns);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S, bool LPV, bool XS>
static int so_fwd(int64_t B, int64_t T, const void* A, int A_batched, const void* zi, const void* x, void* y,
                  void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  if constexpr (LPV) {
    if (B >= g_so_small_min_rows) return so_small_fwd<S, XS>(B, T, A, A_batched, zi, x, y, zf, ws, wsb, status, st);
  }
  using P = SoFwdP<S, LPV, XS>;
  typename P::Params p;
  p.A = static_cast<const S*>(A);
  p.a_row_stride = A_batched ? (LPV ? 4 * T : 4) : 0;
  p.zi = static_cast<const S*>(zi);
  p.zi_stride = 2;
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  const bool bulk = aligned16(x) && aligned16(y) && (!LPV || aligned16(A)) &&
                    (T * (XS ? 1 : 2) * sizeof(S)) % 16 == 0;
  return launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

template <class S, bool LPV, bool XS>
static int so_bwd(int64_t B, int64_t T, const void* A, int A_batched, const void* zi, const void* y,
                  const void* gy, const void* g_in, void* grad_x, void* grad_A, void* grad_zi, void* ws,
                  int64_t wsb, uint32_t* status, cudaStream_t st, bool gA_shared = false) {
  if (gA_shared && (!LPV || A_batched || !grad_A)) return PTB_ERR_ARG;
  if constexpr (LPV) {
    if (B >= g_so_small_min_rows && (grad_A == nullptr || A_batched || gA_shared))
      return so_small_bwd<S, XS>(B, T, A, A_batched, zi, y, gy, g_in, grad_x, grad_A, grad_zi, ws, wsb, status, st,
                                 gA_shared);
  }
  using P = SoBwdP<S, LPV, XS>;
  typename P::Params p;
  p.A = static_cast<const S*>(A);
  p.a_row_stride = A_batched ? (LPV ? 4 * T : 4) : 0;
  p.zi = static_cast<const S*>(zi);
  p.zi_stride = 2;
  p.y = static_cast<const S*>(y);
  p.gy = static_cast<const S*>(gy);
  p.g_in = static_cast<const S*>(g_in);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_A = LPV ? static_cast<S*>(grad_A) : nullptr;
  p.grad_zi = static_cast<S*>(grad_zi);
  p.T = T;
  p.want_gA = grad_A != nullptr;
  p.gA_shared = gA_shared ? 1 : 0;
  const bool bulk = aligned16(gy) && aligned16(grad_x) && (!LPV || aligned16(A)) &&
                    (!p.want_gA || (aligned16(y) && (!LPV || aligned16(grad_A)))) &&
                    (T * (XS ? 1 : 2) * sizeof(S)) % 16 == 0;
  if (gA_shared && !bulk) return PTB_ERR_ARG;
  void* partial = nullptr;
  int64_t nchunks = 0;
  int rc = launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, &partial, &nchunks);
  if (rc != PTB_OK) return rc;
  if (!LPV && grad_A)
    rc = launch_reduce<S, 4>(partial, B, nchunks, A_batched, StoreSums<S, 4>{static_cast<S*>(grad_A)}, st);
  return rc;
}

// ---------------------------------------------------------------------------- TDF-II section
#ifndef PTB_BQ_FWD_CH
#define PTB_BQ_FWD_CH 13
#define PTB_BQ_FWD_STAGES 2
#define PTB_BQ_FWD_CTAS 2
#endif
#ifndef PTB_BQ_BWD_CH
#define PTB_BQ_BWD_CH 7
#define PTB_BQ_BWD_STAGES 2
#define PTB_BQ_BWD_CTAS 1
#endif
#ifndef PTB_BQ_NT
#define PTB_BQ_NT 256
#endif
template <class S> using BqFwdP = BqFwd<S, PTB_BQ_FWD_CH, PTB_BQ_FWD_STAGES, PTB_BQ_FWD_CTAS, PTB_BQ_NT>;
template <class S> using BqBwdP = BqBwd<S, PTB_BQ_BWD_CH, PTB_BQ_BWD_STAGES, PTB_BQ_BWD_CTAS, PTB_BQ_NT>;

template <class S>
static int bq_fwd(int64_t B, int64_t T, const void* b, const void* a, int batched, const void* zi, const void* x,
                  void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = BqFwdP<S>;
  typename P::Params p;
  p.b = static_cast<const S*>(b); p.b_stride = batched ? 3 : 0;
  p.a = static_cast<const S*>(a); p.a_stride = batched ? 2 : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  const bool bulk = aligned16(x) && aligned16(y) && (T * sizeof(S)) % 16 == 0;
  return launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

template <class S>
static int bq_bwd(int64_t B, int64_t T, const void* b, const void* a, int batched, const void* x, const void* y,
                  const void* gy, const void* g_zf, void* grad_x, void* grad_b, void* grad_a, void* grad_zi,
                  void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = BqBwdP<S>;
  typename P::Params p;
  p.b = static_cast<const S*>(b); p.b_stride = batched ? 3 : 0;
  p.a = static_cast<const S*>(a); p.a_stride = batched ? 2 : 0;
  p.x = static_cast<const S*>(x);
  p.y = static_cast<const S*>(y);
  p.gy = static_cast<const S*>(gy);
  p.g_in = static_cast<const S*>(g_zf);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_zi = static_cast<S*>(grad_zi);
  p.T = T;
  p.want_coef = (grad_b != nullptr) || (grad_a != nullptr);
  const bool bulk = aligned16(gy) && aligned16(grad_x) && (!p.want_coef || (aligned16(x) && aligned16(y))) &&
                    (T * sizeof(S)) % 16 == 0;
  void* partial = nullptr;
  int64_t nchunks = 0;
  int rc = launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, &partial, &nchunks);
  if (rc != PTB_OK) return rc;
  if (p.want_coef) {
    BiquadCoefGrads<S> epi{static_cast<const S*>(a), batched ? 2 : 0, static_cast<S*>(grad_b),
                           static_cast<S*>(grad_a)};
    rc = launch_reduce<S, 5>(partial, B, nchunks, batched, epi, st);
  }
  return rc;
}

// ---------------------------------------------------------------------------- no-allocation variant
// Scratch that lives in the library image instead of being passed in: one array per GPU that loads
// the library, held until the process exits.  On the host the symbol below is only a stand-in;
// the device address is fetched once per device with cudaGetSymbolAddress.
constexpr int64_t kStaticScratchBytes = 2ll << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static void* g_static_scratch_addr[kMaxDevices] = {};

static int static_scratch(void** out) {
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!g_static_scratch_addr[dev]) {
      void* p = nullptr;
      PTB_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));   // device `dev` is current
      g_static_scratch_addr[dev] = p;
    }
  }
  *out = g_static_scratch_addr[dev];
  return PTB_OK;
}

template <class S>
static int fo_fwd_lpv_static(int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
                             const void* x, void* y, void* zf, uint32_t* status, cudaStream_t st) {
  using P = FoFwdP<S, true>;
  const int64_t ntiles = B * ((T + P::TILE - 1) / P::TILE);
  if (ws_layout(ntiles, P::SLOT_WORDS, sizeof(typename P::Partial)).total > kStaticScratchBytes)
    return PTB_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc != PTB_OK) return rc;
  // launch_scan clears the ticket and the look-back records of this call with cudaMemsetAsync
  return fo_fwd<S, true>(B, T, a, a_batched, zi, zi_batched, x, y, zf, scratch, kStaticScratchBytes, status, st);
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
    case PTB_ERR_SCRATCH_LIMIT:
      return "problem exceeds the built-in scratch of the no-allocation entry point "
             "(see ptb_lpv_recur_fwd_static_max_tiles); use the entry point that takes a workspace";
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
  if (dtype == PTB_C64 || dtype == PTB_C128)
    return cx_fo_fwd(dtype, 0, B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace, workspace_bytes, status,
                     (cudaStream_t)stream);
  if (dtype == PTB_F16)
    return fo_fwd<float, false, __half>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace, workspace_bytes, status,
                                       (cudaStream_t)stream);
  if (dtype == PTB_BF16)
    return fo_fwd<float, false, __nv_bfloat16>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace, workspace_bytes,
                                              status, (cudaStream_t)stream);
  PTB_DISPATCH(dtype, (fo_fwd<S, false>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace,
                                        workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lpv_recur_fwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* x, void* y, void* zf, void* workspace,
                      int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !zi || !x || !y) return PTB_ERR_ARG;
  if (dtype == PTB_C64 || dtype == PTB_C128)
    return cx_fo_fwd(dtype, 1, B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace, workspace_bytes, status,
                     (cudaStream_t)stream);
  if (dtype == PTB_F16)
    return fo_fwd<float, true, __half>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace, workspace_bytes, status,
                                       (cudaStream_t)stream);
  if (dtype == PTB_BF16)
    return fo_fwd<float, true, __nv_bfloat16>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace, workspace_bytes,
                                              status, (cudaStream_t)stream);
  PTB_DISPATCH(dtype, (fo_fwd<S, true>(B, T, a, a_batched, zi, zi_batched, x, y, zf, workspace,
                                       workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lpv_recur_carry(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* x,
                        int reverse, void* carry, void* workspace, int64_t workspace_bytes, uint32_t* status,
                        ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0) return PTB_OK;
  if (T == 0 || !a || !x || !carry) return PTB_ERR_ARG;
  switch (dtype) {
    case PTB_F32:
      return reverse ? fo_carry<float, true>(B, T, a, a_batched, x, nullptr, carry, workspace, workspace_bytes, status,
                                             (cudaStream_t)stream)
                     : fo_carry<float, false>(B, T, a, a_batched, x, nullptr, carry, workspace, workspace_bytes, status,
                                              (cudaStream_t)stream);
    case PTB_F64:
      return reverse ? fo_carry<double, true>(B, T, a, a_batched, x, nullptr, carry, workspace, workspace_bytes, status,
                                              (cudaStream_t)stream)
                     : fo_carry<double, false>(B, T, a, a_batched, x, nullptr, carry, workspace, workspace_bytes, status,
                                               (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur_fwd_carry(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* x, void* y,
                            void* carry, void* workspace, int64_t workspace_bytes, uint32_t* status,
                            ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0) return PTB_OK;
  if (T == 0 || !a || !x || !y || !carry) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_carry<S, false, true>(B, T, a, a_batched, x, y, carry, workspace, workspace_bytes,
                                                 status, (cudaStream_t)stream)));
}

int ptb_lpv_recur2_set_small_cta_min_rows(int64_t rows) {
  if (rows < 1) return PTB_ERR_ARG;
  g_so_small_min_rows = rows > 0x7fffffff ? 0x7fffffff : (int)rows;
  return PTB_OK;
}

int ptb_biquad_set_policy(int policy) {
  if (policy < 0 || policy > 1) return PTB_ERR_ARG;
  g_bq_policy = policy;
  return PTB_OK;
}

int ptb_set_wait_limit_ms(int64_t ms) {
  if (ms < 1 || ms > 600000) return PTB_ERR_ARG;
  g_wait_ns = (uint64_t)ms * 1000000ull;
  return PTB_OK;
}

int64_t ptb_selftest_wait_expiry_elems(void) { return 3 * 2 * (int64_t)FoFwdP<float, true>::TILE + 16; }

int ptb_selftest_wait_expiry(void* workspace, int64_t workspace_bytes, void* buf, int64_t buf_elems,
                             uint32_t* status, ptb_stream_t stream) {
  using P = FoFwdP<float, true>;
  const int64_t T = 2 * (int64_t)P::TILE;
  if (!workspace || !buf || !status || buf_elems < 3 * T + 16) return PTB_ERR_ARG;
  float* f = static_cast<float*>(buf);
  typename P::Params p;
  p.a = f; p.a_row_stride = T;
  p.x = f + T;
  p.y = f + 2 * T;
  p.zi = f + 3 * T; p.zi_stride = 1;
  p.zf = nullptr;
  p.T = T;
  return launch_scan<P>(p, 1, T, true, workspace, workspace_bytes, status, (cudaStream_t)stream, nullptr, nullptr,
                        /*skip_first_chunk=*/true);
}

int64_t ptb_lpv_recur_fwd_static_max_tiles(int dtype) {
  if (dtype != PTB_F32 && dtype != PTB_F64) return 0;   // the entry point dispatches real types only
  // header + one look-back record and one (unused) partial slot per tile
  const int64_t per_tile = dtype == PTB_F64 ? (4 * 8 + 8) : (2 * 8 + 4);
  return (kStaticScratchBytes - kHeaderBytes - 2 * 256) / per_tile;
}

int ptb_lpv_recur_fwd_static(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                             int zi_batched, const void* x, void* y, void* zf, uint32_t* status,
                             ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !zi || !x || !y) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_fwd_lpv_static<S>(B, T, a, a_batched, zi, zi_batched, x, y, zf, status,
                                            (cudaStream_t)stream)));
}

int ptb_lti_recur_bwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* y, const void* gy, const void* g_in, void* grad_x,
                      void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !gy || (grad_a && (!y || !zi))) return PTB_ERR_ARG;   // grad_x may be NULL (not wanted)
  if (dtype == PTB_C64 || dtype == PTB_C128)
    return cx_fo_bwd(dtype, 0, B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi, workspace,
                     workspace_bytes, status, (cudaStream_t)stream);
  if (dtype == PTB_F16)
    return fo_bwd<float, false, __half>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi, workspace,
                                       workspace_bytes, status, (cudaStream_t)stream);
  if (dtype == PTB_BF16)
    return fo_bwd<float, false, __nv_bfloat16>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi,
                                              workspace, workspace_bytes, status, (cudaStream_t)stream);
  PTB_DISPATCH(dtype, (fo_bwd<S, false>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a,
                                        grad_zi, workspace, workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lti_recur_reverse_fused(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* x,
                                const void* second, const void* g_in, double scale, void* out, void* first_state,
                                void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !x || !second || !out) return PTB_ERR_ARG;
  PTB_DISPATCH(dtype, (fo_reverse_fused<S>(B, T, a, a_batched, x, second, g_in, scale, out, first_state, workspace,
                                           workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lpv_recur_bwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* y, const void* gy, const void* g_in, void* grad_x,
                      void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !gy || (grad_a && (!y || !zi))) return PTB_ERR_ARG;   // grad_x may be NULL (not wanted)
  if (dtype == PTB_C64 || dtype == PTB_C128)
    return cx_fo_bwd(dtype, 1, B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi, workspace,
                     workspace_bytes, status, (cudaStream_t)stream);
  if (dtype == PTB_F16)
    return fo_bwd<float, true, __half>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi, workspace,
                                       workspace_bytes, status, (cudaStream_t)stream);
  if (dtype == PTB_BF16)
    return fo_bwd<float, true, __nv_bfloat16>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi,
                                              workspace, workspace_bytes, status, (cudaStream_t)stream);
  PTB_DISPATCH(dtype, (fo_bwd<S, true>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a,
                                       grad_zi, workspace, workspace_bytes, status, (cudaStream_t)stream)));
}

int ptb_lpv_recur_bwd_shared(int dtype, int64_t B, int64_t T, const void* a, const void* zi, int zi_batched,
                             const void* y, const void* gy, const void* g_in, void* grad_x, void* grad_a,
                             void* grad_zi, void* workspace, int64_t workspace_bytes, uint32_t* status,
                             ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!a || !gy || !grad_a || !y || !zi) return PTB_ERR_ARG;   // grad_x may be NULL (not wanted)
  if (dtype == PTB_C64 || dtype == PTB_C128)
    return cx_fo_bwd(dtype, 1, B, T, a, 0, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi, workspace,
                     workspace_bytes, status, (cudaStream_t)stream, 1);
  PTB_DISPATCH(dtype, (fo_bwd<S, true>(B, T, a, 0, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi, workspace,
                                       workspace_bytes, status, (cudaStream_t)stream, true)));
}

#define PTB_SO_DISPATCH(dtype, FN, ...)                                                      \
  switch (dtype) {                                                                          \
    case PTB_F32: return x_scalar ? FN<float, kLpv, true>(__VA_ARGS__) : FN<float, kLpv, false>(__VA_ARGS__);   \
    case PTB_F64: return x_scalar ? FN<double, kLpv, true>(__VA_ARGS__) : FN<double, kLpv, false>(__VA_ARGS__); \
    default: return PTB_ERR_ARG;                                                            \
  }

int ptb_lti_recur2_fwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* x, int x_scalar, void* y, void* zf, void* workspace,
                       int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !zi || !x || !y) return PTB_ERR_ARG;
  constexpr bool kLpv = false;
  PTB_SO_DISPATCH(dtype, so_fwd, B, T, A, A_batched, zi, x, y, zf, workspace, workspace_bytes, status,
                  (cudaStream_t)stream);
}

int ptb_lpv_recur2_fwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* x, int x_scalar, void* y, void* zf, void* workspace,
                       int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !zi || !x || !y) return PTB_ERR_ARG;
  constexpr bool kLpv = true;
  PTB_SO_DISPATCH(dtype, so_fwd, B, T, A, A_batched, zi, x, y, zf, workspace, workspace_bytes, status,
                  (cudaStream_t)stream);
}

int ptb_lti_recur2_bwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* y, const void* gy, const void* g_in, int x_scalar, void* grad_x,
                       void* grad_A, void* grad_zi, void* workspace, int64_t workspace_bytes,
                       uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !gy || !grad_x || (grad_A && (!y || !zi))) return PTB_ERR_ARG;
  constexpr bool kLpv = false;
  PTB_SO_DISPATCH(dtype, so_bwd, B, T, A, A_batched, zi, y, gy, g_in, grad_x, grad_A, grad_zi, workspace,
                  workspace_bytes, status, (cudaStream_t)stream);
}

int ptb_lpv_recur2_bwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* y, const void* gy, const void* g_in, int x_scalar, void* grad_x,
                       void* grad_A, void* grad_zi, void* workspace, int64_t workspace_bytes,
                       uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !gy || !grad_x || (grad_A && (!y || !zi))) return PTB_ERR_ARG;
  constexpr bool kLpv = true;
  PTB_SO_DISPATCH(dtype, so_bwd, B, T, A, A_batched, zi, y, gy, g_in, grad_x, grad_A, grad_zi, workspace,
                  workspace_bytes, status, (cudaStream_t)stream);
}

int64_t ptb_lpv_recur2_carry_chunks(int dtype, int64_t T) {
  if (T < 0) return -1;
  switch (dtype) {
    case PTB_F32: return (T + SoSmallSel<float>::C::TILE - 1) / SoSmallSel<float>::C::TILE;
    case PTB_F64: return (T + SoSmallSel<double>::C::TILE - 1) / SoSmallSel<double>::C::TILE;
    default: return -1;
  }
}

int ptb_lpv_recur2_zero_carry(int dtype, int64_t B, int64_t T, const void* A, const void* x, int x_scalar, void* y,
                              void* tile_prod, void* end_state, void* workspace, int64_t workspace_bytes,
                              uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !x || !y || !tile_prod || !end_state) return PTB_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case PTB_F32:
      return x_scalar ? so_small_fwd<float, true>(B, T, A, 1, nullptr, x, y, end_state, workspace, workspace_bytes,
                                                  status, st, tile_prod)
                      : so_small_fwd<float, false>(B, T, A, 1, nullptr, x, y, end_state, workspace, workspace_bytes,
                                                   status, st, tile_prod);
    case PTB_F64:
      return x_scalar ? so_small_fwd<double, true>(B, T, A, 1, nullptr, x, y, end_state, workspace, workspace_bytes,
                                                   status, st, tile_prod)
                      : so_small_fwd<double, false>(B, T, A, 1, nullptr, x, y, end_state, workspace, workspace_bytes,
                                                    status, st, tile_prod);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur2_bwd_shared(int dtype, int64_t B, int64_t T, const void* A, const void* zi, const void* y,
                              const void* gy, const void* g_in, int x_scalar, void* grad_x, void* grad_A,
                              void* grad_zi, void* workspace, int64_t workspace_bytes, uint32_t* status,
                              ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !gy || !grad_x || !grad_A || !y || !zi) return PTB_ERR_ARG;
  constexpr bool kLpv = true;
  PTB_SO_DISPATCH(dtype, so_bwd, B, T, A, 0, zi, y, gy, g_in, grad_x, grad_A, grad_zi, workspace, workspace_bytes,
                  status, (cudaStream_t)stream, true);
}

int ptb_biquad_tdf2_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* zi, const void* x, void* y, void* zf, void* workspace,
                        int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!b || !a || !x || !y) return PTB_ERR_ARG;
  if (g_bq_policy != 1) {   // the kernels whose matrix powers come from a table built in double
    const int rc = biquad_table_fwd(dtype, B, T, b, a, coef_batched, zi, x, y, zf, workspace, workspace_bytes, status,
                                    (cudaStream_t)stream);
    if (rc >= 0) return rc;
  }
  PTB_DISPATCH(dtype, (bq_fwd<S>(B, T, b, a, coef_batched, zi, x, y, zf, workspace, workspace_bytes, status,
                                 (cudaStream_t)stream)));
}

int ptb_biquad_tdf2_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* x, const void* y, const void* gy, const void* g_zf, void* grad_x,
                        void* grad_b, void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                        uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!b || !a || !gy || !grad_x || ((grad_b || grad_a) && (!x || !y))) return PTB_ERR_ARG;
  {   // large batches: the chained kernel of capi_sos.cu (measured faster for the backward pass only)
    const int rc = biquad_chain_bwd(dtype, B, T, b, a, coef_batched, x, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi,
                                    workspace, workspace_bytes, status, (cudaStream_t)stream);
    if (rc >= 0) return rc;
  }
  if (g_bq_policy != 1) {
    const int rc = biquad_table_bwd(dtype, B, T, b, a, coef_batched, x, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi,
                                    workspace, workspace_bytes, status, (cudaStream_t)stream);
    if (rc >= 0) return rc;
  }
  PTB_DISPATCH(dtype, (bq_bwd<S>(B, T, b, a, coef_batched, x, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi,
                                 workspace, workspace_bytes, status, (cudaStream_t)stream)));
}

}  // extern "C"
