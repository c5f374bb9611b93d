// C ABI of the fused time-varying second-order filter (see include/philtorch_b200.h).
#include "launch.cuh"

#include "lpv_biquad.cuh"

namespace ptb {

// (samples per thread, threads per CTA, CTAs per SM)
template <class S> struct LpvSel;
template <> struct LpvSel<float> { using F = LpvBqCfg<float, 15, 64, 6>; using B = LpvBqCfg<float, 15, 64, 6>; };
template <> struct LpvSel<double> { using F = LpvBqCfg<double, 7, 64, 6>; using B = LpvBqCfg<double, 7, 64, 6>; };

template <class S>
static int64_t lpv_ws_bytes(int64_t B, int64_t T) {
  const int64_t nf = B * ((T + LpvSel<S>::F::TILE - 1) / LpvSel<S>::F::TILE);
  const int64_t nb = B * ((T + LpvSel<S>::B::TILE - 1) / LpvSel<S>::B::TILE);
  return std::max(ws_layout(nf, LpvSel<S>::F::SLOT_WORDS, 0).total, ws_layout(nb, LpvSel<S>::B::SLOT_WORDS, 0).total);
}

template <class C, class K, class P>
static int launch_chained(K kernel, int smem, const P& p, int64_t B, int64_t T, void* ws, int64_t wsb, uint32_t* status,
                          bool bulk, cudaStream_t st, bool* attr_set) {
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
  int dev = 0, sms = 0, occ = 1;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!attr_set[dev]) {
      PTB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr_set[dev] = true;
    }
  }
  PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, C::NT, smem));
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, (int64_t)sms * std::max(occ, 1));
  kernel<<<grid, C::NT, smem, st>>>(p, wk, (uint32_t)B, (uint32_t)nchunks, (uint32_t)ntiles, bulk ? 1 : 0, g_wait_ns);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S, bool TDF2>
static int lpv_fwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* zi, const void* x,
                   void* y, void* hp, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using C = typename LpvSel<S>::F;
  using L = LpvBqFwdSmem<C>;
  LpvBqFwdParams<S> p;
  p.a = static_cast<const S*>(a); p.a_row = coef_batched ? 2 * T : 0;
  p.b = static_cast<const S*>(b); p.b_row = coef_batched ? 3 * T : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.hp = static_cast<S*>(hp);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  const bool bulk = aligned16(a) && aligned16(b) && aligned16(x) && aligned16(y) && (!hp || aligned16(hp)) &&
                    (T * sizeof(S)) % 16 == 0;
  static bool attr_set[kMaxDevices] = {};
  return launch_chained<C>(lpv_bq_fwd_kernel<S, C, TDF2>, L::kTotal, p, B, T, ws, wsb, status, bulk, st, attr_set);
}

template <class S, bool TDF2>
static int lpv_bwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x, const void* hp,
                   const void* gy, const void* g_zf, void* grad_x, void* grad_b, void* grad_a, void* grad_zi, void* ws,
                   int64_t wsb, uint32_t* status, cudaStream_t st) {
  using C = typename LpvSel<S>::B;
  using L = LpvBqBwdSmem<C>;
  LpvBqBwdParams<S> p;
  p.a = static_cast<const S*>(a); p.a_row = coef_batched ? 2 * T : 0;
  p.b = static_cast<const S*>(b); p.b_row = coef_batched ? 3 * T : 0;
  p.x = static_cast<const S*>(x);
  p.hp = static_cast<const S*>(hp);
  p.gy = static_cast<const S*>(gy);
  p.g_in = static_cast<const S*>(g_zf);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_a = static_cast<S*>(grad_a);
  p.grad_b = static_cast<S*>(grad_b);
  p.grad_zi = static_cast<S*>(grad_zi);
  p.T = T;
  const bool bulk = aligned16(a) && aligned16(b) && aligned16(x) && aligned16(hp) && aligned16(gy) &&
                    aligned16(grad_x) && aligned16(grad_a) && aligned16(grad_b) && (T * sizeof(S)) % 16 == 0;
  static bool attr_set[kMaxDevices] = {};
  return launch_chained<C>(lpv_bq_bwd_kernel<S, C, TDF2>, L::kTotal, p, B, T, ws, wsb, status, bulk, st, attr_set);
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int64_t ptb_lpv_biquad_workspace_bytes(int dtype, int64_t B, int64_t T) {
  if (B <= 0 || T <= 0) return 0;
  if (dtype == PTB_F32) return lpv_ws_bytes<float>(B, T);
  if (dtype == PTB_F64) return lpv_ws_bytes<double>(B, T);
  return 0;
}

int ptb_lpv_biquad_df2_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* zi, const void* x, void* y, void* hp, void* zf, void* workspace,
                           int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B <= 0 || T <= 0 || !b || !a || !x || !y) return PTB_ERR_ARG;
  if (dtype == PTB_F32)
    return lpv_fwd<float, false>(B, T, b, a, coef_batched, zi, x, y, hp, zf, workspace, workspace_bytes, status,
                          (cudaStream_t)stream);
  if (dtype == PTB_F64)
    return lpv_fwd<double, false>(B, T, b, a, coef_batched, zi, x, y, hp, zf, workspace, workspace_bytes, status,
                           (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

int ptb_lpv_biquad_df2_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* x, const void* hp, const void* gy, const void* g_zf, void* grad_x,
                           void* grad_b, void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                           uint32_t* status, ptb_stream_t stream) {
  if (B <= 0 || T <= 0 || !b || !a || !x || !hp || !gy || !grad_x || !grad_b || !grad_a) return PTB_ERR_ARG;
  if (dtype == PTB_F32)
    return lpv_bwd<float, false>(B, T, b, a, coef_batched, x, hp, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, workspace,
                          workspace_bytes, status, (cudaStream_t)stream);
  if (dtype == PTB_F64)
    return lpv_bwd<double, false>(B, T, b, a, coef_batched, x, hp, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, workspace,
                           workspace_bytes, status, (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

int ptb_lpv_biquad_tdf2_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* zi, const void* x, void* y, void* hp, void* zf, void* workspace,
                           int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B <= 0 || T <= 0 || !b || !a || !x || !y) return PTB_ERR_ARG;
  if (dtype == PTB_F32)
    return lpv_fwd<float, true>(B, T, b, a, coef_batched, zi, x, y, hp, zf, workspace, workspace_bytes, status,
                          (cudaStream_t)stream);
  if (dtype == PTB_F64)
    return lpv_fwd<double, true>(B, T, b, a, coef_batched, zi, x, y, hp, zf, workspace, workspace_bytes, status,
                           (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

int ptb_lpv_biquad_tdf2_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* x, const void* hp, const void* gy, const void* g_zf, void* grad_x,
                           void* grad_b, void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                           uint32_t* status, ptb_stream_t stream) {
  if (B <= 0 || T <= 0 || !b || !a || !x || !hp || !gy || !grad_x || !grad_b || !grad_a) return PTB_ERR_ARG;
  if (dtype == PTB_F32)
    return lpv_bwd<float, true>(B, T, b, a, coef_batched, x, hp, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, workspace,
                          workspace_bytes, status, (cudaStream_t)stream);
  if (dtype == PTB_F64)
    return lpv_bwd<double, true>(B, T, b, a, coef_batched, x, hp, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, workspace,
                           workspace_bytes, status, (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

}  // extern "C"
