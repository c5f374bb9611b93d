// Host side of the first-order kernels: tile geometry and launch wrappers, shared by the real
// (capi.cu) and complex (capi_cx.cu) instantiations.
#pragma once
#include "launch.cuh"

#include "first_order.cuh"

namespace ptb {

// a scalar as N reals (the per-tile partial sums of grad_a are reduced component-wise)
template <class S> struct RealOf { using R = S; static constexpr int N = 1; };
template <class R_> struct RealOf<Cx<R_>> { using R = R_; static constexpr int N = 2; };

// ---------------------------------------------------------------------------- first order
// Tile geometry: an ODD number of 16-byte units per thread and array (bank-conflict-free strided
// access), large tiles (tens of KB per bulk copy are the most DRAM-efficient), one CTA per SM with
// 2-4 stages filling its shared memory.
// (16-byte units per thread and array, stages, CTAs per SM); overridable for tuning experiments
#ifndef PTB_FO_FWD_CH
#define PTB_FO_FWD_CH 9
#define PTB_FO_FWD_STAGES 3
#define PTB_FO_FWD_CTAS 1
#endif
#ifndef PTB_FO_LBW
#define PTB_FO_LBW 1   // look-back warps per CTA: 1, or one per stage
#endif
#ifndef PTB_FO_BWD_CH
#define PTB_FO_BWD_CH 5
#define PTB_FO_BWD_STAGES 3
#define PTB_FO_BWD_CTAS 1
#endif
// time-invariant variants stage fewer arrays per tile: larger tiles / more stages fill shared memory
#ifndef PTB_FOLTI_FWD_CH
#define PTB_FOLTI_FWD_CH 13
#define PTB_FOLTI_FWD_STAGES 4
#define PTB_FOLTI_FWD_CTAS 1
#endif
#ifndef PTB_FOLTI_BWD_CH
#define PTB_FOLTI_BWD_CH 9
#define PTB_FOLTI_BWD_STAGES 3
#define PTB_FOLTI_BWD_CTAS 1
#endif
// the reverse pass fused with its combination stages two inputs per tile and writes over one of them
#ifndef PTB_FOFUSE_CH
#define PTB_FOFUSE_CH PTB_FOLTI_BWD_CH
#define PTB_FOFUSE_STAGES PTB_FOLTI_BWD_STAGES
#endif
template <class S, bool LPV, class G = S> struct FoFwdSel { using type = FoFwd<S, PTB_FO_FWD_CH, PTB_FO_FWD_STAGES, PTB_FO_FWD_CTAS, 1, true>; };
template <class S> struct FoFwdSel<S, false, S> { using type = FoFwd<S, PTB_FOLTI_FWD_CH, PTB_FOLTI_FWD_STAGES, PTB_FOLTI_FWD_CTAS, 1, false>; };
template <class S, bool LPV, class G = S> struct FoBwdSel { using type = FoBwd<S, PTB_FO_BWD_CH, PTB_FO_BWD_STAGES, PTB_FO_BWD_CTAS, 1, true>; };
template <class S> struct FoBwdSel<S, false, S> { using type = FoBwd<S, PTB_FOLTI_BWD_CH, PTB_FOLTI_BWD_STAGES, PTB_FOLTI_BWD_CTAS, 1, false>; };
// 2-byte storage (float16 / bfloat16 arrays, float32 arithmetic): a 16-byte unit holds 8 samples, so
// fewer units per thread keep the register count of the fp32 kernels
#ifndef PTB_FOH_FWD_CH
#define PTB_FOH_FWD_CH 7       // 14336-sample tiles, 28 KB per array (5 units: 0.307 ms, 7 units: 0.267 ms at B=256, T=2^20)
#define PTB_FOH_FWD_STAGES 3
#define PTB_FOH_BWD_CH 5       // 10240-sample tiles, 20 KB per array (3 units: 0.481 ms, 5 units: 0.404 ms)
#define PTB_FOH_BWD_STAGES 3
#endif
// time-invariant coefficients: one staged array less per tile (forward, B=256, T=2^20, float16: 9 units x 3
// stages 0.227 ms, 13 x 3 0.201 ms, 15 x 3 0.198 ms, 17 x 3 0.199 ms; backward: 9 x 3 no better than 7 x 3)
#ifndef PTB_FOH_LTI_FWD_CH
#define PTB_FOH_LTI_FWD_CH 15
#define PTB_FOH_LTI_FWD_STAGES 3
#define PTB_FOH_LTI_BWD_CH (PTB_FOH_BWD_CH + 2)
#define PTB_FOH_LTI_BWD_STAGES PTB_FOH_BWD_STAGES
#endif
template <bool LPV> struct FoFwdSel<float, LPV, __half> { using type = FoFwd<float, LPV ? PTB_FOH_FWD_CH : PTB_FOH_LTI_FWD_CH, LPV ? PTB_FOH_FWD_STAGES : PTB_FOH_LTI_FWD_STAGES, 1, 1, LPV, __half>; };
template <bool LPV> struct FoFwdSel<float, LPV, __nv_bfloat16> { using type = FoFwd<float, LPV ? PTB_FOH_FWD_CH : PTB_FOH_LTI_FWD_CH, LPV ? PTB_FOH_FWD_STAGES : PTB_FOH_LTI_FWD_STAGES, 1, 1, LPV, __nv_bfloat16>; };
template <bool LPV> struct FoBwdSel<float, LPV, __half> { using type = FoBwd<float, LPV ? PTB_FOH_BWD_CH : PTB_FOH_LTI_BWD_CH, LPV ? PTB_FOH_BWD_STAGES : PTB_FOH_LTI_BWD_STAGES, 1, 1, LPV, false, __half>; };
template <bool LPV> struct FoBwdSel<float, LPV, __nv_bfloat16> { using type = FoBwd<float, LPV ? PTB_FOH_BWD_CH : PTB_FOH_LTI_BWD_CH, LPV ? PTB_FOH_BWD_STAGES : PTB_FOH_LTI_BWD_STAGES, 1, 1, LPV, false, __nv_bfloat16>; };
template <class S, bool LPV, class G = S> using FoFwdP = typename FoFwdSel<S, LPV, G>::type;
template <class S, bool LPV, class G = S> using FoBwdP = typename FoBwdSel<S, LPV, G>::type;

constexpr int64_t kFusedReduceMaxTiles = 2048;   // beyond this one warp would take longer than a second launch

// write-out of the per-row sums of a time-invariant gradient in the storage type
template <class S, int N, class G>
struct StoreSumsAs {
  G* out;
  __device__ void operator()(int64_t row, const double* acc) const {
    for (int i = 0; i < N; ++i) out[row * N + i] = Cvt<S, G>::out((S)acc[i]);
  }
};

template <class S, bool LPV, class G = S>
static int fo_fwd(int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
                  const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = FoFwdP<S, LPV, G>;
  typename P::Params p;
  p.a = static_cast<const G*>(a);
  p.a_row_stride = a_batched ? (LPV ? T : 1) : 0;
  p.zi = static_cast<const G*>(zi);
  p.zi_stride = zi_batched ? 1 : 0;
  p.x = static_cast<const G*>(x);
  p.y = static_cast<G*>(y);
  p.zf = static_cast<G*>(zf);
  p.T = T;
  const bool bulk = aligned16(x) && aligned16(y) && (!LPV || aligned16(a)) && (T * sizeof(G)) % 16 == 0;
  // the plain-load path copies 32-bit words: arrays of 2-byte samples must qualify for bulk copies
  if (!bulk && sizeof(G) < 4) return PTB_ERR_ARG;
  return launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

// ga_shared (per-sample coefficients only): grad_a is ONE (T,) array that every row adds its tile
// into (TMA reduce copies); needs the bulk path and 4- or 8-byte scalars, else PTB_ERR_ARG.
template <class S, bool LPV, class G = S>
static int fo_bwd(int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
                  const void* y, const void* gy, const void* g_in, void* grad_x, void* grad_a, void* grad_zi,
                  void* ws, int64_t wsb, uint32_t* status, cudaStream_t st, bool ga_shared = false) {
  using P = FoBwdP<S, LPV, G>;
  typename P::Params p;
  p.a = static_cast<const G*>(a);
  p.a_row_stride = a_batched ? (LPV ? T : 1) : 0;
  p.zi = static_cast<const G*>(zi);
  p.zi_stride = zi_batched ? 1 : 0;
  p.y = static_cast<const G*>(y);
  p.gy = static_cast<const G*>(gy);
  p.g_in = static_cast<const G*>(g_in);
  p.grad_x = static_cast<G*>(grad_x);
  p.grad_a = LPV ? static_cast<G*>(grad_a) : nullptr;
  p.grad_zi = static_cast<G*>(grad_zi);
  p.T = T;
  p.want_ga = grad_a != nullptr;
  p.ga_row_stride = ga_shared ? 0 : T;
  const bool bulk = aligned16(gy) && (!grad_x || aligned16(grad_x)) && (!LPV || aligned16(a)) &&
                    (!p.want_ga || (aligned16(y) && (!LPV || aligned16(grad_a)))) &&
                    (T * sizeof(G)) % 16 == 0;
  if (!bulk && sizeof(G) < 4) return PTB_ERR_ARG;
  if (ga_shared && (!LPV || !bulk || sizeof(G) < 4)) return PTB_ERR_ARG;
  // small launches: the kernel's last warp reduces the per-tile sums of grad_a itself
  bool fused = false;
  if constexpr (!LPV && std::is_arithmetic<S>::value) {
    if (grad_a && B * ((T + P::TILE - 1) / P::TILE) <= kFusedReduceMaxTiles) {
      p.ga_out = static_cast<G*>(grad_a);
      p.ga_batched = a_batched ? 1 : 0;
      p.fuse_reduce = 1;
      fused = true;
    }
  }
  void* partial = nullptr;
  int64_t nchunks = 0;
  int rc = launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, &partial, &nchunks);
  if (rc != PTB_OK) return rc;
  if (!LPV && grad_a && !fused) {
    if constexpr (std::is_same<S, G>::value) {
      rc = launch_reduce<typename RealOf<S>::R, RealOf<S>::N>(
          partial, B, nchunks, a_batched,
          StoreSums<typename RealOf<S>::R, RealOf<S>::N>{static_cast<typename RealOf<S>::R*>(grad_a)}, st);
    } else {
      rc = launch_reduce<S, 1>(partial, B, nchunks, a_batched, StoreSumsAs<S, 1, G>{static_cast<G*>(grad_a)}, st);
    }
  }
  return rc;
}

// Reverse-time time-invariant recurrence fused with the combination out = scale * (g + second - x),
// g[t] = x[t] + a g[t+1]  (g beyond the end: g_in / a, i.e. g[T-1] = x[T-1] + g_in).
template <class S>
static int fo_reverse_fused(int64_t B, int64_t T, const void* a, int a_batched, const void* x, const void* second,
                            const void* g_in, double scale, void* out, void* first_state, void* ws, int64_t wsb,
                            uint32_t* status, cudaStream_t st) {
  using P = FoBwd<S, PTB_FOFUSE_CH, PTB_FOFUSE_STAGES, PTB_FOLTI_BWD_CTAS, 1, false, true>;
  typename P::Params p;
  p.a = static_cast<const S*>(a);
  p.a_row_stride = a_batched ? 1 : 0;
  p.zi = nullptr;
  p.zi_stride = 0;
  p.y = static_cast<const S*>(second);
  p.gy = static_cast<const S*>(x);
  p.g_in = static_cast<const S*>(g_in);
  p.grad_x = static_cast<S*>(out);
  p.grad_a = nullptr;
  p.grad_zi = static_cast<S*>(first_state);
  p.T = T;
  p.want_ga = 0;
  p.fuse_scale = (S)scale;
  const bool bulk = aligned16(x) && aligned16(out) && aligned16(second) && (T * sizeof(S)) % 16 == 0;
  return launch_scan<P>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

}  // namespace ptb
