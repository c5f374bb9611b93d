// C ABI of the comb-filter kernels (see include/philtorch_b200.h).
#include "launch.cuh"

#include "comb.cuh"
#include "comb_slab.cuh"

namespace ptb {

static int comb_blocks_per_row(int64_t D) { return (int)((D + 31) / 32); }   // a block of the lane kernels: 32 phases

// 0: slab kernels where the layout allows and they are expected to pay, 1: lane-per-phase kernels
// only, 2 / 3 / 4: slab kernels with bands of 256 / 128 / 64 phases wherever the layout allows (tests, tuning)
static int g_comb_policy = 0;
static int g_comb_max_stages = 4;   // deepest ring of the slab kernels (3 .. kCombMaxStages)

// steps per slab; the adjoint stages two slabs per step range
#ifndef PTB_COMB_KS_FWD
#define PTB_COMB_KS_FWD 64   // steps per slab (float32; halved for float64): 16-64 KB per tiled copy
#define PTB_COMB_KS_BWD 32
#endif
template <class S, int W, bool BWD> struct CombSlabSel {
  static constexpr int KS = (BWD ? PTB_COMB_KS_BWD : PTB_COMB_KS_FWD) / (int)(sizeof(S) / 4);
  using C = CombSlabCfg<S, W, KS>;
};

template <class S>
static bool comb_slab_ok(int64_t N, int64_t D, std::initializer_list<const void*> arrays) {
  constexpr int64_t V = 16 / (int64_t)sizeof(S);
  if (N % V != 0 || D % V != 0) return false;
  for (const void* q : arrays)
    if (q && !aligned16(q)) return false;
  return true;
}

constexpr int64_t kSmemPerSm = 228 * 1024, kSmemPerCtaMax = 227 * 1024, kSmemCtaOverhead = 1024;

// ---- tensor maps: (phase, step, row) view of a (B, N) signal, box W x KS x 1 ------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  std::lock_guard<std::mutex> init_lock(init_mutex());
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

template <class S>
static bool comb_tensor_map(CUtensorMap* map, const void* base, int64_t B, int64_t N, int64_t D, int64_t K, int W,
                            int KS) {
  const EncodeTiledFn enc = tensor_map_encoder();
  if (!enc || K < 1 || B < 1 || D > 0x7FFFFFFFll || K > 0x7FFFFFFFll || B > 0x7FFFFFFFll) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)K, (cuuint64_t)B};
  const cuuint64_t strides[2] = {(cuuint64_t)D * sizeof(S), (cuuint64_t)N * sizeof(S)};   // bytes, multiples of 16
  if (strides[0] >= (1ull << 40) || strides[1] >= (1ull << 40)) return false;
  const cuuint32_t box[3] = {(cuuint32_t)W, (cuuint32_t)KS, 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r = enc(map, sizeof(S) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 3,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

constexpr int kCombNoTensorMap = -1;   // the tensor maps could not be encoded: the caller uses the other kernels

struct CombPlan {
  int width = 0, stages = 0;
  int64_t ctas = 0;
};

static int comb_sm_count() {
  static int cached[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> init_lock(init_mutex());
  if (!cached[dev]) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    cached[dev] = sms;
  }
  return cached[dev];
}

template <class S, int W, bool BWD>
struct CombSlabLaunch {
  using C = typename CombSlabSel<S, W, BWD>::C;
  // ring depth: what this CTA's share of an SM's shared memory holds, 3 .. g_comb_max_stages (measured:
  // beyond four stages nothing is gained; the slab height matters, 32-64 KB per copy)
  static CombPlan plan(int64_t B, int64_t D) {
    const int64_t sms = comb_sm_count();
    CombPlan pl;
    pl.ctas = B * ((D + W - 1) / W);
    const int64_t per_sm = std::max<int64_t>(1, (pl.ctas + sms - 1) / sms);
    const int64_t slab = (int64_t)(BWD ? 2 : 1) * C::SLAB * (int64_t)sizeof(S);
    const int64_t most = (kSmemPerCtaMax - kCombSlabHeader) / slab;   // deepest ring one CTA can hold
    if (most < 3) return pl;                                          // this band width does not fit: width 0
    const int64_t fit = (std::min(kSmemPerSm / per_sm - kSmemCtaOverhead, kSmemPerCtaMax) - kCombSlabHeader) / slab;
    pl.width = W;
    pl.stages = (int)std::max<int64_t>(3, std::min<int64_t>(std::min<int64_t>(fit, most), g_comb_max_stages));
    return pl;
  }
  static int run(CombSlabParams<S> p, int64_t B, int stages, cudaStream_t st) {
    static int attr_bytes[kMaxDevices] = {};
    int dev = 0;
    PTB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
    const int smem = C::bytes(stages, BWD);
    {
      std::lock_guard<std::mutex> init_lock(init_mutex());
      if (attr_bytes[dev] < smem) {   // the attribute is the largest ring used so far
        const int top = C::bytes(kCombMaxStages, BWD) <= kSmemPerCtaMax ? C::bytes(kCombMaxStages, BWD) : (int)kSmemPerCtaMax;
        if (BWD) PTB_CUDA(cudaFuncSetAttribute(comb_slab_bwd_kernel<S, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, top));
        else PTB_CUDA(cudaFuncSetAttribute(comb_slab_fwd_kernel<S, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, top));
        attr_bytes[dev] = top;
      }
    }
    p.bands = (int)((p.D + W - 1) / W);
    p.stages = stages;
    const unsigned grid = (unsigned)(B * p.bands);
    const int64_t K = p.N / p.D;
    alignas(64) CUtensorMap m0, m1, m2;
    if (BWD) {
      if (!comb_tensor_map<S>(&m0, p.gy, B, p.N, p.D, K, W, C::KS) ||
          !comb_tensor_map<S>(&m1, p.yfwd ? static_cast<const void*>(p.yfwd) : static_cast<const void*>(p.gy), B, p.N,
                              p.D, K, W, C::KS) ||
          !comb_tensor_map<S>(&m2, p.grad_x, B, p.N, p.D, K, W, C::KS))
        return kCombNoTensorMap;
      comb_slab_bwd_kernel<S, C><<<grid, W, smem, st>>>(m0, m1, m2, p);
    } else {
      if (!comb_tensor_map<S>(&m0, p.x, B, p.N, p.D, K, W, C::KS) ||
          !comb_tensor_map<S>(&m1, p.y, B, p.N, p.D, K, W, C::KS))
        return kCombNoTensorMap;
      comb_slab_fwd_kernel<S, C><<<grid, W, smem, st>>>(m0, m1, p);
    }
    PTB_CUDA(cudaGetLastError());
    return PTB_OK;
  }
};

// Band width and ring depth for this problem (width 0: use the lane-per-phase kernels).  The widest
// band that still puts a CTA on most SMs: measured at delay 1000, T = 2^22, fwd+bwd, 64 rows: 0.90 ms
// with 256 phases per band, 0.94 with 128, 1.02 with 64 (1.28 lane per phase); 16 rows: 0.35 / 0.27 /
// 0.28 ms (0.46).
template <class S, bool BWD>
static CombPlan comb_plan(int64_t B, int64_t N, int64_t D) {
  const CombPlan p256 = CombSlabLaunch<S, 256, BWD>::plan(B, D), p128 = CombSlabLaunch<S, 128, BWD>::plan(B, D),
                 p64 = CombSlabLaunch<S, 64, BWD>::plan(B, D);
  CombPlan none;
  if (N / D < 1) return none;   // no full step: nothing for a tensor of steps to describe
  if (g_comb_policy == 2) return p256;
  if (g_comb_policy == 3) return p128;
  if (g_comb_policy == 4) return p64;
  if (N / D < 64 || D < 64) return none;   // a few steps or a few phases: the slabs would be mostly padding
  const int64_t enough = (int64_t)(0.8 * comb_sm_count());
  if (p256.width && D > 128 && p256.ctas >= enough) return p256;
  if (p128.width && D > 64 && p128.ctas >= enough) return p128;
  return p64;
}

template <class S, bool BWD>
static int comb_slab_run(const CombPlan& pl, const CombSlabParams<S>& p, int64_t B, cudaStream_t st) {
  switch (pl.width) {
    case 256: return CombSlabLaunch<S, 256, BWD>::run(p, B, pl.stages, st);
    case 128: return CombSlabLaunch<S, 128, BWD>::run(p, B, pl.stages, st);
    default: return CombSlabLaunch<S, 64, BWD>::run(p, B, pl.stages, st);
  }
}

template <class S>
static int comb_fwd(int64_t B, int64_t N, int64_t D, const void* a, int a_batched, const void* zi, int zi_mode,
                    const void* x, void* y, uint32_t* status, cudaStream_t st) {
  CombPlan pl;
  if (g_comb_policy != 1 && comb_slab_ok<S>(N, D, {x, y})) pl = comb_plan<S, false>(B, N, D);
  if (pl.width) {
    CombSlabParams<S> p{};
    p.a = static_cast<const S*>(a); p.a_stride = a_batched ? 1 : 0;
    p.zi = static_cast<const S*>(zi); p.zi_mode = zi_mode;
    p.N = N; p.D = D; p.status = status; p.wait_ns = g_wait_ns;
    p.x = static_cast<const S*>(x); p.y = static_cast<S*>(y);
    const int rc = comb_slab_run<S, false>(pl, p, B, st);
    if (rc != kCombNoTensorMap) return rc;
  }
  const int bpr = comb_blocks_per_row(D);
  comb_fwd_kernel<S><<<(unsigned)(B * bpr), kCombThreads, 0, st>>>(
      static_cast<const S*>(x), static_cast<const S*>(a), a_batched ? 1 : 0, static_cast<const S*>(zi), zi_mode,
      static_cast<S*>(y), N, D, bpr);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int comb_bwd(int64_t B, int64_t N, int64_t D, const void* a, int a_batched, const void* zi, int zi_mode,
                    const void* y, const void* gy, void* grad_x, void* partial, void* grad_state, uint32_t* status,
                    cudaStream_t st) {
  CombPlan pl;
  if (g_comb_policy != 1 && comb_slab_ok<S>(N, D, {gy, y, grad_x})) pl = comb_plan<S, true>(B, N, D);
  if (pl.width) {
    CombSlabParams<S> p{};
    p.a = static_cast<const S*>(a); p.a_stride = a_batched ? 1 : 0;
    p.zi = static_cast<const S*>(zi); p.zi_mode = zi_mode;
    p.N = N; p.D = D; p.status = status; p.wait_ns = g_wait_ns;
    p.gy = static_cast<const S*>(gy); p.yfwd = static_cast<const S*>(y); p.grad_x = static_cast<S*>(grad_x);
    p.partial = static_cast<S*>(partial); p.partial_stride = comb_blocks_per_row(D);
    p.grad_state = static_cast<S*>(grad_state);
    const int rc = comb_slab_run<S, true>(pl, p, B, st);
    if (rc != kCombNoTensorMap) return rc;
  }
  const int bpr = comb_blocks_per_row(D);
  comb_bwd_kernel<S><<<(unsigned)(B * bpr), kCombThreads, 0, st>>>(
      static_cast<const S*>(gy), static_cast<const S*>(y), static_cast<const S*>(a), a_batched ? 1 : 0,
      static_cast<const S*>(zi), zi_mode, static_cast<S*>(grad_x), static_cast<S*>(partial),
      static_cast<S*>(grad_state), N, D, bpr);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int ptb_comb_set_policy(int policy) {
  const int family = policy & 0xFF, depth = policy >> 8;   // bits 8..: deepest ring of the slab kernels (0: default)
  if (policy < 0 || family > 4 || (depth != 0 && (depth < 3 || depth > kCombMaxStages))) return PTB_ERR_ARG;
  g_comb_policy = family;
  g_comb_max_stages = depth ? depth : 4;
  return PTB_OK;
}

int64_t ptb_comb_partial_blocks(int64_t delay) { return delay > 0 ? comb_blocks_per_row(delay) : 0; }

int ptb_comb_fwd(int dtype, int64_t B, int64_t N, int64_t delay, const void* a, int a_batched, const void* zi,
                 int zi_mode, const void* x, void* y, void* workspace, int64_t workspace_bytes, uint32_t* status,
                 ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes;
  if (B < 0 || N < 0 || delay < 1 || zi_mode < 0 || zi_mode > 2) return PTB_ERR_ARG;
  if (B == 0 || N == 0) return PTB_OK;
  if (!a || !x || !y || (zi_mode && !zi)) return PTB_ERR_ARG;
  if (B * (int64_t)comb_blocks_per_row(delay) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_F32: return comb_fwd<float>(B, N, delay, a, a_batched, zi, zi_mode, x, y, status, (cudaStream_t)stream);
    case PTB_F64: return comb_fwd<double>(B, N, delay, a, a_batched, zi, zi_mode, x, y, status, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_comb_bwd(int dtype, int64_t B, int64_t N, int64_t delay, const void* a, int a_batched, const void* zi,
                 int zi_mode, const void* y, const void* gy, void* grad_x, void* partial, void* grad_state,
                 void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes;
  if (B < 0 || N < 0 || delay < 1 || zi_mode < 0 || zi_mode > 2) return PTB_ERR_ARG;
  if (B == 0 || N == 0) return PTB_OK;
  if (!a || !gy || !grad_x || (partial && !y) || (partial && zi_mode && !zi)) return PTB_ERR_ARG;
  if (B * (int64_t)comb_blocks_per_row(delay) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_F32:
      return comb_bwd<float>(B, N, delay, a, a_batched, zi, zi_mode, y, gy, grad_x, partial, grad_state, status,
                             (cudaStream_t)stream);
    case PTB_F64:
      return comb_bwd<double>(B, N, delay, a, a_batched, zi, zi_mode, y, gy, grad_x, partial, grad_state, status,
                              (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

}  // extern "C"
