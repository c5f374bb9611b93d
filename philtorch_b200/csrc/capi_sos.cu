// C ABI of the fused second-order-section cascade (see include/philtorch_b200.h).
#include "launch.cuh"

#include "sos_cascade.cuh"
#include "sos_chain.cuh"

namespace ptb {

// (16-byte units per thread and array, stages)
#ifndef PTB_SOS_FWD_CH
#define PTB_SOS_FWD_CH 9
#define PTB_SOS_FWD_STAGES 3
#define PTB_SOS_FWD_NT 256
#define PTB_SOS_FWD_CTAS 1
#endif
#ifndef PTB_SOS_BWD_CH
#define PTB_SOS_BWD_CH 9
#define PTB_SOS_BWD_STAGES 2
#define PTB_SOS_BWD_NT 256
#define PTB_SOS_BWD_CTAS 1
#endif
// a single section moves a third of the cascade's bytes per sample: larger tiles, two CTAs per SM
#ifndef PTB_SOS1_FWD_CH
#define PTB_SOS1_FWD_CH 13
#define PTB_SOS1_FWD_STAGES 2
#define PTB_SOS1_FWD_CTAS 2
#endif
template <class S, int K> struct SosFwdSel { using type = SosFwd<S, K, PTB_SOS_FWD_CH, PTB_SOS_FWD_STAGES, PTB_SOS_FWD_NT, PTB_SOS_FWD_CTAS>; };
template <class S> struct SosFwdSel<S, 1> { using type = SosFwd<S, 1, PTB_SOS1_FWD_CH, PTB_SOS1_FWD_STAGES, 256, PTB_SOS1_FWD_CTAS>; };
template <class S, int K> using SosFwdP = typename SosFwdSel<S, K>::type;
template <class S, int K> using SosBwdP = SosBwd<S, K, PTB_SOS_BWD_CH, PTB_SOS_BWD_STAGES, PTB_SOS_BWD_NT, PTB_SOS_BWD_CTAS>;

// chained kernels: (16-byte units per thread, threads, output buffers, CTAs per SM) per direction.
// Small CTAs, many per SM: inside a CTA the sections run in lock-step (a barrier per section), the
// overlap of one tile's scan latency with another tile's arithmetic comes from the other CTAs.
#ifndef PTB_CHAINF_CH
#define PTB_CHAINF_CH 9
#define PTB_CHAINF_NT 64
#define PTB_CHAINF_NOUT 1
#define PTB_CHAINF_MINB 8
#endif
#ifndef PTB_CHAINB_CH
#define PTB_CHAINB_CH 9
#define PTB_CHAINB_NT 64
#define PTB_CHAINB_MINB 5
#endif
template <class S, int K> using ChainF = ChainCfg<S, K, PTB_CHAINF_CH, PTB_CHAINF_NT, PTB_CHAINF_NOUT, PTB_CHAINF_MINB>;
template <class S, int K> using ChainB = ChainCfg<S, K, PTB_CHAINB_CH, PTB_CHAINB_NT, 1, PTB_CHAINB_MINB>;
// Few rows: a row keeps at most K + 1 tiles busy, so the CTAs that do run should be larger (measured,
// K = 6, T = 2^18, fwd+bwd: 64 rows 0.504 -> 0.436 ms, 32 rows 0.431 -> 0.354 ms, 128 rows 0.644 -> 0.624 ms)
template <class S, int K> using ChainFFew = ChainCfg<S, K, 9, 128, 1, 4>;
template <class S, int K> using ChainBFew = ChainCfg<S, K, 9, 128, 1, 3>;
static bool chain_few_rows(int64_t B, int sms) { return 10 * B < 11 * (int64_t)sms; }

// 0: pick by batch size, 1: always the decoupled kernels, 2: always the chained kernels
static int g_sos_mode = 0;

static int device_sms(int* sms) {
  static int cached[kMaxDevices] = {};
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return PTB_ERR_ARG;
  std::lock_guard<std::mutex> init_lock(init_mutex());
  if (!cached[dev]) PTB_CUDA(cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev));
  *sms = cached[dev];
  return PTB_OK;
}
// A row keeps at most K + 1 tiles busy in the chained kernels (staggered by one section), so they need
// enough rows to fill the GPU; measured on B200 (K = 6, with the few-row geometry) they win from about
// 32 rows on (32 rows x 2^18: 0.354 ms against 0.449 ms decoupled; 16 rows x 2^20: 0.834 against 0.668 ms).
static bool use_chain(int64_t B, int sms) { return g_sos_mode == 2 || (g_sos_mode == 0 && 6 * B >= (int64_t)sms); }

template <class S, int K, class CF, class CB>
static int64_t chain_ws_bytes_of(int64_t B, int64_t T) {
  const int64_t nf = B * ((T + CF::TILE - 1) / CF::TILE), nb = B * ((T + CB::TILE - 1) / CB::TILE);
  return std::max(align_up(B * CF::ROW * (int64_t)sizeof(S), 256) + ws_layout(nf, CF::SLOT_WORDS, 0).total,
                  align_up(B * CB::ROW * (int64_t)sizeof(S), 256) + ws_layout(nb, CB::SLOT_WORDS, 5 * K * sizeof(S)).total);
}
template <class S, int K>
static int64_t chain_ws_bytes(int64_t B, int64_t T) {
  return std::max(chain_ws_bytes_of<S, K, ChainF<S, K>, ChainB<S, K>>(B, T),
                  chain_ws_bytes_of<S, K, ChainFFew<S, K>, ChainBFew<S, K>>(B, T));
}

template <class S, int K, class C>
static int chain_fwd_cfg(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* zi,
                         const void* x, void* y, void* mid, void* zf, void* ws, int64_t wsb, uint32_t* status,
                         cudaStream_t st) {
  using L = ChainFwdSmem<C>;
  static_assert(L::kTotal <= 227 * 1024, "shared memory of an SM");
  const int64_t rows = coef_batched ? B : 1;
  const int64_t tb = align_up(rows * C::ROW * (int64_t)sizeof(S), 256);
  const int64_t nchunks = (T + C::TILE - 1) / C::TILE;
  const int64_t ntiles = B * nchunks;
  if (ntiles >= 0xFFFFFFFEll || B >= 0xFFFFFFFFll) return PTB_ERR_TOO_LARGE;
  const WsLayout l = ws_layout(ntiles, C::SLOT_WORDS, 0);
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < tb + l.total) return PTB_ERR_WORKSPACE;
  // one warp per block: a thread writes its ~150 table entries with a stride of a table row, and the
  // load/store units of few SMs serialised those (13.5 us with 128-thread blocks at 512 threads)
  chain_setup_kernel<S, C, false><<<(unsigned)((rows * K + 31) / 32), 32, 0, st>>>(
      static_cast<const S*>(b), rows * 3, coef_batched ? 3 : 0, static_cast<const S*>(a), rows * 2,
      coef_batched ? 2 : 0, static_cast<S*>(ws), rows);
  PTB_CUDA(cudaGetLastError());
  char* w = static_cast<char*>(ws) + tb;
  PTB_CUDA(cudaMemsetAsync(w, 0, (size_t)l.part_off, st));
  Workspace wk;
  wk.ticket = reinterpret_cast<uint32_t*>(w);
  wk.error = status ? status : reinterpret_cast<uint32_t*>(w + 4);
  wk.slots = reinterpret_cast<uint64_t*>(w + l.slots_off);
  wk.partial = nullptr;
  ChainFwdParams<S> p;
  p.tab = static_cast<const S*>(ws);
  p.tab_stride = coef_batched ? C::ROW : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.mid = static_cast<S*>(mid);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  p.B = B;
  const bool bulk = aligned16(x) && aligned16(y) && (!mid || aligned16(mid)) && (T * sizeof(S)) % 16 == 0;
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != PTB_OK) return rc;
  static bool attr_set[kMaxDevices] = {};
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!attr_set[dev]) {
      PTB_CUDA(cudaFuncSetAttribute(chain_fwd_kernel<S, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      attr_set[dev] = true;
    }
  }
  int occ = 1;
  PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, chain_fwd_kernel<S, C>, C::NT, L::kTotal));
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, (int64_t)sms * std::max(occ, 1));
  chain_fwd_kernel<S, C><<<grid, C::NT, L::kTotal, st>>>(p, wk, (uint32_t)B, (uint32_t)nchunks, (uint32_t)ntiles,
                                                         bulk ? 1 : 0, g_wait_ns);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S, int K>
static int chain_fwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* zi,
                     const void* x, void* y, void* mid, void* zf, void* ws, int64_t wsb, uint32_t* status,
                     cudaStream_t st) {
  int sms = 0;
  const int rc = device_sms(&sms);
  if (rc != PTB_OK) return rc;
  if (chain_few_rows(B, sms))
    return chain_fwd_cfg<S, K, ChainFFew<S, K>>(B, T, b, a, coef_batched, zi, x, y, mid, zf, ws, wsb, status, st);
  return chain_fwd_cfg<S, K, ChainF<S, K>>(B, T, b, a, coef_batched, zi, x, y, mid, zf, ws, wsb, status, st);
}

template <class S, int K> struct SosCoefGrads;

template <class S, int K>
static int chain_bwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                     const void* mid, const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b,
                     void* grad_a, void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st);

template <class S, int K>
static int64_t table_bytes(int64_t rows) { return align_up(rows * SosDims<K>::ROWTAB * (int64_t)sizeof(S), 256); }

template <class P>
static int64_t scan_ws_bytes(int64_t B, int64_t T) {
  const int64_t ntiles = B * ((T + P::TILE - 1) / P::TILE);
  return ws_layout(ntiles, P::SLOT_WORDS, sizeof(typename P::Partial)).total;
}

template <class S, int K>
static int64_t sos_ws_bytes(int64_t B, int64_t T) {
  return std::max(std::max(table_bytes<S, K>(B) + std::max(scan_ws_bytes<SosFwdP<S, K>>(B, T), scan_ws_bytes<SosBwdP<S, K>>(B, T)),
                           ptb_workspace_bytes(B, T)),
                  chain_ws_bytes<S, K>(B, T));
}

template <class S, int K, bool ADJ>
static int build_table(const void* b, const void* a, int coef_batched, int64_t B, void* tab, int spt,
                       cudaStream_t st) {
  const int64_t rows = coef_batched ? B : 1;
  const int threads = std::max(32, SosDims<K>::NS * SosDims<K>::NS);
  sos_setup_kernel<S, K, ADJ><<<(unsigned)rows, threads, 0, st>>>(
      static_cast<const S*>(b), rows * 3, coef_batched ? 3 : 0, static_cast<const S*>(a), rows * 2,
      coef_batched ? 2 : 0, static_cast<S*>(tab), spt);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S, int K>
static int sos_fwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* zi,
                   const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = SosFwdP<S, K>;
  const int64_t rows = coef_batched ? B : 1;
  const int64_t tb = table_bytes<S, K>(rows);
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < tb) return PTB_ERR_WORKSPACE;
  int rc = build_table<S, K, false>(b, a, coef_batched, B, ws, P::SPT, st);
  if (rc != PTB_OK) return rc;
  typename P::Params p;
  p.tab = static_cast<const S*>(ws);
  p.tab_stride = coef_batched ? SosDims<K>::ROWTAB : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  p.B = B;
  const bool bulk = aligned16(x) && aligned16(y) && (T * sizeof(S)) % 16 == 0;
  return launch_scan<P, false>(p, B, T, bulk, static_cast<char*>(ws) + tb, wsb - tb, status, st, nullptr, nullptr);
}

// With the outputs of the inner sections wanted, the sections run one by one through the
// single-section kernel: each of those passes moves 8 bytes per sample at close to the memory
// bandwidth, and together they write exactly the arrays the fused backward pass reads.
template <class S>
static int sos_fwd_chain(int dtype, int K, int64_t B, int64_t T, const S* b, const S* a, int coef_batched,
                         const S* zi, const S* x, S* y, S* mid, S* zf, void* ws, int64_t wsb, uint32_t* status,
                         ptb_stream_t st) {
  const int64_t rows = coef_batched ? B : 1;
  for (int k = 0; k < K; ++k) {
    const S* in = k == 0 ? x : mid + (int64_t)(k - 1) * B * T;
    S* out = k == K - 1 ? y : mid + (int64_t)k * B * T;
    const int rc = ptb_biquad_tdf2_fwd(dtype, B, T, b + (int64_t)k * rows * 3, a + (int64_t)k * rows * 2, coef_batched,
                                       zi ? zi + (int64_t)k * B * 2 : nullptr, in, out,
                                       zf ? zf + (int64_t)k * B * 2 : nullptr, ws, wsb, status, st);
    if (rc != PTB_OK) return rc;
  }
  return PTB_OK;
}

template <class S, int K>
struct SosCoefGrads {
  const S* a; int64_t a_sec, a_row;
  S* grad_b; S* grad_a;
  int64_t rows;
  __device__ void operator()(int64_t row, const double* acc) const {
    for (int k = 0; k < K; ++k) {
      const double a1 = (double)a[k * a_sec + row * a_row], a2 = (double)a[k * a_sec + row * a_row + 1];
      const double* q = acc + 5 * k;
      if (grad_b) {
        S* gb = grad_b + (k * rows + row) * 3;
        gb[0] = (S)(q[0] - a1 * q[1] - a2 * q[2]);
        gb[1] = (S)q[1];
        gb[2] = (S)q[2];
      }
      if (grad_a) {
        S* ga = grad_a + (k * rows + row) * 2;
        ga[0] = (S)(-q[3]);
        ga[1] = (S)(-q[4]);
      }
    }
  }
};

template <class S, int K, class C>
static int chain_bwd_cfg(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                         const void* mid, const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b,
                         void* grad_a, void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using L = ChainBwdSmem<C>;
  static_assert(L::kTotal <= 227 * 1024, "shared memory of an SM");
  const int64_t rows = coef_batched ? B : 1;
  const int64_t tb = align_up(rows * C::ROW * (int64_t)sizeof(S), 256);
  const int64_t nchunks = (T + C::TILE - 1) / C::TILE;
  const int64_t ntiles = B * nchunks;
  if (ntiles >= 0xFFFFFFFEll || B >= 0xFFFFFFFFll) return PTB_ERR_TOO_LARGE;
  const WsLayout l = ws_layout(ntiles, C::SLOT_WORDS, 5 * K * sizeof(S));
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < tb + l.total) return PTB_ERR_WORKSPACE;
  const bool want_coef = grad_b != nullptr || grad_a != nullptr;
  if (want_coef && (!x || !mid || !y)) return PTB_ERR_ARG;
  chain_setup_kernel<S, C, true><<<(unsigned)((rows * K + 31) / 32), 32, 0, st>>>(
      static_cast<const S*>(b), rows * 3, coef_batched ? 3 : 0, static_cast<const S*>(a), rows * 2,
      coef_batched ? 2 : 0, static_cast<S*>(ws), rows);
  PTB_CUDA(cudaGetLastError());
  char* w = static_cast<char*>(ws) + tb;
  PTB_CUDA(cudaMemsetAsync(w, 0, (size_t)l.part_off, st));
  Workspace wk;
  wk.ticket = reinterpret_cast<uint32_t*>(w);
  wk.error = status ? status : reinterpret_cast<uint32_t*>(w + 4);
  wk.slots = reinterpret_cast<uint64_t*>(w + l.slots_off);
  wk.partial = w + l.part_off;
  ChainBwdParams<S> p;
  p.tab = static_cast<const S*>(ws);
  p.tab_stride = coef_batched ? C::ROW : 0;
  p.gy = static_cast<const S*>(gy);
  p.x = static_cast<const S*>(x);
  p.mid = static_cast<const S*>(mid);
  p.y = static_cast<const S*>(y);
  p.g_in = static_cast<const S*>(g_zf);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_zi = static_cast<S*>(grad_zi);
  p.T = T;
  p.B = B;
  p.want_coef = want_coef ? 1 : 0;
  const bool bulk = aligned16(gy) && aligned16(grad_x) &&
                    (!want_coef || (aligned16(x) && aligned16(mid) && aligned16(y))) && (T * sizeof(S)) % 16 == 0;
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != PTB_OK) return rc;
  static bool attr_set[kMaxDevices] = {};
  int dev = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  {   // first use on this device: one thread fills the cache, the others wait
    std::lock_guard<std::mutex> init_lock(init_mutex());
    if (!attr_set[dev]) {
      PTB_CUDA(cudaFuncSetAttribute(chain_bwd_kernel<S, C>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      attr_set[dev] = true;
    }
  }
  int occ = 1;
  PTB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, chain_bwd_kernel<S, C>, C::NT, L::kTotal));
  const unsigned grid = (unsigned)std::min<int64_t>(ntiles, (int64_t)sms * std::max(occ, 1));
  chain_bwd_kernel<S, C><<<grid, C::NT, L::kTotal, st>>>(p, wk, (uint32_t)B, (uint32_t)nchunks, (uint32_t)ntiles,
                                                         bulk ? 1 : 0, g_wait_ns);
  PTB_CUDA(cudaGetLastError());
  if (!want_coef) return PTB_OK;
  SosCoefGrads<S, K> epi{static_cast<const S*>(a), rows * 2, coef_batched ? 2 : 0, static_cast<S*>(grad_b),
                         static_cast<S*>(grad_a), rows};
  return launch_reduce<S, 5 * K>(wk.partial, B, nchunks, coef_batched, epi, st);
}

template <class S, int K>
static int chain_bwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                     const void* mid, const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b,
                     void* grad_a, void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  int sms = 0;
  const int rc = device_sms(&sms);
  if (rc != PTB_OK) return rc;
  if (chain_few_rows(B, sms))
    return chain_bwd_cfg<S, K, ChainBFew<S, K>>(B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a,
                                                grad_zi, ws, wsb, status, st);
  return chain_bwd_cfg<S, K, ChainB<S, K>>(B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a,
                                           grad_zi, ws, wsb, status, st);
}

template <class S, int K>
static int sos_bwd(int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                   const void* mid, const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b,
                   void* grad_a, void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = SosBwdP<S, K>;
  const int64_t rows = coef_batched ? B : 1;
  const int64_t tb = table_bytes<S, K>(rows);
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < tb + kHeaderBytes) return PTB_ERR_WORKSPACE;
  const bool want_coef = grad_b != nullptr || grad_a != nullptr;
  if (want_coef && (!x || !mid || !y)) return PTB_ERR_ARG;
  int rc = build_table<S, K, true>(b, a, coef_batched, B, ws, P::SPT, st);
  if (rc != PTB_OK) return rc;
  char* scan_ws = static_cast<char*>(ws) + tb;
  typename P::Params p;
  p.tab = static_cast<const S*>(ws);
  p.tab_stride = coef_batched ? SosDims<K>::ROWTAB : 0;
  p.gy = static_cast<const S*>(gy);
  p.x = static_cast<const S*>(x);
  p.mid = static_cast<const S*>(mid);
  p.y = static_cast<const S*>(y);
  p.g_in = static_cast<const S*>(g_zf);
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_zi = static_cast<S*>(grad_zi);
  p.err = status ? status : reinterpret_cast<uint32_t*>(scan_ws + 4);
  p.T = T;
  p.B = B;
  p.want_coef = want_coef ? 1 : 0;
  const bool bulk = aligned16(gy) && aligned16(grad_x) &&
                    (!want_coef || (aligned16(x) && aligned16(mid) && aligned16(y))) && (T * sizeof(S)) % 16 == 0;
  p.bulk = bulk ? 1 : 0;
  void* partial = nullptr;
  int64_t nchunks = 0;
  rc = launch_scan<P, false>(p, B, T, bulk, scan_ws, wsb - tb, status, st, &partial, &nchunks);
  if (rc != PTB_OK || !want_coef) return rc;
  SosCoefGrads<S, K> epi{static_cast<const S*>(a), rows * 2, coef_batched ? 2 : 0, static_cast<S*>(grad_b),
                         static_cast<S*>(grad_a), rows};
  return launch_reduce<S, 5 * K>(partial, B, nchunks, coef_batched, epi, st);
}

}  // namespace ptb

using namespace ptb;

#ifdef PTB_SOS_MINIMAL   // tuning builds: only the six-section float kernels
#define PTB_SOS_DISPATCH(FN, ...)                                            \
  do {                                                                       \
    if (dtype == PTB_F32 && K == 6) return FN<float, 6>(__VA_ARGS__);        \
  } while (0)
#else
#define PTB_SOS_DISPATCH(FN, ...)                                            \
  do {                                                                       \
    if (dtype == PTB_F32) {                                                  \
      switch (K) {                                                           \
        case 2: return FN<float, 2>(__VA_ARGS__);                            \
        case 4: return FN<float, 4>(__VA_ARGS__);                            \
        case 6: return FN<float, 6>(__VA_ARGS__);                            \
        case 8: return FN<float, 8>(__VA_ARGS__);                            \
      }                                                                      \
    } else if (dtype == PTB_F64) {                                           \
      switch (K) {                                                           \
        case 2: return FN<double, 2>(__VA_ARGS__);                           \
        case 4: return FN<double, 4>(__VA_ARGS__);                           \
        case 6: return FN<double, 6>(__VA_ARGS__);                           \
        case 8: return FN<double, 8>(__VA_ARGS__);                           \
      }                                                                      \
    }                                                                        \
  } while (0)
#endif

namespace ptb {
// Single section through the chained backward kernel (K = 1): picked by ptb_biquad_tdf2_bwd for
// large batches when the caller's workspace is large enough (0.43 ms against 0.47 ms at B = 512,
// T = 2^18; the forward pass is faster on the decoupled kernel).  Returns -1 when not applicable.
int biquad_chain_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                     const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b, void* grad_a,
                     void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  int sms = 0;
  if (device_sms(&sms) != PTB_OK || !use_chain(B, sms)) return -1;
  // a row keeps ONE tile of a single section busy: the chained kernel needs about three rows per SM to
  // fill the GPU (B = 128, T = 2^19: 0.308 ms chained against 0.20 ms on the decoupled kernel)
  if (g_sos_mode == 0 && B < 3 * (int64_t)sms) return -1;
  // K = 1: there are no intermediate outputs; the kernel is handed x as Z_0 and y as Z_1
  const void* mid = x;
  if (dtype == PTB_F32) {
    if (wsb < chain_ws_bytes<float, 1>(B, T)) return -1;
    return chain_bwd<float, 1>(B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, ws, wsb,
                               status, st);
  }
  if (dtype == PTB_F64) {
    if (wsb < chain_ws_bytes<double, 1>(B, T)) return -1;
    return chain_bwd<double, 1>(B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, ws,
                                wsb, status, st);
  }
  return -1;
}

// Single section through the decoupled kernels with K = 1: the linear parts of all maps come from
// the row's table of powers M^(SPT 2^i), built in double, so no matrices are multiplied in the
// section's own precision.  (Squaring a rounded power doubles its relative error; after the ~14
// doublings of a thread / warp / tile hierarchy a float32 section with a nearly double pole close to
// the unit circle -- pole angle near 0 or pi, radius ~0.99 -- misses the sequential result by
// ~3e-4 of max|y| when the powers are formed in float32.)  Returns -1 when the caller's workspace
// cannot hold the table (very short rows): the caller then takes the generic 2x2 policy.
int biquad_table_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* zi,
                     const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  const int64_t rows = coef_batched ? B : 1;
  if (dtype == PTB_F32) {
    if (wsb < table_bytes<float, 1>(rows) + scan_ws_bytes<SosFwdP<float, 1>>(B, T)) return -1;
    return sos_fwd<float, 1>(B, T, b, a, coef_batched, zi, x, y, zf, ws, wsb, status, st);
  }
  if (dtype == PTB_F64) {
    if (wsb < table_bytes<double, 1>(rows) + scan_ws_bytes<SosFwdP<double, 1>>(B, T)) return -1;
    return sos_fwd<double, 1>(B, T, b, a, coef_batched, zi, x, y, zf, ws, wsb, status, st);
  }
  return -1;
}

int biquad_table_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched, const void* x,
                     const void* y, const void* gy, const void* g_zf, void* grad_x, void* grad_b, void* grad_a,
                     void* grad_zi, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  const int64_t rows = coef_batched ? B : 1;
  const void* mid = x;   // K = 1: no intermediate outputs (never read)
  if (dtype == PTB_F32) {
    if (wsb < table_bytes<float, 1>(rows) + scan_ws_bytes<SosBwdP<float, 1>>(B, T)) return -1;
    return sos_bwd<float, 1>(B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, ws, wsb,
                             status, st);
  }
  if (dtype == PTB_F64) {
    if (wsb < table_bytes<double, 1>(rows) + scan_ws_bytes<SosBwdP<double, 1>>(B, T)) return -1;
    return sos_bwd<double, 1>(B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, ws, wsb,
                              status, st);
  }
  return -1;
}
}  // namespace ptb

extern "C" {

int ptb_sos_cascade_set_mode(int mode) {
  if (mode < 0 || mode > 2) return PTB_ERR_ARG;
  g_sos_mode = mode;
  return PTB_OK;
}

int64_t ptb_sos_cascade_workspace_bytes(int dtype, int K, int64_t B, int64_t T) {
  if (B <= 0 || T <= 0) return 0;
  PTB_SOS_DISPATCH(sos_ws_bytes, B, T);   // includes the bound of the single-section passes
  return 0;
}

int ptb_sos_cascade_fwd(int dtype, int K, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* zi, const void* x, void* y, void* mid, void* zf, void* workspace,
                        int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B <= 0 || T <= 0 || !b || !a || !x || !y) return PTB_ERR_ARG;
  int sms = 0;
  const int rcs = device_sms(&sms);
  if (rcs != PTB_OK) return rcs;
  if (use_chain(B, sms)) {
    PTB_SOS_DISPATCH(chain_fwd, B, T, b, a, coef_batched, zi, x, y, mid, zf, workspace, workspace_bytes, status,
                     (cudaStream_t)stream);
    return PTB_ERR_ARG;
  }
  if (mid != nullptr) {
    if (K < 2 || K > 8) return PTB_ERR_ARG;
    if (dtype == PTB_F32)
      return sos_fwd_chain<float>(dtype, K, B, T, (const float*)b, (const float*)a, coef_batched, (const float*)zi,
                                  (const float*)x, (float*)y, (float*)mid, (float*)zf, workspace, workspace_bytes,
                                  status, stream);
    if (dtype == PTB_F64)
      return sos_fwd_chain<double>(dtype, K, B, T, (const double*)b, (const double*)a, coef_batched,
                                   (const double*)zi, (const double*)x, (double*)y, (double*)mid, (double*)zf,
                                   workspace, workspace_bytes, status, stream);
    return PTB_ERR_ARG;
  }
  PTB_SOS_DISPATCH(sos_fwd, B, T, b, a, coef_batched, zi, x, y, zf, workspace, workspace_bytes, status,
                   (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

int ptb_sos_cascade_bwd(int dtype, int K, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* x, const void* mid, const void* y, const void* gy, const void* g_zf,
                        void* grad_x, void* grad_b, void* grad_a, void* grad_zi, void* workspace,
                        int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  if (B <= 0 || T <= 0 || !b || !a || !gy || !grad_x) return PTB_ERR_ARG;
  int sms = 0;
  const int rcs = device_sms(&sms);
  if (rcs != PTB_OK) return rcs;
  if (use_chain(B, sms)) {
    PTB_SOS_DISPATCH(chain_bwd, B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi,
                     workspace, workspace_bytes, status, (cudaStream_t)stream);
    return PTB_ERR_ARG;
  }
  PTB_SOS_DISPATCH(sos_bwd, B, T, b, a, coef_batched, x, mid, y, gy, g_zf, grad_x, grad_b, grad_a, grad_zi, workspace,
                   workspace_bytes, status, (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

}  // extern "C"
