// C ABI of the dense N x N recurrences, 2 < N <= 8 (see include/philtorch_b200.h).
#include "launch.cuh"

#include "mat_n.cuh"
#include "mat_n_lti.cuh"

namespace ptb {

// (threads, samples per thread, stages) per padded size and precision: the stage holds
// TILE * (NMAX + NMAX^2) scalars.  An odd number of samples per thread spreads a warp's 16-byte
// shared-memory accesses over the banks (4x4, fp32, B=16, T=2^18, forward + adjoint scan: 1.62 ms with
// 2 samples and 4-byte accesses, 0.84 ms with 16-byte accesses, 0.55 ms with 3 samples, 0.40 ms with 5)
template <class S, int NMAX> struct MatNGeom;
template <> struct MatNGeom<float, 4> { static constexpr int NT = 256, SPT = 5, ST = 2; };
template <> struct MatNGeom<double, 4> { static constexpr int NT = 128, SPT = 3, ST = 3; };
template <> struct MatNGeom<float, 8> { static constexpr int NT = 128, SPT = 3, ST = 2; };
template <> struct MatNGeom<double, 8> { static constexpr int NT = 128, SPT = 1, ST = 2; };
template <class S, int NMAX, bool REV>
using MatNP = MatN<S, NMAX, MatNGeom<S, NMAX>::NT, MatNGeom<S, NMAX>::SPT, MatNGeom<S, NMAX>::ST, REV>;

static int g_matn_lti_tables = 1;   // constant matrices: 1 = table-of-powers policy, 0 = the general policy (tests)

template <class P>
static int64_t matn_ws(int64_t B, int64_t T) {
  const int64_t ntiles = B * ((T + P::TILE - 1) / P::TILE);
  return ws_layout(ntiles, P::SLOT_WORDS, sizeof(typename P::Partial)).total;
}

template <class S, int NMAX, bool REV>
static int matn_run(int N, int64_t B, int64_t T, const void* A, int A_batched, int A_timevar, const void* zi,
                    const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = MatNP<S, NMAX, REV>;
  typename P::Params p;
  p.A = static_cast<const S*>(A);
  p.a_t_stride = A_timevar ? (int64_t)N * N : 0;
  p.a_row_stride = A_batched ? (A_timevar ? T * N * N : (int64_t)N * N) : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  p.N = N;
  const bool bulk = aligned16(x) && aligned16(y) && (!A_timevar || aligned16(A)) && (T * N * sizeof(S)) % 16 == 0 &&
                    ((int64_t)P::TILE * N * sizeof(S)) % 16 == 0;
  return launch_scan<P, false>(p, B, T, bulk, ws, wsb, status, st, nullptr, nullptr);
}

// constant matrices: table-of-powers policy (mat_n_lti.cuh).  (threads, samples per thread, stages)
template <class S, int NMAX> struct MatNLtiGeom;
#ifndef PTB_MATN_LTI_SPT4
#define PTB_MATN_LTI_SPT4 7
#define PTB_MATN_LTI_SPT8 9
#endif
template <> struct MatNLtiGeom<float, 4> { static constexpr int NT = 256, SPT = PTB_MATN_LTI_SPT4, ST = 3; };
template <> struct MatNLtiGeom<double, 4> { static constexpr int NT = 256, SPT = 3, ST = 3; };
template <> struct MatNLtiGeom<float, 8> { static constexpr int NT = 256, SPT = PTB_MATN_LTI_SPT8, ST = 3; };
template <> struct MatNLtiGeom<double, 8> { static constexpr int NT = 256, SPT = 3, ST = 3; };
template <class S, int NMAX, bool REV>
using MatNLtiP = MatNLti<S, NMAX, MatNLtiGeom<S, NMAX>::NT, MatNLtiGeom<S, NMAX>::SPT, MatNLtiGeom<S, NMAX>::ST, REV>;

template <class S, int NMAX>
static int64_t matn_lti_table_bytes(int64_t B) {
  return align_up(B * MatNLtiDims<NMAX>::ROWTAB * (int64_t)sizeof(S), 256);
}

template <class S, int NMAX, bool REV>
static int matn_lti_run(int N, int64_t B, int64_t T, const void* A, int A_batched, const void* zi, const void* x,
                        void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  using P = MatNLtiP<S, NMAX, REV>;
  using D = MatNLtiDims<NMAX>;
  if ((T + P::SPT - 1) / P::SPT >= (1ll << D::NPOW)) return PTB_ERR_TOO_LARGE;
  const int64_t rows = A_batched ? B : 1;
  const int64_t scan_ws = align_up(matn_ws<P>(B, T), 256);
  if (!ws || (reinterpret_cast<uintptr_t>(ws) & 255u) || wsb < scan_ws + matn_lti_table_bytes<S, NMAX>(rows))
    return PTB_ERR_WORKSPACE;
  S* tab = reinterpret_cast<S*>(static_cast<char*>(ws) + scan_ws);
  matn_lti_setup_kernel<S, NMAX, REV><<<(unsigned)rows, D::NN, 0, st>>>(static_cast<const S*>(A), A_batched ? (int64_t)N * N : 0,
                                                                      N, tab, P::SPT);
  PTB_CUDA(cudaGetLastError());
  typename P::Params p;
  p.tab = tab;
  p.tab_stride = A_batched ? D::ROWTAB : 0;
  p.zi = static_cast<const S*>(zi);
  p.x = static_cast<const S*>(x);
  p.y = static_cast<S*>(y);
  p.zf = static_cast<S*>(zf);
  p.T = T;
  p.N = N;
  const bool bulk = aligned16(x) && aligned16(y) && (T * N * sizeof(S)) % 16 == 0 &&
                    ((int64_t)P::TILE * N * sizeof(S)) % 16 == 0;
  return launch_scan<P, false>(p, B, T, bulk, ws, scan_ws, status, st, nullptr, nullptr);
}

template <class S, bool REV>
static int matn_dispatch(int N, int64_t B, int64_t T, const void* A, int A_batched, int A_timevar, const void* zi,
                         const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  if (!A_timevar && g_matn_lti_tables) {
    const int rc = N <= 4 ? matn_lti_run<S, 4, REV>(N, B, T, A, A_batched, zi, x, y, zf, ws, wsb, status, st)
                          : matn_lti_run<S, 8, REV>(N, B, T, A, A_batched, zi, x, y, zf, ws, wsb, status, st);
    if (rc != PTB_ERR_TOO_LARGE) return rc;   // rows beyond 2^24 thread units: the general policy
  }
  if (N <= 4) return matn_run<S, 4, REV>(N, B, T, A, A_batched, A_timevar, zi, x, y, zf, ws, wsb, status, st);
  return matn_run<S, 8, REV>(N, B, T, A, A_batched, A_timevar, zi, x, y, zf, ws, wsb, status, st);
}

template <class S, int NMAX>
static int64_t matn_ws_all(int64_t B, int64_t T) {
  const int64_t general = std::max(matn_ws<MatNP<S, NMAX, false>>(B, T), matn_ws<MatNP<S, NMAX, true>>(B, T));
  const int64_t lti = align_up(std::max(matn_ws<MatNLtiP<S, NMAX, false>>(B, T), matn_ws<MatNLtiP<S, NMAX, true>>(B, T)), 256) +
                      matn_lti_table_bytes<S, NMAX>(B);
  return std::max(general, lti);
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int64_t ptb_recur_n_workspace_bytes(int dtype, int N, int64_t B, int64_t T) {
  if (B <= 0 || T <= 0 || N < 1 || N > 8) return 0;
  if (dtype == PTB_F32) return N <= 4 ? matn_ws_all<float, 4>(B, T) : matn_ws_all<float, 8>(B, T);
  if (dtype == PTB_F64) return N <= 4 ? matn_ws_all<double, 4>(B, T) : matn_ws_all<double, 8>(B, T);
  return 0;
}

int64_t ptb_outer_prev_sum_chunks(int64_t B, int64_t T) {
  if (B <= 0 || T <= 0) return 0;
  // enough blocks to fill the device, chunks of at least 4096 samples
  const int64_t want = (8 * 148 + B - 1) / B;
  const int64_t most = (T + 4095) / 4096;
  return std::max<int64_t>(1, std::min(want, most));
}

int ptb_outer_prev_sum(int dtype, int N, int64_t B, int64_t T, const void* g, const void* h, const void* zi,
                       void* partial, ptb_stream_t stream) {
  if (B < 0 || T < 0 || N < 1 || N > 8) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!g || !h || !zi || !partial) return PTB_ERR_ARG;
  const int64_t chunks = ptb_outer_prev_sum_chunks(B, T);
  const int64_t chunk_len = (T + chunks - 1) / chunks;
  if (B * chunks >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)(B * chunks);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == PTB_F32) {
    if (N <= 4) outer_prev_sum_kernel<float, 4><<<grid, kOuterNT, 0, st>>>((const float*)g, (const float*)h, (const float*)zi, (float*)partial, N, T, (int)chunks, chunk_len);
    else outer_prev_sum_kernel<float, 8><<<grid, kOuterNT, 0, st>>>((const float*)g, (const float*)h, (const float*)zi, (float*)partial, N, T, (int)chunks, chunk_len);
  } else if (dtype == PTB_F64) {
    if (N <= 4) outer_prev_sum_kernel<double, 4><<<grid, kOuterNT, 0, st>>>((const double*)g, (const double*)h, (const double*)zi, (double*)partial, N, T, (int)chunks, chunk_len);
    else outer_prev_sum_kernel<double, 8><<<grid, kOuterNT, 0, st>>>((const double*)g, (const double*)h, (const double*)zi, (double*)partial, N, T, (int)chunks, chunk_len);
  } else {
    return PTB_ERR_ARG;
  }
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

int ptb_recur_n_set_policy(int policy) {
  if (policy < 0 || policy > 1) return PTB_ERR_ARG;
  g_matn_lti_tables = policy == 0 ? 1 : 0;
  return PTB_OK;
}

int ptb_recur_n_fwd(int dtype, int N, int64_t B, int64_t T, const void* A, int A_batched, int A_timevar,
                    const void* zi, const void* x, void* y, void* zf, void* workspace, int64_t workspace_bytes,
                    uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0 || N < 1 || N > 8) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !zi || !x || !y) return PTB_ERR_ARG;
  if (dtype == PTB_F32)
    return matn_dispatch<float, false>(N, B, T, A, A_batched, A_timevar, zi, x, y, zf, workspace, workspace_bytes,
                                       status, (cudaStream_t)stream);
  if (dtype == PTB_F64)
    return matn_dispatch<double, false>(N, B, T, A, A_batched, A_timevar, zi, x, y, zf, workspace, workspace_bytes,
                                        status, (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

int ptb_recur_n_adj(int dtype, int N, int64_t B, int64_t T, const void* A, int A_batched, int A_timevar,
                    const void* gy, const void* g_in, void* g, void* c0, void* workspace, int64_t workspace_bytes,
                    uint32_t* status, ptb_stream_t stream) {
  if (B < 0 || T < 0 || N < 1 || N > 8) return PTB_ERR_ARG;
  if (B == 0 || T == 0) return PTB_OK;
  if (!A || !gy || !g) return PTB_ERR_ARG;
  if (dtype == PTB_F32)
    return matn_dispatch<float, true>(N, B, T, A, A_batched, A_timevar, g_in, gy, g, c0, workspace, workspace_bytes,
                                      status, (cudaStream_t)stream);
  if (dtype == PTB_F64)
    return matn_dispatch<double, true>(N, B, T, A, A_batched, A_timevar, g_in, gy, g, c0, workspace, workspace_bytes,
                                       status, (cudaStream_t)stream);
  return PTB_ERR_ARG;
}

}  // extern "C"
