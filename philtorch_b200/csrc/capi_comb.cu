// C ABI of the comb-filter kernels (see include/philtorch_b200.h).
#include "launch.cuh"

#include "comb.cuh"

namespace ptb {

static int comb_blocks_per_row(int64_t D) { return (int)((D + 31) / 32); }   // a block: 32 phases

template <class S>
static int comb_fwd(int64_t B, int64_t N, int64_t D, const void* a, int a_batched, const void* zi, int zi_mode,
                    const void* x, void* y, cudaStream_t st) {
  const int bpr = comb_blocks_per_row(D);
  comb_fwd_kernel<S><<<(unsigned)(B * bpr), kCombThreads, 0, st>>>(
      static_cast<const S*>(x), static_cast<const S*>(a), a_batched ? 1 : 0, static_cast<const S*>(zi), zi_mode,
      static_cast<S*>(y), N, D, bpr);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int comb_bwd(int64_t B, int64_t N, int64_t D, const void* a, int a_batched, const void* zi, int zi_mode,
                    const void* y, const void* gy, void* grad_x, void* partial, void* grad_state, cudaStream_t st) {
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

int64_t ptb_comb_partial_blocks(int64_t delay) { return delay > 0 ? comb_blocks_per_row(delay) : 0; }

int ptb_comb_fwd(int dtype, int64_t B, int64_t N, int64_t delay, const void* a, int a_batched, const void* zi,
                 int zi_mode, const void* x, void* y, void* workspace, int64_t workspace_bytes, uint32_t* status,
                 ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes; (void)status;
  if (B < 0 || N < 0 || delay < 1 || zi_mode < 0 || zi_mode > 2) return PTB_ERR_ARG;
  if (B == 0 || N == 0) return PTB_OK;
  if (!a || !x || !y || (zi_mode && !zi)) return PTB_ERR_ARG;
  if (B * (int64_t)comb_blocks_per_row(delay) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_F32: return comb_fwd<float>(B, N, delay, a, a_batched, zi, zi_mode, x, y, (cudaStream_t)stream);
    case PTB_F64: return comb_fwd<double>(B, N, delay, a, a_batched, zi, zi_mode, x, y, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_comb_bwd(int dtype, int64_t B, int64_t N, int64_t delay, const void* a, int a_batched, const void* zi,
                 int zi_mode, const void* y, const void* gy, void* grad_x, void* partial, void* grad_state,
                 void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes; (void)status;
  if (B < 0 || N < 0 || delay < 1 || zi_mode < 0 || zi_mode > 2) return PTB_ERR_ARG;
  if (B == 0 || N == 0) return PTB_OK;
  if (!a || !gy || !grad_x || (partial && !y) || (partial && zi_mode && !zi)) return PTB_ERR_ARG;
  if (B * (int64_t)comb_blocks_per_row(delay) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_F32:
      return comb_bwd<float>(B, N, delay, a, a_batched, zi, zi_mode, y, gy, grad_x, partial, grad_state,
                             (cudaStream_t)stream);
    case PTB_F64:
      return comb_bwd<double>(B, N, delay, a, a_batched, zi, zi_mode, y, gy, grad_x, partial, grad_state,
                              (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

}  // extern "C"
