// C ABI of the eigenbasis output map (see include/philtorch_b200.h).
#include "launch.cuh"

#include "modal.cuh"

namespace ptb {

static int64_t modal_blocks_per_row(int64_t N) { return (N + kModalTile - 1) / kModalTile; }

template <class R>
static int modal_fwd(int64_t rows, int64_t M, int64_t N, const void* w, const void* w0, const void* coef,
                     int coef_batched, int real_out, void* y, cudaStream_t st) {
  const int64_t bpr = modal_blocks_per_row(N);
  modal_mix_fwd_kernel<R><<<(unsigned)(rows * bpr), kModalThreads, 0, st>>>(
      static_cast<const Cx<R>*>(w), static_cast<const Cx<R>*>(w0), static_cast<const Cx<R>*>(coef), coef_batched,
      real_out, y, M, N, bpr);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class R>
static int modal_bwd(int64_t rows, int64_t M, int64_t N, const void* w, const void* w0, const void* coef,
                     int coef_batched, int real_out, const void* gy, void* grad_w, void* grad_w0, void* partial,
                     cudaStream_t st) {
  const int64_t bpr = modal_blocks_per_row(N);
  modal_mix_bwd_kernel<R><<<(unsigned)(rows * bpr), kModalThreads, 0, st>>>(
      static_cast<const Cx<R>*>(w), static_cast<const Cx<R>*>(w0), static_cast<const Cx<R>*>(coef), coef_batched,
      real_out, gy, static_cast<Cx<R>*>(grad_w), static_cast<Cx<R>*>(grad_w0), static_cast<Cx<R>*>(partial), M, N,
      bpr);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class R>
static int modal_drive(int64_t rows, int64_t M, int64_t N, const void* x, const void* gain, int gain_batched, void* u,
                       cudaStream_t st) {
  const int64_t bpr = modal_blocks_per_row(N);
  modal_drive_fwd_kernel<R><<<(unsigned)(rows * bpr), kModalThreads, 0, st>>>(
      static_cast<const R*>(x), static_cast<const Cx<R>*>(gain), gain_batched, static_cast<Cx<R>*>(u), M, N, bpr);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int64_t ptb_modal_mix_partial_blocks(int64_t N) { return N > 0 ? modal_blocks_per_row(N) : 0; }

int ptb_modal_mix_fwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* w, const void* w0, const void* coef,
                      int coef_batched, int real_out, void* y, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes; (void)status;
  if (rows < 0 || M < 1 || N < 0) return PTB_ERR_ARG;
  if (rows == 0 || N == 0) return PTB_OK;
  if (!coef || !y || ((N > 1 || !w0) && !w)) return PTB_ERR_ARG;
  if (rows * modal_blocks_per_row(N) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_C64: return modal_fwd<float>(rows, M, N, w, w0, coef, coef_batched, real_out, y, (cudaStream_t)stream);
    case PTB_C128: return modal_fwd<double>(rows, M, N, w, w0, coef, coef_batched, real_out, y, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_modal_drive_fwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* x, const void* gain,
                        int gain_batched, void* u, void* workspace, int64_t workspace_bytes, uint32_t* status,
                        ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes; (void)status;
  if (rows < 0 || M < 1 || N < 0) return PTB_ERR_ARG;
  if (rows == 0 || N == 0) return PTB_OK;
  if (!x || !gain || !u) return PTB_ERR_ARG;
  if (rows * modal_blocks_per_row(N) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_C64: return modal_drive<float>(rows, M, N, x, gain, gain_batched, u, (cudaStream_t)stream);
    case PTB_C128: return modal_drive<double>(rows, M, N, x, gain, gain_batched, u, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_modal_mix_bwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* w, const void* w0, const void* coef,
                      int coef_batched, int real_out, const void* gy, void* grad_w, void* grad_w0, void* partial,
                      void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream) {
  (void)workspace; (void)workspace_bytes; (void)status;
  if (rows < 0 || M < 1 || N < 0) return PTB_ERR_ARG;
  if (rows == 0 || N == 0) return PTB_OK;
  if (!coef || !gy || !grad_w || !grad_w0 || (partial && (!w0 || (N > 1 && !w)))) return PTB_ERR_ARG;
  if (rows * modal_blocks_per_row(N) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_C64:
      return modal_bwd<float>(rows, M, N, w, w0, coef, coef_batched, real_out, gy, grad_w, grad_w0, partial,
                              (cudaStream_t)stream);
    case PTB_C128:
      return modal_bwd<double>(rows, M, N, w, w0, coef, coef_batched, real_out, gy, grad_w, grad_w0, partial,
                               (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

}  // extern "C"
