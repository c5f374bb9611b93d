// C ABI of the eigenbasis output map (see include/philtorch_b200.h).
#include "launch.cuh"

#include "modal.cuh"
#include "modal_bank.cuh"

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

// ---- fused bank of modes (modal_bank.cuh) -------------------------------------------------------------
// tiles of a row that one CTA takes in a row (the per-row tables are then built once per run): as many
// as leave about eight CTAs per SM
#ifndef PTB_BANK_AGG_RUN_DIV
#define PTB_BANK_AGG_RUN_DIV 4
#endif
static int64_t bank_run_length(int64_t rows, int64_t ntiles) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (rows * ntiles) / ((int64_t)sms * 8);
  return std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, 32), ntiles));
}

template <class R, int MMAX>
static int bank_fwd(BankParams<R> p, cudaStream_t st) {
  using C = BankCfg<R, MMAX>;
  const unsigned grid = (unsigned)(p.rows * ((p.ntiles + p.run - 1) / p.run));
  BankParams<R> pa = p;   // the aggregate pass keeps few registers: shorter runs, more CTAs per SM
  pa.run = std::max<int64_t>(1, p.run / PTB_BANK_AGG_RUN_DIV);
  bank_aggregate_kernel<R, MMAX, false><<<(unsigned)(p.rows * ((p.ntiles + pa.run - 1) / pa.run)), kBankNT, 0, st>>>(pa);
  PTB_CUDA(cudaGetLastError());
  bank_fold_kernel<R, false><<<(unsigned)((p.rows * p.M * 32 + 127) / 128), 128, 0, st>>>(p, C::TILE);
  PTB_CUDA(cudaGetLastError());
  bank_forward_kernel<R, MMAX><<<grid, kBankNT, 0, st>>>(p);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class R, int MMAX>
static int bank_bwd(BankParams<R> p, cudaStream_t st) {
  using C = BankCfg<R, MMAX>;
  const unsigned grid = (unsigned)(p.rows * ((p.ntiles + p.run - 1) / p.run));
  BankParams<R> pa = p;
  pa.run = std::max<int64_t>(1, p.run / PTB_BANK_AGG_RUN_DIV);
  bank_aggregate_kernel<R, MMAX, true><<<(unsigned)(p.rows * ((p.ntiles + pa.run - 1) / pa.run)), kBankNT, 0, st>>>(pa);
  PTB_CUDA(cudaGetLastError());
  bank_fold_kernel<R, true><<<(unsigned)((p.rows * p.M * 32 + 127) / 128), 128, 0, st>>>(p, C::TILE);
  PTB_CUDA(cudaGetLastError());
  bank_backward_kernel<R, MMAX><<<grid, kBankNT, 0, st>>>(p);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

static int64_t bank_tile(int64_t M) { return M <= 4 ? BankCfg<float, 4>::TILE : BankCfg<float, 8>::TILE; }

template <class R>
static int bank_run(bool adjoint, int64_t rows, int64_t M, int64_t N, const void* x, const void* gy, const void* lam,
                    const void* gain, const void* coef, const void* d, const void* w0, const void* g_wf, void* chk,
                    const void* fwd_chk, void* y, void* wf, void* partial, int need, cudaStream_t st) {
  BankParams<R> p;
  p.need = need;
  p.rows = rows; p.M = M; p.N = N;
  p.ntiles = (N + bank_tile(M) - 1) / bank_tile(M);
  p.run = bank_run_length(rows, p.ntiles);
  p.x = static_cast<const R*>(x);
  p.gy = static_cast<const R*>(gy);
  p.lam = static_cast<const Cx<R>*>(lam);
  p.gain = static_cast<const Cx<R>*>(gain);
  p.coef = static_cast<const Cx<R>*>(coef);
  p.d = static_cast<const R*>(d);
  p.w0 = static_cast<const Cx<R>*>(w0);
  p.g_wf = static_cast<const Cx<R>*>(g_wf);
  p.chk = static_cast<Cx<R>*>(chk);
  p.fwd_chk = static_cast<const Cx<R>*>(fwd_chk);
  p.y = static_cast<R*>(y);
  p.wf = static_cast<Cx<R>*>(wf);
  p.partial = static_cast<R*>(partial);
  if (M <= 4) return adjoint ? bank_bwd<R, 4>(p, st) : bank_fwd<R, 4>(p, st);
  return adjoint ? bank_bwd<R, 8>(p, st) : bank_fwd<R, 8>(p, st);
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


int64_t ptb_modal_bank_tiles(int64_t M, int64_t N) {
  if (M < 1 || M > 8 || N <= 0) return 0;
  return (N + bank_tile(M) - 1) / bank_tile(M);
}

int ptb_modal_bank_fwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* x, const void* lam,
                       const void* gain, const void* coef, const void* d, const void* w0, void* y, void* wf,
                       void* chk, ptb_stream_t stream) {
  if (rows < 0 || M < 1 || M > 8 || N < 0) return PTB_ERR_ARG;
  if (rows == 0 || N == 0) return PTB_OK;
  if (!x || !lam || !gain || !coef || !w0 || !y || !chk) return PTB_ERR_ARG;
  if (rows * ptb_modal_bank_tiles(M, N) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_F32:
      return bank_run<float>(false, rows, M, N, x, nullptr, lam, gain, coef, d, w0, nullptr, chk, nullptr, y, wf,
                             nullptr, 0, (cudaStream_t)stream);
    case PTB_F64:
      return bank_run<double>(false, rows, M, N, x, nullptr, lam, gain, coef, d, w0, nullptr, chk, nullptr, y, wf,
                              nullptr, 0, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_modal_bank_bwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* x, const void* lam,
                       const void* gain, const void* coef, const void* d, const void* fwd_chk, const void* gy,
                       const void* g_wf, int need, void* grad_x, void* grad_w0, void* partial, void* chk,
                       ptb_stream_t stream) {
  if (rows < 0 || M < 1 || M > 8 || N < 0) return PTB_ERR_ARG;
  if (rows == 0 || N == 0) return PTB_OK;
  if (!x || !lam || !gain || !coef || !fwd_chk || !gy || !grad_x || !grad_w0 || !partial || !chk) return PTB_ERR_ARG;
  if (rows * ptb_modal_bank_tiles(M, N) >= 0x7FFFFFFFll) return PTB_ERR_TOO_LARGE;
  switch (dtype) {
    case PTB_F32:
      return bank_run<float>(true, rows, M, N, x, gy, lam, gain, coef, d, nullptr, g_wf, chk, fwd_chk, grad_x,
                             grad_w0, partial, need, (cudaStream_t)stream);
    case PTB_F64:
      return bank_run<double>(true, rows, M, N, x, gy, lam, gain, coef, d, nullptr, g_wf, chk, fwd_chk, grad_x,
                              grad_w0, partial, need, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

}  // extern "C"
