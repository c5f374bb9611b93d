// Complex instantiations (complex64 / complex128) of the first-order recurrences; the public entry
// points in capi.cu forward here for the dtype codes PTB_C64 / PTB_C128.
#include "first_order_host.cuh"

namespace ptb {

#define PTB_CX_DISPATCH(dtype, CALL)                       \
  switch (dtype) {                                         \
    case PTB_C64: { using S = Cx<float>; return CALL; }    \
    case PTB_C128: { using S = Cx<double>; return CALL; }  \
    default: return PTB_ERR_ARG;                           \
  }

int cx_fo_fwd(int dtype, int lpv, int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
              const void* x, void* y, void* zf, void* ws, int64_t wsb, uint32_t* status, cudaStream_t st) {
  if (lpv) {
    PTB_CX_DISPATCH(dtype, (fo_fwd<S, true>(B, T, a, a_batched, zi, zi_batched, x, y, zf, ws, wsb, status, st)));
  }
  PTB_CX_DISPATCH(dtype, (fo_fwd<S, false>(B, T, a, a_batched, zi, zi_batched, x, y, zf, ws, wsb, status, st)));
}

int cx_fo_bwd(int dtype, int lpv, int64_t B, int64_t T, const void* a, int a_batched, const void* zi, int zi_batched,
              const void* y, const void* gy, const void* g_in, void* grad_x, void* grad_a, void* grad_zi, void* ws,
              int64_t wsb, uint32_t* status, cudaStream_t st, int ga_shared) {
  if (lpv) {
    PTB_CX_DISPATCH(dtype, (fo_bwd<S, true>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi,
                                            ws, wsb, status, st, ga_shared != 0)));
  }
  PTB_CX_DISPATCH(dtype, (fo_bwd<S, false>(B, T, a, a_batched, zi, zi_batched, y, gy, g_in, grad_x, grad_a, grad_zi,
                                           ws, wsb, status, st)));
}

}  // namespace ptb
