// C ABI of the fix-up kernels of the time-split first-order recurrence (see include/philtorch_b200.h).
#include "launch.cuh"

#include "shard_fixup.cuh"
#include "shard_fixup2.cuh"

namespace ptb {

static int fix_grid(int64_t rows, unsigned* grid) {
  int dev = 0, sms = 0;
  PTB_CUDA(cudaGetDevice(&dev));
  PTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  *grid = (unsigned)std::min<int64_t>(rows, (int64_t)sms * 8);
  return PTB_OK;
}

template <class S>
static int fixup_fwd(int64_t B, int64_t nseg, int64_t L, const void* a, int a_batched, void* y, const void* seg_maps,
                     const void* zi, const void* rank_maps, int rank, int world, void* states, cudaStream_t st) {
  FixupParams<S> p{};
  p.B = B; p.nseg = nseg; p.L = L;
  p.a = static_cast<const S*>(a); p.a_row_stride = a_batched ? L : 0;
  p.seg_maps = static_cast<const S*>(seg_maps);
  p.rank_maps = static_cast<const S*>(rank_maps);
  p.rank = rank; p.world = world;
  p.zi = static_cast<const S*>(zi);
  p.y = static_cast<S*>(y);
  p.states = static_cast<S*>(states);
  unsigned grid = 1;
  const int rc = fix_grid(B * nseg, &grid);
  if (rc != PTB_OK) return rc;
  fixup_fwd_kernel<S><<<grid, kFixNT, 0, st>>>(p);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int fixup_bwd(int64_t B, int64_t nseg, int64_t L, const void* a, int a_batched, const void* y,
                     const void* states, const void* seg_maps, const void* rank_maps, int rank, int world,
                     void* grad_x, void* grad_a, void* grad_zi, cudaStream_t st) {
  FixupParams<S> p{};
  p.B = B; p.nseg = nseg; p.L = L;
  p.a = static_cast<const S*>(a); p.a_row_stride = a_batched ? L : 0;
  p.seg_maps = static_cast<const S*>(seg_maps);
  p.rank_maps = static_cast<const S*>(rank_maps);
  p.rank = rank; p.world = world;
  p.y = const_cast<S*>(static_cast<const S*>(y));
  p.states = const_cast<S*>(static_cast<const S*>(states));
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_a = static_cast<S*>(grad_a);
  p.grad_zi = static_cast<S*>(grad_zi);
  unsigned grid = 1;
  const int rc = fix_grid(B * nseg, &grid);
  if (rc != PTB_OK) return rc;
  fixup_bwd_kernel<S><<<grid, kFixNT, 0, st>>>(p);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int fold_maps(int64_t B, int64_t nseg, const void* maps, int reverse, void* out, cudaStream_t st) {
  fold_maps_kernel<S><<<(unsigned)((B + 127) / 128), 128, 0, st>>>(static_cast<const S*>(maps), B, nseg, reverse,
                                                                 static_cast<S*>(out));
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int fixup2_fwd(int64_t B, int64_t nseg, int64_t L, const void* A, void* y, const void* P, const void* e,
                      const void* zi, void* states, cudaStream_t st) {
  Fixup2Params<S> p{};
  p.B = B; p.nseg = nseg; p.L = L;
  p.A = static_cast<const S*>(A);
  p.P = static_cast<const S*>(P);
  p.e = static_cast<const S*>(e);
  p.zi = static_cast<const S*>(zi);
  p.y = static_cast<S*>(y);
  p.states = static_cast<S*>(states);
  unsigned grid = 1;
  const int rc = fix_grid(B * nseg, &grid);
  if (rc != PTB_OK) return rc;
  fixup2_fwd_kernel<S><<<grid, kFix2NT, 0, st>>>(p);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int fixup2_bwd(int64_t B, int64_t nseg, int64_t L, const void* A, const void* y, const void* states,
                      const void* P, const void* e, int x_scalar, void* grad_x, void* grad_A, void* grad_zi,
                      cudaStream_t st) {
  Fixup2Params<S> p{};
  p.B = B; p.nseg = nseg; p.L = L;
  p.A = static_cast<const S*>(A);
  p.P = static_cast<const S*>(P);
  p.e = static_cast<const S*>(e);
  p.y = const_cast<S*>(static_cast<const S*>(y));
  p.states = const_cast<S*>(static_cast<const S*>(states));
  p.x_scalar = x_scalar;
  p.grad_x = static_cast<S*>(grad_x);
  p.grad_A = static_cast<S*>(grad_A);
  p.grad_zi = static_cast<S*>(grad_zi);
  unsigned grid = 1;
  const int rc = fix_grid(B * nseg, &grid);
  if (rc != PTB_OK) return rc;
  fixup2_bwd_kernel<S><<<grid, kFix2NT, 0, st>>>(p);
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

template <class S>
static int fold_tile_products(int64_t R, int64_t nchunks, const void* tile_prod, void* P, cudaStream_t st) {
  fold_tile_products_kernel<S><<<(unsigned)((R + 127) / 128), 128, 0, st>>>(static_cast<const S*>(tile_prod), R, nchunks,
                                                                          static_cast<S*>(P));
  PTB_CUDA(cudaGetLastError());
  return PTB_OK;
}

}  // namespace ptb

using namespace ptb;

extern "C" {

int ptb_lpv_recur_fold_maps(int dtype, int64_t B, int64_t nseg, const void* maps, int reverse, void* out,
                            ptb_stream_t stream) {
  if (B < 0 || nseg < 1) return PTB_ERR_ARG;
  if (B == 0) return PTB_OK;
  if (!maps || !out) return PTB_ERR_ARG;
  switch (dtype) {
    case PTB_F32: return fold_maps<float>(B, nseg, maps, reverse, out, (cudaStream_t)stream);
    case PTB_F64: return fold_maps<double>(B, nseg, maps, reverse, out, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur_fixup_fwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* a, int a_batched, void* y,
                            const void* seg_maps, const void* zi, const void* rank_maps, int rank, int world,
                            void* states, ptb_stream_t stream) {
  if (B < 0 || nseg < 1 || L < 0 || world < 1 || rank < 0 || rank >= world) return PTB_ERR_ARG;
  if (B == 0) return PTB_OK;
  if (!a || !y || !seg_maps || !zi || !states || (world > 1 && !rank_maps)) return PTB_ERR_ARG;
  if (!a_batched && nseg != 1) return PTB_ERR_ARG;   // a shared (L,) array cannot be cut into segment rows
  switch (dtype) {
    case PTB_F32:
      return fixup_fwd<float>(B, nseg, L, a, a_batched, y, seg_maps, zi, world > 1 ? rank_maps : nullptr, rank, world,
                              states, (cudaStream_t)stream);
    case PTB_F64:
      return fixup_fwd<double>(B, nseg, L, a, a_batched, y, seg_maps, zi, world > 1 ? rank_maps : nullptr, rank, world,
                               states, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur_fixup_bwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* a, int a_batched,
                            const void* y, const void* states, const void* seg_maps, const void* rank_maps, int rank,
                            int world, void* grad_x, void* grad_a, void* grad_zi, ptb_stream_t stream) {
  if (B < 0 || nseg < 1 || L < 0 || world < 1 || rank < 0 || rank >= world) return PTB_ERR_ARG;
  if (B == 0) return PTB_OK;
  if (!a || !seg_maps || !grad_x || (grad_a && (!y || !states)) || (world > 1 && !rank_maps)) return PTB_ERR_ARG;
  if (!a_batched && nseg != 1) return PTB_ERR_ARG;
  switch (dtype) {
    case PTB_F32:
      return fixup_bwd<float>(B, nseg, L, a, a_batched, y, states, seg_maps, world > 1 ? rank_maps : nullptr, rank,
                              world, grad_x, grad_a, grad_zi, (cudaStream_t)stream);
    case PTB_F64:
      return fixup_bwd<double>(B, nseg, L, a, a_batched, y, states, seg_maps, world > 1 ? rank_maps : nullptr, rank,
                               world, grad_x, grad_a, grad_zi, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur2_fold_products(int dtype, int64_t R, int64_t nchunks, const void* tile_prod, void* P,
                                 ptb_stream_t stream) {
  if (R < 0 || nchunks < 1) return PTB_ERR_ARG;
  if (R == 0) return PTB_OK;
  if (!tile_prod || !P) return PTB_ERR_ARG;
  switch (dtype) {
    case PTB_F32: return fold_tile_products<float>(R, nchunks, tile_prod, P, (cudaStream_t)stream);
    case PTB_F64: return fold_tile_products<double>(R, nchunks, tile_prod, P, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur2_fixup_fwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* A, void* y, const void* P,
                             const void* e, const void* zi, void* states, ptb_stream_t stream) {
  if (B < 0 || nseg < 1 || L < 0) return PTB_ERR_ARG;
  if (B == 0 || L == 0) return PTB_OK;
  if (!A || !y || !P || !e || !zi || !states) return PTB_ERR_ARG;
  switch (dtype) {
    case PTB_F32: return fixup2_fwd<float>(B, nseg, L, A, y, P, e, zi, states, (cudaStream_t)stream);
    case PTB_F64: return fixup2_fwd<double>(B, nseg, L, A, y, P, e, zi, states, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

int ptb_lpv_recur2_fixup_bwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* A, const void* y,
                             const void* states, const void* P, const void* e, int x_scalar, void* grad_x,
                             void* grad_A, void* grad_zi, ptb_stream_t stream) {
  if (B < 0 || nseg < 1 || L < 0) return PTB_ERR_ARG;
  if (B == 0 || L == 0) return PTB_OK;
  if (!A || !P || !e || !grad_x || (grad_A && (!y || !states))) return PTB_ERR_ARG;
  switch (dtype) {
    case PTB_F32:
      return fixup2_bwd<float>(B, nseg, L, A, y, states, P, e, x_scalar, grad_x, grad_A, grad_zi, (cudaStream_t)stream);
    case PTB_F64:
      return fixup2_bwd<double>(B, nseg, L, A, y, states, P, e, x_scalar, grad_x, grad_A, grad_zi, (cudaStream_t)stream);
    default: return PTB_ERR_ARG;
  }
}

}  // extern "C"
