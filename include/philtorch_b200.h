/*
 * philtorch_b200 -- C ABI of the B200 (sm_100a) linear-recurrence kernels.
 *
 * Drop-in boundary for the differentiable linear-recurrence path of the reference project
 * (philtorch): the functions below are what a binding of that path's native ops would call.
 * Plain pointers and sizes only; no torch types.  All data pointers are DEVICE pointers to
 * dense row-major arrays; every call is asynchronous on `stream`, allocates nothing and
 * synchronises nothing.
 *
 * Common conventions
 *   dtype        PTB_F32 or PTB_F64; all arrays of a call share it.  The first-order recurrences
 *                (ptb_lti_recur_*, ptb_lpv_recur_fwd / _bwd) also take PTB_C64 / PTB_C128: arrays of
 *                interleaved {re, im} pairs, element counts unchanged; their adjoint uses conj(a) and
 *                grad_a = sum g[t] conj(y[t-1]) as the reference's autograd Function does
 *                (philtorch/lti/recur.py:31-57).
 *                They also take PTB_F16 / PTB_BF16 (the reference dispatches both,
 *                philtorch/csrc/lti_recur.cu:135-136, philtorch/csrc/host_recurN.cpp:259-260): every
 *                array of the call holds 2-byte floats, the recurrence runs in float32 registers and
 *                each result is rounded once.  These need rows that qualify for bulk copies (all
 *                base pointers 16-byte aligned, T a multiple of 8), else PTB_ERR_ARG.
 *   recurrence   y[-1] := zi, y[t] = A[t] * y[t-1] + x[t], t = 0..T-1: the coefficient with time
 *                index t multiplies the PREVIOUS state (philtorch/csrc/host_recurN.cpp:254-255).
 *   *_batched    1: the array has a leading batch axis of length B; 0: one copy shared by all rows.
 *   workspace    scratch of at least ptb_workspace_bytes(B, T) bytes, 256-byte aligned, private to
 *                the call until it completes (tile tickets, look-back flags, per-tile carries).
 *   status       device uint32, sticky error bits OR-ed in by the kernels when a bounded device
 *                wait expires (never cleared by the library); read it with ptb_read_status.
 *                May be NULL.
 *   return       PTB_OK or a PTB_ERR_* code; nothing was launched on error.
 */
#ifndef PHILTORCH_B200_H
#define PHILTORCH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* ptb_stream_t; /* a cudaStream_t */

enum { PTB_F32 = 0, PTB_F64 = 1,
       PTB_C64 = 2, PTB_C128 = 3, /* interleaved {re, im}; first-order recurrences only */
       PTB_F16 = 4, PTB_BF16 = 5  /* 2-byte arrays, float32 arithmetic; first-order recurrences only */ };
enum {
  PTB_OK = 0,
  PTB_ERR_ARG = 1,       /* null pointer, negative size, unknown dtype */
  PTB_ERR_WORKSPACE = 2, /* workspace missing, misaligned or too small */
  PTB_ERR_CUDA = 3,      /* a CUDA runtime call failed (see ptb_last_cuda_error) */
  PTB_ERR_TOO_LARGE = 4, /* more than 2^32-2 tiles */
  PTB_ERR_SCRATCH_LIMIT = 5 /* ptb_lpv_recur_fwd_static: problem larger than its built-in scratch */
};

const char* ptb_version(void);
const char* ptb_error_string(int code);
/* cudaError_t of the last failing runtime call made by this library on the calling thread. */
int ptb_last_cuda_error(void);

/* Upper bound of the scratch any entry point needs for B rows of T samples. */
int64_t ptb_workspace_bytes(int64_t B, int64_t T);

/* Copies *status to the host after synchronising `stream` (the only blocking call). */
int ptb_read_status(const uint32_t* status, ptb_stream_t stream, uint32_t* host_out);

/* ---- failure detection ----------------------------------------------------------------------
 * Every device-side wait of the kernels (look-back records of other CTAs, shared-memory barriers)
 * is bounded in time; when a bound expires the kernel sets a bit in `status`, finishes its copies
 * and runs to completion, so the context stays usable.  The bound is 2000 ms by default. */
int ptb_set_wait_limit_ms(int64_t ms);
/* ptb_lpv_recur2_fwd runs on one of two kernels: small CTAs (several per SM) from this many rows on,
 * else one large CTA per SM.  Default 48; process-wide; meant for tests and tuning. */
int ptb_lpv_recur2_set_small_cta_min_rows(int64_t rows);
/* Self-test of that path without faulting anything: runs the first-order forward kernel on two
 * tiles of which the FIRST IS NEVER PROCESSED, so the second one's look-back waits for a record
 * that nothing writes, gives up after the wait limit and reports kErrLookbackTimeout (bit 0) in
 * `status`.  buf: device scratch of at least ptb_selftest_wait_expiry_elems() floats (contents
 * irrelevant, 16-byte aligned); workspace as for the other entry points with B = 1,
 * T = that many samples. */
int64_t ptb_selftest_wait_expiry_elems(void);
int ptb_selftest_wait_expiry(void* workspace, int64_t workspace_bytes, void* buf, int64_t buf_elems,
                             uint32_t* status, ptb_stream_t stream);

/* ---- first-order, time-invariant ------------------------------------------------------------
 * Replaces op philtorch::lti_recur(a, zi, x) -> y
 *   (philtorch/csrc/host_recur2.cpp:170, CPU kernel philtorch/csrc/host_lti_recur.cpp:42-80,
 *    CUDA philtorch/csrc/lti_recur.cu:113-158).
 * a: (B,) if a_batched else (1,); zi: (B,) if zi_batched else (1,); x, y: (B,T);
 * zf: optional (B,), receives y[:, T-1]. */
int ptb_lti_recur_fwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* x, void* y, void* zf, void* workspace,
                      int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* Fused adjoint of the above; replaces LTIRecurrence.backward (philtorch/lti/recur.py:25-59) and
 * _lti_recur_backward (philtorch/__init__.py:115-148), which run the forward op on flipped copies.
 *   g[t] = a*g[t+1] + gy[t];  grad_x = g;  grad_zi = a*g[0];
 *   grad_a = sum_t y[t-1]*g[t] per row, summed over rows as well when !a_batched.
 * y: forward output (B,T); gy: (B,T); g_in: optional (B,), an adjoint state a*g[T] entering from the
 * right (rows that continue on another device); grad_x: (B,T), optional (NULL: not written, 4 bytes
 * per sample less traffic when only coefficient gradients are wanted); grad_a: optional, (B,) or (1,);
 * grad_zi: optional (B,). */
int ptb_lti_recur_bwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* y, const void* gy, const void* g_in, void* grad_x,
                      void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream);

/* Reverse-time first-order time-invariant recurrence fused with a three-term combination: the
 * second pass of the symmetric (causal + anticausal) filters, e.g. the cubic-spline prefilter of
 * philtorch/lti/interp.py:23-57, which the reference evaluates on a mirrored copy of the signal.
 *   g[t]   = x[t] + a * g[t+1],  g[T-1] = x[T-1] + g_in[row]   (g_in may be NULL: 0)
 *   out[t] = scale * (g[t] + second[t] - x[t])
 *   first_state (may be NULL) receives a * g[0] per row.
 * a: (B,) when a_batched, else one value; x, second, out: (B,T).  float32 / float64. */
int ptb_lti_recur_reverse_fused(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* x,
                                const void* second, const void* g_in, double scale, void* out, void* first_state,
                                void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* ---- first-order, per-sample coefficients ---------------------------------------------------
 * Replaces philtorch.lpv.linear_recurrence (philtorch/lpv/recur.py:20-101, pure PyTorch in the
 * reference) and the N = 1 case of op philtorch::recurN (philtorch/csrc/host_recurN.cpp:236-281).
 * a: (B,T) if a_batched else (T,). */
int ptb_lpv_recur_fwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* x, void* y, void* zf, void* workspace,
                      int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* Fused adjoint; replaces MatrixRecurrence.backward with M = 1 (philtorch/lpv/ssm.py:64-99),
 * which materialises transposed, rolled and flipped copies of the coefficients.
 *   g[t] = a[t+1]*g[t+1] + gy[t];  grad_x = g;  grad_a[b,t] = g[t]*y[t-1];  grad_zi = a[0]*g[0].
 * grad_a: optional, always (B,T) (per row; a caller with shared coefficients sums over rows);
 * grad_x: optional (NULL: not written). */
int ptb_lpv_recur_bwd(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                      int zi_batched, const void* y, const void* gy, const void* g_in, void* grad_x,
                      void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream);

/* The same adjoint for coefficients SHARED by the rows (a: (T,)), with the sum over the rows that the
 * reference's rule takes afterwards (philtorch/__init__.py:62-65) done on the way out: every row's
 * tiles of g[t]*y[t-1] are ADDED into the one grad_a (T,) by bulk reduce copies, so no (B,T) array of
 * per-row gradients is written and read again.  grad_a must be zero on entry (it is accumulated
 * into; the order of the additions is not fixed).  Needs rows that qualify for bulk copies (16-byte
 * aligned arrays, T*sizeof a multiple of 16), else PTB_ERR_ARG: use ptb_lpv_recur_bwd and sum. */
int ptb_lpv_recur_bwd_shared(int dtype, int64_t B, int64_t T, const void* a, const void* zi, int zi_batched,
                             const void* y, const void* gy, const void* g_in, void* grad_x, void* grad_a,
                             void* grad_zi, void* workspace, int64_t workspace_bytes, uint32_t* status,
                             ptb_stream_t stream);

/* ---- carry pass of a first-order scan whose time axis is split across devices --------------------
 * New with the time-sharded mode (the reference has no multi-device code).  Reads a shard's
 * coefficients and inputs once and returns, per row, the shard's total affine map
 *   carry[b] = { prod_t a[b,t],  end state of the shard started from zero }
 * without writing the sequence.  reverse = 0: the forward recurrence (x = inputs);
 * reverse = 1: the adjoint recurrence c[t] = a[t] (gy[t] + c[t+1]) run from the shard's end
 * (x = gy).  a: (B,T) if a_batched else (T,); carry: (B,2). */
int ptb_lpv_recur_carry(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* x,
                        int reverse, void* carry, void* workspace, int64_t workspace_bytes, uint32_t* status,
                        ptb_stream_t stream);

/* Local scan of a time shard and its total map in ONE pass: y = the recurrence started from a ZERO
 * state, carry[b] = { prod_t a[b,t], y[b,T-1] }.  With the true incoming state s of the shard,
 * y_true[t] = y[t] + (prod_{u<=t} a[u]) s; the correction dies out where the running product
 * underflows, so it is applied to a prefix only (philtorch_b200/sharded.py). */
int ptb_lpv_recur_fwd_carry(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* x, void* y,
                            void* carry, void* workspace, int64_t workspace_bytes, uint32_t* status,
                            ptb_stream_t stream);

/* ---- fix-up of a first-order scan cut into pieces along time --------------------------------------
 * New with the time-sharded mode (the reference has no multi-device code; its scalar recurrence is
 * philtorch/lpv/recur.py:20-101).  A row is cut into `world` time shards (one per device, in rank
 * order) and every shard into `nseg` segments of L samples, which the scan kernels treat as
 * B * nseg independent rows (kernel row r = b * nseg + j) started from a ZERO state.  These three
 * entry points turn such zero-start results into the results of the uncut recurrence without any
 * host round trip.  They need no workspace and are asynchronous on `stream`.
 *
 * ptb_lpv_recur_fold_maps: total map of every row's nseg pieces, out (B,2) = fold of maps (B,nseg,2)
 *   = {P_k, e_k}: s -> P_k s + e_k taken over k = 0..nseg-1 (reverse = 0) or nseg-1..0 (reverse = 1,
 *   the adjoint maps).  This is what a rank contributes to the all-gather over the shards.
 *
 * ptb_lpv_recur_fixup_fwd: for every kernel row, the state s entering it is folded from zi (B,), the
 *   shards' maps rank_maps (world,B,2) of ranks < rank (NULL when world == 1) and the maps
 *   seg_maps (B*nseg,2) of the segments before it; s is written to states (B*nseg,) and
 *   y[t] += (prod_{u<=t} a[u]) s is applied in place, block by block, until the running correction
 *   is exactly zero (it stays zero from there on, so stopping is exact).
 *   a: (B*nseg, L) if a_batched, else (L,) shared by the rows (then nseg must be 1).
 *
 * ptb_lpv_recur_fixup_bwd: the mirror image for the adjoint.  seg_maps (B*nseg,2) = {P_k, adjoint
 *   state leaving segment k on its left when nothing enters on its right}, rank_maps those of the
 *   shards; the adjoint state c entering a segment from its right is folded from the pieces to its
 *   right and  grad_x[t] += d[t],  grad_a[t] += d[t] y[t-1]  (y[-1] = states[r]),
 *   d[t] = c prod_{t<u<L} a[u], walking from the segment's end until d is exactly zero.
 *   grad_a: optional; (B*nseg, L), or (L,) with shared coefficients (atomic adds).
 *   grad_zi: optional (B,), receives the adjoint state leaving the shard on its left (the gradient
 *   of zi on rank 0). */
int ptb_lpv_recur_fold_maps(int dtype, int64_t B, int64_t nseg, const void* maps, int reverse, void* out,
                            ptb_stream_t stream);
int ptb_lpv_recur_fixup_fwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* a, int a_batched, void* y,
                            const void* seg_maps, const void* zi, const void* rank_maps, int rank, int world,
                            void* states, ptb_stream_t stream);
int ptb_lpv_recur_fixup_bwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* a, int a_batched,
                            const void* y, const void* states, const void* seg_maps, const void* rank_maps, int rank,
                            int world, void* grad_x, void* grad_a, void* grad_zi, ptb_stream_t stream);

/* ---- first-order forward without any caller-side or library-side allocation -----------------
 * No counterpart in the reference.  Same computation and arguments as ptb_lpv_recur_fwd for
 * PTB_F32 and PTB_F64 (the complex codes return PTB_ERR_ARG here, and
 * ptb_lpv_recur_fwd_static_max_tiles returns 0 for them), minus the workspace: the look-back scratch is a fixed 2 MiB array inside the library image (every GPU
 * that loads the library holds it until the process exits).  It is for callers whose processing
 * call is not allowed to allocate device memory -- a real-time audio or DSP callback, where
 * cudaMalloc may stall the whole device for an unbounded time, or a host application that has
 * handed all device memory to its own pool -- and that have no workspace to pass either.
 *   - Limit: B * ceil(T / tile) <= ptb_lpv_recur_fwd_static_max_tiles(dtype), the tile being 9216
 *     samples (fp32) or 4608 (fp64): about 9.6e8 fp32 samples of long rows.  Larger problems return
 *     PTB_ERR_SCRATCH_LIMIT and launch nothing.
 *   - The first call on each device looks up the array's device address (that device must be
 *     current, as for every entry point); make that first call before any stream capture.
 *   - All calls on a device share the one array; the part a call uses is cleared on `stream`
 *     before its kernel runs, and it keeps the last call's records afterwards.  Two calls that may
 *     overlap on the GPU (different streams without an ordering between them) race: serialise them.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine. */
int64_t ptb_lpv_recur_fwd_static_max_tiles(int dtype);
int ptb_lpv_recur_fwd_static(int dtype, int64_t B, int64_t T, const void* a, int a_batched, const void* zi,
                             int zi_batched, const void* x, void* y, void* zf, uint32_t* status,
                             ptb_stream_t stream);

/* ---- 2x2, time-invariant ---------------------------------------------------------------------
 * Replaces op philtorch::lti_recur2(A, zi, x) -> y (philtorch/csrc/host_recur2.cpp:166, CPU kernel
 * philtorch/csrc/host_lti_recurN.cpp:63-108, CUDA philtorch/csrc/lti_recur2.cu:66-113).
 * A: (B,2,2) if A_batched else (2,2), row-major; zi: (B,2); y: (B,T,2); zf: optional (B,2).
 * x: (B,T,2), or (B,T) when x_scalar (the sequence feeds state 0 only, as
 * philtorch/lti/ssm.py:187-191 does by zero-padding). */
int ptb_lti_recur2_fwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* x, int x_scalar, void* y, void* zf, void* workspace,
                       int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* Fused adjoint; replaces LTIMatrixRecurrence.backward (philtorch/lti/ssm.py:67-96) and
 * _lti_recurN_backward (philtorch/__init__.py:76-112).
 *   g[t] = A^T g[t+1] + gy[t];  grad_x = g (state 0 only when x_scalar, then (B,T));
 *   grad_zi = A^T g[0];  grad_A = sum_t g[t] (x) y[t-1], also summed over rows when !A_batched.
 * grad_A: optional, (B,2,2) or (2,2); g_in: optional (B,2); grad_zi: optional (B,2). */
int ptb_lti_recur2_bwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* y, const void* gy, const void* g_in, int x_scalar, void* grad_x,
                       void* grad_A, void* grad_zi, void* workspace, int64_t workspace_bytes,
                       uint32_t* status, ptb_stream_t stream);

/* ---- 2x2, per-sample coefficients --------------------------------------------------------------
 * Replaces op philtorch::recur2(A, zi, x) -> y (philtorch/csrc/host_recur2.cpp:164, CPU kernel
 * philtorch/csrc/host_recurN.cpp:236-281, CUDA philtorch/csrc/recur2.cu:69-117).
 * A: (B,T,2,2) if A_batched else (T,2,2). */
int ptb_lpv_recur2_fwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* x, int x_scalar, void* y, void* zf, void* workspace,
                       int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* Fused adjoint; replaces MatrixRecurrence.backward (philtorch/lpv/ssm.py:64-99) and
 * _recurN_backward (philtorch/__init__.py:34-73).
 *   g[t] = A[t+1]^T g[t+1] + gy[t];  grad_A[b,t] = g[t] (x) y[t-1];  grad_zi = A[0]^T g[0].
 * grad_A: optional, always (B,T,2,2) (per row; a caller with shared coefficients sums over rows). */
int ptb_lpv_recur2_bwd(int dtype, int64_t B, int64_t T, const void* A, int A_batched, const void* zi,
                       const void* y, const void* gy, const void* g_in, int x_scalar, void* grad_x,
                       void* grad_A, void* grad_zi, void* workspace, int64_t workspace_bytes,
                       uint32_t* status, ptb_stream_t stream);

/* The same adjoint for matrices SHARED by the rows (A: (T,2,2)), with the sum over the rows that the
 * reference's rule takes afterwards (philtorch/__init__.py:62-65) done on the way out: every row ADDS
 * its tiles of g[t] (x) y[t-1] into the one grad_A (T,2,2) by bulk reduce copies.  grad_A must be zero
 * on entry (the order of the additions is not fixed).  Needs arrays that qualify for bulk copies
 * (16-byte aligned, row length in bytes a multiple of 16), else PTB_ERR_ARG: use ptb_lpv_recur2_bwd
 * and sum. */
int ptb_lpv_recur2_bwd_shared(int dtype, int64_t B, int64_t T, const void* A, const void* zi, const void* y,
                              const void* gy, const void* g_in, int x_scalar, void* grad_x, void* grad_A,
                              void* grad_zi, void* workspace, int64_t workspace_bytes, uint32_t* status,
                              ptb_stream_t stream);

/* ---- 2x2, per-sample coefficients: rows cut into segments along time ------------------------------
 * No counterpart in the reference (its recurrence is philtorch/csrc/recur2.cu:69-117).  A handful of
 * long rows is cut into nseg segments of L samples each, which the scan kernel treats as B * nseg
 * independent rows (kernel row r = b * nseg + j) started from a ZERO state; the fix-up turns the
 * zero-start results into those of the uncut recurrence on the device.
 *
 * ptb_lpv_recur2_zero_carry: the forward scan of R kernel rows of T samples from a zero state
 *   (A (R,T,2,2), x (R,T,2) or (R,T) if x_scalar) -> y (R,T,2), end_state (R,2) = y[:, T-1], and
 *   tile_prod (R, ptb_lpv_recur2_carry_chunks(dtype, T), 4): the ordered product of the matrices
 *   of every tile of every row.  Workspace as for ptb_lpv_recur2_fwd.
 * ptb_lpv_recur2_fold_products: P (R,4) = the ordered product of a row's tile products
 *   = A[T-1] ... A[0].
 * ptb_lpv_recur2_fixup_fwd: the state s entering kernel row (b, j) is folded from zi (B,2) and the
 *   maps s -> P_i s + e_i of the segments before it; s goes to states (B*nseg,2) and
 *   y[t] += k[t], k[t] = A[t] k[t-1], k[-1] = s, is applied in place block by block until k is
 *   exactly zero (it stays zero from there on, so stopping is exact).
 * ptb_lpv_recur2_fixup_bwd: the mirror image for the adjoint.  e (B*nseg,2) = the adjoint state
 *   leaving every segment on its left when nothing enters on its right (grad_zi of
 *   ptb_lpv_recur2_bwd run on the kernel rows with zi = states); the state c entering a segment
 *   from its right is folded with P^T from the segments to its right, and
 *   grad_x[t] += d[t], grad_A[t] += d[t] (x) y[t-1] (y[-1] = states[r]), d[L-1] = c,
 *   d[t-1] = A[t]^T d[t], from the segment's end until d is exactly zero.  grad_x: (B*nseg,L,2), or
 *   (B*nseg,L) if x_scalar (component 0 only); grad_A optional; grad_zi (B,2) optional. */
int64_t ptb_lpv_recur2_carry_chunks(int dtype, int64_t T);
int ptb_lpv_recur2_zero_carry(int dtype, int64_t B, int64_t T, const void* A, const void* x, int x_scalar, void* y,
                              void* tile_prod, void* end_state, void* workspace, int64_t workspace_bytes,
                              uint32_t* status, ptb_stream_t stream);
int ptb_lpv_recur2_fold_products(int dtype, int64_t R, int64_t nchunks, const void* tile_prod, void* P,
                                 ptb_stream_t stream);
int ptb_lpv_recur2_fixup_fwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* A, void* y, const void* P,
                             const void* e, const void* zi, void* states, ptb_stream_t stream);
int ptb_lpv_recur2_fixup_bwd(int dtype, int64_t B, int64_t nseg, int64_t L, const void* A, const void* y,
                             const void* states, const void* P, const void* e, int x_scalar, void* grad_x,
                             void* grad_A, void* grad_zi, ptb_stream_t stream);

/* ---- dense N x N recurrences, 2 < N <= 8 ---------------------------------------------------------
 * Replace ops philtorch::recurN / philtorch::lti_recurN for state dimensions above two
 * (philtorch/csrc/host_recur2.cpp:165,168; CPU kernels philtorch/csrc/host_recurN.cpp:81-140,236-281 and
 * philtorch/csrc/host_lti_recurN.cpp:63-108; the reference has no GPU kernel for them).
 *   h[t] = A[t] h[t-1] + x[t],  h[-1] = zi.
 * A: row-major (N,N) matrices; A_timevar = 1: one per sample, (B,T,N,N) if A_batched else (T,N,N);
 * A_timevar = 0: constant along time, (B,N,N) if A_batched else (N,N).  zi (B,N); x, y (B,T,N);
 * zf optional (B,N).  N = 1 and 2 are accepted too (the dedicated kernels are faster).
 * Workspace: ptb_recur_n_workspace_bytes (the look-back records hold N x N maps).
 *
 * ptb_recur_n_adj is the scan inside the adjoint rules MatrixRecurrence.backward
 * (philtorch/lpv/ssm.py:64-99) and LTIMatrixRecurrence.backward (philtorch/lti/ssm.py:67-96):
 *   g[t] = gy[t] + c[t+1],  c[t] = A[t]^T g[t],  c[T] = g_in (optional (B,N), zero if NULL);
 * g (B,T,N) is grad_x, c0 (optional (B,N)) is grad_zi.  grad_A = g[t] (x) h[t-1] (summed over t for a
 * time-invariant A) is left to the caller: per row it is an (N x T)(T x N) matrix product.
 *
 * Constant matrices (A_timevar = 0) run on a policy whose maps carry only the N-vector offset and
 * their length; the linear part A^n comes from a per-row table of powers built in double at the
 * start of the call (csrc/mat_n_lti.cuh): N^2 work per sample instead of N^3.
 * ptb_recur_n_set_policy(1) sends them to the general kernels instead (process-wide; tests). */
int64_t ptb_recur_n_workspace_bytes(int dtype, int N, int64_t B, int64_t T);
int ptb_recur_n_set_policy(int policy);
/* grad_A of a constant matrix (LTIMatrixRecurrence.backward, philtorch/lti/ssm.py:84-92):
 *   partial[b][c] = sum over the samples t of time chunk c of  g[b,t] (x) h[b,t-1],   h[b,-1] = zi[b];
 * partial is (B, ptb_outer_prev_sum_chunks(B, T), N, N) and the caller adds the chunks of a row (and the
 * rows, when the matrix is shared).  Reads g and h (B,T,N) once; no workspace. */
int64_t ptb_outer_prev_sum_chunks(int64_t B, int64_t T);
int ptb_outer_prev_sum(int dtype, int N, int64_t B, int64_t T, const void* g, const void* h, const void* zi,
                       void* partial, ptb_stream_t stream);
int ptb_recur_n_fwd(int dtype, int N, int64_t B, int64_t T, const void* A, int A_batched, int A_timevar,
                    const void* zi, const void* x, void* y, void* zf, void* workspace, int64_t workspace_bytes,
                    uint32_t* status, ptb_stream_t stream);
int ptb_recur_n_adj(int dtype, int N, int64_t B, int64_t T, const void* A, int A_batched, int A_timevar,
                    const void* gy, const void* g_in, void* g, void* c0, void* workspace, int64_t workspace_bytes,
                    uint32_t* status, ptb_stream_t stream);

/* ---- one second-order section, transposed direct form II, scalar in / scalar out --------------
 * Replaces the whole lfilter(b, a, x, zi, form="tdf2") call stack for order <= 2
 * (philtorch/lti/filtering.py:211-333 -> philtorch/lti/ssm.py:386-510 -> op lti_recur2), a0 = 1:
 *   y[t] = h0[t-1] + b0 x[t];  h0[t] = -a1 h0[t-1] + h1[t-1] + (b1-b0 a1) x[t];
 *   h1[t] = -a2 h0[t-1] + (b2-b0 a2) x[t].
 * b: (B,3) / (3,), a: (B,2) / (2,) (coef_batched applies to both); zi: optional (B,2), zero if
 * NULL; x, y: (B,T); zf: optional (B,2) final state. */
int ptb_biquad_tdf2_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* zi, const void* x, void* y, void* zf, void* workspace,
                        int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);
/* The single-section entry points run on kernels that take the powers of the section's 2x2 matrix
 * from a per-row table built in double precision (policy 0, default); policy 1 forces the generic
 * 2x2 scan, which multiplies matrices in the data's precision and loses accuracy in float32 for
 * nearly double poles close to the unit circle.  Process-wide; meant for tests. */
int ptb_biquad_set_policy(int policy);

/* Adjoint of the section above (what autograd derives in the reference through the state-space
 * glue).  Reads gy, x and the forward OUTPUT y only; no state sequence is stored.
 * g_zf: optional (B,2) gradient w.r.t. zf; grad_x: (B,T); grad_b: optional (B,3)/(3,);
 * grad_a: optional (B,2)/(2,); grad_zi: optional (B,2). */
int ptb_biquad_tdf2_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* x, const void* y, const void* gy, const void* g_zf, void* grad_x,
                        void* grad_b, void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                        uint32_t* status, ptb_stream_t stream);

/* ---- cascade of K second-order sections, fused -------------------------------------------------
 * All K sections of a cascade in ONE pass over the signal per direction.  The reference runs a
 * cascade as K chained lfilter(b_k, a_k, ., form="tdf2") calls (philtorch/lti/filtering.py:304-317,
 * philtorch/lti/ssm.py:466-504); results equal that chain's up to floating-point re-association.
 *   K            number of sections: 2, 4, 6 or 8 (callers pad an odd cascade with the identity
 *                section b = {1,0,0}, a = {0,0} and split longer ones)
 *   b, a         (K,B,3), (K,B,2) when coef_batched, else (K,3), (K,2); a0 = 1 implicit
 *   zi / zf      optional (K,B,2) states of every section before the first / after the last sample
 *   x, y         (B,T)
 *   mid          optional (K-1,B,T): outputs of sections 0..K-2, needed by the backward pass for
 *                coefficient gradients
 * Backward: gy (B,T), g_zf optional (K,B,2) -> grad_x (B,T), grad_b / grad_a shaped like b / a
 * (optional, both or none; need x, mid, y), grad_zi optional (K,B,2).
 * Workspace: ptb_sos_cascade_workspace_bytes (holds the per-row table of matrix powers too).
 * Two families of kernels serve these entry points: chained ones (a tile takes over the end states
 * of its predecessor; fastest when there are at least as many rows as SMs) and decoupled ones
 * (look-back over aggregates; for few long rows).  ptb_sos_cascade_set_mode: 0 picks by batch size
 * (default), 1 / 2 force the decoupled / chained family (process-wide; meant for tests). */
int ptb_sos_cascade_set_mode(int mode);
int64_t ptb_sos_cascade_workspace_bytes(int dtype, int K, int64_t B, int64_t T);
int ptb_sos_cascade_fwd(int dtype, int K, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* zi, const void* x, void* y, void* mid, void* zf, void* workspace,
                        int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);
int ptb_sos_cascade_bwd(int dtype, int K, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                        const void* x, const void* mid, const void* y, const void* gy, const void* g_zf,
                        void* grad_x, void* grad_b, void* grad_a, void* grad_zi, void* workspace,
                        int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* ---- time-varying second-order filter, direct form II, fused -------------------------------------
 * philtorch.lpv.lfilter(b, a, x, zi, form="df2") for orders <= 2 (philtorch/lpv/filtering.py:288-313,
 * philtorch/lpv/ssm.py:413-500) in one pass per direction.
 *   b, a     per-sample coefficients (B,T,3), (B,T,2) when coef_batched, else (T,3), (T,2); a0 = 1
 *   zi / zf  optional (B,2);  x, y (B,T)
 *   hp       optional (B,T,2): the state before every sample, which the backward pass needs
 * Backward: gy (B,T), g_zf optional (B,2) -> grad_x (B,T), grad_b (B,T,3) and grad_a (B,T,2) PER
 * ROW (a caller with shared coefficients sums them over the rows), grad_zi optional (B,2).
 * Small CTAs with decoupled look-back: meant for batches of at least a few dozen rows.
 * Workspace: ptb_lpv_biquad_workspace_bytes. */
int64_t ptb_lpv_biquad_workspace_bytes(int dtype, int64_t B, int64_t T);
int ptb_lpv_biquad_df2_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* zi, const void* x, void* y, void* hp, void* zf, void* workspace,
                           int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);
int ptb_lpv_biquad_df2_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* x, const void* hp, const void* gy, const void* g_zf, void* grad_x,
                           void* grad_b, void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                           uint32_t* status, ptb_stream_t stream);
/* the same for form="tdf2" (philtorch/lpv/filtering.py:314-326): identical arguments */
int ptb_lpv_biquad_tdf2_fwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* zi, const void* x, void* y, void* hp, void* zf, void* workspace,
                           int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);
int ptb_lpv_biquad_tdf2_bwd(int dtype, int64_t B, int64_t T, const void* b, const void* a, int coef_batched,
                           const void* x, const void* hp, const void* gy, const void* g_zf, void* grad_x,
                           void* grad_b, void* grad_a, void* grad_zi, void* workspace, int64_t workspace_bytes,
                           uint32_t* status, ptb_stream_t stream);

/* ---- feedback comb filter (replaces the fold / transpose route of philtorch/lti/filtering.py:15-71,
 *      comb_filter) -------------------------------------------------------------------------------
 * y[t] = x[t] - a * y[t - delay] on the signal's own (B, N) layout: one thread per (row, phase).
 *   a         (B,) when a_batched, else one value
 *   zi_mode   0: zero initial state; 1: zi is (delay,) shared by the rows; 2: zi is (B, delay).
 *             zi[..., k] is the output k + 1 samples before the start (the reference's order).
 * Adjoint: grad_x (B, N); `partial` (may be NULL) receives B * ptb_comb_partial_blocks(delay)
 * partial sums of grad_a, row-major (row, block): grad_a[row] is the sum over its blocks, a shared
 * coefficient sums all of them; `grad_state` (may be NULL) receives the (B, delay) gradient of the
 * initial state in zi's order.  workspace and status are unused (no device-side waits) and may be NULL.
 * float32 / float64. */
int64_t ptb_comb_partial_blocks(int64_t delay);
/* Kernel family (process-wide; for tests and tuning), low byte of `policy`: 0 = slab kernels
 * (csrc/comb_slab.cuh: bands of neighbouring phases staged by tiled TMA copies) when delay and N are
 * multiples of 16 bytes of samples, the arrays are 16-byte aligned and the signal has at least 64 steps
 * of at least 64 phases, else one lane per phase (csrc/comb.cuh); 1 = lane per phase only; 2 / 3 / 4 =
 * slab kernels with bands of 256 / 128 / 64 phases wherever the layout allows.  Bits 8 and up: deepest
 * shared-memory ring of the slab kernels, 3..16 (0: the default, 4). */
int ptb_comb_set_policy(int policy);
int ptb_comb_fwd(int dtype, int64_t B, int64_t N, int64_t delay, const void* a, int a_batched, const void* zi,
                 int zi_mode, const void* x, void* y, void* workspace, int64_t workspace_bytes, uint32_t* status,
                 ptb_stream_t stream);
int ptb_comb_bwd(int dtype, int64_t B, int64_t N, int64_t delay, const void* a, int a_batched, const void* zi,
                 int zi_mode, const void* y, const void* gy, void* grad_x, void* partial, void* grad_state,
                 void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* ---- output map of a state-space model in its eigenbasis (replaces V w, the shifting
 *      concatenation and the complex product with C of philtorch/lti/ssm.py:805-830) ---------------
 * y[r, t] = sum_m coef[r, m] * w[r, m, t-1], with w[r, m, -1] = w0[r, m]; the real part only when
 * real_out.  ptb_modal_mix_fwd with w0 == NULL applies no delay: y[r, t] = sum_m coef[r, m] * w[r, m, t]
 * (the transposed input map, i.e. the gradient of a real input broadcast into the modes).
 * dtype PTB_C64 / PTB_C128: w (rows, M, N), w0 (rows, M), coef (M,) or (rows, M) when
 * coef_batched are complex; y and gy are (rows, N), real of the matching precision when real_out,
 * else complex.  Adjoint: grad_w (rows, M, N), grad_w0 (rows, M); `partial` (may be NULL) receives
 * rows * ptb_modal_mix_partial_blocks(N) * M complex partial sums of grad_coef, (row, block, m).
 * workspace and status are unused and may be NULL. */
int64_t ptb_modal_mix_partial_blocks(int64_t N);
int ptb_modal_mix_fwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* w, const void* w0, const void* coef,
                      int coef_batched, int real_out, void* y, void* workspace, int64_t workspace_bytes,
                      uint32_t* status, ptb_stream_t stream);
/* Input map for a real scalar input: u[r, m, t] = gain[r, m] * x[r, t]; x real (rows, N) of the
 * precision matching dtype (PTB_C64: float, PTB_C128: double), gain (M,) or (rows, M) complex,
 * u (rows, M, N) complex (philtorch/lti/ssm.py:783-788).  Its adjoint w.r.t. x is
 * ptb_modal_mix_fwd with w0 == NULL, coef = conj(gain) and real_out = 1. */
int ptb_modal_drive_fwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* x, const void* gain,
                        int gain_batched, void* u, void* workspace, int64_t workspace_bytes, uint32_t* status,
                        ptb_stream_t stream);
int ptb_modal_mix_bwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* w, const void* w0, const void* coef,
                      int coef_batched, int real_out, const void* gy, void* grad_w, void* grad_w0, void* partial,
                      void* workspace, int64_t workspace_bytes, uint32_t* status, ptb_stream_t stream);

/* ---- a state-space model with a scalar input and a real scalar output in its eigenbasis, fused ------
 * The whole of philtorch/lti/ssm.py:590-850 (diag_state_space) for that case in one read of x and one
 * write of y; the (rows, M, N) complex mode signals are never formed:
 *   w_m[t] = lam_m w_m[t-1] + gain_m x[t],  w_m[-1] = w0_m;   y[t] = Re(sum_m coef_m w_m[t-1]) + d x[t].
 * dtype PTB_F32 / PTB_F64 = the precision R of the real arrays x, y, d (rows,) (d may be NULL);
 * lam, gain, coef, w0, wf are (rows, M) complex of that precision, 1 <= M <= 8.
 * chk: (rows, ptb_modal_bank_tiles(M, N), M) complex; on return it holds the modes entering every
 * tile, which the adjoint needs (keep it until then).  wf (may be NULL): the modes after the last
 * sample.  Adjoint (gy real (rows, N); g_wf optional gradient of wf): grad_x (rows, N), grad_w0
 * (rows, M); `partial` receives (rows, tiles, 6 M + 1) reals per tile: {grad_gain, grad_lam, grad_coef}
 * as interleaved complex (M each) followed by grad_d -- the caller sums them over the tiles (a run of
 * consecutive tiles may store its sums with its last tile and zeros with the others); `need`
 * selects the parameter sums that are computed (bit 0 grad_gain, bit 1 grad_lam, bit 2 grad_coef); chk for
 * the adjoint is a second scratch array of the same size as the forward one (fwd_chk). */
int64_t ptb_modal_bank_tiles(int64_t M, int64_t N);
int ptb_modal_bank_fwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* x, const void* lam,
                       const void* gain, const void* coef, const void* d, const void* w0, void* y, void* wf,
                       void* chk, ptb_stream_t stream);
int ptb_modal_bank_bwd(int dtype, int64_t rows, int64_t M, int64_t N, const void* x, const void* lam,
                       const void* gain, const void* coef, const void* d, const void* fwd_chk, const void* gy,
                       const void* g_wf, int need, void* grad_x, void* grad_w0, void* partial, void* chk,
                       ptb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PHILTORCH_B200_H */
