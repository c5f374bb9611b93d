// Time-varying 2x2 recurrence  h[t] = A[t] h[t-1] + x[t]  (philtorch::recur2,
// philtorch/csrc/recur2.cu:69-117) in small CTAs: the single-pass scan with decoupled look-back of
// lpv_biquad.cuh (64 threads, several CTAs per SM, operands in registers, one tile prefetched)
// with the plain matrix recurrence as the per-sample step.  Batches of a few dozen rows and more
// run faster here than on the one-CTA-per-SM engine (the scan and look-back latency of one tile
// overlaps other tiles' arithmetic); the host picks.
#pragma once
#include "lpv_biquad.cuh"

namespace ptb {

template <class S>
struct SoSmallFwdParams {
  const S* A; int64_t a_row;   // (B,T,2,2) or (T,2,2): row stride 4T or 0
  const S* zi;                 // (B,2)
  const S* x;                  // (B,T) into state 0 (XS) or (B,T,2)
  S* y;                        // (B,T,2)
  S* zf;                       // optional (B,2)
  int64_t T;
  S* tile_prod;                // optional (B, nchunks, 4): the ordered product of every tile's matrices
};

template <class C, bool XS>
struct SoSmallFwdSmem {
  static constexpr int kA = 0;                               // [TILE][4]
  static constexpr int kX = kA + 4 * C::XB;                  // [TILE] or [TILE][2]
  static constexpr int kY = kX + (XS ? 1 : 2) * C::XB;       // [TILE][2] out
  static constexpr int kBar = kY + 2 * C::XB;                // u64 full[2]
  static constexpr int kMisc = kBar + 16;                    // u32 ticket[2], ok
  static constexpr int kHin = kMisc + 16;                    // S hin[2]
  static constexpr int kWtot = kHin + 16;                    // S wtot[NW][6]
  static constexpr int kTotal = kWtot + C::NW * 6 * 8 + 16;
};

template <class S> struct Vec4T;
template <> struct Vec4T<float> {
  static __device__ __forceinline__ void ld(const float* p, float* r) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    r[0] = q.x; r[1] = q.y; r[2] = q.z; r[3] = q.w;
  }
};
template <> struct Vec4T<double> {
  static __device__ __forceinline__ void ld(const double* p, double* r) {
    const double2 q = *reinterpret_cast<const double2*>(p), t = *reinterpret_cast<const double2*>(p + 2);
    r[0] = q.x; r[1] = q.y; r[2] = t.x; r[3] = t.y;
  }
};

template <class S, class C, bool XS>
__global__ void __launch_bounds__(C::NT, C::MINB)
so_small_fwd_kernel(const SoSmallFwdParams<S> p, const Workspace ws, const uint32_t B, const uint32_t nchunks,
                    const uint32_t ntiles, const int bulk, const uint64_t wait_ns) {
  using L = SoSmallFwdSmem<C, XS>;
  using V2 = typename Vec2T<S>::type;
  constexpr int SPT = C::SPT, TILE = C::TILE, NT = C::NT, XW = XS ? 1 : 2;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBar);
  volatile uint32_t* sm_ticket = reinterpret_cast<volatile uint32_t*>(smem + L::kMisc);
  volatile uint32_t* sm_ok = sm_ticket + 2;
  S* sm_hin = reinterpret_cast<S*>(smem + L::kHin);
  S* sm_wtot = reinterpret_cast<S*>(smem + L::kWtot);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    fence_mbar_init();
  }
  __syncthreads();
  auto coords = [&](uint32_t ticket, uint32_t& chunk, uint32_t& row, int64_t& t0, int& nvalid) {
    chunk = ticket / B;
    row = ticket - chunk * B;
    t0 = (int64_t)chunk * TILE;
    const int64_t rem = p.T - t0;
    nvalid = rem < (int64_t)TILE ? (int)rem : TILE;
  };
  auto issue = [&](int s, uint32_t ticket) {
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    mbar_arrive_expect_tx(&full[s], (4 + XW) * bytes);
    bulk_g2s(smem + L::kA, p.A + (int64_t)row * p.a_row + 4 * t0, 4 * bytes, &full[s]);
    bulk_g2s(smem + L::kX, p.x + ((int64_t)row * p.T + t0) * XW, XW * bytes, &full[s]);
  };
  if (tid == 0) {
    const uint32_t t = atomicAdd(ws.ticket, 1u);
    sm_ticket[0] = t < ntiles ? t : kNoTile;
    if (t < ntiles && bulk) issue(0, t);
  }
  __syncthreads();

  for (uint32_t n = 0;; ++n) {
    const int s = n & 1;
    const uint32_t ticket = sm_ticket[s];
    if (ticket == kNoTile) break;
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    const uint32_t nbytes = (uint32_t)nvalid * sizeof(S);
    if (bulk) {
      if (tid == 0) {
        const bool ok = mbar_wait_bounded(&full[s], (n >> 1) & 1u, wait_ns);
        if (!ok) atomicOr(ws.error, kErrLoadTimeout);
        *sm_ok = ok ? 1u : 0u;
      }
    } else {
      auto copy = [&](int off, const S* g, uint32_t words) {
        const uint32_t* gg = reinterpret_cast<const uint32_t*>(g);
        uint32_t* d = reinterpret_cast<uint32_t*>(smem + off);
        for (uint32_t w = tid; w < words; w += NT) d[w] = __ldg(gg + w);
      };
      copy(L::kA, p.A + (int64_t)row * p.a_row + 4 * t0, 4 * nbytes / 4);
      copy(L::kX, p.x + ((int64_t)row * p.T + t0) * XW, XW * nbytes / 4);
      if (tid == 0) *sm_ok = 1u;
    }
    __syncthreads();
    if (*sm_ok == 0u) {   // results are invalid from here on: stop taking work
      if (tid == 0) sm_ticket[s ^ 1] = kNoTile;
      __syncthreads();
      continue;
    }
    if (bulk) mbar_test_wait(&full[s], (n >> 1) & 1u);   // every thread observes the completed phase itself

    int nv = nvalid - tid * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    S A[SPT][4], x0[SPT], x1[SPT];
    {
      const S* pa = reinterpret_cast<const S*>(smem + L::kA) + tid * SPT * 4;
      const S* px = reinterpret_cast<const S*>(smem + L::kX) + tid * SPT * XW;
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        Vec4T<S>::ld(pa + 4 * j, A[j]);
        if (XS) { x0[j] = px[j]; x1[j] = S(0); }
        else { const V2 v = reinterpret_cast<const V2*>(px)[j]; x0[j] = v.x; x1[j] = v.y; }
      }
    }
    __syncthreads();   // everyone holds its samples: the tile buffers are free
    if (tid == 0) {    // fetch the tile after this one
      const uint32_t t = atomicAdd(ws.ticket, 1u);
      sm_ticket[s ^ 1] = t < ntiles ? t : kNoTile;
      if (t < ntiles && bulk) {
        fence_proxy_async_smem();
        issue(s ^ 1, t);
      }
    }
    // phase A: my samples as one affine map (samples beyond the end of the row are skipped)
    S m[6] = {S(1), S(0), S(0), S(1), S(0), S(0)};
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      if (j < nv) {
        const S n0 = A[j][0] * m[0] + A[j][1] * m[2], n1 = A[j][0] * m[1] + A[j][1] * m[3];
        const S n2 = A[j][2] * m[0] + A[j][3] * m[2], n3 = A[j][2] * m[1] + A[j][3] * m[3];
        const S n4 = A[j][0] * m[4] + A[j][1] * m[5] + x0[j], n5 = A[j][2] * m[4] + A[j][3] * m[5] + x1[j];
        m[0] = n0; m[1] = n1; m[2] = n2; m[3] = n3; m[4] = n4; m[5] = n5;
      }
    }
    affine_warp_scan<S>(m, lane);
    S e[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) e[i] = __shfl_up_sync(0xffffffffu, m[i], 1);
    if (lane == 0) { e[0] = S(1); e[1] = S(0); e[2] = S(0); e[3] = S(1); e[4] = S(0); e[5] = S(0); }
    if (lane == 31) {
#pragma unroll
      for (int i = 0; i < 6; ++i) sm_wtot[warp * 6 + i] = m[i];
    }
    if (tid == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous tile's outputs have left
    __syncthreads();
    if (p.tile_prod != nullptr && tid == NT - 1) {   // rows cut into segments: the fix-up needs the segment's matrix
      S q0 = S(1), q1 = S(0), q2 = S(0), q3 = S(1);
      for (int w = 0; w < C::NW; ++w) {
        const S* t = sm_wtot + w * 6;
        const S n0 = t[0] * q0 + t[1] * q2, n1 = t[0] * q1 + t[1] * q3;
        const S n2 = t[2] * q0 + t[3] * q2, n3 = t[2] * q1 + t[3] * q3;
        q0 = n0; q1 = n1; q2 = n2; q3 = n3;
      }
      S* o = p.tile_prod + ((int64_t)row * nchunks + chunk) * 4;
      o[0] = q0; o[1] = q1; o[2] = q2; o[3] = q3;
    }
    if (warp == 0) {
      S z0 = S(0), z1 = S(0);
      if (chunk == 0 && p.zi != nullptr) { z0 = __ldg(p.zi + (int64_t)row * 2); z1 = __ldg(p.zi + (int64_t)row * 2 + 1); }
      const typename LpvLb<S>::State hin =
          lpv_tile_state<S, C::NW>(ws, sm_wtot, ticket, chunk, nchunks, B, lane, z0, z1, wait_ns);
      if (lane == 0) { sm_hin[0] = hin.v[0]; sm_hin[1] = hin.v[1]; }
    }
    __syncthreads();
    S h0 = sm_hin[0], h1 = sm_hin[1];
    for (int w = 0; w < warp; ++w) {
      const S* t = sm_wtot + w * 6;
      const S g0 = t[0] * h0 + t[1] * h1 + t[4], g1 = t[2] * h0 + t[3] * h1 + t[5];
      h0 = g0; h1 = g1;
    }
    {
      const S g0 = e[0] * h0 + e[1] * h1 + e[4], g1 = e[2] * h0 + e[3] * h1 + e[5];
      h0 = g0; h1 = g1;
    }
    // phase B: replay; the states after every sample are the output
    {
      V2* py = reinterpret_cast<V2*>(smem + L::kY) + tid * SPT;
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        if (j < nv) {
          const S n0 = A[j][0] * h0 + A[j][1] * h1 + x0[j], n1 = A[j][2] * h0 + A[j][3] * h1 + x1[j];
          h0 = n0; h1 = n1;
          V2 hv; hv.x = h0; hv.y = h1;
          py[j] = hv;
        }
      }
    }
    if (p.zf != nullptr && nv > 0 && (t0 + (int64_t)tid * SPT + nv == p.T)) {
      p.zf[(int64_t)row * 2] = h0;
      p.zf[(int64_t)row * 2 + 1] = h1;
    }
    S* gy = p.y + ((int64_t)row * p.T + t0) * 2;
    if (bulk) {
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        bulk_s2g(gy, smem + L::kY, 2 * nbytes);
        bulk_commit();
      }
    } else {
      __syncthreads();
      const uint32_t* sy = reinterpret_cast<const uint32_t*>(smem + L::kY);
      uint32_t* oy = reinterpret_cast<uint32_t*>(gy);
      for (uint32_t w = tid; w < 2 * nbytes / 4; w += NT) oy[w] = sy[w];
      __syncthreads();
    }
  }
  if (tid == 0) bulk_wait_all();
}

// ------------------------------------------------------------------------------------ backward
// Adjoint of the recurrence with the carried quantity c[t] = A[t]^T g[t] in descending time
// (g[t] = gy[t] + c[t+1]; grad_x = g; grad_A[t] = g[t] (x) h[t-1]; grad_zi = c[0];
// philtorch/lpv/ssm.py:64-99).  The operands stay in shared memory and the gradients replace them
// in place (every thread only touches its own samples).
template <class S>
struct SoSmallBwdParams {
  const S* A; int64_t a_row;
  const S* zi;       // (B,2): h[-1], for grad_A[0]
  const S* y;        // forward states (B,T,2), needed only when grad_A is wanted
  const S* gy;       // (B,T,2)
  const S* g_in;     // optional (B,2): c entering from the right end
  S* grad_x;         // (B,T,2), or (B,T) when XS
  S* grad_A;         // optional (B,T,2,2); (T,2,2) when gA_shared
  S* grad_zi;        // optional (B,2)
  int64_t T;
  int gA_shared;     // the rows ADD their tiles of grad_A into one (T,2,2) array (bulk path only)
};

template <class C, bool XS>
struct SoSmallBwdSmem {
  static constexpr int kG = 0;                               // [TILE][2]  gy in, grad_x out (vector x)
  static constexpr int kA = kG + 2 * C::XB;                  // [TILE][4]  A in, grad_A out
  static constexpr int kY = kA + 4 * C::XB;                  // [TILE][2]  forward states
  static constexpr int kGX = kY + 2 * C::XB;                 // [TILE]     grad_x out (scalar x)
  static constexpr int kBar = kGX + (XS ? 1 : 0) * C::XB;    // u64 full
  static constexpr int kMisc = kBar + 16;                    // u32 ticket, ok
  static constexpr int kHin = kMisc + 16;                    // S hin[2], yprev[2]
  static constexpr int kWtot = kHin + 32;                    // S wtot[NW][6]
  static constexpr int kTotal = kWtot + C::NW * 6 * 8 + 16;
};

template <class S, class C, bool XS>
__global__ void __launch_bounds__(C::NT, C::MINB)
so_small_bwd_kernel(const SoSmallBwdParams<S> p, const Workspace ws, const uint32_t B, const uint32_t nchunks,
                    const uint32_t ntiles, const int bulk, const uint64_t wait_ns) {
  using L = SoSmallBwdSmem<C, XS>;
  using V2 = typename Vec2T<S>::type;
  constexpr int SPT = C::SPT, TILE = C::TILE, NT = C::NT;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBar);
  volatile uint32_t* sm_ticket = reinterpret_cast<volatile uint32_t*>(smem + L::kMisc);
  volatile uint32_t* sm_ok = sm_ticket + 1;
  S* sm_hin = reinterpret_cast<S*>(smem + L::kHin);
  S* sm_wtot = reinterpret_cast<S*>(smem + L::kWtot);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tpos = NT - 1 - tid;   // time runs against the scan order
  const bool want_gA = p.grad_A != nullptr;

  if (tid == 0) {
    mbar_init(full, 1);
    fence_mbar_init();
  }
  __syncthreads();

  for (uint32_t n = 0;; ++n) {
    if (tid == 0) {
      const uint32_t t = atomicAdd(ws.ticket, 1u);
      *sm_ticket = t < ntiles ? t : kNoTile;
    }
    __syncthreads();
    const uint32_t ticket = *sm_ticket;
    if (ticket == kNoTile) break;
    const uint32_t chunk = ticket / B, row = ticket - chunk * B;
    const int64_t t0 = (int64_t)(nchunks - 1 - chunk) * TILE;
    const int64_t rem = p.T - t0;
    const int nvalid = rem < (int64_t)TILE ? (int)rem : TILE;
    const uint32_t nbytes = (uint32_t)nvalid * sizeof(S);
    const int64_t off = (int64_t)row * p.T + t0;
    const S* gA_ = p.A + (int64_t)row * p.a_row + 4 * t0;
    if (bulk) {
      if (tid == 0) {
        bulk_wait_read_all();   // the previous tile's gradients have left the buffers
        fence_proxy_async_smem();
        mbar_arrive_expect_tx(full, (want_gA ? 8 : 6) * nbytes);
        bulk_g2s(smem + L::kG, p.gy + 2 * off, 2 * nbytes, full);
        bulk_g2s(smem + L::kA, gA_, 4 * nbytes, full);
        if (want_gA) bulk_g2s(smem + L::kY, p.y + 2 * off, 2 * nbytes, full);
        const bool ok = mbar_wait_bounded(full, n & 1u, wait_ns);
        if (!ok) atomicOr(ws.error, kErrLoadTimeout);
        *sm_ok = ok ? 1u : 0u;
      }
    } else {
      auto copy = [&](int o, const S* g, uint32_t words) {
        const uint32_t* gg = reinterpret_cast<const uint32_t*>(g);
        uint32_t* d = reinterpret_cast<uint32_t*>(smem + o);
        for (uint32_t w = tid; w < words; w += NT) d[w] = __ldg(gg + w);
      };
      copy(L::kG, p.gy + 2 * off, 2 * nbytes / 4);
      copy(L::kA, gA_, 4 * nbytes / 4);
      if (want_gA) copy(L::kY, p.y + 2 * off, 2 * nbytes / 4);
      if (tid == 0) *sm_ok = 1u;
    }
    if (tid == 0 && want_gA) {   // h[t0-1]: the state before the tile's first sample
      const S* q = t0 > 0 ? p.y + 2 * (off - 1) : p.zi + (int64_t)row * 2;
      sm_hin[2] = __ldg(q);
      sm_hin[3] = __ldg(q + 1);
    }
    __syncthreads();
    if (*sm_ok == 0u) break;   // results are invalid; nothing of this CTA is in flight
    if (bulk) mbar_test_wait(full, n & 1u);

    int nv = nvalid - tpos * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    S* pa = reinterpret_cast<S*>(smem + L::kA) + tpos * SPT * 4;
    V2* pg = reinterpret_cast<V2*>(smem + L::kG) + tpos * SPT;
    const V2* py = reinterpret_cast<const V2*>(smem + L::kY) + tpos * SPT;

    // phase A: c_out = A_j^T (gy_j + c_in) over my samples, descending
    S m[6] = {S(1), S(0), S(0), S(1), S(0), S(0)};
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      if (j < nv) {
        S a[4];
        Vec4T<S>::ld(pa + 4 * j, a);
        const V2 g = pg[j];
        const S u0 = m[4] + g.x, u1 = m[5] + g.y;
        const S n0 = a[0] * m[0] + a[2] * m[2], n1 = a[0] * m[1] + a[2] * m[3];
        const S n2 = a[1] * m[0] + a[3] * m[2], n3 = a[1] * m[1] + a[3] * m[3];
        m[0] = n0; m[1] = n1; m[2] = n2; m[3] = n3;
        m[4] = a[0] * u0 + a[2] * u1;
        m[5] = a[1] * u0 + a[3] * u1;
      }
    }
    affine_warp_scan<S>(m, lane);
    S e[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) e[i] = __shfl_up_sync(0xffffffffu, m[i], 1);
    if (lane == 0) { e[0] = S(1); e[1] = S(0); e[2] = S(0); e[3] = S(1); e[4] = S(0); e[5] = S(0); }
    if (lane == 31) {
#pragma unroll
      for (int i = 0; i < 6; ++i) sm_wtot[warp * 6 + i] = m[i];
    }
    __syncthreads();
    if (warp == 0) {
      S z0 = S(0), z1 = S(0);
      if (chunk == 0 && p.g_in) { z0 = __ldg(p.g_in + (int64_t)row * 2); z1 = __ldg(p.g_in + (int64_t)row * 2 + 1); }
      const typename LpvLb<S>::State hin =
          lpv_tile_state<S, C::NW>(ws, sm_wtot, ticket, chunk, nchunks, B, lane, z0, z1, wait_ns);
      if (lane == 0) { sm_hin[0] = hin.v[0]; sm_hin[1] = hin.v[1]; }
    }
    __syncthreads();
    S c0 = sm_hin[0], c1 = sm_hin[1];
    for (int w = 0; w < warp; ++w) {
      const S* t = sm_wtot + w * 6;
      const S g0 = t[0] * c0 + t[1] * c1 + t[4], g1 = t[2] * c0 + t[3] * c1 + t[5];
      c0 = g0; c1 = g1;
    }
    {
      const S g0 = e[0] * c0 + e[1] * c1 + e[4], g1 = e[2] * c0 + e[3] * c1 + e[5];
      c0 = g0; c1 = g1;
    }
    // phase B: replay; gradients in place
    S yp0 = S(0), yp1 = S(0);   // h before my first sample
    if (want_gA && nv > 0) {
      if (tpos > 0) { const V2 v = py[-1]; yp0 = v.x; yp1 = v.y; }
      else { yp0 = sm_hin[2]; yp1 = sm_hin[3]; }
    }
    S* pgx = reinterpret_cast<S*>(smem + L::kGX) + tpos * SPT;
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      if (j < nv) {
        S a[4];
        Vec4T<S>::ld(pa + 4 * j, a);
        const V2 g = pg[j];
        const S g0 = g.x + c0, g1 = g.y + c1;
        if (XS) pgx[j] = g0;
        else { V2 gv; gv.x = g0; gv.y = g1; pg[j] = gv; }
        if (want_gA) {
          S y0 = yp0, y1 = yp1;
          if (j > 0) { const V2 v = py[j - 1]; y0 = v.x; y1 = v.y; }
          pa[4 * j] = g0 * y0; pa[4 * j + 1] = g0 * y1; pa[4 * j + 2] = g1 * y0; pa[4 * j + 3] = g1 * y1;
        }
        c0 = a[0] * g0 + a[2] * g1;
        c1 = a[1] * g0 + a[3] * g1;
      }
    }
    if (tid == NT - 1 && chunk + 1 == nchunks && p.grad_zi) {
      p.grad_zi[(int64_t)row * 2] = c0;
      p.grad_zi[(int64_t)row * 2 + 1] = c1;
    }
    S* ox = XS ? p.grad_x + off : p.grad_x + 2 * off;
    S* oa = want_gA ? p.grad_A + 4 * (p.gA_shared ? t0 : off) : nullptr;
    if (bulk) {
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        if (XS) bulk_s2g(ox, smem + L::kGX, nbytes);
        else bulk_s2g(ox, smem + L::kG, 2 * nbytes);
        if (want_gA) {
          if (!p.gA_shared) bulk_s2g(oa, smem + L::kA, 4 * nbytes);
          else if (sizeof(S) == 4) bulk_s2g_add_f32(oa, smem + L::kA, 4 * nbytes);
          else bulk_s2g_add_f64(oa, smem + L::kA, 4 * nbytes);
        }
        bulk_commit();
      }
    } else {
      __syncthreads();
      auto put = [&](S* g, int o, uint32_t words) {
        const uint32_t* sdat = reinterpret_cast<const uint32_t*>(smem + o);
        uint32_t* gg = reinterpret_cast<uint32_t*>(g);
        for (uint32_t w = tid; w < words; w += NT) gg[w] = sdat[w];
      };
      if (XS) put(ox, L::kGX, nbytes / 4);
      else put(ox, L::kG, 2 * nbytes / 4);
      if (want_gA) put(oa, L::kA, 4 * nbytes / 4);
    }
    __syncthreads();
  }
  if (tid == 0) bulk_wait_all();
}

}  // namespace ptb
