// Time-varying (parameter-varying) second-order filter, direct form II (and transposed direct form
// II, TDF2 = true: h' = A_t^T h + (b_t[1:] - b0_t a_t) x_t, y_t = h0 + b0_t x_t, adjoint likewise),
// scalar in and scalar out, with per-sample coefficients: the whole of
// philtorch.lpv.lfilter(form="df2" | "tdf2") for orders <= 2
// (philtorch/lpv/filtering.py:288-313 builds companion(a_t), C_t = b_t[1:] - b0_t a_t, D_t = b0_t;
// philtorch/lpv/ssm.py:413-500 runs  h_t = A_t h_{t-1} + e0 x_t,  y_t = C_t . h_{t-1} + D_t x_t
// as a dozen full passes over (B,T,2,2) / (B,T,2) tensors) in ONE pass per direction:
//     y[t]  = (b1 - b0 a1) h0 + (b2 - b0 a2) h1 + b0 x[t]        (h = state before sample t)
//     h0'   = -a1 h0 - a2 h1 + x[t],   h1' = h0
// Forward reads a (2), b (3), x and writes y and, for the backward pass, the states before every
// sample.  Backward (lam_t = dL/dh_t, descending time):
//     lam_{t-1} = A_t^T lam_t + C_t gy_t
//     grad_x = lam0 + b0 gy,  grad_C = gy h,  grad_a = -lam0 h - b0 grad_C,
//     grad_b0 = gy x - a . grad_C,  grad_b[1:] = grad_C
// all per sample, so nothing is reduced.
//
// Single-pass scan with decoupled look-back in small CTAs: a CTA takes one tile of one row
// (chunk-major tickets, as in scan_engine.cuh); every thread folds its SPT samples into a 2x2 affine
// map (phase A), the maps are scanned over the lanes and warps, warp 0 publishes the tile's
// aggregate and looks back over the row's earlier tiles (scan_engine.cuh's lookback: aggregates
// until an end state is met, bounded waits), publishes the tile's end state, and every thread
// replays its samples from its true state (phase B).
// SPT is odd: per-thread strides of 2 SPT, 3 SPT and SPT words make the 8-byte / 4-byte shared
// memory accesses conflict-free.  Small CTAs, several per SM, overlap one tile's scan latency with
// another tile's arithmetic.
#pragma once
#include "sos_chain.cuh"
#include "second_order.cuh"

namespace ptb {

// the look-back's view of the maps: second_order.cuh's 2x2 affine algebra
template <class S>
struct LpvLb : MatAffine<S> {
  static constexpr int SLOT_WORDS = Words<typename MatAffine<S>::Map>::W;
};

template <class S, int SPT_, int NT_, int MINB_>
struct LpvBqCfg {
  static_assert(SPT_ % 2 == 1, "odd per-thread sample count: conflict-free strided shared-memory accesses");
  static constexpr int SPT = SPT_, NT = NT_, NW = NT_ / 32, MINB = MINB_;
  static constexpr int TILE = NT * SPT;
  static constexpr int XB = TILE * (int)sizeof(S);   // bytes of a tile of a scalar array
  static constexpr int SLOT_WORDS = LpvLb<S>::SLOT_WORDS;
  static_assert(XB % 16 == 0, "bulk copies move multiples of 16 bytes");
};

template <class S> struct Vec2T;
template <> struct Vec2T<float> { using type = float2; };
template <> struct Vec2T<double> { using type = double2; };

// 2x2 affine maps {m00 m01 m10 m11 v0 v1}: apply `f` first, then `g`
template <class S>
__device__ __forceinline__ void affine_compose(const S* f, const S* g, S* r) {
  const S r0 = g[0] * f[0] + g[1] * f[2], r1 = g[0] * f[1] + g[1] * f[3];
  const S r2 = g[2] * f[0] + g[3] * f[2], r3 = g[2] * f[1] + g[3] * f[3];
  const S r4 = g[0] * f[4] + g[1] * f[5] + g[4], r5 = g[2] * f[4] + g[3] * f[5] + g[5];
  r[0] = r0; r[1] = r1; r[2] = r2; r[3] = r3; r[4] = r4; r[5] = r5;
}
// inclusive scan of the maps over the lanes of a warp
template <class S>
__device__ __forceinline__ void affine_warp_scan(S* m, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    S o[6];
#pragma unroll
    for (int i = 0; i < 6; ++i) o[i] = __shfl_up_sync(0xffffffffu, m[i], d);
    if (lane >= d) affine_compose<S>(o, m, m);
  }
}

// Warp 0, after the warps' totals are in shared memory: tile aggregate, look-back, end state.
// Returns (in every lane) the state entering the tile; zi: the row's initial state (chunk 0).
template <class S, int NW>
__device__ __forceinline__ typename LpvLb<S>::State lpv_tile_state(const Workspace& ws, const S* wtot, uint32_t ticket,
                                                                   uint32_t chunk, uint32_t nchunks, uint32_t B,
                                                                   int lane, S zi0, S zi1, uint64_t wait_ns) {
  using P = LpvLb<S>;
  typename P::Map agg = P::identity();
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    typename P::Map t;
#pragma unroll
    for (int i = 0; i < 6; ++i) t.v[i] = wtot[w * 6 + i];
    agg = P::compose(agg, t);
  }
  uint64_t* slot = ws.slots + (size_t)ticket * P::SLOT_WORDS;
  typename P::State hin;
  if (chunk == 0) {
    hin.v[0] = zi0; hin.v[1] = zi1;
  } else {
    if (lane == 0 && chunk + 1 < nchunks) slot_store(slot, agg, 1u);
    uint32_t failed = 0;
    hin = lookback<P>(0, ws, ticket, chunk, B, lane, failed, 8, wait_ns);
  }
  if (lane == 0 && chunk + 1 < nchunks) slot_store(slot, P::apply(agg, hin), 2u);
  return hin;
}

// ------------------------------------------------------------------------------------ forward
template <class S>
struct LpvBqFwdParams {
  const S* a; int64_t a_row;   // (B,T,2) or (T,2): row stride 2T or 0
  const S* b; int64_t b_row;   // (B,T,3) or (T,3): row stride 3T or 0
  const S* zi;                 // optional (B,2)
  const S* x;
  S* y;
  S* hp;                       // optional (B,T,2): the state before every sample (kept for the backward pass)
  S* zf;                       // optional (B,2)
  int64_t T;
};

template <class C>
struct LpvBqFwdSmem {
  static constexpr int kA = 0;                          // [TILE][2]
  static constexpr int kB = kA + 2 * C::XB;             // [TILE][3]
  static constexpr int kX = kB + 3 * C::XB;             // [TILE]
  static constexpr int kY = kX + C::XB;                 // [TILE]     out
  static constexpr int kH = kY + C::XB;                 // [TILE][2]  out
  static constexpr int kBar = kH + 2 * C::XB;           // u64 full[2]
  static constexpr int kMisc = kBar + 16;               // u32 ticket[2], ok
  static constexpr int kHin = kMisc + 16;               // S hin[2]
  static constexpr int kWtot = kHin + 16;               // S wtot[NW][6]
  static constexpr int kTotal = kWtot + C::NW * 6 * 8 + 16;
};

template <class S, class C, bool TDF2>
__global__ void __launch_bounds__(C::NT, C::MINB)
lpv_bq_fwd_kernel(const LpvBqFwdParams<S> p, const Workspace ws, const uint32_t B, const uint32_t nchunks,
                  const uint32_t ntiles, const int bulk, const uint64_t wait_ns) {
  using L = LpvBqFwdSmem<C>;
  using V2 = typename Vec2T<S>::type;
  constexpr int SPT = C::SPT, TILE = C::TILE, NT = C::NT;
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
  auto issue = [&](int s, uint32_t ticket) {   // one thread: bulk loads of a tile's a, b and x
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    mbar_arrive_expect_tx(&full[s], 6 * bytes);
    bulk_g2s(smem + L::kA, p.a + (int64_t)row * p.a_row + 2 * t0, 2 * bytes, &full[s]);
    bulk_g2s(smem + L::kB, p.b + (int64_t)row * p.b_row + 3 * t0, 3 * bytes, &full[s]);
    bulk_g2s(smem + L::kX, p.x + (int64_t)row * p.T + t0, bytes, &full[s]);
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
      copy(L::kA, p.a + (int64_t)row * p.a_row + 2 * t0, 2 * nbytes / 4);
      copy(L::kB, p.b + (int64_t)row * p.b_row + 3 * t0, 3 * nbytes / 4);
      copy(L::kX, p.x + (int64_t)row * p.T + t0, nbytes / 4);
      if (tid == 0) *sm_ok = 1u;
    }
    __syncthreads();
    if (*sm_ok == 0u) {   // results are invalid from here on: stop taking work
      if (tid == 0) sm_ticket[s ^ 1] = kNoTile;
      __syncthreads();
      continue;
    }
    if (bulk) mbar_test_wait(&full[s], (n >> 1) & 1u);   // every thread observes the completed phase itself

    // this thread's samples and coefficients; beyond the end of the row: zero input, identity-free
    // coefficients of zero (the states of such samples are never used)
    int nv = nvalid - tid * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    S a1[SPT], a2[SPT], c0[SPT], c1[SPT], d0[SPT], x[SPT];
    {
      const V2* pa = reinterpret_cast<const V2*>(smem + L::kA) + tid * SPT;
      const S* pb = reinterpret_cast<const S*>(smem + L::kB) + tid * SPT * 3;
      const S* px = reinterpret_cast<const S*>(smem + L::kX) + tid * SPT;
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        const V2 av = pa[j];
        const S b0 = pb[3 * j], b1 = pb[3 * j + 1], b2 = pb[3 * j + 2];
        const bool in = j < nv;
        a1[j] = in ? av.x : S(0);
        a2[j] = in ? av.y : S(0);
        d0[j] = in ? b0 : S(0);
        c0[j] = in ? b1 - b0 * av.x : S(0);
        c1[j] = in ? b2 - b0 * av.y : S(0);
        x[j] = in ? px[j] : S(0);
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
    // phase A: my samples as one affine map
    S m[6] = {S(1), S(0), S(0), S(1), S(0), S(0)};
#pragma unroll
    for (int j = 0; j < SPT; ++j) {
      if (!TDF2) {   // h' = [[-a1,-a2],[1,0]] h + [x, 0]
        const S n0 = -a1[j] * m[0] - a2[j] * m[2], n1 = -a1[j] * m[1] - a2[j] * m[3];
        const S n4 = -a1[j] * m[4] - a2[j] * m[5] + x[j];
        m[2] = m[0]; m[3] = m[1]; m[5] = m[4];
        m[0] = n0; m[1] = n1; m[4] = n4;
      } else {       // h' = [[-a1,1],[-a2,0]] h + [c0, c1] x
        const S n0 = -a1[j] * m[0] + m[2], n1 = -a1[j] * m[1] + m[3], n4 = -a1[j] * m[4] + m[5] + c0[j] * x[j];
        const S n2 = -a2[j] * m[0], n3 = -a2[j] * m[1], n5 = -a2[j] * m[4] + c1[j] * x[j];
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
    if (warp == 0) {
      S z0 = S(0), z1 = S(0);
      if (chunk == 0 && p.zi) { z0 = __ldg(p.zi + (int64_t)row * 2); z1 = __ldg(p.zi + (int64_t)row * 2 + 1); }
      const typename LpvLb<S>::State hin =
          lpv_tile_state<S, C::NW>(ws, sm_wtot, ticket, chunk, nchunks, B, lane, z0, z1, wait_ns);
      if (lane == 0) { sm_hin[0] = hin.v[0]; sm_hin[1] = hin.v[1]; }
    }
    __syncthreads();
    // state entering my warp, then my thread
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
    // phase B: replay; outputs to shared memory
    {
      S* py = reinterpret_cast<S*>(smem + L::kY) + tid * SPT;
      V2* ph = reinterpret_cast<V2*>(smem + L::kH) + tid * SPT;
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        if (j < nv) {
          if (p.hp) { V2 hv; hv.x = h0; hv.y = h1; ph[j] = hv; }
          if (!TDF2) {
            py[j] = c0[j] * h0 + c1[j] * h1 + d0[j] * x[j];
            const S n0 = -a1[j] * h0 - a2[j] * h1 + x[j];
            h1 = h0;
            h0 = n0;
          } else {
            py[j] = h0 + d0[j] * x[j];
            const S n0 = -a1[j] * h0 + h1 + c0[j] * x[j];
            h1 = -a2[j] * h0 + c1[j] * x[j];
            h0 = n0;
          }
        }
      }
    }
    if (p.zf != nullptr && nv > 0 && (t0 + (int64_t)tid * SPT + nv == p.T)) {
      p.zf[(int64_t)row * 2] = h0;
      p.zf[(int64_t)row * 2 + 1] = h1;
    }
    S* gy = p.y + (int64_t)row * p.T + t0;
    S* gh = p.hp ? p.hp + ((int64_t)row * p.T + t0) * 2 : nullptr;
    if (bulk) {
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        bulk_s2g(gy, smem + L::kY, nbytes);
        if (gh) bulk_s2g(gh, smem + L::kH, 2 * nbytes);
        bulk_commit();
      }
    } else {
      __syncthreads();
      const uint32_t* sy = reinterpret_cast<const uint32_t*>(smem + L::kY);
      uint32_t* oy = reinterpret_cast<uint32_t*>(gy);
      for (uint32_t w = tid; w < nbytes / 4; w += NT) oy[w] = sy[w];
      if (gh) {
        const uint32_t* sh = reinterpret_cast<const uint32_t*>(smem + L::kH);
        uint32_t* oh = reinterpret_cast<uint32_t*>(gh);
        for (uint32_t w = tid; w < 2 * nbytes / 4; w += NT) oh[w] = sh[w];
      }
      __syncthreads();
    }
  }
  if (tid == 0) bulk_wait_all();
}

// ------------------------------------------------------------------------------------ backward
template <class S>
struct LpvBqBwdParams {
  const S* a; int64_t a_row;
  const S* b; int64_t b_row;
  const S* x;
  const S* hp;     // (B,T,2) states before every sample, from the forward pass
  const S* gy;
  const S* g_in;   // optional (B,2): gradient w.r.t. the final state
  S* grad_x;
  S* grad_a;       // (B,T,2), per row even when the coefficients are shared
  S* grad_b;       // (B,T,3)
  S* grad_zi;      // optional (B,2)
  int64_t T;
};

template <class C>
struct LpvBqBwdSmem {
  static constexpr int kG = 0;                          // [TILE]     gy in, grad_x out
  static constexpr int kA = kG + C::XB;                 // [TILE][2]  a in, grad_a out
  static constexpr int kB = kA + 2 * C::XB;             // [TILE][3]  b in, grad_b out
  static constexpr int kX = kB + 3 * C::XB;             // [TILE]
  static constexpr int kH = kX + C::XB;                 // [TILE][2]
  static constexpr int kBar = kH + 2 * C::XB;           // u64 full
  static constexpr int kMisc = kBar + 16;               // u32 ticket, ok
  static constexpr int kHin = kMisc + 16;               // S hin[2]
  static constexpr int kWtot = kHin + 16;               // S wtot[NW][6]
  static constexpr int kTotal = kWtot + C::NW * 6 * 8 + 16;
};

template <class S, class C, bool TDF2>
__global__ void __launch_bounds__(C::NT, C::MINB)
lpv_bq_bwd_kernel(const LpvBqBwdParams<S> p, const Workspace ws, const uint32_t B, const uint32_t nchunks,
                  const uint32_t ntiles, const int bulk, const uint64_t wait_ns) {
  using L = LpvBqBwdSmem<C>;
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
    const S* ga_ = p.a + (int64_t)row * p.a_row + 2 * t0;
    const S* gb_ = p.b + (int64_t)row * p.b_row + 3 * t0;
    const int64_t off = (int64_t)row * p.T + t0;
    if (bulk) {
      if (tid == 0) {
        bulk_wait_read_all();   // the previous tile's gradients have left the buffers
        fence_proxy_async_smem();
        mbar_arrive_expect_tx(full, 9 * nbytes);
        bulk_g2s(smem + L::kG, p.gy + off, nbytes, full);
        bulk_g2s(smem + L::kA, ga_, 2 * nbytes, full);
        bulk_g2s(smem + L::kB, gb_, 3 * nbytes, full);
        bulk_g2s(smem + L::kX, p.x + off, nbytes, full);
        bulk_g2s(smem + L::kH, p.hp + 2 * off, 2 * nbytes, full);
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
      copy(L::kG, p.gy + off, nbytes / 4);
      copy(L::kA, ga_, 2 * nbytes / 4);
      copy(L::kB, gb_, 3 * nbytes / 4);
      copy(L::kX, p.x + off, nbytes / 4);
      copy(L::kH, p.hp + 2 * off, 2 * nbytes / 4);
      if (tid == 0) *sm_ok = 1u;
    }
    __syncthreads();
    if (*sm_ok == 0u) break;   // results are invalid; nothing of this CTA is in flight
    if (bulk) mbar_test_wait(full, n & 1u);

    int nv = nvalid - tpos * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    V2* pa = reinterpret_cast<V2*>(smem + L::kA) + tpos * SPT;
    S* pb = reinterpret_cast<S*>(smem + L::kB) + tpos * SPT * 3;
    S* pg = reinterpret_cast<S*>(smem + L::kG) + tpos * SPT;
    const S* px = reinterpret_cast<const S*>(smem + L::kX) + tpos * SPT;
    const V2* ph = reinterpret_cast<const V2*>(smem + L::kH) + tpos * SPT;
    // the gradient entering through the final state belongs to the thread that owns sample T-1
    const bool owner = p.g_in != nullptr && nv > 0 && (t0 + (int64_t)tpos * SPT + nv == p.T);
    S gi0 = S(0), gi1 = S(0);
    if (owner) { gi0 = __ldg(p.g_in + (int64_t)row * 2); gi1 = __ldg(p.g_in + (int64_t)row * 2 + 1); }

    // phase A: my samples (descending) as one affine map of lam
    S m[6] = {S(1), S(0), S(0), S(1), S(0), S(0)};
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      if (j < nv) {
        const V2 av = pa[j];
        const S b0 = pb[3 * j], b1 = pb[3 * j + 1], b2 = pb[3 * j + 2], g = pg[j];
        if (!TDF2) {   // lam' = [[-a1,1],[-a2,0]] lam + C gy
          const S c0 = b1 - b0 * av.x, c1 = b2 - b0 * av.y;
          const S n0 = -av.x * m[0] + m[2], n1 = -av.x * m[1] + m[3], n4 = -av.x * m[4] + m[5] + c0 * g;
          const S n2 = -av.y * m[0], n3 = -av.y * m[1], n5 = -av.y * m[4] + c1 * g;
          m[0] = n0; m[1] = n1; m[2] = n2; m[3] = n3; m[4] = n4; m[5] = n5;
        } else {       // lam' = [[-a1,-a2],[1,0]] lam + [gy, 0]
          const S n0 = -av.x * m[0] - av.y * m[2], n1 = -av.x * m[1] - av.y * m[3];
          const S n4 = -av.x * m[4] - av.y * m[5] + g;
          m[2] = m[0]; m[3] = m[1]; m[5] = m[4];
          m[0] = n0; m[1] = n1; m[4] = n4;
        }
      }
    }
    if (owner) {   // its incoming state is g_in, not zero: as seen by the threads after it
      m[4] += m[0] * gi0 + m[1] * gi1;
      m[5] += m[2] * gi0 + m[3] * gi1;
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
      const typename LpvLb<S>::State hin =
          lpv_tile_state<S, C::NW>(ws, sm_wtot, ticket, chunk, nchunks, B, lane, S(0), S(0), wait_ns);
      if (lane == 0) { sm_hin[0] = hin.v[0]; sm_hin[1] = hin.v[1]; }
    }
    __syncthreads();
    S l0 = sm_hin[0], l1 = sm_hin[1];
    for (int w = 0; w < warp; ++w) {
      const S* t = sm_wtot + w * 6;
      const S g0 = t[0] * l0 + t[1] * l1 + t[4], g1 = t[2] * l0 + t[3] * l1 + t[5];
      l0 = g0; l1 = g1;
    }
    {
      const S g0 = e[0] * l0 + e[1] * l1 + e[4], g1 = e[2] * l0 + e[3] * l1 + e[5];
      l0 = g0 + gi0; l1 = g1 + gi1;
    }
    // phase B: replay; the gradients replace the operands in place
#pragma unroll
    for (int j = SPT - 1; j >= 0; --j) {
      if (j < nv) {
        const V2 av = pa[j];
        const S b0 = pb[3 * j], b1 = pb[3 * j + 1], b2 = pb[3 * j + 2], g = pg[j], xj = px[j];
        const V2 hv = ph[j];
        const S c0 = b1 - b0 * av.x, c1 = b2 - b0 * av.y;
        if (!TDF2) {
          const S gc0 = g * hv.x, gc1 = g * hv.y;   // gradient w.r.t. C_t
          pg[j] = l0 + b0 * g;
          V2 gav;
          gav.x = -l0 * hv.x - b0 * gc0;
          gav.y = -l0 * hv.y - b0 * gc1;
          pa[j] = gav;
          pb[3 * j] = g * xj - av.x * gc0 - av.y * gc1;
          pb[3 * j + 1] = gc0;
          pb[3 * j + 2] = gc1;
          const S n0 = -av.x * l0 + l1 + c0 * g, n1 = -av.y * l0 + c1 * g;
          l0 = n0; l1 = n1;
        } else {
          const S gb0 = xj * l0, gb1 = xj * l1;     // gradient w.r.t. B_t
          pg[j] = c0 * l0 + c1 * l1 + b0 * g;
          V2 gav;
          gav.x = -l0 * hv.x - b0 * gb0;
          gav.y = -l1 * hv.x - b0 * gb1;
          pa[j] = gav;
          pb[3 * j] = g * xj - av.x * gb0 - av.y * gb1;
          pb[3 * j + 1] = gb0;
          pb[3 * j + 2] = gb1;
          const S n0 = -av.x * l0 - av.y * l1 + g;
          l1 = l0;
          l0 = n0;
        }
      }
    }
    if (tid == NT - 1 && chunk + 1 == nchunks && p.grad_zi) {
      p.grad_zi[(int64_t)row * 2] = l0;
      p.grad_zi[(int64_t)row * 2 + 1] = l1;
    }
    S* ox = p.grad_x + off;
    S* oa = p.grad_a + 2 * off;
    S* ob = p.grad_b + 3 * off;
    if (bulk) {
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        bulk_s2g(ox, smem + L::kG, nbytes);
        bulk_s2g(oa, smem + L::kA, 2 * nbytes);
        bulk_s2g(ob, smem + L::kB, 3 * nbytes);
        bulk_commit();
      }
    } else {
      __syncthreads();
      auto put = [&](S* g, int o, uint32_t words) {
        const uint32_t* sdat = reinterpret_cast<const uint32_t*>(smem + o);
        uint32_t* gg = reinterpret_cast<uint32_t*>(g);
        for (uint32_t w = tid; w < words; w += NT) gg[w] = sdat[w];
      };
      put(ox, L::kG, nbytes / 4);
      put(oa, L::kA, 2 * nbytes / 4);
      put(ob, L::kB, 3 * nbytes / 4);
    }
    __syncthreads();
  }
  if (tid == 0) bulk_wait_all();
}

}  // namespace ptb
