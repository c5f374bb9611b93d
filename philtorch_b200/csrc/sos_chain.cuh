// Cascade of K second-order sections (transposed direct form II) for LARGE BATCHES: one pass per
// direction in which a CTA takes a tile of one row through all K sections, section after section,
// and hands the 2K end states to the tile that follows it in the row.
//
// This is the chained (not decoupled) form of the scan: a tile needs the END STATE of its
// predecessor, not an aggregate.  Tiles are handed out chunk-major (ticket -> chunk = ticket / B,
// row = ticket % B) and a CTA works on one tile at a time, so with at least as many rows as
// resident CTAs the predecessor (B tickets older) has finished before its successor starts and
// nothing ever waits; with fewer rows CTAs wait for one another and the decoupled kernels of
// sos_cascade.cuh are the better choice (the host picks).  States travel section by section
// ({flag, payload} words as in scan_engine.cuh), so a successor can start section k as soon as
// its predecessor has finished section k.
//
// Why it is cheap: per section the recurrence is 2x2 and time-invariant, so inside a tile
//   phase A  every thread runs its SPT samples from a zero state (2 numbers out),
//   scan     2 shuffles + 4 multiply-adds per step over the lanes with the constant powers
//            D^(2^d) of the section's SPT-sample matrix D, warp totals exchanged through shared
//            memory (one CTA barrier per section),
//   phase B  every thread replays its samples from its true incoming state
// with the thread's samples in registers throughout; the output of section k is the input of
// section k+1 in the same registers.  The loop over sections is not unrolled: the hot code is one
// section's worth of instructions.
//
// Per-row constants (chain_setup_kernel, in double): per section the derived coefficients, D^l
// for l = 0..31 (lane offsets and scan steps) and D^(32 w) for w = 0..NW (warp offsets).
#pragma once
#include "biquad.cuh"

namespace ptb {

template <class S, int K_, int CH_, int NT_, int NOUT_ = 1, int MINB_ = 2>
struct ChainCfg {
  static_assert(NOUT_ == 1 || (NOUT_ == 2 && K_ % 2 == 0), "two output buffers alternate per section across tiles");
  using Scalar = S;
  static constexpr int K = K_, CH = CH_, NT = NT_, NW = NT_ / 32;
  static constexpr int NOUT = NOUT_;   // forward: tile buffers for section outputs on their way out
  static constexpr int MINB = MINB_;   // CTAs per SM the kernels are built for
  static constexpr int V = Vec16<S>::V;
  static constexpr int SPT = V * CH;
  static constexpr int TILE = NT * SPT;
  static constexpr int TILE_BYTES = TILE * (int)sizeof(S);
  // one section's block of a table row (scalars)
  static constexpr int T_DL = 8;                     // D^l, l = 0..31
  static constexpr int T_DW = T_DL + 4 * 32;         // D^(32 w), w = 0..NW
  static constexpr int SEC = T_DW + 4 * (NW + 1);
  static constexpr int ROW = K * SEC;
  static constexpr int ROW_BYTES = ROW * (int)sizeof(S);
  static constexpr int ROWB = ((ROW_BYTES + 127) / 128) * 128;
  static constexpr int SLOT_WORDS = 2 * K * (int)(sizeof(S) / 4);   // one 64-bit word per 32 payload bits
  static_assert(SEC % 4 == 0, "table rows stay 16-byte aligned");
};

template <class S> struct Ld4s;   // four consecutive scalars from shared memory
template <> struct Ld4s<float> {
  static __device__ __forceinline__ void ld(const float* p, float* m) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    m[0] = q.x; m[1] = q.y; m[2] = q.z; m[3] = q.w;
  }
};
template <> struct Ld4s<double> {
  static __device__ __forceinline__ void ld(const double* p, double* m) {
    const double2 q = *reinterpret_cast<const double2*>(p), r = *reinterpret_cast<const double2*>(p + 2);
    m[0] = q.x; m[1] = q.y; m[2] = r.x; m[3] = r.y;
  }
};

// One thread per (row, section).  ADJ: powers of the adjoint's matrix [[-a1,-a2],[1,0]] instead of
// the forward [[-a1,1],[-a2,0]].
template <class S, class C, bool ADJ>
__global__ void chain_setup_kernel(const S* __restrict__ b, int64_t b_sec, int64_t b_row, const S* __restrict__ a,
                                   int64_t a_sec, int64_t a_row, S* __restrict__ tab, int64_t rows) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * C::K) return;
  const int64_t row = i / C::K;
  const int k = (int)(i % C::K);
  S d[5];
  BqCoef<S>::derive(b + k * b_sec + row * b_row, 0, a + k * a_sec + row * a_row, 0, 0, d);
  S* out = tab + row * C::ROW + (int64_t)k * C::SEC;
  for (int j = 0; j < 5; ++j) out[j] = d[j];
  for (int j = 5; j < 8; ++j) out[j] = S(0);
  const double na1 = (double)d[3], na2 = (double)d[4];
  const double A[4] = {na1, ADJ ? na2 : 1.0, ADJ ? 1.0 : na2, 0.0};
  auto mul = [](const double* x, const double* y, double* r) {   // r = x y
    const double r0 = x[0] * y[0] + x[1] * y[2], r1 = x[0] * y[1] + x[1] * y[3];
    const double r2 = x[2] * y[0] + x[3] * y[2], r3 = x[2] * y[1] + x[3] * y[3];
    r[0] = r0; r[1] = r1; r[2] = r2; r[3] = r3;
  };
  double D[4] = {1.0, 0.0, 0.0, 1.0};
  for (int n = 0; n < C::SPT; ++n) mul(A, D, D);
  double P[4] = {1.0, 0.0, 0.0, 1.0};
  for (int l = 0; l < 32; ++l) {
    for (int j = 0; j < 4; ++j) out[C::T_DL + 4 * l + j] = (S)P[j];
    mul(D, P, P);
  }
  const double W[4] = {P[0], P[1], P[2], P[3]};   // D^32
  double Q[4] = {1.0, 0.0, 0.0, 1.0};
  for (int w = 0; w <= C::NW; ++w) {
    for (int j = 0; j < 4; ++j) out[C::T_DW + 4 * w + j] = (S)Q[j];
    mul(W, Q, Q);
  }
}

// ---- pieces shared by the two directions ---------------------------------------------------------
// inclusive scan over the lanes of the 2-vectors (a0, a1) under  s -> D s + a  per lane
template <class S, class C>
__device__ __forceinline__ void chain_warp_scan(const S* sec, int lane, S& a0, S& a1) {
#pragma unroll
  for (int d = 0; d < 5; ++d) {
    const S o0 = __shfl_up_sync(0xffffffffu, a0, 1 << d), o1 = __shfl_up_sync(0xffffffffu, a1, 1 << d);
    S m[4];
    Ld4s<S>::ld(sec + C::T_DL + 4 * (1 << d), m);
    if (lane >= (1 << d)) {
      a0 += m[0] * o0 + m[1] * o1;
      a1 += m[2] * o0 + m[3] * o1;
    }
  }
}
// state entering this thread: tile-incoming state carried over the warps before this one and the
// lanes before this one, plus the zero-state contributions of those warps (wt) and lanes (e0, e1)
template <class S, class C>
__device__ __forceinline__ void chain_thread_state(const S* sec, const S* wt, const S* hin, int warp, int lane, S e0,
                                                   S e1, S& h0, S& h1) {
  S m[4];
  Ld4s<S>::ld(sec + C::T_DW + 4 * warp, m);
  S z0 = m[0] * hin[0] + m[1] * hin[1], z1 = m[2] * hin[0] + m[3] * hin[1];
  for (int w = 0; w < warp; ++w) {
    Ld4s<S>::ld(sec + C::T_DW + 4 * (warp - 1 - w), m);
    const S t0 = wt[2 * w], t1 = wt[2 * w + 1];
    z0 += m[0] * t0 + m[1] * t1;
    z1 += m[2] * t0 + m[3] * t1;
  }
  Ld4s<S>::ld(sec + C::T_DL + 4 * lane, m);
  h0 = m[0] * z0 + m[1] * z1 + e0;
  h1 = m[2] * z0 + m[3] * z1 + e1;
}
// the two states of one section of one tile as {flag = 2, payload} words
template <class S>
__device__ __forceinline__ void chain_publish(uint64_t* slot, S h0, S h1) {
  Pod<S, 2> v; v.v[0] = h0; v.v[1] = h1;
  slot_store(slot, v, 2u);
}
// one look without waiting; false when they are not there yet
template <class S>
__device__ __forceinline__ bool chain_try_fetch(const uint64_t* slot, S& h0, S& h1) {
  constexpr int W = Words<Pod<S, 2>>::W;
  uint64_t raw[W];
#pragma unroll
  for (int i = 0; i < W; ++i) raw[i] = ld_relaxed_u64(slot + i);
  bool ok = true;
  typename Words<Pod<S, 2>>::U u;
#pragma unroll
  for (int i = 0; i < W; ++i) { ok = ok && ((uint32_t)(raw[i] >> 32) == 2u); u.w[i] = (uint32_t)raw[i]; }
  h0 = u.t.v[0]; h1 = u.t.v[1];
  return ok;
}
// waits (bounded) for them; false when the wait ran out
template <class S>
__device__ __forceinline__ bool chain_fetch(const uint64_t* slot, S& h0, S& h1, uint64_t wait_ns) {
  constexpr int W = Words<Pod<S, 2>>::W;
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint64_t raw[W];
#pragma unroll
    for (int i = 0; i < W; ++i) raw[i] = ld_relaxed_u64(slot + i);
    bool ok = true;
    typename Words<Pod<S, 2>>::U u;
#pragma unroll
    for (int i = 0; i < W; ++i) { ok = ok && ((uint32_t)(raw[i] >> 32) == 2u); u.w[i] = (uint32_t)raw[i]; }
    if (ok) { h0 = u.t.v[0]; h1 = u.t.v[1]; return true; }
    if (it > 1) __nanosleep(it > 64 ? 400 : 100);
    if (it == 64) t0 = globaltimer_ns();
    if (it > 64 && globaltimer_ns() - t0 > wait_ns) { h0 = S(0); h1 = S(0); return false; }
  }
}

// ------------------------------------------------------------------------------------ forward
template <class S>
struct ChainFwdParams {
  const S* tab; int64_t tab_stride;
  const S* zi;    // optional (K,B,2)
  const S* x;
  S* y;
  S* mid;         // optional (K-1,B,T)
  S* zf;          // optional (K,B,2)
  int64_t T, B;
};

template <class C>
struct ChainFwdSmem {
  static constexpr int kXin = 0;                                   // [TILE]     samples of the tile being loaded
  static constexpr int kRowc = kXin + C::TILE_BYTES;               // [2][ROWB]  table rows of this tile and the next
  static constexpr int kOut = kRowc + 2 * C::ROWB;                 // [NOUT][TILE] section outputs on their way out
  static constexpr int kBar = kOut + C::NOUT * C::TILE_BYTES;      // u64 full[2]
  static constexpr int kMisc = kBar + 16;                          // u32 ticket[2], ok
  static constexpr int kHin = kMisc + 16;                          // S hin[2][2]
  static constexpr int kWtot = kHin + 4 * 8;                       // S wtot[2][NW][2]
  static constexpr int kPre = kWtot + 2 * C::NW * 2 * 8;           // S pre[K][2], u32 pre_ok[K]: states found at tile start
  static constexpr int kTotal = kPre + C::K * (2 * 8 + 4) + 16;
};

template <class S, class C>
__global__ void __launch_bounds__(C::NT, C::MINB)
chain_fwd_kernel(const ChainFwdParams<S> p, const Workspace ws, const uint32_t B, const uint32_t nchunks,
                 const uint32_t ntiles, const int bulk, const uint64_t wait_ns) {
  using L = ChainFwdSmem<C>;
  constexpr int K = C::K, CH = C::CH, V = C::V, SPT = C::SPT, TILE = C::TILE, NT = C::NT, NW = C::NW;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBar);
  volatile uint32_t* sm_ticket = reinterpret_cast<volatile uint32_t*>(smem + L::kMisc);
  volatile uint32_t* sm_ok = sm_ticket + 2;
  S* sm_hin = reinterpret_cast<S*>(smem + L::kHin);
  S* sm_wtot = reinterpret_cast<S*>(smem + L::kWtot);
  S* sm_pre = reinterpret_cast<S*>(smem + L::kPre);
  volatile uint32_t* sm_pre_ok = reinterpret_cast<volatile uint32_t*>(smem + L::kPre + C::K * 2 * 8);
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
  auto issue = [&](int s, uint32_t ticket) {   // one thread: bulk loads of a tile's samples and table row
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    mbar_arrive_expect_tx(&full[s], bytes + C::ROW_BYTES);
    bulk_g2s(smem + L::kXin, p.x + (int64_t)row * p.T + t0, bytes, &full[s]);
    bulk_g2s(smem + L::kRowc + s * C::ROWB, p.tab + (int64_t)row * p.tab_stride, C::ROW_BYTES, &full[s]);
  };
  if (tid == 0) {
    const uint32_t t = atomicAdd(ws.ticket, 1u);
    sm_ticket[0] = t < ntiles ? t : kNoTile;
    if (t < ntiles && bulk) issue(0, t);
  }
  __syncthreads();

  uint32_t failed = 0;
  for (uint32_t n = 0;; ++n) {
    const int s = n & 1;
    const uint32_t ticket = sm_ticket[s];
    if (ticket == kNoTile) break;
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    unsigned char* xin = smem + L::kXin;
    S* rowc = reinterpret_cast<S*>(smem + L::kRowc + s * C::ROWB);
    if (bulk) {
      if (tid == 0) {
        const bool ok = mbar_wait_bounded(&full[s], (n >> 1) & 1u, failed ? kWaitNsAfterError : wait_ns);
        if (!ok) atomicOr(ws.error, kErrLoadTimeout);
        *sm_ok = ok ? 1u : 0u;
      }
    } else {
      const uint32_t* gx = reinterpret_cast<const uint32_t*>(p.x + (int64_t)row * p.T + t0);
      uint32_t* dx = reinterpret_cast<uint32_t*>(xin);
      for (uint32_t w = tid; w < (uint32_t)nvalid * (sizeof(S) / 4); w += NT) dx[w] = __ldg(gx + w);
      const uint32_t* gt = reinterpret_cast<const uint32_t*>(p.tab + (int64_t)row * p.tab_stride);
      uint32_t* dt = reinterpret_cast<uint32_t*>(rowc);
      for (uint32_t w = tid; w < (uint32_t)(C::ROW_BYTES / 4); w += NT) dt[w] = __ldg(gt + w);
      if (tid == 0) *sm_ok = 1u;
    }
    __syncthreads();
    if (*sm_ok == 0u) failed = 1;
    if (failed) {   // results are invalid from here on: stop taking work
      if (tid == 0) sm_ticket[s ^ 1] = kNoTile;
      __syncthreads();
      continue;
    }
    if (bulk) mbar_test_wait(&full[s], (n >> 1) & 1u);   // every thread observes the completed phase itself

    // this thread's samples, zero beyond the end of the row
    S x[SPT];
    int nv = nvalid - tid * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    {
      const unsigned char* px = xin + (size_t)tid * SPT * sizeof(S);
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<S, V>::ld(px + 16 * c, &x[c * V]);
      if (nv < SPT) {
#pragma unroll
        for (int j = 0; j < SPT; ++j)
          if (j >= nv) x[j] = S(0);
      }
    }
    const uint64_t* pred = ws.slots + ((size_t)ticket - B) * C::SLOT_WORDS;   // read only when chunk > 0
    // The predecessor has normally finished: one look at all its K records now (K lanes, one round
    // trip) instead of a round trip per section later; what is missing is waited for section by section.
    if (tid < K) {
      S q0 = S(0), q1 = S(0);
      const bool ok = chunk > 0 && chain_try_fetch<S>(pred + tid * (C::SLOT_WORDS / K), q0, q1);
      sm_pre[2 * tid] = q0;
      sm_pre[2 * tid + 1] = q1;
      sm_pre_ok[tid] = ok ? 1u : 0u;
    }
    __syncthreads();   // everyone holds its samples: the tile buffer is free
    if (tid == 0) {    // fetch the tile after this one
      const uint32_t t = atomicAdd(ws.ticket, 1u);
      sm_ticket[s ^ 1] = t < ntiles ? t : kNoTile;
      if (t < ntiles && bulk) {
        fence_proxy_async_smem();
        issue(s ^ 1, t);
      }
    }
    const bool owner = p.zf != nullptr && nv > 0 && (t0 + (int64_t)tid * SPT + nv == p.T);
    const bool full_tile = nvalid == TILE;
    uint64_t* mine_slot = ws.slots + (size_t)ticket * C::SLOT_WORDS;

#pragma unroll 1
    for (int k = 0; k < K; ++k) {
      const S* sec = rowc + k * C::SEC;
      BqCoef<S> c;
      c.load(reinterpret_cast<const unsigned char*>(sec));
      // phase A: my samples from a zero state
      S a0 = S(0), a1 = S(0);
#pragma unroll
      for (int j = 0; j < SPT; ++j) {
        const S t = a1 + c.B0 * x[j];   // off the chain through a0
        a1 = c.na2 * a0 + c.B1 * x[j];
        a0 = c.na1 * a0 + t;
      }
      chain_warp_scan<S, C>(sec, lane, a0, a1);
      S e0 = __shfl_up_sync(0xffffffffu, a0, 1), e1 = __shfl_up_sync(0xffffffffu, a1, 1);
      if (lane == 0) { e0 = S(0); e1 = S(0); }
      S* wt = sm_wtot + (k & 1) * NW * 2;
      S* hin = sm_hin + (k & 1) * 2;
      if (lane == 31) { wt[2 * warp] = a0; wt[2 * warp + 1] = a1; }
      if (tid == 0) {
        S h0 = S(0), h1 = S(0);
        if (chunk == 0) {
          if (p.zi) {
            h0 = __ldg(p.zi + ((int64_t)k * p.B + row) * 2);
            h1 = __ldg(p.zi + ((int64_t)k * p.B + row) * 2 + 1);
          }
        } else if (sm_pre_ok[k]) {
          h0 = sm_pre[2 * k];
          h1 = sm_pre[2 * k + 1];
        } else if (!chain_fetch<S>(pred + k * (C::SLOT_WORDS / K), h0, h1, wait_ns)) {
          atomicOr(ws.error, kErrLookbackTimeout);
        }
        hin[0] = h0; hin[1] = h1;
        // the bulk store that last read this section's output buffer has finished
        if (C::NOUT == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
      __syncthreads();
      S h0, h1;
      chain_thread_state<S, C>(sec, wt, hin, warp, lane, e0, e1, h0, h1);
      // phase B: replay from the true state; x becomes the section's output
      if (full_tile) {
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
          const S xj = x[j];
          x[j] = h0 + c.b0 * xj;
          const S t = h1 + c.B0 * xj;
          h1 = c.na2 * h0 + c.B1 * xj;
          h0 = c.na1 * h0 + t;
        }
      } else {
#pragma unroll
        for (int j = 0; j < SPT; ++j) {
          if (j < nv) {
            const S xj = x[j];
            x[j] = h0 + c.b0 * xj;
            const S t = h1 + c.B0 * xj;
            h1 = c.na2 * h0 + c.B1 * xj;
            h0 = c.na1 * h0 + t;
          }
        }
      }
      if (tid == NT - 1 && chunk + 1 < nchunks) chain_publish<S>(mine_slot + k * (C::SLOT_WORDS / K), h0, h1);
      if (owner) {
        p.zf[((int64_t)k * p.B + row) * 2] = h0;
        p.zf[((int64_t)k * p.B + row) * 2 + 1] = h1;
      }
      const bool store = (k == K - 1) || (p.mid != nullptr);
      unsigned char* ob = smem + L::kOut + (C::NOUT == 2 ? (k & 1) : 0) * C::TILE_BYTES;
      if (store) {
        unsigned char* po = ob + (size_t)tid * SPT * sizeof(S);
#pragma unroll
        for (int q = 0; q < CH; ++q) VecIO<S, V>::st(po + 16 * q, &x[q * V]);
      }
      S* dst = (k == K - 1 ? p.y : p.mid + (int64_t)k * p.B * p.T) + (int64_t)row * p.T + t0;
      if (bulk) {
        if (store) {
          fence_proxy_async_smem();
          __syncthreads();
        }
        if (tid == 0) {
          if (store) bulk_s2g(dst, ob, (uint32_t)nvalid * sizeof(S));
          bulk_commit();   // one group per section, stored or not: the read-wait above counts groups
        }
      } else if (store) {
        __syncthreads();
        const uint32_t* so = reinterpret_cast<const uint32_t*>(ob);
        uint32_t* go = reinterpret_cast<uint32_t*>(dst);
        for (uint32_t w = tid; w < (uint32_t)nvalid * (sizeof(S) / 4); w += NT) go[w] = so[w];
      }
    }
    __syncthreads();   // the tile's stage and scratch are free
  }
  if (tid == 0) bulk_wait_all();
}

// ------------------------------------------------------------------------------------ backward
// Adjoint of the cascade, sections K-1 .. 0 in descending time (see biquad.cuh for one section's
// adjoint).  Scan position `tid` owns the samples of tile position NT-1-tid.  With coefficient
// gradients the section inputs/outputs Z_0 = x, Z_m = output of section m-1 (Z_K = y) stream
// through a ring of three tile buffers: section k reads Z_k and Z_{k+1} while Z_{k-1} is on its way.
template <class S>
struct ChainBwdParams {
  const S* tab; int64_t tab_stride;   // ADJOINT table
  const S* gy;
  const S* x;
  const S* mid;
  const S* y;
  const S* g_in;     // optional (K,B,2): gradient w.r.t. the final states
  S* grad_x;
  S* grad_zi;        // optional (K,B,2)
  int64_t T, B;
  int want_coef;
};

template <class C>
struct ChainBwdSmem {
  static constexpr int kGin = 0;                                   // [TILE]     gy of the tile being loaded
  static constexpr int kRowc = kGin + C::TILE_BYTES;               // [2][ROWB]
  static constexpr int kZ = kRowc + 2 * C::ROWB;                   // [3][TILE]  ring of section inputs/outputs; grad_x leaves from [2]
  static constexpr int kBar = kZ + 3 * C::TILE_BYTES;              // u64 full[2], zbar[K+1]
  static constexpr int kMisc = kBar + 8 * (2 + C::K + 1);          // u32 ticket[2], ok
  static constexpr int kHin = kMisc + 16;                          // S hin[2][2]
  static constexpr int kWtot = kHin + 4 * 8;                       // S wtot[2][NW][2]
  static constexpr int kPsum = kWtot + 2 * C::NW * 2 * 8;          // S psum[2][NW][5]
  static constexpr int kPre = kPsum + 2 * C::NW * 5 * 8;           // S pre[K][2], u32 pre_ok[K]: states found at tile start
  static constexpr int kTotal = kPre + C::K * (2 * 8 + 4) + 16;
};

template <class S, class C>
__global__ void __launch_bounds__(C::NT, C::MINB)
chain_bwd_kernel(const ChainBwdParams<S> p, const Workspace ws, const uint32_t B, const uint32_t nchunks,
                 const uint32_t ntiles, const int bulk, const uint64_t wait_ns) {
  using L = ChainBwdSmem<C>;
  constexpr int K = C::K, CH = C::CH, V = C::V, SPT = C::SPT, TILE = C::TILE, NT = C::NT, NW = C::NW;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* zbar = full + 2;
  volatile uint32_t* sm_ticket = reinterpret_cast<volatile uint32_t*>(smem + L::kMisc);
  volatile uint32_t* sm_ok = sm_ticket + 2;
  S* sm_hin = reinterpret_cast<S*>(smem + L::kHin);
  S* sm_wtot = reinterpret_cast<S*>(smem + L::kWtot);
  S* sm_psum = reinterpret_cast<S*>(smem + L::kPsum);
  S* sm_pre = reinterpret_cast<S*>(smem + L::kPre);
  volatile uint32_t* sm_pre_ok = reinterpret_cast<volatile uint32_t*>(smem + L::kPre + C::K * 2 * 8);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tpos = NT - 1 - tid;   // time runs against the scan order

  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    for (int m = 0; m <= K; ++m) mbar_init(&zbar[m], 1);
    fence_mbar_init();
  }
  __syncthreads();
  auto coords = [&](uint32_t ticket, uint32_t& chunk, uint32_t& row, int64_t& t0, int& nvalid) {
    chunk = ticket / B;
    row = ticket - chunk * B;
    t0 = (int64_t)(nchunks - 1 - chunk) * TILE;
    const int64_t rem = p.T - t0;
    nvalid = rem < (int64_t)TILE ? (int)rem : TILE;
  };
  auto issue = [&](int s, uint32_t ticket) {
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    const uint32_t bytes = (uint32_t)nvalid * sizeof(S);
    mbar_arrive_expect_tx(&full[s], bytes + C::ROW_BYTES);
    bulk_g2s(smem + L::kGin, p.gy + (int64_t)row * p.T + t0, bytes, &full[s]);
    bulk_g2s(smem + L::kRowc + s * C::ROWB, p.tab + (int64_t)row * p.tab_stride, C::ROW_BYTES, &full[s]);
  };
  auto zrow = [&](int m, int64_t row) -> const S* {
    if (m == 0) return p.x + row * p.T;
    if (m == K) return p.y + row * p.T;
    return p.mid + ((int64_t)(m - 1) * p.B + row) * p.T;
  };
  auto zbuf = [&](int m) -> unsigned char* { return smem + L::kZ + (m % 3) * C::TILE_BYTES; };
  if (tid == 0) {
    const uint32_t t = atomicAdd(ws.ticket, 1u);
    sm_ticket[0] = t < ntiles ? t : kNoTile;
    if (t < ntiles && bulk) issue(0, t);
  }
  __syncthreads();

  uint32_t failed = 0;
  for (uint32_t n = 0;; ++n) {
    const int s = n & 1;
    const uint32_t par = n & 1u;   // every Z barrier completes once per tile
    const uint32_t ticket = sm_ticket[s];
    if (ticket == kNoTile) break;
    uint32_t chunk, row; int64_t t0; int nvalid;
    coords(ticket, chunk, row, t0, nvalid);
    unsigned char* gin = smem + L::kGin;
    S* rowc = reinterpret_cast<S*>(smem + L::kRowc + s * C::ROWB);
    const uint32_t tile_bytes = (uint32_t)nvalid * sizeof(S);
    auto zrequest = [&](int m) {   // one thread: array Z_m of this tile into its ring buffer
      mbar_arrive_expect_tx(&zbar[m], tile_bytes);
      bulk_g2s(zbuf(m), zrow(m, row) + t0, tile_bytes, &zbar[m]);
    };
    auto zcopy = [&](int m) {      // all threads: the same with plain loads
      const uint32_t* g = reinterpret_cast<const uint32_t*>(zrow(m, row) + t0);
      uint32_t* d = reinterpret_cast<uint32_t*>(zbuf(m));
      for (uint32_t w = tid; w < tile_bytes / 4; w += NT) d[w] = __ldg(g + w);
    };
    if (bulk) {
      if (tid == 0) {
        if (p.want_coef && !failed) {
          bulk_wait_read_all();   // grad_x of the previous tile has left ring buffer 2
          fence_proxy_async_smem();
          zrequest(K);
          zrequest(K - 1);
        }
        const bool ok = mbar_wait_bounded(&full[s], (n >> 1) & 1u, failed ? kWaitNsAfterError : wait_ns);
        if (!ok) atomicOr(ws.error, kErrLoadTimeout);
        *sm_ok = ok ? 1u : 0u;
      }
    } else {
      const uint32_t* gg = reinterpret_cast<const uint32_t*>(p.gy + (int64_t)row * p.T + t0);
      uint32_t* dg = reinterpret_cast<uint32_t*>(gin);
      for (uint32_t w = tid; w < tile_bytes / 4; w += NT) dg[w] = __ldg(gg + w);
      const uint32_t* gt = reinterpret_cast<const uint32_t*>(p.tab + (int64_t)row * p.tab_stride);
      uint32_t* dt = reinterpret_cast<uint32_t*>(rowc);
      for (uint32_t w = tid; w < (uint32_t)(C::ROW_BYTES / 4); w += NT) dt[w] = __ldg(gt + w);
      if (p.want_coef) { zcopy(K); zcopy(K - 1); }
      if (tid == 0) *sm_ok = 1u;
    }
    __syncthreads();
    if (*sm_ok == 0u) failed = 1;
    if (failed) {
      if (tid == 0) sm_ticket[s ^ 1] = kNoTile;
      __syncthreads();
      continue;
    }
    if (bulk) mbar_test_wait(&full[s], (n >> 1) & 1u);   // every thread observes the completed phase itself

    S g[SPT];
    int nv = nvalid - tpos * SPT;
    nv = nv < 0 ? 0 : (nv > SPT ? SPT : nv);
    unsigned char* pg = gin + (size_t)tpos * SPT * sizeof(S);
    {
#pragma unroll
      for (int c = 0; c < CH; ++c) VecIO<S, V>::ld(pg + 16 * c, &g[c * V]);
      if (nv < SPT) {
#pragma unroll
        for (int j = 0; j < SPT; ++j)
          if (j >= nv) g[j] = S(0);
      }
    }
    const uint64_t* pred = ws.slots + ((size_t)ticket - B) * C::SLOT_WORDS;
    if (tid < K) {   // one early look at all K records of the predecessor (see the forward kernel)
      S q0 = S(0), q1 = S(0);
      const bool ok = chunk > 0 && chain_try_fetch<S>(pred + tid * (C::SLOT_WORDS / K), q0, q1);
      sm_pre[2 * tid] = q0;
      sm_pre[2 * tid + 1] = q1;
      sm_pre_ok[tid] = ok ? 1u : 0u;
    }
    __syncthreads();   // everyone holds its samples: the tile buffer is free
    if (tid == 0) {    // fetch the tile after this one
      const uint32_t t = atomicAdd(ws.ticket, 1u);
      sm_ticket[s ^ 1] = t < ntiles ? t : kNoTile;
      if (t < ntiles && bulk) {
        fence_proxy_async_smem();
        issue(s ^ 1, t);
      }
    }
    // the gradient entering through the final states is injected by the thread that owns sample T-1
    const bool owner = p.g_in != nullptr && nv > 0 && (t0 + (int64_t)tpos * SPT + nv == p.T);
    const bool full_tile = nvalid == TILE;
    uint64_t* mine_slot = ws.slots + (size_t)ticket * C::SLOT_WORDS;
    S* part = static_cast<S*>(ws.partial) + ((size_t)row * nchunks + chunk) * (5 * K);

#pragma unroll 1
    for (int k = K - 1; k >= 0; --k) {
      const S* sec = rowc + k * C::SEC;
      BqCoef<S> c;
      c.load(reinterpret_cast<const unsigned char*>(sec));
      S gi0 = S(0), gi1 = S(0);
      if (owner) {
        gi0 = __ldg(p.g_in + ((int64_t)k * p.B + row) * 2);
        gi1 = __ldg(p.g_in + ((int64_t)k * p.B + row) * 2 + 1);
      }
      // phase A: my samples from a zero state (padded samples are skipped, not run with zero drive:
      // an injected state must not move)
      S a0 = gi0, a1 = gi1;
      if (full_tile) {
#pragma unroll
        for (int j = SPT - 1; j >= 0; --j) {
          const S t = c.na2 * a1 + g[j];   // off the chain through a0
          a1 = a0;
          a0 = c.na1 * a0 + t;
        }
      } else {
#pragma unroll
        for (int j = SPT - 1; j >= 0; --j) {
          if (j < nv) {
            const S t = c.na2 * a1 + g[j];
            a1 = a0;
            a0 = c.na1 * a0 + t;
          }
        }
      }
      chain_warp_scan<S, C>(sec, lane, a0, a1);
      S e0 = __shfl_up_sync(0xffffffffu, a0, 1), e1 = __shfl_up_sync(0xffffffffu, a1, 1);
      if (lane == 0) { e0 = S(0); e1 = S(0); }
      S* wt = sm_wtot + (k & 1) * NW * 2;
      S* hin = sm_hin + (k & 1) * 2;
      if (lane == 31) { wt[2 * warp] = a0; wt[2 * warp + 1] = a1; }
      if (tid == 0) {
        S h0 = S(0), h1 = S(0);
        if (chunk > 0) {
          if (sm_pre_ok[k]) {
            h0 = sm_pre[2 * k];
            h1 = sm_pre[2 * k + 1];
          } else if (!chain_fetch<S>(pred + k * (C::SLOT_WORDS / K), h0, h1, wait_ns)) {
            atomicOr(ws.error, kErrLookbackTimeout);
          }
        }
        hin[0] = h0; hin[1] = h1;
        if (p.want_coef && bulk) {
          bool ok = true;
          if (k == K - 1) ok = mbar_wait_bounded(&zbar[K], par, wait_ns);
          ok = mbar_wait_bounded(&zbar[k], par, wait_ns) && ok;
          if (!ok) atomicOr(ws.error, kErrLoadTimeout);
        }
      }
      __syncthreads();   // (A) warp totals, incoming state and the section's arrays are in place
      if (p.want_coef && bulk) {   // every thread observes the completed phases itself
        if (k == K - 1) mbar_test_wait(&zbar[K], par);
        mbar_test_wait(&zbar[k], par);
      }
      if (p.want_coef && k >= 1) {
        // Z_{k-1} goes where Z_{k+2} was: every thread is through with section k+1
        if (bulk) {
          if (tid == 0) {
            fence_proxy_async_smem();
            zrequest(k - 1);
          }
        }
      }
      // the sums of the section before this one (in processing order) leave the chip
      if (p.want_coef && k < K - 1 && tid < 5) {
        const S* ps = sm_psum + ((k + 1) & 1) * NW * 5;
        S t = ps[tid];
        for (int w = 1; w < NW; ++w) t += ps[w * 5 + tid];
        part[5 * (k + 1) + tid] = t;
      }
      S l0, l1;
      chain_thread_state<S, C>(sec, wt, hin, warp, lane, e0, e1, l0, l1);
      l0 += gi0;
      l1 += gi1;
      // phase B: replay from the true state; g becomes the gradient w.r.t. the section's input
      S s0 = S(0), s1 = S(0), s2 = S(0), s3 = S(0), s4 = S(0);
      auto replay = [&](auto full_tag) {
        constexpr bool FULL = decltype(full_tag)::value;
        if (p.want_coef) {
          const unsigned char* xs = zbuf(k) + (size_t)tpos * SPT * sizeof(S);
          const unsigned char* ys = zbuf(k + 1) + (size_t)tpos * SPT * sizeof(S);
          // float32: (s1, s2) and (s3, s4) as packed pairs, two sums per fma.rn.f32x2 (1.074 -> 1.055 ms at K = 6)
          float2 sx = make_float2(0.f, 0.f), sy = make_float2(0.f, 0.f);
#pragma unroll
          for (int cc = CH - 1; cc >= 0; --cc) {
            S xv[V], yv[V];
            VecIO<S, V>::ld(xs + 16 * cc, xv);
            VecIO<S, V>::ld(ys + 16 * cc, yv);
#pragma unroll
            for (int q = V - 1; q >= 0; --q) {
              const int j = cc * V + q;
              if (FULL || j < nv) {
                const S gj = g[j];
                g[j] = c.b0 * gj + c.B0 * l0 + c.B1 * l1;
                s0 += gj * xv[q];
                if constexpr (std::is_same<S, float>::value) {
                  const float2 l = make_float2(l0, l1);
                  sx = __ffma2_rn(make_float2(xv[q], xv[q]), l, sx);
                  sy = __ffma2_rn(make_float2(yv[q], yv[q]), l, sy);
                } else {
                  s1 += xv[q] * l0;
                  s2 += xv[q] * l1;
                  s3 += yv[q] * l0;
                  s4 += yv[q] * l1;
                }
                const S t = c.na2 * l1 + gj;
                l1 = l0;
                l0 = c.na1 * l0 + t;
              }
            }
          }
          if constexpr (std::is_same<S, float>::value) { s1 += sx.x; s2 += sx.y; s3 += sy.x; s4 += sy.y; }
        } else {
#pragma unroll
          for (int j = SPT - 1; j >= 0; --j) {
            if (FULL || j < nv) {
              const S gj = g[j];
              g[j] = c.b0 * gj + c.B0 * l0 + c.B1 * l1;
              const S t = c.na2 * l1 + gj;
              l1 = l0;
              l0 = c.na1 * l0 + t;
            }
          }
        }
      };
      if (full_tile) replay(std::true_type{});
      else replay(std::false_type{});
      if (tid == NT - 1) {
        if (chunk + 1 < nchunks) chain_publish<S>(mine_slot + k * (C::SLOT_WORDS / K), l0, l1);
        else if (p.grad_zi) {
          p.grad_zi[((int64_t)k * p.B + row) * 2] = l0;
          p.grad_zi[((int64_t)k * p.B + row) * 2 + 1] = l1;
        }
      }
      if (p.want_coef) {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
          s0 += __shfl_down_sync(0xffffffffu, s0, d);
          s1 += __shfl_down_sync(0xffffffffu, s1, d);
          s2 += __shfl_down_sync(0xffffffffu, s2, d);
          s3 += __shfl_down_sync(0xffffffffu, s3, d);
          s4 += __shfl_down_sync(0xffffffffu, s4, d);
        }
        if (lane == 0) {
          S* ps = sm_psum + (k & 1) * NW * 5 + warp * 5;
          ps[0] = s0; ps[1] = s1; ps[2] = s2; ps[3] = s3; ps[4] = s4;
        }
        if (!bulk && k >= 1) {   // plain-load path: the next section's input array, after everyone left its buffer
          __syncthreads();
          zcopy(k - 1);
        }
      }
    }
    // grad_x out through ring buffer 2 (free since section 1; the tile buffer already holds the next tile)
    unsigned char* gout = smem + L::kZ + 2 * C::TILE_BYTES;
    if (!p.want_coef && bulk && tid == 0) bulk_wait_read_all();   // (with the sums: waited for before the ring was refilled)
    if (!p.want_coef) __syncthreads();
    {
      unsigned char* po = gout + (size_t)tpos * SPT * sizeof(S);
#pragma unroll
      for (int cc = 0; cc < CH; ++cc) VecIO<S, V>::st(po + 16 * cc, &g[cc * V]);
    }
    if (bulk) fence_proxy_async_smem();
    __syncthreads();
    if (p.want_coef && tid < 5) {   // the sums of section 0
      const S* ps = sm_psum;
      S t = ps[tid];
      for (int w = 1; w < NW; ++w) t += ps[w * 5 + tid];
      part[tid] = t;
    }
    S* dst = p.grad_x + (int64_t)row * p.T + t0;
    if (bulk) {
      if (tid == 0) {
        bulk_s2g(dst, gout, tile_bytes);
        bulk_commit();
      }
    } else {
      const uint32_t* so = reinterpret_cast<const uint32_t*>(gout);
      uint32_t* go = reinterpret_cast<uint32_t*>(dst);
      for (uint32_t w = tid; w < tile_bytes / 4; w += NT) go[w] = so[w];
    }
    __syncthreads();   // the tile's scratch is free
  }
  if (tid == 0) bulk_wait_all();
}

}  // namespace ptb
