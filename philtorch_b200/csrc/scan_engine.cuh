// Single-pass chunked scan engine with decoupled look-back for affine recurrences
//     h[t] = A[t] * h[t-1] + v[t]          (scalar or 2x2, forward or reversed in time)
// on B independent rows of length T.
//
// Work decomposition
//   * A row is cut into time chunks ("tiles") of P::TILE samples.  Tiles are handed out by an
//     atomic ticket in chunk-major order (ticket -> chunk = ticket / B, row = ticket % B), so the
//     predecessor of a tile (same row, previous chunk) is B tickets older and has normally
//     published its end state before the tile asks for it; a CTA only ever waits on OLDER
//     tickets, which are held by running CTAs, so the look-back cannot deadlock.
//   * One CTA = P::NT compute threads + one DMA warp.  Lane 0 of the DMA warp owns the ticket
//     counter, issues the 1-D bulk (TMA) loads of a tile's operands into a ring of P::STAGES
//     shared-memory stages (mbarrier transaction counts signal arrival) and, once the compute
//     warps have written the tile's results back into the same stage, issues the bulk stores.
//   * Compute thread i owns P::SPT consecutive samples of the tile.  P::SPT is chosen so that the
//     per-thread footprint of every staged array is an ODD number of 16-byte (or 8-byte) units,
//     which makes the strided 128-bit / 64-bit shared-memory accesses bank-conflict free without
//     swizzling.  Each thread folds its samples into one affine map, maps are scanned with warp
//     shuffles, warp totals are scanned by warp 0, the tile aggregate is published
//     (flag 1) and warp 0 looks back over predecessor tiles -- 32 at a time -- until it meets
//     an end state (flag 2).  The tile's end state is published (flag 2) and every thread
//     replays its samples from its own incoming state.
//
// All waits are bounded; on expiry an error bit is set in the workspace and the kernel runs to
// completion (results are then invalid, the host reports the error).
//
// The association order of the look-back depends on which predecessors had already published
// an end state, so floating-point results can differ in the last bits from run to run, as with
// any decoupled look-back scan.
#pragma once
#include "ptx.cuh"

namespace ptb {

constexpr uint32_t kNoTile = 0xFFFFFFFFu;
constexpr uint32_t kErrLookbackTimeout = 1u;
constexpr uint32_t kErrLoadTimeout = 2u;
constexpr uint32_t kErrDrainTimeout = 4u;
constexpr uint32_t kSpinLimit = 1u << 22;   // polls (each >= 64 ns once backed off): a few tenths of a second
constexpr uint32_t kSpinLimitAfterError = 1u << 8;

struct Workspace {
  uint32_t* ticket;   // [1]   zeroed before launch
  uint32_t* error;    // [1]   sticky error bits
  uint32_t* flags;    // [ntiles] zeroed before launch: 0 empty, 1 aggregate ready, 2 end state ready
  void* agg;          // [ntiles] Map
  void* incl;         // [ntiles] State
  void* partial;      // [ntiles] P::Partial (policy specific), may be null
};

constexpr int kMaxIo = 4;
struct IoPlan {
  uint32_t ld_soff[kMaxIo];
  uint32_t ld_bytes[kMaxIo];
  const char* ld_g[kMaxIo];
  int nld;
  uint32_t st_soff[kMaxIo];
  uint32_t st_bytes[kMaxIo];
  char* st_g[kMaxIo];
  int nst;
  __device__ __forceinline__ void load(uint32_t soff, const void* g, uint32_t bytes) {
    ld_soff[nld] = soff; ld_g[nld] = static_cast<const char*>(g); ld_bytes[nld] = bytes; ++nld;
  }
  __device__ __forceinline__ void store(uint32_t soff, void* g, uint32_t bytes) {
    st_soff[nst] = soff; st_g[nst] = static_cast<char*>(g); st_bytes[nst] = bytes; ++nst;
  }
};

// ---- small helpers on POD structs made of scalars `v[N]` ---------------------------------------
template <class T>
__device__ __forceinline__ T shfl_up_pod(const T& x, int d) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = __shfl_up_sync(0xffffffffu, x.v[i], d);
  return r;
}
template <class T>
__device__ __forceinline__ T shfl_down_pod(const T& x, int d) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = __shfl_down_sync(0xffffffffu, x.v[i], d);
  return r;
}
template <class T>
__device__ __forceinline__ T shfl_pod(const T& x, int src) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = __shfl_sync(0xffffffffu, x.v[i], src);
  return r;
}
template <class T>
__device__ __forceinline__ void st_cg_pod(T* p, const T& x) {
#pragma unroll
  for (int i = 0; i < T::N; ++i) __stcg(&p->v[i], x.v[i]);
}
template <class T>
__device__ __forceinline__ T ld_cg_pod(const T* p) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = __ldcg(&p->v[i]);
  return r;
}

template <class P>
__device__ __forceinline__ typename P::Map warp_scan_inclusive(typename P::Map m, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    typename P::Map o = shfl_up_pod(m, d);
    if (lane >= d) m = P::compose(o, m);
  }
  return m;
}

// Look-back executed by all 32 lanes of compute warp 0.  Returns (in every lane) the state
// entering the tile.
template <class P>
__device__ __forceinline__ typename P::State lookback(const Workspace& ws, uint32_t ticket,
                                                      uint32_t chunk, uint32_t B, int lane,
                                                      uint32_t& failed) {
  using Map = typename P::Map;
  using State = typename P::State;
  const Map* aggs = static_cast<const Map*>(ws.agg);
  const State* incls = static_cast<const State*>(ws.incl);
  Map acc = P::identity();   // meaningful in lane 0: maps nearer to the tile than the window
  uint32_t base = 1;
  State result;
  while (true) {
    const uint32_t k = base + lane;
    const bool valid = k <= chunk;
    const size_t idx = valid ? (size_t)ticket - (size_t)k * B : 0;
    uint32_t flag = 0;
    if (valid) {
      const uint32_t limit = failed ? kSpinLimitAfterError : kSpinLimit;
      for (uint32_t it = 0; it < limit; ++it) {
        flag = ld_acquire_u32(ws.flags + idx);
        if (flag != 0) break;
        if (it > 16) __nanosleep(it > 256 ? 256 : 32);
      }
    }
    const bool timed_out = valid && flag == 0;
    if (__any_sync(0xffffffffu, timed_out)) {
      failed = 1;
      if (lane == 0) atomicOr(ws.error, kErrLookbackTimeout);
    }
    const uint32_t m2 = __ballot_sync(0xffffffffu, (valid && flag == 2) || timed_out || !valid);
    if (m2 & 1u) {   // common case: the immediate predecessor already has its end state
      State s = P::zero_state();
      if (lane == 0 && valid && flag == 2) s = ld_cg_pod(incls + idx);
      s = shfl_pod(s, 0);
      // fold with the nearer maps gathered so far (identity on the first window)
      Map a0 = shfl_pod(acc, 0);
      result = P::apply(a0, s);
      break;
    }
    const int j = m2 ? (__ffs(m2) - 1) : 32;
    Map m = P::identity();
    if (lane < j) {
      m = ld_cg_pod(aggs + idx);
    } else if (lane == j) {
      State s = P::zero_state();
      if (valid && flag == 2) s = ld_cg_pod(incls + idx);
      m = P::const_map(s);
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {   // ordered reduction: higher lane = earlier in the sequence
      Map o = shfl_down_pod(m, d);
      if (lane + d < 32) m = P::compose(o, m);
    }
    acc = P::compose(m, acc);   // window first, then the nearer maps
    if (m2) {
      Map a0 = shfl_pod(acc, 0);
      result = P::apply(a0, P::zero_state());   // acc ends in a constant map: its offset is the state
      break;
    }
    base += 32;
  }
  return result;
}

// --------------------------------------------------------------------------------------------------
// Policy requirements (see first_order.cuh for a worked example):
//   types   S, Map{S v[N]}, State{S v[N]}, Partial{S v[N]}, Params, Thread
//   consts  NT (compute threads, multiple of 32), SPT, TILE = NT*SPT, STAGES, STAGE_BYTES,
//           MIN_CTAS, REVERSE (process time descending), HAS_PARTIAL
//   static  identity(), zero_state(), const_map(State), compose(first, second), apply(Map, State),
//           plan(prm, bulk, row, t0, nvalid, IoPlan&), row_init(prm, row), row_final(prm, row, State)
//   Thread  load(prm, stage, tpos, row, t0, nvalid), aggregate() -> Map,
//           finish(prm, State in, stage, tpos, nvalid) -> Partial
// --------------------------------------------------------------------------------------------------
template <class P>
struct EngineSmem {
  static constexpr int kStagesBytes = P::STAGES * P::STAGE_BYTES;
  static constexpr int kNW = P::NT / 32;
  // after the stages:
  static constexpr int kFullOff = kStagesBytes;                       // u64 full[STAGES]
  static constexpr int kDoneOff = kFullOff + 8 * P::STAGES;           // u64 done[STAGES]
  static constexpr int kTicketOff = kDoneOff + 8 * P::STAGES;         // u32 tile_ticket[STAGES]
  static constexpr int kScratchOff = ((kTicketOff + 4 * P::STAGES + 15) / 16) * 16;
  static constexpr int kWtotOff = kScratchOff;                                          // Map wtot[NW]
  static constexpr int kWpreOff = kWtotOff + (int)sizeof(typename P::Map) * kNW;        // Map wpre[NW]
  static constexpr int kHinOff = kWpreOff + (int)sizeof(typename P::Map) * kNW;         // State hin
  static constexpr int kPartOff = ((kHinOff + (int)sizeof(typename P::State) + 15) / 16) * 16;  // Partial[NW]
  static constexpr int kTotal = kPartOff + (int)sizeof(typename P::Partial) * kNW + 16;
};

template <class P>
__device__ __forceinline__ void tile_coords(const typename P::Params& prm, uint32_t ticket, uint32_t B,
                                            uint32_t nchunks, int64_t T, uint32_t& chunk, uint32_t& row,
                                            int64_t& t0, int& nvalid) {
  chunk = ticket / B;
  row = ticket - chunk * B;
  const uint32_t tc = P::REVERSE ? (nchunks - 1 - chunk) : chunk;
  t0 = (int64_t)tc * P::TILE;
  const int64_t rem = T - t0;
  nvalid = rem < (int64_t)P::TILE ? (int)rem : P::TILE;
}

template <class P>
__global__ void __launch_bounds__(P::NT + 32, P::MIN_CTAS)
scan_kernel(const typename P::Params prm, const Workspace ws, const uint32_t B, const int64_t T,
            const uint32_t nchunks, const uint32_t ntiles, const int bulk) {
  using Map = typename P::Map;
  using State = typename P::State;
  using Partial = typename P::Partial;
  using L = EngineSmem<P>;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kFullOff);
  uint64_t* done = reinterpret_cast<uint64_t*>(smem + L::kDoneOff);
  volatile uint32_t* tile_ticket = reinterpret_cast<volatile uint32_t*>(smem + L::kTicketOff);
  Map* wtot = reinterpret_cast<Map*>(smem + L::kWtotOff);
  Map* wpre = reinterpret_cast<Map*>(smem + L::kWpreOff);
  State* sm_hin = reinterpret_cast<State*>(smem + L::kHinOff);
  Partial* sm_part = reinterpret_cast<Partial*>(smem + L::kPartOff);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  constexpr int NT = P::NT;
  constexpr int NW = NT / 32;
  constexpr int D = P::STAGES;

  if (tid == 0) {
    for (int s = 0; s < D; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], NT);
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (warp == NW) {
    // ======================================================================= DMA warp
    if (lane != 0) return;
    uint32_t failed = 0;
    uint32_t next = atomicAdd(ws.ticket, 1u);
    uint32_t n = 0;
    auto drain = [&](uint32_t j) {   // results of the j-th tile of this CTA are in its stage
      const int s = j % D;
      const uint32_t limit = failed ? kSpinLimitAfterError : kSpinLimit;
      if (!mbar_wait_bounded(&done[s], (j / D) & 1u, limit)) {
        failed = 1;
        atomicOr(ws.error, kErrDrainTimeout);
      }
      if (bulk) {
        uint32_t chunk, row; int64_t t0; int nvalid;
        tile_coords<P>(prm, tile_ticket[s], B, nchunks, T, chunk, row, t0, nvalid);
        IoPlan io; io.nld = 0; io.nst = 0;
        P::plan(prm, true, row, t0, nvalid, io);
        unsigned char* stage = smem + s * P::STAGE_BYTES;
        for (int i = 0; i < io.nst; ++i)
          if (io.st_bytes[i]) bulk_s2g(io.st_g[i], stage + io.st_soff[i], io.st_bytes[i]);
        bulk_commit();
        bulk_wait_read_all();   // the stage may be overwritten from here on
      }
    };
    for (;; ++n) {
      const int s = n % D;
      if (n >= (uint32_t)D) drain(n - D);
      const uint32_t ticket = next;
      if (ticket >= ntiles) {
        tile_ticket[s] = kNoTile;
        mbar_arrive(&full[s]);
        break;
      }
      next = atomicAdd(ws.ticket, 1u);
      tile_ticket[s] = ticket;
      if (bulk) {
        uint32_t chunk, row; int64_t t0; int nvalid;
        tile_coords<P>(prm, ticket, B, nchunks, T, chunk, row, t0, nvalid);
        IoPlan io; io.nld = 0; io.nst = 0;
        P::plan(prm, true, row, t0, nvalid, io);
        uint32_t total = 0;
        for (int i = 0; i < io.nld; ++i) total += io.ld_bytes[i];
        mbar_arrive_expect_tx(&full[s], total);
        unsigned char* stage = smem + s * P::STAGE_BYTES;
        for (int i = 0; i < io.nld; ++i)
          if (io.ld_bytes[i]) bulk_g2s(stage + io.ld_soff[i], io.ld_g[i], io.ld_bytes[i], &full[s]);
      } else {
        mbar_arrive(&full[s]);
      }
    }
    // n = index of the terminal slot; tiles n-D+1 .. n-1 are still in their stages
    for (uint32_t j = (n >= (uint32_t)D ? n - D + 1 : 0); j < n; ++j) drain(j);
    if (bulk) bulk_wait_all();
    return;
  }

  // ========================================================================= compute warps
  uint32_t failed = 0;
  for (uint32_t n = 0;; ++n) {
    const int s = n % D;
    {
      const uint32_t limit = failed ? kSpinLimitAfterError : kSpinLimit;
      if (!mbar_wait_bounded(&full[s], (n / D) & 1u, limit)) {
        failed = 1;
        if (lane == 0) atomicOr(ws.error, kErrLoadTimeout);
      }
    }
    const uint32_t ticket = tile_ticket[s];
    if (ticket == kNoTile) break;
    uint32_t chunk, row; int64_t t0; int nvalid;
    tile_coords<P>(prm, ticket, B, nchunks, T, chunk, row, t0, nvalid);
    unsigned char* stage = smem + s * P::STAGE_BYTES;

    if (!bulk) {   // operands that are not 16-byte aligned: cooperative word copies
      IoPlan io; io.nld = 0; io.nst = 0;
      P::plan(prm, false, row, t0, nvalid, io);
      for (int i = 0; i < io.nld; ++i) {
        const uint32_t* g = reinterpret_cast<const uint32_t*>(io.ld_g[i]);
        uint32_t* d = reinterpret_cast<uint32_t*>(stage + io.ld_soff[i]);
        const uint32_t nw = io.ld_bytes[i] >> 2;
        for (uint32_t w = tid; w < nw; w += NT) d[w] = __ldg(g + w);
      }
      bar_sync(1, NT);
    }

    const int tpos = P::REVERSE ? (NT - 1 - tid) : tid;
    typename P::Thread th;
    th.load(prm, stage, tpos, row, t0, nvalid);
    const Map mine = th.aggregate();
    const Map inc = warp_scan_inclusive<P>(mine, lane);
    if (lane == 31) wtot[warp] = inc;
    Map exc = shfl_up_pod(inc, 1);
    if (lane == 0) exc = P::identity();
    bar_sync(1, NT);   // (A) warp totals visible, every thread holds its operands in registers

    if (warp == 0) {
      Map w = lane < NW ? wtot[lane] : P::identity();
      const Map winc = warp_scan_inclusive<P>(w, lane);
      Map wexc = shfl_up_pod(winc, 1);
      if (lane == 0) wexc = P::identity();
      if (lane < NW) wpre[lane] = wexc;
      const Map tile_agg = shfl_pod(winc, NW - 1);
      State hin;
      if (chunk == 0) {
        hin = P::row_init(prm, row);
      } else {
        if (lane == 0) {
          st_cg_pod(static_cast<Map*>(ws.agg) + ticket, tile_agg);
          st_release_u32(ws.flags + ticket, 1u);
        }
        hin = lookback<P>(ws, ticket, chunk, B, lane, failed);
      }
      if (lane == 0) {
        const State hend = P::apply(tile_agg, hin);
        st_cg_pod(static_cast<State*>(ws.incl) + ticket, hend);
        st_release_u32(ws.flags + ticket, 2u);
        *sm_hin = hin;
        if (chunk == nchunks - 1) P::row_final(prm, row, hend);
      }
    }
    bar_sync(1, NT);   // (B) incoming state and warp prefixes visible

    const State hin = *sm_hin;
    const Map pre = P::compose(wpre[warp], exc);
    Partial part = th.finish(prm, P::apply(pre, hin), stage, tpos, nvalid);

    if (P::HAS_PARTIAL) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        Partial o = shfl_down_pod(part, d);
#pragma unroll
        for (int i = 0; i < Partial::N; ++i) part.v[i] += o.v[i];
      }
      if (lane == 0) sm_part[warp] = part;
    }

    if (bulk) {
      fence_proxy_async_smem();
      mbar_arrive(&done[s]);
      if (P::HAS_PARTIAL) {
        bar_sync(1, NT);
        if (tid == 0) {
          Partial tot = sm_part[0];
          for (int w2 = 1; w2 < NW; ++w2)
#pragma unroll
            for (int i = 0; i < Partial::N; ++i) tot.v[i] += sm_part[w2].v[i];
          static_cast<Partial*>(ws.partial)[(size_t)row * nchunks + chunk] = tot;
        }
      }
    } else {
      bar_sync(1, NT);
      if (P::HAS_PARTIAL && tid == 0) {
        Partial tot = sm_part[0];
        for (int w2 = 1; w2 < NW; ++w2)
#pragma unroll
          for (int i = 0; i < Partial::N; ++i) tot.v[i] += sm_part[w2].v[i];
        static_cast<Partial*>(ws.partial)[(size_t)row * nchunks + chunk] = tot;
      }
      IoPlan io; io.nld = 0; io.nst = 0;
      P::plan(prm, false, row, t0, nvalid, io);
      for (int i = 0; i < io.nst; ++i) {
        uint32_t* g = reinterpret_cast<uint32_t*>(io.st_g[i]);
        const uint32_t* d = reinterpret_cast<const uint32_t*>(stage + io.st_soff[i]);
        const uint32_t nw = io.st_bytes[i] >> 2;
        for (uint32_t w = tid; w < nw; w += NT) g[w] = d[w];
      }
      mbar_arrive(&done[s]);
    }
  }
}

}  // namespace ptb
