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
//   * One CTA = P::NT compute threads + P::LBW look-back warps + one DMA warp, decoupled by
//     shared-memory mbarriers (no CTA-wide barrier on the bulk path):
//       DMA warp (lane 0)   owns the ticket counter, issues the 1-D bulk (TMA) loads of a tile's
//                           operands into a ring of P::STAGES shared-memory stages and, once the
//                           compute warps have written the tile's results back into the stage,
//                           the bulk stores.
//       compute warps       event loop.  Phase 1 (as soon as a tile's operands have landed): every
//                           thread folds its P::SPT consecutive samples into one affine map, maps
//                           are scanned with warp shuffles, the last warp to arrive scans the warp
//                           totals and PUBLISHES the tile aggregate (flag 1) at once, so successors
//                           never wait for this CTA's look-back.  Phase 2 (as soon as the tile's
//                           incoming state is known): every thread replays its samples from its
//                           own incoming state and writes the results into the stage.
//       look-back warp      starts as soon as the tile's ticket is known (it needs nothing from the
//                           tile's own operands, so it overlaps their load): looks back over
//                           predecessor tiles, one per lane, until it meets an end state (flag 2),
//                           hands the incoming state to the compute warps and, once the tile
//                           aggregate is known, publishes the tile's end state.
//   * Tiles are large (tens of KB per array and bulk copy) and there is one CTA per SM: large
//     contiguous requests are what the memory system serves fastest; 2-4 stages fill the SM's
//     shared memory.
//   * P::SPT is chosen so that the per-thread footprint of every staged array is an ODD number of
//     16-byte (or 8-byte) units: the strided 128-bit / 64-bit shared-memory accesses are then
//     bank-conflict free without swizzling.
//   * Published records need no fences: every 32-bit payload word travels in its own 64-bit word
//     next to the flag, written and read with single relaxed 64-bit accesses; a reader accepts a
//     record only when all its words carry the same flag.
//
// All waits are bounded; on expiry an error bit is set and the kernel runs to completion
// (results are then invalid, the host reports the error).
//
// The association order of the look-back depends on which predecessors had already published
// an end state, so floating-point results can differ in the last bits from run to run, as with
// any decoupled look-back scan.
#pragma once
#include "ptx.cuh"
#include "complex.cuh"

#include <type_traits>

namespace ptb {

// Policies whose maps are self-contained (they carry their own linear part) need no context:
// this macro, expanded inside the algebra struct after compose/apply, supplies the context-taking
// forms the engine calls.  Policies whose linear part is implicit (a per-row table of matrix
// powers, see sos_cascade.cuh) define Ctx, ctx_stage, ctx_row and the three functions themselves.
#define PTB_NO_CTX                                                                                       \
  using Ctx = int;                                                                                       \
  static __device__ __forceinline__ Ctx ctx_stage(const unsigned char*) { return 0; }                    \
  template <class Pr_>                                                                                   \
  static __device__ __forceinline__ Ctx ctx_row(const Pr_&, int64_t) { return 0; }                       \
  static __device__ __forceinline__ Map compose(Ctx, const Map& a, const Map& b) { return compose(a, b); } \
  static __device__ __forceinline__ State apply(Ctx, const Map& m, const State& s) { return apply(m, s); } \
  static __device__ __forceinline__ State thread_state(Ctx, const Map& wp, const Map& e, const State& hin, \
                                                       int) {                                            \
    return apply(compose(wp, e), hin);                                                                   \
  }                                                                                                      \
  /* inclusive scan over the lanes of a warp (level 0: threads of a warp, 1: warps of a tile) */         \
  static __device__ __forceinline__ Map warp_scan(Ctx, Map m, int lane, int) {                           \
    _Pragma("unroll") for (int d = 1; d < 32; d <<= 1) {                                                 \
      Map o = shfl_up_pod(m, d);                                                                         \
      if (lane >= d) m = compose(o, m);                                                                  \
    }                                                                                                    \
    return m;                                                                                            \
  }

// Optional policy member FINAL_REDUCE = true with wants_final_reduce(prm) and
// final_reduce(prm, partial, B, nchunks, lane): the last compute warp of the whole grid to finish adds
// up the per-tile partial sums (one warp, fixed order) instead of a second launch.
template <class P, class = void>
struct FinalReduceOf { static constexpr bool value = false; };
template <class P>
struct FinalReduceOf<P, std::void_t<decltype(P::FINAL_REDUCE)>> { static constexpr bool value = P::FINAL_REDUCE; };

// Optional policy members: EXTRA_SMEM bytes of policy-owned shared memory behind the engine's
// (with init_extra / prefetch / finish_x hooks, see scan_kernel).
template <class P, class = void>
struct ExtraSmemOf { static constexpr int value = 0; };
template <class P>
struct ExtraSmemOf<P, std::void_t<decltype(P::EXTRA_SMEM)>> { static constexpr int value = P::EXTRA_SMEM; };

constexpr uint32_t kNoTile = 0xFFFFFFFFu;
constexpr uint32_t kErrLookbackTimeout = 1u;
constexpr uint32_t kErrLoadTimeout = 2u;
constexpr uint32_t kErrDrainTimeout = 4u;
constexpr uint32_t kErrPipeTimeout = 8u;
constexpr uint64_t kDefaultWaitNs = 2000000000ull;  // any single device-side wait gives up after 2 s (default)
constexpr uint64_t kWaitNsAfterError = 1000000ull;   // ... or after 1 ms once this CTA has seen an error

// Optional role-level timing (compile with -DPTB_PROFILE): cycles each role spends waiting,
// summed over CTAs into 64-bit counters that follow the workspace header.
#ifdef PTB_PROFILE
#define PTB_PROF_DECL(name) long long name = 0
#define PTB_PROF_BEGIN(t) const long long t = clock64()
#define PTB_PROF_END(name, t) name += clock64() - t
#define PTB_PROF_FLUSH(idx, name) atomicAdd(reinterpret_cast<unsigned long long*>(ws.ticket) + 8 + (idx), (unsigned long long)(name))
#else
#define PTB_PROF_DECL(name)
#define PTB_PROF_BEGIN(t)
#define PTB_PROF_END(name, t)
#define PTB_PROF_FLUSH(idx, name)
#endif

// Optional event trace of CTA 0 (compile with -DPTB_TRACE): {clock:48 | tile:12 | event:4} words
// written over the (otherwise unused) partial area of the workspace.
#ifdef PTB_TRACE
#define PTB_EV(type, n)                                                                         \
  do {                                                                                          \
    if (blockIdx.x == 0) {                                                                      \
      const unsigned ei_ = atomicAdd(sm_trace_cnt, 1u);                                         \
      if (ei_ < 8000u)                                                                          \
        reinterpret_cast<unsigned long long*>(ws.partial)[ei_] =                                \
            ((unsigned long long)clock64() << 16) | (((unsigned long long)(n) & 0xfffu) << 4) | (type); \
    }                                                                                           \
  } while (0)
#else
#define PTB_EV(type, n)
#endif

struct Workspace {
  uint32_t* ticket;   // [1]   zeroed before launch
  uint32_t* error;    // [1]   sticky error bits
  uint64_t* slots;    // [ntiles][P::SLOT_WORDS] zeroed before launch: {flag:32 | payload word:32}
  void* partial;      // [ntiles] P::Partial (policy specific)
  uint32_t* done = nullptr;   // [1] zeroed before launch: compute warps that have finished (policies with a final reduction)
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
  int st_add[kMaxIo];   // 0: plain store; 4 / 8: add into the destination as 4- / 8-byte floats (bulk path only)
  int nst;
  __device__ __forceinline__ void load(uint32_t soff, const void* g, uint32_t bytes) {
    ld_soff[nld] = soff; ld_g[nld] = static_cast<const char*>(g); ld_bytes[nld] = bytes; ++nld;
  }
  __device__ __forceinline__ void store(uint32_t soff, void* g, uint32_t bytes, int add = 0) {
    st_soff[nst] = soff; st_g[nst] = static_cast<char*>(g); st_bytes[nst] = bytes; st_add[nst] = add; ++nst;
  }
};

// ---- small helpers on POD structs made of scalars `v[N]` ---------------------------------------
template <class T>
__device__ __forceinline__ T shfl_up_pod(const T& x, int d) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = shfl_up_s(x.v[i], d);
  return r;
}
template <class T>
__device__ __forceinline__ T shfl_down_pod(const T& x, int d) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = shfl_down_s(x.v[i], d);
  return r;
}
template <class T>
__device__ __forceinline__ T shfl_pod(const T& x, int src) {
  T r;
#pragma unroll
  for (int i = 0; i < T::N; ++i) r.v[i] = shfl_s(x.v[i], src);
  return r;
}

// ---- published records --------------------------------------------------------------------------
template <class T>
struct Words {
  static constexpr int W = (int)(sizeof(T) / 4);
  union U { T t; uint32_t w[W]; };
};
template <class T>
__device__ __forceinline__ void slot_store(uint64_t* slot, const T& v, uint32_t flag) {
  typename Words<T>::U u;
  u.t = v;
#pragma unroll
  for (int i = 0; i < Words<T>::W; ++i) st_relaxed_u64(slot + i, ((uint64_t)flag << 32) | u.w[i]);
}
// fetch the raw words of a record (all loads in flight together) ...
template <class Map>
__device__ __forceinline__ void slot_fetch(const uint64_t* slot, uint64_t* r) {
#pragma unroll
  for (int i = 0; i < Words<Map>::W; ++i) r[i] = ld_relaxed_u64(slot + i);
}
// ... and decode them.  0: nothing usable yet, 1: aggregate in `m`, 2: end state in `st`
template <class Map, class State>
__device__ __forceinline__ uint32_t slot_decode(const uint64_t* r, Map& m, State& st) {
  constexpr int WM = Words<Map>::W, WS = Words<State>::W;
  static_assert(WS <= WM, "end states are stored in the first words of the aggregate's slot");
  const uint32_t f0 = (uint32_t)(r[0] >> 32);
  bool ok2 = true, ok1 = true;
  typename Words<State>::U us;
  typename Words<Map>::U um;
#pragma unroll
  for (int i = 0; i < WS; ++i) { ok2 = ok2 && ((uint32_t)(r[i] >> 32) == 2u); us.w[i] = (uint32_t)r[i]; }
#pragma unroll
  for (int i = 0; i < WM; ++i) { ok1 = ok1 && ((uint32_t)(r[i] >> 32) == 1u); um.w[i] = (uint32_t)r[i]; }
  st = us.t;
  m = um.t;
  return (f0 == 2u && ok2) ? 2u : ((f0 == 1u && ok1) ? 1u : 0u);
}

// Look-back executed by all 32 lanes of a look-back warp; returns (in every lane) the state
// entering the tile.  Windows of predecessors (one per lane, all loads in flight together) are
// folded until one contains an end state.  The look-back starts as soon as the tile's ticket is
// known, usually before the predecessors have published anything, so the first window is only
// `first_window` lanes wide (8 when the batch is large enough that a row has few tiles in flight,
// 32 for a handful of long rows) and polls with a back-off: that keeps the polling traffic in L2
// small.  Later windows are 32 wide.
template <class P>
__device__ __forceinline__ typename P::State lookback(const typename P::Ctx& ctx, const Workspace& ws, uint32_t ticket,
                                                      uint32_t chunk, uint32_t B, int lane,
                                                      uint32_t& failed, int first_window, uint64_t kWaitNs) {
  using Map = typename P::Map;
  using State = typename P::State;
  Map acc = P::identity();
  uint32_t base = 1;
  int wsize = first_window;
  State result;
  while (true) {
    const uint32_t k = base + lane;
    const bool active = lane < wsize;
    const bool valid = active && k <= chunk;
    const size_t idx = valid ? (size_t)ticket - (size_t)k * B : 0;
    uint32_t flag = 0;
    Map m = P::identity();
    State st = P::zero_state();
    if (valid) {
      const uint64_t* slot = ws.slots + idx * P::SLOT_WORDS;
      const uint64_t limit = failed ? kWaitNsAfterError : kWaitNs;
      uint64_t t0 = 0;
      for (uint32_t it = 0;; ++it) {
        uint64_t raw[Words<Map>::W];
        slot_fetch<Map>(slot, raw);
        flag = slot_decode<Map, State>(raw, m, st);
        if (flag != 0) break;
        if (it > 1) __nanosleep(it > 64 ? 400 : 100);
        if (it == 64) t0 = globaltimer_ns();
        if (it > 64 && globaltimer_ns() - t0 > limit) break;
      }
    }
    const bool timed_out = valid && flag == 0;
    if (__any_sync(0xffffffffu, timed_out)) {
      failed = 1;
      if (lane == 0) atomicOr(ws.error, kErrLookbackTimeout);
    }
    // lanes of the window that end the walk: an end state, a wait that expired, the row start
    const uint32_t m2 = __ballot_sync(0xffffffffu, active && ((valid && flag == 2) || timed_out || !valid));
    if (m2 & 1u) {
      const State s = shfl_pod(st, 0);
      const Map a0 = shfl_pod(acc, 0);
      result = P::apply(ctx, a0, s);
      break;
    }
    const int j = m2 ? (__ffs(m2) - 1) : 32;
    if (lane == j) m = P::const_map((valid && flag == 2) ? st : P::zero_state());
    else if (lane > j || !active) m = P::identity();
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      Map o = shfl_down_pod(m, d);
      if (lane + d < 32) m = P::compose(ctx, o, m);
    }
    acc = P::compose(ctx, m, acc);
    if (m2) {
      const Map a0 = shfl_pod(acc, 0);
      result = P::apply(ctx, a0, P::zero_state());
      break;
    }
    base += wsize;
    wsize = 32;
  }
  return result;
}

// --------------------------------------------------------------------------------------------------
// Policy requirements (see first_order.cuh for a worked example):
//   types   S, Map{S v[N]}, State{S v[N]}, Partial{S v[N]}, Params
//   consts  NT (compute threads, multiple of 32), SPT, TILE = NT*SPT, STAGES, STAGE_BYTES,
//           MIN_CTAS, REVERSE (process time descending), HAS_PARTIAL, SLOT_WORDS,
//           NROWC / ROWC_OFF / row_constants(prm, row, Scalar*): per-row constants the DMA warp
//           places at ROWC_OFF of the stage (0 = none)
//   static  identity(), zero_state(), const_map(State), compose(first, second), apply(Map, State),
//           plan(prm, bulk, row, t0, nvalid, IoPlan&), row_init(prm, row), row_final(prm, row, State),
//           aggregate(prm, stage, tpos, row, t0, nvalid) -> Map          (phase 1, reads the stage)
//           finish(prm, State in, stage, tpos, row, t0, nvalid) -> Partial (phase 2, reads and
//                                                                          overwrites the stage)
//           Ctx, ctx_stage(stage), ctx_row(prm, row), compose/apply(ctx, ...), thread_state(ctx,
//           warp prefix, thread prefix, tile-incoming state, lane), warp_scan(ctx, map, lane, level):
//           PTB_NO_CTX unless the linear
//           part of the maps lives in a per-row table
//   optional EXTRA_SMEM > 0: init_extra(extra) (one thread, before the first tile),
//           prefetch(prm, extra, seq, warp, lane, row, t0, nvalid) (per warp, once per tile, after
//           the previous tile's phase 2), finish_x(prm, in, stage, extra, seq, warp, lane, row, t0,
//           nvalid, wait_ns) instead of finish; seq = number of tiles this CTA finished before
// --------------------------------------------------------------------------------------------------
template <class P>
struct EngineSmem {
  static constexpr int D = P::STAGES;
  static constexpr int kStagesBytes = D * P::STAGE_BYTES;
  static constexpr int kNW = P::NT / 32;
  static constexpr int kMapB = (int)sizeof(typename P::Map);
  static constexpr int kStateB = (int)sizeof(typename P::State);
  static constexpr int kFullOff = kStagesBytes;            // u64 full[D]      operands landed
  static constexpr int kDoneOff = kFullOff + 8 * D;        // u64 done[D]      results written to the stage
  static constexpr int kAggOff = kDoneOff + 8 * D;         // u64 agg_ready[D] tile aggregate known
  static constexpr int kLbOff = kAggOff + 8 * D;           // u64 lb_done[D]   incoming state known
  static constexpr int kIssuedOff = kLbOff + 8 * D;        // u64 issued[D]    ticket of the stage known
  static constexpr int kSyncOff = kIssuedOff + 8 * D;      // u64 sync_bar[3]  barriers among the compute threads
  static constexpr int kTicketOff = kSyncOff + 8 * 3;      // u32 tile_ticket[D]
  static constexpr int kCntOff = kTicketOff + 4 * D;       // u32 arrived[D]
  static constexpr int kAbortOff = kCntOff + 4 * D;        // u32 abort, u32 trace counter
  static constexpr int kWtotOff = ((kAbortOff + 8 + 15) / 16) * 16;   // Map wtot[D][NW]
  static constexpr int kWpreOff = kWtotOff + D * kMapB * kNW;         // Map wpre[D][NW]
  static constexpr int kTaggOff = kWpreOff + D * kMapB * kNW;         // Map tile_agg[D]
  static constexpr int kHinOff = kTaggOff + D * kMapB;                // State hin[D]
  static constexpr int kPcntOff = kHinOff + D * kStateB;              // u32 partial arrivals[D]
  static constexpr int kPartOff = ((kPcntOff + 4 * D + 15) / 16) * 16;   // Partial[D][NW]
  static constexpr int kExtraOff = ((kPartOff + (int)sizeof(typename P::Partial) * kNW * D + 16 + 127) / 128) * 128;
  static constexpr int kExtra = ExtraSmemOf<P>::value;   // policy-owned area
  static constexpr int kTotal = kExtraOff + kExtra;
};

struct TileCoords {
  uint32_t ticket, chunk, row;
  int64_t t0;
  int nvalid;
};

template <class P>
__device__ __forceinline__ TileCoords tile_coords(uint32_t ticket, uint32_t B, uint32_t nchunks, int64_t T) {
  TileCoords c;
  c.ticket = ticket;
  c.chunk = ticket / B;
  c.row = ticket - c.chunk * B;
  const uint32_t tc = P::REVERSE ? (nchunks - 1 - c.chunk) : c.chunk;
  c.t0 = (int64_t)tc * P::TILE;
  const int64_t rem = T - c.t0;
  c.nvalid = rem < (int64_t)P::TILE ? (int)rem : P::TILE;
  return c;
}

template <class P>
__global__ void __launch_bounds__(P::NT + 32 * (P::LBW + 1), P::MIN_CTAS)
scan_kernel(const typename P::Params prm, const Workspace ws, const uint32_t B, const int64_t T,
            const uint32_t nchunks, const uint32_t ntiles, const int bulk, const int lb_first, const uint64_t kWaitNs) {
  using Map = typename P::Map;
  using State = typename P::State;
  using Partial = typename P::Partial;
  using L = EngineSmem<P>;
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kFullOff);
  uint64_t* done = reinterpret_cast<uint64_t*>(smem + L::kDoneOff);
  uint64_t* agg_ready = reinterpret_cast<uint64_t*>(smem + L::kAggOff);
  uint64_t* lb_done = reinterpret_cast<uint64_t*>(smem + L::kLbOff);
  uint64_t* issued = reinterpret_cast<uint64_t*>(smem + L::kIssuedOff);
  uint64_t* sync_bar = reinterpret_cast<uint64_t*>(smem + L::kSyncOff);
  volatile uint32_t* tile_ticket = reinterpret_cast<volatile uint32_t*>(smem + L::kTicketOff);
  uint32_t* sm_cnt = reinterpret_cast<uint32_t*>(smem + L::kCntOff);
  volatile uint32_t* sm_abort = reinterpret_cast<volatile uint32_t*>(smem + L::kAbortOff);
#ifdef PTB_TRACE
  uint32_t* sm_trace_cnt = reinterpret_cast<uint32_t*>(smem + L::kAbortOff + 4);
  if (threadIdx.x == 0) *sm_trace_cnt = 0;
#endif
  Map* wtot = reinterpret_cast<Map*>(smem + L::kWtotOff);
  Map* wpre = reinterpret_cast<Map*>(smem + L::kWpreOff);
  Map* sm_tagg = reinterpret_cast<Map*>(smem + L::kTaggOff);
  State* sm_hin = reinterpret_cast<State*>(smem + L::kHinOff);
  Partial* sm_part = reinterpret_cast<Partial*>(smem + L::kPartOff);
  uint32_t* sm_pcnt = reinterpret_cast<uint32_t*>(smem + L::kPcntOff);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  constexpr int NT = P::NT;
  constexpr int NW = NT / 32;
  constexpr int D = P::STAGES;
  static_assert(D >= 2, "at least two stages");

  if (tid == 0) {
    for (int s = 0; s < D; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], NT + 1);   // compute threads + the stage's look-back warp
      mbar_init(&agg_ready[s], 1);
      mbar_init(&lb_done[s], 1);
      mbar_init(&issued[s], 1);
      sm_cnt[s] = 0;
      sm_pcnt[s] = 0;
    }
    for (int i = 0; i < 3; ++i) mbar_init(&sync_bar[i], NT);
    if constexpr (L::kExtra > 0) P::init_extra(smem + L::kExtraOff);
    *sm_abort = 0;
    fence_mbar_init();
  }
  __syncthreads();

  constexpr int LBW = P::LBW;
  static_assert(LBW == 1 || LBW == D, "one look-back warp, or one per stage");
  if (warp == NW + LBW) {
    // ======================================================================= DMA warp
    if (lane != 0) return;
    uint32_t failed = 0;
    uint32_t next = atomicAdd(ws.ticket, 1u);
    uint32_t n = 0;
    // per-row constants (time-invariant coefficients) of the NEXT tile, fetched one iteration ahead
    // so that their latency hides behind the drain of an older tile; they travel with the stage
    constexpr int NR = P::NROWC;
    typename P::Scalar rc[NR > 0 ? NR : 1];
    if (NR > 0 && next < ntiles) P::row_constants(prm, (int64_t)(next % B), rc);
    PTB_PROF_DECL(t_wait_done); PTB_PROF_DECL(t_wait_read); PTB_PROF_DECL(t_dma_total);
    PTB_PROF_BEGIN(tdma0);
    auto drain = [&](uint32_t j) {   // results of the j-th tile of this CTA are in its stage
      const int s = j % D;
      const uint64_t limit = (failed || *sm_abort) ? kWaitNsAfterError : kWaitNs;
      PTB_PROF_BEGIN(tw0);
      if (!mbar_wait_bounded(&done[s], (j / D) & 1u, limit)) {
        failed = 1;
        atomicOr(ws.error, kErrDrainTimeout);
        return;   // the stage was not completed: nothing to store
      }
      PTB_PROF_END(t_wait_done, tw0);
      PTB_EV(8, j);
      if (bulk) {
        const TileCoords c = tile_coords<P>(tile_ticket[s], B, nchunks, T);
        IoPlan io; io.nld = 0; io.nst = 0;
        P::plan(prm, true, c.row, c.t0, c.nvalid, io);
        unsigned char* stage = smem + s * P::STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < kMaxIo; ++i)
          if (i < io.nst && io.st_bytes[i]) {
            if (io.st_add[i] == 4) bulk_s2g_add_f32(io.st_g[i], stage + io.st_soff[i], io.st_bytes[i]);
            else if (io.st_add[i] == 8) bulk_s2g_add_f64(io.st_g[i], stage + io.st_soff[i], io.st_bytes[i]);
            else bulk_s2g(io.st_g[i], stage + io.st_soff[i], io.st_bytes[i]);
          }
        bulk_commit();
        PTB_PROF_BEGIN(tr0);
        bulk_wait_read_all();   // the stage may be overwritten from here on
        PTB_PROF_END(t_wait_read, tr0);
        PTB_EV(9, j);
      }
    };
    for (;; ++n) {
      const int s = n % D;
      if (n >= (uint32_t)D) drain(n - D);
      const uint32_t ticket = (failed || *sm_abort) ? ntiles : next;   // stop handing out work after an error
      if (ticket >= ntiles) break;
      next = atomicAdd(ws.ticket, 1u);
      tile_ticket[s] = ticket;
      if (NR > 0) {
        typename P::Scalar* dst = reinterpret_cast<typename P::Scalar*>(smem + s * P::STAGE_BYTES + P::ROWC_OFF);
#pragma unroll
        for (int i = 0; i < NR; ++i) dst[i] = rc[i];
        if (next < ntiles) P::row_constants(prm, (int64_t)(next % B), rc);
      }
      PTB_EV(1, n);
      mbar_arrive(&issued[s]);   // the look-back of this tile may start: it needs nothing from the tile
      if (bulk) {
        const TileCoords c = tile_coords<P>(ticket, B, nchunks, T);
        IoPlan io; io.nld = 0; io.nst = 0;
        P::plan(prm, true, c.row, c.t0, c.nvalid, io);
        uint32_t total = 0;
#pragma unroll
        for (int i = 0; i < kMaxIo; ++i)
          if (i < io.nld) total += io.ld_bytes[i];
        mbar_arrive_expect_tx(&full[s], total);
        unsigned char* stage = smem + s * P::STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < kMaxIo; ++i)
          if (i < io.nld && io.ld_bytes[i]) bulk_g2s(stage + io.ld_soff[i], io.ld_g[i], io.ld_bytes[i], &full[s]);
      } else {
        mbar_arrive(&full[s]);
      }
    }
    // n = first index without a tile: put the end marker into every stage (with one look-back
    // warp per stage each watches its own), draining the tiles still held by the stages on the way
    for (uint32_t k = 0; k < (uint32_t)D; ++k) {
      const uint32_t m = n + k;
      const int s = m % D;
      if (k > 0 && m >= (uint32_t)D) drain(m - D);
      tile_ticket[s] = kNoTile;
      mbar_arrive(&issued[s]);
      mbar_arrive(&full[s]);
    }
    if (failed || *sm_abort) {
      // make sure no bulk load of this CTA is still writing shared memory when the CTA exits
      for (uint32_t j = (n >= (uint32_t)D ? n - D : 0); j < n; ++j)
        mbar_wait_bounded(&full[j % D], (j / D) & 1u, kWaitNs);
    }
    if (bulk) bulk_wait_all();
    PTB_PROF_END(t_dma_total, tdma0);
    PTB_PROF_FLUSH(0, t_wait_done); PTB_PROF_FLUSH(1, t_wait_read); PTB_PROF_FLUSH(2, t_dma_total);
    PTB_PROF_FLUSH(3, (long long)n);
    return;
  }

  if (warp >= NW) {
    // ======================================================================= look-back warps
    // Warp w handles the CTA's tiles w, w + LBW, w + 2 LBW, ...: all of them with LBW == 1, those of
    // stage w with LBW == D (the look-backs of the stages then overlap one another).
    uint32_t failed = 0;
    PTB_PROF_DECL(t_lb_wait_full); PTB_PROF_DECL(t_lb_wait_agg); PTB_PROF_DECL(t_lb_look); PTB_PROF_DECL(t_lb_total);
    PTB_PROF_BEGIN(tlb0);
    for (uint32_t n = warp - NW;; n += LBW) {
      const int s = n % D;
      const uint32_t par = (n / D) & 1u;
      uint64_t limit = (failed || *sm_abort) ? kWaitNsAfterError : kWaitNs;
      PTB_PROF_BEGIN(tf0);
      if (!mbar_wait_bounded(&issued[s], par, limit)) {
        if (lane == 0) { atomicOr(ws.error, kErrLoadTimeout); *sm_abort = 1; }
        break;
      }
      PTB_PROF_END(t_lb_wait_full, tf0);
      const uint32_t ticket = tile_ticket[s];
      if (ticket == kNoTile) break;
      const TileCoords c = tile_coords<P>(ticket, B, nchunks, T);
      PTB_PROF_BEGIN(tl0);
      if (lane == 0) PTB_EV(4, n);
      State hin;
      if (c.chunk == 0) hin = P::row_init(prm, c.row);   // its end state is published in phase 1
      else hin = lookback<P>(P::ctx_row(prm, c.row), ws, ticket, c.chunk, B, lane, failed, lb_first, kWaitNs);
      if (lane == 0) {
        sm_hin[s] = hin;
        mbar_arrive(&lb_done[s]);
        PTB_EV(5, n);
      }
      PTB_PROF_END(t_lb_look, tl0);
      limit = (failed || *sm_abort) ? kWaitNsAfterError : kWaitNs;
      PTB_PROF_BEGIN(ta0);
      if (!mbar_wait_bounded(&agg_ready[s], par, limit)) {
        if (lane == 0) { atomicOr(ws.error, kErrPipeTimeout); *sm_abort = 1; }
        break;
      }
      PTB_PROF_END(t_lb_wait_agg, ta0);
      if (lane == 0) {
        if (c.chunk > 0 || nchunks == 1) {
          const State hend = P::apply(P::ctx_row(prm, c.row), sm_tagg[s], hin);
          if (c.chunk + 1 < nchunks) slot_store(ws.slots + (size_t)ticket * P::SLOT_WORDS, hend, 2u);
          else P::row_final(prm, c.row, hend);
        }
        mbar_arrive(&done[s]);   // this warp is through with the stage's scratch
      }
      __syncwarp();
    }
    PTB_PROF_END(t_lb_total, tlb0);
    if (lane == 0 && warp == NW) {
      PTB_PROF_FLUSH(4, t_lb_wait_full); PTB_PROF_FLUSH(5, t_lb_wait_agg); PTB_PROF_FLUSH(6, t_lb_look);
      PTB_PROF_FLUSH(7, t_lb_total);
    }
    return;
  }

  // ========================================================================= compute warps
  // Event loop per warp: finish (phase 2) the oldest aggregated tile as soon as its incoming state
  // is known; otherwise aggregate (phase 1) the next tile as soon as its operands have landed.
  // Every landed tile therefore publishes its aggregate without waiting for older look-backs.
  const int tpos = P::REVERSE ? (NT - 1 - tid) : tid;
  Map exc[D];                // this thread's exclusive prefix inside the tile held by each stage
  uint32_t p1 = 0, p2 = 0;   // tiles aggregated / finished so far by this warp
  uint32_t sync_par0 = 0, sync_par1 = 0;
  // barrier among the compute threads, bounded like every other wait of the kernel
  auto cta_sync = [&](int id, uint32_t& par) {
    mbar_arrive(&sync_bar[id]);
    if (!mbar_wait_bounded(&sync_bar[id], par, (*sm_abort) ? kWaitNsAfterError : kWaitNs)) {
      if (lane == 0) { atomicOr(ws.error, kErrPipeTimeout); *sm_abort = 1; }
    }
    par ^= 1u;
  };
  PTB_PROF_DECL(t_c_idle); PTB_PROF_DECL(t_c_total);
  PTB_PROF_BEGIN(tc0);

  auto phase1 = [&](const int s, uint32_t ticket) {
    const TileCoords c = tile_coords<P>(ticket, B, nchunks, T);
    unsigned char* stage = smem + s * P::STAGE_BYTES;
    if (tid == 0) PTB_EV(2, p1);
    if (!bulk) {   // operands that are not 16-byte aligned: cooperative word copies
      IoPlan io; io.nld = 0; io.nst = 0;
      P::plan(prm, false, c.row, c.t0, c.nvalid, io);
#pragma unroll
      for (int i = 0; i < kMaxIo; ++i) {
        if (i < io.nld) {
          const uint32_t* g = reinterpret_cast<const uint32_t*>(io.ld_g[i]);
          uint32_t* d = reinterpret_cast<uint32_t*>(stage + io.ld_soff[i]);
          const uint32_t nw = io.ld_bytes[i] >> 2;
          for (uint32_t w = tid; w < nw; w += NT) d[w] = __ldg(g + w);
        }
      }
      cta_sync(0, sync_par0);
    }
    const typename P::Ctx ctx = P::ctx_stage(stage);
    const Map mine = P::aggregate(prm, stage, tpos, c.row, c.t0, c.nvalid);
    if (tid == 0) PTB_EV(10, p1);
    const Map inc = P::warp_scan(ctx, mine, lane, 0);
    if (tid == 0) PTB_EV(11, p1);
    uint32_t order = 0;
    if (lane == 31) {
      wtot[s * NW + warp] = inc;
      __threadfence_block();
      order = atomicAdd(&sm_cnt[s], 1u);
    }
    order = __shfl_sync(0xffffffffu, order, 31);
    Map e = shfl_up_pod(inc, 1);
    if (lane == 0) e = P::identity();
    // this thread's exclusive prefix inside its warp, kept for phase 2 (select chain: the stage
    // index is dynamic, the register array must be indexed statically)
#pragma unroll
    for (int i = 0; i < D; ++i)
      if (i == s) exc[i] = e;
    if (order == (uint32_t)(NW - 1)) {
      // last warp of the tile: scan the warp totals and publish the tile's record right away
      __threadfence_block();
      const Map w = lane < NW ? wtot[s * NW + lane] : P::identity();
      const Map winc = P::warp_scan(ctx, w, lane, 1);
      Map wexc = shfl_up_pod(winc, 1);
      if (lane == 0) wexc = P::identity();
      if (lane < NW) wpre[s * NW + lane] = wexc;
      if (lane == NW - 1) {
        sm_tagg[s] = winc;
        sm_cnt[s] = 0;
        uint64_t* slot = ws.slots + (size_t)c.ticket * P::SLOT_WORDS;
        if (c.chunk > 0) {
          slot_store(slot, winc, 1u);
        } else if (nchunks > 1) {
          slot_store(slot, P::apply(ctx, winc, P::row_init(prm, c.row)), 2u);
        }
      }
      __syncwarp();
      if (lane == NW - 1) { mbar_arrive(&agg_ready[s]); PTB_EV(3, p1); }
    }
  };

  auto phase2 = [&](const int s) {
    const TileCoords c = tile_coords<P>(tile_ticket[s], B, nchunks, T);
    unsigned char* stage = smem + s * P::STAGE_BYTES;
    const State hin = sm_hin[s];
    if (tid == 0) PTB_EV(6, p2);
    Map e = exc[0];
#pragma unroll
    for (int i = 1; i < D; ++i)
      if (i == s) e = exc[i];
    const State mine = P::thread_state(P::ctx_stage(stage), wpre[s * NW + warp], e, hin, lane);
    if (tid == 0) PTB_EV(12, p2);
    Partial part;
    if constexpr (L::kExtra > 0)
      part = P::finish_x(prm, mine, stage, smem + L::kExtraOff, p2, warp, lane, c.row, c.t0, c.nvalid, kWaitNs);
    else
      part = P::finish(prm, mine, stage, tpos, c.row, c.t0, c.nvalid);

    if (P::HAS_PARTIAL) {
      // per-tile sum for time-invariant gradients: warp shuffle, then the last warp to arrive adds
      // the warp sums in a fixed order (deterministic) and writes the tile's partial.  This is done
      // before the stage is released, so the per-stage scratch cannot be overwritten meanwhile.
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        Partial o = shfl_down_pod(part, d);
#pragma unroll
        for (int i = 0; i < Partial::N; ++i) part.v[i] += o.v[i];
      }
      uint32_t order = 0;
      if (lane == 0) {
        sm_part[s * NW + warp] = part;
        __threadfence_block();
        order = atomicAdd(&sm_pcnt[s], 1u);
      }
      order = __shfl_sync(0xffffffffu, order, 0);
      if (order == (uint32_t)(NW - 1) && lane == 0) {
        __threadfence_block();
        Partial tot = sm_part[s * NW];
        for (int w2 = 1; w2 < NW; ++w2)
#pragma unroll
          for (int i = 0; i < Partial::N; ++i) tot.v[i] += sm_part[s * NW + w2].v[i];
        static_cast<Partial*>(ws.partial)[(size_t)c.row * nchunks + c.chunk] = tot;
        sm_pcnt[s] = 0;
      }
      __syncwarp();
    }
    if (bulk) {
      fence_proxy_async_smem();
      mbar_arrive(&done[s]);
      if (tid == 0) PTB_EV(7, p2);
    } else {
      cta_sync(1, sync_par1);
      IoPlan io; io.nld = 0; io.nst = 0;
      P::plan(prm, false, c.row, c.t0, c.nvalid, io);
#pragma unroll
      for (int i = 0; i < kMaxIo; ++i) {
        if (i < io.nst) {
          uint32_t* g = reinterpret_cast<uint32_t*>(io.st_g[i]);
          const uint32_t* d = reinterpret_cast<const uint32_t*>(stage + io.st_soff[i]);
          const uint32_t nw = io.st_bytes[i] >> 2;
          for (uint32_t w = tid; w < nw; w += NT) g[w] = d[w];
        }
      }
      mbar_arrive(&done[s]);
    }
  };

  bool ended = false;
  uint32_t pf = 0;           // tiles whose phase-2 operands this warp has requested (policies with a prefetch hook)
  uint32_t idle = 0;
  uint64_t idle_t0 = 0;
  // On the plain-load path both phases contain barriers among the compute threads, so all warps
  // must take the phases in one fixed order: a tile is aggregated only when nothing is pending.
  const uint32_t ahead = bulk ? (uint32_t)D : 1u;
  while (true) {
    bool progressed = false;
    if constexpr (L::kExtra > 0) {
      // operands that phase 2 streams through the policy's own buffers: requested as soon as the
      // previous tile has left them, long before the tile's incoming state is known
      if (pf == p2 && p2 < p1) {
        const TileCoords c = tile_coords<P>(tile_ticket[p2 % D], B, nchunks, T);
        P::prefetch(prm, smem + L::kExtraOff, p2, warp, lane, c.row, c.t0, c.nvalid);
        ++pf;
      }
    }
    if (p2 < p1) {
      const int s2 = p2 % D;
      // the warp prefixes need every warp's phase 1 (agg_ready), the incoming state the look-back
      if (__all_sync(0xffffffffu, mbar_test_wait(&agg_ready[s2], (p2 / D) & 1u) &&
                                      mbar_test_wait(&lb_done[s2], (p2 / D) & 1u))) {
        phase2(s2);
        ++p2;
        progressed = true;
      }
    }
    if (!progressed && !ended && p1 < p2 + ahead) {
      const int s1 = p1 % D;
      if (__all_sync(0xffffffffu, mbar_test_wait(&full[s1], (p1 / D) & 1u))) {
        const uint32_t ticket = tile_ticket[s1];
        if (ticket == kNoTile) {
          ended = true;
        } else {
          phase1(s1, ticket);
          ++p1;
        }
        progressed = true;
      }
    }
    if (ended && p2 == p1) break;
    if (progressed) {
      idle = 0;
    } else {
      ++idle;
      if (idle > 32) __nanosleep(idle > 256 ? 100 : 20);
      if (idle == 256) idle_t0 = globaltimer_ns();
      if (idle > 256 && (idle & 63u) == 0 &&
          globaltimer_ns() - idle_t0 > ((*sm_abort) ? kWaitNsAfterError : kWaitNs)) {
        if (lane == 0) { atomicOr(ws.error, kErrPipeTimeout); *sm_abort = 1; }
        break;
      }
#ifdef PTB_PROFILE
      t_c_idle += 1;
#endif
    }
  }
  if constexpr (L::kExtra > 0) bulk_wait_all();   // bulk copies issued by the policy's hooks
  if constexpr (FinalReduceOf<P>::value) {
    if (P::wants_final_reduce(prm)) {
      // every warp's partial sums precede its own count; the warp that completes the count sees them all
      __threadfence();
      uint32_t cnt = 0;
      if (lane == 0) cnt = atomicAdd(ws.done, 1u);
      cnt = __shfl_sync(0xffffffffu, cnt, 0);
      if (cnt == gridDim.x * (uint32_t)NW - 1u) {
        __threadfence();
        P::final_reduce(prm, ws.partial, B, nchunks, lane);
      }
    }
  }
  PTB_PROF_END(t_c_total, tc0);
  if (tid == 0) {
    PTB_PROF_FLUSH(8, t_c_idle); PTB_PROF_FLUSH(10, t_c_total);
  }
}

}  // namespace ptb
