// Hand-written sm_100a kernel for fused graphs WITH a reduce-by-row: persistent CTAs walk contiguous
// runs of merge-path tiles; each tile's row-end offsets, index arrays and (two-phase graphs) per-edge
// tensors are staged into shared memory by 1-D bulk async copies (TMA, mbarrier complete_tx) that a
// producer warp issues STAGES tiles ahead.
//   Two-phase graphs (plain SpMV and every graph whose map needs no per-row data): phase 1, lanes on
//   consecutive edges -- each thread copies IPT edges from the stage to registers, hands the stage back,
//   gathers, runs the generated map and writes the products to shared memory; phase 2, one thread per
//   row sums its products and stores the row; rows longer than kShortRowMax are summed by whole warps.
//   Row-mode graphs (a selector equals the row id: spring-mass, fluxes): in tiles without long rows one
//   thread per row loads the row's own record once, gathers and maps its edges in register batches and
//   stores the row; in tiles with a long row whole warps take the rows one at a time (lanes 32 edges
//   apart, shuffle tree).  Nothing of a row-mode graph passes through a shared-memory product buffer.
// The carry of a row that spans tiles travels inside the CTA in shared memory; the only cross-CTA state
// is one carry per CTA, folded in by the last CTA to finish (ticket counter), in CTA order.  No atomics
// on the output, no pre-zeroed output, run-to-run deterministic.
//
// Replaces (reference, paths inside the FlexSpmv project): SpmvKernel
// include/merged_spmv_kernels.cuh:110-128 and AgentFlexSpmv::ConsumeTile / reduce<>
// cuda_template/reducer/merged_agent_spmv_template.cuh:180-445 (CUB BlockScan + per-row atomicAdd).
#pragma once
#include "flex_common.cuh"
#include "flex_tensor.cuh"
#include <type_traits>

namespace flex {

template <int BLOCK_, int IPT_, int STAGES_, int MIN_CTAS_, int BATCH_ = 8, bool PIPELINE_ = false>
struct TileCfg {
  // software pipelining across tiles (gathers of tile k in flight while tile k-1 is reduced); measured
  // slower than the plain loop on B200 (58% against 68% of the HBM peak on the 7-point fp64 SpMV: one
  // CTA less per SM for the second s_prod / s_rel buffer), so it is off by default
  static constexpr bool kPipeline = PIPELINE_;
  // producer-warp L1 prefetch of the records the next tile's gathers will read: measured slower on B200
  // (62% against 67% of the HBM peak on the 7-point fp64 SpMV, 16% against 21% on the power-law matrix: the
  // prefetches add L1 traffic and delay the producer's next bulk copies), so it is off unless requested
#ifdef FLEX_GATHER_PREFETCH
  static constexpr bool kPrefetchGathers = true;
#else
  static constexpr bool kPrefetchGathers = false;
#endif
  static constexpr int kBlock = BLOCK_;
  static constexpr int kIpt = IPT_;
  static constexpr int kStages = STAGES_;
  static constexpr int kMinCtas = MIN_CTAS_;
  static constexpr int kTile = BLOCK_ * IPT_;
  static constexpr int kWarps = BLOCK_ / 32;
  static constexpr int kBatch = BATCH_;   // edges of one row whose gathers are in flight together (short-row tiles)
};

constexpr int kMaxCtas = 2048;            // capacity of the per-CTA carry arrays in the workspace
#ifndef FLEX_SHORT_ROW_MAX
#define FLEX_SHORT_ROW_MAX 64
#endif
constexpr int kShortRowMax = FLEX_SHORT_ROW_MAX;              // tiles whose rows are all at most this long reduce one thread per row
constexpr uint64_t kWaitPolls = 1000000000ull;  // bound on every mbarrier wait: one second of %globaltimer

template <class G>
struct SmemTile {
  const char* base[G::kNumStreams > 0 ? G::kNumStreams : 1];
  __device__ __forceinline__ void advance(int records) {
    static_for<G::kNumStreams>([&](auto I) { base[I.value] += (size_t)records * G::template stream_bytes<I.value>(); });
  }
  template <int I, class T>
  __device__ __forceinline__ const T* stream(int le) const {
    return reinterpret_cast<const T*>(base[I] + (size_t)le * G::template stream_bytes<I>());
  }
};

// Direct mode: the per-edge arrays are read straight from global memory with coalesced loads (lanes on
// consecutive edges); `le` is relative to the tile's first edge.
template <class G>
struct DirectTile {
  const typename G::Params* p;
  long long nz0;
  __device__ __forceinline__ void advance(int records) { nz0 += records; }
  template <int I, class T>
  __device__ __forceinline__ const T* stream(long long le) const {
    return reinterpret_cast<const T*>(G::template stream_ptr<I>(*p) + (size_t)(nz0 + le) * G::template stream_bytes<I>());
  }
};

template <class G, bool WIN> struct WinBytesOf { static constexpr int value = 0; };
template <class G> struct WinBytesOf<G, true> { static constexpr int value = G::kWinBytes; };

template <class G, typename OffsetT, class Cfg, bool WIN = false>
struct TileSmemLayout {
  using V = typename G::V;
  static constexpr int kAcc = G::kAccDim;
  static constexpr int kBytesPerEdge = G::kStreamBytesPerEdge;
  static constexpr int kPerItem = (int(sizeof(OffsetT)) > kBytesPerEdge) ? int(sizeof(OffsetT)) : kBytesPerEdge;
  // each staged window may grow by < 32 bytes from aligning both ends to 16
  static constexpr int kStreamBytes =
      G::kDirectLoads ? 0 : int(align_up(uint64_t(Cfg::kTile) * kPerItem + 32u * (G::kNumStreams + 1) + 16, 128));
  // gather windows (WIN): the segments of the gathered vector follow the streams in every stage
  static constexpr int kWinBytes = int(align_up(uint64_t(WinBytesOf<G, WIN>::value), 128));
  static constexpr int kStageBytes = kStreamBytes + kWinBytes;
  struct alignas(16) Ctl {   // read by every consumer thread of every tile: whole 16-byte words (see acquire)
    long long row0, nz0;
    int nrows, nnz;
    int win;            // the tile gathers from the window area and its index stream holds 16-bit positions
    uint32_t roff_off;
    uint32_t stream_off[G::kNumStreams > 0 ? G::kNumStreams : 1];
  };
  static constexpr int kOffBars = 0;
  static constexpr int kOffCtl = int(align_up(kOffBars + 16 * Cfg::kStages, 16));
  static constexpr int kOffXs = int(align_up(kOffCtl + sizeof(Ctl) * Cfg::kStages, 16));
  static constexpr int kOffWKey = int(align_up(kOffXs + 4 * (Cfg::kBlock + 1), 16));
  static constexpr int kOffWVal = int(align_up(kOffWKey + 4 * Cfg::kWarps, 16));
  static constexpr int kOffCarry = int(align_up(kOffWVal + sizeof(V) * kAcc * Cfg::kWarps, 16));
  static constexpr int kOffFlag = int(align_up(kOffCarry + sizeof(V) * kAcc * 2, 16));
  // rows longer than kShortRowMax inside the current tile: [0..1] counters by tile parity, [2..] local rows
  static constexpr int kMaxLong = Cfg::kTile / (kShortRowMax + 1) + 2;
  static constexpr int kOffLong = int(align_up(kOffFlag + 16, 16));
  static constexpr int kBuffers = (!G::kGatherNeedsRow && Cfg::kPipeline) ? 2 : 1;   // s_rel / s_prod / long-row list double-buffered when tiles are pipelined
  static constexpr int kOffRel = int(align_up(kOffLong + 4 * (4 + kMaxLong * kBuffers), 16));
  // Row-mode graphs (a selector equals the row id) reduce in registers in every tile: no product buffer.  The
  // shared memory a kernel does not claim stays L1 cache, and the number of gather misses an SM can have in
  // flight grows with that cache (measured on B200: 63 / 130 / 183 / 225 / 265 G random 4-byte gathers per
  // second at 228 / 196 / 164 / 132 / <= 32 KB of shared memory per SM).
  static constexpr int kOffProd = int(align_up(kOffRel + 4 * (Cfg::kTile + 1) * kBuffers, 16));
  static constexpr int kOffStages = int(align_up(kOffProd + (G::kGatherNeedsRow ? 0 : sizeof(V) * kAcc * Cfg::kTile * kBuffers), 128));
  static constexpr int kTotal = kOffStages + kStageBytes * Cfg::kStages;
};

struct TileKernelArgs {
  const void* row_offsets;  // leading 0 included
  const void* coords;       // (num_tiles + 1) pairs of OffsetT
  WorkspaceHeader* header;
  long long* carry_row;     // [kMaxCtas]
  void* carry_val;          // [kMaxCtas][kAcc] of V
  long long num_rows;
  long long num_edges;
  long long num_tiles;
  const int* win_table;                // gather windows (WIN kernels): per-tile segment table,
  const unsigned short* win_index;     // per-edge positions inside the window area,
  long long num_vertices;              // rows of the gathered array
};

// One staged window: `count` elements of `eb` bytes starting at element `first` of an array of
// `total` elements at `gbase` (16-byte aligned).  The bulk copy covers whole 16-byte chunks that lie
// inside the array; a ragged tail (the array's last < 16 bytes) is fetched with plain loads.
struct Window {
  const char* src;     // 16-byte aligned start of the bulk part
  uint32_t bulk_bytes; // multiple of 16 (may be 0)
  uint32_t lead;       // bytes between src and the first wanted element
  uint32_t span;       // smem bytes reserved (multiple of 16)
  const char* tail_src;
  uint32_t tail_bytes; // multiple of the element size
};
__device__ __forceinline__ Window make_window(const void* gbase, uint32_t eb, long long first, long long count,
                                              long long total) {
  Window w;
  const uintptr_t addr0 = (uintptr_t)gbase + (uintptr_t)first * eb;
  const uintptr_t addr1 = addr0 + (uintptr_t)count * eb;
  const uintptr_t a0 = addr0 & ~(uintptr_t)15;
  const uintptr_t a1 = (addr1 + 15) & ~(uintptr_t)15;
  const uintptr_t arr_floor = ((uintptr_t)gbase + (uintptr_t)total * eb) & ~(uintptr_t)15;
  uintptr_t bulk_end = a1 < arr_floor ? a1 : arr_floor;
  if (bulk_end < a0) bulk_end = a0;
  w.src = (const char*)a0;
  w.lead = (uint32_t)(addr0 - a0);
  w.span = count > 0 ? (uint32_t)(a1 - a0) : 0u;
  w.bulk_bytes = count > 0 ? (uint32_t)(bulk_end - a0) : 0u;
  const uintptr_t t0 = bulk_end > addr0 ? bulk_end : addr0;
  w.tail_src = (const char*)t0;
  w.tail_bytes = (count > 0 && addr1 > t0) ? (uint32_t)(addr1 - t0) : 0u;
  return w;
}

template <class G, typename OffsetT, class Cfg, bool WIN = false>
__global__ void __launch_bounds__(Cfg::kBlock + (G::kDirectLoads ? 0 : 32), Cfg::kMinCtas)
flex_tile_kernel(const typename G::Params p, const TileKernelArgs a) {
  using V = typename G::V;
  using L = TileSmemLayout<G, OffsetT, Cfg, WIN>;
  static_assert(!WIN || (!G::kDirectLoads && !G::kGatherNeedsRow && !Cfg::kPipeline), "gather windows: staged two-phase loop only");
  using Ctl = typename L::Ctl;
  constexpr int kAcc = G::kAccDim;
  constexpr int NS = G::kNumStreams;
  constexpr int BLOCK = Cfg::kBlock, IPT = Cfg::kIpt, S = Cfg::kStages;
  constexpr bool DIRECT = G::kDirectLoads;   // narrow per-edge records: coalesced loads, no staging, no producer warp

  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBars);    // "full": a stage's copies have landed
  uint64_t* empty = bars + S;                                          // "empty": the consumers released a stage
  Ctl* ctls = reinterpret_cast<Ctl*>(smem + L::kOffCtl);
  int* s_wkey = reinterpret_cast<int*>(smem + L::kOffWKey);
  V* s_wval = reinterpret_cast<V*>(smem + L::kOffWVal);
  V* s_carry = reinterpret_cast<V*>(smem + L::kOffCarry);
  int* s_flag = reinterpret_cast<int*>(smem + L::kOffFlag);
  int* s_nlong = reinterpret_cast<int*>(smem + L::kOffLong);
  int* s_long = s_nlong + 4;
  int* s_rel = reinterpret_cast<int*>(smem + L::kOffRel);
  V* s_prod = reinterpret_cast<V*>(smem + L::kOffProd);
  unsigned char* s_stage = smem + L::kOffStages;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const OffsetT* row_offsets = static_cast<const OffsetT*>(a.row_offsets);
  const OffsetT* coords = static_cast<const OffsetT*>(a.coords);

  // With a programmatic dependent launch the CTA may have been placed while the kernel before this one on the stream
  // was still draining: wait for its results (and for this workspace's ticket) before the first global access.
  pdl_wait();
  pdl_launch_dependents();

  // contiguous run of tiles of this CTA
  const long long q = a.num_tiles / gridDim.x, rem = a.num_tiles % gridDim.x;
  const long long t_begin = (long long)blockIdx.x * q + ((long long)blockIdx.x < rem ? blockIdx.x : rem);
  const int count = (int)(q + ((long long)blockIdx.x < rem ? 1 : 0));

  // The producer warp asks for its first coordinates together with the header (two round trips become one).  The
  // words lie inside the workspace whether it was planned or not; nothing is done with them before the check below.
  OffsetT first_coords[4] = {0, 0, 0, 0};
  if constexpr (!DIRECT) {
    if (warp == Cfg::kWarps && count) {
#pragma unroll
      for (int i = 0; i < 4; ++i) first_coords[i] = coords[2 * t_begin + i];
    }
  }

  // a workspace that was never planned for this problem holds no usable coordinates: every CTA
  // sees the same header, so all of them leave here and the ticket stays untouched
  if (a.header->magic != kMagic || a.header->num_tiles != a.num_tiles || a.header->num_rows != a.num_rows ||
      a.header->num_edges != a.num_edges || a.header->offset_bits != (int)(8 * sizeof(OffsetT))) {
    if (tid == 0 && blockIdx.x == 0) raise_not_planned(a.header);
    return;
  }

  const bool win_ready = WIN && a.header->win_ready == 1;   // until the window plan has run every tile gathers globally
  (void)win_ready;

  // ---- producer ------------------------------------------------------------------------------------------
  // Table entry of a tile's gather windows, one piece per lane: the segment count in every lane, segment j in
  // lane 16 + j (read one tile ahead, like the coordinates).
  struct WinEnt { int nseg, first, len; };
  auto load_win_entry = [&](long long tile_id) -> WinEnt {
    WinEnt e{0, 0, 0};
    if constexpr (WIN) {
      static_assert(NS + 1 <= 16 && kWinMaxSegs <= 16, "lanes 0..NS stage the streams, lanes 16.. the window segments");
      if (win_ready) {
        const int* ent = a.win_table + tile_id * kWinEntryInts;
        e.nseg = ent[0];
        if (lane >= 16 && lane - 16 < kWinMaxSegs) { e.first = ent[2 + 2 * (lane - 16)]; e.len = ent[3 + 2 * (lane - 16)]; }
      }
    }
    (void)tile_id;
    return e;
  };
  // Stages one tile; executed by the whole producer warp: lane i prepares window i (lane 0: row-end offsets,
  // lane 1+I: stream I, lane 16+j: gather-window segment j), a shuffle prefix sum places the windows in the
  // stage, lane 0 posts the byte count, then every lane issues its own bulk copy.
  auto issue = [&](long long row0, long long nz0, long long row1, long long nz1, int s, const WinEnt& we) {
    unsigned char* dst = s_stage + (size_t)s * L::kStageBytes;
    Window w;
    w.src = nullptr; w.bulk_bytes = 0; w.lead = 0; w.span = 0; w.tail_src = nullptr; w.tail_bytes = 0;
    const int nseg = we.nseg;
    if constexpr (WIN) {
      if (lane >= 16 && lane - 16 < nseg) w = make_window(G::gather_base(p), G::kGatherRecBytes, we.first, we.len, a.num_vertices);
    }
    if (lane == 0) w = make_window(row_offsets, sizeof(OffsetT), row0 + 1, row1 - row0, a.num_rows + 1);
    static_for<NS>([&](auto I) {
      if (lane == I.value + 1) {
        bool local = false;
        if constexpr (WIN) local = (I.value == G::kIdxStream) && nseg > 0;
        if (local) w = make_window(a.win_index, 2, nz0, nz1 - nz0, a.num_edges);
        else w = make_window(G::template stream_ptr<I.value>(p), G::template stream_bytes<I.value>(), nz0, nz1 - nz0, a.num_edges);
      }
    });
    uint32_t off = w.span;   // exclusive prefix sum of the spans over lanes 0..NS (streams) and 16.. (segments)
#pragma unroll
    for (int d = 1; d <= (WIN ? 8 : NS); d <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, off, d);
      if ((lane & 15) >= d) off += t;
    }
    off -= w.span;
    if constexpr (WIN) { if (lane >= 16) off += L::kStreamBytes; }
    uint32_t total = w.bulk_bytes;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
    Ctl& c = ctls[s];
    if (lane == 0) { c.row0 = row0; c.nz0 = nz0; c.nrows = (int)(row1 - row0); c.nnz = (int)(nz1 - nz0); c.roff_off = off + w.lead; c.win = nseg > 0; }
    static_for<NS>([&](auto I) { if (lane == I.value + 1) c.stream_off[I.value] = off + w.lead; });
    // the ragged tail (last < 16 bytes of an array) is fetched with plain loads BEFORE the arrive below,
    // whose release (after the warp barrier) makes it and the control block visible to the consumers
    if (w.tail_bytes) {
      const uint32_t so = off + (uint32_t)(w.tail_src - w.src);
      if (((uint32_t)reinterpret_cast<uintptr_t>(w.tail_src) | w.tail_bytes) & 3u) {   // 2-byte elements (window positions)
        for (uint32_t b = 0; b < w.tail_bytes; b += 2)
          *reinterpret_cast<uint16_t*>(dst + so + b) = *reinterpret_cast<const uint16_t*>(w.tail_src + b);
      } else {
        for (uint32_t b = 0; b < w.tail_bytes; b += 4)
          *reinterpret_cast<uint32_t*>(dst + so + b) = *reinterpret_cast<const uint32_t*>(w.tail_src + b);
      }
    }
    fence_proxy_async_smem();   // earlier generic accesses to this stage are ordered before the bulk copies
    __syncwarp();
    if (lane == 0) mbar_expect_tx(&bars[s], total);
    __syncwarp();
    if (w.bulk_bytes) bulk_g2s(dst + off, w.src, w.bulk_bytes, &bars[s]);
#ifdef FLEX_PREFETCH_DIRECT
    if constexpr (G::kHasDirectEdgeTensors) G::prefetch_direct(p, nz0, nz1, lane);
#endif
  };

  // Producer warp, one tile ahead of the consumers: once tile j's index arrays have landed in shared memory,
  // prefetch into L1 every vertex record its gathers will read, so that the consumers' gathers hit L1
  // instead of paying an L2 round trip in the middle of the tile.
  auto prefetch_gathers = [&](int j) {
    if constexpr (G::kHasEdgeGather && S >= 2 && Cfg::kPrefetchGathers) {
      const int s = j % S;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(&bars[s], (uint32_t)(j / S) & 1u, kWaitPolls))) return;
      const Ctl& c = ctls[s];
      const unsigned char* stage = s_stage + (size_t)s * L::kStageBytes;
      SmemTile<G> tile;
      static_for<NS>([&](auto I) { tile.base[I.value] = reinterpret_cast<const char*>(stage + c.stream_off[I.value]); });
      const int nnz = c.nnz;
      for (int e = lane; e < nnz; e += 32) G::prefetch_edge(p, tile, e);
    }
  };

  if constexpr (!DIRECT) {
    if (tid == 0) {
#pragma unroll
      for (int s = 0; s < S; ++s) { mbar_init(&bars[s], 1); mbar_init(&empty[s], Cfg::kWarps); }   // empty: one arrive per consumer warp
      mbar_fence_init();
    }
  }
  if (tid < 2 * kAcc) s_carry[tid] = V(0);
  if (tid < 4) s_nlong[tid] = 0;
  if (tid == 0) s_flag[1] = (a.header->snapped_grid == (int)gridDim.x) ? 1 : 0;   // no row spans two CTAs of this launch
  __syncthreads();   // the only barrier that includes the producer warp

  // ---- producer warp: runs up to S tiles ahead of the consumers, off their critical path -----------
  if (!DIRECT && warp == Cfg::kWarps) {
    {
      int issued = 0;
      bool pfail = false;
      // coordinates are read one tile ahead, so their load latency overlaps the wait for a free stage
      long long c_row = (long long)first_coords[0], c_nz = (long long)first_coords[1];
      long long n_row = (long long)first_coords[2], n_nz = (long long)first_coords[3];
      WinEnt c_we = count ? load_win_entry(t_begin) : WinEnt{0, 0, 0};
      // testing aid (flexspmv_debug_withhold_stage): the stage of tile `withhold - 1` and of every later tile is
      // never filled, so that the consumers' bounded wait runs out and the error path can be exercised
      const unsigned long long withhold = a.header->debug[7];
      for (int k = 0; k < count; ++k) {
        if (withhold && (unsigned long long)(t_begin + k) + 1ull >= withhold) break;
        const int s = k % S;
        long long nn_row = 0, nn_nz = 0;
        if (k + 1 < count) { nn_row = (long long)coords[2 * (t_begin + k + 2)]; nn_nz = (long long)coords[2 * (t_begin + k + 2) + 1]; }
        const WinEnt n_we = (k + 1 < count) ? load_win_entry(t_begin + k + 1) : WinEnt{0, 0, 0};
        if (k >= S) {
          const bool ok = mbar_wait_bounded(&empty[s], (uint32_t)(k / S - 1) & 1u, kWaitPolls);
          if (!__all_sync(0xffffffffu, ok)) { pfail = true; break; }
        }
        issue(c_row, c_nz, n_row, n_nz, s, c_we);
        c_row = n_row; c_nz = n_nz; n_row = nn_row; n_nz = nn_nz; c_we = n_we;
        issued = k + 1;
        if (k >= 1) prefetch_gathers(k - 1);   // tile k-1 has (almost certainly) landed: warm L1 for its gathers
      }
      if (!pfail && count >= 1) prefetch_gathers(count - 1);
      if (pfail && lane == 0) {   // the consumers never released a stage: flag it, let copies in flight land, leave
        raise_status(a.header, FLEXSPMV_ERR_TIMEOUT);
        a.header->debug[4] = (uint32_t)issued; a.header->debug[5] = blockIdx.x;
        for (int j = issued > S ? issued - S : 0; j < issued; ++j)
          mbar_wait_bounded(&bars[j % S], (uint32_t)(j / S) & 1u, kWaitPolls);
      }
    }
    return;
  }

  // ---- consumers (threads 0 .. BLOCK-1); their barriers are the named barrier 1 ---------------------
  using TileT = std::conditional_t<DIRECT, DirectTile<G>, SmemTile<G>>;
  struct TileRef { long long row0, nz0; int nrows, nnz; int win; };
  const unsigned char* xwin = nullptr;   // WIN: the current tile's window area
  bool failed = false;
  long long last_row1 = 0;

  // direct mode: tile coordinates are read one tile ahead into registers
  long long d_row = 0, d_nz = 0, d_row1 = 0, d_nz1 = 0;
  if constexpr (DIRECT) {
    if (count) {
      d_row = (long long)coords[2 * t_begin]; d_nz = (long long)coords[2 * t_begin + 1];
      d_row1 = (long long)coords[2 * t_begin + 2]; d_nz1 = (long long)coords[2 * t_begin + 3];
    }
  }

  // Makes tile k available: waits (bounded) for its stage, or takes its coordinates in direct mode.
  auto acquire = [&](int k, TileRef& t, TileT& tile, const OffsetT*& rend) -> bool {
    if constexpr (DIRECT) {
      t.row0 = d_row; t.nz0 = d_nz; t.nrows = (int)(d_row1 - d_row); t.nnz = (int)(d_nz1 - d_nz); t.win = 0;
      d_row = d_row1; d_nz = d_nz1;
      if (k + 1 < count) { d_row1 = (long long)coords[2 * (t_begin + k + 2)]; d_nz1 = (long long)coords[2 * (t_begin + k + 2) + 1]; }
      tile.p = &p; tile.nz0 = t.nz0;
      rend = row_offsets + t.row0 + 1;
      named_bar_sync(1, BLOCK);   // the previous tile's readers of the shared arrays are done
      return true;
    } else {
      const int s = k % S;
      const bool ok = named_bar_and(1, BLOCK, mbar_wait_bounded(&bars[s], (uint32_t)(k / S) & 1u, kWaitPolls));
      if (!ok) {
        if (tid == 0) {
          raise_status(a.header, FLEXSPMV_ERR_TIMEOUT);
          a.header->debug[0] = (uint32_t)(t_begin + k); a.header->debug[1] = (uint32_t)s; a.header->debug[2] = blockIdx.x;
        }
        return false;
      }
      // one 16-byte shared load per 16 bytes of the control block instead of one load per field: the kernel
      // is bound by shared-memory wavefronts, and every thread of every tile reads this
      Ctl c;
      {
        constexpr int kWords = int(sizeof(Ctl) / 16);
        const int4* src = reinterpret_cast<const int4*>(&ctls[s]);
        int4* dst16 = reinterpret_cast<int4*>(&c);
#pragma unroll
        for (int i = 0; i < kWords; ++i) dst16[i] = src[i];
      }
      t.row0 = c.row0; t.nz0 = c.nz0; t.nrows = c.nrows; t.nnz = c.nnz; t.win = c.win;
      const unsigned char* stage = s_stage + (size_t)s * L::kStageBytes;
      xwin = stage + L::kStreamBytes;
      rend = reinterpret_cast<const OffsetT*>(stage + c.roff_off);
      static_for<NS>([&](auto I) { tile.base[I.value] = reinterpret_cast<const char*>(stage + c.stream_off[I.value]); });
      return true;
    }
  };
  // This warp needs nothing more from stage s: the producer refills it once every warp has said so.
  auto release = [&](int k) {
    if constexpr (!DIRECT) {
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[k % S]);
    }
  };
  // Row ends as 32-bit edge indices relative to the tile, with a sentinel behind the last row.  Returns
  // whether this thread saw a long row (or a long trailing partial row).
  // With list >= 0 the long rows are also appended (in any order) to buffer lbuf of s_long, counted in
  // s_nlong[list].
  auto convert = [&](const TileRef& t, const OffsetT* rend, int* srel, int list, int lbuf = 0) -> bool {
    int* rows_long = s_long + lbuf * L::kMaxLong;
    bool my_long = false;
    for (int r = tid; r < t.nrows; r += BLOCK) {
      const long long end_r = (long long)rend[r];
      const long long beg_r = r ? (long long)rend[r - 1] : t.nz0;
      srel[r] = (int)(end_r - t.nz0);
      if ((end_r - beg_r) > kShortRowMax) {
        my_long = true;
        if (list >= 0) rows_long[atomicAdd(&s_nlong[list], 1)] = r;
      }
    }
    if (tid == 0) {
      srel[t.nrows] = 0x7fffffff;
      const long long beg_t = t.nrows ? (long long)rend[t.nrows - 1] : t.nz0;
      if ((t.nz0 + t.nnz - beg_t) > kShortRowMax) {
        my_long = true;
        if (list >= 0) rows_long[atomicAdd(&s_nlong[list], 1)] = t.nrows;
      }
    }
    return my_long;
  };
  auto store_row = [&](long long row, const V* v) {
    static_for<G::kNumReducers>([&](auto R) {
      constexpr int d = G::template red_dim<R.value>();
      constexpr int o = G::template red_off<R.value>();
      V* dst = G::template red_out<R.value>(p) + (size_t)row * d;
#pragma unroll
      for (int j = 0; j < d; ++j) dst[j] = v[o + j];
    });
  };

  // ---- phase 1 pieces: lanes on consecutive edges ------------------------------------------------------
  auto map_load = [&](const TileRef& t, const TileT& tile, typename G::EReg (&er)[IPT]) {
    auto ttile = tile;
    ttile.advance(tid);   // element `tid` at offset 0: the unrolled accesses are base + constant
#pragma unroll
    for (int i = 0; i < IPT; ++i)
      if (i * BLOCK + tid < t.nnz) G::load_edge(p, ttile, i * BLOCK, t.nz0 + (i * BLOCK + tid), er[i]);
  };
  auto map_gather = [&](const TileRef& t, const typename G::EReg (&er)[IPT], typename G::GEdge (&ge)[IPT],
                        typename G::GRow (&gr)[G::kGatherNeedsRow ? IPT : 1]) {
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (i * BLOCK + tid < t.nnz) {
#ifndef FLEX_EXP_SKIP_GATHER
        G::gather_edge(p, er[i], ge[i]);
#else
        memset(&ge[i], 0, sizeof(ge[i]));
#endif
      }
    }
  };
  auto map_products = [&](const TileRef& t, const typename G::EReg (&er)[IPT], const typename G::GEdge (&ge)[IPT],
                          const typename G::GRow (&gr)[G::kGatherNeedsRow ? IPT : 1], V* sprod) {
    V* tprod = sprod + tid;
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (i * BLOCK + tid < t.nnz) {
        V prod[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) prod[j] = V(0);
        G::map(p, er[i], t.nz0 + (i * BLOCK + tid), gr[G::kGatherNeedsRow ? i : 0], ge[i], prod);
#pragma unroll
        for (int j = 0; j < kAcc; ++j) tprod[j * Cfg::kTile + i * BLOCK] = prod[j];
      }
    }
  };

  // ---- phase 1 of a tile with gather windows: 16-bit positions instead of column indices, gathers from the
  //      window area of the stage (so the stage goes back to the producer after the gathers, not before) ----
  auto map_load_gather_win = [&](const TileRef& t, const TileT& tile, typename G::EReg (&er)[IPT], typename G::GEdge (&ge)[IPT]) {
    if constexpr (WIN) {
      auto ttile = tile;
      ttile.advance(tid);
      unsigned short pos[IPT];
#pragma unroll
      for (int i = 0; i < IPT; ++i)
        if (i * BLOCK + tid < t.nnz) {
          G::load_edge_vals(p, ttile, i * BLOCK, t.nz0 + (i * BLOCK + tid), er[i]);   // the index stream holds 16-bit positions here
          pos[i] = reinterpret_cast<const unsigned short*>(tile.base[G::kIdxStream])[i * BLOCK + tid];
        }
#pragma unroll
      for (int i = 0; i < IPT; ++i)
        if (i * BLOCK + tid < t.nnz) G::gather_edge_win(xwin, pos[i], ge[i]);
    }
  };

  // ---- phase 2, short rows: one thread per row sums its products left to right and stores the row
  //      (coalesced); local row 0 continues the CTA's carry (buffer kpar), the trailing partial row
  //      (local row `nrows`) becomes the next carry ---------------------------------------------------------
  //      With list >= 0 the rows in s_long (longer than kShortRowMax) are left to whole warps: lanes sum
  //      strided, a shuffle tree combines them.
  auto reduce_short = [&](const TileRef& t, int kpar, const V* sprod, const int* srel, int list, int lbuf = 0) {
    const int* rows_long = s_long + lbuf * L::kMaxLong;
#ifdef FLEX_EXP_SKIP_REDUCE
    return;
#endif
    if (list >= 0) {
      const int n_long = s_nlong[list];
      for (int i = warp; i < n_long; i += Cfg::kWarps) {
        const int r = rows_long[i];
        const int lo = r ? srel[r - 1] : 0;
        const int hi = r < t.nrows ? srel[r] : t.nnz;
        V sum[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) sum[j] = V(0);
        for (int e = lo + lane; e < hi; e += 32) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) sum[j] += sprod[j * Cfg::kTile + e];
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) sum[j] += shfl_down_any(sum[j], off);
        }
        if (lane == 0) {
          if (r == 0) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) sum[j] = s_carry[kpar * kAcc + j] + sum[j];
          }
          if (r < t.nrows) {
            store_row(t.row0 + r, sum);
          } else {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) s_carry[(kpar ^ 1) * kAcc + j] = sum[j];
          }
        }
      }
    }
    for (int r = tid; r <= t.nrows; r += BLOCK) {
      const int lo = r ? srel[r - 1] : 0;
      const int hi = r < t.nrows ? srel[r] : t.nnz;
      int n = hi - lo;
      if (list >= 0 && n > kShortRowMax) continue;
      V sum[kAcc];
#pragma unroll
      for (int j = 0; j < kAcc; ++j) sum[j] = (r == 0) ? s_carry[kpar * kAcc + j] : V(0);
      const V* q = sprod + lo;
      // rows of up to kUnroll edges (the common case) without a loop: every load is issued before the first add,
      // and threads whose rows differ in length do not diverge
      constexpr int kUnroll = (kAcc * sizeof(V) <= 8) ? 8 : ((kAcc * sizeof(V) <= 16) ? 4 : 2);
      if (n <= kUnroll) {
        V v[kUnroll][kAcc];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) v[u][j] = (u < n) ? q[j * Cfg::kTile + u] : V(0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (u < n) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) sum[j] += v[u][j];
          }
        }
        n = 0;
      }
      for (; n >= 4; n -= 4, q += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) sum[j] += q[j * Cfg::kTile + u];
        }
      }
      for (; n > 0; --n, ++q) {
#pragma unroll
        for (int j = 0; j < kAcc; ++j) sum[j] += q[j * Cfg::kTile];
      }
      if (r < t.nrows) {
        store_row(t.row0 + r, sum);
      } else {
#pragma unroll
        for (int j = 0; j < kAcc; ++j) s_carry[(kpar ^ 1) * kAcc + j] = sum[j];
      }
    }
  };

  // ---- phase 2, long rows: every thread reduces its merge-path span: exactly n_items steps, each
  //      consuming one edge (accumulate) or one row end (store the row, reset); the carries are combined
  //      by a warp-shuffle segmented scan and a cross-warp fold (one barrier inside) -------------------
  auto reduce_long = [&](const TileRef& t, int kpar, const V* sprod, const int* srel, int xs, int ys, int n_items) {
    V acc[kAcc], first_val[kAcc];
#pragma unroll
    for (int j = 0; j < kAcc; ++j) { acc[j] = V(0); first_val[j] = V(0); }
    int row = xs;
    {
      int nz = ys, re = srel[xs];
#pragma unroll
      for (int i = 0; i < IPT; ++i) {
        if (i < n_items) {
          if (nz < re) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) acc[j] += sprod[j * Cfg::kTile + nz];
            ++nz;
          } else {
            // the first row a thread closes may have begun in earlier threads: keep it for after the scan
            if (row == xs) {
#pragma unroll
              for (int j = 0; j < kAcc; ++j) first_val[j] = acc[j];
            } else {
              store_row(t.row0 + row, acc);
            }
#pragma unroll
            for (int j = 0; j < kAcc; ++j) acc[j] = V(0);
            ++row;
            re = srel[row];
          }
        }
      }
    }
    // segmented inclusive scan of the carries (key = row the carry belongs to)
    const int key = row;
    V val[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; ++i) val[i] = acc[i];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int k2 = __shfl_up_sync(0xffffffffu, key, off);
#pragma unroll
      for (int i = 0; i < kAcc; ++i) {
        const V v2 = shfl_up_any(val[i], off);
        if (lane >= off && k2 == key) val[i] += v2;
      }
    }
    if (lane == 31) {
      s_wkey[warp] = key;
#pragma unroll
      for (int i = 0; i < kAcc; ++i) s_wval[warp * kAcc + i] = val[i];
    }
    const int pk = __shfl_up_sync(0xffffffffu, key, 1);
    V pv[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; ++i) pv[i] = shfl_up_any(val[i], 1);
    named_bar_sync(1, BLOCK);   // [B] warp aggregates visible
    // fold: CTA carry (belongs to local row 0) then the aggregates of the warps before this one
    int fk = 0;
    V fv[kAcc];
#pragma unroll
    for (int i = 0; i < kAcc; ++i) fv[i] = s_carry[kpar * kAcc + i];
    for (int w = 0; w < warp; ++w) {
      const int wk = s_wkey[w];
      if (wk == fk) {
#pragma unroll
        for (int i = 0; i < kAcc; ++i) fv[i] += s_wval[w * kAcc + i];
      } else {
        fk = wk;
#pragma unroll
        for (int i = 0; i < kAcc; ++i) fv[i] = s_wval[w * kAcc + i];
      }
    }
    if (tid == BLOCK - 1) {   // carry into the next tile = inclusive value of the last thread
#pragma unroll
      for (int i = 0; i < kAcc; ++i) s_carry[(kpar ^ 1) * kAcc + i] = (fk == key) ? fv[i] + val[i] : val[i];
    }
    if (lane > 0) {
      if (pk == fk) {
#pragma unroll
        for (int i = 0; i < kAcc; ++i) fv[i] += pv[i];
      } else {
#pragma unroll
        for (int i = 0; i < kAcc; ++i) fv[i] = pv[i];
      }
    }
    if (row > xs) {   // first closed row = what earlier threads / tiles carried + this thread's part
#pragma unroll
      for (int i = 0; i < kAcc; ++i) first_val[i] = fv[i] + first_val[i];
      store_row(t.row0 + xs, first_val);
    }
  };
  auto thread_span = [&](const TileRef& t, const int* srel, int& xs, int& ys, int& n_items) {
    const int total_items = t.nrows + t.nnz;
    const int d0 = min(tid * IPT, total_items);
    n_items = min(d0 + IPT, total_items) - d0;
    merge_path_search<int, int>(d0, srel, 0, t.nrows, t.nnz, xs, ys);
  };

  if constexpr (!G::kGatherNeedsRow && !Cfg::kPipeline) {
    // ---- plain loop: stage -> registers -> gathers -> products -> classify -> reduce --------------------
    for (int k = 0; k < count; ++k) {
      TileRef t{0, 0, 0, 0, 0};
      TileT tile;
      const OffsetT* rend = nullptr;
      if (!acquire(k, t, tile, rend)) { failed = true; break; }
      last_row1 = t.row0 + t.nrows;
#ifdef FLEX_STREAM_ONLY
      release(k);
      continue;
#endif
      if (tid == 0) s_nlong[(k + 1) & 1] = 0;   // the previous tile's list has been consumed (barrier in acquire)
      const bool my_long = convert(t, rend, s_rel, k & 1);
      {
        typename G::EReg er[IPT];
        typename G::GEdge ge[IPT];
        typename G::GRow gr[1];
        if (WIN && t.win) {
          map_load_gather_win(t, tile, er, ge);
          release(k);
        } else {
          map_load(t, tile, er);
          release(k);     // as early as possible: the refill latency of this stage is what bounds the kernel
          map_gather(t, er, ge, gr);
        }
        map_products(t, er, ge, gr, s_prod);
      }
      const bool long_tile = named_bar_or(1, BLOCK, my_long);   // [P] products, s_rel and the long-row list complete
#ifdef FLEX_MERGE_WALK_REDUCE
      if (long_tile) {
        int xs, ys, n_items;
        thread_span(t, s_rel, xs, ys, n_items);
        reduce_long(t, k & 1, s_prod, s_rel, xs, ys, n_items);
        continue;
      }
#endif
      reduce_short(t, k & 1, s_prod, s_rel, long_tile ? (k & 1) : -1);   // the next tile's first barrier orders these reads
    }
  } else if constexpr (!G::kGatherNeedsRow) {
    // ---- software-pipelined loop: the gathers of tile k are in flight while tile k-1 is reduced.
    //      s_rel and s_prod are double-buffered by tile parity; one classifying barrier per tile. -------
    TileRef prev{0, 0, 0, 0, 0};
    bool prev_long = false;
    for (int k = 0; k <= count; ++k) {
      const bool have = k < count;
      TileRef cur{0, 0, 0, 0, 0};
      bool my_long = false;
      typename G::EReg er[IPT];
      typename G::GEdge ge[IPT];
      typename G::GRow gr[1];
      int* srel_k = s_rel + (k & 1) * (Cfg::kTile + 1);
      V* sprod_k = s_prod + (size_t)(k & 1) * kAcc * Cfg::kTile;
      if (have) {
        TileT tile;
        const OffsetT* rend = nullptr;
        if (!acquire(k, cur, tile, rend)) { failed = true; break; }
        last_row1 = cur.row0 + cur.nrows;
#ifdef FLEX_STREAM_ONLY
        release(k);
        continue;
#endif
        // long-row counters rotate over three slots: k % 3 is filled now, (k - 1) % 3 is read by the reduction
        // below, (k + 1) % 3 was last read before the barrier in acquire and is cleared for the next tile
        if (tid == 0) s_nlong[(k + 1) % 3] = 0;
        my_long = convert(cur, rend, srel_k, k % 3, k & 1);
        map_load(cur, tile, er);
        release(k);
        map_gather(cur, er, ge, gr);
      }
      if (k > 0) {
        const int* srel_p = s_rel + ((k - 1) & 1) * (Cfg::kTile + 1);
        const V* sprod_p = s_prod + (size_t)((k - 1) & 1) * kAcc * Cfg::kTile;
        reduce_short(prev, (k - 1) & 1, sprod_p, srel_p, prev_long ? (k - 1) % 3 : -1, (k - 1) & 1);
      }
      if (have) map_products(cur, er, ge, gr, sprod_k);
      prev_long = named_bar_or(1, BLOCK, my_long);   // [P] products, s_rel and long-row list of tile k complete
      prev = cur;
    }
  } else {
    // ---- the map needs per-row data (row-identity selectors) ---------------------------------------------
    for (int k = 0; k < count; ++k) {
      TileRef t{0, 0, 0, 0, 0};
      TileT tile;
      const OffsetT* rend = nullptr;
      if (!acquire(k, t, tile, rend)) { failed = true; break; }
      last_row1 = t.row0 + t.nrows;
      const bool my_long = convert(t, rend, s_rel, -1);
#ifdef FLEX_FORCE_EDGE_PARALLEL
      const bool long_tile = named_bar_or(1, BLOCK, true);      // experiment: every tile takes the edge-parallel path
#else
      const bool long_tile = named_bar_or(1, BLOCK, my_long);   // [R] s_rel complete, tile classified
#endif
      if (!long_tile) {
        // short rows: one thread per row does gather + map + sum in registers (the row's own vertex data is
        // loaded once) and stores the row; local row 0 continues the CTA's carry, local row `nrows`
        // (partial) becomes the next carry
        for (int r = tid; r <= t.nrows; r += BLOCK) {
          const int lo = r ? s_rel[r - 1] : 0;
          const int hi = r < t.nrows ? s_rel[r] : t.nnz;
          V sum[kAcc];
#pragma unroll
          for (int j = 0; j < kAcc; ++j) sum[j] = (r == 0) ? s_carry[(k & 1) * kAcc + j] : V(0);
          typename G::GRow grow;
          if (lo < hi) G::gather_row(p, t.row0 + r, grow);
          for (int e0 = lo; e0 < hi; e0 += Cfg::kBatch) {
            typename G::EReg er[Cfg::kBatch];
            typename G::GEdge ge[Cfg::kBatch];
#pragma unroll
            for (int b = 0; b < Cfg::kBatch; ++b)
              if (e0 + b < hi) { G::load_edge(p, tile, e0 + b, t.nz0 + e0 + b, er[b]); G::gather_edge(p, er[b], ge[b]); }
#pragma unroll
            for (int b = 0; b < Cfg::kBatch; ++b)
              if (e0 + b < hi) G::map(p, er[b], t.nz0 + e0 + b, grow, ge[b], sum);
          }
          if (r < t.nrows) {
            store_row(t.row0 + r, sum);
          } else {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) s_carry[((k + 1) & 1) * kAcc + j] = sum[j];
          }
        }
        release(k);
        continue;
      }
      // a tile with a long row: whole warps take the rows one at a time -- every lane holds the row's own record,
      // lanes map edges 32 apart, a shuffle tree folds the lanes' partial sums (no shared-memory buffers)
      for (int r = warp; r <= t.nrows; r += Cfg::kWarps) {
        const int lo = r ? s_rel[r - 1] : 0;
        const int hi = r < t.nrows ? s_rel[r] : t.nnz;
        V sum[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) sum[j] = V(0);
        if (lo < hi) {
          typename G::GRow grow;
          G::gather_row(p, t.row0 + r, grow);
          for (int e = lo + lane; e < hi; e += 32) {
            typename G::EReg er;
            typename G::GEdge ge;
            G::load_edge(p, tile, e, t.nz0 + e, er);
            G::gather_edge(p, er, ge);
            G::map(p, er, t.nz0 + e, grow, ge, sum);
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) sum[j] += shfl_down_any(sum[j], off);
          }
        }
        if (lane == 0) {
          if (r == 0) {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) sum[j] = s_carry[(k & 1) * kAcc + j] + sum[j];
          }
          if (r < t.nrows) {
            store_row(t.row0 + r, sum);
          } else {
#pragma unroll
            for (int j = 0; j < kAcc; ++j) s_carry[((k + 1) & 1) * kAcc + j] = sum[j];
          }
        }
      }
      release(k);
    }
  }

  // ---- hand the CTA's carry to the last CTA ---------------------------------------------------------
  // (nothing to hand over when the plan put the boundaries between this launch's CTAs on row ends)
  if (s_flag[1]) return;
  named_bar_sync(1, BLOCK);
  if (tid < kAcc) {
    V* cv = static_cast<V*>(a.carry_val) + (size_t)blockIdx.x * kAcc;
    cv[tid] = failed ? V(0) : s_carry[(count & 1) * kAcc + tid];
  }
  if (tid == 0) a.carry_row[blockIdx.x] = (failed || count == 0) ? a.num_rows : last_row1;
  named_bar_sync(1, BLOCK);
  if (tid == 0) {
    // one fence after the barrier orders every consumer thread's stores (rows, carries) before the ticket
    __threadfence();
    const unsigned t = atomicAdd(&a.header->ticket, 1u);
    s_flag[0] = (t == gridDim.x - 1) ? 1 : 0;
  }
  named_bar_sync(1, BLOCK);
  if (s_flag[0]) {
    __threadfence();
    const int n_cta = gridDim.x;
    const V* cvals = static_cast<const V*>(a.carry_val);
    for (int c = tid; c < n_cta; c += BLOCK) {
      // the CTA's row, its neighbours' rows and its value are requested together: one memory round trip
      const long long row = __ldcg(a.carry_row + c);
      const long long row_before = c > 0 ? __ldcg(a.carry_row + c - 1) : -1;
      long long row_after = c + 1 < n_cta ? __ldcg(a.carry_row + c + 1) : -1;
      V sum[kAcc];
#pragma unroll
      for (int i = 0; i < kAcc; ++i) sum[i] = __ldcg(cvals + (size_t)c * kAcc + i);
      if (row >= a.num_rows) continue;
      if (row_before == row) continue;   // not the head of its run
      for (int c2 = c + 1; c2 < n_cta && row_after == row; ++c2, row_after = c2 < n_cta ? __ldcg(a.carry_row + c2) : -1) {
#pragma unroll
        for (int i = 0; i < kAcc; ++i) sum[i] += __ldcg(cvals + (size_t)c2 * kAcc + i);
      }
      static_for<G::kNumReducers>([&](auto R) {
        constexpr int d = G::template red_dim<R.value>();
        constexpr int o = G::template red_off<R.value>();
        V* dst = G::template red_out<R.value>(p) + (size_t)row * d;
#pragma unroll
        for (int i = 0; i < d; ++i) dst[i] = __ldcg(dst + i) + sum[o + i];
      });
    }
    if (tid == 0) a.header->ticket = 0;
  }
}

}  // namespace flex
