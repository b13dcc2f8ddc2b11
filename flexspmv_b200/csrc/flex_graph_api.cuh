// Host side of one generated graph: workspace sizing, planning (merge-path partition into the
// workspace), launch.  FLEXSPMV_DEFINE_GRAPH(symbol_suffix, GraphStruct, Cfg) emits the five
// extern "C" entry points declared by FLEXSPMV_DECLARE_GRAPH in include/flexspmv.h.
//
// Replaces the reference's host dispatch (merged_spmv_dispatch / merged_spmv_launch,
// include/merged_spmv.cuh:22-182): no per-call device-attribute queries, no per-call temp-storage
// allocation, one kernel launch per operator call, partition cached in the caller's workspace.
#pragma once
#include <cstdlib>
#include <mutex>

#include "flex_common.cuh"
#include "flex_edge_kernel.cuh"
#include "flex_tile_kernel.cuh"
#include "flex_warp_kernel.cuh"

namespace flex {

// implemented in flex_core.cu
int partition_launch(const void* d_row_offsets, int offset_bits, long long num_rows, long long num_edges,
                     int tile_items, void* d_coords, cudaStream_t stream);
int device_sm_count();
int header_init_launch(void* ws, const WorkspaceHeader& h, cudaStream_t stream);
int snap_cta_boundaries_launch(const void* d_row_offsets, int offset_bits, long long num_rows, long long num_tiles, int grid,
                               void* d_coords, void* ws, cudaStream_t stream);
int window_plan_launch(const void* d_coords, int offset_bits, long long num_tiles, const int* d_idx, int rec_bytes,
                       int win_bytes, void* d_table, void* d_local_idx, cudaStream_t st);
int window_ready_launch(void* ws, cudaStream_t st);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// FLEXSPMV_NO_PDL=1 in the environment launches the tile kernel without the programmatic-dependent-launch attribute.
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("FLEXSPMV_NO_PDL"); return !(e && e[0] == '1'); }();
  return on;
}

struct NoWindows {   // in place of CfgWin: the gather-window variant of the kernel is not built and the flag is ignored
  static constexpr int kTile = 0;
};

struct NoLean {      // in place of CfgLean: the warp kernel for matrices with random columns is not built
  static constexpr int kChunk = 0;
};

template <class G, class Cfg, class CfgWin = Cfg, class CfgLean = NoLean>
struct GraphApi {
  static constexpr bool kWindowsBuilt = !std::is_same_v<CfgWin, NoWindows>;
  static constexpr bool kLeanBuilt = !std::is_same_v<CfgLean, NoLean>;
  using V = typename G::V;
  // edge kernel: 256 threads x 4 edges per thread (measured on B200, 2^27 edges: 2 / 4 / 8 edges per thread give
  // 91.5 / 90.8 / 62.9 % of the HBM peak for a product + global sum and 76.4 / 94.2 / 77.9 % for a gather written in place)
  static constexpr int kEdgeBlock = 256, kEdgeIpt = 4;
  // Row-mode graphs run one thread per row, the trailing partial row of the tile included: on a mesh with
  // exactly kIpt merge items per row (3 edges + the row end at kIpt = 4) a full tile holds kBlock rows plus
  // that partial row, which would cost a second pass over the rows for one thread's worth of work (measured
  // on the shallow-water model graph: 40.7 % -> 48.7 % of the HBM peak).  One row less per tile avoids it.
  static constexpr int kDefaultTile = Cfg::kTile - (G::kHasReducer && G::kGatherNeedsRow ? Cfg::kIpt : 0);

  // Gather windows are used when the graph supports them and the caller asked for them in the descriptor.
  static bool use_win(const flexspmv_desc* d) {
    if constexpr (G::kHasReducer && kWindowsBuilt) return G::kWindowGather && (d->reserved & FLEXSPMV_FLAG_GATHER_WINDOWS) != 0;
    return false;
  }
  // The warp kernel (flex_warp_kernel.cuh) is used when it was built for the graph and the caller says that the
  // gathers have no locality; it wins over the gather windows when both flags are set.
  static bool use_lean(const flexspmv_desc* d) {
    if constexpr (G::kHasReducer && kLeanBuilt) return (d->reserved & FLEXSPMV_FLAG_RANDOM_GATHER) != 0;
    return false;
  }
  static int compiled_tile(const flexspmv_desc* d) {
    if (use_lean(d)) return CfgLean::kChunk;
    return use_win(d) ? CfgWin::kTile : Cfg::kTile;
  }
  // The tile kernel's shared-memory carve-up is compiled for Cfg::kTile items; a smaller tile is allowed
  // (tests exercise odd sizes), a larger one is not.  (Shrinking the default tile on small problems until every
  // CTA gets the same number of tiles was measured on B200 and changed nothing: 13.1 us against 13.0 us per
  // launch on the 2-D Poisson 512^2 matrix.)
  static int tile_items(const flexspmv_desc* d) {
    if (d->tile_items > 0) return d->tile_items;
    if (use_lean(d)) return CfgLean::kChunk;
    return use_win(d) ? CfgWin::kTile : kDefaultTile;
  }
  static int max_ctas(const flexspmv_desc* d, int resident) {
    int m = d->max_ctas > 0 ? d->max_ctas : device_sm_count() * resident;
    return m > kMaxCtas ? kMaxCtas : (m < 1 ? 1 : m);
  }
  static int check_desc(const flexspmv_desc* d) {
    if (!d) return FLEXSPMV_ERR_BAD_ARG;
    if (d->num_rows < 0 || d->num_edges < 0) return FLEXSPMV_ERR_BAD_ARG;
    if (G::kHasReducer && d->offset_bits != 32 && d->offset_bits != 64) return FLEXSPMV_ERR_BAD_ARG;
    if (G::kHasReducer && d->tile_items > compiled_tile(d)) return FLEXSPMV_ERR_TOO_LARGE;
    if (G::kHasReducer && d->offset_bits == 32 && d->num_rows + d->num_edges >= (1ll << 31)) return FLEXSPMV_ERR_TOO_LARGE;
    return 0;
  }
  static long long num_tiles(const flexspmv_desc* d) {
    if (!G::kHasReducer) return 0;
    const long long t = tile_items(d);
    return (d->num_rows + d->num_edges + t - 1) / t;
  }
  static void layout(const flexspmv_desc* d, WorkspaceHeader& h) {
    const long long tiles = num_tiles(d);
    const uint64_t pair = (d->offset_bits == 64 ? 16u : 8u);
    h.coords_offset = sizeof(WorkspaceHeader);
    h.carry_row_offset = align_up(h.coords_offset + (uint64_t)(tiles + 1) * pair, 256);
    const uint64_t carries = use_lean(d) ? kMaxWarpCarries : kMaxCtas;      // one carry per CTA, or per warp
    h.carry_val_offset = align_up(h.carry_row_offset + carries * 8u, 256);
    const int width = G::kHasReducer ? G::kAccDim : (G::kAggDim > 0 ? G::kAggDim : 1);
    h.total_bytes = align_up(h.carry_val_offset + carries * width * sizeof(V), 256);
    h.win_table_offset = h.win_index_offset = 0;
    if (use_win(d) && !use_lean(d)) {
      h.win_table_offset = h.total_bytes;
      h.win_index_offset = align_up(h.win_table_offset + (uint64_t)tiles * kWinEntryInts * 4u, 256);
      h.total_bytes = align_up(h.win_index_offset + (uint64_t)d->num_edges * 2u, 256);
    }
  }

  static int info(flexspmv_graph_info* o) {
    if (!o) return FLEXSPMV_ERR_BAD_ARG;
    o->num_values = G::kNumValues; o->num_indices = G::kNumIndices; o->num_outputs = G::kNumOutputs;
    o->has_reducer = G::kHasReducer ? 1 : 0; o->value_bytes = (int)sizeof(V);
    o->default_tile_items = kDefaultTile; o->block_threads = Cfg::kBlock; o->items_per_thread = Cfg::kIpt;
    o->stages = Cfg::kStages;
    o->smem_bytes = 0;
    if constexpr (G::kHasReducer) o->smem_bytes = TileSmemLayout<G, long long, Cfg>::kTotal;
    o->acc_dim = G::kHasReducer ? G::kAccDim : G::kAggDim;
    o->reserved = 0;
    // bit 0: the graph can use gather windows, bit 1: the warp kernel for random columns is built
    if constexpr (G::kHasReducer) o->reserved = ((G::kWindowGather && kWindowsBuilt) ? 1 : 0) | (kLeanBuilt ? 2 : 0);
    return 0;
  }

  static int workspace_bytes(const flexspmv_desc* d, size_t* bytes) {
    if (int e = check_desc(d)) return e;
    if (!bytes) return FLEXSPMV_ERR_BAD_ARG;
    WorkspaceHeader h{};
    layout(d, h);
    *bytes = (size_t)h.total_bytes;
    return 0;
  }

  static int plan(const flexspmv_desc* d, const void* row_offsets, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (int e = check_desc(d)) return e;
    if (!ws) return FLEXSPMV_ERR_WORKSPACE;
    WorkspaceHeader h{};
    layout(d, h);
    if (ws_bytes < h.total_bytes) return FLEXSPMV_ERR_WORKSPACE;
    if (!aligned16(ws)) return FLEXSPMV_ERR_ALIGN;
    h.magic = kMagic; h.ticket = 0; h.status = 0; h.offset_bits = d->offset_bits;
    h.num_rows = d->num_rows; h.num_edges = d->num_edges; h.num_tiles = num_tiles(d);
    h.tile_items = tile_items(d); h.max_ctas = d->max_ctas;
    if (int e = header_init_launch(ws, h, st)) return e;   // a one-thread kernel: stream-ordered, no host sync
    if (G::kHasReducer) {
      if (!row_offsets) return FLEXSPMV_ERR_BAD_ARG;
      if (!aligned16(row_offsets)) return FLEXSPMV_ERR_ALIGN;
      if (int e = partition_launch(row_offsets, d->offset_bits, d->num_rows, d->num_edges, tile_items(d),
                                   static_cast<char*>(ws) + h.coords_offset, st)) return e;
      // the tile kernel: boundaries between the CTAs of its grid moved onto row ends where the tiles have room
      if (!use_lean(d) && h.num_tiles > 1) {
        int resident = 0;
        int e = 0;
        bool win = false;
        if constexpr (G::kWindowGather && kWindowsBuilt) win = use_win(d);
        if constexpr (G::kWindowGather && kWindowsBuilt) {
          if (win) e = d->offset_bits == 64 ? resident_ctas<long long, CfgWin, true>(&resident) : resident_ctas<int, CfgWin, true>(&resident);
        }
        if (!win) e = d->offset_bits == 64 ? resident_ctas<long long>(&resident) : resident_ctas<int>(&resident);
        if (e) return e;
        long long grid = max_ctas(d, resident);
        if (grid > h.num_tiles) grid = h.num_tiles;
        return snap_cta_boundaries_launch(row_offsets, d->offset_bits, d->num_rows, h.num_tiles, (int)grid,
                                          static_cast<char*>(ws) + h.coords_offset, ws, st);
      }
      return 0;
    }
    return 0;
  }

  // CTAs of the tile kernel that one SM holds.  The shared-memory opt-in and the occupancy are per device: looked up
  // once for each device of the process.
  template <typename OffsetT, class C = Cfg, bool WIN = false>
  static int resident_ctas(int* out) {
    using L = TileSmemLayout<G, OffsetT, C, WIN>;
    static_assert(L::kTotal <= 227 * 1024, "tile kernel needs more shared memory than one sm_100a CTA can have");
    auto kernel = flex_tile_kernel<G, OffsetT, C, WIN>;
    constexpr int kThreads = C::kBlock + (G::kDirectLoads ? 0 : 32);
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static int resident_of[kMaxDevices] = {};      // 0: not initialised yet
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return FLEXSPMV_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (resident_of[dev] == 0) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
      int r = 0;
      if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, kernel, kThreads, L::kTotal);
      if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
      resident_of[dev] = r < 1 ? -1 : r;
    }
    if (resident_of[dev] < 1) return FLEXSPMV_ERR_TOO_LARGE;
    *out = resident_of[dev];
    return 0;
  }

  template <typename OffsetT, class C = Cfg, bool WIN = false>
  static int launch_tiles(const flexspmv_desc* d, const typename G::Params& p, const void* row_offsets, void* ws,
                          const WorkspaceHeader& h, cudaStream_t st) {
    using L = TileSmemLayout<G, OffsetT, C, WIN>;
    auto kernel = flex_tile_kernel<G, OffsetT, C, WIN>;
    constexpr int kThreads = C::kBlock + (G::kDirectLoads ? 0 : 32);   // staged mode adds the producer warp
    int resident = 0;
    if (int e = resident_ctas<OffsetT, C, WIN>(&resident)) return e;
    const long long tiles = h.num_tiles;
    if (tiles == 0) return 0;
    long long grid = max_ctas(d, resident);
    if (grid > tiles) grid = tiles;
    TileKernelArgs a;
    a.row_offsets = row_offsets;
    a.coords = static_cast<char*>(ws) + h.coords_offset;
    a.header = static_cast<WorkspaceHeader*>(ws);
    a.carry_row = reinterpret_cast<long long*>(static_cast<char*>(ws) + h.carry_row_offset);
    a.carry_val = static_cast<char*>(ws) + h.carry_val_offset;
    a.num_rows = d->num_rows; a.num_edges = d->num_edges; a.num_tiles = tiles;
    a.win_table = nullptr; a.win_index = nullptr; a.num_vertices = d->num_vertices;
    if constexpr (WIN) {
      if (d->num_vertices <= 0) return FLEXSPMV_ERR_BAD_ARG;
      if (!aligned16(G::gather_base(p))) return FLEXSPMV_ERR_ALIGN;   // window sources are 16-byte aligned only then
      a.win_table = reinterpret_cast<const int*>(static_cast<char*>(ws) + h.win_table_offset);
      a.win_index = reinterpret_cast<const unsigned short*>(static_cast<char*>(ws) + h.win_index_offset);
    }
    // Programmatic dependent launch: the CTAs may be placed while the kernel before this one on the stream drains; the
    // kernel touches no global memory before its griddepcontrol.wait.  Back-to-back launches of small problems
    // (a time-stepping loop) then overlap one launch's set-up with the tail of the one before.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = L::kTotal; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, p, a);
  }

  template <typename OffsetT>
  static int launch_lean(const flexspmv_desc* d, const typename G::Params& p, const void* row_offsets, void* ws,
                         const WorkspaceHeader& h, cudaStream_t st) {
    if constexpr (G::kHasReducer && kLeanBuilt) {
      auto kernel = flex_warp_kernel<G, OffsetT, CfgLean>;
      // per warp: the product slots and marker words of one chunk (WarpSmem, the layout of flex_warp_kernel)
      constexpr int kSmem = WarpSmem<G, CfgLean>::template cta_bytes<OffsetT>();
      constexpr int kMaxDevices = 64;
      static std::mutex mu;
      static int resident_of[kMaxDevices] = {};      // 0: not initialised yet
      int dev = 0;
      if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return (int)e;
      if (dev < 0 || dev >= kMaxDevices) return FLEXSPMV_ERR_BAD_ARG;
      int resident = 0;
      {
        std::lock_guard<std::mutex> lock(mu);
        if (resident_of[dev] == 0) {
          cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
          int r = 0;
          if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&r, kernel, CfgLean::kBlock, kSmem);
          if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
          resident_of[dev] = r < 1 ? -1 : r;
        }
        resident = resident_of[dev];
      }
      if (resident < 1) return FLEXSPMV_ERR_TOO_LARGE;
      const long long chunks = h.num_tiles;
      if (chunks == 0) return 0;
      long long grid = d->max_ctas > 0 ? d->max_ctas : (long long)device_sm_count() * resident;
      const long long need = (chunks + CfgLean::kWarps - 1) / CfgLean::kWarps;
      if (grid > need) grid = need;
      if (grid > kMaxWarpCarries / CfgLean::kWarps) grid = kMaxWarpCarries / CfgLean::kWarps;
      if (grid < 1) grid = 1;
      WarpKernelArgs a;
      a.row_offsets = row_offsets;
      a.coords = static_cast<char*>(ws) + h.coords_offset;
      a.header = static_cast<WorkspaceHeader*>(ws);
      a.carry_row = reinterpret_cast<long long*>(static_cast<char*>(ws) + h.carry_row_offset);
      a.carry_val = static_cast<char*>(ws) + h.carry_val_offset;
      a.num_rows = d->num_rows; a.num_edges = d->num_edges; a.num_chunks = chunks;
      kernel<<<(unsigned)grid, CfgLean::kBlock, kSmem, st>>>(p, a);
      return (int)cudaGetLastError();
    } else {
      (void)d; (void)p; (void)row_offsets; (void)ws; (void)h; (void)st;
      return FLEXSPMV_ERR_BAD_ARG;
    }
  }

  // Second planning step for descriptors with FLEXSPMV_FLAG_GATHER_WINDOWS (after plan, same workspace): reads the
  // index array of the graph's one gather and fills the per-tile segment table and the per-edge positions.
  // Until it has run, a launch treats every tile as having no windows.
  static int plan_windows(const flexspmv_desc* d, const void* const* indices, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (int e = check_desc(d)) return e;
    if (!use_win(d) || use_lean(d)) return 0;          // nothing to do for graphs / descriptors without windows
    if constexpr (G::kHasReducer && G::kWindowGather && kWindowsBuilt) {
      if (!ws) return FLEXSPMV_ERR_WORKSPACE;
      if (!indices || !indices[0]) return FLEXSPMV_ERR_BAD_ARG;
      WorkspaceHeader h{};
      layout(d, h);
      if (ws_bytes < h.total_bytes) return FLEXSPMV_ERR_WORKSPACE;
      char* base = static_cast<char*>(ws);
      if (int e = window_plan_launch(base + h.coords_offset, d->offset_bits, num_tiles(d), static_cast<const int*>(indices[0]),
                                     G::kGatherRecBytes, G::kWinBytes, base + h.win_table_offset, base + h.win_index_offset, st))
        return e;
      return window_ready_launch(ws, st);
    }
    return 0;
  }

  static int launch(const flexspmv_desc* d, const void* const* values, const void* const* indices,
                    const void* row_offsets, void* const* outputs, void* ws, size_t ws_bytes, cudaStream_t st) {
    if (int e = check_desc(d)) return e;
    if (!ws) return FLEXSPMV_ERR_WORKSPACE;
    if ((G::kNumValues && !values) || (G::kNumIndices && !indices) || (G::kNumOutputs && !outputs)) return FLEXSPMV_ERR_BAD_ARG;
    WorkspaceHeader h{};
    layout(d, h);
    if (ws_bytes < h.total_bytes) return FLEXSPMV_ERR_WORKSPACE;
    h.num_tiles = num_tiles(d);
    for (int i = 0; i < G::kNumValues; ++i) if (!values[i]) return FLEXSPMV_ERR_BAD_ARG;
    for (int i = 0; i < G::kNumIndices; ++i) if (!indices[i]) return FLEXSPMV_ERR_BAD_ARG;
    for (int i = 0; i < G::kNumOutputs; ++i) if (!outputs[i]) return FLEXSPMV_ERR_BAD_ARG;
    typename G::Params p = G::make_params(values, indices, outputs);
    if (!G::pointers_aligned(p)) return FLEXSPMV_ERR_ALIGN;
    if constexpr (G::kHasReducer) {
      if (!row_offsets) return FLEXSPMV_ERR_BAD_ARG;
      if (!aligned16(row_offsets)) return FLEXSPMV_ERR_ALIGN;
      if (use_lean(d)) {
        if (d->offset_bits == 64) return launch_lean<long long>(d, p, row_offsets, ws, h, st);
        return launch_lean<int>(d, p, row_offsets, ws, h, st);
      }
      if constexpr (G::kWindowGather && kWindowsBuilt) {
        if (use_win(d)) {
          if (d->offset_bits == 64) return launch_tiles<long long, CfgWin, true>(d, p, row_offsets, ws, h, st);
          return launch_tiles<int, CfgWin, true>(d, p, row_offsets, ws, h, st);
        }
      }
      if (d->offset_bits == 64) return launch_tiles<long long>(d, p, row_offsets, ws, h, st);
      return launch_tiles<int>(d, p, row_offsets, ws, h, st);
    } else {
    if (d->num_edges == 0 && G::kAggDim == 0) return 0;
    const long long tile_edges = (long long)kEdgeBlock * kEdgeIpt;
    long long grid = (d->num_edges + tile_edges - 1) / tile_edges;
    const long long cap = max_ctas(d, 2048 / kEdgeBlock);
    if (grid > cap) grid = cap;
    if (grid < 1) grid = 1;
    EdgeKernelArgs a;
    a.header = static_cast<WorkspaceHeader*>(ws);
    a.partials = static_cast<char*>(ws) + h.carry_val_offset;
    a.num_edges = d->num_edges;
    flex_edge_kernel<G, kEdgeBlock, kEdgeIpt><<<(unsigned)grid, kEdgeBlock, 0, st>>>(p, a);
    return (int)cudaGetLastError();
    }
  }

  static int device_status(const void* ws, int32_t* d_out, cudaStream_t st) {
    if (!ws || !d_out) return FLEXSPMV_ERR_BAD_ARG;
    const char* src = static_cast<const char*>(ws) + offsetof(WorkspaceHeader, status);
    return (int)cudaMemcpyAsync(d_out, src, sizeof(int32_t), cudaMemcpyDefault, st);
  }
};

}  // namespace flex

#define FLEXSPMV_DEFINE_GRAPH(SYM, GRAPH, CFG, CFGWIN, CFGLEAN)                                                          \
  extern "C" {                                                                                                  \
  int flexspmv_##SYM##_info(flexspmv_graph_info* info) { return flex::GraphApi<GRAPH, CFG, CFGWIN, CFGLEAN>::info(info); } \
  int flexspmv_##SYM##_workspace_bytes(const flexspmv_desc* d, size_t* b) {                                     \
    return flex::GraphApi<GRAPH, CFG, CFGWIN, CFGLEAN>::workspace_bytes(d, b);                                           \
  }                                                                                                             \
  int flexspmv_##SYM##_plan(const flexspmv_desc* d, const void* ro, void* ws, size_t wb, void* st) {            \
    return flex::GraphApi<GRAPH, CFG, CFGWIN, CFGLEAN>::plan(d, ro, ws, wb, static_cast<cudaStream_t>(st));              \
  }                                                                                                             \
  int flexspmv_##SYM##_plan_windows(const flexspmv_desc* d, const void* const* ix, void* ws, size_t wb, void* st) { \
    return flex::GraphApi<GRAPH, CFG, CFGWIN, CFGLEAN>::plan_windows(d, ix, ws, wb, static_cast<cudaStream_t>(st));      \
  }                                                                                                             \
  int flexspmv_##SYM##_launch(const flexspmv_desc* d, const void* const* v, const void* const* ix,              \
                              const void* ro, void* const* o, void* ws, size_t wb, void* st) {                  \
    return flex::GraphApi<GRAPH, CFG, CFGWIN, CFGLEAN>::launch(d, v, ix, ro, o, ws, wb, static_cast<cudaStream_t>(st));  \
  }                                                                                                             \
  int flexspmv_##SYM##_device_status(const void* ws, int32_t* out, void* st) {                                  \
    return flex::GraphApi<GRAPH, CFG, CFGWIN, CFGLEAN>::device_status(ws, out, static_cast<cudaStream_t>(st));           \
  }                                                                                                             \
  }


// ---- an entry point for callers that cannot allocate device memory -----------------------------------
// FLEXSPMV_DEFINE_STATIC_SCRATCH_LAUNCH(symbol_suffix, GraphStruct, Cfg, BYTES) expands, inside the
// translation unit of one graph, to a file-scope device array of BYTES bytes and to
//   int flexspmv_<suffix>_launch_static(desc, values, indices, row_offsets, outputs, stream)
// which plans the problem into that array and launches the fused pass, calling no allocator of any kind.
// The array's name is only a host-side handle for the symbol; its device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and cached.
#define FLEXSPMV_DEFINE_STATIC_SCRATCH_LAUNCH(SYM, GRAPH, CFG, BYTES)                                           \
  static __device__ __align__(256) unsigned char flexspmv_static_scratch_##SYM[BYTES];                          \
  namespace {                                                                                                   \
  struct StaticScratch_##SYM {                                                                                  \
    std::mutex mu;                                                                                              \
    void* ptr[64] = {};                                                                                         \
    int lookup(void** out) {                                                                                    \
      int dev = -1;                                                                                             \
      cudaError_t e = cudaGetDevice(&dev);                                                                      \
      if (e != cudaSuccess) return (int)e;                                                                      \
      if (dev < 0 || dev >= 64) return FLEXSPMV_ERR_BAD_ARG;                                                    \
      std::lock_guard<std::mutex> lock(mu);                                                                     \
      if (!ptr[dev]) {                                                                                          \
        void* p = nullptr;                                                                                      \
        e = cudaGetSymbolAddress(&p, flexspmv_static_scratch_##SYM);                                            \
        if (e != cudaSuccess) return (int)e;                                                                    \
        ptr[dev] = p;                                                                                           \
      }                                                                                                         \
      *out = ptr[dev];                                                                                          \
      return 0;                                                                                                 \
    }                                                                                                           \
  } static_scratch_##SYM;                                                                                       \
  }                                                                                                             \
  extern "C" int flexspmv_##SYM##_launch_static(const flexspmv_desc* d_in, const void* const* v,                \
                                                const void* const* ix, const void* ro, void* const* o,          \
                                                void* st) {                                                     \
    using Api = flex::GraphApi<GRAPH, CFG, flex::NoWindows>;                                                    \
    if (!d_in) return FLEXSPMV_ERR_BAD_ARG;                                                                     \
    flexspmv_desc desc = *d_in;                                                                                 \
    desc.reserved = 0; /* gather windows need a second planning step and 2 bytes of scratch per edge: not here */ \
    const flexspmv_desc* d = &desc;                                                                             \
    size_t need = 0;                                                                                            \
    if (int e = Api::workspace_bytes(d, &need)) return e;                                                       \
    if (need > (size_t)(BYTES)) return FLEXSPMV_ERR_STATIC_SCRATCH;                                             \
    void* ws = nullptr;                                                                                         \
    if (int e = static_scratch_##SYM.lookup(&ws)) return e;                                                     \
    cudaStream_t stream = static_cast<cudaStream_t>(st);                                                        \
    /* the array keeps the previous call's contents: planning rewrites the header (ticket, status) and */      \
    /* every tile coordinate this problem reads; the carry slots are written before they are read      */      \
    if (int e = Api::plan(d, ro, ws, (size_t)(BYTES), stream)) return e;                                        \
    return Api::launch(d, v, ix, ro, o, ws, (size_t)(BYTES), stream);                                           \
  }                                                                                                             \
  extern "C" int flexspmv_##SYM##_static_device_status(int32_t* d_out, void* st) {                              \
    void* ws = nullptr;                                                                                         \
    if (int e = static_scratch_##SYM.lookup(&ws)) return e;                                                     \
    return flex::GraphApi<GRAPH, CFG, flex::NoWindows>::device_status(ws, d_out, static_cast<cudaStream_t>(st)); \
  }
