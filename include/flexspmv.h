/*
 * flexspmv.h -- C ABI of the B200 (sm_100a) fused gather -> per-edge map -> segmented reduce-by-row
 * library (libflexspmv_b200.so).
 *
 * Conventions for every entry point:
 *   - plain C, no exceptions cross the boundary; the return value is a status:
 *       0 = success, negative = FLEXSPMV_ERR_* below, positive = a cudaError_t from the runtime;
 *   - all device work is enqueued on the caller's stream (a cudaStream_t passed as void*); nothing
 *     synchronises the device or the stream and nothing is allocated or freed: scratch memory comes
 *     from the caller ("workspace"), sized by the matching *_workspace_bytes call;
 *   - device pointers of streamed arrays (per-edge tensors, index arrays, row offsets) must be
 *     16-byte aligned (bulk-copy staging); gather sources and outputs need only their natural
 *     alignment;
 *   - row offsets always include the leading 0 (length num_rows + 1), as the reference operator
 *     receives them (the callee skips it: include/merged_spmv.cuh:169,
 *     cpu_template/merged_spmv_template_reducer.h:97).
 *
 * Reference interfaces replaced (paths inside the FlexSpmv project):
 *   merged::merged_spmv_launch<ValueT,OffsetT>(FlexParams, void* d_temp, size_t& bytes, bool, stream)
 *       include/merged_spmv.cuh:149-182 (two-phase temp-storage convention) and its dispatch
 *       merged_spmv_dispatch include/merged_spmv.cuh:22-144      -> flexspmv_<graph>_* below
 *   SpmvSearchKernel / MergePathSearch  include/merged_spmv_kernels.cuh:19-99 -> flexspmv_partition
 *   FlexParams pointer bundle           include/merged_utils.cuh:243-262      -> flexspmv_desc + the
 *       three pointer arrays of flexspmv_<graph>_launch
 */
#ifndef FLEXSPMV_H_
#define FLEXSPMV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLEXSPMV_ABI_VERSION 1

enum {
  FLEXSPMV_OK = 0,
  FLEXSPMV_ERR_BAD_ARG = -1,       /* null pointer, negative size, unsupported offset width        */
  FLEXSPMV_ERR_ALIGN = -2,         /* a streamed array is not 16-byte aligned                      */
  FLEXSPMV_ERR_WORKSPACE = -3,     /* workspace missing or smaller than *_workspace_bytes reports  */
  FLEXSPMV_ERR_TOO_LARGE = -4,     /* size beyond what the entry point supports                    */
  FLEXSPMV_ERR_BAD_CSR = -5,       /* row offsets not monotone / inconsistent with num_edges       */
  FLEXSPMV_ERR_TIMEOUT = -6,       /* a bounded device-side wait ran out (read via *_device_status)*/
  FLEXSPMV_ERR_NOT_PLANNED = -7,   /* launch called on a workspace that was never planned          */
  FLEXSPMV_ERR_STATIC_SCRATCH = -8 /* problem needs more scratch than the built-in static array     */
};

/* Problem descriptor shared by the plan / launch calls of every graph. */
typedef struct flexspmv_desc {
  int64_t num_rows;      /* rows of the reduce-by-row (0 for graphs without a reducer)              */
  int64_t num_edges;     /* edges = non-zeros = length of every per-edge array                      */
  int64_t num_vertices;  /* rows of the gather sources (informational; used by validation)          */
  int32_t offset_bits;   /* 32 or 64: width of the row-offset entries                               */
  int32_t tile_items;    /* merge items (rows + edges) per tile; 0 = the graph's compiled default   */
  int32_t max_ctas;      /* cap on persistent CTAs; 0 = SM count x resident CTAs per SM.  plan() lays the tile
                            boundaries between the CTAs of THIS grid on row ends where it can; a launch with
                            another value still works but hands carries between its CTAs            */
  int32_t reserved;      /* flags: 0 or an OR of the FLEXSPMV_FLAG_* below (field name kept from ABI 1) */
} flexspmv_desc;

/*
 * Gather windows (no reference counterpart; graphs whose flexspmv_graph_info.reserved has bit 0 set).
 * With this flag in the descriptor -- the same descriptor for workspace_bytes, plan, plan_windows and
 * launch -- the workspace also holds, per tile, up to 12 column segments that cover every column the
 * tile gathers from and, per edge, the 16-bit position of its column in those segments (2 bytes per
 * edge of extra workspace).  The kernel then stages the segments of the gathered array with bulk
 * copies and gathers from shared memory, and it streams the positions instead of the 4-byte column
 * indices.  Pays on stencil / banded matrices that are applied many times; tiles that touch too many
 * separate column ranges (random columns) keep their global gathers.  The gathered array must be
 * 16-byte aligned and num_vertices must be its number of rows.  Results are bit-identical to the
 * plain path run with the same tile size and CTA count.
 */
#define FLEXSPMV_FLAG_GATHER_WINDOWS 1

/*
 * Random gathers (no reference counterpart; graphs whose flexspmv_graph_info.reserved has bit 1 set).
 * The caller states that the columns of the matrix have no locality (consecutive edges gather from unrelated
 * cache lines: power-law graphs, random sparse matrices).  With this flag in the descriptor -- the same for
 * workspace_bytes, plan and launch -- a kernel without shared-memory staging runs instead: on such matrices
 * the bound is the number of gather misses an SM has in flight, which grows with the part of the L1 /
 * shared-memory array that stays cache.  The plan then splits the merge path into chunks of 32 x
 * (items per lane) items, one warp each.  Results agree with the plain path to the parity tolerance (the
 * summation order inside a row differs); run-to-run deterministic.  Ignored by graphs that were not built
 * with that kernel.  On stencil / banded matrices the plain path is faster.
 */
#define FLEXSPMV_FLAG_RANDOM_GATHER 2

/* ---- library-wide ----------------------------------------------------------------------------- */

/* ABI version of the loaded library (FLEXSPMV_ABI_VERSION it was built with). */
int flexspmv_abi_version(void);

/* Static, NUL-terminated description of a status returned by this library. */
const char *flexspmv_error_string(int status);

/*
 * Merge-path partition: coordinates (row, edge) where the diagonals t * tile_items, t in
 * [0, num_tiles], cross the merge path of (row END offsets) x (0..num_edges-1); num_tiles =
 * ceil((num_rows + num_edges) / tile_items).  Output: (num_tiles + 1) pairs of int32 (offset_bits 32)
 * or int64 (offset_bits 64) in device memory, bit-identical to the reference search.
 * Replaces SpmvSearchKernel, include/merged_spmv_kernels.cuh:60-99 (MergePathSearch :19-50).
 */
int flexspmv_partition_bytes(int64_t num_rows, int64_t num_edges, int32_t offset_bits,
                             int32_t tile_items, size_t *bytes);
int flexspmv_partition(const void *d_row_offsets, int32_t offset_bits, int64_t num_rows,
                       int64_t num_edges, int32_t tile_items, void *d_coords, void *stream);

/*
 * nnz-balanced contiguous row blocks for the multi-GPU split: d_first_row[k] (int64, parts + 1
 * entries, device) = lower_bound(row_offsets, k * nnz / parts), rounded to the nearest multiple of
 * `snap` rows (snap <= 1: no rounding); d_first_row[0] = 0, d_first_row[parts] = num_rows.
 * No counterpart in the reference (it has no multi-GPU code); the search is the same lower-bound
 * family as MergePathSearch.
 */
int flexspmv_row_blocks(const void *d_row_offsets, int32_t offset_bits, int64_t num_rows,
                        int32_t parts, int64_t snap, int64_t *d_first_row, void *stream);

/*
 * Testing aid for the bounded device-side waits: after this call, launches on the planned workspace never
 * fill the stage of tile `first_tile_plus_one - 1` nor of any later tile (0 switches the aid off; plan
 * resets it).  The consumers of such a tile wait for their bounded time (one second), the kernel sets
 * FLEXSPMV_ERR_TIMEOUT in the workspace status (read it with *_device_status) and returns; rows of the
 * withheld tiles are not written.  No reference counterpart (its kernels have no waits).
 */
int flexspmv_debug_withhold_stage(void *d_workspace, uint32_t first_tile_plus_one, void *stream);

/*
 * Measurement aid: the rate at which the GPU gathers 4-byte records without locality.  Streams d_idx / d_vals
 * (num_edges entries, coalesced), gathers d_x[d_idx[e]] and accumulates; writes nothing (d_out needs `ctas` floats
 * and stays untouched).  `smem_bytes_per_cta` of unused dynamic shared memory per 256-thread CTA shrink the L1
 * that is left to the misses in flight (the driver sizes the carve-out for 8 such CTAs per SM).  Time it with
 * events: num_edges / time is the bound of any kernel that gathers this index array.  No reference counterpart.
 */
int flexspmv_probe_gather(const int32_t *d_idx, const float *d_vals, const float *d_x, int64_t num_edges,
                          float *d_out, int32_t ctas, int32_t smem_bytes_per_cta, void *stream);

/*
 * Host-visible copy of a workspace's status word.  `pinned_host_status` is an int32 in page-locked host
 * memory (cudaHostAlloc / cudaHostRegister; NULL removes the registration).  From then on a kernel that
 * raises FLEXSPMV_ERR_TIMEOUT or FLEXSPMV_ERR_NOT_PLANNED on this workspace also stores the code there, so
 * the host can notice a failed launch by reading one int -- no copy, no synchronisation on the launch path.
 * The call itself stores the current status (normally 0).  Planning the workspace again drops the
 * registration.  After FLEXSPMV_ERR_TIMEOUT the outputs of that launch are undefined (rows of the tiles
 * that were not reached are not written).  No reference counterpart (its kernels cannot fail this way).
 */
int flexspmv_workspace_status_mirror(void *d_workspace, int32_t *pinned_host_status, void *stream);

/*
 * Halo plan of a 1-D row-block partition (host only, pure integers): given the world + 1 block
 * boundaries and, per block, the smallest and largest global column its rows reference (for an empty
 * block: row_begin and row_begin - 1), computes for every rank how many vector entries it needs from
 * the block below / above (halo_lo / halo_hi) and how many of its own head / tail entries the
 * neighbours need (send_lo / send_hi).  The local vector of a rank is laid out
 * [halo_lo | owned rows | halo_hi]; global column - (row_begin - halo_lo) indexes it.
 * FLEXSPMV_ERR_TOO_LARGE when a halo reaches beyond the neighbouring block (matrix not banded enough
 * for a nearest-neighbour exchange).  No counterpart in the reference (it has no multi-GPU code).
 */
typedef struct flexspmv_halo_plan_t {
  int64_t row_begin, row_end;
  int64_t halo_lo, halo_hi;
  int64_t send_lo, send_hi;
} flexspmv_halo_plan_t;
int flexspmv_halo_plan(const int64_t *first_row, const int64_t *min_col, const int64_t *max_col,
                       int32_t world, flexspmv_halo_plan_t *plans);

/*
 * Debug validator: checks on the device that row offsets start at 0, are non-decreasing and end at
 * num_edges, and (when d_index != NULL) that every index lies in [0, num_vertices).  Writes 0 or a
 * FLEXSPMV_ERR_* to the int32 *d_status (device).  No reference counterpart (the reference never
 * validates: python_wrapper/dynamic_replace_submodule.py:20-41 assumes sorted rows).
 */
int flexspmv_validate_csr(const void *d_row_offsets, int32_t offset_bits, int64_t num_rows,
                          int64_t num_edges, const int32_t *d_index, int64_t num_vertices,
                          int32_t *d_status, void *stream);

/*
 * Sorted COO row ids (the Reducer's index, int32 or int64) -> CSR row offsets with the leading 0
 * (num_rows + 1 entries, int32 or int64): what _coo_rows_to_csr_ptr computes with bincount + cumsum
 * (python_wrapper/dynamic_replace_submodule.py:20-41), on the device in one launch.  Unlike the
 * reference it checks its precondition: *d_status (device int32) becomes FLEXSPMV_ERR_BAD_CSR when
 * the ids are not ascending, FLEXSPMV_ERR_BAD_ARG when one lies outside [0, num_rows), else 0.
 */
int flexspmv_coo_rows_to_csr(const void *d_row_ids, int32_t id_bits, int64_t num_edges,
                             int64_t num_rows, void *d_row_offsets, int32_t offset_bits,
                             int32_t *d_status, void *stream);

/*
 * Unsorted reducers: a stable sort of the edges by row id.  d_perm (int32, num_edges entries) receives the
 * permutation -- d_perm[k] = original position of the edge that comes k-th when the edges are ordered by row,
 * edges of one row keeping their input order (a stable argsort) -- and d_row_offsets the CSR offsets with the
 * leading 0 of the sorted order.  The caller permutes its per-edge arrays once with flexspmv_permute_edges
 * (dst[k] = src[d_perm[k]], records of record_bytes bytes, a multiple of 4) and then uses the CSR kernels.
 * Scratch: flexspmv_sort_rows_bytes(num_edges) bytes, 16-byte aligned.  *d_status (device int32) becomes
 * FLEXSPMV_ERR_BAD_ARG when an id lies outside [0, num_rows), else 0.  num_edges and num_rows < 2^31.
 * The reference has no counterpart: its _coo_rows_to_csr_ptr assumes ascending ids and is silently wrong
 * otherwise (python_wrapper/dynamic_replace_submodule.py:20-41).
 */
int flexspmv_sort_rows_bytes(int64_t num_edges, size_t *bytes);
int flexspmv_sort_rows(const void *d_row_ids, int32_t id_bits, int64_t num_edges, int64_t num_rows,
                       int32_t *d_perm, void *d_row_offsets, int32_t offset_bits, void *d_scratch,
                       size_t scratch_bytes, int32_t *d_status, void *stream);
int flexspmv_permute_edges(const void *d_src, void *d_dst, const int32_t *d_perm, int64_t num_edges,
                           int32_t record_bytes, void *stream);

/*
 * One Runge-Kutta stage of the per-cell arithmetic of the reference's shallow-water model
 * (shallow_water_equation/swe_main.py:100-146), which the reference leaves to torch element-wise
 * kernels: with r = the three interior reducer sums and rb = the two boundary sums,
 *   d_k   = -(r_k [+ rb_k]) / area                      (k = h, uh, vh; rb only for uh, vh)
 *   acc_k = first ? d_k : acc_k + d_k
 *   last  ? x_k += w * acc_k  :  stage_k = x_k + c * d_k
 * d_r, d_x, d_acc, d_stage: 3 device pointers each; d_rb: 2; value_bytes 4 | 8; all arrays n long.
 */
int flexspmv_swe_rk_stage(int32_t value_bytes, const void *const *d_r, const void *const *d_rb,
                          const void *d_area, void *const *d_x, void *const *d_acc,
                          void *const *d_stage, double c, double w, int64_t n, int32_t first,
                          int32_t last, void *stream);

/* ---- per fused graph ---------------------------------------------------------------------------
 * One set of five symbols per (graph, value type); the per-edge map is compiled into the kernel, so
 * a graph is identified by its symbol prefix.  For graph G and value type T (f32 | f64 | i64):
 *
 *   flexspmv_G_T_info            sizes of the three pointer arrays and of the compiled defaults
 *   flexspmv_G_T_workspace_bytes scratch size for a problem (first phase of the reference's
 *                                two-phase temp-storage call, include/merged_spmv.cuh:84-92)
 *   flexspmv_G_T_plan            partitions the problem into the workspace (cacheable while the row
 *                                offsets do not change; replaces the per-call search kernel,
 *                                include/merged_spmv.cuh:98-119)
 *   flexspmv_G_T_plan_windows    second planning step of descriptors with FLEXSPMV_FLAG_GATHER_WINDOWS,
 *                                after plan on the same workspace; takes the index arrays of launch.
 *                                A no-op (returns 0) for other descriptors and graphs.
 *   flexspmv_G_T_launch          one fused pass (replaces SpmvKernel + AgentFlexSpmv::ConsumeTile,
 *                                include/merged_spmv_kernels.cuh:110-128,
 *                                cuda_template/reducer/merged_agent_spmv_template.cuh:350-445, and
 *                                the aggregator flavour cuda_template/aggregator/...:348-409).
 *                                Every output element is written (outputs need no zero fill).
 *   flexspmv_G_T_device_status   copies the workspace's device status word into *d_status_out
 *                                (int32 in device or page-locked host memory) without synchronising
 *
 * Pointer arrays of launch (device pointers; order = the operator's positional order,
 * codegen/merged_gen_binding.py:65-78):
 *   values[]  non-gather value inputs then gather value inputs
 *   indices[] one int32 index array per distinct selector target
 *   outputs[] one array per graph output (reducer (num_rows, dim), sum (dim), per-edge (ne, dim))
 */
typedef struct flexspmv_graph_info {
  int32_t num_values;
  int32_t num_indices;
  int32_t num_outputs;
  int32_t has_reducer;
  int32_t value_bytes;
  int32_t default_tile_items;
  int32_t block_threads;
  int32_t items_per_thread;
  int32_t stages;
  int32_t smem_bytes;
  int32_t acc_dim;
  int32_t reserved;
} flexspmv_graph_info;

#define FLEXSPMV_DECLARE_GRAPH(G)                                                                   \
  int flexspmv_##G##_info(flexspmv_graph_info *info);                                               \
  int flexspmv_##G##_workspace_bytes(const flexspmv_desc *desc, size_t *bytes);                     \
  int flexspmv_##G##_plan(const flexspmv_desc *desc, const void *d_row_offsets, void *d_workspace,  \
                          size_t workspace_bytes, void *stream);                                    \
  int flexspmv_##G##_plan_windows(const flexspmv_desc *desc, const void *const *indices,            \
                                  void *d_workspace, size_t workspace_bytes, void *stream);         \
  int flexspmv_##G##_launch(const flexspmv_desc *desc, const void *const *values,                   \
                            const void *const *indices, const void *d_row_offsets,                  \
                            void *const *outputs, void *d_workspace, size_t workspace_bytes,        \
                            void *stream);                                                          \
  int flexspmv_##G##_device_status(const void *d_workspace, int32_t *d_status_out, void *stream);

/* graphs built into libflexspmv_b200.so (the benchmark configurations and the unit-test graphs) */
FLEXSPMV_DECLARE_GRAPH(spmv_f32)
FLEXSPMV_DECLARE_GRAPH(spmv_f64)
FLEXSPMV_DECLARE_GRAPH(spmv_i64)
FLEXSPMV_DECLARE_GRAPH(spring_mass_f32)
FLEXSPMV_DECLARE_GRAPH(spring_mass_f64)
FLEXSPMV_DECLARE_GRAPH(rusanov_f64)
FLEXSPMV_DECLARE_GRAPH(rusanov_f32)
FLEXSPMV_DECLARE_GRAPH(swe_delta_f64)
FLEXSPMV_DECLARE_GRAPH(swe_delta_f32)
FLEXSPMV_DECLARE_GRAPH(swe_boundary_f64)
FLEXSPMV_DECLARE_GRAPH(swe_boundary_f32)
FLEXSPMV_DECLARE_GRAPH(swe_components_i64)
FLEXSPMV_DECLARE_GRAPH(swe_init_edges_f64)
FLEXSPMV_DECLARE_GRAPH(swe_init_cells_f64)
FLEXSPMV_DECLARE_GRAPH(swe_init_boundary_f64)
FLEXSPMV_DECLARE_GRAPH(mixed_dims_f32)
FLEXSPMV_DECLARE_GRAPH(mixed_dims_f64)
FLEXSPMV_DECLARE_GRAPH(mixed_dims_i64)
FLEXSPMV_DECLARE_GRAPH(ops_zoo_f32)
FLEXSPMV_DECLARE_GRAPH(ops_zoo_f64)
FLEXSPMV_DECLARE_GRAPH(edge_sum_f32)
FLEXSPMV_DECLARE_GRAPH(edge_sum_f64)
FLEXSPMV_DECLARE_GRAPH(edge_sum_i64)
FLEXSPMV_DECLARE_GRAPH(edge_copy_f32)
FLEXSPMV_DECLARE_GRAPH(edge_copy_f64)
FLEXSPMV_DECLARE_GRAPH(edge_copy_i64)

/*
 * flexspmv_spmv_f64_launch_static -- the fused fp64 SpMV for callers that must not allocate.
 *
 * No counterpart in the reference: its operator allocates temporary storage with cudaMalloc on every
 * call (cuda_template/merged_binding_template.cu:42-49).  Some hosts of this library cannot do that at
 * all -- code running inside a region where the CUDA allocator is off limits (a stream-ordered
 * pipeline whose memory was fixed at start-up, a plug-in that only receives pointers from its host
 * application, a real-time loop that may not take the allocator's locks).  They pass inputs and
 * outputs as usual; the scratch the kernels need (tile coordinates, per-CTA carries, a status block)
 * lives in a device array compiled into the library, FLEXSPMV_STATIC_SCRATCH_BYTES (2 MiB) per GPU
 * that loads the library, held until the process exits.
 *
 *   - Same arguments and results as flexspmv_spmv_f64_plan followed by flexspmv_spmv_f64_launch, minus
 *     the workspace: every call partitions the problem into the static array (two small kernels) and
 *     runs the fused pass, all on `stream`.  It calls no cudaMalloc, cudaFree or allocating library
 *     routine.  FLEXSPMV_FLAG_GATHER_WINDOWS in the descriptor is ignored (the windows need a second
 *     planning step and two more bytes of scratch per edge).
 *   - flexspmv_spmv_f64_static_device_status copies the array's status word (0, FLEXSPMV_ERR_TIMEOUT
 *     or FLEXSPMV_ERR_NOT_PLANNED, as raised by the kernels of the most recent call) into *d_status_out
 *     (int32 in device or page-locked host memory) on `stream`, without synchronising: the error
 *     channel that flexspmv_spmv_f64_device_status gives callers who own a workspace.
 *   - Problems whose scratch need (flexspmv_spmv_f64_workspace_bytes) exceeds the array are refused
 *     with FLEXSPMV_ERR_STATIC_SCRATCH; with the default tile size that is about 160 million rows +
 *     non-zeros with 64-bit offsets, twice that with 32-bit offsets.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array, which still holds the previous call's contents; each
 *     call rewrites what it needs, but two calls whose kernels overlap on the GPU (different streams
 *     without an ordering between them) race on it.  Order such calls, or use the workspace API.
 */
#define FLEXSPMV_STATIC_SCRATCH_BYTES (2u << 20)
int flexspmv_spmv_f64_launch_static(const flexspmv_desc *desc, const void *const *values,
                                    const void *const *indices, const void *d_row_offsets,
                                    void *const *outputs, void *stream);
int flexspmv_spmv_f64_static_device_status(int32_t *d_status_out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* FLEXSPMV_H_ */
