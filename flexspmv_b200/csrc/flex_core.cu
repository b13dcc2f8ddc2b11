// Library-wide entry points of the C ABI: merge-path partition, nnz-balanced row blocks, CSR
// validation, status strings.  Integer-only kernels; results are bit-identical to the reference's
// search (include/merged_spmv_kernels.cuh:19-99).
#include <cuda_runtime.h>

#include "flex_common.cuh"

namespace flex {

int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// One thread per tile boundary: coordinate of diagonal t * tile_items (clamped to rows + edges).
template <typename OffsetT>
__global__ void partition_kernel(const OffsetT* __restrict__ row_offsets, long long num_rows, long long num_edges,
                                 long long tile_items, long long num_tiles, OffsetT* __restrict__ coords) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t > num_tiles) return;
  long long d = t * tile_items;
  if (d > num_rows + num_edges) d = num_rows + num_edges;
  OffsetT x, y;
  merge_path_search<OffsetT, OffsetT>((OffsetT)d, row_offsets + 1, (OffsetT)0, (OffsetT)num_rows, (OffsetT)num_edges, x, y);
  coords[2 * t] = x;
  coords[2 * t + 1] = y;
}

// One CTA.  A launch of `grid` CTAs gives CTA c the tiles [c q + min(c, r), ...), q = tiles / grid, r = tiles % grid.
// The boundary in front of each such run usually cuts a row in two, which costs the launch a carry hand-over
// between CTAs (fence, ticket, fix-up by the last CTA).  When the part of the cut row in front of the boundary fits
// into the tile behind it -- which has room for as many extra edges as it holds row ends -- the boundary is moved
// back to the row's first edge instead.  All boundaries or none: the header records the grid size it was done for.
template <typename OffsetT>
__global__ void snap_cta_boundaries_kernel(const OffsetT* __restrict__ row_offsets, long long num_rows, long long num_tiles,
                                           int grid, OffsetT* __restrict__ coords, WorkspaceHeader* h) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const long long q = num_tiles / grid, r = num_tiles % grid;
  for (int c = 1 + threadIdx.x; c < grid; c += blockDim.x) {
    const long long t = c * q + (c < r ? c : r);
    const long long x = (long long)coords[2 * t], y = (long long)coords[2 * t + 1];
    if (x >= num_rows) continue;                                    // behind the last row end: nothing is cut
    const long long begin = (long long)row_offsets[x];              // first edge of the row the boundary cuts
    const long long rows_behind = (long long)coords[2 * t + 2] - x; // row ends in the tile behind the boundary
    const long long y_before = (long long)coords[2 * t - 1];        // where the tile in front of it starts
    if (y - begin > rows_behind || begin < y_before) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return;
  for (int c = 1 + threadIdx.x; c < grid; c += blockDim.x) {
    const long long t = c * q + (c < r ? c : r);
    const long long x = (long long)coords[2 * t];
    if (x < num_rows) coords[2 * t + 1] = row_offsets[x];
  }
  if (threadIdx.x == 0) h->snapped_grid = grid;
}

int snap_cta_boundaries_launch(const void* d_row_offsets, int offset_bits, long long num_rows, long long num_tiles, int grid,
                               void* d_coords, void* ws, cudaStream_t stream) {
  if (grid < 2 || num_tiles < grid) return 0;
  if (offset_bits == 32)
    snap_cta_boundaries_kernel<int><<<1, 256, 0, stream>>>(static_cast<const int*>(d_row_offsets), num_rows, num_tiles, grid,
                                                           static_cast<int*>(d_coords), static_cast<WorkspaceHeader*>(ws));
  else
    snap_cta_boundaries_kernel<long long><<<1, 256, 0, stream>>>(static_cast<const long long*>(d_row_offsets), num_rows,
                                                                 num_tiles, grid, static_cast<long long*>(d_coords),
                                                                 static_cast<WorkspaceHeader*>(ws));
  return (int)cudaGetLastError();
}

int partition_launch(const void* d_row_offsets, int offset_bits, long long num_rows, long long num_edges,
                     int tile_items, void* d_coords, cudaStream_t stream) {
  if (!d_row_offsets || !d_coords || tile_items <= 0 || num_rows < 0 || num_edges < 0) return FLEXSPMV_ERR_BAD_ARG;
  if (offset_bits != 32 && offset_bits != 64) return FLEXSPMV_ERR_BAD_ARG;
  if (offset_bits == 32 && num_rows + num_edges >= (1ll << 31)) return FLEXSPMV_ERR_TOO_LARGE;
  const long long tiles = (num_rows + num_edges + tile_items - 1) / tile_items;
  const int block = 128;
  const long long grid = (tiles + 1 + block - 1) / block;
  if (grid > 0x7fffffffLL) return FLEXSPMV_ERR_TOO_LARGE;
  if (offset_bits == 32)
    partition_kernel<int><<<(unsigned)grid, block, 0, stream>>>(static_cast<const int*>(d_row_offsets), num_rows, num_edges,
                                                                tile_items, tiles, static_cast<int*>(d_coords));
  else
    partition_kernel<long long><<<(unsigned)grid, block, 0, stream>>>(static_cast<const long long*>(d_row_offsets), num_rows,
                                                                      num_edges, tile_items, tiles,
                                                                      static_cast<long long*>(d_coords));
  return (int)cudaGetLastError();
}

__global__ void header_init_kernel(WorkspaceHeader* dst, const WorkspaceHeader h) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *dst = h;
}
__global__ void debug_withhold_kernel(WorkspaceHeader* h, uint32_t first_tile_plus_one) {
  if (threadIdx.x == 0 && blockIdx.x == 0) h->debug[7] = first_tile_plus_one;
}
__global__ void window_ready_kernel(WorkspaceHeader* h) {
  if (threadIdx.x == 0 && blockIdx.x == 0) h->win_ready = 1;
}
__global__ void status_mirror_kernel(WorkspaceHeader* h, int32_t* mirror) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    h->status_mirror = reinterpret_cast<uint64_t>(mirror);
    if (mirror) { *reinterpret_cast<volatile int32_t*>(mirror) = h->status; __threadfence_system(); }
  }
}
int window_ready_launch(void* ws, cudaStream_t st) {
  window_ready_kernel<<<1, 32, 0, st>>>(static_cast<WorkspaceHeader*>(ws));
  return (int)cudaGetLastError();
}
int header_init_launch(void* ws, const WorkspaceHeader& h, cudaStream_t stream) {
  header_init_kernel<<<1, 32, 0, stream>>>(static_cast<WorkspaceHeader*>(ws), h);
  return (int)cudaGetLastError();
}

template <typename OffsetT>
__global__ void row_blocks_kernel(const OffsetT* __restrict__ row_offsets, long long num_rows, int parts, long long snap,
                                  long long* __restrict__ first_row) {
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k > parts) return;
  if (k == 0) { first_row[0] = 0; return; }
  if (k == parts) { first_row[parts] = num_rows; return; }
  const long long nnz = (long long)row_offsets[num_rows];
  // k * nnz / parts without overflow: nnz < 2^63 / parts is guaranteed by parts <= 1024 and nnz < 2^52
  const long long target = (long long)(((unsigned __int128)nnz * (unsigned)k) / (unsigned)parts);
  long long lo = 0, hi = num_rows;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if ((long long)row_offsets[mid] < target) lo = mid + 1; else hi = mid;
  }
  if (snap > 1) lo = ((lo + snap / 2) / snap) * snap;
  if (lo > num_rows) lo = num_rows;
  first_row[k] = lo;
}
// rounding can make neighbours cross; enforce monotonicity in one thread (parts is tiny)
__global__ void row_blocks_fix_kernel(long long* first_row, int parts) {
  if (threadIdx.x == 0 && blockIdx.x == 0)
    for (int k = 1; k <= parts; ++k)
      if (first_row[k] < first_row[k - 1]) first_row[k] = first_row[k - 1];
}

template <typename OffsetT>
__global__ void validate_kernel(const OffsetT* __restrict__ row_offsets, long long num_rows, long long num_edges,
                                const int* __restrict__ index, long long num_vertices, int* status) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool bad_csr = false, bad_idx = false;
  if (i == 0) bad_csr = (row_offsets[0] != 0) || ((long long)row_offsets[num_rows] != num_edges);
  for (long long r = i; r < num_rows; r += stride) bad_csr |= row_offsets[r + 1] < row_offsets[r];
  if (index)
    for (long long e = i; e < num_edges; e += stride) bad_idx |= (index[e] < 0) || ((long long)index[e] >= num_vertices);
  if (bad_csr) atomicCAS(status, 0, FLEXSPMV_ERR_BAD_CSR);
  else if (bad_idx) atomicCAS(status, 0, FLEXSPMV_ERR_BAD_ARG);
}

// ---- gather-window plan (see flex_common.cuh) ----------------------------------------------------------
// One CTA per tile (grid-stride).  Columns are bucketed by 16; the distinct buckets go into a small hash
// table (a tile that touches more than kWinMaxBuckets of them keeps its global gathers: random columns
// leave after the first pass), are rank-sorted, and runs of adjacent buckets become segments whose exact
// column bounds come from a second pass over the edges.
constexpr int kWinMaxBuckets = 160;
constexpr int kWinHashSlots = 1024;
template <typename OffsetT>
__global__ void __launch_bounds__(256) window_plan_kernel(const OffsetT* __restrict__ coords, long long num_tiles,
                                                          const int* __restrict__ idx, int rec_bytes, int win_bytes,
                                                          int* __restrict__ table, unsigned short* __restrict__ local_idx) {
  __shared__ int s_hash[kWinHashSlots];
  __shared__ int s_bk[kWinMaxBuckets], s_sorted[kWinMaxBuckets];
  __shared__ int s_cnt, s_nseg;
  __shared__ int s_b0[kWinMaxSegs + 1], s_lo[kWinMaxSegs], s_hi[kWinMaxSegs], s_eoff[kWinMaxSegs];
  const int tid = threadIdx.x;
  for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const long long nz0 = (long long)coords[2 * t + 1], nz1 = (long long)coords[2 * t + 3];
    const int n = (int)(nz1 - nz0);
    for (int i = tid; i < kWinHashSlots; i += blockDim.x) s_hash[i] = -1;
    if (tid == 0) { s_cnt = 0; s_nseg = 0; }
    __syncthreads();
    for (int e = tid; e < n; e += blockDim.x) {
      const int b = idx[nz0 + e] >> 4;
      unsigned h = ((unsigned)b * 2654435761u >> 20) & (kWinHashSlots - 1);
      for (int probe = 0; probe < kWinHashSlots; ++probe) {
        if (s_cnt > kWinMaxBuckets) break;                      // already known not to be windowable
        const int old = atomicCAS(&s_hash[h], -1, b);
        if (old == -1) {
          const int pos = atomicAdd(&s_cnt, 1);
          if (pos < kWinMaxBuckets) s_bk[pos] = b;
          break;
        }
        if (old == b) break;
        h = (h + 1) & (kWinHashSlots - 1);
      }
    }
    __syncthreads();
    const int nb = s_cnt;
    bool ok = nb <= kWinMaxBuckets && n > 0;
    if (ok) {
      for (int i = tid; i < nb; i += blockDim.x) {              // rank sort of the distinct buckets
        const int v = s_bk[i];
        int rank = 0;
        for (int j = 0; j < nb; ++j) rank += s_bk[j] < v;
        s_sorted[rank] = v;
      }
    }
    __syncthreads();
    if (ok && tid == 0) {
      int ns = 0;
      for (int i = 0; i < nb; ++i) {
        if (i == 0 || s_sorted[i] - s_sorted[i - 1] > 2) {      // a gap of more than one empty bucket starts a segment
          if (ns < kWinMaxSegs) { s_b0[ns] = s_sorted[i]; s_lo[ns] = 0x7fffffff; s_hi[ns] = -1; }
          ++ns;
        }
      }
      s_nseg = ns;
    }
    __syncthreads();
    const int ns = s_nseg;
    ok = ok && ns <= kWinMaxSegs;
    if (ok) {
      for (int e = tid; e < n; e += blockDim.x) {
        const int c = idx[nz0 + e], b = c >> 4;
        int k = 0;
        for (int j = 1; j < ns; ++j) k += s_b0[j] <= b;
        atomicMin(&s_lo[k], c);
        atomicMax(&s_hi[k], c);
      }
    }
    __syncthreads();
    if (tid == 0) {
      unsigned off = 0;
      if (ok) {
        for (int k = 0; k < ns; ++k) {
          const int len = s_hi[k] - s_lo[k] + 1;
          s_eoff[k] = (int)((off + win_lead(s_lo[k], rec_bytes)) / (unsigned)rec_bytes);
          off += win_span(s_lo[k], len, rec_bytes);
        }
        ok = off <= (unsigned)win_bytes && off / (unsigned)rec_bytes <= 65535u;
      }
      int* ent = table + t * kWinEntryInts;
      ent[0] = ok ? ns : 0;
      ent[1] = (int)off;
      for (int k = 0; k < kWinMaxSegs; ++k) {
        ent[2 + 2 * k] = (ok && k < ns) ? s_lo[k] : 0;
        ent[3 + 2 * k] = (ok && k < ns) ? s_hi[k] - s_lo[k] + 1 : 0;
      }
      s_nseg = ok ? ns : 0;
    }
    __syncthreads();
    const int ns2 = s_nseg;
    for (int e = tid; e < n; e += blockDim.x) {
      unsigned short pos = 0;
      if (ns2 > 0) {
        const int c = idx[nz0 + e], b = c >> 4;
        int k = 0;
        for (int j = 1; j < ns2; ++j) k += s_b0[j] <= b;
        pos = (unsigned short)(s_eoff[k] + (c - s_lo[k]));
      }
      local_idx[nz0 + e] = pos;
    }
    __syncthreads();
  }
}

int window_plan_launch(const void* d_coords, int offset_bits, long long num_tiles, const int* d_idx, int rec_bytes,
                       int win_bytes, void* d_table, void* d_local_idx, cudaStream_t st) {
  if (num_tiles <= 0) return 0;
  long long grid = num_tiles;
  const long long cap = (long long)device_sm_count() * 8;
  if (grid > cap) grid = cap;
  if (offset_bits == 64)
    window_plan_kernel<long long><<<(unsigned)grid, 256, 0, st>>>(static_cast<const long long*>(d_coords), num_tiles, d_idx,
                                                                  rec_bytes, win_bytes, static_cast<int*>(d_table),
                                                                  static_cast<unsigned short*>(d_local_idx));
  else
    window_plan_kernel<int><<<(unsigned)grid, 256, 0, st>>>(static_cast<const int*>(d_coords), num_tiles, d_idx, rec_bytes,
                                                            win_bytes, static_cast<int*>(d_table),
                                                            static_cast<unsigned short*>(d_local_idx));
  return (int)cudaGetLastError();
}

// Sorted COO row ids -> CSR row offsets with the leading 0: offsets[r] = number of ids < r (a lower bound
// per row), plus the checks the conversion depends on: ids ascending (else BAD_CSR) and inside
// [0, num_rows) (else BAD_ARG).
template <typename IdT, typename OffsetT>
__global__ void coo_rows_to_csr_kernel(const IdT* __restrict__ ids, long long num_edges, long long num_rows,
                                       OffsetT* __restrict__ offsets, int* status) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (long long r = i; r <= num_rows; r += stride) {
    long long lo = 0, hi = num_edges;
    while (lo < hi) {
      const long long mid = (lo + hi) >> 1;
      if ((long long)ids[mid] < r) lo = mid + 1; else hi = mid;
    }
    offsets[r] = (OffsetT)lo;
  }
  bool unsorted = false, out_of_range = false;
  for (long long e = i; e < num_edges; e += stride) {
    const long long v = (long long)ids[e];
    out_of_range |= v < 0 || v >= num_rows;
    if (e + 1 < num_edges) unsorted |= (long long)ids[e + 1] < v;
  }
  if (unsorted) atomicCAS(status, 0, FLEXSPMV_ERR_BAD_CSR);
  else if (out_of_range) atomicCAS(status, 0, FLEXSPMV_ERR_BAD_ARG);
}

// One Runge-Kutta stage of the shallow-water model's per-cell arithmetic, fused: the reducers' sums
// become the stage's increments d = -(r [+ r_boundary]) / area, the running sum of increments is
// extended, and either the next stage's state x + c d or (last stage) the step x += w sum is written.
// Every operation is a separate IEEE operation in the order the model's torch expressions evaluate.
template <typename V>
struct SweStageArgs {
  const V* r[3];        // interior reducer sums (h, uh, vh)
  const V* rb[2];       // boundary reducer sums (uh, vh)
  const V* area;
  V* x[3];              // state (read; written by the last stage)
  V* acc[3];            // running d1 + d2 + ...
  V* stage[3];          // state for the next delta evaluation (not written by the last stage)
  V c, w;
  long long n;
  int first, last;
};
template <typename V>
__global__ void __launch_bounds__(256) swe_stage_kernel(const SweStageArgs<V> a) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += stride) {
    const V area = a.area[i];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      V sum = a.r[k][i];
      if (k > 0) sum = sum + a.rb[k - 1][i];
      const V d = (-sum) / area;
      const V acc = a.first ? d : a.acc[k][i] + d;
      const V x = a.x[k][i];
      if (a.last) {
        a.x[k][i] = x + a.w * acc;
      } else {
        a.acc[k][i] = acc;
        a.stage[k][i] = x + a.c * d;
      }
    }
  }
}
template <typename V>
int swe_stage_launch(const void* const* r, const void* const* rb, const void* area, void* const* x, void* const* acc,
                     void* const* stage, double c, double w, long long n, int first, int last, cudaStream_t st) {
  SweStageArgs<V> a;
  for (int k = 0; k < 3; ++k) {
    a.r[k] = static_cast<const V*>(r[k]);
    a.x[k] = static_cast<V*>(x[k]);
    a.acc[k] = static_cast<V*>(acc[k]);
    a.stage[k] = static_cast<V*>(stage[k]);
    if (!a.r[k] || !a.x[k] || !a.acc[k] || !a.stage[k]) return FLEXSPMV_ERR_BAD_ARG;
  }
  for (int k = 0; k < 2; ++k) {
    a.rb[k] = static_cast<const V*>(rb[k]);
    if (!a.rb[k]) return FLEXSPMV_ERR_BAD_ARG;
  }
  a.area = static_cast<const V*>(area);
  a.c = (V)c; a.w = (V)w; a.n = n; a.first = first; a.last = last;
  if (n == 0) return 0;
  long long grid = (n + 255) / 256;
  if (grid > 148 * 8) grid = 148 * 8;
  swe_stage_kernel<V><<<(unsigned)grid, 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}

// Measurement aid (flexspmv_probe_gather): streams idx / vals with coalesced loads, gathers x[idx] and accumulates.
// Nothing is written unless the sum hits a sentinel, so the kernel measures the rate at which an SM can issue
// gathers; `smem_bytes` of dynamic shared memory (unused) shrink the L1 that is left to the misses in flight.
__global__ void __launch_bounds__(256) probe_gather_kernel(const int* __restrict__ idx, const float* __restrict__ vals,
                                                           const float* __restrict__ x, long long n, float* out) {
  extern __shared__ float probe_dummy[];
  constexpr int U = 4;
  float acc = 0.f;
  const long long chunk = (long long)blockDim.x * U;
  for (long long base = (long long)blockIdx.x * chunk; base < n; base += (long long)gridDim.x * chunk) {
    int id[U];
    float v[U], g[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long e = base + (long long)u * blockDim.x + threadIdx.x;
      id[u] = 0; v[u] = 1.f;
      if (e < n) { id[u] = __ldcs(idx + e); v[u] = __ldcs(vals + e); }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) g[u] = __ldg(x + id[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) acc += v[u] * g[u];
  }
  if (acc == 123.456f) out[blockIdx.x] = acc + probe_dummy[0];
}

}  // namespace flex

extern "C" {

int flexspmv_probe_gather(const int32_t* d_idx, const float* d_vals, const float* d_x, int64_t num_edges, float* d_out,
                          int32_t ctas, int32_t smem_bytes_per_cta, void* stream) {
  if (!d_idx || !d_vals || !d_x || !d_out || num_edges < 0 || ctas < 1 || smem_bytes_per_cta < 0 || smem_bytes_per_cta > 227 * 1024)
    return FLEXSPMV_ERR_BAD_ARG;
  const int smem = smem_bytes_per_cta < 16 ? 16 : smem_bytes_per_cta;
  cudaError_t e = cudaFuncSetAttribute(flex::probe_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
  flex::probe_gather_kernel<<<ctas, 256, smem, static_cast<cudaStream_t>(stream)>>>(d_idx, d_vals, d_x, num_edges, d_out);
  return (int)cudaGetLastError();
}

int flexspmv_abi_version(void) { return FLEXSPMV_ABI_VERSION; }

const char* flexspmv_error_string(int status) {
  switch (status) {
    case FLEXSPMV_OK: return "success";
    case FLEXSPMV_ERR_BAD_ARG: return "bad argument (null pointer, negative size, unsupported offset width or index out of range)";
    case FLEXSPMV_ERR_ALIGN: return "a device pointer is not aligned as required (streamed arrays: 16 bytes)";
    case FLEXSPMV_ERR_WORKSPACE: return "workspace missing or too small";
    case FLEXSPMV_ERR_TOO_LARGE: return "problem size beyond what this entry point supports";
    case FLEXSPMV_ERR_BAD_CSR: return "row offsets are not a valid CSR offset array";
    case FLEXSPMV_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case FLEXSPMV_ERR_NOT_PLANNED: return "workspace was not planned for this problem";
    case FLEXSPMV_ERR_STATIC_SCRATCH:
      return "problem too large for the built-in static scratch array (FLEXSPMV_STATIC_SCRATCH_BYTES); use the workspace API";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown flexspmv status";
}

int flexspmv_partition_bytes(int64_t num_rows, int64_t num_edges, int32_t offset_bits, int32_t tile_items, size_t* bytes) {
  if (!bytes || tile_items <= 0 || num_rows < 0 || num_edges < 0 || (offset_bits != 32 && offset_bits != 64))
    return FLEXSPMV_ERR_BAD_ARG;
  const int64_t tiles = (num_rows + num_edges + tile_items - 1) / tile_items;
  *bytes = (size_t)(tiles + 1) * (offset_bits == 64 ? 16u : 8u);
  return 0;
}

int flexspmv_partition(const void* d_row_offsets, int32_t offset_bits, int64_t num_rows, int64_t num_edges,
                       int32_t tile_items, void* d_coords, void* stream) {
  return flex::partition_launch(d_row_offsets, offset_bits, num_rows, num_edges, tile_items, d_coords,
                                static_cast<cudaStream_t>(stream));
}

int flexspmv_row_blocks(const void* d_row_offsets, int32_t offset_bits, int64_t num_rows, int32_t parts, int64_t snap,
                        int64_t* d_first_row, void* stream) {
  if (!d_row_offsets || !d_first_row || parts < 1 || parts > 1024 || num_rows < 0) return FLEXSPMV_ERR_BAD_ARG;
  if (offset_bits != 32 && offset_bits != 64) return FLEXSPMV_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int block = 128, grid = (parts + 1 + block - 1) / block;
  if (offset_bits == 32)
    flex::row_blocks_kernel<int><<<grid, block, 0, st>>>(static_cast<const int*>(d_row_offsets), num_rows, parts, snap,
                                                         reinterpret_cast<long long*>(d_first_row));
  else
    flex::row_blocks_kernel<long long><<<grid, block, 0, st>>>(static_cast<const long long*>(d_row_offsets), num_rows, parts,
                                                               snap, reinterpret_cast<long long*>(d_first_row));
  flex::row_blocks_fix_kernel<<<1, 32, 0, st>>>(reinterpret_cast<long long*>(d_first_row), parts);
  return (int)cudaGetLastError();
}

int flexspmv_debug_withhold_stage(void* d_workspace, uint32_t first_tile_plus_one, void* stream) {
  if (!d_workspace) return FLEXSPMV_ERR_WORKSPACE;
  flex::debug_withhold_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<flex::WorkspaceHeader*>(d_workspace),
                                                                               first_tile_plus_one);
  return (int)cudaGetLastError();
}

int flexspmv_workspace_status_mirror(void* d_workspace, int32_t* pinned_host_status, void* stream) {
  if (!d_workspace) return FLEXSPMV_ERR_WORKSPACE;
  int32_t* alias = nullptr;
  if (pinned_host_status) {
    void* dptr = nullptr;
    cudaError_t e = cudaHostGetDevicePointer(&dptr, pinned_host_status, 0);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return (int)e; }
    alias = static_cast<int32_t*>(dptr);
  }
  flex::status_mirror_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<flex::WorkspaceHeader*>(d_workspace), alias);
  return (int)cudaGetLastError();
}

int flexspmv_halo_plan(const int64_t* first_row, const int64_t* min_col, const int64_t* max_col, int32_t world,
                       flexspmv_halo_plan_t* plans) {
  if (!first_row || !min_col || !max_col || !plans || world < 1) return FLEXSPMV_ERR_BAD_ARG;
  for (int r = 0; r < world; ++r) {
    if (first_row[r + 1] < first_row[r]) return FLEXSPMV_ERR_BAD_ARG;
    flexspmv_halo_plan_t& p = plans[r];
    p.row_begin = first_row[r]; p.row_end = first_row[r + 1];
    p.halo_lo = p.row_begin > min_col[r] ? p.row_begin - min_col[r] : 0;
    p.halo_hi = max_col[r] + 1 > p.row_end ? max_col[r] + 1 - p.row_end : 0;
    p.send_lo = p.send_hi = 0;
  }
  for (int r = 0; r < world; ++r) {
    if (plans[r].halo_lo) {
      if (r == 0 || plans[r].halo_lo > plans[r - 1].row_end - plans[r - 1].row_begin) return FLEXSPMV_ERR_TOO_LARGE;
      plans[r - 1].send_hi = plans[r].halo_lo;
    }
    if (plans[r].halo_hi) {
      if (r == world - 1 || plans[r].halo_hi > plans[r + 1].row_end - plans[r + 1].row_begin) return FLEXSPMV_ERR_TOO_LARGE;
      plans[r + 1].send_lo = plans[r].halo_hi;
    }
  }
  return 0;
}

int flexspmv_validate_csr(const void* d_row_offsets, int32_t offset_bits, int64_t num_rows, int64_t num_edges,
                          const int32_t* d_index, int64_t num_vertices, int32_t* d_status, void* stream) {
  if (!d_row_offsets || !d_status || num_rows < 0 || num_edges < 0) return FLEXSPMV_ERR_BAD_ARG;
  if (offset_bits != 32 && offset_bits != 64) return FLEXSPMV_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(d_status, 0, sizeof(int32_t), st);
  if (e != cudaSuccess) return (int)e;
  const int block = 256;
  long long work = num_rows > num_edges ? num_rows : num_edges;
  long long grid = (work + block - 1) / block;
  if (grid < 1) grid = 1;
  if (grid > 148 * 8) grid = 148 * 8;
  if (offset_bits == 32)
    flex::validate_kernel<int><<<(unsigned)grid, block, 0, st>>>(static_cast<const int*>(d_row_offsets), num_rows, num_edges,
                                                                 d_index, num_vertices, d_status);
  else
    flex::validate_kernel<long long><<<(unsigned)grid, block, 0, st>>>(static_cast<const long long*>(d_row_offsets), num_rows,
                                                                       num_edges, d_index, num_vertices, d_status);
  return (int)cudaGetLastError();
}

int flexspmv_coo_rows_to_csr(const void* d_row_ids, int32_t id_bits, int64_t num_edges, int64_t num_rows,
                             void* d_row_offsets, int32_t offset_bits, int32_t* d_status, void* stream) {
  if (!d_row_offsets || !d_status || num_edges < 0 || num_rows < 0 || (num_edges > 0 && !d_row_ids)) return FLEXSPMV_ERR_BAD_ARG;
  if ((id_bits != 32 && id_bits != 64) || (offset_bits != 32 && offset_bits != 64)) return FLEXSPMV_ERR_BAD_ARG;
  if (offset_bits == 32 && num_edges > 0x7fffffffLL) return FLEXSPMV_ERR_TOO_LARGE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(d_status, 0, sizeof(int32_t), st);
  if (e != cudaSuccess) return (int)e;
  const int block = 256;
  const long long work = (num_rows + 1) > num_edges ? (num_rows + 1) : num_edges;
  long long grid = (work + block - 1) / block;
  if (grid > 148 * 16) grid = 148 * 16;
  const unsigned g = (unsigned)grid;
  if (id_bits == 32 && offset_bits == 32)
    flex::coo_rows_to_csr_kernel<int, int><<<g, block, 0, st>>>(static_cast<const int*>(d_row_ids), num_edges, num_rows, static_cast<int*>(d_row_offsets), d_status);
  else if (id_bits == 32)
    flex::coo_rows_to_csr_kernel<int, long long><<<g, block, 0, st>>>(static_cast<const int*>(d_row_ids), num_edges, num_rows, static_cast<long long*>(d_row_offsets), d_status);
  else if (offset_bits == 32)
    flex::coo_rows_to_csr_kernel<long long, int><<<g, block, 0, st>>>(static_cast<const long long*>(d_row_ids), num_edges, num_rows, static_cast<int*>(d_row_offsets), d_status);
  else
    flex::coo_rows_to_csr_kernel<long long, long long><<<g, block, 0, st>>>(static_cast<const long long*>(d_row_ids), num_edges, num_rows, static_cast<long long*>(d_row_offsets), d_status);
  return (int)cudaGetLastError();
}

int flexspmv_swe_rk_stage(int32_t value_bytes, const void* const* d_r, const void* const* d_rb, const void* d_area,
                          void* const* d_x, void* const* d_acc, void* const* d_stage, double c, double w, int64_t n,
                          int32_t first, int32_t last, void* stream) {
  if (!d_r || !d_rb || !d_area || !d_x || !d_acc || !d_stage || n < 0) return FLEXSPMV_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (value_bytes == 8) return flex::swe_stage_launch<double>(d_r, d_rb, d_area, d_x, d_acc, d_stage, c, w, n, first, last, st);
  if (value_bytes == 4) return flex::swe_stage_launch<float>(d_r, d_rb, d_area, d_x, d_acc, d_stage, c, w, n, first, last, st);
  return FLEXSPMV_ERR_BAD_ARG;
}

}  // extern "C"
