// Shared device/host definitions: workspace layout, merge-path search, sm_100a PTX wrappers
// (mbarrier + 1-D bulk async copy), bounded waits.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "flexspmv.h"   // the public C header (include/ of the project; the build passes -I for it)

namespace flex {

// ---- compile-time loop ---------------------------------------------------------------------------
template <int I>
struct IntC {
  static constexpr int value = I;
};
template <int N, int I = 0, class F>
__host__ __device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(IntC<I>{});
    static_for<N, I + 1>(static_cast<F&&>(f));
  }
}

// ---- workspace -----------------------------------------------------------------------------------
// [ WorkspaceHeader (256 B) | tile coordinates (tiles+1 pairs) | per-CTA carry rows (int64) |
//   per-CTA carry / partial values (max_ctas x acc_dim x 8 B) ]
struct WorkspaceHeader {
  uint32_t magic;          // kMagic once planned
  uint32_t ticket;         // CTAs finished in the current launch; the last one resets it to 0
  int32_t status;          // 0 or FLEXSPMV_ERR_* raised by a kernel (sticky until re-planned)
  int32_t offset_bits;
  int64_t num_rows;
  int64_t num_edges;
  int64_t num_tiles;
  int32_t tile_items;
  int32_t max_ctas;
  uint64_t coords_offset;  // byte offsets from the workspace base
  uint64_t carry_row_offset;
  uint64_t carry_val_offset;
  uint64_t total_bytes;
  uint32_t debug[8];       // where a bounded wait gave up: {tile, stage, ...}
  uint64_t win_table_offset;   // gather windows (0: not planned): per-tile segment table ...
  uint64_t win_index_offset;   // ... and per-edge 16-bit positions inside the tile's window area
  int32_t win_ready;           // 1 once the window plan has filled them
  int32_t snapped_grid;        // > 0: the tile boundaries in front of the CTAs of a grid of this size sit on row
                               // ends (no row spans two CTAs of such a launch: no carries to hand over)
  uint64_t status_mirror;      // device alias of a pinned host int32 that receives a copy of `status` when a
                               // kernel raises an error (0: none); lets the host notice without a sync or a copy
  char pad[256 - 4 * 4 - 3 * 8 - 2 * 4 - 4 * 8 - 8 * 4 - 2 * 8 - 2 * 4 - 8];
};
static_assert(sizeof(WorkspaceHeader) == 256, "header is one 256-byte block");
constexpr uint32_t kMagic = 0x464c5831u;  // "FLX1"

// Raises `err` in the workspace header (first error wins, sticky until the workspace is planned again) and
// copies it to the host-visible mirror when one is registered.
__device__ __forceinline__ void raise_status(WorkspaceHeader* h, int err) {
  if (atomicCAS(&h->status, 0, err) == 0) {
    volatile int32_t* m = reinterpret_cast<volatile int32_t*>(h->status_mirror);
    if (m) { *m = err; __threadfence_system(); }
  }
}

// A launch found a header that does not describe its problem.  A header that was planned for another problem
// is otherwise intact; one that was never planned holds arbitrary bytes, so only the status word is written.
__device__ __forceinline__ void raise_not_planned(WorkspaceHeader* h) {
  if (h->magic == kMagic) raise_status(h, FLEXSPMV_ERR_NOT_PLANNED);
  else h->status = FLEXSPMV_ERR_NOT_PLANNED;
}

// ---- gather windows ---------------------------------------------------------------------------------
// On matrices whose tiles touch only a few contiguous column ranges (stencils, banded meshes) the plan can
// record, per tile, up to kWinMaxSegs column segments that cover every column of the tile and, per edge, the
// 16-bit position of its column inside the concatenation of those segments.  The tile kernel then stages the
// segments of the gathered vector into shared memory with bulk copies (like every other stream) and gathers
// from there, and it streams the 2-byte positions instead of the 4-byte column indices.
// Table entry of one tile: ints [0] = number of segments (0: the tile keeps its global gathers),
// [2 + 2j] = first column, [3 + 2j] = length of segment j.  In the window area segment j starts at the next
// 16-byte boundary after segment j-1 plus `lead_j = (first_j * record_bytes) & 15` (its source is 16-byte
// aligned that way when the gathered array is), so the layout is a function of the table entry alone.
constexpr int kWinMaxSegs = 12;
constexpr int kWinEntryInts = 28;          // 112 bytes per tile
__host__ __device__ __forceinline__ uint32_t win_lead(int first, int rec_bytes) { return ((uint32_t)first * (uint32_t)rec_bytes) & 15u; }
__host__ __device__ __forceinline__ uint32_t win_span(int first, int len, int rec_bytes) {
  return (win_lead(first, rec_bytes) + (uint32_t)len * (uint32_t)rec_bytes + 15u) & ~15u;
}

__host__ __device__ constexpr uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

// ---- merge-path search ---------------------------------------------------------------------------
// Coordinate (x = rows consumed, y = edges consumed) at which `diagonal` crosses the merge path of
// a[0..a_len) (row END offsets, relative to `b_base`) and the counting sequence b_base + 0..b_len-1.
// Same arithmetic as the reference search (include/merged_spmv_kernels.cuh:19-50): the largest x
// with a[x-1] <= b[diagonal - x], found by bisection; results must be bit-identical to it.
template <typename OffsetT, typename AT>
__host__ __device__ __forceinline__ void merge_path_search(OffsetT diagonal, const AT* a, OffsetT b_base,
                                                           OffsetT a_len, OffsetT b_len, OffsetT& x, OffsetT& y) {
  OffsetT lo = diagonal - b_len > 0 ? diagonal - b_len : 0;
  OffsetT hi = diagonal < a_len ? diagonal : a_len;
  while (lo < hi) {
    OffsetT mid = (lo + hi) >> 1;
    if ((OffsetT)a[mid] <= b_base + (diagonal - mid - 1)) lo = mid + 1;
    else hi = mid;
  }
  x = lo < a_len ? lo : a_len;
  y = diagonal - lo;
}

// ---- PTX wrappers (sm_90+/sm_100a) ---------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Named barriers over a subset of the CTA's threads (count must be a multiple of 32).
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ bool named_bar_and(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(id), "r"(count)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ bool named_bar_or(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "r"(id), "r"(count)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: polls until the phase completes or ~`limit_ns` of wall time (%globaltimer) have
// passed.  Returns false when the phase never completed (the caller raises ERR_TIMEOUT and leaves).
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 0 && global_timer_ns() - t0 > limit_ns) return false;
  }
}
// 1-D bulk async copy global -> this CTA's shared memory, completion counted on an mbarrier.
// dst, src 16-byte aligned, bytes a positive multiple of 16.  No multicast qualifier.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  // The staged arrays are read once per launch: evict_first in L2 leaves the cache to the gathered
  // records (measured on B200: +11% on a random-column matrix whose x is half the L2, neutral on stencils;
  // marking the gathers evict_last on top of it was slower).
  uint64_t pol;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
               : "memory");
}
// Programmatic dependent launch: a kernel launched with the programmatic-stream-serialization attribute may
// start while the kernel before it on the stream is still running; everything it does before pdl_wait() must
// touch no global memory.  pdl_wait() returns once that kernel has completed and its writes are visible (at
// once when the launch carried no such attribute); pdl_launch_dependents() lets the next such launch start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Orders earlier generic-proxy shared-memory accesses before later async-proxy (bulk copy) ones.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ T shfl_up_any(T v, int delta) {
  return __shfl_up_sync(0xffffffffu, v, delta);
}
template <typename T>
__device__ __forceinline__ T shfl_down_any(T v, int delta) {
  return __shfl_down_sync(0xffffffffu, v, delta);
}

}  // namespace flex
