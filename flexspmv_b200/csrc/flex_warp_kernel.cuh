// Hand-written sm_100a kernel for reduce-by-row graphs whose gathers have no locality (random columns).
//
// On such matrices every gathered record costs its own L1 miss, and what bounds the kernel is how many
// misses an SM can have in flight: its L1 tag stage accepts one cache line per clock, and every miss
// in flight holds one line of the L1 / shared-memory array.  Measured on B200 (4-byte gathers from a 64 MB
// vector): 265 G gathers/s per GPU with at most 32 KB of shared memory per SM, 225 at 132 KB, 183 at 164 KB,
// 130 at 196 KB, 63 at 228 KB.  So this kernel keeps shared memory small and the miss queue full:
//   * no staging: every warp works alone on merge-path chunks of 32 x IPT items (coordinates planned per
//     chunk), reads its index / value records with coalesced streaming loads straight into registers --
//     one chunk ahead of the chunk whose gathers are in flight -- and gathers from registers;
//   * the only shared memory is one product slot per item (the strided -> row-wise transposition):
//     lanes take consecutive edges for loads and gathers, then one lane per row sums the row's products
//     left to right; rows longer than 32 edges and the chunk's trailing partial row are summed by the
//     whole warp (lanes 32 apart, shuffle tree);
//   * a warp owns a contiguous run of chunks, so the carry of a row that spans chunks stays in a register;
//     one carry per warp reaches global memory and the last CTA to finish folds them, in order.
// No barriers between warps, no atomics on the output, run-to-run deterministic.
//
// Replaces, for those matrices, the same reference code as flex_tile_kernel.cuh (SpmvKernel +
// AgentFlexSpmv::ConsumeTile / reduce<>, include/merged_spmv_kernels.cuh:110-128,
// cuda_template/reducer/merged_agent_spmv_template.cuh:180-445).
#pragma once
#include "flex_common.cuh"
#include "flex_tensor.cuh"
#include "flex_tile_kernel.cuh"

namespace flex {

template <int BLOCK_, int IPT_, int MIN_CTAS_>
struct WarpCfg {
  static constexpr int kBlock = BLOCK_;
  static constexpr int kIpt = IPT_;
  static constexpr int kMinCtas = MIN_CTAS_;
  static constexpr int kWarps = BLOCK_ / 32;
  static constexpr int kChunk = 32 * IPT_;        // merge items per warp chunk ("tile" of the plan)
};

constexpr int kMaxWarpCarries = 16384;            // capacity of the per-warp carry arrays in the workspace
constexpr int kWarpLongRow = 32;                  // rows longer than this are summed by the whole warp

// Streaming accessor for the per-edge arrays: plain global pointers read with evict-first loads, so that the
// lines of the streams do not compete with the gathered records for L1 and L2.
template <typename T>
struct StreamRef {
  const T* ptr;
  __device__ __forceinline__ T operator*() const { return __ldcs(ptr); }
  __device__ __forceinline__ T operator[](int i) const { return __ldcs(ptr + i); }
};
template <class G>
struct StreamTile {
  const typename G::Params* p;
  template <int I, class T>
  __device__ __forceinline__ StreamRef<T> stream(long long e) const {
    return StreamRef<T>{reinterpret_cast<const T*>(G::template stream_ptr<I>(*p) + (size_t)e * G::template stream_bytes<I>())};
  }
};

struct WarpKernelArgs {
  const void* row_offsets;  // leading 0 included
  const void* coords;       // (num_chunks + 1) pairs of OffsetT
  WorkspaceHeader* header;
  long long* carry_row;     // [kMaxWarpCarries]
  void* carry_val;          // [kMaxWarpCarries][kAcc] of V
  long long num_rows;
  long long num_edges;
  long long num_chunks;
};

template <class G, typename OffsetT, class Cfg>
__global__ void __launch_bounds__(Cfg::kBlock, Cfg::kMinCtas)
flex_warp_kernel(const typename G::Params p, const WarpKernelArgs a) {
  using V = typename G::V;
  constexpr int kAcc = G::kAccDim;
  constexpr int IPT = Cfg::kIpt, CH = Cfg::kChunk;
  static_assert(!G::kGatherNeedsRow, "the warp kernel takes graphs whose gathers all depend on the edge");

  extern __shared__ __align__(16) unsigned char smem_w[];
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  V* sp = reinterpret_cast<V*>(smem_w) + (size_t)warp * kAcc * CH;      // this warp's product slots, [kAcc][CH]
  const OffsetT* ro = static_cast<const OffsetT*>(a.row_offsets);
  const OffsetT* coords = static_cast<const OffsetT*>(a.coords);

  if (a.header->magic != kMagic || a.header->num_tiles != a.num_chunks || a.header->num_rows != a.num_rows ||
      a.header->num_edges != a.num_edges || a.header->offset_bits != (int)(8 * sizeof(OffsetT))) {
    if (tid == 0 && blockIdx.x == 0) raise_not_planned(a.header);
    return;
  }

  // contiguous run of chunks of this warp
  const long long n_warps = (long long)gridDim.x * Cfg::kWarps;
  const long long g = (long long)blockIdx.x * Cfg::kWarps + warp;
  const long long q = a.num_chunks / n_warps, rem = a.num_chunks % n_warps;
  const long long c_begin = g * q + (g < rem ? g : rem);
  const int count = (int)(q + (g < rem ? 1 : 0));

  StreamTile<G> tile{&p};
  V carry[kAcc];
#pragma unroll
  for (int j = 0; j < kAcc; ++j) carry[j] = V(0);
  long long end_row = a.num_rows;      // row the final carry belongs to (num_rows: none)

  // chunk coordinates, two chunks ahead: lanes 0..3 hold (row, edge) of the chunk's begin and end
  auto load_coords = [&](long long c) -> long long { return (lane < 4) ? (long long)coords[2 * c + lane] : 0; };
  // per-edge records of one chunk into registers (lanes on consecutive edges)
  auto load_edges = [&](long long y0, int ne, typename G::EReg (&er)[IPT]) {
#pragma unroll
    for (int i = 0; i < IPT; ++i)
      if (i * 32 + lane < ne) G::load_edge(p, tile, y0 + (i * 32 + lane), y0 + (i * 32 + lane), er[i]);
  };

  long long cw = count ? load_coords(c_begin) : 0;
  long long cw_next = count > 1 ? load_coords(c_begin + 1) : 0;
  typename G::EReg er[IPT];
  {
    const long long y0 = __shfl_sync(0xffffffffu, cw, 1), y1 = __shfl_sync(0xffffffffu, cw, 3);
    if (count) load_edges(y0, (int)(y1 - y0), er);
  }

  for (int k = 0; k < count; ++k) {
    const long long x0 = __shfl_sync(0xffffffffu, cw, 0), y0 = __shfl_sync(0xffffffffu, cw, 1);
    const long long x1 = __shfl_sync(0xffffffffu, cw, 2), y1 = __shfl_sync(0xffffffffu, cw, 3);
    const int ne = (int)(y1 - y0), nr = (int)(x1 - x0);

    // gathers of this chunk go out first
    typename G::GEdge ge[IPT];
#pragma unroll
    for (int i = 0; i < IPT; ++i)
      if (i * 32 + lane < ne) G::gather_edge(p, er[i], ge[i]);

    // while they fly: the next chunk's records, the coordinates after that, this chunk's row bounds
    typename G::EReg er_next[IPT];
    cw = cw_next;
    if (k + 1 < count) {
      const long long ny0 = __shfl_sync(0xffffffffu, cw, 1), ny1 = __shfl_sync(0xffffffffu, cw, 3);
      load_edges(ny0, (int)(ny1 - ny0), er_next);
    }
    cw_next = (k + 2 < count) ? load_coords(c_begin + k + 2) : 0;

    // products into this warp's slots
    typename G::GRow gr;
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      if (i * 32 + lane < ne) {
        V prod[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) prod[j] = V(0);
        G::map(p, er[i], y0 + (i * 32 + lane), gr, ge[i], prod);
#pragma unroll
        for (int j = 0; j < kAcc; ++j) sp[j * CH + i * 32 + lane] = prod[j];
      }
    }
    __syncwarp();

    // rows that end inside the chunk: one lane per row; the first one continues the warp's carry
    long long tail_begin = y0;                         // first edge of the trailing partial row
    for (int r0 = 0; r0 < nr; r0 += 32) {
      const int r = r0 + lane;
      const bool have = r < nr;
      long long beg = 0, end = 0;
      if (have) {
        end = (long long)ro[x0 + r + 1];
        beg = r ? (long long)ro[x0 + r] : y0;          // row x0 may have begun in an earlier chunk
        if (beg < y0) beg = y0;
      }
      const int lo = (int)(beg - y0), len = (int)(end - beg);
      V sum[kAcc];
#pragma unroll
      for (int j = 0; j < kAcc; ++j) sum[j] = V(0);
      const bool is_long = have && len > kWarpLongRow;
      if (have && !is_long) {
        const V* qv = sp + lo;
        for (int n = 0; n < len; ++n) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) sum[j] += qv[j * CH + n];
        }
      }
      unsigned longs = __ballot_sync(0xffffffffu, is_long);
      while (longs) {                                  // long rows: lanes 32 apart, shuffle tree, result to the row's lane
        const int src = __ffs(longs) - 1;
        longs &= longs - 1;
        const int llo = __shfl_sync(0xffffffffu, lo, src), llen = __shfl_sync(0xffffffffu, len, src);
        V part[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) part[j] = V(0);
        for (int n = lane; n < llen; n += 32) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) part[j] += sp[j * CH + llo + n];
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) part[j] += shfl_down_any(part[j], off);
        }
#pragma unroll
        for (int j = 0; j < kAcc; ++j) {
          const V tot = __shfl_sync(0xffffffffu, part[j], 0);
          if (lane == src) sum[j] = tot;
        }
      }
      if (have) {
        if (r == 0) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) sum[j] = carry[j] + sum[j];
        }
        static_for<G::kNumReducers>([&](auto R) {
          constexpr int d = G::template red_dim<R.value>();
          constexpr int o = G::template red_off<R.value>();
          V* dst = G::template red_out<R.value>(p) + (size_t)(x0 + r) * d;
#pragma unroll
          for (int j = 0; j < d; ++j) dst[j] = sum[o + j];
        });
      }
      if (r0 + 32 >= nr) {                             // the last row's end is where the trailing partial row begins
        const long long last_end = __shfl_sync(0xffffffffu, end, (nr - 1) & 31);
        tail_begin = last_end > y0 ? last_end : y0;
      }
    }

    // trailing partial row (all of the chunk when no row ends in it): whole warp, then into the carry
    {
      const int tlo = (int)(tail_begin - y0);
      V part[kAcc];
#pragma unroll
      for (int j = 0; j < kAcc; ++j) part[j] = V(0);
      for (int n = tlo + lane; n < ne; n += 32) {
#pragma unroll
        for (int j = 0; j < kAcc; ++j) part[j] += sp[j * CH + n];
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int j = 0; j < kAcc; ++j) part[j] += shfl_down_any(part[j], off);
      }
#pragma unroll
      for (int j = 0; j < kAcc; ++j) {
        const V tot = __shfl_sync(0xffffffffu, part[j], 0);
        carry[j] = (nr > 0) ? tot : carry[j] + tot;
      }
    }
    end_row = x1;
    __syncwarp();                                      // the slots are rewritten by the next chunk
#pragma unroll
    for (int i = 0; i < IPT; ++i) er[i] = er_next[i];
  }

  // ---- hand the warp's carry to the last CTA -----------------------------------------------------------
  if (lane == 0) {
    V* cv = static_cast<V*>(a.carry_val) + (size_t)g * kAcc;
#pragma unroll
    for (int j = 0; j < kAcc; ++j) cv[j] = carry[j];
    a.carry_row[g] = count ? end_row : a.num_rows;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned t = atomicAdd(&a.header->ticket, 1u);
    s_last = (t == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    const int n_carry = (int)n_warps;
    const V* cvals = static_cast<const V*>(a.carry_val);
    for (int c = tid; c < n_carry; c += Cfg::kBlock) {
      const long long row = __ldcg(a.carry_row + c);
      if (row >= a.num_rows) continue;
      if (c > 0 && __ldcg(a.carry_row + c - 1) == row) continue;   // not the head of its run
      V sum[kAcc];
#pragma unroll
      for (int i = 0; i < kAcc; ++i) sum[i] = __ldcg(cvals + (size_t)c * kAcc + i);
      for (int c2 = c + 1; c2 < n_carry && __ldcg(a.carry_row + c2) == row; ++c2) {
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
