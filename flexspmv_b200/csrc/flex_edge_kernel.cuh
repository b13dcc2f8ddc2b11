// Hand-written sm_100a kernel for fused graphs WITHOUT a reduce-by-row (the reference's "aggregator"
// flavour: per-edge map outputs, in-place per-edge writes and global `sum` aggregators).  Edges are
// independent, so tiles are plain runs of consecutive edges read with coalesced loads straight from
// global memory; `sum` aggregators are reduced per thread, per warp (shuffles), per CTA (shared
// memory) and finally across CTAs by the last CTA to finish, in CTA order: no atomics on the output,
// no pre-zeroed output, deterministic.
//
// Replaces (reference): the aggregator agent's ConsumeTile + BlockReduce + atomicAdd,
// cuda_template/aggregator/merged_agent_spmv_template.cuh:348-409 and
// codegen/merged_gen_gpu.py:308-332.
#pragma once
#include "flex_common.cuh"
#include "flex_tensor.cuh"

namespace flex {

template <class G>
struct GlobalTile {
  const typename G::Params* p;
  template <int I, class T>
  __device__ __forceinline__ const T* stream(long long e) const {
    return reinterpret_cast<const T*>(G::template stream_ptr<I>(*p) + (size_t)e * G::template stream_bytes<I>());
  }
};

struct EdgeKernelArgs {
  WorkspaceHeader* header;
  void* partials;        // [kMaxCtas][kAggDim] of V
  long long num_edges;
};

template <class G, int BLOCK, int IPT>
__global__ void __launch_bounds__(BLOCK) flex_edge_kernel(const typename G::Params p, const EdgeKernelArgs a) {
  using V = typename G::V;
  constexpr int kAgg = G::kAggDim > 0 ? G::kAggDim : 1;
  constexpr int kWarps = BLOCK / 32;
  __shared__ V s_part[kWarps * kAgg];
  __shared__ int s_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // a workspace that was not planned for this problem holds an arbitrary ticket: every CTA sees the same
  // header, so all of them leave here and nothing is written
  if (a.header->magic != kMagic || a.header->num_edges != a.num_edges || a.header->num_tiles != 0) {
    if (tid == 0 && blockIdx.x == 0) raise_not_planned(a.header);
    return;
  }
  GlobalTile<G> tile{&p};
  V agg[kAgg];
#pragma unroll
  for (int i = 0; i < kAgg; ++i) agg[i] = V(0);

  const long long tile_edges = (long long)BLOCK * IPT;
  for (long long base = (long long)blockIdx.x * tile_edges; base < a.num_edges; base += (long long)gridDim.x * tile_edges) {
    typename G::EReg er[IPT];
    typename G::GEdge g[IPT];
    typename G::GRow gr[IPT];    // a graph without a reducer has no rows: a row-identity selector reads entry e
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      const long long e = base + (long long)i * BLOCK + tid;
      if (e < a.num_edges) { G::load_edge(p, tile, e, e, er[i]); G::gather_row(p, e, gr[i]); G::gather_edge(p, er[i], g[i]); }
    }
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
      const long long e = base + (long long)i * BLOCK + tid;
      if (e < a.num_edges) G::map(p, er[i], e, gr[i], g[i], agg);
    }
  }

  if constexpr (G::kAggDim > 0) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int i = 0; i < kAgg; ++i) agg[i] += __shfl_down_sync(0xffffffffu, agg[i], off);
    }
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < kAgg; ++i) s_part[warp * kAgg + i] = agg[i];
    }
    __syncthreads();
    V* partials = static_cast<V*>(a.partials);
    if (tid < kAgg) {
      V s = V(0);
      for (int w = 0; w < kWarps; ++w) s += s_part[w * kAgg + tid];
      partials[(size_t)blockIdx.x * kAgg + tid] = s;
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned t = atomicAdd(&a.header->ticket, 1u);
      s_flag = (t == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_flag) {
      // the last CTA folds the per-CTA partial sums: every thread takes the CTAs tid, tid + BLOCK, ..., then lanes and
      // warps are combined in a fixed order (the same sum from launch to launch)
      __threadfence();
#pragma unroll
      for (int i = 0; i < kAgg; ++i) {
        V s = V(0);
        for (unsigned c = tid; c < gridDim.x; c += BLOCK) s += __ldcg(partials + (size_t)c * kAgg + i);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
        if (lane == 0) s_part[warp * kAgg + i] = s;
      }
      __syncthreads();
      if (tid < kAgg) {
        V s = V(0);
        for (int w = 0; w < kWarps; ++w) s += s_part[w * kAgg + tid];
        G::store_aggregate(p, tid, s);
      }
      if (tid == 0) a.header->ticket = 0;
    }
  }
}

}  // namespace flex
