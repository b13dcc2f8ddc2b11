// Hand-written sm_100a kernel for reduce-by-row graphs whose gathers have no locality (random columns).
//
// On such matrices every gathered record costs its own L1 miss, and what bounds the kernel is how many
// misses an SM can have in flight: its L1 tag stage accepts one cache line per clock, and every miss
// in flight holds one line of the L1 / shared-memory array.  Measured on B200 (4-byte gathers from a 64 MB
// vector): 235 - 265 G gathers/s per GPU with at most 32 KB of shared memory per SM, 213 - 225 at 64 - 164 KB,
// 177 - 183 at 196 KB, 130 at 224 KB.  So this kernel keeps shared memory small and the miss queue full:
//   * no staging: every warp works alone on merge-path chunks of 32 x IPT items (coordinates planned per
//     chunk), reads its index / value records with coalesced streaming loads straight into registers --
//     one chunk ahead of the chunk whose gathers are in flight -- and gathers from registers;
//   * the only shared memory per item is one product slot and one marker byte (the strided -> blocked
//     transposition): lanes take consecutive edges for loads and gathers; then every lane takes IPT
//     consecutive items, sums them left to right and closes the rows whose last edge is marked inside its
//     span, and a warp-shuffle segmented scan of the lanes' open partial sums supplies what a row received
//     from the lanes before (every lane is busy whatever the row lengths are);
//   * a CTA owns a contiguous range of chunks and hands it to its warps in runs of consecutive chunks, long runs
//     first and short ones at the end (each 1/32 of what is left), so the warps finish together although their
//     speeds differ; inside a run the carry of a row that spans chunks stays in a register.  One carry per run
//     goes to shared memory and the CTA folds them itself; one carry per CTA reaches global memory and the last
//     CTA to finish folds those, in order.
// No barriers between warps while they work, no atomics on the output, run-to-run deterministic (the sequence of
// runs depends on the range only, not on which warp takes which).
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

// Shared memory of one warp: a product slot per item and accumulator component, then 8 marker bytes per lane.
template <class G, class Cfg>
struct WarpSmem {
  static constexpr int kBytes = int(align_up(uint64_t(G::kAccDim) * Cfg::kChunk * sizeof(typename G::V) + 256, 16));
  static constexpr int kMaxRuns = 224;      // runs a CTA hands out to its warps (one carry each, folded by the CTA)
  // dynamic shared memory of a CTA: the warps' areas, then a row and kAccDim partial sums per run
  template <typename OffsetT>
  static constexpr int cta_bytes() {
    return Cfg::kWarps * kBytes + kMaxRuns * int(sizeof(OffsetT) + G::kAccDim * sizeof(typename G::V));
  }
};

constexpr int kMaxWarpCarries = 16384;            // capacity of the per-warp carry arrays in the workspace

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
  long long* carry_row;     // one per CTA (capacity kMaxWarpCarries): the row its range left open
  void* carry_val;          // [..][kAcc] of V: the partial sums of that row
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
  __shared__ unsigned long long s_next;
  constexpr int kMaxRuns = WarpSmem<G, Cfg>::kMaxRuns;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  static_assert(CH <= 255, "row numbers inside a chunk are kept in marker bytes");
  static_assert(IPT <= 8, "a lane's markers are read as one 8-byte word");
  constexpr int kWarpBytes = WarpSmem<G, Cfg>::kBytes;
  unsigned char* wbase = smem_w + (size_t)warp * kWarpBytes;
  V* sp = reinterpret_cast<V*>(wbase);                                   // this warp's product slots, [kAcc][CH]
  // per item: the row (inside the chunk) whose last edge it is, or 0xff; the IPT items of a lane sit in one 8-byte word
  unsigned char* mk = wbase + (size_t)kAcc * CH * sizeof(V);
  const OffsetT* ro = static_cast<const OffsetT*>(a.row_offsets);
  const OffsetT* coords = static_cast<const OffsetT*>(a.coords);

  if (a.header->magic != kMagic || a.header->num_tiles != a.num_chunks || a.header->num_rows != a.num_rows ||
      a.header->num_edges != a.num_edges || a.header->offset_bits != (int)(8 * sizeof(OffsetT))) {
    if (tid == 0 && blockIdx.x == 0) raise_not_planned(a.header);
    return;
  }

  // The CTA owns a contiguous range of chunks.  Its warps take runs of consecutive chunks from it one after the other
  // (s_next: next free chunk of the range in the low half, runs handed out so far in the high half).  A run is
  // 1/kWarps of what is left, at least min_run chunks: long runs first, short ones at the end, so that the warps of
  // the CTA finish together whatever their speeds were.  The sequence of runs depends only on the range, not on
  // which warp takes which, so results stay the same from launch to launch.
  const long long q = a.num_chunks / gridDim.x, rem = a.num_chunks % gridDim.x;
  const long long cta_begin = (long long)blockIdx.x * q + (blockIdx.x < rem ? blockIdx.x : rem);
  const unsigned cta_chunks = (unsigned)(q + (blockIdx.x < rem ? 1 : 0));
  OffsetT* s_run_row = reinterpret_cast<OffsetT*>(smem_w + (size_t)Cfg::kWarps * kWarpBytes);   // [kMaxRuns] row a run left open
  V* s_run_val = reinterpret_cast<V*>(s_run_row + kMaxRuns);                                     // [kMaxRuns][kAcc] its partial sums
  const unsigned min_run = cta_chunks >= 16u * Cfg::kWarps ? 4u : 1u;     // a run pays for one pipeline start
  if (tid == 0) s_next = 0ull;
  __syncthreads();

  StreamTile<G> tile{&p};
  for (;;) {
    unsigned run_pos = 0, run_len = 0, run_id = 0;
    if (lane == 0) {
      unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(&s_next);
      for (;;) {
        const unsigned pos = (unsigned)seen, id = (unsigned)(seen >> 32);
        if (pos >= cta_chunks) break;
        const unsigned left = cta_chunks - pos;
        unsigned len = left / Cfg::kWarps;
        if (len < min_run) len = min_run;
        if (len > left || id == (unsigned)kMaxRuns - 1) len = left;
        const unsigned long long want = ((unsigned long long)(id + 1) << 32) | (pos + len);
        const unsigned long long got = atomicCAS(&s_next, seen, want);
        if (got == seen) { run_pos = pos; run_len = len; run_id = id; break; }
        seen = got;
      }
    }
    run_pos = __shfl_sync(0xffffffffu, run_pos, 0);
    run_len = __shfl_sync(0xffffffffu, run_len, 0);
    run_id = __shfl_sync(0xffffffffu, run_id, 0);
    if (run_len == 0) break;
    const long long c_begin = cta_begin + run_pos;
    const int count = (int)run_len;

    V carry[kAcc];
#pragma unroll
    for (int j = 0; j < kAcc; ++j) carry[j] = V(0);
    long long end_row = a.num_rows;      // row the run's carry belongs to

    // A chunk boundary is a (row, edge) pair; every lane reads the same pair (one broadcast transaction, no shuffles).
    auto load_pair = [&](long long c, OffsetT& x, OffsetT& y) {
      if constexpr (sizeof(OffsetT) == 4) {
        const int2 v = __ldg(reinterpret_cast<const int2*>(coords) + c);
        x = v.x; y = v.y;
      } else {
        const longlong2 v = __ldg(reinterpret_cast<const longlong2*>(coords) + c);
        x = v.x; y = v.y;
      }
    };
    // per-edge records of one chunk into registers (lanes on consecutive edges)
    auto load_edges = [&](OffsetT y0, int ne, typename G::EReg (&er)[IPT]) {
      const long long e0 = (long long)y0 + lane;
#pragma unroll
      for (int i = 0; i < IPT; ++i)
        if (i * 32 + lane < ne) G::load_edge(p, tile, e0 + i * 32, e0 + i * 32, er[i]);
    };

    // boundaries of the current chunk (x0, y0) .. (x1, y1) and the two after it
    OffsetT x0 = 0, y0 = 0, x1 = 0, y1 = 0, x2 = 0, y2 = 0;
    if (count) { load_pair(c_begin, x0, y0); load_pair(c_begin + 1, x1, y1); }
    if (count > 1) load_pair(c_begin + 2, x2, y2);
    typename G::EReg er[IPT];
    if (count) load_edges(y0, (int)(y1 - y0), er);
    // the end of row x0 + lane (the first 32 rows that end inside the chunk), requested one chunk ahead like the records:
    // the row offsets stream from DRAM as the records do
    OffsetT row_end = 0;
    if (count && lane < (int)(x1 - x0)) row_end = ro[(long long)x0 + 1 + lane];

    for (int k = 0; k < count; ++k) {
      const int ne = (int)(y1 - y0), nr = (int)(x1 - x0);

      // gathers of this chunk go out first
      typename G::GEdge ge[IPT];
#pragma unroll
      for (int i = 0; i < IPT; ++i)
        if (i * 32 + lane < ne) G::gather_edge(p, er[i], ge[i]);

      // while they fly: the next chunk's records, the boundary after that, this chunk's row ends
      typename G::EReg er_next[IPT];
      if (k + 1 < count) load_edges(y1, (int)(y2 - y1), er_next);
      OffsetT x3 = 0, y3 = 0;
      if (k + 3 <= count) load_pair(c_begin + k + 3, x3, y3);

      OffsetT row_end_next = 0;
      if (k + 1 < count && lane < (int)(x2 - x1)) row_end_next = ro[(long long)x1 + 1 + lane];

      // end of row x0 + lane relative to the chunk's first edge (rows past the chunk: unused)
      const OffsetT* ro0 = ro + x0 + 1;
      int rel_end = 0;
      if (lane < nr) rel_end = (int)(row_end - y0);
      reinterpret_cast<uint2*>(mk)[lane] = make_uint2(0xffffffffu, 0xffffffffu);
      __syncwarp();

      // rows that end inside the chunk, one lane per row: the last edge of a row is marked with the row's number;
      // a row without edges in this chunk is finished here (row x0 then takes the whole carry)
      const bool seed_used = __any_sync(0xffffffffu, lane == 0 && nr > 0 && rel_end == 0);
      int before = 0;                                      // where the row before this batch's first row ended
      for (int r0 = 0; r0 < nr; r0 += 32) {
        const int r = r0 + lane;
        if (r0) {
          before = __shfl_sync(0xffffffffu, rel_end, 31);
          rel_end = 0;
          if (r < nr) rel_end = (int)(ro0[r] - y0);
        }
        int prev = __shfl_up_sync(0xffffffffu, rel_end, 1);
        if (lane == 0) prev = before;
        if (r < nr) {
          if (rel_end > prev) {
            const int q = rel_end - 1, owner = q / IPT;
            mk[owner * 8 + (q - owner * IPT)] = (unsigned char)r;
          } else {
            static_for<G::kNumReducers>([&](auto R) {
              constexpr int d = G::template red_dim<R.value>();
              constexpr int o = G::template red_off<R.value>();
              V* dst = G::template red_out<R.value>(p) + (size_t)((long long)x0 + r) * d;
#pragma unroll
              for (int j = 0; j < d; ++j) dst[j] = (r == 0) ? carry[o + j] : V(0);
            });
          }
        }
      }
      if (seed_used) {
#pragma unroll
        for (int j = 0; j < kAcc; ++j) carry[j] = V(0);
      }

      // products into this warp's slots (lanes on consecutive edges; slots past the chunk's edges hold zero)
      typename G::GRow gr;
#pragma unroll
      for (int i = 0; i < IPT; ++i) {
        V prod[kAcc];
#pragma unroll
        for (int j = 0; j < kAcc; ++j) prod[j] = V(0);
        if (i * 32 + lane < ne) G::map(p, er[i], (long long)y0 + (i * 32 + lane), gr, ge[i], prod);
#pragma unroll
        for (int j = 0; j < kAcc; ++j) sp[j * CH + i * 32 + lane] = prod[j];
      }
      __syncwarp();

      // blocked pass: every lane sums IPT consecutive items and closes the rows that end inside its span
      V run[kAcc], first[kAcc];
#pragma unroll
      for (int j = 0; j < kAcc; ++j) { run[j] = V(0); first[j] = V(0); }
      int first_row = -1;
      {
        V pv[IPT][kAcc];
        int pm[IPT];
        const uint2 mw = reinterpret_cast<const uint2*>(mk)[lane];
#pragma unroll
        for (int i = 0; i < IPT; ++i) {
          pm[i] = (int)(((i < 4 ? mw.x : mw.y) >> (8 * (i & 3))) & 0xffu);
#pragma unroll
          for (int j = 0; j < kAcc; ++j) pv[i][j] = sp[j * CH + lane * IPT + i];
        }
#pragma unroll
        for (int i = 0; i < IPT; ++i) {
#pragma unroll
          for (int j = 0; j < kAcc; ++j) run[j] += pv[i][j];
          if (pm[i] != 0xff) {
            if (first_row < 0) {                         // may have begun in earlier lanes: finished after the scan
              first_row = pm[i];
#pragma unroll
              for (int j = 0; j < kAcc; ++j) first[j] = run[j];
            } else {
              static_for<G::kNumReducers>([&](auto R) {
                constexpr int d = G::template red_dim<R.value>();
                constexpr int o = G::template red_off<R.value>();
                V* dst = G::template red_out<R.value>(p) + (size_t)((long long)x0 + pm[i]) * d;
#pragma unroll
                for (int j = 0; j < d; ++j) dst[j] = run[o + j];
              });
            }
#pragma unroll
            for (int j = 0; j < kAcc; ++j) run[j] = V(0);
          }
        }
      }
      // segmented inclusive scan of the open partial sums: a lane that closed a row passes on only what follows it.
      // Which lanes closed a row is one ballot; a lane takes a value from `d` lanes down only while that lane is not
      // before the nearest closing lane at or below it (lane 0 when there is none).
      const unsigned closed = __ballot_sync(0xffffffffu, first_row >= 0);
      const unsigned closed_le = closed & (0xffffffffu >> (31 - lane));
      const int reach = lane - (closed_le ? 31 - __clz(closed_le) : 0);      // lanes below this one in its segment
      V scan[kAcc];
#pragma unroll
      for (int j = 0; j < kAcc; ++j) scan[j] = run[j];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
        for (int j = 0; j < kAcc; ++j) {
          const V v_up = shfl_up_any(scan[j], d);
          if (reach >= d) scan[j] = v_up + scan[j];
        }
      }
      // what the lanes before this one left open (plus the warp's carry when none of them closed a row)
      const bool f_ex = (closed_le & ~(1u << lane)) != 0;
      V in[kAcc];
#pragma unroll
      for (int j = 0; j < kAcc; ++j) {
        V v_ex = shfl_up_any(scan[j], 1);
        if (lane == 0) v_ex = V(0);
        in[j] = f_ex ? v_ex : carry[j] + v_ex;
      }
      if (first_row >= 0) {
        static_for<G::kNumReducers>([&](auto R) {
          constexpr int d = G::template red_dim<R.value>();
          constexpr int o = G::template red_off<R.value>();
          V* dst = G::template red_out<R.value>(p) + (size_t)((long long)x0 + first_row) * d;
#pragma unroll
          for (int j = 0; j < d; ++j) dst[j] = in[o + j] + first[o + j];
        });
      }
      // the warp's new carry: what is still open behind the last lane
      {
        const bool f31 = closed != 0;
#pragma unroll
        for (int j = 0; j < kAcc; ++j) {
          const V v31 = __shfl_sync(0xffffffffu, scan[j], 31);
          carry[j] = f31 ? v31 : carry[j] + v31;
        }
      }
      end_row = x1;
      __syncwarp();                                      // the slots are rewritten by the next chunk
#pragma unroll
      for (int i = 0; i < IPT; ++i) er[i] = er_next[i];
      row_end = row_end_next;
      x0 = x1; y0 = y1; x1 = x2; y1 = y2; x2 = x3; y2 = y3;
    }

    // the run's carry: the row it left open and the partial sums of that row
    if (lane == 0) {
      s_run_row[run_id] = (OffsetT)end_row;
#pragma unroll
      for (int j = 0; j < kAcc; ++j) s_run_val[run_id * kAcc + j] = carry[j];
    }
  }  // runs of this warp

  // ---- the CTA folds the carries of its runs; what its last run left open goes to the last CTA -------------------
  __syncthreads();
  {
    const int n_runs = (int)(s_next >> 32);
    const long long tail_row = n_runs ? (long long)s_run_row[n_runs - 1] : a.num_rows;
    for (int c = tid; c < n_runs; c += Cfg::kBlock) {
      const long long row = (long long)s_run_row[c];
      if (c > 0 && (long long)s_run_row[c - 1] == row) continue;     // not the first carry of its row
      V sum[kAcc];
#pragma unroll
      for (int i = 0; i < kAcc; ++i) sum[i] = s_run_val[c * kAcc + i];
      for (int c2 = c + 1; c2 < n_runs && (long long)s_run_row[c2] == row; ++c2) {
#pragma unroll
        for (int i = 0; i < kAcc; ++i) sum[i] += s_run_val[c2 * kAcc + i];
      }
      if (row == tail_row) {
        // still open at the end of the range (or no row at all): another CTA may finish it, so it waits for all of them
        V* cv = static_cast<V*>(a.carry_val) + (size_t)blockIdx.x * kAcc;
#pragma unroll
        for (int i = 0; i < kAcc; ++i) cv[i] = sum[i];
      } else {
        // finished by a later run of this CTA: every store to it is behind the barrier above
        static_for<G::kNumReducers>([&](auto R) {
          constexpr int d = G::template red_dim<R.value>();
          constexpr int o = G::template red_off<R.value>();
          V* dst = G::template red_out<R.value>(p) + (size_t)row * d;
#pragma unroll
          for (int i = 0; i < d; ++i) dst[i] = dst[i] + sum[o + i];
        });
      }
    }
    if (tid == 0) a.carry_row[blockIdx.x] = tail_row;
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
    const int n_carry = (int)gridDim.x;
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
