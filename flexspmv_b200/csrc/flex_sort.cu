// Unsorted reducers: a stable sort of the edges by row id on the device, so that a Reducer whose index is not
// ascending can still be served by the CSR kernels.  The reference converts COO row ids to CSR offsets with
// bincount + cumsum and silently assumes the ids are already sorted
// (python_wrapper/dynamic_replace_submodule.py:20-41); here the permutation that sorts them is computed once,
// the per-edge arrays are permuted with it, and the CSR offsets come from the sorted ids.
//
// Least-significant-digit radix sort, 4 bits per pass, keys = row ids (dense, so ceil(log2(num_rows) / 4)
// passes), values = original edge positions.  Every pass is stable: a block owns a contiguous run of keys,
// every thread a contiguous piece of that run; per-thread digit counts are scanned in (digit, thread) order
// inside the block and in (digit, block) order across blocks, so equal digits keep their input order and the
// final permutation equals a stable argsort (bit-exact against numpy.argsort(kind="stable")).
// Integer-only, bandwidth-bound passes; not on the per-call path of the operator.
#include <cuda_runtime.h>

#include "flex_common.cuh"

namespace flex {

constexpr int kSortThreads = 256;
constexpr int kSortKeysPerThread = 8;
constexpr int kSortTile = kSortThreads * kSortKeysPerThread;
constexpr int kRadixBits = 4;
constexpr int kRadix = 1 << kRadixBits;

__device__ __forceinline__ int digit_of(unsigned key, int shift) { return (int)((key >> shift) & (kRadix - 1)); }

// ids -> 32-bit keys and identity values; flags ids outside [0, num_rows)
template <typename IdT>
__global__ void sort_init_kernel(const IdT* __restrict__ ids, long long n, long long num_rows, unsigned* __restrict__ keys,
                                 int* __restrict__ vals, int* status) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  bool bad = false;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    const long long v = (long long)ids[e];
    bad |= v < 0 || v >= num_rows;
    keys[e] = (unsigned)v;
    vals[e] = (int)e;
  }
  if (bad) atomicCAS(status, 0, FLEXSPMV_ERR_BAD_ARG);
}

// per block: number of keys with each digit -> hist[digit * num_blocks + block]
__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(const unsigned* __restrict__ keys, long long n, int shift,
                                                                 int num_blocks, unsigned* __restrict__ hist) {
  __shared__ unsigned s_cnt[kRadix];
  if (threadIdx.x < kRadix) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const long long base = (long long)blockIdx.x * kSortTile + (long long)threadIdx.x * kSortKeysPerThread;
  unsigned local[kRadix];
#pragma unroll
  for (int d = 0; d < kRadix; ++d) local[d] = 0;
#pragma unroll
  for (int i = 0; i < kSortKeysPerThread; ++i)
    if (base + i < n) {
      const int dg = digit_of(keys[base + i], shift);
#pragma unroll
      for (int d = 0; d < kRadix; ++d) local[d] += (d == dg);
    }
#pragma unroll
  for (int d = 0; d < kRadix; ++d)
    if (local[d]) atomicAdd(&s_cnt[d], local[d]);       // integer counts: order does not matter
  __syncthreads();
  if (threadIdx.x < kRadix) hist[(size_t)threadIdx.x * num_blocks + blockIdx.x] = s_cnt[threadIdx.x];
}

// exclusive scan of the (digit, block) histogram in place, one block (the array has 16 x num_blocks entries)
__global__ void __launch_bounds__(1024) sort_scan_kernel(unsigned* hist, long long total) {
  __shared__ unsigned s_warp[32];
  __shared__ unsigned s_run;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_run = 0;
  __syncthreads();
  for (long long base = 0; base < total; base += 1024) {
    const long long i = base + tid;
    const unsigned v = i < total ? hist[i] : 0u;
    unsigned x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += t;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    if (warp == 0) {
      unsigned w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
      }
      s_warp[lane] = w;
    }
    __syncthreads();
    const unsigned before = s_run + (warp ? s_warp[warp - 1] : 0u) + (x - v);
    if (i < total) hist[i] = before;
    __syncthreads();
    if (tid == 1023) s_run = before + v;
    __syncthreads();
  }
}

// stable scatter of one pass
__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(const unsigned* __restrict__ keys_in, const int* __restrict__ vals_in,
                                                                    long long n, int shift, int num_blocks,
                                                                    const unsigned* __restrict__ hist, unsigned* __restrict__ keys_out,
                                                                    int* __restrict__ vals_out) {
  __shared__ unsigned short s_cnt[kRadix][kSortThreads + 1];
  __shared__ unsigned s_digit_base[kRadix];
  const int tid = threadIdx.x;
  const long long base = (long long)blockIdx.x * kSortTile + (long long)tid * kSortKeysPerThread;
  unsigned k[kSortKeysPerThread];
  int v[kSortKeysPerThread];
  unsigned short local[kRadix];
#pragma unroll
  for (int d = 0; d < kRadix; ++d) local[d] = 0;
#pragma unroll
  for (int i = 0; i < kSortKeysPerThread; ++i) {
    k[i] = 0; v[i] = 0;
    if (base + i < n) {
      k[i] = keys_in[base + i];
      v[i] = vals_in[base + i];
      const int dg = digit_of(k[i], shift);
#pragma unroll
      for (int d = 0; d < kRadix; ++d) local[d] += (d == dg);
    }
  }
#pragma unroll
  for (int d = 0; d < kRadix; ++d) s_cnt[d][tid] = local[d];
  __syncthreads();
  // exclusive scan over threads for each digit: warp w scans digit w and digit w + 8 (8 warps, 16 digits)
  {
    const int lane = tid & 31, warp = tid >> 5;
    for (int d = warp; d < kRadix; d += kSortThreads / 32) {
      unsigned run = 0;
      for (int t0 = 0; t0 < kSortThreads; t0 += 32) {
        const unsigned c = s_cnt[d][t0 + lane];
        unsigned x = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned t = __shfl_up_sync(0xffffffffu, x, o);
          if (lane >= o) x += t;
        }
        s_cnt[d][t0 + lane] = (unsigned short)(run + x - c);
        run += __shfl_sync(0xffffffffu, x, 31);
      }
      if (lane == 0) s_digit_base[d] = hist[(size_t)d * num_blocks + blockIdx.x];
    }
  }
  __syncthreads();
  unsigned next[kRadix];
#pragma unroll
  for (int d = 0; d < kRadix; ++d) next[d] = s_digit_base[d] + s_cnt[d][tid];
#pragma unroll
  for (int i = 0; i < kSortKeysPerThread; ++i)
    if (base + i < n) {
      const int dg = digit_of(k[i], shift);
      unsigned pos = 0;
#pragma unroll
      for (int d = 0; d < kRadix; ++d)
        if (d == dg) pos = next[d]++;
      keys_out[pos] = k[i];
      vals_out[pos] = v[i];
    }
}

// dst[e] = src[perm[e]] for records of `bytes` bytes (4, 8 or a multiple of 4)
__global__ void permute_kernel(const unsigned* __restrict__ src, unsigned* __restrict__ dst, const int* __restrict__ perm,
                               long long n, int words) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n * words; i += stride) {
    const long long e = i / words;
    const int w = (int)(i - e * words);
    dst[i] = src[(long long)perm[e] * words + w];
  }
}

__global__ void copy_u32_kernel(const unsigned* __restrict__ src, unsigned* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[i];
}

static int grid_for(long long work, int block) {
  long long g = (work + block - 1) / block;
  const long long cap = 148ll * 16;
  if (g > cap) g = cap;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace flex

extern "C" {

int flexspmv_sort_rows_bytes(int64_t num_edges, size_t* bytes) {
  if (!bytes || num_edges < 0) return FLEXSPMV_ERR_BAD_ARG;
  if (num_edges > 0x7fffffffLL) return FLEXSPMV_ERR_TOO_LARGE;
  const uint64_t blocks = (uint64_t)(num_edges + flex::kSortTile - 1) / flex::kSortTile;
  // keys (2 buffers), values (1 extra buffer; the other is the caller's permutation array), digit x block histogram
  *bytes = (size_t)(flex::align_up((uint64_t)num_edges * 4u, 256) * 3 + flex::align_up(blocks * flex::kRadix * 4u, 256) + 256);
  return 0;
}

int flexspmv_sort_rows(const void* d_row_ids, int32_t id_bits, int64_t num_edges, int64_t num_rows, int32_t* d_perm,
                       void* d_row_offsets, int32_t offset_bits, void* d_scratch, size_t scratch_bytes, int32_t* d_status,
                       void* stream) {
  if (!d_perm || !d_row_offsets || !d_status || num_edges < 0 || num_rows < 0 || (num_edges > 0 && !d_row_ids))
    return FLEXSPMV_ERR_BAD_ARG;
  if ((id_bits != 32 && id_bits != 64) || (offset_bits != 32 && offset_bits != 64)) return FLEXSPMV_ERR_BAD_ARG;
  if (num_edges > 0x7fffffffLL || num_rows > 0x7fffffffLL) return FLEXSPMV_ERR_TOO_LARGE;
  size_t need = 0;
  if (int e = flexspmv_sort_rows_bytes(num_edges, &need)) return e;
  if (!d_scratch || scratch_bytes < need) return FLEXSPMV_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(d_scratch) & 15u) return FLEXSPMV_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaError_t e = cudaMemsetAsync(d_status, 0, sizeof(int32_t), st); e != cudaSuccess) return (int)e;
  const uint64_t seg = flex::align_up((uint64_t)num_edges * 4u, 256);
  char* base = static_cast<char*>(d_scratch);
  unsigned* keys[2] = {reinterpret_cast<unsigned*>(base), reinterpret_cast<unsigned*>(base + seg)};
  int* vals[2] = {d_perm, reinterpret_cast<int*>(base + 2 * seg)};
  unsigned* hist = reinterpret_cast<unsigned*>(base + 3 * seg);
  const int blocks = (int)((num_edges + flex::kSortTile - 1) / flex::kSortTile);
  int cur = 0;
  if (num_edges > 0) {
    const int g = flex::grid_for(num_edges, 256);
    if (id_bits == 32)
      flex::sort_init_kernel<int><<<g, 256, 0, st>>>(static_cast<const int*>(d_row_ids), num_edges, num_rows, keys[0], vals[0], d_status);
    else
      flex::sort_init_kernel<long long><<<g, 256, 0, st>>>(static_cast<const long long*>(d_row_ids), num_edges, num_rows, keys[0],
                                                           vals[0], d_status);
    int bits = 0;
    while (bits < 31 && (1ll << bits) < num_rows) ++bits;
    for (int shift = 0; shift < bits; shift += flex::kRadixBits) {
      flex::sort_hist_kernel<<<blocks, flex::kSortThreads, 0, st>>>(keys[cur], num_edges, shift, blocks, hist);
      flex::sort_scan_kernel<<<1, 1024, 0, st>>>(hist, (long long)blocks * flex::kRadix);
      flex::sort_scatter_kernel<<<blocks, flex::kSortThreads, 0, st>>>(keys[cur], vals[cur], num_edges, shift, blocks, hist,
                                                                       keys[cur ^ 1], vals[cur ^ 1]);
      cur ^= 1;
    }
    if (cur == 1)     // an odd number of passes left the permutation in the scratch buffer
      flex::copy_u32_kernel<<<g, 256, 0, st>>>(reinterpret_cast<const unsigned*>(vals[1]), reinterpret_cast<unsigned*>(d_perm), num_edges);
  }
  if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return (int)e;
  // CSR offsets from the sorted ids (also re-checks that they ascend); its status word is a scratch int so that an
  // out-of-range id reported above is not overwritten
  int32_t* st2 = reinterpret_cast<int32_t*>(base + 3 * seg + flex::align_up((uint64_t)blocks * flex::kRadix * 4u, 256));
  return flexspmv_coo_rows_to_csr(keys[cur], 32, num_edges, num_rows, d_row_offsets, offset_bits, st2, stream);
}

int flexspmv_permute_edges(const void* d_src, void* d_dst, const int32_t* d_perm, int64_t num_edges, int32_t record_bytes,
                           void* stream) {
  if (num_edges < 0 || record_bytes <= 0 || (record_bytes & 3)) return FLEXSPMV_ERR_BAD_ARG;
  if (num_edges == 0) return 0;
  if (!d_src || !d_dst || !d_perm || d_src == d_dst) return FLEXSPMV_ERR_BAD_ARG;
  const int words = record_bytes / 4;
  flex::permute_kernel<<<flex::grid_for(num_edges * words, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned*>(d_src), static_cast<unsigned*>(d_dst), d_perm, num_edges, words);
  return (int)cudaGetLastError();
}

}  // extern "C"
