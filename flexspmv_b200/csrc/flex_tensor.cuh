// Per-edge value arithmetic used by the generated map code.
//
// The reference defines the meaning of every map operation through its Tensor<ValueT,Dim> value type
// (data_struct_shared.cuh).  Here the code generator resolves, at generation time, WHICH of that
// type's overloads an expression would pick (equal widths -> member operator, different widths ->
// index-modulo broadcast template, scalar on the left / right) and emits an explicitly named call, so
// this header needs no operator overloading:
//
//   zip(a, b, Op)      tensor (.) tensor, out width max(N, M), operands indexed modulo their width
//                      (data_struct_shared.cuh:611-625); for equal widths this is the member operator
//   zip_vs(a, s, Op)   tensor (.) scalar      (data_struct_shared.cuh:214-253)
//   zip_sv(s, b, Op)   scalar (.) tensor      (data_struct_shared.cuh:386-417)
//   Op = Add, Sub, Mul, Div (IEEE divide), DivGuard (0 where the divisor is 0,
//        data_struct_shared.cuh:194-200,402-408), Pow, Lt, Gt (0/1 in ValueT, :311-329,643-659)
//   where3(c, x, y)    select on c != 0 with modulo broadcast (:425-449)
//   norm(a)            sum of squares accumulated left to right, one sqrt (:346-353)
//
// No fast-math anywhere: + - * / sqrt are single IEEE operations written with the round-to-nearest
// intrinsics, which the compiler neither contracts into fused multiply-adds nor replaces by the
// approximate forms of --use_fast_math, so a map chain evaluates exactly as the reference's CPU code
// does whatever flags the translation unit is built with (only the order of the per-row summation
// differs).  pow and exp are the CUDA math library's and do follow the build flags.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fx {

template <typename V, int D>
struct Vec {
  V v[D];
};

template <typename V, int D>
__device__ __forceinline__ Vec<V, D> splat(V s) {
  Vec<V, D> r;
#pragma unroll
  for (int i = 0; i < D; ++i) r.v[i] = s;
  return r;
}

// ---- math helpers per value type -----------------------------------------------------------------
__device__ __forceinline__ float vpow(float a, float b) { return powf(a, b); }
__device__ __forceinline__ double vpow(double a, double b) { return pow(a, b); }
__device__ __forceinline__ long long vpow(long long a, long long b) { return (long long)pow((double)a, (double)b); }
__device__ __forceinline__ float vexp(float a) { return expf(a); }
__device__ __forceinline__ double vexp(double a) { return exp(a); }
__device__ __forceinline__ long long vexp(long long a) { return (long long)exp((double)a); }
__device__ __forceinline__ float vsqrt(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ double vsqrt(double a) { return __dsqrt_rn(a); }
__device__ __forceinline__ long long vsqrt(long long a) { return (long long)sqrt((double)a); }
__device__ __forceinline__ float vabs(float a) { return fabsf(a); }
__device__ __forceinline__ double vabs(double a) { return fabs(a); }
__device__ __forceinline__ long long vabs(long long a) { return a < 0 ? -a : a; }

__device__ __forceinline__ float vadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double vadd(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ long long vadd(long long a, long long b) { return a + b; }
__device__ __forceinline__ float vsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double vsub(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ long long vsub(long long a, long long b) { return a - b; }
__device__ __forceinline__ float vmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double vmul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ long long vmul(long long a, long long b) { return a * b; }
__device__ __forceinline__ float vdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double vdiv(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ long long vdiv(long long a, long long b) { return a / b; }

struct Add { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return vadd(a, b); } };
struct Sub { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return vsub(a, b); } };
struct Mul { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return vmul(a, b); } };
struct Div { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return vdiv(a, b); } };
struct DivGuard {
  template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return (b != V(0)) ? vdiv(a, b) : V(0); }
};
struct Pow { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return vpow(a, b); } };
// pow(a, 0.5) as one correctly rounded sqrt; the two IEEE special cases where pow and sqrt differ
// (pow(-0, .5) = +0, pow(-inf, .5) = +inf) are kept as pow defines them
struct PowHalf {
  template <typename V> __device__ __forceinline__ V operator()(V a, V) const {
    if (a == V(0)) return V(0);
    if (a < V(0) && vmul(a, V(0.5)) == a) return -a;   // -inf
    return vsqrt(a);
  }
};
struct Lt { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return a < b ? V(1) : V(0); } };
struct Gt { template <typename V> __device__ __forceinline__ V operator()(V a, V b) const { return a > b ? V(1) : V(0); } };

template <typename V, int N, int M, class Op>
__device__ __forceinline__ Vec<V, (N > M ? N : M)> zip(const Vec<V, N>& a, const Vec<V, M>& b, Op op) {
  constexpr int O = (N > M ? N : M);
  Vec<V, O> r;
#pragma unroll
  for (int i = 0; i < O; ++i) r.v[i] = op(a.v[i % N], b.v[i % M]);
  return r;
}
template <typename V, int N, class Op>
__device__ __forceinline__ Vec<V, N> zip_vs(const Vec<V, N>& a, V s, Op op) {
  Vec<V, N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = op(a.v[i], s);
  return r;
}
template <typename V, int N, class Op>
__device__ __forceinline__ Vec<V, N> zip_sv(V s, const Vec<V, N>& b, Op op) {
  Vec<V, N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = op(s, b.v[i]);
  return r;
}

template <typename V, int N>
__device__ __forceinline__ Vec<V, N> neg(const Vec<V, N>& a) {
  Vec<V, N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = -a.v[i];
  return r;
}
template <typename V, int N>
__device__ __forceinline__ Vec<V, N> vec_exp(const Vec<V, N>& a) {
  Vec<V, N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = vexp(a.v[i]);
  return r;
}
template <typename V, int N>
__device__ __forceinline__ Vec<V, N> vec_abs(const Vec<V, N>& a) {
  Vec<V, N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = vabs(a.v[i]);
  return r;
}
template <typename V, int N>
__device__ __forceinline__ Vec<V, N> vec_sign(const Vec<V, N>& a) {
  Vec<V, N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = (a.v[i] > V(0)) ? V(1) : ((a.v[i] < V(0)) ? V(-1) : V(0));
  return r;
}
template <typename V, int N>
__device__ __forceinline__ V norm(const Vec<V, N>& a) {
  V s = V(0);
#pragma unroll
  for (int i = 0; i < N; ++i) s = vadd(s, vmul(a.v[i], a.v[i]));
  return vsqrt(s);
}
template <typename V, int N>
__device__ __forceinline__ Vec<V, 1> item(const Vec<V, N>& a, int i) {
  Vec<V, 1> r;
  r.v[0] = a.v[i];
  return r;
}

// where(c, x, y) with any mix of tensor / scalar for x and y
template <typename V, int C, int X, int Y>
__device__ __forceinline__ Vec<V, (C > X ? (C > Y ? C : Y) : (X > Y ? X : Y))> where3(const Vec<V, C>& c, const Vec<V, X>& x,
                                                                                     const Vec<V, Y>& y) {
  constexpr int O = (C > X ? (C > Y ? C : Y) : (X > Y ? X : Y));
  Vec<V, O> r;
#pragma unroll
  for (int i = 0; i < O; ++i) r.v[i] = (c.v[i % C] != V(0)) ? x.v[i % X] : y.v[i % Y];
  return r;
}
template <typename V, int C, int X>
__device__ __forceinline__ Vec<V, (C > X ? C : X)> where3(const Vec<V, C>& c, const Vec<V, X>& x, V y) {
  constexpr int O = (C > X ? C : X);
  Vec<V, O> r;
#pragma unroll
  for (int i = 0; i < O; ++i) r.v[i] = (c.v[i % C] != V(0)) ? x.v[i % X] : y;
  return r;
}
template <typename V, int C, int Y>
__device__ __forceinline__ Vec<V, (C > Y ? C : Y)> where3(const Vec<V, C>& c, V x, const Vec<V, Y>& y) {
  constexpr int O = (C > Y ? C : Y);
  Vec<V, O> r;
#pragma unroll
  for (int i = 0; i < O; ++i) r.v[i] = (c.v[i % C] != V(0)) ? x : y.v[i % Y];
  return r;
}
template <typename V, int C>
__device__ __forceinline__ Vec<V, C> where3(const Vec<V, C>& c, V x, V y) {
  Vec<V, C> r;
#pragma unroll
  for (int i = 0; i < C; ++i) r.v[i] = (c.v[i] != V(0)) ? x : y;
  return r;
}

// ---- loads / stores --------------------------------------------------------------------------------
// Widest power-of-two chunk (<= 16 bytes) that divides the element group; the C ABI checks that
// gather-source and output base pointers are aligned to it.
template <typename V, int D>
struct VecIO {
  static constexpr int kBytes = int(sizeof(V)) * D;
  static constexpr int kChunk = (kBytes % 16 == 0) ? 16 : (kBytes % 8 == 0) ? 8 : 4;
};

template <typename V, int D>
__device__ __forceinline__ Vec<V, D> ldg_vec(const V* p) {   // read-only global (gather sources)
  Vec<V, D> r;
  constexpr int C = VecIO<V, D>::kChunk;
  if constexpr (C == 16) {
    const int4* q = reinterpret_cast<const int4*>(p);
    int4* o = reinterpret_cast<int4*>(r.v);
#pragma unroll
    for (int i = 0; i < VecIO<V, D>::kBytes / 16; ++i) o[i] = __ldg(q + i);
  } else if constexpr (C == 8) {
    const int2* q = reinterpret_cast<const int2*>(p);
    int2* o = reinterpret_cast<int2*>(r.v);
#pragma unroll
    for (int i = 0; i < VecIO<V, D>::kBytes / 8; ++i) o[i] = __ldg(q + i);
  } else {
    const int* q = reinterpret_cast<const int*>(p);
    int* o = reinterpret_cast<int*>(r.v);
#pragma unroll
    for (int i = 0; i < VecIO<V, D>::kBytes / 4; ++i) o[i] = __ldg(q + i);
  }
  return r;
}

// L1 prefetch of one gathered record (every 32-byte sector it touches)
template <typename V, int D>
__device__ __forceinline__ void prefetch_l1(const V* p) {
  const char* c = reinterpret_cast<const char*>(p);
  constexpr int kBytes = int(sizeof(V)) * D;
  asm volatile("prefetch.global.L1 [%0];" ::"l"(c));
  if constexpr (kBytes > 32) {
#pragma unroll
    for (int o = 32; o < kBytes; o += 32) asm volatile("prefetch.global.L1 [%0];" ::"l"(c + o));
  }
  if constexpr (kBytes > 4 && kBytes <= 32) {   // a record that is not sector-aligned may straddle two sectors
    if ((reinterpret_cast<uintptr_t>(c) & 31) + kBytes > 32) asm volatile("prefetch.global.L1 [%0];" ::"l"(c + kBytes - 1));
  }
}

// L2 prefetch of the byte range [b, e) by one warp (one request per 128-byte line)
__device__ __forceinline__ void prefetch_l2_range(const void* b, const void* e, int lane) {
  const char* q = reinterpret_cast<const char*>(reinterpret_cast<uintptr_t>(b) & ~(uintptr_t)127) + lane * 128;
  for (; q < reinterpret_cast<const char*>(e); q += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(q));
}

template <typename V, int D, class P>
__device__ __forceinline__ Vec<V, D> ld_vec(P p) {   // plain load through anything indexable (shared / global pointer, streaming accessor)
  Vec<V, D> r;
#pragma unroll
  for (int i = 0; i < D; ++i) r.v[i] = p[i];
  return r;
}

template <typename V, int D>
__device__ __forceinline__ void st_vec(V* p, const Vec<V, D>& a) {
  // records of whole 16-byte chunks go out as 16-byte stores when the destination allows it (map-only gather of
  // 16-byte records written in place: 70.7 -> 93.2 % of the HBM peak; 8-byte vector stores of fp32 pairs measured
  // slower than two 4-byte stores, 79.4 against 85.7 %, and are not used)
  if constexpr ((sizeof(V) * D) % 16 == 0) {
    if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
      const int4* src = reinterpret_cast<const int4*>(a.v);
      int4* dst = reinterpret_cast<int4*>(p);
#pragma unroll
      for (int i = 0; i < int(sizeof(V) * D / 16); ++i) dst[i] = src[i];
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < D; ++i) p[i] = a.v[i];
}

template <int OFF, typename V, int D>
__device__ __forceinline__ void accumulate(V* acc, const Vec<V, D>& a) {
#pragma unroll
  for (int i = 0; i < D; ++i) acc[OFF + i] = vadd(acc[OFF + i], a.v[i]);
}
template <int OFF, int D, typename V>
__device__ __forceinline__ void accumulate_scalar(V* acc, V s) {
#pragma unroll
  for (int i = 0; i < D; ++i) acc[OFF + i] = vadd(acc[OFF + i], s);
}

}  // namespace fx
