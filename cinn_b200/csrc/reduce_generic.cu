// Reductions for the element types the fp32 kernels of reduce_kernels.cu do not cover: float16 / bfloat16
// (accumulated in fp32, rounded once at the end), float64, int32 / int64 (wrapping, as C) and bool
// (reduce_all / reduce_any).  Same semantics as cinn/hlir/pe/reduction.cc:139-227: the accumulator starts at the
// op's initial value of cinn/lang/builtin.cc:123-143 (0, 1, the type's lowest / largest finite value, true,
// false), max / min are compare + select.  The reference accumulates 16-bit floats in their own type, serially;
// a tree in fp32 is closer to the exact result and stays inside the 1e-2 tolerance of those types.
//
// Two layouts, as in reduce_kernels.cu: rows (inner == 1: a warp or a CTA per row) and columns (inner > 1: a
// thread per 16 bytes of columns, eight row loads in flight).  16-byte loads when the buffers allow it.
#include <cstdint>
#include <type_traits>

#include "device_math.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

// ---- element types: storage T, accumulator type, conversion ------------------------------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<__half> {
  using Acc = float;
  __device__ static Acc load(__half v) { return __half2float(v); }
  __device__ static __half store(Acc v) { return __float2half_rn(v); }
  __device__ static Acc lowest() { return -65504.0f; }
  __device__ static Acc largest() { return 65504.0f; }
};
template <>
struct Elem<__nv_bfloat16> {
  using Acc = float;
  __device__ static Acc load(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 store(Acc v) { return __float2bfloat16_rn(v); }
  __device__ static Acc lowest() { return -__uint_as_float(0x7f7f0000u); }
  __device__ static Acc largest() { return __uint_as_float(0x7f7f0000u); }
};
template <>
struct Elem<float> {  // second pass of the reductions that leave float32 partials (chain_reduce.cu)
  using Acc = float;
  __device__ static Acc load(float v) { return v; }
  __device__ static float store(Acc v) { return v; }
  __device__ static Acc lowest() { return -3.402823466e38f; }
  __device__ static Acc largest() { return 3.402823466e38f; }
};
template <>
struct Elem<double> {
  using Acc = double;
  __device__ static Acc load(double v) { return v; }
  __device__ static double store(Acc v) { return v; }
  __device__ static Acc lowest() { return -1.7976931348623157e308; }
  __device__ static Acc largest() { return 1.7976931348623157e308; }
};
template <>
struct Elem<int32_t> {
  using Acc = int32_t;
  __device__ static Acc load(int32_t v) { return v; }
  __device__ static int32_t store(Acc v) { return v; }
  __device__ static Acc lowest() { return (int32_t)0x80000000; }
  __device__ static Acc largest() { return 0x7fffffff; }
};
template <>
struct Elem<long long> {
  using Acc = long long;
  __device__ static Acc load(long long v) { return v; }
  __device__ static long long store(Acc v) { return v; }
  __device__ static Acc lowest() { return (long long)0x8000000000000000ull; }
  __device__ static Acc largest() { return 0x7fffffffffffffffll; }
};
template <>
struct Elem<uint8_t> {  // bool
  using Acc = int32_t;
  __device__ static Acc load(uint8_t v) { return v != 0; }
  __device__ static uint8_t store(Acc v) { return v != 0; }
  __device__ static Acc lowest() { return 0; }
  __device__ static Acc largest() { return 1; }
};

// ---- ops ----------------------------------------------------------------------------------------------------------
struct GSum {
  template <typename T> __device__ static typename Elem<T>::Acc identity() { return 0; }
  // unsigned arithmetic for integers: wrapping without undefined behaviour
  __device__ static float apply(float a, float b) { return a + b; }
  __device__ static double apply(double a, double b) { return a + b; }
  __device__ static int32_t apply(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
  __device__ static long long apply(long long a, long long b) { return (long long)((unsigned long long)a + (unsigned long long)b); }
};
struct GProd {
  template <typename T> __device__ static typename Elem<T>::Acc identity() { return 1; }
  __device__ static float apply(float a, float b) { return a * b; }
  __device__ static double apply(double a, double b) { return a * b; }
  __device__ static int32_t apply(int32_t a, int32_t b) { return (int32_t)((uint32_t)a * (uint32_t)b); }
  __device__ static long long apply(long long a, long long b) { return (long long)((unsigned long long)a * (unsigned long long)b); }
};
struct GMax {
  template <typename T> __device__ static typename Elem<T>::Acc identity() { return Elem<T>::lowest(); }
  template <typename A> __device__ static A apply(A a, A b) { return a > b ? a : b; }
};
struct GMin {
  template <typename T> __device__ static typename Elem<T>::Acc identity() { return Elem<T>::largest(); }
  template <typename A> __device__ static A apply(A a, A b) { return a < b ? a : b; }
};
struct GAll {
  template <typename T> __device__ static typename Elem<T>::Acc identity() { return 1; }
  __device__ static int32_t apply(int32_t a, int32_t b) { return a && b; }
};
struct GAny {
  template <typename T> __device__ static typename Elem<T>::Acc identity() { return 0; }
  __device__ static int32_t apply(int32_t a, int32_t b) { return a || b; }
};

// acc (+)= v for one stored element.  A sum of 16-bit floats uses the mixed-precision add of sm_100 (add.f32.f16 /
// add.f32.bf16: the operand is widened inside the instruction), one instruction instead of a conversion on the
// XU pipe plus an add; the result is the same bit for bit (the widening is exact, the add rounds once).
template <typename T, class Op>
__device__ __forceinline__ typename Elem<T>::Acc fold_elem(typename Elem<T>::Acc acc, T v) {
  if constexpr (std::is_same<Op, GSum>::value && std::is_same<T, __half>::value) {
    asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(acc) : "h"(__half_as_ushort(v)));
    return acc;
  } else if constexpr (std::is_same<Op, GSum>::value && std::is_same<T, __nv_bfloat16>::value) {
    asm("add.rn.f32.bf16 %0, %1, %0;" : "+f"(acc) : "h"(__bfloat16_as_ushort(v)));
    return acc;
  } else {
    return Op::apply(acc, Elem<T>::load(v));
  }
}

template <typename T, class Op>
__device__ __forceinline__ void fold16(const uint4& u, typename Elem<T>::Acc& acc) {
  constexpr int V = 16 / sizeof(T);
  if constexpr (std::is_same<T, uint8_t>::value && (std::is_same<Op, GAll>::value || std::is_same<Op, GAny>::value)) {
    // sixteen bools at once: "any" is a non-zero word; "all" is a word without a zero byte
    // ((w - 0x01010101) & ~w & 0x80808080 is non-zero exactly when some byte of w is zero)
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if constexpr (std::is_same<Op, GAny>::value) acc = acc | (w[q] != 0u ? 1 : 0);
      else acc = acc & ((((w[q] - 0x01010101u) & ~w[q] & 0x80808080u) == 0u) ? 1 : 0);
    }
    return;
  }
  const T* e      = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < V; ++i) acc = fold_elem<T, Op>(acc, e[i]);
}

template <typename A, class Op>
__device__ __forceinline__ A warp_fold(A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- rows: y[row] = fold over x[row, 0..r) -------------------------------------------------------------------------
// `group` = 32: a warp per row (8 rows per CTA of 256); `group` = 256: a CTA per row.
template <typename T, class Op>
__global__ void __launch_bounds__(256)
    k_reduce_generic_row(const T* __restrict__ x, T* __restrict__ y, long long rows, long long r, long long group,
                         long long vec_ok) {
  using A         = typename Elem<T>::Acc;
  constexpr int V = 16 / sizeof(T);
  __shared__ A part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool per_warp   = group == 32;
  const long long first = per_warp ? (long long)blockIdx.x * 8 + warp : blockIdx.x;
  const long long step  = per_warp ? (long long)gridDim.x * 8 : gridDim.x;
  const int t = per_warp ? lane : (int)threadIdx.x, nt = per_warp ? 32 : 256;
  for (long long row = first; row < rows; row += step) {  // uniform per CTA in the CTA-per-row form
    const T* px = x + row * r;
    A acc       = Op::template identity<T>();
    long long done = 0;
    if (vec_ok) {  // r % V == 0 and 16-byte aligned base: every row starts on a 16-byte boundary
      const uint4* pv    = reinterpret_cast<const uint4*>(px);
      const long long nv = r / V;
      long long v        = t;
      for (; v + 3 * nt < nv; v += 4 * nt) {
        uint4 u[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) u[q] = __ldcs(pv + v + q * nt);
#pragma unroll
        for (int q = 0; q < 4; ++q) fold16<T, Op>(u[q], acc);
      }
      for (; v < nv; v += nt) fold16<T, Op>(__ldcs(pv + v), acc);
      done = nv * V;
    }
    for (long long i = done + t; i < r; i += nt) acc = fold_elem<T, Op>(acc, px[i]);
    acc = warp_fold<A, Op>(acc);
    if (per_warp) {
      if (lane == 0) y[row] = Elem<T>::store(acc);
    } else {
      if (lane == 0) part[warp] = acc;
      __syncthreads();
      if (threadIdx.x == 0) {
        A total = part[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) total = Op::apply(total, part[w]);
        y[row] = Elem<T>::store(total);
      }
      __syncthreads();
    }
  }
}

// ---- columns: y[o, c] = fold over x[o, 0..r, c] --------------------------------------------------------------------
template <typename T, class Op>
__global__ void __launch_bounds__(256)
    k_reduce_generic_col(const T* __restrict__ x, T* __restrict__ y, long long outer, long long r_total,
                         long long inner, long long rows_per_split, long long vec_ok) {
  using A         = typename Elem<T>::Acc;
  constexpr int V = 16 / sizeof(T);
  // blockIdx.z = split of the reduced axis: rows [k0, k0 + r) go to partial result z (y holds [splits][outer][inner])
  const long long k0 = (long long)blockIdx.z * rows_per_split;
  const long long r  = min(rows_per_split, r_total - k0);
  for (long long o = blockIdx.y; o < outer; o += gridDim.y) {
    const T* px = x + (o * r_total + k0) * inner;
    T* py       = y + ((long long)blockIdx.z * outer + o) * inner;
    if (vec_ok) {  // inner % V == 0, 16-byte aligned bases
      const long long nv = inner / V;
      const long long c  = (long long)blockIdx.x * blockDim.x + threadIdx.x;
      if (c < nv) {
        A acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = Op::template identity<T>();
        const uint4* pv = reinterpret_cast<const uint4*>(px) + c;
        long long k     = 0;
        for (; k + 8 <= r; k += 8) {
          uint4 u[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) u[q] = __ldcs(pv + (k + q) * nv);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const T* e = reinterpret_cast<const T*>(&u[q]);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = fold_elem<T, Op>(acc[i], e[i]);
          }
        }
        for (; k < r; ++k) {
          const uint4 u = __ldcs(pv + k * nv);
          const T* e    = reinterpret_cast<const T*>(&u);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] = fold_elem<T, Op>(acc[i], e[i]);
        }
        uint4 out;
        T* e = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int i = 0; i < V; ++i) e[i] = Elem<T>::store(acc[i]);
        reinterpret_cast<uint4*>(py)[c] = out;
      }
    } else {
      for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < inner; c += (long long)gridDim.x * blockDim.x) {
        A a0 = Op::template identity<T>(), a1 = a0, a2 = a0, a3 = a0;
        long long k = 0;
        for (; k + 4 <= r; k += 4) {
          a0 = fold_elem<T, Op>(a0, px[(k + 0) * inner + c]);
          a1 = fold_elem<T, Op>(a1, px[(k + 1) * inner + c]);
          a2 = fold_elem<T, Op>(a2, px[(k + 2) * inner + c]);
          a3 = fold_elem<T, Op>(a3, px[(k + 3) * inner + c]);
        }
        for (; k < r; ++k) a0 = fold_elem<T, Op>(a0, px[k * inner + c]);
        py[c] = Elem<T>::store(Op::apply(Op::apply(a0, a1), Op::apply(a2, a3)));
      }
    }
  }
}

// ---- fold of few columns: y[c] = fold over x[0..r, c] with the rows spread over the warps of a CTA ----------------------
// The second step of a split column reduction has r = number of splits (tens to hundreds) and only inner / V column
// groups: with a thread per column group it would run on a handful of CTAs, each walking all the rows eight at a
// time.  Here a CTA takes 32 column groups (a warp reads 512 contiguous bytes of a row) and its 8 warps take the
// rows k = warp, warp + 8, ... (up to four loads in flight each); the warps' accumulators meet in shared memory and
// warp 0 folds them in warp order.  Needs inner % V == 0 (the planner checks) and a 16-byte aligned x.
template <typename T, class Op>
__global__ void __launch_bounds__(256)
    k_reduce_generic_col_fold(const T* __restrict__ x, T* __restrict__ y, long long r, long long inner) {
  using A         = typename Elem<T>::Acc;
  constexpr int V = 16 / sizeof(T);
  __shared__ A part[8][32][V + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long nv = inner / V;
  const long long c  = (long long)blockIdx.x * 32 + lane;
  A acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = Op::template identity<T>();
  if (c < nv) {
    const uint4* pv = reinterpret_cast<const uint4*>(x) + c;
    long long k     = warp;
    for (; k + 24 < r; k += 32) {
      uint4 u[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) u[q] = __ldcs(pv + (k + 8 * q) * nv);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const T* e = reinterpret_cast<const T*>(&u[q]);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fold_elem<T, Op>(acc[i], e[i]);
      }
    }
    for (; k < r; k += 8) {
      const uint4 u = __ldcs(pv + k * nv);
      const T* e    = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = fold_elem<T, Op>(acc[i], e[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) part[warp][lane][i] = acc[i];
  __syncthreads();
  if (warp == 0 && c < nv) {
#pragma unroll
    for (int w = 1; w < 8; ++w)
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = Op::apply(acc[i], part[w][lane][i]);
    uint4 out;
    T* e = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int i = 0; i < V; ++i) e[i] = Elem<T>::store(acc[i]);
    if ((reinterpret_cast<uintptr_t>(y) & 15u) == 0) {
      reinterpret_cast<uint4*>(y)[c] = out;
    } else {  // the group's output may sit at any address; the partials this kernel reads are always aligned
#pragma unroll
      for (int i = 0; i < V; ++i) y[c * V + i] = e[i];
    }
  }
}

}  // namespace

#define REG_GENERIC(OPNAME, OP, TNAME, T)                                                                       \
  CINN_B200_REGISTER_KERNEL("reduce_generic_row_" OPNAME "_" TNAME, 6, 256, k_reduce_generic_row<T, OP>);      \
  CINN_B200_REGISTER_KERNEL("reduce_generic_col_" OPNAME "_" TNAME, 7, 256, k_reduce_generic_col<T, OP>);      \
  CINN_B200_REGISTER_KERNEL("reduce_generic_col_fold_" OPNAME "_" TNAME, 4, 256, k_reduce_generic_col_fold<T, OP>)
#define REG_GENERIC_ARITH(TNAME, T)   \
  REG_GENERIC("sum", GSum, TNAME, T);  \
  REG_GENERIC("prod", GProd, TNAME, T); \
  REG_GENERIC("max", GMax, TNAME, T);  \
  REG_GENERIC("min", GMin, TNAME, T)

REG_GENERIC_ARITH("f32", float);
REG_GENERIC_ARITH("f16", __half);
REG_GENERIC_ARITH("bf16", __nv_bfloat16);
REG_GENERIC_ARITH("f64", double);
REG_GENERIC_ARITH("i32", int32_t);
REG_GENERIC_ARITH("i64", long long);
REG_GENERIC("all", GAll, "bool", uint8_t);
REG_GENERIC("any", GAny, "bool", uint8_t);

}  // namespace cinn_b200
