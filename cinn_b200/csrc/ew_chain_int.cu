// Integer form of the generic elementwise chain (see ew_chain.cu for the float form and ew_chain.h for the program
// encoding): the chain value and its side operands are int32, int64 or uint8 values, bool travels as 0 / 1,
// immediates are signed 32-bit integers (truncated to the value type).  uint8 follows the unsigned instructions the
// reference's LLVM code generator picks for `uint` types (cinn/backends/llvm/codegen_llvm.cc:205-216, 280-340,
// 1449-1457: UDiv / URem, unsigned compares, logical right shift, zero-extending casts); + - * wrap modulo 256.  Arithmetic is what the reference generates for integer tensors:
// + - * wrap, `divide` truncates toward zero (ir::Div), max / min are compare + select, mod takes the sign of the
// divisor and floor_divide rounds toward minus infinity (cinn/lang/builtin.cc:108-121,
// cinn/runtime/cuda/cinn_cuda_runtime_source.cuh:160-183), shifts and bitwise ops are the C operators
// (cinn/hlir/pe/broadcast.cc:256-266), logical_right_shift shifts the unsigned value, clz / popc count bits
// (cinn/runtime/cpu/host_intrinsics.cc:240-262).  A divisor of zero gives 0 (the reference's x86 code would trap).
#include <cstdint>
#include <type_traits>

#include "device_math.cuh"
#include "ew_chain.h"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

template <typename T>
struct UnsignedOf;
template <>
struct UnsignedOf<int32_t> {
  using type = uint32_t;
};
template <>
struct UnsignedOf<long long> {
  using type = unsigned long long;
};
template <>
struct UnsignedOf<uint8_t> {
  using type = uint8_t;
};
// The storage type of a uint8 OUTPUT (uint8_t itself names the one-byte bool output of these kernels).
struct u8_out {
  uint8_t v;
};

template <typename T>
__device__ __forceinline__ T int_unary(int op, T x) {
  using U = typename UnsignedOf<T>::type;
  switch (op) {
    case EW_NEG: return (T)(U(0) - (U)x);
    case EW_ABS: return x > 0 ? x : (T)(U(0) - (U)x);
    case EW_LNOT: return x == 0 ? 1 : 0;
    case EW_TO_BOOL: return x != 0 ? 1 : 0;
    case EW_BNOT: return (T)~x;
    case EW_CLZ: return sizeof(T) == 4 ? (T)__clz((int)x) : (T)__clzll((long long)x);
    case EW_POPC: return sizeof(T) == 4 ? (T)__popc((unsigned)x) : (T)__popcll((unsigned long long)x);
    default: return x;
  }
}

// Integer pow as the reference's host intrinsics define it (cinn/runtime/cpu/host_intrinsics.cc:234-239, 255):
// (T)pow((double)x, (double)y) with the truncating x86 conversion, which yields the most negative value for
// anything out of range; int32 alone returns -1 for 0 to a negative power.  Computed exactly in integers: the
// magnitude by repeated squaring in 64 bits with overflow detection, then rounded once to double (to nearest even)
// and converted back.  Everything a double holds exactly -- every int32 result, int64 results up to 2^53 -- equals
// the host function; beyond 2^53 the host returns glibc's pow, which is within one ulp of the true power but not
// always the nearest double (9^17 lies exactly between two doubles and glibc returns the upper one), so results
// there may differ by one step of the double grid.
template <typename T>
__device__ __noinline__ T int_pow(T x, T y) {
  constexpr bool k32 = sizeof(T) == 4;
  const T kMin       = k32 ? (T)INT32_MIN : (T)INT64_MIN;
  // the exponent as double: beyond 2^53 every double is an even integer
  const unsigned long long ymag = y < 0 ? 0ull - (unsigned long long)y : (unsigned long long)y;
  const bool odd                = ymag <= (1ull << 53) && (ymag & 1);
  if (y < 0) {
    if (x == 0) return k32 ? (T)-1 : kMin;  // int64: pow(0, -n) is infinite
    if (x == 1) return 1;
    if (x == -1) return odd ? (T)-1 : (T)1;
    return 0;  // |x| >= 2: a magnitude below one truncates to zero
  }
  unsigned long long base = x < 0 ? 0ull - (unsigned long long)(long long)x : (unsigned long long)x;
  unsigned long long mag = 1, e = ymag;
  bool over = false;
  while (e) {
    if (e & 1) {
      over |= __umul64hi(mag, base) != 0;
      mag *= base;
    }
    e >>= 1;
    if (e) {
      over |= __umul64hi(base, base) != 0;
      base *= base;
    }
  }
  const bool neg = x < 0 && odd;
  if (k32) {
    if (over || mag > 0x80000000ull || (!neg && mag == 0x80000000ull)) return kMin;
    return (T)(neg ? 0ll - (long long)mag : (long long)mag);
  }
  const double d = __ull2double_rn(mag);
  if (over || d >= 9223372036854775808.0) return kMin;
  const long long v = __double2ll_rz(d);
  return (T)(neg ? -v : v);
}

template <typename T>
__device__ __forceinline__ bool is_minus_one(T v) {
  if constexpr (std::is_signed<T>::value) return v == (T)-1;
  return false;
}
template <typename T>
__device__ __forceinline__ bool is_negative(T v) {
  if constexpr (std::is_signed<T>::value) return v < 0;
  return false;
}

template <typename T>
__device__ __forceinline__ T int_binary(int op, T l, T r) {
  using U = typename UnsignedOf<T>::type;
  constexpr int kBits = sizeof(T) * 8;
  switch (op) {
    case EW_ADD: return (T)((U)l + (U)r);
    case EW_SUB: return (T)((U)l - (U)r);
    case EW_MUL: return (T)((U)l * (U)r);
    case EW_DIV: return r == 0 ? (T)0 : (is_minus_one(r) ? (T)(U(0) - (U)l) : (T)(l / r));
    case EW_MAX: return l > r ? l : r;
    case EW_MIN: return l < r ? l : r;
    case EW_POW: return sizeof(T) == 1 ? l : int_pow<typename std::conditional<sizeof(T) == 1, int32_t, T>::type>(l, r);
    case EW_EQ: return l == r;
    case EW_NE: return l != r;
    case EW_GT: return l > r;
    case EW_LT: return l < r;
    case EW_GE: return l >= r;
    case EW_LE: return l <= r;
    case EW_MOD: {
      if (r == 0 || is_minus_one(r)) return 0;
      T res = (T)(l % r);
      if (res != 0 && is_negative((T)(r ^ res))) res = (T)(res + r);
      return res;
    }
    case EW_FLOOR_DIV: {
      if (r == 0) return 0;
      if (is_minus_one(r)) return (T)(U(0) - (U)l);
      const T div = (T)(l / r), mod = (T)(l % r);
      return ((l > 0 && r > 0) || (is_negative(l) && is_negative(r))) ? div : (mod == 0 ? div : (T)(div - 1));
    }
    case EW_LAND: return (l != 0 && r != 0) ? 1 : 0;
    case EW_LOR: return (l != 0 || r != 0) ? 1 : 0;
    case EW_LXOR: return ((l != 0) != (r != 0)) ? 1 : 0;
    case EW_BAND: return (T)(l & r);
    case EW_BOR: return (T)(l | r);
    case EW_BXOR: return (T)(l ^ r);
    // shift counts are taken modulo the width, as the x86 shift instructions do
    case EW_SHL: return (T)((U)l << ((int)r & (kBits - 1)));
    case EW_SHR: return (T)(l >> ((int)r & (kBits - 1)));
    case EW_LSHR: return (T)((U)l >> ((int)r & (kBits - 1)));
    case EW_COPY: return r;
    default: return l;
  }
}

template <typename T>
__device__ __forceinline__ T load_int(const void* p, int dtype, long long idx) {
  switch (dtype) {
    case EW_BOOL: return static_cast<const uint8_t*>(p)[idx] != 0 ? 1 : 0;
    case EW_I32: return (T) static_cast<const int32_t*>(p)[idx];
    case EW_U8: return (T) static_cast<const uint8_t*>(p)[idx];
    default: return (T) static_cast<const long long*>(p)[idx];
  }
}

// Four consecutive elements starting at idx (idx % 4 == 0, pointer 16-byte aligned).
template <typename T>
__device__ __forceinline__ void load_int4(const void* p, int dtype, long long idx, bool stream, T (&v)[4]) {
  if (dtype == EW_BOOL) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p) + idx);
    const uint32_t u  = stream ? __ldcs(q) : __ldg(q);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ((u >> (8 * i)) & 0xffu) != 0 ? 1 : 0;
  } else if (dtype == EW_U8) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p) + idx);
    const uint32_t u  = stream ? __ldcs(q) : __ldg(q);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (T)((u >> (8 * i)) & 0xffu);
  } else if (dtype == EW_I32) {
    const int4* q = reinterpret_cast<const int4*>(static_cast<const int32_t*>(p) + idx);
    const int4 u  = stream ? __ldcs(q) : __ldg(q);
    v[0] = (T)u.x; v[1] = (T)u.y; v[2] = (T)u.z; v[3] = (T)u.w;
  } else {
    const longlong2* q = reinterpret_cast<const longlong2*>(static_cast<const long long*>(p) + idx);
    const longlong2 u0 = stream ? __ldcs(q) : __ldg(q);
    const longlong2 u1 = stream ? __ldcs(q + 1) : __ldg(q + 1);
    v[0] = (T)u0.x; v[1] = (T)u0.y; v[2] = (T)u1.x; v[3] = (T)u1.y;
  }
}

template <typename T, typename OutT>
__device__ __forceinline__ OutT convert_out(T v);
template <> __device__ __forceinline__ int32_t convert_out<int32_t, int32_t>(int32_t v) { return v; }
template <> __device__ __forceinline__ long long convert_out<int32_t, long long>(int32_t v) { return v; }
template <> __device__ __forceinline__ uint8_t convert_out<int32_t, uint8_t>(int32_t v) { return v != 0; }
template <> __device__ __forceinline__ float convert_out<int32_t, float>(int32_t v) { return (float)v; }
template <> __device__ __forceinline__ int32_t convert_out<long long, int32_t>(long long v) { return (int32_t)v; }
template <> __device__ __forceinline__ long long convert_out<long long, long long>(long long v) { return v; }
template <> __device__ __forceinline__ uint8_t convert_out<long long, uint8_t>(long long v) { return v != 0; }
template <> __device__ __forceinline__ float convert_out<long long, float>(long long v) { return (float)v; }
template <> __device__ __forceinline__ u8_out convert_out<uint8_t, u8_out>(uint8_t v) { return u8_out{v}; }
template <> __device__ __forceinline__ uint8_t convert_out<uint8_t, uint8_t>(uint8_t v) { return v != 0; }
template <> __device__ __forceinline__ int32_t convert_out<uint8_t, int32_t>(uint8_t v) { return v; }
template <> __device__ __forceinline__ long long convert_out<uint8_t, long long>(uint8_t v) { return v; }
template <> __device__ __forceinline__ float convert_out<uint8_t, float>(uint8_t v) { return (float)v; }
template <> __device__ __forceinline__ u8_out convert_out<int32_t, u8_out>(int32_t v) { return u8_out{(uint8_t)v}; }
template <> __device__ __forceinline__ u8_out convert_out<long long, u8_out>(long long v) { return u8_out{(uint8_t)v}; }

template <typename T, typename OutT>
__device__ __forceinline__ void store_int4(OutT* p, long long idx, const T (&v)[4]) {
  // one store of 4 / 16 bytes, or two of 16 for 8-byte elements (the buffers are only known to be 16-byte aligned)
  constexpr int kHalf = sizeof(OutT) == 8 ? 2 : 4;
  struct alignas(sizeof(OutT) * kHalf) Pack {
    OutT e[kHalf];
  };
#pragma unroll
  for (int h = 0; h < 4 / kHalf; ++h) {
    Pack pk;
#pragma unroll
    for (int i = 0; i < kHalf; ++i) pk.e[i] = convert_out<T, OutT>(v[h * kHalf + i]);
    *reinterpret_cast<Pack*>(p + idx + h * kHalf) = pk;
  }
}

struct SideSpec {
  const void* ptr;
  int dtype, mode;
  long long mid, inner;
};

__device__ __forceinline__ long long side_index(long long i, long long inner, long long mid) {
  if (((i | inner | mid) >> 31) == 0) return (long long)(((unsigned)i / (unsigned)inner) % (unsigned)mid);
  return (i / inner) % mid;
}

template <typename T, int VEC>
__device__ __forceinline__ void load_side(const SideSpec& s, long long i0, T (&f)[VEC]) {
  if (VEC == 4 && s.mode == EW_SIDE_FULL) {
    load_int4<T>(s.ptr, s.dtype, i0, true, *reinterpret_cast<T(*)[4]>(&f[0]));
  } else if (VEC == 4 && s.mode == EW_SIDE_PERIODIC_VEC) {
    load_int4<T>(s.ptr, s.dtype, side_index(i0, 1, s.mid), false, *reinterpret_cast<T(*)[4]>(&f[0]));
  } else if (s.mode == EW_SIDE_ONE_PER_VEC || s.mode == EW_SIDE_SCALAR) {
    const T v = load_int<T>(s.ptr, s.dtype, s.mode == EW_SIDE_SCALAR ? 0 : side_index(i0, s.inner, s.mid));
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = v;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = load_int<T>(s.ptr, s.dtype, side_index(i0 + i, s.inner, s.mid));
  }
}

// ONE step of an integer chain program on VEC values (the fields of the step's word decoded by the caller: at run
// time by the interpreter, as constants by the kernels specialised at build time).  Returns true when the step used
// the next word's immediate.
// NS = how many side inputs the kernel variant carries (0, 1 or 3): the registers of absent sides are never touched.
// NT = 2: two temporaries (operand selectors 5 and 6, written by EW_STASH) for expression trees, as in the float form.
template <typename T, int VEC, int NS, int NT>
__device__ __forceinline__ bool int_chain_step(int op, int asel, int bsel, int role, T imm, T imm2, const T (&s1)[VEC],
                                               const T (&s2)[VEC], const T (&s3)[VEC], T (&acc)[VEC],
                                               T (&ta)[NT > 0 ? VEC : 1], T (&tb)[NT > 0 ? VEC : 1]) {
  if (op == EW_NOP) return false;
  if (op >= EW_FIRST_UNARY) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = int_unary<T>(op, acc[i]);
    return false;
  }
  if (NT > 0 && op == EW_STASH) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) (asel == 5 ? ta : tb)[NT > 0 ? i : 0] = acc[i];
    return false;
  }
  T o[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    o[i] = (NS >= 1 && asel == 1) ? s1[i] : ((NS >= 2 && asel == 2) ? s2[i] : ((NS >= 3 && asel == 3) ? s3[i] : (asel == 4 ? acc[i] : imm)));
    if (NT > 0) o[i] = asel == 5 ? ta[NT > 0 ? i : 0] : (asel == 6 ? tb[NT > 0 ? i : 0] : o[i]);
  }
  if (op == EW_SELECT) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      T b = (NS >= 1 && bsel == 1) ? s1[i] : ((NS >= 2 && bsel == 2) ? s2[i] : ((NS >= 3 && bsel == 3) ? s3[i] : (bsel == 4 ? acc[i] : imm2)));
      if (NT > 0) b = bsel == 5 ? ta[NT > 0 ? i : 0] : (bsel == 6 ? tb[NT > 0 ? i : 0] : b);
      const T c = role == 0 ? acc[i] : o[i];
      const T t = role == 0 ? o[i] : (role == 1 ? acc[i] : b);
      const T f = role == 2 ? acc[i] : b;
      acc[i]    = c != 0 ? t : f;
    }
    return bsel == 0;
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i)
    acc[i] = (role != 0 && op != EW_COPY) ? int_binary<T>(op, o[i], acc[i]) : int_binary<T>(op, acc[i], o[i]);
  return false;
}

template <typename T>
__device__ __forceinline__ T int_imm(long long word) { return (T)(int32_t)(word >> 32); }

// The interpreter's program: everything comes from kernel parameters.
template <typename T>
struct DynIntProgram {
  const long long* steps;
  int nsteps;
  long long meta;
  __device__ __forceinline__ int in_type() const { return (int)((meta >> 24) & 15); }
  __device__ __forceinline__ int side_dtype(int k) const { return (int)((meta >> (8 * (k - 1))) & 15); }
  __device__ __forceinline__ int side_mode(int k) const { return (int)((meta >> (8 * (k - 1) + 4)) & 15); }
  template <int VEC, int NS, int NT>
  __device__ __forceinline__ void run(const T (&s1)[VEC], const T (&s2)[VEC], const T (&s3)[VEC], T (&acc)[VEC]) const {
    T ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
    if (NT > 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0;
    }
    for (int k = 0; k < nsteps; ++k) {
      const long long st = steps[k];
      if (int_chain_step<T, VEC, NS, NT>((int)(st & 0xff), (int)((st >> 8) & 0xff), (int)((st >> 16) & 0xff),
                                         (int)((st >> 24) & 3), int_imm<T>(st), int_imm<T>(steps[k + 1]), s1, s2, s3,
                                         acc, ta, tb))
        ++k;
    }
  }
};

// A program whose structure was fixed when the library was built (see ew_static.cu for the scheme).
template <typename T, unsigned long long META, uint32_t... SIG>
struct StaticIntProgram {
  const long long* steps;
  __device__ __forceinline__ constexpr int in_type() const { return (int)((META >> 24) & 15); }
  __device__ __forceinline__ constexpr int side_dtype(int k) const { return (int)((META >> (8 * (k - 1))) & 15); }
  __device__ __forceinline__ constexpr int side_mode(int k) const { return (int)((META >> (8 * (k - 1) + 4)) & 15); }
  template <int VEC, int NS, int NT, int K>
  __device__ __forceinline__ void from(const T (&s1)[VEC], const T (&s2)[VEC], const T (&s3)[VEC], T (&acc)[VEC],
                                       T (&ta)[NT > 0 ? VEC : 1], T (&tb)[NT > 0 ? VEC : 1]) const {
    constexpr int N = (int)sizeof...(SIG);
    if constexpr (K < N) {
      constexpr uint32_t sig[N] = {SIG...};
      constexpr uint32_t w      = sig[K];
      constexpr int op = (int)(w & 0xff), asel = (int)((w >> 8) & 0xff), bsel = (int)((w >> 16) & 0xff),
                    role = (int)((w >> 24) & 3);
      constexpr bool two = op == EW_SELECT && bsel == 0;
      (void)int_chain_step<T, VEC, NS, NT>(op, asel, bsel, role, int_imm<T>(steps[K]),
                                           int_imm<T>(steps[K + 1 < EW_MAX_STEPS ? K + 1 : K]), s1, s2, s3, acc, ta, tb);
      from<VEC, NS, NT, K + (two ? 2 : 1)>(s1, s2, s3, acc, ta, tb);
    }
  }
  template <int VEC, int NS, int NT>
  __device__ __forceinline__ void run(const T (&s1)[VEC], const T (&s2)[VEC], const T (&s3)[VEC], T (&acc)[VEC]) const {
    T ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
    if (NT > 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0;
    }
    from<VEC, NS, NT, 0>(s1, s2, s3, acc, ta, tb);
  }
};

template <typename T, typename OutT, int NS, int NT, class Prog>
__device__ __forceinline__ void int_chain_body(const Prog& prog, const void* __restrict__ in0,
                                               const void* __restrict__ p1, const void* __restrict__ p2,
                                               const void* __restrict__ p3, OutT* __restrict__ out, long long n,
                                               long long vec_ok, long long mid1, long long inner1, long long mid2,
                                               long long inner2, long long mid3, long long inner3) {
  const int in_type  = prog.in_type();
  const SideSpec sd1 = {p1, prog.side_dtype(1), prog.side_mode(1), mid1, inner1};
  const SideSpec sd2 = {p2, prog.side_dtype(2), prog.side_mode(2), mid2, inner2};
  const SideSpec sd3 = {p3, prog.side_dtype(3), prog.side_mode(3), mid3, inner3};
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (vec_ok) {
    const long long nvec = n >> 2;
    // 32-bit values: two vectors (8 elements) per thread iteration, all loads issued before the program runs.
    constexpr int NV = (sizeof(T) == 4 && NT == 0) ? 2 : 1;  // one vector with temporaries: they cost registers
    long long v      = tid;
    for (; v + (NV - 1) * stride < nvec; v += NV * stride) {
      T acc[4 * NV], s1[4 * NV], s2[4 * NV], s3[4 * NV];
#pragma unroll
      for (int j = 0; j < NV; ++j)
        if (in_type != EW_NO_INPUT) load_int4<T>(in0, in_type, (v + j * stride) << 2, true, *reinterpret_cast<T(*)[4]>(&acc[4 * j]));
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const long long i0 = (v + j * stride) << 2;
        if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<T, 4>(sd1, i0, *reinterpret_cast<T(*)[4]>(&s1[4 * j]));
        if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<T, 4>(sd2, i0, *reinterpret_cast<T(*)[4]>(&s2[4 * j]));
        if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<T, 4>(sd3, i0, *reinterpret_cast<T(*)[4]>(&s3[4 * j]));
      }
      prog.template run<4 * NV, NS, NT>(s1, s2, s3, acc);
#pragma unroll
      for (int j = 0; j < NV; ++j) store_int4<T, OutT>(out, (v + j * stride) << 2, *reinterpret_cast<T(*)[4]>(&acc[4 * j]));
    }
    for (; v < nvec; v += stride) {
      const long long i0 = v << 2;
      T acc[4], s1[4], s2[4], s3[4];
      if (in_type != EW_NO_INPUT) load_int4<T>(in0, in_type, i0, true, acc);
      if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<T, 4>(sd1, i0, s1);
      if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<T, 4>(sd2, i0, s2);
      if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<T, 4>(sd3, i0, s3);
      prog.template run<4, NS, NT>(s1, s2, s3, acc);
      store_int4<T, OutT>(out, i0, acc);
    }
    done = nvec << 2;
  }
  for (long long i = done + tid; i < n; i += stride) {
    T acc[1], s1[1], s2[1], s3[1];
    acc[0] = in_type != EW_NO_INPUT ? load_int<T>(in0, in_type, i) : 0;
    if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<T, 1>(sd1, i, s1);
    if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<T, 1>(sd2, i, s2);
    if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<T, 1>(sd3, i, s3);
    prog.template run<1, NS, NT>(s1, s2, s3, acc);
    out[i] = convert_out<T, OutT>(acc[0]);
  }
}

#define INT_CHAIN_PARAMS                                                                                              \
  const void *__restrict__ in0, const void *__restrict__ p1, const void *__restrict__ p2, const void *__restrict__ p3, \
      OutT *__restrict__ out, long long n, long long vec_ok, long long meta, long long mid1, long long inner1,        \
      long long mid2, long long inner2, long long mid3, long long inner3, long long nsteps_ll, long long t0,         \
      long long t1, long long t2, long long t3, long long t4, long long t5, long long t6, long long t7, long long t8, \
      long long t9, long long t10, long long t11, long long t12, long long t13, long long t14, long long t15

// Same parameter list as the float form (k_ew_chain): meta bits 0-3 / 4-7 dtype / mode of side 1, 8-15 side 2,
// 16-23 side 3, 24-27 dtype of in0.
template <typename T, typename OutT, int NS, int NT = 0>
__global__ void __launch_bounds__(256) k_ew_chain_int(INT_CHAIN_PARAMS) {
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0};
  const DynIntProgram<T> prog = {steps, (int)nsteps_ll, meta};
  int_chain_body<T, OutT, NS, NT>(prog, in0, p1, p2, p3, out, n, vec_ok, mid1, inner1, mid2, inner2, mid3, inner3);
}

template <typename T, typename OutT, int NS, int NT, unsigned long long META, uint32_t... SIG>
__global__ void __launch_bounds__(256) k_ew_chain_int_static(INT_CHAIN_PARAMS) {
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0};
  const StaticIntProgram<T, META, SIG...> prog = {steps};
  int_chain_body<T, OutT, NS, NT>(prog, in0, p1, p2, p3, out, n, vec_ok, mid1, inner1, mid2, inner2, mid3, inner3);
}

template <uint32_t... SIG>
StaticChainKey MakeKey(const char* base, long long meta) {
  StaticChainKey k = {base, meta, (int)sizeof...(SIG), {SIG...}};
  return k;
}

}  // namespace

#define REG_INT_CHAIN_NS(TNAME, T, NSNAME, NS)                                                                       \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_i32_" NSNAME, 31, 256, k_ew_chain_int<T, int32_t, NS>);        \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_i64_" NSNAME, 31, 256, k_ew_chain_int<T, long long, NS>);      \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_bool_" NSNAME, 31, 256, k_ew_chain_int<T, uint8_t, NS>);       \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_f32_" NSNAME, 31, 256, k_ew_chain_int<T, float, NS>)
#define REG_INT_CHAIN(TNAME, T)                                                                                     \
  REG_INT_CHAIN_NS(TNAME, T, "s0", 0);                                                                              \
  REG_INT_CHAIN_NS(TNAME, T, "s1", 1);                                                                              \
  REG_INT_CHAIN_NS(TNAME, T, "s3", 3);                                                                              \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_i32_s3t", 31, 256, k_ew_chain_int<T, int32_t, 3, 2>);          \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_i64_s3t", 31, 256, k_ew_chain_int<T, long long, 3, 2>);        \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_bool_s3t", 31, 256, k_ew_chain_int<T, uint8_t, 3, 2>);         \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_f32_s3t", 31, 256, k_ew_chain_int<T, float, 3, 2>)

#define REG_U8_OUT(TNAME, T)                                                                                \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_u8_s0", 31, 256, k_ew_chain_int<T, u8_out, 0>);        \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_u8_s1", 31, 256, k_ew_chain_int<T, u8_out, 1>);        \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_u8_s3", 31, 256, k_ew_chain_int<T, u8_out, 3>);        \
  CINN_B200_REGISTER_KERNEL("ew_chain_int_" TNAME "_u8_s3t", 31, 256, k_ew_chain_int<T, u8_out, 3, 2>)

REG_INT_CHAIN("i32", int32_t);
REG_INT_CHAIN("i64", long long);
REG_INT_CHAIN("u8", uint8_t);
REG_U8_OUT("u8", uint8_t);
REG_U8_OUT("i32", int32_t);
REG_U8_OUT("i64", long long);

}  // namespace cinn_b200

namespace cinn_b200 {
#define STATIC_INT_CHAIN(ID, BASE, T, OutT, NS, NT, META, ...)                                                      \
  CINN_B200_REGISTER_KERNEL("ew_int_static_" #ID, 31, 256, k_ew_chain_int_static<T, OutT, NS, NT, META##ull, __VA_ARGS__>); \
  static int cinn_b200_static_int_chain_##ID = RegisterStaticChain(MakeKey<__VA_ARGS__>(BASE, META##ll), "ew_int_static_" #ID)
#include "ew_int_static_table.inc"
}  // namespace cinn_b200
