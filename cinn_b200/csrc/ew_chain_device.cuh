// Device side of the elementwise-chain interpreter, shared by the kernels that run a chain program: the plain chain
// kernel (ew_chain.cu) and the reductions with a chain as their first stage (chain_reduce.cu).  Loads of every storage
// type into fp32 registers, side-operand addressing, and run_chain(), which applies the program to VEC values.
#pragma once

#include <cstdint>

#include "device_math.cuh"
#include "ew_chain.h"

namespace cinn_b200 {
namespace {

// Rarely used, code-heavy functions stay out of line so that the interpreter's unrolled body stays small enough
// for the instruction cache (each inlined copy of erff / sinf / powf is hundreds of instructions).
__device__ __noinline__ float heavy_unary(int op, float x) {
  switch (op) {
    case EW_ERF: return erff(x);
    case EW_SIN: return sinf(x);
    case EW_COS: return cosf(x);
    case EW_LOG2: return log2f(x);
    case EW_LOG10: return log10f(x);
    // The functions below are evaluated in double precision and rounded once: the host library the x86 path calls
    // is within an ulp of the correctly rounded result, which CUDA's single-precision versions (2-4 ulp) are not.
    // cinn/backends/llvm/llvm_intrin_rule.h:126-175: tan = sin / cos, sinh / cosh from two exps
    case EW_TAN: return (float)sin((double)x) / (float)cos((double)x);
    case EW_SINH: return ((float)exp((double)x) - (float)exp((double)(x * -1.0f))) / 2.0f;
    case EW_COSH: return ((float)exp((double)x) + (float)exp((double)(x * -1.0f))) / 2.0f;
    // cinn/optim/map_extern_call.cc:42-74: the host's asinf ... atanhf
    case EW_ASIN: return (float)asin((double)x);
    case EW_ACOS: return (float)acos((double)x);
    case EW_ATAN: return (float)atan((double)x);
    case EW_ASINH: return (float)asinh((double)x);
    case EW_ACOSH: return (float)acosh((double)x);
    case EW_ATANH: return (float)atanh((double)x);
    // cinn/runtime/cpu/host_intrinsics.cc:216: the double-precision cbrt of the promoted argument
    case EW_CBRT: return (float)cbrt((double)x);
    default: return x;
  }
}
__device__ __noinline__ float heavy_pow(float l, float r) { return powf(l, r); }
// cinn/runtime/cuda/cinn_cuda_runtime_source.cuh:84-88: the result takes the sign of the divisor
__device__ __noinline__ float heavy_mod(float l, float r) {
  float res = fmodf(l, r);
  if ((res != 0.0f) && ((res < 0.0f) != (r < 0.0f))) res += r;
  return res;
}
// cinn/hlir/pe/broadcast.cc:275-291
__device__ __noinline__ float heavy_atan2(float a, float b) {
  const float at = (float)atan((double)(a / b));
  const float pi = (float)3.14159265358979323846, half_pi = (float)(3.14159265358979323846 / 2);
  if (b == 0.0f) return a == 0.0f ? 0.0f : (a > 0.0f ? half_pi : -half_pi);
  return b > 0.0f ? at : (a >= 0.0f ? at + pi : at - pi);
}

// FAST: exp / tanh / sigmoid through the hardware's approximate exponential and reciprocal (relative error about
// 1e-6).  Only the specialised reductions use it: their result is judged at the reduction tolerance (1e-5 relative),
// which a sum of such terms keeps with a wide margin, and the full-precision forms make those kernels issue-bound.
// INL: the caller knows `op` at build time, so the error function is expanded in place (the same erff as the
// out-of-line copy, without a call per element); the interpreter keeps the call to hold its code size down.
template <int VEC, bool FAST = false, bool INL = false>
__device__ __forceinline__ void apply_unary(int op, float imm, float (&a)[VEC]) {
  if (INL && op == EW_ERF) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) a[i] = erff(a[i]);
    return;
  }
#define EW_UNARY_CASE(code, expr) \
  case code:                      \
    _Pragma("unroll") for (int i = 0; i < VEC; ++i) { const float x = a[i]; a[i] = (expr); } \
    break;
  switch (op) {
    EW_UNARY_CASE(EW_EXP, FAST ? exp_for_16bit_out(x) : expf(x))
    EW_UNARY_CASE(EW_TANH, FAST ? x86_tanh_for_16bit_out(x) : x86_tanh(x))
    EW_UNARY_CASE(EW_SIGMOID, FAST ? rcp_approx(1.0f + exp_for_16bit_out(-x)) : x86_sigmoid(x))
    EW_UNARY_CASE(EW_RSQRT, x86_rsqrt(x))
    EW_UNARY_CASE(EW_SQRT, sqrtf(x))
    EW_UNARY_CASE(EW_RELU, x86_max(x, 0.0f))
    EW_UNARY_CASE(EW_NEG, -x)
    EW_UNARY_CASE(EW_ABS, fabsf(x))
    EW_UNARY_CASE(EW_LOG, logf(x))
    EW_UNARY_CASE(EW_FLOOR, floorf(x))
    EW_UNARY_CASE(EW_CEIL, ceilf(x))
    EW_UNARY_CASE(EW_RECIP, 1.0f / x)
    EW_UNARY_CASE(EW_ROUND, nearbyintf(x))
    EW_UNARY_CASE(EW_TRUNC, truncf(x))
    EW_UNARY_CASE(EW_SIGN, x < 0.0f ? -1.0f : (x > 0.0f ? 1.0f : (x == 0.0f ? 0.0f : x)))
    EW_UNARY_CASE(EW_RELU6, x86_min(x86_max(x, 0.0f), imm))
    EW_UNARY_CASE(EW_ROUND_F16, __half2float(__float2half_rn(x)))
    EW_UNARY_CASE(EW_ROUND_BF16, __bfloat162float(__float2bfloat16_rn(x)))
    // cinn/backends/llvm/llvm_intrin_rule.h:78-104 and cinn/lang/builtin.cc:212-259
    EW_UNARY_CASE(EW_ISNAN, x != x ? 1.0f : 0.0f)
    EW_UNARY_CASE(EW_ISINF, (fabsf(x) == __int_as_float(0x7f800000) && !(x != x)) ? 1.0f : 0.0f)
    EW_UNARY_CASE(EW_ISFINITE, (fabsf(x) == __int_as_float(0x7f800000) || x != x) ? 0.0f : 1.0f)
    EW_UNARY_CASE(EW_LNOT, x == 0.0f ? 1.0f : 0.0f)
    EW_UNARY_CASE(EW_TO_BOOL, x != 0.0f ? 1.0f : 0.0f)
    case EW_IDENTITY:
      break;
    default:  // the code-heavy functions
#pragma unroll
      for (int i = 0; i < VEC; ++i) a[i] = heavy_unary(op, a[i]);
      break;
  }
#undef EW_UNARY_CASE
}

// acc (op) o, or o (op) acc when swapped: the operand order of the reference expression is kept because
// max/min/sub/div/pow and the comparisons are not symmetric (max(a,b) = a > b ? a : b).
template <int VEC>
__device__ __forceinline__ void apply_binary(int op, bool swap, const float (&o)[VEC], float (&a)[VEC]) {
#define EW_BINARY_CASE(code, expr)                                 \
  case code:                                                       \
    _Pragma("unroll") for (int i = 0; i < VEC; ++i) {              \
      const float l = swap ? o[i] : a[i], r = swap ? a[i] : o[i];  \
      a[i] = (expr);                                               \
    }                                                              \
    break;
  switch (op) {
    EW_BINARY_CASE(EW_ADD, l + r)
    EW_BINARY_CASE(EW_SUB, l - r)
    EW_BINARY_CASE(EW_MUL, l * r)
    EW_BINARY_CASE(EW_DIV, l / r)
    EW_BINARY_CASE(EW_MAX, x86_max(l, r))
    EW_BINARY_CASE(EW_MIN, x86_min(l, r))
    EW_BINARY_CASE(EW_POW, heavy_pow(l, r))
    EW_BINARY_CASE(EW_EQ, l == r ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_NE, l != r ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_GT, l > r ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_LT, l < r ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_GE, l >= r ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_LE, l <= r ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_MOD, heavy_mod(l, r))
    EW_BINARY_CASE(EW_FLOOR_DIV, floorf(l / r))
    EW_BINARY_CASE(EW_ATAN2, heavy_atan2(l, r))
    EW_BINARY_CASE(EW_LAND, (l != 0.0f && r != 0.0f) ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_LOR, (l != 0.0f || r != 0.0f) ? 1.0f : 0.0f)
    EW_BINARY_CASE(EW_LXOR, ((l != 0.0f) != (r != 0.0f)) ? 1.0f : 0.0f)
    case EW_COPY:
#pragma unroll
      for (int i = 0; i < VEC; ++i) a[i] = o[i];
      break;
    default:
      break;
  }
#undef EW_BINARY_CASE
}

__device__ __forceinline__ float load_scalar(const void* p, int dtype, long long idx) {
  switch (dtype) {
    case EW_F32: return static_cast<const float*>(p)[idx];
    case EW_F16: return __half2float(static_cast<const __half*>(p)[idx]);
    case EW_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    case EW_BOOL: return static_cast<const uint8_t*>(p)[idx] != 0 ? 1.0f : 0.0f;
    case EW_I32: return (float)static_cast<const int32_t*>(p)[idx];  // the cast op's own rounding (to nearest even)
    case EW_U8: return (float)static_cast<const uint8_t*>(p)[idx];
    default: return (float)static_cast<const long long*>(p)[idx];
  }
}

// Four consecutive elements starting at idx (idx % 4 == 0, pointer 16-byte aligned).
__device__ __forceinline__ void load_vec4(const void* p, int dtype, long long idx, bool stream, float (&f)[4]) {
  if (dtype == EW_F32) {
    const uint4* q = reinterpret_cast<const uint4*>(static_cast<const float*>(p) + idx);
    unpack4(stream ? __ldcs(q) : __ldg(q), f);
  } else if (dtype == EW_F16 || dtype == EW_BF16) {
    const uint2* q = reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + idx);
    uint2 u        = stream ? __ldcs(q) : __ldg(q);
    if (dtype == EW_F16) {
      unpack_h2(u.x, f[0], f[1]);
      unpack_h2(u.y, f[2], f[3]);
    } else {
      unpack_bf2(u.x, f[0], f[1]);
      unpack_bf2(u.y, f[2], f[3]);
    }
  } else if (dtype == EW_BOOL) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p) + idx);
    const uint32_t u  = stream ? __ldcs(q) : __ldg(q);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = ((u >> (8 * i)) & 0xffu) != 0 ? 1.0f : 0.0f;
  } else if (dtype == EW_U8) {
    const uint32_t* q = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p) + idx);
    const uint32_t u  = stream ? __ldcs(q) : __ldg(q);
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = (float)((u >> (8 * i)) & 0xffu);
  } else if (dtype == EW_I32) {
    const int4* q = reinterpret_cast<const int4*>(static_cast<const int32_t*>(p) + idx);
    const int4 u  = stream ? __ldcs(q) : __ldg(q);
    f[0] = (float)u.x; f[1] = (float)u.y; f[2] = (float)u.z; f[3] = (float)u.w;
  } else {
    const longlong2* q = reinterpret_cast<const longlong2*>(static_cast<const long long*>(p) + idx);
    const longlong2 u0 = stream ? __ldcs(q) : __ldg(q);
    const longlong2 u1 = stream ? __ldcs(q + 1) : __ldg(q + 1);
    f[0] = (float)u0.x; f[1] = (float)u0.y; f[2] = (float)u1.x; f[3] = (float)u1.y;
  }
}

// float -> integer as the x86 conversion instruction does it (cvttss2si): toward zero; NaN and values out of
// range give the most negative integer.
__device__ __forceinline__ int32_t x86_f2i32(float x) {
  return (x >= -2147483648.0f && x < 2147483648.0f) ? (int32_t)x : (int32_t)0x80000000;
}
__device__ __forceinline__ long long x86_f2i64(float x) {
  return (x >= -9223372036854775808.0f && x < 9223372036854775808.0f) ? (long long)x : (long long)0x8000000000000000ull;
}

template <typename OutT>
__device__ __forceinline__ void store_vec4(OutT* p, long long idx, const float (&f)[4]);
template <>
__device__ __forceinline__ void store_vec4<float>(float* p, long long idx, const float (&f)[4]) {
  __stcs(reinterpret_cast<uint4*>(p + idx), pack4(f));
}
template <>
__device__ __forceinline__ void store_vec4<__half>(__half* p, long long idx, const float (&f)[4]) {
  __stcs(reinterpret_cast<uint2*>(p + idx), make_uint2(pack_h2(f[0], f[1]), pack_h2(f[2], f[3])));
}
template <>
__device__ __forceinline__ void store_vec4<__nv_bfloat16>(__nv_bfloat16* p, long long idx, const float (&f)[4]) {
  __stcs(reinterpret_cast<uint2*>(p + idx), make_uint2(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3])));
}
template <>
__device__ __forceinline__ void store_vec4<uint8_t>(uint8_t* p, long long idx, const float (&f)[4]) {
  uint32_t u = (f[0] != 0.0f ? 1u : 0u) | (f[1] != 0.0f ? 1u << 8 : 0u) | (f[2] != 0.0f ? 1u << 16 : 0u) |
               (f[3] != 0.0f ? 1u << 24 : 0u);
  *reinterpret_cast<uint32_t*>(p + idx) = u;
}
template <>
__device__ __forceinline__ void store_vec4<int32_t>(int32_t* p, long long idx, const float (&f)[4]) {
  __stcs(reinterpret_cast<int4*>(p + idx), make_int4(x86_f2i32(f[0]), x86_f2i32(f[1]), x86_f2i32(f[2]), x86_f2i32(f[3])));
}
template <>
__device__ __forceinline__ void store_vec4<long long>(long long* p, long long idx, const float (&f)[4]) {
  __stcs(reinterpret_cast<longlong2*>(p + idx), make_longlong2(x86_f2i64(f[0]), x86_f2i64(f[1])));
  __stcs(reinterpret_cast<longlong2*>(p + idx) + 1, make_longlong2(x86_f2i64(f[2]), x86_f2i64(f[3])));
}
template <typename OutT>
__device__ __forceinline__ void store_one(OutT* p, long long idx, float v) {
  Io<OutT>::store1(p + idx, v);
}
template <>
__device__ __forceinline__ void store_one<uint8_t>(uint8_t* p, long long idx, float v) {
  p[idx] = v != 0.0f ? 1 : 0;
}
template <>
__device__ __forceinline__ void store_one<int32_t>(int32_t* p, long long idx, float v) {
  p[idx] = x86_f2i32(v);
}
template <>
__device__ __forceinline__ void store_one<long long>(long long* p, long long idx, float v) {
  p[idx] = x86_f2i64(v);
}

struct SideSpec {
  const void* ptr;
  int dtype, mode;
  long long mid, inner;
  // Set by kernels that walk rows: the flat index at which the current row starts and the row's length.  A vector
  // operand whose period is the row length is then indexed by the offset within the row, without a division.
  long long row_base, row_len;
};

// (i / inner) % mid, in 32-bit arithmetic whenever the operands allow it (64-bit division is several times dearer).
__device__ __forceinline__ long long side_index(long long i, long long inner, long long mid) {
  if (((i | inner | mid) >> 31) == 0) return (long long)(((unsigned)i / (unsigned)inner) % (unsigned)mid);
  return (i / inner) % mid;
}

// stream: a full-size operand is read once (evict-first); false when the same threads read it again shortly after
// (the later passes of a row program), so that it stays in L1.
template <int VEC>
__device__ __forceinline__ void load_side(const SideSpec& s, long long i0, float (&f)[VEC], bool stream = true) {
  if (VEC == 4 && s.mode == EW_SIDE_FULL) {
    load_vec4(s.ptr, s.dtype, i0, stream, *reinterpret_cast<float(*)[4]>(&f[0]));
  } else if (VEC == 4 && s.mode == EW_SIDE_PERIODIC_VEC) {
    const long long idx = s.mid == s.row_len ? i0 - s.row_base : side_index(i0, 1, s.mid);
    load_vec4(s.ptr, s.dtype, idx, false, *reinterpret_cast<float(*)[4]>(&f[0]));
  } else if (s.mode == EW_SIDE_ONE_PER_VEC || s.mode == EW_SIDE_SCALAR) {
    const float v = load_scalar(s.ptr, s.dtype, s.mode == EW_SIDE_SCALAR ? 0 : side_index(i0, s.inner, s.mid));
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = v;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = load_scalar(s.ptr, s.dtype, side_index(i0 + i, s.inner, s.mid));
  }
}

// NS = how many side inputs the kernel variant carries (0, 1 or 3): the registers of absent sides are never touched.
// Where EW_STORE2 writes: the group's second output, its storage type (EwDType) and the flat index of acc[0].
struct Store2 {
  void* ptr;
  int dtype;
  long long i0;
  long long i1;  // VEC = 8 only: the flat index of acc[4] (the second vector)
};

template <int VEC>
__device__ __forceinline__ void store_second(const Store2& st, const float (&a)[VEC]) {
  if constexpr (VEC == 8) {
    store_second<4>(Store2{st.ptr, st.dtype, st.i0, 0}, *reinterpret_cast<const float(*)[4]>(&a[0]));
    store_second<4>(Store2{st.ptr, st.dtype, st.i1, 0}, *reinterpret_cast<const float(*)[4]>(&a[4]));
    return;
  }
  if (VEC == 4 && st.dtype == EW_F32) {
    __stcs(reinterpret_cast<uint4*>(static_cast<float*>(st.ptr) + st.i0), pack4(*reinterpret_cast<const float(*)[4]>(&a[0])));
  } else if (VEC == 4 && st.dtype == EW_F16) {
    __stcs(reinterpret_cast<uint2*>(static_cast<__half*>(st.ptr) + st.i0), make_uint2(pack_h2(a[0], a[1]), pack_h2(a[2], a[3])));
  } else if (VEC == 4 && st.dtype == EW_BF16) {
    __stcs(reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(st.ptr) + st.i0), make_uint2(pack_bf2(a[0], a[1]), pack_bf2(a[2], a[3])));
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (st.dtype == EW_F32) static_cast<float*>(st.ptr)[st.i0 + i] = a[i];
      else if (st.dtype == EW_F16) static_cast<__half*>(st.ptr)[st.i0 + i] = __float2half_rn(a[i]);
      else if (st.dtype == EW_BF16) static_cast<__nv_bfloat16*>(st.ptr)[st.i0 + i] = __float2bfloat16_rn(a[i]);
      else static_cast<uint8_t*>(st.ptr)[st.i0 + i] = a[i] != 0.0f ? 1 : 0;
    }
  }
}

// Operand of a step by its selector: 0 the immediate, 1..3 a side input, 4 the chain value, 5 / 6 a temporary.
template <int VEC, int NS, int NT>
__device__ __forceinline__ void pick_operand(int sel, float imm, const float (&s1)[VEC], const float (&s2)[VEC],
                                             const float (&s3)[VEC], const float (&acc)[VEC],
                                             const float (&ta)[NT > 0 ? VEC : 1], const float (&tb)[NT > 0 ? VEC : 1],
                                             float (&o)[VEC]) {
  switch (sel) {  // one uniform branch per step instead of a select chain per element
    case 1:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = NS >= 1 ? s1[i] : imm;
      break;
    case 2:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = NS >= 2 ? s2[i] : imm;
      break;
    case 3:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = NS >= 3 ? s3[i] : imm;
      break;
    case 4:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = acc[i];
      break;
    case 5:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = NT > 0 ? ta[NT > 0 ? i : 0] : imm;
      break;
    case 6:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = NT > 0 ? tb[NT > 0 ? i : 0] : imm;
      break;
    default:
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = imm;
      break;
  }
}

// ONE step of a chain program on VEC values.  op / asel / bsel / role are the fields of the step's word, imm its
// immediate and imm2 the immediate of the next word.  Returns true when the step used the next word as its second
// immediate (the caller then skips it).  The interpreter calls this with values decoded at run time; the kernels
// specialised at build time call it with constants, so that both execute the same arithmetic by construction.
// NT = 2: two temporaries (operand selectors 5 and 6, written by EW_STASH) for expression trees.
// ST2: the program may hold EW_STORE2 steps (st2 then says where they write).
template <int VEC, int NS, int NT, bool ST2, bool FAST = false, bool INL = false>
__device__ __forceinline__ bool chain_step(int op, int asel, int bsel, int role, float imm, float imm2,
                                           const float (&s1)[VEC], const float (&s2)[VEC], const float (&s3)[VEC],
                                           float (&acc)[VEC], float (&ta)[NT > 0 ? VEC : 1],
                                           float (&tb)[NT > 0 ? VEC : 1], const Store2* st2) {
  if (op == EW_NOP) return false;
  if (op >= EW_FIRST_UNARY) {
    apply_unary<VEC, FAST, INL>(op, imm, acc);
    return false;
  }
  if (ST2 && op == EW_STORE2) {
    if (st2) store_second<VEC>(*st2, acc);
    return false;
  }
  if (NT > 0 && op == EW_STASH) {
    if (asel == 5) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) ta[NT > 0 ? i : 0] = acc[i];
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) tb[NT > 0 ? i : 0] = acc[i];
    }
    return false;
  }
  float o[VEC];
  pick_operand<VEC, NS, NT>(asel, imm, s1, s2, s3, acc, ta, tb, o);
  if (op == EW_FMA) {
    // acc = fma(acc, A, B); B is a side operand, a temporary or the immediate of the next program slot.
    float b[VEC];
    pick_operand<VEC, NS, NT>(bsel == 4 ? 0 : bsel, imm2, s1, s2, s3, acc, ta, tb, b);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(acc[i], o[i], b[i]);
    return bsel == 0;
  }
  if (op == EW_SELECT) {
    // cinn/hlir/pe/elementwise.cc Select: cond ? true_value : false_value; the chain value is one of the three.
    // The operand and role decisions are uniform: they are taken once per step, outside the element loops.
    float b[VEC];
    pick_operand<VEC, NS, NT>(bsel, imm2, s1, s2, s3, acc, ta, tb, b);
    if (role == 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = acc[i] != 0.0f ? o[i] : b[i];
    } else if (role == 1) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = o[i] != 0.0f ? acc[i] : b[i];
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = o[i] != 0.0f ? b[i] : acc[i];
    }
    return bsel == 0;
  }
  if (op == EW_SCALE_PRE) {
    // imm * (acc + imm2): scale with bias_after_scale = false
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = imm * (acc[i] + imm2);
    return true;
  }
  apply_binary<VEC>(op, role != 0, o, acc);
  return false;
}

// The interpreter: decodes the program's words at run time.
template <int VEC, int NS, int NT = 0, bool ST2 = (NT > 0)>
__device__ __forceinline__ void run_chain(const long long* steps, int nsteps, const float (&s1)[VEC],
                                          const float (&s2)[VEC], const float (&s3)[VEC], float (&acc)[VEC],
                                          const Store2* st2 = nullptr) {
  float ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
  if (NT > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0.0f;
  }
  for (int k = 0; k < nsteps; ++k) {
    const long long st = steps[k];
    const float imm    = __uint_as_float((uint32_t)(st >> 32));
    const float imm2   = __uint_as_float((uint32_t)(steps[k + 1] >> 32));
    if (chain_step<VEC, NS, NT, ST2>((int)(st & 0xff), (int)((st >> 8) & 0xff), (int)((st >> 16) & 0xff),
                                     (int)((st >> 24) & 3), imm, imm2, s1, s2, s3, acc, ta, tb, st2))
      ++k;
  }
}

// The same program with its words' low halves (op, selectors, role) known at build time: SIG... are those 32-bit
// halves, the immediates still come from the kernel's parameters.  Every branch of chain_step folds away.
template <int VEC, int NS, int NT, bool ST2, bool FAST, int K, uint32_t... SIG>
__device__ __forceinline__ void run_chain_static_from(const long long* steps, const float (&s1)[VEC],
                                                      const float (&s2)[VEC], const float (&s3)[VEC],
                                                      float (&acc)[VEC], float (&ta)[NT > 0 ? VEC : 1],
                                                      float (&tb)[NT > 0 ? VEC : 1], const Store2* st2) {
  constexpr int N = (int)sizeof...(SIG);
  if constexpr (K < N) {
    constexpr uint32_t sig[N] = {SIG...};
    constexpr uint32_t w      = sig[K];
    constexpr int op = (int)(w & 0xff), asel = (int)((w >> 8) & 0xff), bsel = (int)((w >> 16) & 0xff),
                  role = (int)((w >> 24) & 3);
    // what chain_step would return, as a constant: the step reads the next word's immediate
    constexpr bool two = ((op == EW_FMA || op == EW_SELECT) && bsel == 0) || op == EW_SCALE_PRE;
    const float imm  = __uint_as_float((uint32_t)(steps[K] >> 32));
    const float imm2 = __uint_as_float((uint32_t)(steps[K + 1 < EW_MAX_STEPS ? K + 1 : K] >> 32));
    (void)chain_step<VEC, NS, NT, ST2, FAST, true>(op, asel, bsel, role, imm, imm2, s1, s2, s3, acc, ta, tb, st2);
    run_chain_static_from<VEC, NS, NT, ST2, FAST, K + (two ? 2 : 1), SIG...>(steps, s1, s2, s3, acc, ta, tb, st2);
  }
}
template <int VEC, int NS, int NT, bool ST2, bool FAST, uint32_t... SIG>
__device__ __forceinline__ void run_chain_static(const long long* steps, const float (&s1)[VEC],
                                                 const float (&s2)[VEC], const float (&s3)[VEC], float (&acc)[VEC],
                                                 const Store2* st2 = nullptr) {
  float ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
  if (NT > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0.0f;
  }
  run_chain_static_from<VEC, NS, NT, ST2, FAST, 0, SIG...>(steps, s1, s2, s3, acc, ta, tb, st2);
}
}  // namespace
}  // namespace cinn_b200
