// Generic elementwise / broadcast fused group: a linear chain of ops evaluated in registers, one HBM pass.
//
// This is the catch-all for kElementWise / kBroadcast groups that have no dedicated kernel: the group's
// expression is linearised by the matcher into a short program (at most 16 steps) that starts from one input
// ("the chain") and applies one op per step with, at most, side operands taken from up to three other inputs
// or immediates.  It covers what the reference generates for such groups after inlining
// (cinn/hlir/framework/op_lowering.cc:247-310) with the x86 path's arithmetic: unary math as in
// cinn/hlir/pe/elementwise.cc:33-108 and cinn/backends/llvm/llvm_intrin_rule.h, binary ops with the broadcast
// index rule of cinn/hlir/pe/broadcast.cc:35-273, scale (cinn/hlir/op/elementwise.cc:149-163), cast
// (cinn/hlir/pe/elementwise.cc:213-217) and the Mul+Add -> fma contraction of cinn/optim/lower_intrin.cc:41-59.
// The program is interpreted per 4-element vector; every thread of a warp takes the same branch, so the cost
// of the dispatch is shared by the vector.
#include "device_math.cuh"
#include "ew_chain.h"
#include "kernel_registry.h"

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
    default: return x;
  }
}
__device__ __noinline__ float heavy_pow(float l, float r) { return powf(l, r); }

template <int VEC>
__device__ __forceinline__ void apply_unary(int op, float imm, float (&a)[VEC]) {
#define EW_UNARY_CASE(code, expr) \
  case code:                      \
    _Pragma("unroll") for (int i = 0; i < VEC; ++i) { const float x = a[i]; a[i] = (expr); } \
    break;
  switch (op) {
    EW_UNARY_CASE(EW_EXP, expf(x))
    EW_UNARY_CASE(EW_TANH, x86_tanh(x))
    EW_UNARY_CASE(EW_SIGMOID, x86_sigmoid(x))
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
    case EW_ERF:
    case EW_SIN:
    case EW_COS:
    case EW_LOG2:
    case EW_LOG10:
#pragma unroll
      for (int i = 0; i < VEC; ++i) a[i] = heavy_unary(op, a[i]);
      break;
    default:
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
    default:
      break;
  }
#undef EW_BINARY_CASE
}

__device__ __forceinline__ float load_scalar(const void* p, int dtype, long long idx) {
  if (dtype == 0) return static_cast<const float*>(p)[idx];
  if (dtype == 1) return __half2float(static_cast<const __half*>(p)[idx]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

// Four consecutive elements starting at idx (idx % 4 == 0, pointer 16-byte aligned for fp32 / 8 for 16-bit).
__device__ __forceinline__ void load_vec4(const void* p, int dtype, long long idx, bool stream, float (&f)[4]) {
  if (dtype == 0) {
    const uint4* q = reinterpret_cast<const uint4*>(static_cast<const float*>(p) + idx);
    unpack4(stream ? __ldcs(q) : __ldg(q), f);
  } else {
    const uint2* q = reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + idx);
    uint2 u        = stream ? __ldcs(q) : __ldg(q);
    if (dtype == 1) {
      unpack_h2(u.x, f[0], f[1]);
      unpack_h2(u.y, f[2], f[3]);
    } else {
      unpack_bf2(u.x, f[0], f[1]);
      unpack_bf2(u.y, f[2], f[3]);
    }
  }
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
template <typename OutT>
__device__ __forceinline__ void store_one(OutT* p, long long idx, float v) {
  Io<OutT>::store1(p + idx, v);
}
template <>
__device__ __forceinline__ void store_one<uint8_t>(uint8_t* p, long long idx, float v) {
  p[idx] = v != 0.0f ? 1 : 0;
}

struct SideSpec {
  const void* ptr;
  int dtype, mode;
  long long mid, inner;
};

// (i / inner) % mid, in 32-bit arithmetic whenever the operands allow it (64-bit division is several times dearer).
__device__ __forceinline__ long long side_index(long long i, long long inner, long long mid) {
  if (((i | inner | mid) >> 31) == 0) return (long long)(((unsigned)i / (unsigned)inner) % (unsigned)mid);
  return (i / inner) % mid;
}

template <int VEC>
__device__ __forceinline__ void load_side(const SideSpec& s, long long i0, float (&f)[VEC]) {
  if (VEC == 4 && s.mode == EW_SIDE_FULL) {
    load_vec4(s.ptr, s.dtype, i0, true, *reinterpret_cast<float(*)[4]>(&f[0]));
  } else if (VEC == 4 && s.mode == EW_SIDE_PERIODIC_VEC) {
    load_vec4(s.ptr, s.dtype, side_index(i0, 1, s.mid), false, *reinterpret_cast<float(*)[4]>(&f[0]));
  } else if (s.mode == EW_SIDE_ONE_PER_VEC || s.mode == EW_SIDE_SCALAR) {
    const float v = load_scalar(s.ptr, s.dtype, s.mode == EW_SIDE_SCALAR ? 0 : side_index(i0, s.inner, s.mid));
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = v;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = load_scalar(s.ptr, s.dtype, side_index(i0 + i, s.inner, s.mid));
  }
}

template <int VEC>
__device__ __forceinline__ void run_chain(const long long* steps, int nsteps, const float (&s1)[VEC],
                                          const float (&s2)[VEC], const float (&s3)[VEC], float (&acc)[VEC]) {
  for (int k = 0; k < nsteps; ++k) {
    const long long st = steps[k];
    const int op       = (int)(st & 0xff);
    const int asel     = (int)((st >> 8) & 0xff);
    const int bsel     = (int)((st >> 16) & 0xff);
    const bool swap    = ((st >> 24) & 1) != 0;
    const float imm    = __uint_as_float((uint32_t)(st >> 32));
    if (op == EW_NOP) continue;
    if (op >= EW_FIRST_UNARY) {
      apply_unary<VEC>(op, imm, acc);
      continue;
    }
    float o[VEC];
    switch (asel) {  // one uniform branch per step instead of a select chain per element
      case 1:
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = s1[i];
        break;
      case 2:
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = s2[i];
        break;
      case 3:
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = s3[i];
        break;
      case 4:
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = acc[i];
        break;
      default:
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = imm;
        break;
    }
    if (op == EW_FMA) {
      // acc = fma(acc, A, B); B is a side operand or the immediate of the next program slot.
      const float imm2 = __uint_as_float((uint32_t)(steps[k + 1] >> 32));
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float b = bsel == 1 ? s1[i] : (bsel == 2 ? s2[i] : (bsel == 3 ? s3[i] : imm2));
        acc[i]        = fmaf(acc[i], o[i], b);
      }
      if (bsel == 0) ++k;
    } else if (op == EW_SCALE_PRE) {
      // imm * (acc + imm2): scale with bias_after_scale = false
      const float imm2 = __uint_as_float((uint32_t)(steps[k + 1] >> 32));
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = imm * (acc[i] + imm2);
      ++k;
    } else {
      apply_binary<VEC>(op, swap, o, acc);
    }
  }
}

template <typename InT>
struct DTypeCode;
template <>
struct DTypeCode<float> {
  static constexpr int v = 0;
};
template <>
struct DTypeCode<__half> {
  static constexpr int v = 1;
};
template <>
struct DTypeCode<__nv_bfloat16> {
  static constexpr int v = 2;
};

// meta: bits 0-3 dtype of side 1, 4-7 mode of side 1, 8-11 / 12-15 side 2, 16-19 / 20-23 side 3.
template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
    k_ew_chain(const InT* __restrict__ in0, const void* __restrict__ p1, const void* __restrict__ p2,
               const void* __restrict__ p3, OutT* __restrict__ out, long long n, long long vec_ok, long long meta,
               long long mid1, long long inner1, long long mid2, long long inner2, long long mid3, long long inner3,
               long long nsteps_ll, long long t0, long long t1, long long t2, long long t3, long long t4,
               long long t5, long long t6, long long t7, long long t8, long long t9, long long t10, long long t11,
               long long t12, long long t13, long long t14, long long t15) {
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0};
  const int nsteps = (int)nsteps_ll;
  const SideSpec sd1 = {p1, (int)(meta & 15), (int)((meta >> 4) & 15), mid1, inner1};
  const SideSpec sd2 = {p2, (int)((meta >> 8) & 15), (int)((meta >> 12) & 15), mid2, inner2};
  const SideSpec sd3 = {p3, (int)((meta >> 16) & 15), (int)((meta >> 20) & 15), mid3, inner3};
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (vec_ok) {
    const long long nvec = n >> 2;
    // Two vectors (8 elements) per thread iteration: all of their loads are issued before the program runs,
    // and one pass of the interpreter serves the eight elements.
    long long v = tid;
    for (; v + stride < nvec; v += 2 * stride) {
      float acc[8], s1[8], s2[8], s3[8];
#pragma unroll
      for (int j = 0; j < 2; ++j)
        load_vec4(in0, DTypeCode<InT>::v, (v + j * stride) << 2, true, *reinterpret_cast<float(*)[4]>(&acc[4 * j]));
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const long long i0 = (v + j * stride) << 2;
        if (sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, *reinterpret_cast<float(*)[4]>(&s1[4 * j]));
        if (sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, *reinterpret_cast<float(*)[4]>(&s2[4 * j]));
        if (sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, *reinterpret_cast<float(*)[4]>(&s3[4 * j]));
      }
      run_chain<8>(steps, nsteps, s1, s2, s3, acc);
#pragma unroll
      for (int j = 0; j < 2; ++j)
        store_vec4<OutT>(out, (v + j * stride) << 2, *reinterpret_cast<float(*)[4]>(&acc[4 * j]));
    }
    for (; v < nvec; v += stride) {
      const long long i0 = v << 2;
      float acc[4], s1[4], s2[4], s3[4];
      load_vec4(in0, DTypeCode<InT>::v, i0, true, acc);
      if (sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, s1);
      if (sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, s2);
      if (sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, s3);
      run_chain<4>(steps, nsteps, s1, s2, s3, acc);
      store_vec4<OutT>(out, i0, acc);
    }
    done = nvec << 2;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float acc[1], s1[1], s2[1], s3[1];
    acc[0] = load_scalar(in0, DTypeCode<InT>::v, i);
    if (sd1.mode != EW_SIDE_NONE) load_side<1>(sd1, i, s1);
    if (sd2.mode != EW_SIDE_NONE) load_side<1>(sd2, i, s2);
    if (sd3.mode != EW_SIDE_NONE) load_side<1>(sd3, i, s3);
    run_chain<1>(steps, nsteps, s1, s2, s3, acc);
    store_one<OutT>(out, i, acc[0]);
  }
}

}  // namespace

#define REG_CHAIN(INNAME, InT, OUTNAME, OutT) \
  CINN_B200_REGISTER_KERNEL("ew_chain_" INNAME "_" OUTNAME, 31, 256, k_ew_chain<InT, OutT>)
#define REG_CHAIN_IN(INNAME, InT)            \
  REG_CHAIN(INNAME, InT, "f32", float);      \
  REG_CHAIN(INNAME, InT, "f16", __half);     \
  REG_CHAIN(INNAME, InT, "bf16", __nv_bfloat16); \
  REG_CHAIN(INNAME, InT, "bool", uint8_t)

REG_CHAIN_IN("f32", float);
REG_CHAIN_IN("f16", __half);
REG_CHAIN_IN("bf16", __nv_bfloat16);

}  // namespace cinn_b200
