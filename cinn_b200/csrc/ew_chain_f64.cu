// float64 form of the generic elementwise chain (ew_chain.cu is the fp32 form, ew_chain.h the program encoding).
// The chain value and its operands are doubles; bool travels as 0.0 / 1.0.  A 32-bit field cannot hold a double,
// so the immediate field of a word is an index into a table of eight doubles passed after the program words.
// Arithmetic follows the same x86 rules as the fp32 form, in double precision: tanh / sigmoid / sinh / cosh / tan
// composed from exp, sin, cos (cinn/backends/llvm/llvm_intrin_rule.h:105-175), rsqrt = 1 / sqrt, max / min as
// compare + select, Mul followed by Add as one fused multiply-add (cinn/optim/lower_intrin.cc:41-59).
#include <cstdint>

#include "device_math.cuh"
#include "ew_chain.h"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

constexpr int kMaxImm = 8;

__device__ __noinline__ double d_unary_heavy(int op, double x) {
  switch (op) {
    case EW_EXP: return exp(x);
    case EW_TANH:
      if (x >= 0.0) {
        const double e = exp(-2.0 * x);
        return (1.0 - e) / (1.0 + e);
      } else {
        const double e = exp(2.0 * x);
        return (e - 1.0) / (e + 1.0);
      }
    case EW_SIGMOID: return 1.0 / (1.0 + exp(-x));
    case EW_LOG: return log(x);
    case EW_ERF: return erf(x);
    case EW_SIN: return sin(x);
    case EW_COS: return cos(x);
    case EW_LOG2: return log2(x);
    case EW_LOG10: return log10(x);
    case EW_TAN: return sin(x) / cos(x);
    case EW_SINH: return (exp(x) - exp(x * -1.0)) / 2.0;
    case EW_COSH: return (exp(x) + exp(x * -1.0)) / 2.0;
    case EW_ASIN: return asin(x);
    case EW_ACOS: return acos(x);
    case EW_ATAN: return atan(x);
    case EW_ASINH: return asinh(x);
    case EW_ACOSH: return acosh(x);
    case EW_ATANH: return atanh(x);
    case EW_CBRT: return cbrt(x);
    default: return x;
  }
}

__device__ __forceinline__ double d_unary(int op, double imm, double x) {
  const double inf = __longlong_as_double(0x7ff0000000000000ll);
  switch (op) {
    case EW_RSQRT: return 1.0 / sqrt(x);
    case EW_SQRT: return sqrt(x);
    case EW_RELU: return x > 0.0 ? x : 0.0;
    case EW_NEG: return -x;
    case EW_ABS: return fabs(x);
    case EW_FLOOR: return floor(x);
    case EW_CEIL: return ceil(x);
    case EW_RECIP: return 1.0 / x;
    case EW_ROUND: return nearbyint(x);
    case EW_TRUNC: return trunc(x);
    case EW_SIGN: return x < 0.0 ? -1.0 : (x > 0.0 ? 1.0 : (x == 0.0 ? 0.0 : x));
    case EW_RELU6: {
      const double r = x > 0.0 ? x : 0.0;
      return r < imm ? r : imm;
    }
    case EW_ISNAN: return x != x ? 1.0 : 0.0;
    case EW_ISINF: return (fabs(x) == inf && !(x != x)) ? 1.0 : 0.0;
    case EW_ISFINITE: return (fabs(x) == inf || x != x) ? 0.0 : 1.0;
    case EW_LNOT: return x == 0.0 ? 1.0 : 0.0;
    case EW_TO_BOOL: return x != 0.0 ? 1.0 : 0.0;
    case EW_IDENTITY: return x;
    default: return d_unary_heavy(op, x);
  }
}

__device__ __noinline__ double d_binary_heavy(int op, double l, double r) {
  switch (op) {
    case EW_POW: return pow(l, r);
    case EW_MOD: {
      double res = fmod(l, r);
      if ((res != 0.0) && ((res < 0.0) != (r < 0.0))) res += r;
      return res;
    }
    default: {  // EW_ATAN2, cinn/hlir/pe/broadcast.cc:275-291
      const double at = atan(l / r), pi = 3.14159265358979323846, half_pi = 3.14159265358979323846 / 2;
      if (r == 0.0) return l == 0.0 ? 0.0 : (l > 0.0 ? half_pi : -half_pi);
      return r > 0.0 ? at : (l >= 0.0 ? at + pi : at - pi);
    }
  }
}

__device__ __forceinline__ double d_binary(int op, double l, double r) {
  switch (op) {
    case EW_ADD: return l + r;
    case EW_SUB: return l - r;
    case EW_MUL: return l * r;
    case EW_DIV: return l / r;
    case EW_MAX: return l > r ? l : r;
    case EW_MIN: return l < r ? l : r;
    case EW_EQ: return l == r ? 1.0 : 0.0;
    case EW_NE: return l != r ? 1.0 : 0.0;
    case EW_GT: return l > r ? 1.0 : 0.0;
    case EW_LT: return l < r ? 1.0 : 0.0;
    case EW_GE: return l >= r ? 1.0 : 0.0;
    case EW_LE: return l <= r ? 1.0 : 0.0;
    case EW_FLOOR_DIV: return floor(l / r);
    case EW_LAND: return (l != 0.0 && r != 0.0) ? 1.0 : 0.0;
    case EW_LOR: return (l != 0.0 || r != 0.0) ? 1.0 : 0.0;
    case EW_LXOR: return ((l != 0.0) != (r != 0.0)) ? 1.0 : 0.0;
    case EW_COPY: return r;
    default: return d_binary_heavy(op, l, r);
  }
}

__device__ __forceinline__ double load_d(const void* p, int dtype, long long idx) {
  switch (dtype) {
    case EW_F64: return static_cast<const double*>(p)[idx];
    case EW_F32: return (double)static_cast<const float*>(p)[idx];
    case EW_BOOL: return static_cast<const uint8_t*>(p)[idx] != 0 ? 1.0 : 0.0;
    case EW_I32: return (double)static_cast<const int32_t*>(p)[idx];
    default: return (double)static_cast<const long long*>(p)[idx];
  }
}

// Four consecutive elements starting at idx (idx % 4 == 0, pointer 16-byte aligned).
__device__ __forceinline__ void load_d4(const void* p, int dtype, long long idx, bool stream, double (&v)[4]) {
  if (dtype == EW_F64) {
    const double2* q = reinterpret_cast<const double2*>(static_cast<const double*>(p) + idx);
    const double2 a  = stream ? __ldcs(q) : __ldg(q);
    const double2 b  = stream ? __ldcs(q + 1) : __ldg(q + 1);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  } else if (dtype == EW_F32) {
    const float4* q = reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx);
    const float4 a  = stream ? __ldcs(q) : __ldg(q);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = load_d(p, dtype, idx + i);
  }
}

template <typename OutT>
__device__ __forceinline__ OutT out_of(double v);
template <> __device__ __forceinline__ double out_of<double>(double v) { return v; }
template <> __device__ __forceinline__ float out_of<float>(double v) { return (float)v; }
template <> __device__ __forceinline__ uint8_t out_of<uint8_t>(double v) { return v != 0.0; }

template <typename OutT>
__device__ __forceinline__ void store_d4(OutT* p, long long idx, const double (&v)[4]) {
  constexpr int kHalf = sizeof(OutT) == 8 ? 2 : 4;
  struct alignas(sizeof(OutT) * kHalf) Pack {
    OutT e[kHalf];
  };
#pragma unroll
  for (int h = 0; h < 4 / kHalf; ++h) {
    Pack pk;
#pragma unroll
    for (int i = 0; i < kHalf; ++i) pk.e[i] = out_of<OutT>(v[h * kHalf + i]);
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

template <int VEC>
__device__ __forceinline__ void load_side(const SideSpec& s, long long i0, double (&f)[VEC]) {
  if (VEC == 4 && s.mode == EW_SIDE_FULL) {
    load_d4(s.ptr, s.dtype, i0, true, *reinterpret_cast<double(*)[4]>(&f[0]));
  } else if (VEC == 4 && s.mode == EW_SIDE_PERIODIC_VEC) {
    load_d4(s.ptr, s.dtype, side_index(i0, 1, s.mid), false, *reinterpret_cast<double(*)[4]>(&f[0]));
  } else if (s.mode == EW_SIDE_ONE_PER_VEC || s.mode == EW_SIDE_SCALAR) {
    const double v = load_d(s.ptr, s.dtype, s.mode == EW_SIDE_SCALAR ? 0 : side_index(i0, s.inner, s.mid));
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = v;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) f[i] = load_d(s.ptr, s.dtype, side_index(i0 + i, s.inner, s.mid));
  }
}

// NS = how many side inputs the kernel variant carries (0, 1 or 3): the registers of absent sides are never touched.
// NT = 2: two temporaries (operand selectors 5 and 6, written by EW_STASH) for expression trees, as in the float form.
template <int VEC, int NS, int NT = 0>
__device__ __forceinline__ void run_chain(const long long* steps, int nsteps, const double* imms,
                                          const double (&s1)[VEC], const double (&s2)[VEC], const double (&s3)[VEC],
                                          double (&acc)[VEC]) {
  double ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
  if (NT > 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0.0;
  }
  for (int k = 0; k < nsteps; ++k) {
    const long long st = steps[k];
    const int op       = (int)(st & 0xff);
    const int asel     = (int)((st >> 8) & 0xff);
    const int bsel     = (int)((st >> 16) & 0xff);
    const int role     = (int)((st >> 24) & 3);
    const double imm   = imms[(int)(st >> 32) & (kMaxImm - 1)];
    if (op == EW_NOP) continue;
    if (op >= EW_FIRST_UNARY) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = d_unary(op, imm, acc[i]);
      continue;
    }
    if (NT > 0 && op == EW_STASH) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) (asel == 5 ? ta : tb)[NT > 0 ? i : 0] = acc[i];
      continue;
    }
    double o[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      o[i] = (NS >= 1 && asel == 1) ? s1[i] : ((NS >= 2 && asel == 2) ? s2[i] : ((NS >= 3 && asel == 3) ? s3[i] : (asel == 4 ? acc[i] : imm)));
      if (NT > 0) o[i] = asel == 5 ? ta[NT > 0 ? i : 0] : (asel == 6 ? tb[NT > 0 ? i : 0] : o[i]);
    }
    const double imm2 = imms[(int)(steps[k + 1] >> 32) & (kMaxImm - 1)];
    if (op == EW_FMA) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        double b = (NS >= 1 && bsel == 1) ? s1[i] : ((NS >= 2 && bsel == 2) ? s2[i] : ((NS >= 3 && bsel == 3) ? s3[i] : imm2));
        if (NT > 0) b = bsel == 5 ? ta[NT > 0 ? i : 0] : (bsel == 6 ? tb[NT > 0 ? i : 0] : b);
        acc[i] = fma(acc[i], o[i], b);
      }
      if (bsel == 0) ++k;
    } else if (op == EW_SCALE_PRE) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = imm * (acc[i] + imm2);
      ++k;
    } else if (op == EW_SELECT) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        double b = (NS >= 1 && bsel == 1) ? s1[i] : ((NS >= 2 && bsel == 2) ? s2[i] : ((NS >= 3 && bsel == 3) ? s3[i] : (bsel == 4 ? acc[i] : imm2)));
        if (NT > 0) b = bsel == 5 ? ta[NT > 0 ? i : 0] : (bsel == 6 ? tb[NT > 0 ? i : 0] : b);
        const double c = role == 0 ? acc[i] : o[i];
        const double t = role == 0 ? o[i] : (role == 1 ? acc[i] : b);
        const double f = role == 2 ? acc[i] : b;
        acc[i]         = c != 0.0 ? t : f;
      }
      if (bsel == 0) ++k;
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        acc[i] = (role != 0 && op != EW_COPY) ? d_binary(op, o[i], acc[i]) : d_binary(op, acc[i], o[i]);
    }
  }
}

// The fp32 form's parameter list followed by the table of double immediates.
template <typename OutT, int NS, int NT = 0>
__global__ void __launch_bounds__(256)
    k_ew_chain_f64(const void* __restrict__ in0, const void* __restrict__ p1, const void* __restrict__ p2,
                   const void* __restrict__ p3, OutT* __restrict__ out, long long n, long long vec_ok, long long meta,
                   long long mid1, long long inner1, long long mid2, long long inner2, long long mid3,
                   long long inner3, long long nsteps_ll, long long t0, long long t1, long long t2, long long t3,
                   long long t4, long long t5, long long t6, long long t7, long long t8, long long t9, long long t10,
                   long long t11, long long t12, long long t13, long long t14, long long t15, double d0, double d1,
                   double d2, double d3, double d4, double d5, double d6, double d7) {
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0};
  const double imms[kMaxImm]              = {d0, d1, d2, d3, d4, d5, d6, d7};
  const int nsteps  = (int)nsteps_ll;
  const int in_type = (int)((meta >> 24) & 15);
  const SideSpec sd1 = {p1, (int)(meta & 15), (int)((meta >> 4) & 15), mid1, inner1};
  const SideSpec sd2 = {p2, (int)((meta >> 8) & 15), (int)((meta >> 12) & 15), mid2, inner2};
  const SideSpec sd3 = {p3, (int)((meta >> 16) & 15), (int)((meta >> 20) & 15), mid3, inner3};
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (vec_ok) {
    const long long nvec = n >> 2;
    for (long long v = tid; v < nvec; v += stride) {
      const long long i0 = v << 2;
      double acc[4], s1[4], s2[4], s3[4];
      if (in_type != EW_NO_INPUT) load_d4(in0, in_type, i0, true, acc);
      if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, s1);
      if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, s2);
      if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, s3);
      run_chain<4, NS, NT>(steps, nsteps, imms, s1, s2, s3, acc);
      store_d4<OutT>(out, i0, acc);
    }
    done = nvec << 2;
  }
  for (long long i = done + tid; i < n; i += stride) {
    double acc[1], s1[1], s2[1], s3[1];
    acc[0] = in_type != EW_NO_INPUT ? load_d(in0, in_type, i) : 0.0;
    if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<1>(sd1, i, s1);
    if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<1>(sd2, i, s2);
    if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<1>(sd3, i, s3);
    run_chain<1, NS, NT>(steps, nsteps, imms, s1, s2, s3, acc);
    out[i] = out_of<OutT>(acc[0]);
  }
}

}  // namespace

#define REG_F64_CHAIN(NSNAME, NS)                                                                  \
  CINN_B200_REGISTER_KERNEL("ew_chain_f64_f64_" NSNAME, 39, 256, k_ew_chain_f64<double, NS>);     \
  CINN_B200_REGISTER_KERNEL("ew_chain_f64_f32_" NSNAME, 39, 256, k_ew_chain_f64<float, NS>);      \
  CINN_B200_REGISTER_KERNEL("ew_chain_f64_bool_" NSNAME, 39, 256, k_ew_chain_f64<uint8_t, NS>)
REG_F64_CHAIN("s0", 0);
REG_F64_CHAIN("s1", 1);
REG_F64_CHAIN("s3", 3);
CINN_B200_REGISTER_KERNEL("ew_chain_f64_f64_s3t", 39, 256, k_ew_chain_f64<double, 3, 2>);
CINN_B200_REGISTER_KERNEL("ew_chain_f64_f32_s3t", 39, 256, k_ew_chain_f64<float, 3, 2>);
CINN_B200_REGISTER_KERNEL("ew_chain_f64_bool_s3t", 39, 256, k_ew_chain_f64<uint8_t, 3, 2>);

}  // namespace cinn_b200
