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
    case EW_U8: return (double)static_cast<const uint8_t*>(p)[idx];
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
// One step of the program; returns true when the step also used the next word's immediate.
template <int VEC, int NS, int NT>
__device__ __forceinline__ bool d_chain_step(int op, int asel, int bsel, int role, double imm, double imm2,
                                             const double (&s1)[VEC], const double (&s2)[VEC], const double (&s3)[VEC],
                                             double (&acc)[VEC], double (&ta)[NT > 0 ? VEC : 1],
                                             double (&tb)[NT > 0 ? VEC : 1]) {
  if (op == EW_NOP) return false;
  if (op >= EW_FIRST_UNARY) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = d_unary(op, imm, acc[i]);
    return false;
  }
  if (NT > 0 && op == EW_STASH) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) (asel == 5 ? ta : tb)[NT > 0 ? i : 0] = acc[i];
    return false;
  }
  double o[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    o[i] = (NS >= 1 && asel == 1) ? s1[i] : ((NS >= 2 && asel == 2) ? s2[i] : ((NS >= 3 && asel == 3) ? s3[i] : (asel == 4 ? acc[i] : imm)));
    if (NT > 0) o[i] = asel == 5 ? ta[NT > 0 ? i : 0] : (asel == 6 ? tb[NT > 0 ? i : 0] : o[i]);
  }
  if (op == EW_FMA) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      double b = (NS >= 1 && bsel == 1) ? s1[i] : ((NS >= 2 && bsel == 2) ? s2[i] : ((NS >= 3 && bsel == 3) ? s3[i] : imm2));
      if (NT > 0) b = bsel == 5 ? ta[NT > 0 ? i : 0] : (bsel == 6 ? tb[NT > 0 ? i : 0] : b);
      acc[i] = fma(acc[i], o[i], b);
    }
    return bsel == 0;
  }
  if (op == EW_SCALE_PRE) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = imm * (acc[i] + imm2);
    return true;
  }
  if (op == EW_SELECT) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      double b = (NS >= 1 && bsel == 1) ? s1[i] : ((NS >= 2 && bsel == 2) ? s2[i] : ((NS >= 3 && bsel == 3) ? s3[i] : (bsel == 4 ? acc[i] : imm2)));
      if (NT > 0) b = bsel == 5 ? ta[NT > 0 ? i : 0] : (bsel == 6 ? tb[NT > 0 ? i : 0] : b);
      const double c = role == 0 ? acc[i] : o[i];
      const double t = role == 0 ? o[i] : (role == 1 ? acc[i] : b);
      const double f = role == 2 ? acc[i] : b;
      acc[i]         = c != 0.0 ? t : f;
    }
    return bsel == 0;
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i)
    acc[i] = (role != 0 && op != EW_COPY) ? d_binary(op, o[i], acc[i]) : d_binary(op, acc[i], o[i]);
  return false;
}

// The program read from the kernel's parameters at run time.
struct DynF64Program {
  const long long* steps;
  int nsteps;
  long long meta_;
  const double* imms;
  __device__ __forceinline__ long long meta() const { return meta_; }
  template <int VEC, int NS, int NT>
  __device__ __forceinline__ void run(const double (&s1)[VEC], const double (&s2)[VEC], const double (&s3)[VEC],
                                      double (&acc)[VEC]) const {
    double ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
    if (NT > 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0.0;
    }
    for (int k = 0; k < nsteps; ++k) {
      const long long st = steps[k];
      const double imm   = imms[(int)(st >> 32) & (kMaxImm - 1)];
      const double imm2  = imms[(int)(steps[k + 1] >> 32) & (kMaxImm - 1)];
      if (d_chain_step<VEC, NS, NT>((int)(st & 0xff), (int)((st >> 8) & 0xff), (int)((st >> 16) & 0xff),
                                    (int)((st >> 24) & 3), imm, imm2, s1, s2, s3, acc, ta, tb))
        ++k;
    }
  }
};

// Entry `idx` of the immediates without indexing the array at run time (which would move it to local memory).
__device__ __forceinline__ double pick_imm(const double* imms, int idx) {
  const double a = (idx & 1) ? imms[1] : imms[0], b = (idx & 1) ? imms[3] : imms[2];
  const double c = (idx & 1) ? imms[5] : imms[4], d = (idx & 1) ? imms[7] : imms[6];
  const double ab = (idx & 2) ? b : a, cd = (idx & 2) ? d : c;
  return (idx & 4) ? cd : ab;
}

// The program fixed at build time: META and the low halves of the step words (op, selectors, role) are template
// constants; which immediate a step takes still comes from the parameters.
template <unsigned long long META, uint32_t... SIG>
struct StaticF64Program {
  const long long* steps;
  const double* imms;
  static constexpr int kSteps = (int)sizeof...(SIG);
  __host__ __device__ static constexpr uint32_t word(int k) {
    constexpr uint32_t w[kSteps + 1] = {SIG..., 0u};
    return w[k < kSteps ? k : kSteps];
  }
  __host__ __device__ static constexpr bool uses_imm(int k) {
    const uint32_t w = word(k);
    const int op = (int)(w & 0xff), asel = (int)((w >> 8) & 0xff);
    return op >= EW_FIRST_UNARY || op == EW_SCALE_PRE || asel == 0;
  }
  __host__ __device__ static constexpr bool uses_next(int k) {
    const uint32_t w = word(k);
    const int op = (int)(w & 0xff), bsel = (int)((w >> 16) & 0xff);
    return op == EW_SCALE_PRE || ((op == EW_FMA || op == EW_SELECT) && bsel == 0);
  }
  __device__ __forceinline__ long long meta() const { return (long long)META; }
  template <int VEC, int NS, int NT, int K>
  __device__ __forceinline__ void from(const double (&s1)[VEC], const double (&s2)[VEC], const double (&s3)[VEC],
                                       double (&acc)[VEC], double (&ta)[NT > 0 ? VEC : 1],
                                       double (&tb)[NT > 0 ? VEC : 1]) const {
    if constexpr (K < kSteps) {
      constexpr uint32_t w = word(K);
      const double imm  = uses_imm(K) ? pick_imm(imms, (int)(steps[K] >> 32)) : 0.0;
      const double imm2 = uses_next(K) ? pick_imm(imms, (int)(steps[K + 1 < EW_MAX_STEPS ? K + 1 : K] >> 32)) : 0.0;
      (void)d_chain_step<VEC, NS, NT>((int)(w & 0xff), (int)((w >> 8) & 0xff), (int)((w >> 16) & 0xff),
                                      (int)((w >> 24) & 3), imm, imm2, s1, s2, s3, acc, ta, tb);
      from<VEC, NS, NT, K + (uses_next(K) ? 2 : 1)>(s1, s2, s3, acc, ta, tb);
    }
  }
  template <int VEC, int NS, int NT>
  __device__ __forceinline__ void run(const double (&s1)[VEC], const double (&s2)[VEC], const double (&s3)[VEC],
                                      double (&acc)[VEC]) const {
    double ta[NT > 0 ? VEC : 1], tb[NT > 0 ? VEC : 1];
    if (NT > 0) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) ta[i] = tb[i] = 0.0;
    }
    from<VEC, NS, NT, 0>(s1, s2, s3, acc, ta, tb);
  }
};

// The fp32 form's parameter list followed by the table of double immediates.
#define F64_CHAIN_PARAMS                                                                                              \
  const void *__restrict__ in0, const void *__restrict__ p1, const void *__restrict__ p2, const void *__restrict__ p3, \
      OutT *__restrict__ out, long long n, long long vec_ok, long long meta_ll, long long mid1, long long inner1,    \
      long long mid2, long long inner2, long long mid3, long long inner3, long long nsteps_ll, long long t0,         \
      long long t1, long long t2, long long t3, long long t4, long long t5, long long t6, long long t7, long long t8, \
      long long t9, long long t10, long long t11, long long t12, long long t13, long long t14, long long t15,        \
      double d0, double d1, double d2, double d3, double d4, double d5, double d6, double d7
#define F64_CHAIN_TABLES                                                                                              \
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0}; \
  const double imms[kMaxImm]              = {d0, d1, d2, d3, d4, d5, d6, d7}

struct F64Geometry {
  long long n, vec_ok, mid1, inner1, mid2, inner2, mid3, inner3;
};

template <typename OutT, int NS, int NT, class Prog>
__device__ __forceinline__ void f64_chain_body(const Prog& prog, const void* in0, const void* p1, const void* p2,
                                               const void* p3, OutT* out, const F64Geometry& geo) {
  const long long meta = prog.meta(), n = geo.n;
  const int in_type = (int)((meta >> 24) & 15);
  const SideSpec sd1 = {p1, (int)(meta & 15), (int)((meta >> 4) & 15), geo.mid1, geo.inner1};
  const SideSpec sd2 = {p2, (int)((meta >> 8) & 15), (int)((meta >> 12) & 15), geo.mid2, geo.inner2};
  const SideSpec sd3 = {p3, (int)((meta >> 16) & 15), (int)((meta >> 20) & 15), geo.mid3, geo.inner3};
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (geo.vec_ok) {
    const long long nvec = n >> 2;
    for (long long v = tid; v < nvec; v += stride) {
      const long long i0 = v << 2;
      double acc[4], s1[4], s2[4], s3[4];
      if (in_type != EW_NO_INPUT) load_d4(in0, in_type, i0, true, acc);
      if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, s1);
      if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, s2);
      if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, s3);
      prog.template run<4, NS, NT>(s1, s2, s3, acc);
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
    prog.template run<1, NS, NT>(s1, s2, s3, acc);
    out[i] = out_of<OutT>(acc[0]);
  }
}

template <typename OutT, int NS, int NT = 0>
__global__ void __launch_bounds__(256) k_ew_chain_f64(F64_CHAIN_PARAMS) {
  grid_dependency_sync();
  F64_CHAIN_TABLES;
  const DynF64Program prog = {steps, (int)nsteps_ll, meta_ll, imms};
  f64_chain_body<OutT, NS, NT>(prog, in0, p1, p2, p3, out, F64Geometry{n, vec_ok, mid1, inner1, mid2, inner2, mid3, inner3});
}

// The same with the program fixed at build time (see ew_static.cu for the scheme).
template <typename OutT, int NS, int NT, unsigned long long META, uint32_t... SIG>
__global__ void __launch_bounds__(256) k_ew_chain_f64_static(F64_CHAIN_PARAMS) {
  grid_dependency_sync();
  F64_CHAIN_TABLES;
  const StaticF64Program<META, SIG...> prog = {steps, imms};
  f64_chain_body<OutT, NS, NT>(prog, in0, p1, p2, p3, out, F64Geometry{n, vec_ok, mid1, inner1, mid2, inner2, mid3, inner3});
}

template <uint32_t... SIG>
StaticChainKey MakeF64Key(const char* base, long long meta) {
  StaticChainKey k = {base, meta, (int)sizeof...(SIG), {SIG...}};
  return k;
}

}  // namespace

#define REG_F64_CHAIN(NSNAME, NS)                                                                  \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_f64_f64_" NSNAME, 39, 256, k_ew_chain_f64<double, NS>);     \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_f64_f32_" NSNAME, 39, 256, k_ew_chain_f64<float, NS>);      \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_f64_bool_" NSNAME, 39, 256, k_ew_chain_f64<uint8_t, NS>)
REG_F64_CHAIN("s0", 0);
REG_F64_CHAIN("s1", 1);
REG_F64_CHAIN("s3", 3);
CINN_B200_REGISTER_KERNEL_PDL("ew_chain_f64_f64_s3t", 39, 256, k_ew_chain_f64<double, 3, 2>);
CINN_B200_REGISTER_KERNEL_PDL("ew_chain_f64_f32_s3t", 39, 256, k_ew_chain_f64<float, 3, 2>);
CINN_B200_REGISTER_KERNEL_PDL("ew_chain_f64_bool_s3t", 39, 256, k_ew_chain_f64<uint8_t, 3, 2>);


#define STATIC_F64_CHAIN(ID, BASE, OutT, NS, NT, META, ...)                                                        \
  CINN_B200_REGISTER_KERNEL_PDL("ew_f64_static_" #ID, 39, 256, k_ew_chain_f64_static<OutT, NS, NT, META##ull, __VA_ARGS__>); \
  static int cinn_b200_static_f64_chain_##ID = RegisterStaticChain(MakeF64Key<__VA_ARGS__>(BASE, META##ll), "ew_f64_static_" #ID)
#include "ew_f64_static_table.inc"

}  // namespace cinn_b200
