/*
 * CPU restatement of the arithmetic that CINN's x86 path (DefaultHostTarget:
 * CINN IR -> LowerIntrin -> CodeGenX86 -> LLVM -O3 without fast-math) performs
 * for elementwise, broadcast and reduction fused groups.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the GPU kernels are
 * compared against and the CPU baseline that the benchmark times.  Nothing in
 * the product library calls it.
 *
 * Parity status: the reference cannot be built or imported offline (it needs
 * LLVM 11, isl, glog, ... fetched at configure time) and it stores no golden
 * numeric vectors for this path, so the arithmetic here is pinned only by the
 * known-answer relations the reference's own tests use (libm closeness 1e-5,
 * A+(A+B)==2A+B, serial-loop batch-norm and reduce references) and, for the
 * LLVM -O3 behaviour, by JIT-compiling the IR the reference would emit with
 * llvmlite in the development container.  "parity unpinned" against the
 * reference's own x86 output.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -mfma -mf16c -fopenmp -shared -fPIC
 * (-ffp-contract=off so that a*b+c is fused ONLY where fmaf is written, which is
 * exactly where the reference creates llvm.fmuladd).
 *
 * Rules followed (file:line are paths inside the reference project):
 *  - float Add with a Mul operand -> fused multiply-add      cinn/optim/lower_intrin.cc:41-59
 *  - tanh(x) = x>=0 ? (1-e^-2x)/(1+e^-2x) : (e^2x-1)/(e^2x+1) cinn/backends/llvm/llvm_intrin_rule.h:136-154
 *  - rsqrt(x) = 1/sqrt(x)                                     cinn/backends/llvm/llvm_intrin_rule.h:105-113
 *  - sigmoid(x) = 1/(1+exp(-x))                               cinn/lang/builtin.h:79-82
 *  - exp/log/sqrt/floor/ceil... -> LLVM intrinsics -> libm    cinn/backends/llvm/llvm_intrin_rule.h:48-63
 *  - max(a,b) = a>b ? a : b ; min(a,b) = a<b ? a : b           cinn/backends/llvm/codegen_llvm.cc:310-340
 *  - relu(x) = max(x, 0)                                       cinn/lang/builtin.h:106-108, cinn/hlir/pe/nn.cc:61-64
 *  - scale: s*x+b (bias_after_scale) or s*(x+b)                cinn/hlir/op/elementwise.cc:149-163
 *  - casts are fptrunc/fpext, round-to-nearest-even            cinn/backends/llvm/codegen_llvm.cc:454-455
 *  - reductions: acc = acc (op) x in increasing index order,
 *    init 0 / lowest(), accumulator in the tensor's dtype      cinn/ir/tensor.cc:325-349, cinn/lang/builtin.cc:123-143
 *  - batch_norm: (x-mean)*scale/sqrt(var+eps)+bias             cinn/hlir/pe/nn.cc:700-721
 *  - softmax: exp(x)/sum_j exp(x_j), no max subtraction        cinn/hlir/pe/nn.cc:755-796
 *  - layer_norm composition                                    cinn/frontend/op_mappers/paddle/layer_norm.cc:84-139
 */
#include <float.h>
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

typedef uint16_t f16bits;

/* fptrunc / fpext (codegen_llvm.cc:454-455): IEEE round-to-nearest-even via F16C. */
static inline f16bits f32_to_f16(float v) { return (f16bits)_cvtss_sh(v, _MM_FROUND_TO_NEAREST_INT); }
static inline float f16_to_f32(f16bits h) { return _cvtsh_ss(h); }

/* bfloat16 <-> float: fptrunc to bf16 is round-to-nearest-even on the upper 16 bits. */
static inline uint16_t f32_to_bf16(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); /* quiet NaN */
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float v;
  memcpy(&v, &u, 4);
  return v;
}

static inline float x86_max(float a, float b) { return a > b ? a : b; } /* fcmp ogt + select */
static inline float x86_min(float a, float b) { return a < b ? a : b; } /* fcmp olt + select */

/* llvm_intrin_rule.h:136-154 */
static inline float x86_tanh(float x) {
  if (x >= 0.0f) {
    float e = expf(-2.0f * x);
    return (1.0f - e) / (1.0f + e);
  } else {
    float e = expf(2.0f * x);
    return (e - 1.0f) / (e + 1.0f);
  }
}
/* llvm_intrin_rule.h:105-113 */
static inline float x86_rsqrt(float x) { return 1.0f / sqrtf(x); }
/* builtin.h:79-82 */
static inline float x86_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------------------------------
 * Op-at-a-time evaluators.  An operand is addressed as p[(i / inner) % mid] for flat output index i:
 * a full-size operand has mid = n, inner = 1; a vector broadcast on the last axis has mid = its
 * length, inner = 1; a per-channel vector of an NCHW tensor has mid = C, inner = H*W; a scalar has
 * mid = 1.  This is the index subset rule of pe::Broadcast (cinn/hlir/pe/broadcast.cc:35-239).
 * ---------------------------------------------------------------------------------------------- */
static inline int64_t bidx(int64_t i, int64_t mid, int64_t inner) { return (i / inner) % mid; }

enum {
  ORC_EXP = 0, ORC_TANH, ORC_SIGMOID, ORC_RSQRT, ORC_SQRT, ORC_RELU, ORC_NEG, ORC_ABS, ORC_IDENTITY, ORC_LOG,
  ORC_FLOOR, ORC_CEIL, ORC_ERF, ORC_SIN, ORC_COS, ORC_RECIPROCAL, ORC_ROUND, ORC_TRUNC, ORC_LOG2, ORC_LOG10,
  ORC_SIGN
};

static inline float unary1(int op, float x) {
  switch (op) {
    case ORC_EXP: return expf(x);
    case ORC_TANH: return x86_tanh(x);
    case ORC_SIGMOID: return x86_sigmoid(x);
    case ORC_RSQRT: return x86_rsqrt(x);
    case ORC_SQRT: return sqrtf(x);
    case ORC_RELU: return x86_max(x, 0.0f);
    case ORC_NEG: return -x;
    case ORC_ABS: return fabsf(x);
    case ORC_IDENTITY: return x;
    case ORC_LOG: return logf(x);
    case ORC_FLOOR: return floorf(x);
    case ORC_CEIL: return ceilf(x);
    case ORC_ERF: return erff(x);  /* cinn/optim/map_extern_call.cc:42-74 -> host erff */
    case ORC_SIN: return sinf(x);
    case ORC_COS: return cosf(x);
    case ORC_RECIPROCAL: return 1.0f / x; /* cinn/hlir/op/elementwise.cc reciprocal: 1/x */
    case ORC_ROUND: return nearbyintf(x); /* llvm.nearbyint, llvm_intrin_rule.h:48-63 */
    case ORC_TRUNC: return truncf(x);
    case ORC_LOG2: return log2f(x);
    case ORC_LOG10: return log10f(x);
    case ORC_SIGN: return x < 0.0f ? -1.0f : (x > 0.0f ? 1.0f : (x == 0.0f ? 0.0f : x)); /* builtin.h:84-92 */
    default: return NAN;
  }
}

int orc_unary_f32(int op, const float* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = unary1(op, x[i]);
  return 0;
}

enum { ORC_ADD = 0, ORC_SUB, ORC_MUL, ORC_DIV, ORC_MAX, ORC_MIN, ORC_POW };

static inline float binary1(int op, float a, float b) {
  switch (op) {
    case ORC_ADD: return a + b;
    case ORC_SUB: return a - b;
    case ORC_MUL: return a * b;
    case ORC_DIV: return a / b;
    case ORC_MAX: return x86_max(a, b);
    case ORC_MIN: return x86_min(a, b);
    case ORC_POW: return powf(a, b);
    default: return NAN;
  }
}

int orc_binary_f32(int op, const float* a, int64_t a_mid, int64_t a_inner, const float* b, int64_t b_mid,
                   int64_t b_inner, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = binary1(op, a[bidx(i, a_mid, a_inner)], b[bidx(i, b_mid, b_inner)]);
  return 0;
}

/* y = fma(a, b, c): the result of lower_intrin.cc:41-59 on Add(Mul(a,b), c) or Add(c, Mul(a,b)). */
int orc_fma_f32(const float* a, int64_t a_mid, int64_t a_inner, const float* b, int64_t b_mid, int64_t b_inner,
                const float* c, int64_t c_mid, int64_t c_inner, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i)
    y[i] = fmaf(a[bidx(i, a_mid, a_inner)], b[bidx(i, b_mid, b_inner)], c[bidx(i, c_mid, c_inner)]);
  return 0;
}

/* scale op, cinn/hlir/op/elementwise.cc:149-163; the bias_after_scale form is Add(Mul,..) => fma. */
int orc_scale_f32(const float* x, float scale, float bias, int bias_after_scale, float* y, int64_t n) {
  if (bias_after_scale) {
    for (int64_t i = 0; i < n; ++i) y[i] = fmaf(scale, x[i], bias);
  } else {
    for (int64_t i = 0; i < n; ++i) y[i] = scale * (x[i] + bias);
  }
  return 0;
}

int orc_cast_f32_f16(const float* x, f16bits* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = f32_to_f16(x[i]);
  return 0;
}
int orc_cast_f16_f32(const f16bits* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = f16_to_f32(x[i]);
  return 0;
}
int orc_cast_f32_bf16(const float* x, uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = f32_to_bf16(x[i]);
  return 0;
}
int orc_cast_bf16_f32(const uint16_t* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) y[i] = bf16_to_f32(x[i]);
  return 0;
}

/* ------------------------------------------------------------------------------------------------
 * Reductions over the middle axis of a tensor viewed as [outer, r, inner] -> [outer, inner].
 * Serial, increasing index, accumulator fp32 (cinn/ir/tensor.cc:325-349; init values
 * cinn/lang/builtin.cc:123-143: 0 for sum, 1 for prod, lowest()/max() for max/min).
 * `threads` > 1 splits OUTPUT elements over OpenMP threads; each output keeps its serial order,
 * so the result does not depend on the thread count.
 * ---------------------------------------------------------------------------------------------- */
enum { ORC_RSUM = 0, ORC_RPROD, ORC_RMAX, ORC_RMIN };

int orc_reduce_f32(int kind, const float* x, int64_t outer, int64_t r, int64_t inner, float* y, int threads) {
  const int64_t nout = outer * inner;
  if (kind < 0 || kind > ORC_RMIN) return -1;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t o = 0; o < nout; ++o) {
    const int64_t oo = o / inner, ii = o % inner;
    const float* p   = x + oo * r * inner + ii;
    float acc;
    switch (kind) {
      case ORC_RSUM:
        acc = 0.0f;
        for (int64_t k = 0; k < r; ++k) acc = acc + p[k * inner];
        break;
      case ORC_RPROD:
        acc = 1.0f;
        for (int64_t k = 0; k < r; ++k) acc = acc * p[k * inner];
        break;
      case ORC_RMAX:
        acc = -FLT_MAX;
        for (int64_t k = 0; k < r; ++k) acc = x86_max(acc, p[k * inner]);
        break;
      default:
        acc = FLT_MAX;
        for (int64_t k = 0; k < r; ++k) acc = x86_min(acc, p[k * inner]);
        break;
    }
    y[o] = acc;
  }
  return 0;
}

/* Arbiter for the reduction tolerance: the same sum with a double accumulator, result in double. */
int orc_reduce_sum_f64acc(const float* x, int64_t outer, int64_t r, int64_t inner, double* y, int threads) {
  const int64_t nout = outer * inner;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t o = 0; o < nout; ++o) {
    const int64_t oo = o / inner, ii = o % inner;
    const float* p   = x + oo * r * inner + ii;
    double acc       = 0.0;
    for (int64_t k = 0; k < r; ++k) acc += (double)p[k * inner];
    y[o] = acc;
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------------
 * Fused single-pass loops for the benchmark groups: what LLVM compiles after every producer in the
 * group has been inlined into the output expression.  Used as the timed CPU baseline and
 * cross-checked in the tests against the op-at-a-time evaluators above.
 * ---------------------------------------------------------------------------------------------- */

/* relu(A+B), fp32. */
int orc_add_relu_f32(const float* a, const float* b, float* y, int64_t n, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t i = 0; i < n; ++i) y[i] = x86_max(a[i] + b[i], 0.0f);
  return 0;
}

/* cast_fp16(tanh(scale*(X + bias[col]) + shift)), bias broadcast on the last axis of length `cols`. */
int orc_bias_scale_tanh_f16(const float* x, const float* bias, int64_t rows, int64_t cols, float scale, float shift,
                            f16bits* y, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    f16bits* yr     = y + r * cols;
    for (int64_t c = 0; c < cols; ++c) {
      float t = fmaf(scale, xr[c] + bias[c], shift);
      yr[c]   = f32_to_f16(x86_tanh(t));
    }
  }
  return 0;
}

/* softmax along the last axis, fp32 I/O: exp(x)/sum exp(x) (pe/nn.cc:755-796). */
int orc_softmax_f32(const float* x, int64_t rows, int64_t cols, float* y, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr       = y + r * cols;
    float s         = 0.0f;
    for (int64_t c = 0; c < cols; ++c) s = s + expf(xr[c]);
    for (int64_t c = 0; c < cols; ++c) yr[c] = expf(xr[c]) / s;
  }
  return 0;
}

/* fp16 I/O: cast to fp32, fp32 softmax, cast back. */
int orc_softmax_f16(const f16bits* x, int64_t rows, int64_t cols, f16bits* y, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t r = 0; r < rows; ++r) {
    const f16bits* xr = x + r * cols;
    f16bits* yr       = y + r * cols;
    float s           = 0.0f;
    for (int64_t c = 0; c < cols; ++c) s = s + expf(f16_to_f32(xr[c]));
    for (int64_t c = 0; c < cols; ++c) yr[c] = f32_to_f16(expf(f16_to_f32(xr[c])) / s);
  }
  return 0;
}

/*
 * layer_norm along the last axis:
 *   s1 = sum x; mean = s1/N; s2 = sum (x*x) with x*x materialised (a producer of a reduce is not
 *   inlined, cinn/hlir/framework/op_lowering_util.cc:757-761); var = max(s2/N - mean*mean, 0);
 *   r = 1/sqrt(var+eps); y = fma((x-mean)*r, gamma, beta).
 */
static inline void ln_stats(const float* xr, int64_t cols, float eps, float* mean_o, float* rstd_o) {
  float s1 = 0.0f, s2 = 0.0f;
  for (int64_t c = 0; c < cols; ++c) s1 = s1 + xr[c];
  for (int64_t c = 0; c < cols; ++c) {
    float t = xr[c] * xr[c];
    s2      = s2 + t;
  }
  const float n    = (float)cols;
  const float mean = s1 / n;
  const float m2   = s2 / n;
  const float mm   = mean * mean;
  const float var  = x86_max(m2 - mm, 0.0f);
  *mean_o          = mean;
  *rstd_o          = x86_rsqrt(var + eps);
}

int orc_layernorm_f32(const float* x, const float* gamma, const float* beta, int64_t rows, int64_t cols, float eps,
                      float* y, int threads) {
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    float* yr       = y + r * cols;
    float mean, rstd;
    ln_stats(xr, cols, eps, &mean, &rstd);
    for (int64_t c = 0; c < cols; ++c) yr[c] = fmaf((xr[c] - mean) * rstd, gamma[c], beta[c]);
  }
  return 0;
}

int orc_layernorm_f16(const f16bits* x, const float* gamma, const float* beta, int64_t rows, int64_t cols, float eps,
                      f16bits* y, float* row_scratch, int threads) {
  /* row_scratch: threads*cols floats holding the fp32 cast of one row per thread. */
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t r = 0; r < rows; ++r) {
#ifdef _OPENMP
    float* xr = row_scratch + (int64_t)omp_get_thread_num() * cols;
#else
    float* xr = row_scratch;
#endif
    const f16bits* xh = x + r * cols;
    f16bits* yr       = y + r * cols;
    for (int64_t c = 0; c < cols; ++c) xr[c] = f16_to_f32(xh[c]);
    float mean, rstd;
    ln_stats(xr, cols, eps, &mean, &rstd);
    for (int64_t c = 0; c < cols; ++c) yr[c] = f32_to_f16(fmaf((xr[c] - mean) * rstd, gamma[c], beta[c]));
  }
  return 0;
}

/* relu(batch_norm_infer(X)) on NCHW, fp32: max(((x-mean)*scale)/sqrt(var+eps)+bias, 0) (pe/nn.cc:715-717). */
int orc_bn_relu_nchw_f32(const float* x, const float* scale, const float* bias, const float* mean, const float* var,
                         int64_t n, int64_t c, int64_t hw, float eps, float* y, int threads) {
  const int64_t planes = n * c;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t p = 0; p < planes; ++p) {
    const int64_t ch = p % c;
    const float* xp  = x + p * hw;
    float* yp        = y + p * hw;
    for (int64_t i = 0; i < hw; ++i) {
      float t = ((xp[i] - mean[ch]) * scale[ch]) / sqrtf(var[ch] + eps) + bias[ch];
      yp[i]   = x86_max(t, 0.0f);
    }
  }
  return 0;
}

/* fp16 I/O variant: cast16(relu(bn(cast32(x)))) with fp32 parameters. */
int orc_bn_relu_nchw_f16(const f16bits* x, const float* scale, const float* bias, const float* mean,
                         const float* var, int64_t n, int64_t c, int64_t hw, float eps, f16bits* y, int threads) {
  const int64_t planes = n * c;
#pragma omp parallel for schedule(static) num_threads(threads > 0 ? threads : 1)
  for (int64_t p = 0; p < planes; ++p) {
    const int64_t ch  = p % c;
    const f16bits* xp = x + p * hw;
    f16bits* yp       = y + p * hw;
    for (int64_t i = 0; i < hw; ++i) {
      float t = ((f16_to_f32(xp[i]) - mean[ch]) * scale[ch]) / sqrtf(var[ch] + eps) + bias[ch];
      yp[i]   = f32_to_f16(x86_max(t, 0.0f));
    }
  }
  return 0;
}

/* ------------------------------------------------------------------------------------------------
 * Comparison helpers used by the tests (so that full-size comparisons do not run in Python loops).
 * ---------------------------------------------------------------------------------------------- */
static inline int32_t ordered_bits(float f) {
  int32_t i;
  memcpy(&i, &f, 4);
  return i < 0 ? (int32_t)0x80000000 - i : i;
}

/* Largest distance in units in the last place between two fp32 arrays; NaN anywhere gives INT64_MAX. */
int64_t orc_max_ulp_f32(const float* a, const float* b, int64_t n) {
  int64_t worst = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (isnan(a[i]) || isnan(b[i])) {
      if (isnan(a[i]) && isnan(b[i])) continue;
      return INT64_MAX;
    }
    int64_t d = (int64_t)ordered_bits(a[i]) - (int64_t)ordered_bits(b[i]);
    if (d < 0) d = -d;
    if (d > worst) worst = d;
  }
  return worst;
}

/* Number of elements with |a-b| > atol + rtol*|b|, and the largest such excess ratio through *worst. */
int64_t orc_count_not_close_f32(const float* a, const float* b, int64_t n, double rtol, double atol, double* worst) {
  int64_t bad = 0;
  double w    = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    double d   = fabs((double)a[i] - (double)b[i]);
    double lim = atol + rtol * fabs((double)b[i]);
    if (!(d <= lim)) ++bad;
    double q = lim > 0 ? d / lim : (d > 0 ? INFINITY : 0.0);
    if (q > w) w = q;
  }
  if (worst) *worst = w;
  return bad;
}

int64_t orc_count_not_close_f16(const f16bits* a, const f16bits* b, int64_t n, double rtol, double atol,
                                double* worst) {
  int64_t bad = 0;
  double w    = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    double x = f16_to_f32(a[i]), y = f16_to_f32(b[i]);
    double d   = fabs(x - y);
    double lim = atol + rtol * fabs(y);
    if (!(d <= lim)) ++bad;
    double q = lim > 0 ? d / lim : (d > 0 ? INFINITY : 0.0);
    if (q > w) w = q;
  }
  if (worst) *worst = w;
  return bad;
}
