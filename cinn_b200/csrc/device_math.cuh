// Device-side arithmetic and memory helpers shared by all fused-group kernels.
//
// The scalar formulas restate what CINN's x86 path computes (that path is the parity target), not
// what CUDA's libm would: tanh is the two-branch exp formula, rsqrt is 1/sqrt, max/min are
// compare+select.  The translation units that include this file are compiled with -fmad=false so
// that a*b+c is fused only where fmaf() is written; division and sqrt are the IEEE-rounded forms
// (nvcc defaults -prec-div=true -prec-sqrt=true, no fast-math, no flush-to-zero).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cinn_b200 {

// First statement of the kernels that may be launched with programmatic stream serialisation: wait until the
// kernel launched before this one on the stream has completed and its writes are visible (a no-op for an ordinary
// launch), then allow the NEXT kernel of the stream to be scheduled early in turn.  The dependents are released only
// after this wait, so at most one kernel ever sits waiting behind a running one.
__device__ __forceinline__ void grid_dependency_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}


// cinn/backends/llvm/codegen_llvm.cc:310-340: fcmp ogt/olt + select.
__device__ __forceinline__ float x86_max(float a, float b) { return a > b ? a : b; }
__device__ __forceinline__ float x86_min(float a, float b) { return a < b ? a : b; }

// cinn/backends/llvm/llvm_intrin_rule.h:136-154.  Both branches evaluate exp(-2|x|); the negative
// branch (e-1)/(e+1) is the exact negation of (1-e)/(1+e).
__device__ __forceinline__ float x86_tanh(float x) {
  if (x >= 0.0f) {
    float e = expf(-2.0f * x);
    return (1.0f - e) / (1.0f + e);
  } else {
    float e = expf(2.0f * x);
    return (e - 1.0f) / (e + 1.0f);
  }
}
// The same function for kernels whose OUTPUT is a 16-bit float (tolerance 1e-2 relative): one ex2.approx and
// one rcp.approx instead of the full-accuracy expf and the IEEE division.  fp32 relative error of the quotient
// is about 2^-21, far below the 2^-11 spacing of fp16 / 2^-8 of bf16; close to zero, where 1-e cancels, the
// odd series a - a^3/3 is used instead (relative error < 2e-8 for |a| < 0.02).
// 1 / y by the hardware's approximate reciprocal alone (1 ulp; no range fix-ups: for y in [1, 2], or where an
// infinite y may give 0).
__device__ __forceinline__ float rcp_approx(float y) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(y));
  return r;
}
__device__ __forceinline__ float x86_tanh_for_16bit_out(float x) {
  const float a = fabsf(x);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(a * -2.885390082f));  // exp(-2a) = 2^(-2a*log2(e))
  // (the approximate division, not a bare rcp.approx through inline assembly: measured on the streamed headline
  // kernel, 6525 GB/s against 6115 GB/s)
  float r       = __fdividef(1.0f - e, 1.0f + e);
  const float s = a * fmaf(a * a, -0.33333334f, 1.0f);
  r             = a < 0.02f ? s : r;
  return x < 0.0f ? -r : r;
}
// exp for kernels whose output is a 16-bit float: ex2.approx of x*log2(e).  The product's rounding error is
// |x|*2^-24 in the exponent, i.e. a relative error of about |x|*4e-8 in the result, plus 2 ulp of ex2.approx.
__device__ __forceinline__ float exp_for_16bit_out(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * 1.4426950408889634f));
  return e;
}
// cinn/backends/llvm/llvm_intrin_rule.h:105-113.
__device__ __forceinline__ float x86_rsqrt(float x) { return 1.0f / sqrtf(x); }
// cinn/lang/builtin.h:79-82.
__device__ __forceinline__ float x86_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- 128-bit global memory access -------------------------------------------------------------
// Inputs of these groups are read once and outputs written once, so both use the streaming
// (evict-first) cache policy; small broadcast operands use the default policy and stay in L1/L2.
__device__ __forceinline__ uint4 ld_stream16(const void* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st_stream16(void* p, uint4 v) { __stcs(reinterpret_cast<uint4*>(p), v); }
__device__ __forceinline__ uint2 ld_stream8(const void* p) { return __ldcs(reinterpret_cast<const uint2*>(p)); }
__device__ __forceinline__ void st_stream8(void* p, uint2 v) { __stcs(reinterpret_cast<uint2*>(p), v); }
__device__ __forceinline__ uint4 ld_keep16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void unpack4(uint4 u, float (&f)[4]) {
  f[0] = __uint_as_float(u.x);
  f[1] = __uint_as_float(u.y);
  f[2] = __uint_as_float(u.z);
  f[3] = __uint_as_float(u.w);
}
__device__ __forceinline__ uint4 pack4(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
// fp16 pairs: fpext is exact, fptrunc is round-to-nearest-even (cinn/backends/llvm/codegen_llvm.cc:454-455).
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void unpack_h2(uint32_t u, float& lo, float& hi) {
  __half2 h = *reinterpret_cast<__half2*>(&u);
  float2 f  = __half22float2(h);
  lo        = f.x;
  hi        = f.y;
}
__device__ __forceinline__ void unpack8h(uint4 u, float (&f)[8]) {
  unpack_h2(u.x, f[0], f[1]);
  unpack_h2(u.y, f[2], f[3]);
  unpack_h2(u.z, f[4], f[5]);
  unpack_h2(u.w, f[6], f[7]);
}
__device__ __forceinline__ uint4 pack8h(const float (&f)[8]) {
  return make_uint4(pack_h2(f[0], f[1]), pack_h2(f[2], f[3]), pack_h2(f[4], f[5]), pack_h2(f[6], f[7]));
}
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void unpack_bf2(uint32_t u, float& lo, float& hi) {
  lo = __uint_as_float(u << 16);
  hi = __uint_as_float(u & 0xffff0000u);
}

// Element type traits: how many elements a 16-byte vector holds and how to convert it to/from fp32.
template <typename T>
struct Io;
template <>
struct Io<float> {
  static constexpr int kVec = 4;
  __device__ static __forceinline__ void unpack(uint4 u, float* f) {
    f[0] = __uint_as_float(u.x);
    f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z);
    f[3] = __uint_as_float(u.w);
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  __device__ static __forceinline__ float load1(const float* p) { return *p; }
  __device__ static __forceinline__ void store1(float* p, float v) { *p = v; }
};
template <>
struct Io<__half> {
  static constexpr int kVec = 8;
  __device__ static __forceinline__ void unpack(uint4 u, float* f) {
    unpack_h2(u.x, f[0], f[1]);
    unpack_h2(u.y, f[2], f[3]);
    unpack_h2(u.z, f[4], f[5]);
    unpack_h2(u.w, f[6], f[7]);
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack_h2(f[0], f[1]), pack_h2(f[2], f[3]), pack_h2(f[4], f[5]), pack_h2(f[6], f[7]));
  }
  __device__ static __forceinline__ float load1(const __half* p) { return __half2float(*p); }
  __device__ static __forceinline__ void store1(__half* p, float v) { *p = __float2half_rn(v); }
};
template <>
struct Io<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static __forceinline__ void unpack(uint4 u, float* f) {
    unpack_bf2(u.x, f[0], f[1]);
    unpack_bf2(u.y, f[2], f[3]);
    unpack_bf2(u.z, f[4], f[5]);
    unpack_bf2(u.w, f[6], f[7]);
  }
  __device__ static __forceinline__ uint4 pack(const float* f) {
    return make_uint4(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3]), pack_bf2(f[4], f[5]), pack_bf2(f[6], f[7]));
  }
  __device__ static __forceinline__ float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ static __forceinline__ void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

// ---- warp / CTA reductions ---------------------------------------------------------------------
// A reduction op has two faces: accum(acc, x) folds one INPUT element into an accumulator, apply(a, b) combines two
// partial results.  For the plain ops they coincide; the composite ops below apply an elementwise producer to the
// element first (the producer of a reduce is materialised in the reference, cinn/hlir/framework/
// op_lowering_util.cc:757-761, so its result is rounded to fp32 before it is accumulated: x*x then +, no fma).
struct SumOp {
  __device__ static __forceinline__ float identity() { return 0.0f; }
  __device__ static __forceinline__ float apply(float a, float b) { return a + b; }
  __device__ static __forceinline__ float accum(float a, float x) { return a + x; }
};
struct ProdOp {
  __device__ static __forceinline__ float identity() { return 1.0f; }
  __device__ static __forceinline__ float apply(float a, float b) { return a * b; }
  __device__ static __forceinline__ float accum(float a, float x) { return a * x; }
};
// cinn/lang/builtin.cc:123-143: the initial value of max is lowest() (= -FLT_MAX), not -inf.
struct MaxOp {
  __device__ static __forceinline__ float identity() { return -3.402823466e+38f; }
  __device__ static __forceinline__ float apply(float a, float b) { return x86_max(a, b); }
  __device__ static __forceinline__ float accum(float a, float x) { return x86_max(a, x); }
};
struct MinOp {
  __device__ static __forceinline__ float identity() { return 3.402823466e+38f; }
  __device__ static __forceinline__ float apply(float a, float b) { return x86_min(a, b); }
  __device__ static __forceinline__ float accum(float a, float x) { return x86_min(a, x); }
};
struct SumSquareOp : SumOp {  // reduce_sum(x * x)
  __device__ static __forceinline__ float accum(float a, float x) { return a + x * x; }
};
struct SumAbsOp : SumOp {  // reduce_sum(abs(x))
  __device__ static __forceinline__ float accum(float a, float x) { return a + fabsf(x); }
};
struct SumExpOp : SumOp {  // reduce_sum(exp(x))
  __device__ static __forceinline__ float accum(float a, float x) { return a + expf(x); }
};
struct MaxAbsOp : MaxOp {  // reduce_max(abs(x))
  __device__ static __forceinline__ float accum(float a, float x) { return x86_max(a, fabsf(x)); }
};

template <class Op>
__device__ __forceinline__ float warp_allreduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// All threads of the CTA get the result.  `scratch` holds at least 32 floats of shared memory and may
// be reused after the call returns (a trailing barrier is included).
template <class Op>
__device__ __forceinline__ float cta_allreduce(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_allreduce<Op>(v);
  if (nwarps == 1) return v;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < nwarps ? scratch[lane] : Op::identity();
  r       = warp_allreduce<Op>(r);
  __syncthreads();
  return r;
}

}  // namespace cinn_b200
