// Elementwise / broadcast fused-group kernels (one pass over HBM, 128-bit accesses).
//
// These stand in for the kernels the reference generates for kElementWise / kBroadcast groups after
// inlining every producer into the output expression (cinn/hlir/framework/op_lowering.cc:247-310,
// schedule cinn/hlir/pe/ir_schedule_pe.cc:42-86: one element per thread, 1024-thread blocks, scalar
// accesses).  Here each thread moves 16-byte vectors, keeps several loads in flight, and the
// per-channel / per-column operands are read through L1.
//
// Kernel parameters are flat (pointers, then 64-bit integers, then doubles) so that the launch
// primitive can pass them from a cinn_pod_value_t array (floats travel as double in that array,
// cinn/runtime/cinn_runtime.cc:274-281).
#include "device_math.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {

// ------------------------------------------------------------------------------------------------
// relu(a + b), fp32.   cinn/hlir/pe/broadcast.cc:216-273 (add), cinn/hlir/pe/nn.cc:61-64 (relu).
// vec_ok != 0: all three pointers are 16-byte aligned.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_add_relu_f32(const float* __restrict__ a, const float* __restrict__ b,
                                                      float* __restrict__ y, long long n, long long vec_ok) {
  grid_dependency_sync();
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (vec_ok) {
    const long long nvec = n >> 2;
    for (long long v = tid; v < nvec; v += stride) {
      float fa[4], fb[4], fy[4];
      unpack4(ld_stream16(a + 4 * v), fa);
      unpack4(ld_stream16(b + 4 * v), fb);
#pragma unroll
      for (int i = 0; i < 4; ++i) fy[i] = x86_max(fa[i] + fb[i], 0.0f);
      st_stream16(y + 4 * v, pack4(fy));
    }
    done = nvec << 2;
  }
  for (long long i = done + tid; i < n; i += stride) y[i] = x86_max(a[i] + b[i], 0.0f);
}
CINN_B200_REGISTER_KERNEL_PDL("ew_add_relu_f32", 5, 256, k_add_relu_f32);

// ------------------------------------------------------------------------------------------------
// out = cast<OutT>(tanh(scale * (x + bias[col]) + shift)), bias broadcast along the last axis.
// add: cinn/hlir/pe/broadcast.cc:216-273; scale: cinn/hlir/op/elementwise.cc:149-163 (Mul+Add -> fma by
// cinn/optim/lower_intrin.cc:41-59); tanh: the x86 rule; cast: cinn/hlir/pe/elementwise.cc:213-217.
// Each thread-iteration handles 8 consecutive elements: two 16-byte loads of x, two of bias (L1), one
// 16-byte store for 16-bit outputs (two for fp32).  vec_ok != 0: pointers 16-byte aligned and cols % 8 == 0.
// ------------------------------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ void store8(OutT* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&f)[8]) {
  st_stream16(p, pack8h(f));
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  st_stream16(p, Io<__nv_bfloat16>::pack(f));
}
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  st_stream16(p, make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3])));
  st_stream16(p + 4,
              make_uint4(__float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7])));
}

// 16-bit outputs use the reduced-cost tanh (accuracy matched to the output type), fp32 outputs the exact x86 form.
template <typename OutT>
__device__ __forceinline__ float tanh_for(float t) {
  return x86_tanh_for_16bit_out(t);
}
template <>
__device__ __forceinline__ float tanh_for<float>(float t) {
  return x86_tanh(t);
}

template <typename OutT>
__global__ void __launch_bounds__(256)
    k_bias_scale_tanh_cast(const float* __restrict__ x, const float* __restrict__ bias, OutT* __restrict__ y,
                           long long n, long long cols, long long vec_ok, double scale_d, double shift_d) {
  grid_dependency_sync();
  const float scale      = (float)scale_d;
  const float shift      = (float)shift_d;
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (vec_ok) {
    const long long nvec      = n >> 3;
    const unsigned cols_vec   = (unsigned)(cols >> 3);
    // Two vectors per iteration: four independent 16-byte streaming loads in flight per thread.
    long long v = tid;
    for (; v + stride < nvec; v += 2 * stride) {
      const long long v1 = v + stride;
      uint4 r0 = ld_stream16(x + 8 * v), r1 = ld_stream16(x + 8 * v + 4);
      uint4 r2 = ld_stream16(x + 8 * v1), r3 = ld_stream16(x + 8 * v1 + 4);
      const unsigned c0 = (unsigned)(v % cols_vec) << 3, c1 = (unsigned)(v1 % cols_vec) << 3;
      float fx[8], fb[8], fy[8];
      unpack4(r0, *reinterpret_cast<float(*)[4]>(&fx[0]));
      unpack4(r1, *reinterpret_cast<float(*)[4]>(&fx[4]));
      unpack4(ld_keep16(bias + c0), *reinterpret_cast<float(*)[4]>(&fb[0]));
      unpack4(ld_keep16(bias + c0 + 4), *reinterpret_cast<float(*)[4]>(&fb[4]));
#pragma unroll
      for (int i = 0; i < 8; ++i) fy[i] = tanh_for<OutT>(fmaf(scale, fx[i] + fb[i], shift));
      store8<OutT>(y + 8 * v, fy);
      unpack4(r2, *reinterpret_cast<float(*)[4]>(&fx[0]));
      unpack4(r3, *reinterpret_cast<float(*)[4]>(&fx[4]));
      unpack4(ld_keep16(bias + c1), *reinterpret_cast<float(*)[4]>(&fb[0]));
      unpack4(ld_keep16(bias + c1 + 4), *reinterpret_cast<float(*)[4]>(&fb[4]));
#pragma unroll
      for (int i = 0; i < 8; ++i) fy[i] = tanh_for<OutT>(fmaf(scale, fx[i] + fb[i], shift));
      store8<OutT>(y + 8 * v1, fy);
    }
    for (; v < nvec; v += stride) {
      const unsigned c0 = (unsigned)(v % cols_vec) << 3;
      float fx[8], fb[8], fy[8];
      unpack4(ld_stream16(x + 8 * v), *reinterpret_cast<float(*)[4]>(&fx[0]));
      unpack4(ld_stream16(x + 8 * v + 4), *reinterpret_cast<float(*)[4]>(&fx[4]));
      unpack4(ld_keep16(bias + c0), *reinterpret_cast<float(*)[4]>(&fb[0]));
      unpack4(ld_keep16(bias + c0 + 4), *reinterpret_cast<float(*)[4]>(&fb[4]));
#pragma unroll
      for (int i = 0; i < 8; ++i) fy[i] = tanh_for<OutT>(fmaf(scale, fx[i] + fb[i], shift));
      store8<OutT>(y + 8 * v, fy);
    }
    done = nvec << 3;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float t = tanh_for<OutT>(fmaf(scale, x[i] + bias[i % cols], shift));
    Io<OutT>::store1(y + i, t);
  }
}
CINN_B200_REGISTER_KERNEL_PDL("ew_bias_scale_tanh_cast_f32_f16", 8, 256, k_bias_scale_tanh_cast<__half>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bias_scale_tanh_cast_f32_bf16", 8, 256, k_bias_scale_tanh_cast<__nv_bfloat16>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bias_scale_tanh_cast_f32_f32", 8, 256, k_bias_scale_tanh_cast<float>);

// ------------------------------------------------------------------------------------------------
// out = [relu](batch_norm_infer(x)) on NCHW: max(((x - mean[c]) * scale[c]) / sqrt(var[c] + eps) + bias[c], 0).
// cinn/hlir/pe/nn.cc:700-721 (operation order kept: true division, no pre-folded affine form), fused relu
// cinn/hlir/pe/nn.cc:61-64.  T is the storage type of x and out (fp32, or fp16 with the arithmetic in fp32);
// the parameters are fp32.  A CTA owns one chunk of one (n, c) plane, so the channel index and the four
// parameters are computed once per CTA.  vec_ok != 0: x and out are 16-byte aligned and hw % (16/sizeof(T)) == 0.
// ------------------------------------------------------------------------------------------------
// TRAIN: the normalisation step of the decomposed batch_norm_train (cinn/frontend/decomposer/batch_norm.cc:160-166),
// y = ((x - mean) * rsqrt(var + eps)) * scale + bias with mean / var the batch statistics: rsqrt is 1 / sqrt, the last
// multiply and add contract to one fused multiply-add (cinn/optim/lower_intrin.cc:41-59).
template <typename T, bool RELU, bool TRAIN = false>
__global__ void __launch_bounds__(256)
    k_bn_nchw(const T* __restrict__ x, const float* __restrict__ scale, const float* __restrict__ bias,
              const float* __restrict__ mean, const float* __restrict__ var, T* __restrict__ y, long long planes,
              long long channels, long long hw, long long chunks, long long vec_ok, double eps_d) {
  grid_dependency_sync();
  constexpr int V        = Io<T>::kVec;
  const long long n_ctas = planes * chunks;
  for (long long cta = blockIdx.x; cta < n_ctas; cta += gridDim.x) {
    const long long plane = cta / chunks;
    const int chunk       = (int)(cta - plane * chunks);
    const int c           = (int)(plane % channels);
    const float m = mean[c], s = scale[c], b = bias[c];
    const float d = sqrtf(var[c] + (float)eps_d);
    // 16-bit storage: multiply by the reciprocal (one rounding more than the division, far inside 1e-2).
    const float inv_d = 1.0f / d;
    const T* xp   = x + plane * hw;
    T* yp         = y + plane * hw;
    if (vec_ok) {
      const int nvec  = (int)(hw / V);
      const int per   = (int)((nvec + chunks - 1) / chunks);
      const int begin = chunk * per;
      const int end   = min(begin + per, nvec);
      const int B     = blockDim.x;
      // Four predicated vectors per iteration, all loads issued before the first use.
      for (int v = begin + threadIdx.x; v < end; v += 4 * B) {
        uint4 r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (v + j * B < end) r[j] = ld_stream16(xp + (long long)(v + j * B) * V);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (v + j * B < end) {
            float f[V];
            Io<T>::unpack(r[j], f);
#pragma unroll
            for (int i = 0; i < V; ++i) {
              if (TRAIN) f[i] = fmaf((f[i] - m) * inv_d, s, b);
              else f[i] = sizeof(T) == 2 ? ((f[i] - m) * s) * inv_d + b : ((f[i] - m) * s) / d + b;
              if (RELU) f[i] = x86_max(f[i], 0.0f);
            }
            st_stream16(yp + (long long)(v + j * B) * V, Io<T>::pack(f));
          }
        }
      }
    } else {
      const long long per   = (hw + chunks - 1) / chunks;
      const long long begin = chunk * per;
      const long long end   = min(begin + per, hw);
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
        float f = Io<T>::load1(xp + i);
        if (TRAIN) f = fmaf((f - m) * inv_d, s, b);
        else f = sizeof(T) == 2 ? ((f - m) * s) * inv_d + b : ((f - m) * s) / d + b;
        if (RELU) f = x86_max(f, 0.0f);
        Io<T>::store1(yp + i, f);
      }
    }
  }
}
// ------------------------------------------------------------------------------------------------
// x_grad of the decomposed batch_norm_grad (cinn/frontend/decomposer/batch_norm.cc:212-238), NCHW fp32:
//     x_grad = tmp0 * ((dy * nhw - bias_grad) - ((x - mean) * S) / (var + eps))
// with per-channel tmp0 = (scale * rsqrt(var + eps)) / nhw, bias_grad = sum(dy), S = sum(dy * (x - mean)).
// Two streamed inputs, one output; the per-channel values are formed once per CTA, in the reference's operation
// order (rsqrt = 1 / sqrt; subtractions and the division are not contracted).  t0_form / vae_form = 1: tmp0 / var+eps
// are computed here from scale and var; 0: they are given as per-channel inputs.
// ------------------------------------------------------------------------------------------------
// T: storage type of x, dy and the result (float, or a 16-bit float between the casts of the AutoCast pass).
template <typename T>
__global__ void __launch_bounds__(256)
    k_bn_grad_apply(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ mean,
                    const float* __restrict__ sum_s, const float* __restrict__ bias_grad, const float* __restrict__ vae_in,
                    const float* __restrict__ t0_in, const float* __restrict__ var0, T* __restrict__ y,
                    long long planes, long long channels, long long hw, long long chunks, long long vec_ok,
                    long long t0_form, long long vae_form, double count_d, double eps_d) {
  grid_dependency_sync();
  const long long n_ctas = planes * chunks;
  const float count = (float)count_d, eps = (float)eps_d;
  for (long long cta = blockIdx.x; cta < n_ctas; cta += gridDim.x) {
    const long long plane = cta / chunks;
    const int chunk       = (int)(cta - plane * chunks);
    const int c           = (int)(plane % channels);
    const float m = mean[c], S = sum_s[c], db = bias_grad[c];
    const float vae = vae_form ? vae_in[c] + eps : vae_in[c];
    const float t0  = t0_form ? (t0_in[c] * (1.0f / sqrtf(var0[c] + eps))) / count : t0_in[c];
    const T* xp  = x + plane * hw;
    const T* dp  = dy + plane * hw;
    T* yp        = y + plane * hw;
    constexpr int V = Io<T>::kVec;
    if (vec_ok) {
      const int nvec  = (int)(hw / V);
      const int per   = (int)((nvec + chunks - 1) / chunks);
      const int begin = chunk * per;
      const int end   = min(begin + per, nvec);
      const int B     = blockDim.x;
      // four predicated vectors of each input per iteration: eight 16-byte loads in flight per thread
      constexpr int U = 4;
      for (int v = begin + threadIdx.x; v < end; v += U * B) {
        uint4 rx[U], rd[U];
#pragma unroll
        for (int j = 0; j < U; ++j)
          if (v + j * B < end) {
            rx[j] = ld_stream16(xp + (long long)(v + j * B) * V);
            rd[j] = ld_stream16(dp + (long long)(v + j * B) * V);
          }
#pragma unroll
        for (int j = 0; j < U; ++j) {
          if (v + j * B < end) {
            float fx[V], fd[V];
            Io<T>::unpack(rx[j], fx);
            Io<T>::unpack(rd[j], fd);
#pragma unroll
            for (int i = 0; i < V; ++i) fx[i] = t0 * (((fd[i] * count) - db) - (((fx[i] - m) * S) / vae));
            st_stream16(yp + (long long)(v + j * B) * V, Io<T>::pack(fx));
          }
        }
      }
    } else {
      const long long per   = (hw + chunks - 1) / chunks;
      const long long begin = chunk * per;
      const long long end   = min(begin + per, hw);
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x)
        Io<T>::store1(yp + i, t0 * (((Io<T>::load1(dp + i) * count) - db) - (((Io<T>::load1(xp + i) - m) * S) / vae)));
    }
  }
}
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_grad_apply_nchw_f32", 18, 256, k_bn_grad_apply<float>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_grad_apply_nchw_f16", 18, 256, k_bn_grad_apply<__half>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_grad_apply_nchw_bf16", 18, 256, k_bn_grad_apply<__nv_bfloat16>);

CINN_B200_REGISTER_KERNEL_PDL("ew_bn_relu_nchw_f32", 12, 256, k_bn_nchw<float, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_relu_nchw_f16", 12, 256, k_bn_nchw<__half, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_nchw_f32", 12, 256, k_bn_nchw<float, false>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_nchw_f16", 12, 256, k_bn_nchw<__half, false>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_relu_nchw_bf16", 12, 256, k_bn_nchw<__nv_bfloat16, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_nchw_bf16", 12, 256, k_bn_nchw<__nv_bfloat16, false>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_train_apply_nchw_f32", 12, 256, k_bn_nchw<float, false, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_train_apply_relu_nchw_f32", 12, 256, k_bn_nchw<float, true, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_train_apply_nchw_f16", 12, 256, k_bn_nchw<__half, false, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_train_apply_relu_nchw_f16", 12, 256, k_bn_nchw<__half, true, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_train_apply_nchw_bf16", 12, 256, k_bn_nchw<__nv_bfloat16, false, true>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bn_train_apply_relu_nchw_bf16", 12, 256, k_bn_nchw<__nv_bfloat16, true, true>);

}  // namespace cinn_b200
