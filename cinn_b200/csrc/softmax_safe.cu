// Row softmax with the row maximum subtracted first: the decomposed form of the softmax op in every mode other than
// "fast" (cinn/frontend/decomposer/activation.cc:104-116):
//     x_max = reduce_max(x); x_exp = exp(x - x_max); out = exp(x - x_max) / reduce_sum(x_exp)
// The reference runs it as several kernels (two reductions, each refusing to fuse with its broadcast consumer above
// 1024 columns); here one CTA keeps the row in registers and makes the three passes (maximum, exponentials and their
// sum, output) over registers: x is read once and the result written once.  The maximum is compare + select
// starting from the lowest finite value (cinn/lang/builtin.cc:123-143); this group is in the reduction tolerance
// class, so the quotient is a multiplication by 1 / sum and 16-bit outputs use the fast exponential.
// (Measured on B200 with fp16 storage, 16384 x 4096, 0.87 of the HBM peak: a body without the per-vector tests for
// rows of exactly this length gave 0.85, and one barrier per row -- exponentials relative to the warp's maximum, the
// barrier combining (maximum, sum) pairs -- 0.84; both left out.)
#include "device_math.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

// Reduction over the CTA with ONE barrier: every warp leaves its partial in shared memory, and after the barrier
// every thread folds the (at most 16) partials itself, in a fixed order.  `slot` alternates between two buffers so
// that the next reduction may start writing while slow warps still read this one.
template <class Op>
__device__ __forceinline__ float cta_fold(float v, float (*buf)[16], int slot) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  v = warp_allreduce<Op>(v);
  if (lane == 0) buf[slot][warp] = v;
  __syncthreads();
  // 4, 8 or 16 warps: whole float4 reads (broadcast), folded pairwise
  const float4* q = reinterpret_cast<const float4*>(&buf[slot][0]);
  float4 a        = q[0];
  float r         = Op::apply(Op::apply(a.x, a.y), Op::apply(a.z, a.w));
  for (int w = 1; w < (nwarps >> 2); ++w) {
    a = q[w];
    r = Op::apply(r, Op::apply(Op::apply(a.x, a.y), Op::apply(a.z, a.w)));
  }
  return r;
}

// One CTA of blockDim.x threads per row; thread t holds vectors t, t + blockDim.x, ... (VPT of them at most).
// vec_ok != 0: 16-byte aligned buffers and cols % V == 0 (16-byte accesses); otherwise the same register layout is
// filled and drained element by element, positions at or beyond `cols` masked out.
// SUBMAX = false: the plain form exp(x) / sum(exp(x)) of the softmax op itself (cinn/hlir/pe/nn.cc:755-796).
template <typename T, int VPT, bool SUBMAX = true>
__global__ void __launch_bounds__(512)
    k_softmax_safe(const T* __restrict__ x, T* __restrict__ y, long long rows, long long cols, long long vec_ok) {
  grid_dependency_sync();
  constexpr int V = Io<T>::kVec;
  __shared__ __align__(16) float max_buf[2][16], sum_buf[2][16];
  int parity     = 0;
  const int nvec = (int)((cols + V - 1) / V);
  const int G    = blockDim.x;
  // The vectors of the NEXT row of this CTA are requested before the current row is reduced, so that the two
  // barriers of a row do not leave the memory pipe idle.
  uint4 raw[VPT];
  if (vec_ok && blockIdx.x < rows) {
#pragma unroll
    for (int j = 0; j < VPT; ++j)
      if ((int)threadIdx.x + j * G < nvec) raw[j] = __ldcs(reinterpret_cast<const uint4*>(x + (long long)blockIdx.x * cols) + threadIdx.x + j * G);
  }
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * cols;
    T* yr       = y + row * cols;
    float f[VPT][V];
    float mx = MaxOp::identity();
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = (int)threadIdx.x + j * G;
      if (v < nvec) {
        if (vec_ok) {
          Io<T>::unpack(raw[j], f[j]);
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i) f[j][i] = (long long)v * V + i < cols ? Io<T>::load1(xr + (long long)v * V + i) : MaxOp::identity();
        }
#pragma unroll
        for (int i = 0; i < V; ++i) mx = x86_max(mx, f[j][i]);
      }
    }
    if (vec_ok && row + gridDim.x < rows) {
      const uint4* pn = reinterpret_cast<const uint4*>(xr + (long long)gridDim.x * cols);
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if ((int)threadIdx.x + j * G < nvec) raw[j] = __ldcs(pn + threadIdx.x + j * G);
    }
    mx = SUBMAX ? cta_fold<MaxOp>(mx, max_buf, parity) : 0.0f;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = (int)threadIdx.x + j * G;
      if (v < nvec) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float d = SUBMAX ? f[j][i] - mx : f[j][i];
          const float e = sizeof(T) == 2 ? exp_for_16bit_out(d) : expf(d);
          f[j][i]       = (vec_ok || (long long)v * V + i < cols) ? e : 0.0f;
          sum           = sum + f[j][i];
        }
      }
    }
    sum             = cta_fold<SumOp>(sum, sum_buf, parity);
    parity ^= 1;
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = (int)threadIdx.x + j * G;
      if (v < nvec) {
#pragma unroll
        for (int i = 0; i < V; ++i) f[j][i] = f[j][i] * inv;
        if (vec_ok) {
          __stcs(reinterpret_cast<uint4*>(yr) + v, Io<T>::pack(f[j]));
        } else {
#pragma unroll
          for (int i = 0; i < V; ++i)
            if ((long long)v * V + i < cols) Io<T>::store1(yr + (long long)v * V + i, f[j][i]);
        }
      }
    }
  }
}

}  // namespace

#define REG_SAFE(TNAME, T)                                                                      \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_safe_" TNAME "_v1", 5, 512, k_softmax_safe<T, 1>);        \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_safe_" TNAME "_v2", 5, 512, k_softmax_safe<T, 2>);        \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_safe_" TNAME "_v4", 5, 512, k_softmax_safe<T, 4>);        \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_safe_" TNAME "_v8", 5, 512, k_softmax_safe<T, 8>)
#define REG_PLAIN(TNAME, T)                                                                        \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_plain_" TNAME "_v1", 5, 512, k_softmax_safe<T, 1, false>);   \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_plain_" TNAME "_v2", 5, 512, k_softmax_safe<T, 2, false>);   \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_plain_" TNAME "_v4", 5, 512, k_softmax_safe<T, 4, false>);   \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_plain_" TNAME "_v8", 5, 512, k_softmax_safe<T, 8, false>)
REG_PLAIN("f32", float);
REG_PLAIN("f16", __half);
REG_PLAIN("bf16", __nv_bfloat16);
REG_SAFE("f32", float);
REG_SAFE("f16", __half);
REG_SAFE("bf16", __nv_bfloat16);

}  // namespace cinn_b200
