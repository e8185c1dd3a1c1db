// Row-normalisation fused groups: softmax and layer_norm along the last axis, one pass over HBM.
//
// The reference fuses a reduce with its broadcast consumers only when the reduced extent is <= 1024
// (cinn/hlir/pass/op_fusion_pass_util.h:263-265, cinn/hlir/pass/fusion_merge_pass_util.h:400-403); longer rows
// become two kernels that read x twice, and its softmax op recomputes the row sum per output element
// (cinn/hlir/pe/nn.cc:755-796, schedule cinn/hlir/op/nn.cc:1934-1957).  Here a row lives in the registers of a
// group of G threads (or, for very long rows, in the shared memory of a thread-block cluster), so x is read
// once and the result written once whatever the row length.
//
// Arithmetic (the x86 path's, in fp32; T is only the storage type of x and out):
//   softmax     e = exp(x); out = e / sum(e)                       (no max subtraction: pe/nn.cc:755-796)
//   layer_norm  mean = sum(x)/N; var = max(sum(x*x)/N - mean*mean, 0); rstd = 1/sqrt(var+eps);
//               out = fma((x-mean)*rstd, gamma, beta)              (cinn/frontend/op_mappers/paddle/layer_norm.cc:84-139
//               with rsqrt+multiply in place of sqrt+divide; x*x is rounded before it is summed because a
//               producer of a reduce is materialised, cinn/hlir/framework/op_lowering_util.cc:757-761)
#include <cooperative_groups.h>

#include "device_math.cuh"
#include "kernel_registry.h"

namespace cg = cooperative_groups;

namespace cinn_b200 {

// A row is owned by G threads: a warp when G == 32 (several rows per CTA), otherwise the whole CTA.
template <int G, class Op>
__device__ __forceinline__ float group_allreduce(float v, float* scratch) {
  if (G == 32) return warp_allreduce<Op>(v);
  return cta_allreduce<Op>(v, scratch);
}

template <int G>
__device__ __forceinline__ void row_iteration_space(long long& first_row, long long& row_stride, int& t) {
  if (G == 32) {
    first_row  = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    row_stride = ((long long)gridDim.x * blockDim.x) >> 5;
    t          = threadIdx.x & 31;
  } else {
    first_row  = blockIdx.x;
    row_stride = gridDim.x;
    t          = threadIdx.x;
  }
}

// ------------------------------------------------------------------------------------------------
// softmax, row in registers.  Requires cols % V == 0, 16-byte aligned pointers, cols <= G*VPT*V.
// ------------------------------------------------------------------------------------------------
template <typename T, int G, int VPT>
__global__ void __launch_bounds__(G == 32 ? 256 : G)
    k_softmax_row(const T* __restrict__ x, T* __restrict__ y, long long rows, long long cols) {
  constexpr int V = Io<T>::kVec;
  __shared__ float scratch[32];
  long long row, row_stride;
  int t;
  row_iteration_space<G>(row, row_stride, t);
  const int nvec = (int)(cols / V);
  for (; row < rows; row += row_stride) {
    const uint4* px = reinterpret_cast<const uint4*>(x + row * cols);
    uint4* py       = reinterpret_cast<uint4*>(y + row * cols);
    uint4 raw[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (v < nvec) raw[j] = __ldcs(px + v);
    }
    float e[VPT][V];
    float local = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (v < nvec) {
        Io<T>::unpack(raw[j], e[j]);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          e[j][i] = sizeof(T) == 2 ? exp_for_16bit_out(e[j][i]) : expf(e[j][i]);
          local   = local + e[j][i];
        }
      }
    }
    const float s = group_allreduce<G, SumOp>(local, scratch);
    // e * (1/s) instead of e / s: at most one more rounding (1.5 ulp), inside the 1e-5 bar of a reduction group.
    const float inv_s = 1.0f / s;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (v < nvec) {
#pragma unroll
        for (int i = 0; i < V; ++i) e[j][i] = e[j][i] * inv_s;
        __stcs(py + v, Io<T>::pack(e[j]));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// layer_norm, row in registers.  gamma/beta are fp32 and stay in L1 across the rows a CTA processes.
// ------------------------------------------------------------------------------------------------
template <typename T, int G, int VPT>
__global__ void __launch_bounds__(G == 32 ? 256 : G)
    k_layernorm_row(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                    T* __restrict__ y, long long rows, long long cols, double eps_d) {
  constexpr int V = Io<T>::kVec;
  __shared__ float scratch[32];
  long long row, row_stride;
  int t;
  row_iteration_space<G>(row, row_stride, t);
  const int nvec  = (int)(cols / V);
  const float eps = (float)eps_d;
  const float n   = (float)cols;
  for (; row < rows; row += row_stride) {
    const uint4* px = reinterpret_cast<const uint4*>(x + row * cols);
    uint4* py       = reinterpret_cast<uint4*>(y + row * cols);
    uint4 raw[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (v < nvec) raw[j] = __ldcs(px + v);
    }
    float f[VPT][V];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (v < nvec) {
        Io<T>::unpack(raw[j], f[j]);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          s1 = s1 + f[j][i];
          s2 = s2 + f[j][i] * f[j][i];
        }
      }
    }
    s1 = group_allreduce<G, SumOp>(s1, scratch);
    s2 = group_allreduce<G, SumOp>(s2, scratch);
    const float mean = s1 / n;
    const float var  = x86_max(s2 / n - mean * mean, 0.0f);
    const float rstd = x86_rsqrt(var + eps);
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (v < nvec) {
        float g[V], b[V];
#pragma unroll
        for (int q = 0; q < V / 4; ++q) {
          Io<float>::unpack(ld_keep16(gamma + (long long)v * V + 4 * q), g + 4 * q);
          Io<float>::unpack(ld_keep16(beta + (long long)v * V + 4 * q), b + 4 * q);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) f[j][i] = fmaf((f[j][i] - mean) * rstd, g[i], b[i]);
        __stcs(py + v, Io<T>::pack(f[j]));
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Any row length / alignment: a thread-block cluster owns a row.  Each CTA converts its segment of the row
// to fp32 in dynamic shared memory (seg floats), the per-CTA partial sums are exchanged through distributed
// shared memory (every CTA writes its partial into slot [rank] of every peer), and each CTA then normalises
// its own segment out of shared memory.  Cluster size 1 is the plain "row in shared memory" case.
// mode 0: softmax (gamma/beta unused); mode 1: layer_norm.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(512)
    k_rownorm_cluster(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                      T* __restrict__ y, long long rows, long long cols, long long seg, long long mode,
                      double eps_d) {
  extern __shared__ __align__(16) float row_smem[];
  __shared__ float scratch[32];
  __shared__ float part1[16], part2[16];
  cg::cluster_group cluster  = cg::this_cluster();
  const unsigned rank        = cluster.block_rank();
  const unsigned csize       = cluster.num_blocks();
  const long long n_clusters = gridDim.x / csize;
  const long long begin      = (long long)rank * seg;
  const long long end        = min(begin + seg, cols);
  const float eps            = (float)eps_d;
  for (long long row = blockIdx.x / csize; row < rows; row += n_clusters) {
    const T* px = x + row * cols;
    T* py       = y + row * cols;
    float s1 = 0.0f, s2 = 0.0f;
    for (long long c = begin + threadIdx.x; c < end; c += blockDim.x) {
      float f = Io<T>::load1(px + c);
      if (mode == 0) {
        f  = expf(f);
        s1 = s1 + f;
      } else {
        s1 = s1 + f;
        s2 = s2 + f * f;
      }
      row_smem[c - begin] = f;
    }
    s1 = cta_allreduce<SumOp>(s1, scratch);
    s2 = cta_allreduce<SumOp>(s2, scratch);
    if (threadIdx.x < csize) {
      cluster.map_shared_rank(part1, threadIdx.x)[rank] = s1;
      cluster.map_shared_rank(part2, threadIdx.x)[rank] = s2;
    }
    cluster.sync();
    float t1 = 0.0f, t2 = 0.0f;
    for (unsigned q = 0; q < csize; ++q) {  // same order in every CTA: identical totals
      t1 = t1 + part1[q];
      t2 = t2 + part2[q];
    }
    if (mode == 0) {
      for (long long c = begin + threadIdx.x; c < end; c += blockDim.x)
        Io<T>::store1(py + c, row_smem[c - begin] / t1);
    } else {
      const float n    = (float)cols;
      const float mean = t1 / n;
      const float var  = x86_max(t2 / n - mean * mean, 0.0f);
      const float rstd = x86_rsqrt(var + eps);
      for (long long c = begin + threadIdx.x; c < end; c += blockDim.x)
        Io<T>::store1(py + c, fmaf((row_smem[c - begin] - mean) * rstd, gamma[c], beta[c]));
    }
    cluster.sync();  // part1/part2 and row_smem are rewritten by the next row
  }
}

#define REG_ROWNORM_G(TNAME, T, G)                                                                             \
  CINN_B200_REGISTER_KERNEL("softmax_row_" TNAME "_g" #G "_v1", 4, (G == 32 ? 256 : G), k_softmax_row<T, G, 1>); \
  CINN_B200_REGISTER_KERNEL("softmax_row_" TNAME "_g" #G "_v2", 4, (G == 32 ? 256 : G), k_softmax_row<T, G, 2>); \
  CINN_B200_REGISTER_KERNEL("softmax_row_" TNAME "_g" #G "_v4", 4, (G == 32 ? 256 : G), k_softmax_row<T, G, 4>); \
  CINN_B200_REGISTER_KERNEL("layernorm_row_" TNAME "_g" #G "_v1", 7, (G == 32 ? 256 : G), k_layernorm_row<T, G, 1>); \
  CINN_B200_REGISTER_KERNEL("layernorm_row_" TNAME "_g" #G "_v2", 7, (G == 32 ? 256 : G), k_layernorm_row<T, G, 2>); \
  CINN_B200_REGISTER_KERNEL("layernorm_row_" TNAME "_g" #G "_v4", 7, (G == 32 ? 256 : G), k_layernorm_row<T, G, 4>)

#define REG_ROWNORM_T(TNAME, T) \
  REG_ROWNORM_G(TNAME, T, 32);  \
  REG_ROWNORM_G(TNAME, T, 128); \
  REG_ROWNORM_G(TNAME, T, 256); \
  REG_ROWNORM_G(TNAME, T, 512); \
  REG_ROWNORM_G(TNAME, T, 1024); \
  CINN_B200_REGISTER_KERNEL("rownorm_cluster_" TNAME, 9, 512, k_rownorm_cluster<T>)

REG_ROWNORM_T("f32", float);
REG_ROWNORM_T("f16", __half);

}  // namespace cinn_b200
