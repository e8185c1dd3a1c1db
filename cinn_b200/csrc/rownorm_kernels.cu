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
//   layer_norm  mean = sum(x)/N; var = max(sum(x*x)/N - mean*mean, 0); rstd = 1/sqrt(var+eps)  [see k_rownorm_reg
//               for the cheaper per-row forms used inside the 1e-5 reduction tolerance];
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
// softmax / layer_norm with the rows in registers.  Requires cols % V == 0, 16-byte aligned pointers and
// cols <= G*VPT*V.  A group of G threads owns R consecutive rows per iteration; all R*VPT 16-byte loads of a
// thread are issued before the first use.  The rows are kept PACKED in registers (4 registers per 16 bytes
// whatever the element type) and unpacked once for the statistics and once for the output, which is what
// keeps the register count low enough for five 256-thread CTAs per SM.  For layer_norm the fp32 gamma/beta
// slices are read through L1 once per iteration and reused for the R rows; the sums of the R rows are reduced
// together with a single barrier (scratch double-buffered by iteration parity).
// ------------------------------------------------------------------------------------------------
// Resident CTAs per SM asked of the compiler: enough threads for about 80 KiB of loads in flight per SM.
constexpr int RownormMinBlocks(int g, int vpt, int r) {
  if (g == 32) return 5;
  if (g >= 1024) return 1;
  int threads = 5120 / (vpt * r);
  if (threads > 2048) threads = 2048;
  int blocks = (threads + g - 1) / g;
  return blocks < 1 ? 1 : blocks;
}

// EXACT: every row is exactly VPT vectors per thread of its group and the row count a multiple of R -- no test per
// vector, so the loads of a thread's vectors are issued together and their arithmetic interleaves (with the tests
// every vector is a basic block of its own).
template <typename T, int G, int VPT, int R, bool LAYERNORM, bool EXACT>
__device__ __forceinline__ void rownorm_reg_body(const T* __restrict__ x, const float* __restrict__ gamma,
                                                 const float* __restrict__ beta, T* __restrict__ y, long long rows,
                                                 long long cols, double eps_d, double inv_n_d) {
  constexpr int V      = Io<T>::kVec;
  constexpr int NWARPS = G == 32 ? 1 : G / 32;
  // layer_norm keeps the rows packed; softmax keeps exp(x) in fp32 (it is needed again for the output and
  // costs a transcendental to recompute).
  constexpr int KEEP = LAYERNORM ? 1 : V;
  __shared__ __align__(16) float2 partial[2][R][32];
  long long grp, grp_stride;
  int t;
  row_iteration_space<G>(grp, grp_stride, t);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec    = (int)(cols / V);
  const float eps   = (float)eps_d;
  const float inv_n = (float)inv_n_d;
  for (int it = 0; grp * R < rows; grp += grp_stride, ++it) {
    const long long row0 = grp * R;
    uint4 raw[R][VPT];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint4* px = reinterpret_cast<const uint4*>(x + (row0 + r) * cols);
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = t + j * G;
        if (EXACT || (v < nvec && row0 + r < rows)) raw[r][j] = __ldcs(px + v);
      }
    }
    float ev[R][VPT][KEEP];
    float s1[R], s2[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      s1[r] = 0.0f;
      s2[r] = 0.0f;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = t + j * G;
        if (EXACT || (v < nvec && row0 + r < rows)) {
          float f[V];
          Io<T>::unpack(raw[r][j], f);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            if (LAYERNORM) {
              s1[r] = s1[r] + f[i];
              // 16-bit storage (1e-2 tolerance): the square is accumulated with one fused multiply-add.
              s2[r] = sizeof(T) == 2 ? fmaf(f[i], f[i], s2[r]) : s2[r] + f[i] * f[i];
            } else {
              f[i]            = sizeof(T) == 2 ? exp_for_16bit_out(f[i]) : expf(f[i]);
              ev[r][j][i % KEEP] = f[i];
              s1[r]           = s1[r] + f[i];
            }
          }
        }
      }
      s1[r] = warp_allreduce<SumOp>(s1[r]);
      if (LAYERNORM) s2[r] = warp_allreduce<SumOp>(s2[r]);
    }
    if (G != 32) {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) partial[it & 1][r][warp] = make_float2(s1[r], s2[r]);
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (NWARPS <= 8) {
          // Every thread adds the per-warp partials itself (broadcast shared-memory reads, fixed order).
          const float4* pp = reinterpret_cast<const float4*>(&partial[it & 1][r][0]);
          float t1 = 0.0f, t2 = 0.0f;
#pragma unroll
          for (int w = 0; w < NWARPS / 2; ++w) {
            const float4 q = pp[w];
            t1             = (t1 + q.x) + q.z;
            t2             = (t2 + q.y) + q.w;
          }
          s1[r] = t1;
          s2[r] = t2;
        } else {
          float2 p = lane < NWARPS ? partial[it & 1][r][lane] : make_float2(0.0f, 0.0f);
          s1[r]    = warp_allreduce<SumOp>(p.x);
          if (LAYERNORM) s2[r] = warp_allreduce<SumOp>(p.y);
        }
      }
    }
    // Per-row scalars.  These groups are in the reduction tolerance class (1e-5 relative), so the row
    // statistics use a multiplication by 1/N and the hardware reciprocal square root (2 ulp) instead of two
    // IEEE divisions and a square root per row and warp; softmax multiplies by 1/sum.
    float a[R], m[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (LAYERNORM) {
        m[r]            = s1[r] * inv_n;
        const float var = x86_max(s2[r] * inv_n - m[r] * m[r], 0.0f);
        a[r]            = rsqrtf(var + eps);
      } else {
        a[r] = 1.0f / s1[r];
        m[r] = 0.0f;
      }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (EXACT || v < nvec) {
        float g[V], b[V];
        if (LAYERNORM) {
#pragma unroll
          for (int q = 0; q < V / 4; ++q) {
            Io<float>::unpack(ld_keep16(gamma + (long long)v * V + 4 * q), g + 4 * q);
            Io<float>::unpack(ld_keep16(beta + (long long)v * V + 4 * q), b + 4 * q);
          }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (EXACT || row0 + r < rows) {
            float f[V];
            if (LAYERNORM) {
              Io<T>::unpack(raw[r][j], f);
#pragma unroll
              for (int i = 0; i < V; ++i)
                f[i] = sizeof(T) == 2 ? fmaf(fmaf(f[i], a[r], -m[r] * a[r]), g[i], b[i])
                                      : fmaf((f[i] - m[r]) * a[r], g[i], b[i]);
            } else {
#pragma unroll
              for (int i = 0; i < V; ++i) f[i] = ev[r][j][i % KEEP] * a[r];
            }
            __stcs(reinterpret_cast<uint4*>(y + (row0 + r) * cols) + v, Io<T>::pack(f));
          }
        }
      }
    }
  }
}

// The kernel holds both bodies (deliberately: compiled alone, the straight-line body is packed into fewer registers
// with its loads and arithmetic less interleaved -- measured on the row programs, row_prog_body.cuh).  Measured on
// B200, 16384 x 4096: softmax with fp16 storage 0.94 -> 0.97 of the HBM peak, layer_norm fp32 0.95 -> 0.96, softmax
// fp32 unchanged (0.99).
template <typename T, int G, int VPT, int R, bool LAYERNORM>
__global__ void __launch_bounds__(G == 32 ? 256 : G, RownormMinBlocks(G, VPT, R))
    k_rownorm_reg(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                  T* __restrict__ y, long long rows, long long cols, double eps_d, double inv_n_d) {
  grid_dependency_sync();
  // (not for layer_norm with 16-bit storage: measured, its two-rows-per-iteration form does not gain)
  if (!(LAYERNORM && sizeof(T) == 2) && cols == (long long)G * VPT * Io<T>::kVec && rows % R == 0)
    rownorm_reg_body<T, G, VPT, R, LAYERNORM, true>(x, gamma, beta, y, rows, cols, eps_d, inv_n_d);
  else
    rownorm_reg_body<T, G, VPT, R, LAYERNORM, false>(x, gamma, beta, y, rows, cols, eps_d, inv_n_d);
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
  grid_dependency_sync();
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

#define REG_ROWNORM_ONE(TNAME, T, G, VPT, R)                                                                     \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_row_" TNAME "_g" #G "_v" #VPT "_r" #R, 8, (G == 32 ? 256 : G),               \
                            k_rownorm_reg<T, G, VPT, R, false>);                                                  \
  CINN_B200_REGISTER_KERNEL_PDL("layernorm_row_" TNAME "_g" #G "_v" #VPT "_r" #R, 8, (G == 32 ? 256 : G),             \
                            k_rownorm_reg<T, G, VPT, R, true>)
#define REG_ROWNORM_G(TNAME, T, G)    \
  REG_ROWNORM_ONE(TNAME, T, G, 1, 1); \
  REG_ROWNORM_ONE(TNAME, T, G, 2, 1); \
  REG_ROWNORM_ONE(TNAME, T, G, 4, 1); \
  REG_ROWNORM_ONE(TNAME, T, G, 1, 2); \
  REG_ROWNORM_ONE(TNAME, T, G, 2, 2); \
  REG_ROWNORM_ONE(TNAME, T, G, 4, 2); \
  REG_ROWNORM_ONE(TNAME, T, G, 1, 4); \
  REG_ROWNORM_ONE(TNAME, T, G, 2, 4)

#define REG_ROWNORM_T(TNAME, T)       \
  REG_ROWNORM_ONE(TNAME, T, 32, 1, 1); \
  REG_ROWNORM_ONE(TNAME, T, 32, 2, 1); \
  REG_ROWNORM_ONE(TNAME, T, 32, 4, 1); \
  REG_ROWNORM_G(TNAME, T, 128);       \
  REG_ROWNORM_G(TNAME, T, 256);       \
  REG_ROWNORM_G(TNAME, T, 512);       \
  REG_ROWNORM_ONE(TNAME, T, 1024, 1, 1); \
  REG_ROWNORM_ONE(TNAME, T, 1024, 2, 1); \
  REG_ROWNORM_ONE(TNAME, T, 1024, 4, 1); \
  CINN_B200_REGISTER_KERNEL_PDL("rownorm_cluster_" TNAME, 9, 512, k_rownorm_cluster<T>)

REG_ROWNORM_T("f32", float);
REG_ROWNORM_T("f16", __half);
REG_ROWNORM_T("bf16", __nv_bfloat16);

}  // namespace cinn_b200
