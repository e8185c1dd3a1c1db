// Reduction fused-group kernels: reduce_{sum,prod,max,min} over a tensor viewed as [outer, r, inner].
//
// inner == 1 is the "row" (last-axis) reduction the reference lowers with TwoStepBlockReduceInternal /
// BlockReduceInternal and cinn_block_reduce_*_internal (cinn/hlir/pe/reduction.cc:304-362, 668-834,
// cinn/runtime/cuda/cinn_cuda_runtime_source.cuh:459-575); inner > 1 is the "column" reduction it lowers as
// a per-thread serial loop or a block-shuffle two-step (cinn/hlir/pe/reduction.cc:546-644,
// cinn/hlir/pe/ir_schedule_pe.cc:306-353).  Initial values follow cinn/lang/builtin.cc:123-143.
//
// Design: every thread issues several independent 16-byte loads before it combines them; a row is owned by
// a warp (short rows), a CTA (long rows) or a thread-block cluster that merges per-CTA partials through
// distributed shared memory (very long rows); reductions with too few outputs to fill 148 SMs are split
// along r into partials in caller-provided scratch memory and finished by a second launch.
#include <cooperative_groups.h>

#include "device_math.cuh"
#include "kernel_registry.h"

namespace cg = cooperative_groups;

namespace cinn_b200 {

template <class Op>
__device__ __forceinline__ float combine4(float acc, uint4 u) {
  acc = Op::accum(acc, __uint_as_float(u.x));
  acc = Op::accum(acc, __uint_as_float(u.y));
  acc = Op::accum(acc, __uint_as_float(u.z));
  acc = Op::accum(acc, __uint_as_float(u.w));
  return acc;
}

// ------------------------------------------------------------------------------------------------
// Row reduction, one warp per row, ITERS 16-byte loads per lane all issued before the first combine.
// Vector path (vec_ok != 0): r % 4 == 0, r <= ITERS*128, 16-byte aligned base.  Otherwise scalar loads,
// coalesced across the warp, for any r and alignment.  y[row] for row < rows.
// ------------------------------------------------------------------------------------------------
template <class Op, int ITERS>
__global__ void __launch_bounds__(256) k_row_reduce_warp(const float* __restrict__ x, float* __restrict__ y,
                                                         long long rows, long long r, long long vec_ok) {
  grid_dependency_sync();
  const int lane         = threadIdx.x & 31;
  const long long warp   = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec         = (int)(r >> 2);
  for (long long row = warp; row < rows; row += nwarps) {
    float acc = Op::identity();
    if (vec_ok) {
      const uint4* p = reinterpret_cast<const uint4*>(x + row * r);
      uint4 u[ITERS];
#pragma unroll
      for (int j = 0; j < ITERS; ++j) {
        const int v = lane + 32 * j;
        if (v < nvec) u[j] = __ldcs(p + v);
      }
#pragma unroll
      for (int j = 0; j < ITERS; ++j) {
        const int v = lane + 32 * j;
        if (v < nvec) acc = combine4<Op>(acc, u[j]);
      }
    } else {
      const float* p = x + row * r;
      for (long long c = lane; c < r; c += 32) acc = Op::accum(acc, p[c]);
    }
    acc = warp_allreduce<Op>(acc);
    if (lane == 0) y[row] = acc;
  }
}

// Per-thread partial over the segment [begin, end) of one row; the vector body needs x+begin 16-byte aligned.
template <class Op>
__device__ __forceinline__ float segment_partial(const float* __restrict__ p, long long begin, long long end,
                                                 bool vec_ok) {
  float acc = Op::identity();
  if (vec_ok) {
    const uint4* pv      = reinterpret_cast<const uint4*>(p + begin);
    const long long nvec = (end - begin) >> 2;
    const long long B    = blockDim.x;
    for (long long v = threadIdx.x; v < nvec; v += 4 * B) {
      uint4 u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v + j * B < nvec) u[j] = __ldcs(pv + v + j * B);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (v + j * B < nvec) acc = combine4<Op>(acc, u[j]);
    }
    for (long long c = begin + (nvec << 2) + threadIdx.x; c < end; c += blockDim.x) acc = Op::accum(acc, p[c]);
  } else {
    for (long long c = begin + threadIdx.x; c < end; c += blockDim.x) acc = Op::accum(acc, p[c]);
  }
  return acc;
}

// ------------------------------------------------------------------------------------------------
// Row reduction, one CTA per (row, split): y[row*splits + split] = reduce over the split's segment.
// With splits == 1 this writes the final result; with splits > 1 `y` is scratch [rows, splits] that a
// second (warp-per-row) launch finishes.  seg is a multiple of 4 so that segments stay 16-byte aligned.
// ------------------------------------------------------------------------------------------------
template <class Op>
__global__ void __launch_bounds__(512) k_row_reduce_cta(const float* __restrict__ x, float* __restrict__ y,
                                                        long long rows, long long r, long long splits,
                                                        long long seg, long long vec_ok) {
  grid_dependency_sync();
  __shared__ float scratch[32];
  const long long n_ctas = rows * splits;
  for (long long cta = blockIdx.x; cta < n_ctas; cta += gridDim.x) {
    const long long row   = cta / splits;
    const long long split = cta - row * splits;
    const long long begin = split * seg;
    const long long end   = min(begin + seg, r);
    float acc             = begin < end ? segment_partial<Op>(x + row * r, begin, end, vec_ok != 0) : Op::identity();
    acc                   = cta_allreduce<Op>(acc, scratch);
    if (threadIdx.x == 0) y[cta] = acc;
  }
}

// ------------------------------------------------------------------------------------------------
// Row reduction, one thread-block cluster per row: each CTA of the cluster reduces one segment of the row,
// stores its partial into the shared memory of the cluster's rank-0 CTA (distributed shared memory), and
// after a cluster barrier rank 0 combines the partials and writes the result.  One launch, no scratch.
// gridDim.x = rows_per_wave * cluster size; cluster dimension given at launch.
// ------------------------------------------------------------------------------------------------
template <class Op>
__global__ void __launch_bounds__(512) k_row_reduce_cluster(const float* __restrict__ x, float* __restrict__ y,
                                                            long long rows, long long r, long long seg,
                                                            long long vec_ok) {
  grid_dependency_sync();
  __shared__ float scratch[32];
  __shared__ float partials[16];
  cg::cluster_group cluster  = cg::this_cluster();
  const unsigned rank        = cluster.block_rank();
  const unsigned csize       = cluster.num_blocks();
  const long long n_clusters = gridDim.x / csize;
  const long long cluster_id = blockIdx.x / csize;
  for (long long row = cluster_id; row < rows; row += n_clusters) {
    const long long begin = (long long)rank * seg;
    const long long end   = min(begin + seg, r);
    float acc             = begin < end ? segment_partial<Op>(x + row * r, begin, end, vec_ok != 0) : Op::identity();
    acc                   = cta_allreduce<Op>(acc, scratch);
    if (threadIdx.x == 0) {
      float* remote = cluster.map_shared_rank(partials, 0);
      remote[rank]  = acc;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x < 32) {
      float v = threadIdx.x < csize ? partials[threadIdx.x] : Op::identity();
      v       = warp_allreduce<Op>(v);
      if (threadIdx.x == 0) y[row] = v;
    }
    cluster.sync();  // partials of rank 0 are reused by the next row
  }
}

// ------------------------------------------------------------------------------------------------
// Column reduction: x viewed as [outer, r, inner]; out[(split*outer + o)*inner + i] = reduce over the
// split's rows k of x[(o*r + k)*inner + i].  One thread per 16-byte column group (vec_ok: inner % 4 == 0 and
// aligned pointers) or per column element, eight row loads in flight per thread; consecutive threads read
// consecutive addresses.  splits > 1 writes partials into scratch that a second launch of the same
// kernel reduces as [1, splits, outer*inner].
// grid = (column groups, min(outer, 65535), splits).
// ------------------------------------------------------------------------------------------------
template <class Op>
__global__ void __launch_bounds__(256) k_col_reduce(const float* __restrict__ x, float* __restrict__ y,
                                                    long long outer, long long r, long long inner,
                                                    long long rows_per_split, long long vec_ok) {
  grid_dependency_sync();
  const long long split  = blockIdx.z;
  const long long k0     = split * rows_per_split;
  const long long k1     = min(k0 + rows_per_split, r);
  const long long col0   = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long cstep  = (long long)gridDim.x * blockDim.x;  // the grid is sized for the vector path
  if (vec_ok) {
    const long long inner_v = inner >> 2;
    const long long col = col0;  // the grid covers every column group of the vector path
    if (col >= inner_v) return;
    for (long long o = blockIdx.y; o < outer; o += gridDim.y) {
      const uint4* p = reinterpret_cast<const uint4*>(x + o * r * inner) + col;
      float a0 = Op::identity(), a1 = a0, a2 = a0, a3 = a0;
      long long k = k0;
      for (; k + 8 <= k1; k += 8) {
        uint4 u[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) u[j] = __ldcs(p + (k + j) * inner_v);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          a0 = Op::accum(a0, __uint_as_float(u[j].x));
          a1 = Op::accum(a1, __uint_as_float(u[j].y));
          a2 = Op::accum(a2, __uint_as_float(u[j].z));
          a3 = Op::accum(a3, __uint_as_float(u[j].w));
        }
      }
      for (; k < k1; ++k) {
        uint4 u = __ldcs(p + k * inner_v);
        a0      = Op::accum(a0, __uint_as_float(u.x));
        a1      = Op::accum(a1, __uint_as_float(u.y));
        a2      = Op::accum(a2, __uint_as_float(u.z));
        a3      = Op::accum(a3, __uint_as_float(u.w));
      }
      uint4 out = make_uint4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3));
      reinterpret_cast<uint4*>(y + (split * outer + o) * inner)[col] = out;
    }
  } else {
    for (long long col = col0; col < inner; col += cstep)
    for (long long o = blockIdx.y; o < outer; o += gridDim.y) {
      const float* p = x + o * r * inner + col;
      float acc      = Op::identity();
      long long k    = k0;
      for (; k + 4 <= k1; k += 4) {
        float f0 = p[k * inner], f1 = p[(k + 1) * inner], f2 = p[(k + 2) * inner], f3 = p[(k + 3) * inner];
        acc = Op::accum(Op::accum(Op::accum(Op::accum(acc, f0), f1), f2), f3);
      }
      for (; k < k1; ++k) acc = Op::accum(acc, p[k * inner]);
      y[(split * outer + o) * inner + col] = acc;
    }
  }
}

#define REG_REDUCE_FAMILY(OPNAME, OP)                                                                       \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_warp1_" OPNAME "_f32", 5, 256, k_row_reduce_warp<OP, 1>);           \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_warp2_" OPNAME "_f32", 5, 256, k_row_reduce_warp<OP, 2>);           \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_warp4_" OPNAME "_f32", 5, 256, k_row_reduce_warp<OP, 4>);           \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_warp8_" OPNAME "_f32", 5, 256, k_row_reduce_warp<OP, 8>);           \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_warp16_" OPNAME "_f32", 5, 256, k_row_reduce_warp<OP, 16>);         \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_cta_" OPNAME "_f32", 7, 512, k_row_reduce_cta<OP>);                 \
  CINN_B200_REGISTER_KERNEL_PDL("row_reduce_cluster_" OPNAME "_f32", 6, 512, k_row_reduce_cluster<OP>);         \
  CINN_B200_REGISTER_KERNEL_PDL("col_reduce_" OPNAME "_f32", 7, 256, k_col_reduce<OP>)

REG_REDUCE_FAMILY("sum", SumOp);
REG_REDUCE_FAMILY("prod", ProdOp);
REG_REDUCE_FAMILY("max", MaxOp);
REG_REDUCE_FAMILY("min", MinOp);
// Reductions with an elementwise producer folded into the first pass (second passes over partials use the plain op).
REG_REDUCE_FAMILY("sumsq", SumSquareOp);
REG_REDUCE_FAMILY("sumabs", SumAbsOp);
REG_REDUCE_FAMILY("sumexp", SumExpOp);
REG_REDUCE_FAMILY("maxabs", MaxAbsOp);

}  // namespace cinn_b200
