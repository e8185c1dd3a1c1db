// Reductions that keep a middle axis: x viewed as [A, B, I], reduced over A and I, result [B].  This is the
// per-channel statistic of an NCHW tensor (A = N, B = C, I = H*W: reduce over dims 0, 2, 3), the reduction
// batch_norm_train is decomposed into (cinn/frontend/decomposer/batch_norm.cc:60-92: mean = reduce_sum(x) / nhw,
// variance = reduce_sum(x * x) / nhw - mean * mean).  The reference lowers it as a reduce over non-adjacent axes
// (cinn/hlir/pe/reduction.cc:139-227, serial per output element); two such reduces of the same tensor are fused
// horizontally into one kernel there (cinn/hlir/pass/fusion_merge_pass.cc:85-460).
//
// Here one launch streams x once: CTA (b, s) walks the work items (a, chunk of I) s, s + splits, ... of channel b
// with four 16-byte loads in flight per thread and writes one partial per accumulation to scratch [splits][B];
// a column reduction over the splits finishes.  The DUAL form keeps two accumulations, sum and sum of squares, for
// the two-output group {reduce_sum(x), reduce_sum(x * x)}.  Squares are rounded products added without fma, as a
// materialised producer would be.
#include "device_math.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

template <class OpA, class OpB, bool DUAL>
__global__ void __launch_bounds__(256)
    k_mid_keep_reduce(const float* __restrict__ x, float* __restrict__ pa, float* __restrict__ pb, long long A,
                      long long B, long long I, long long chunks, long long splits, long long vec_ok) {
  __shared__ float scratch[32];
  const long long b = blockIdx.x % B, s = blockIdx.x / B;
  const long long items = A * chunks;
  float a0 = OpA::identity(), a1 = OpB::identity();
  if (vec_ok) {
    const int nvec = (int)(I >> 2);
    const int per  = (int)((nvec + chunks - 1) / chunks);
    for (long long it = s; it < items; it += splits) {
      const long long a = it / chunks;
      const int chunk   = (int)(it - a * chunks);
      const int begin = chunk * per, end = min(begin + per, nvec);
      const uint4* px = reinterpret_cast<const uint4*>(x + (a * B + b) * I);
      const int T     = blockDim.x;
      for (int v = begin + threadIdx.x; v < end; v += 4 * T) {
        uint4 r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (v + j * T < end) r[j] = __ldcs(px + v + j * T);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (v + j * T < end) {
            float f[4];
            unpack4(r[j], f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              a0 = OpA::accum(a0, f[i]);
              if (DUAL) a1 = OpB::accum(a1, f[i]);
            }
          }
        }
      }
    }
  } else {
    const long long per = (I + chunks - 1) / chunks;
    for (long long it = s; it < items; it += splits) {
      const long long a = it / chunks, chunk = it - a * chunks;
      const long long begin = chunk * per, end = min(begin + per, I);
      const float* px = x + (a * B + b) * I;
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float f = px[i];
        a0            = OpA::accum(a0, f);
        if (DUAL) a1 = OpB::accum(a1, f);
      }
    }
  }
  a0 = cta_allreduce<OpA>(a0, scratch);
  if (DUAL) a1 = cta_allreduce<OpB>(a1, scratch);
  if (threadIdx.x == 0) {
    pa[s * B + b] = a0;
    if (DUAL) pb[s * B + b] = a1;
  }
}

}  // namespace

#define REG_MID(OPNAME, OP) \
  CINN_B200_REGISTER_KERNEL("mid_keep_reduce_" OPNAME "_f32", 9, 256, k_mid_keep_reduce<OP, OP, false>)
REG_MID("sum", SumOp);
REG_MID("prod", ProdOp);
REG_MID("max", MaxOp);
REG_MID("min", MinOp);
REG_MID("sumsq", SumSquareOp);
REG_MID("sumabs", SumAbsOp);
REG_MID("maxabs", MaxAbsOp);
CINN_B200_REGISTER_KERNEL("mid_keep_reduce_sum_sumsq_f32", 9, 256, k_mid_keep_reduce<SumOp, SumSquareOp, true>);

}  // namespace cinn_b200
