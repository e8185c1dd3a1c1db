// Reductions that keep a middle axis: x viewed as [A, B, I], reduced over A and I, result [B].  This is the
// per-channel statistic of an NCHW tensor (A = N, B = C, I = H*W: reduce over dims 0, 2, 3), the reduction
// batch_norm_train is decomposed into (cinn/frontend/decomposer/batch_norm.cc:60-92: mean = reduce_sum(x) / nhw,
// variance = reduce_sum(x * x) / nhw - mean * mean).  The reference lowers it as a reduce over non-adjacent axes
// (cinn/hlir/pe/reduction.cc:139-227, serial per output element); two such reduces of the same tensor are fused
// horizontally into one kernel there (cinn/hlir/pass/fusion_merge_pass.cc:85-460).
//
// Here one launch streams x once: CTA (b, s) walks the work items (a, chunk of I) s, s + splits, ... of channel b as
// one flat list of 16-byte vectors with four loads in flight per thread, and writes one partial per accumulation
// to scratch [splits][B].  The last CTA of a channel to finish (a ticket counter per channel in scratch, zero
// between launches) folds the channel's partials in a fixed order and writes the result, so there is no second
// launch and the result does not depend on which CTA came last.  The DUAL form keeps two accumulations, sum and sum
// of squares, for the two-output group {reduce_sum(x), reduce_sum(x * x)}.  Squares are rounded products added
// without fma, as a materialised producer would be.
#include <type_traits>
#include "device_math.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

// GRAD: the statistics pass of the decomposed batch_norm_grad (cinn/frontend/decomposer/batch_norm.cc:62-72): x is
// y_grad, x2 the forward input, `mean` the saved per-channel mean; the two accumulations are
// reduce_sum(y_grad) and reduce_sum(y_grad * (x2 - mean)), difference and product rounded, no fma.
// The vector walk of k_mid_keep_reduce: the work items s, s + splits, ... of channel b as one flat list of 16-byte
// vectors.  (k, v) = (item, vector inside the item) of the flat index, advanced incrementally: no division per load.
// Four vectors in flight per thread and stream (eight were slower, with and without the per-vector tests: fewer,
// longer iterations per CTA -- 16-bit statistics 0.79 against 0.84 of the HBM peak).  IdxT: the type
// of the index arithmetic.
template <class OpA, class OpB, bool DUAL, bool GRAD, typename T, typename IdxT>
__device__ __forceinline__ void walk_vectors(const uint4* __restrict__ px, const uint4* __restrict__ px2, float mu,
                                             long long A_, long long B_, long long I_, long long chunks_,
                                             long long splits_, long long b_, long long s_, long long my_items,
                                             float& a0, float& a1) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 4;
  const IdxT B = (IdxT)B_, chunks = (IdxT)chunks_, splits = (IdxT)splits_, b = (IdxT)b_, s = (IdxT)s_;
  const IdxT T_    = (IdxT)blockDim.x;
  const IdxT nvec  = (IdxT)(I_ / V);
  const IdxT per   = (nvec + chunks - 1) / chunks;
  const IdxT total = (IdxT)my_items * per;
  IdxT k = (IdxT)threadIdx.x / per, v = (IdxT)threadIdx.x - k * per;
  const IdxT step_k = T_ / per, step_v = T_ - step_k * per;  // one stride of T_ vectors
  // one loaded vector into the accumulators
  auto fold = [&](const uint4& rv, const uint4& rv2) {
    if constexpr (sizeof(T) == 2 && DUAL && !GRAD && std::is_same<OpA, SumOp>::value &&
                  std::is_same<OpB, SumSquareOp>::value) {
      // sum and sum of squares of 16-bit values with the mixed-precision add / fma of sm_100 (the operand is
      // widened inside the instruction: no conversion instructions; x * x is exact in fp32, so the fma rounds
      // exactly where a + x * x does)
      const unsigned short* h = reinterpret_cast<const unsigned short*>(&rv);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        if constexpr (std::is_same<T, __half>::value) {
          asm("add.rn.f32.f16 %0, %1, %0;" : "+f"(a0) : "h"(h[i]));
          asm("fma.rn.f32.f16 %0, %1, %1, %0;" : "+f"(a1) : "h"(h[i]));
        } else {
          asm("add.rn.f32.bf16 %0, %1, %0;" : "+f"(a0) : "h"(h[i]));
          asm("fma.rn.f32.bf16 %0, %1, %1, %0;" : "+f"(a1) : "h"(h[i]));
        }
      }
    } else {
      float f[V], f2[V];
      Io<T>::unpack(rv, f);
      if (GRAD) Io<T>::unpack(rv2, f2);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        a0 = OpA::accum(a0, f[i]);
        if (GRAD) a1 = a1 + f[i] * (f2[i] - mu);
        else if (DUAL) a1 = OpB::accum(a1, f[i]);
      }
    }
  };
  for (IdxT idx = threadIdx.x; idx < total; idx += U * T_) {
    uint4 r[U], r2[GRAD ? U : 1];
    if (chunks == 1 && idx + (IdxT)(U - 1) * T_ < total) {
      // Whole items (no chunking) and all U vectors in range -- every iteration of a thread but its last: no test
      // per vector, so the U loads are issued together and the folds run straight through.
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const IdxT at = ((s + k * splits) * B + b) * nvec + v;
        r[j]          = __ldcs(px + at);
        if (GRAD) r2[GRAD ? j : 0] = __ldcs(px2 + at);
        k += step_k;
        v += step_v;
        if (v >= per) {
          v -= per;
          ++k;
        }
      }
#pragma unroll
      for (int j = 0; j < U; ++j) fold(r[j], r2[GRAD ? j : 0]);
      continue;
    }
    bool ok[U];
#pragma unroll
    for (int j = 0; j < U; ++j) {
      ok[j] = false;
      if (idx + (IdxT)j * T_ < total) {
        const IdxT it = s + k * splits;
        IdxT a = it, chunk = 0;
        if (chunks != 1) {
          a     = (unsigned)it / (unsigned)chunks;  // items < 2^31 (checked by the planner)
          chunk = it - a * chunks;
        }
        const IdxT vv = chunk * per + v;
        if (vv < nvec) {
          const IdxT at = (a * B + b) * nvec + vv;
          r[j]          = __ldcs(px + at);
          if (GRAD) r2[GRAD ? j : 0] = __ldcs(px2 + at);
          ok[j] = true;
        }
      }
      k += step_k;
      v += step_v;
      if (v >= per) {
        v -= per;
        ++k;
      }
    }
#pragma unroll
    for (int j = 0; j < U; ++j)
      if (ok[j]) fold(r[j], r2[GRAD ? j : 0]);
  }
}

// T: storage type of x (and x2): float, or a 16-bit float widened on load as the casts the AutoCast pass puts around
// batch_norm_train / batch_norm_grad would (cinn/frontend/pass/auto_cast.cc:138-214); everything else is float32.
template <class OpA, class OpB, bool DUAL, bool GRAD = false, typename T = float>
__global__ void __launch_bounds__(256)
    k_mid_keep_reduce(const T* __restrict__ x, const T* __restrict__ x2, const float* __restrict__ mean,
                      float* __restrict__ pa, float* __restrict__ pb, unsigned int* __restrict__ tickets,
                      float* __restrict__ ya, float* __restrict__ yb, long long A, long long B, long long I,
                      long long chunks, long long splits, long long vec_ok) {
  __shared__ float scratch[32];
  __shared__ unsigned int ticket;
  const long long b = blockIdx.x % B, s = blockIdx.x / B;
  const float mu    = GRAD ? mean[b] : 0.0f;
  const long long items    = A * chunks;
  const long long my_items = s < items ? (items - s + splits - 1) / splits : 0;
  float a0 = OpA::identity(), a1 = OpB::identity();
  const int T_ = blockDim.x;
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte vector
  if (vec_ok) {
    const uint4* px  = reinterpret_cast<const uint4*>(x);
    const uint4* px2 = reinterpret_cast<const uint4*>(x2);
    // Index arithmetic in 32 bits whenever the tensor has fewer than 2^31 vectors (64-bit multiplies per load cost
    // as much as the arithmetic on the loaded values, and with 16-bit storage made the kernel issue-bound).
    if (A * B * (I / V) < (1ll << 31))
      walk_vectors<OpA, OpB, DUAL, GRAD, T, unsigned>(px, px2, mu, A, B, I, chunks, splits, b, s, my_items, a0, a1);
    else
      walk_vectors<OpA, OpB, DUAL, GRAD, T, long long>(px, px2, mu, A, B, I, chunks, splits, b, s, my_items, a0, a1);
  } else {
    const long long per = (I + chunks - 1) / chunks;
    for (long long it = s; it < items; it += splits) {
      const long long a = it / chunks, chunk = it - a * chunks;
      const long long begin = chunk * per, end = min(begin + per, I);
      const T* px = x + (a * B + b) * I;
      for (long long i = begin + threadIdx.x; i < end; i += T_) {
        const float f = Io<T>::load1(px + i);
        a0            = OpA::accum(a0, f);
        if (GRAD) a1 = a1 + f * (Io<T>::load1(x2 + (a * B + b) * I + i) - mu);
        else if (DUAL) a1 = OpB::accum(a1, f);
      }
    }
  }
  a0 = cta_allreduce<OpA>(a0, scratch);
  if (DUAL) a1 = cta_allreduce<OpB>(a1, scratch);
  if (threadIdx.x == 0) {
    pa[s * B + b] = a0;
    if (DUAL) pb[s * B + b] = a1;
    __threadfence();
    ticket = atomicAdd(&tickets[b], 1u);
  }
  __syncthreads();
  if (ticket != (unsigned)(splits - 1)) return;
  // Last CTA of channel b: every partial of the channel is visible (fence + ticket); fold them in split order.
  __threadfence();
  float t0 = OpA::identity(), t1 = OpB::identity();
  for (long long k = threadIdx.x; k < splits; k += T_) {
    t0 = OpA::apply(t0, __ldcg(pa + k * B + b));
    if (DUAL) t1 = OpB::apply(t1, __ldcg(pb + k * B + b));
  }
  t0 = cta_allreduce<OpA>(t0, scratch);
  if (DUAL) t1 = cta_allreduce<OpB>(t1, scratch);
  if (threadIdx.x == 0) {
    ya[b] = t0;
    if (DUAL) yb[b] = t1;
    tickets[b] = 0;  // ready for the next launch
  }
}

}  // namespace

#define REG_MID(OPNAME, OP) \
  CINN_B200_REGISTER_KERNEL("mid_keep_reduce_" OPNAME "_f32", 14, 256, k_mid_keep_reduce<OP, OP, false>)
REG_MID("sum", SumOp);
REG_MID("prod", ProdOp);
REG_MID("max", MaxOp);
REG_MID("min", MinOp);
REG_MID("sumsq", SumSquareOp);
REG_MID("sumabs", SumAbsOp);
REG_MID("maxabs", MaxAbsOp);
CINN_B200_REGISTER_KERNEL("mid_keep_reduce_sum_sumsq_f32", 14, 256, k_mid_keep_reduce<SumOp, SumSquareOp, true>);
CINN_B200_REGISTER_KERNEL("bn_grad_stats_f32", 14, 256, k_mid_keep_reduce<SumOp, SumOp, true, true>);
CINN_B200_REGISTER_KERNEL("mid_keep_reduce_sum_sumsq_f16", 14, 256, k_mid_keep_reduce<SumOp, SumSquareOp, true, false, __half>);
CINN_B200_REGISTER_KERNEL("mid_keep_reduce_sum_sumsq_bf16", 14, 256, k_mid_keep_reduce<SumOp, SumSquareOp, true, false, __nv_bfloat16>);
CINN_B200_REGISTER_KERNEL("bn_grad_stats_f16", 14, 256, k_mid_keep_reduce<SumOp, SumOp, true, true, __half>);
CINN_B200_REGISTER_KERNEL("bn_grad_stats_bf16", 14, 256, k_mid_keep_reduce<SumOp, SumOp, true, true, __nv_bfloat16>);

}  // namespace cinn_b200
