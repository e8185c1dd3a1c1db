// Generic elementwise / broadcast fused group: a linear chain of ops evaluated in registers, one HBM pass.
//
// This is the catch-all for kElementWise / kBroadcast groups that have no dedicated kernel: the group's
// expression is linearised by the matcher into a short program (at most 16 steps) that starts from one input
// ("the chain") and applies one op per step with, at most, side operands taken from up to three other inputs
// or immediates.  It covers what the reference generates for such groups after inlining
// (cinn/hlir/framework/op_lowering.cc:247-310) with the x86 path's arithmetic: unary math as in
// cinn/hlir/pe/elementwise.cc:33-108 and cinn/backends/llvm/llvm_intrin_rule.h, binary ops with the broadcast
// index rule of cinn/hlir/pe/broadcast.cc:35-273, scale (cinn/hlir/op/elementwise.cc:149-163), cast
// (cinn/hlir/pe/elementwise.cc:213-217) and the Mul+Add -> fma contraction of cinn/optim/lower_intrin.cc:41-59.
// The program is interpreted per 4-element vector; every thread of a warp takes the same branch, so the cost
// of the dispatch is shared by the vector.
#include "ew_chain_body.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

// meta: bits 0-3 dtype of side 1, 4-7 mode of side 1, 8-11 / 12-15 side 2, 16-19 / 20-23 side 3, 24-27 dtype of in0,
// 36-39 storage type of the second output `out2` (written by EW_STORE2; kernels with temporaries only).
// NT = 2: the variant with two temporaries for expression trees; it takes one vector per iteration so that the
// temporaries fit the same register budget.
// ST2: the variant whose programs may store a second output (EW_STORE2) into `out2`.
template <typename OutT, int NS, int NT = 0, bool ST2 = (NT > 0)>
__global__ void __launch_bounds__(256, NS == 0 ? 6 : (NS == 1 ? 5 : 4))
    k_ew_chain(const void* __restrict__ in0, const void* __restrict__ p1, const void* __restrict__ p2,
               const void* __restrict__ p3, OutT* __restrict__ out, long long n, long long vec_ok, long long meta,
               long long mid1, long long inner1, long long mid2, long long inner2, long long mid3, long long inner3,
               long long nsteps_ll, long long t0, long long t1, long long t2, long long t3, long long t4,
               long long t5, long long t6, long long t7, long long t8, long long t9, long long t10, long long t11,
               long long t12, long long t13, long long t14, long long t15, void* __restrict__ out2) {
  grid_dependency_sync();
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0};
  const DynProgram prog    = {steps, (int)nsteps_ll, meta};
  const ChainGeometry geo  = {n, vec_ok, mid1, inner1, mid2, inner2, mid3, inner3};
  // Two vectors (8 elements) per thread iteration: all of their loads are issued before the program runs, and one
  // pass of the interpreter serves the eight elements.
  ew_chain_body<OutT, NS, NT, ST2, 2>(prog, in0, p1, p2, p3, out, geo, out2);
}

}  // namespace

#define REG_CHAIN(OUTNAME, OutT)                                                               \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_" OUTNAME "_s0", 32, 256, k_ew_chain<OutT, 0>);        \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_" OUTNAME "_s1", 32, 256, k_ew_chain<OutT, 1>);        \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_" OUTNAME "_s3", 32, 256, k_ew_chain<OutT, 3>);        \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_" OUTNAME "_s3t", 32, 256, k_ew_chain<OutT, 3, 2>);    \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_" OUTNAME "_s1o", 32, 256, k_ew_chain<OutT, 1, 0, true>); \
  CINN_B200_REGISTER_KERNEL_PDL("ew_chain_" OUTNAME "_s3o", 32, 256, k_ew_chain<OutT, 3, 0, true>)
REG_CHAIN("f32", float);
REG_CHAIN("f16", __half);
REG_CHAIN("bf16", __nv_bfloat16);
REG_CHAIN("bool", uint8_t);
REG_CHAIN("i32", int32_t);
REG_CHAIN("i64", long long);

}  // namespace cinn_b200
