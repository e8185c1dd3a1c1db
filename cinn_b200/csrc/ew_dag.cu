// Elementwise / broadcast groups that are not chains: a register program over up to eight inputs and four outputs.
//
// The reference fuses any connected set of elementwise and broadcast ops into one kernel, including values that are
// used more than once and groups with several outputs (cinn/hlir/pass/op_fusion_pass.cc:211-317 vertical fusion,
// cinn/hlir/pass/fusion_merge_pass.cc:85-460 horizontal fusion of consumers; lowered by inlining every producer,
// cinn/hlir/framework/op_lowering.cc:247-310).  The chain kernels cover one value flowing through a sequence of ops;
// this kernel covers the rest: the matcher (MatchDag in chain_match.cc) orders the group's ops, assigns each live value
// one of eight vector registers, and emits LOAD / op / STORE steps (ew_chain.h).  Every value is evaluated at the
// output's flat index, so an operand computed at a smaller shape (bias + bias, then broadcast) is simply recomputed
// per element from inputs addressed by the broadcast rule of cinn/hlir/pe/broadcast.cc:35-273.  The arithmetic is
// that of the chain kernels (apply_unary / apply_binary of ew_chain_device.cuh: the x86 path's formulas, fused
// multiply-add only where the reference contracts, 16-bit values rounded after every op).
//
// Two forms, as for the chains: the interpreting kernel decodes the steps at run time and keeps its registers in
// local memory (a catch-all, not fast); programs listed in ew_dag_static_table.inc are also compiled with the
// steps as template arguments, where every register index is a constant and the registers are real ones.
#include "ew_chain_body.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

struct DagInputs {
  const void* ptr[DAG_MAX_IN];
  long long mid[DAG_MAX_IN], inner[DAG_MAX_IN];
};
struct DagOutputs {
  void* ptr[DAG_MAX_OUT];
};

template <int VEC>
__device__ __forceinline__ void dag_operand(int sel, float imm, float imm2, const float (&regs)[DAG_REGS][VEC],
                                            float (&o)[VEC]) {
  if (sel < DAG_REGS) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = regs[sel][i];
  } else {
    const float v = sel == DAG_IMM ? imm : imm2;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = v;
  }
}

// One step on VEC elements starting at flat index i0.  Returns true when the step used the next word's immediate.
template <int VEC>
__device__ __forceinline__ bool dag_step(unsigned w, float imm, float imm2, unsigned long long meta,
                                         const DagInputs& in, const DagOutputs& out, long long i0,
                                         float (&regs)[DAG_REGS][VEC]) {
  const int op = (int)(w & 0xff), dst = (int)((w >> 8) & 15), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31),
            c = (int)((w >> 22) & 31);
  if (op == EW_NOP) return false;
  if (op == DAG_LOAD) {
    const SideSpec s = {in.ptr[a], (int)((meta >> (6 * a)) & 7), (int)((meta >> (6 * a + 3)) & 7), in.mid[a], in.inner[a]};
    load_side<VEC>(s, i0, regs[dst]);
    return false;
  }
  if (op == DAG_STORE) {
    const Store2 st = {out.ptr[dst], (int)((meta >> (48 + 3 * dst)) & 7), i0, 0};
    store_second<VEC>(st, regs[a]);
    return false;
  }
  const bool two = a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE;
  float x[VEC];
  dag_operand<VEC>(a, imm, imm2, regs, x);
  if (op >= EW_FIRST_UNARY) {
    apply_unary<VEC>(op, imm, x);
  } else if (op == EW_FMA) {
    float y[VEC], z[VEC];
    dag_operand<VEC>(b, imm, imm2, regs, y);
    dag_operand<VEC>(c, imm, imm2, regs, z);
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = fmaf(x[i], y[i], z[i]);
  } else if (op == EW_SELECT) {
    float y[VEC], z[VEC];
    dag_operand<VEC>(b, imm, imm2, regs, y);
    dag_operand<VEC>(c, imm, imm2, regs, z);
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = x[i] != 0.0f ? y[i] : z[i];
  } else if (op == EW_SCALE_PRE) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = imm * (x[i] + imm2);
  } else {
    float y[VEC];
    dag_operand<VEC>(b, imm, imm2, regs, y);
    apply_binary<VEC>(op, false, y, x);  // x = x (op) y
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) regs[dst][i] = x[i];
  return two;
}

__device__ __forceinline__ float word_imm(long long w) { return __uint_as_float((uint32_t)(w >> 32)); }

struct DynDag {
  const long long* steps;
  int nsteps;
  unsigned long long meta;
  template <int VEC>
  __device__ __forceinline__ void run(const DagInputs& in, const DagOutputs& out, long long i0) const {
    float regs[DAG_REGS][VEC];
    for (int k = 0; k < nsteps; ++k)
      if (dag_step<VEC>((unsigned)steps[k], word_imm(steps[k]), word_imm(steps[k + 1]), meta, in, out, i0, regs)) ++k;
  }
};

template <int VEC, unsigned long long META, int K, uint32_t... SIG>
__device__ __forceinline__ void dag_run_static(const long long* steps, const DagInputs& in, const DagOutputs& out,
                                               long long i0, float (&regs)[DAG_REGS][VEC]) {
  constexpr int N = (int)sizeof...(SIG);
  if constexpr (K < N) {
    constexpr uint32_t sig[N] = {SIG...};
    constexpr uint32_t w = sig[K];
    constexpr int op = (int)(w & 0xff), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31), c = (int)((w >> 22) & 31);
    constexpr bool two = op != EW_NOP && op != DAG_LOAD && op != DAG_STORE &&
                         (a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE);
    (void)dag_step<VEC>(w, word_imm(steps[K]), word_imm(steps[K + 1 < DAG_MAX_STEPS ? K + 1 : K]), META, in, out, i0, regs);
    dag_run_static<VEC, META, K + (two ? 2 : 1), SIG...>(steps, in, out, i0, regs);
  }
}
template <unsigned long long META, uint32_t... SIG>
struct StaticDag {
  const long long* steps;
  template <int VEC>
  __device__ __forceinline__ void run(const DagInputs& in, const DagOutputs& out, long long i0) const {
    float regs[DAG_REGS][VEC];
    dag_run_static<VEC, META, 0, SIG...>(steps, in, out, i0, regs);
  }
};

// SEP vectors of four elements per thread iteration, each run through the program on its own.
template <int SEP, class Prog>
__device__ __forceinline__ void dag_body(const Prog& prog, const DagInputs& in, const DagOutputs& out, long long n,
                                         long long vec_ok) {
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long done         = 0;
  if (vec_ok) {
    const long long nvec = n >> 2;
    long long v          = tid;
    if constexpr (SEP == 2) {
      for (; v + stride < nvec; v += 2 * stride) {
        prog.template run<4>(in, out, v << 2);
        prog.template run<4>(in, out, (v + stride) << 2);
      }
    }
    for (; v < nvec; v += stride) prog.template run<4>(in, out, v << 2);
    done = nvec << 2;
  }
  for (long long i = done + tid; i < n; i += stride) prog.template run<1>(in, out, i);
}

#define DAG_PARAMS                                                                                                    \
  const void *__restrict__ i0, const void *__restrict__ i1, const void *__restrict__ i2, const void *__restrict__ i3, \
      const void *__restrict__ i4, const void *__restrict__ i5, const void *__restrict__ i6,                         \
      const void *__restrict__ i7, void *__restrict__ o0, void *__restrict__ o1, void *__restrict__ o2,              \
      void *__restrict__ o3, long long n, long long vec_ok, long long meta, long long m0, long long n0,              \
      long long m1, long long n1, long long m2, long long n2, long long m3, long long n3, long long m4, long long n4, \
      long long m5, long long n5, long long m6, long long n6, long long m7, long long n7, long long nsteps_ll,       \
      long long t0, long long t1, long long t2, long long t3, long long t4, long long t5, long long t6, long long t7, \
      long long t8, long long t9, long long t10, long long t11, long long t12, long long t13, long long t14,          \
      long long t15, long long t16, long long t17, long long t18, long long t19, long long t20, long long t21,        \
      long long t22, long long t23, long long t24, long long t25, long long t26, long long t27, long long t28,        \
      long long t29
#define DAG_UNPACK                                                                                                    \
  const DagInputs in = {{i0, i1, i2, i3, i4, i5, i6, i7}, {m0, m1, m2, m3, m4, m5, m6, m7},                          \
                        {n0, n1, n2, n3, n4, n5, n6, n7}};                                                            \
  const DagOutputs out = {{o0, o1, o2, o3}};                                                                          \
  const long long steps[DAG_MAX_STEPS + 1] = {t0,  t1,  t2,  t3,  t4,  t5,  t6,  t7,  t8,  t9,  t10, t11, t12, t13, t14, t15, \
                                              t16, t17, t18, t19, t20, t21, t22, t23, t24, t25, t26, t27, t28, t29, 0}

__global__ void __launch_bounds__(256) k_ew_dag(DAG_PARAMS) {
  grid_dependency_sync();
  DAG_UNPACK;
  const DynDag prog = {steps, (int)nsteps_ll, (unsigned long long)meta};
  dag_body<1>(prog, in, out, n, vec_ok);
}

template <unsigned long long META, uint32_t... SIG>
__global__ void __launch_bounds__(256) k_ew_dag_static(DAG_PARAMS) {
  grid_dependency_sync();
  DAG_UNPACK;
  const StaticDag<META, SIG...> prog = {steps};
  dag_body<2>(prog, in, out, n, vec_ok);
}

template <uint32_t... SIG>
StaticChainKey MakeKey(const char* base, long long meta) {
  StaticChainKey k = {base, meta, (int)sizeof...(SIG), {SIG...}};
  return k;
}

}  // namespace

CINN_B200_REGISTER_KERNEL_PDL("ew_dag", 62, 256, k_ew_dag);

#define STATIC_DAG(ID, META, ...)                                                                     \
  CINN_B200_REGISTER_KERNEL_PDL("ew_dag_static_" #ID, 62, 256, k_ew_dag_static<META##ull, __VA_ARGS__>); \
  static int cinn_b200_static_dag_##ID = RegisterStaticChain(MakeKey<__VA_ARGS__>("ew_dag", META##ll), "ew_dag_static_" #ID)

#include "ew_dag_static_table.inc"

}  // namespace cinn_b200
