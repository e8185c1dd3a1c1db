// Row programs (the kernels' code; row_prog.cu and row_prog_half.cu instantiate them): groups with reductions over the trailing axes and elementwise ops before, between and after them,
// as ONE kernel that keeps a row's traffic to HBM at one read and one write.
//
// The reference fuses a reduce with its elementwise producers, with other reduces of the same shape and with the
// broadcast / elementwise consumers of the reduced values while a row fits one thread block of 1024 threads
// (cinn/hlir/pass/op_fusion_pass.cc:258-276, op_fusion_pass_util.h:190-265, fusion_merge_pass_util.h:400-555; lowered
// by cinn/hlir/framework/op_lowering.cc:312-389).  Softmax and layer_norm have dedicated kernels here; this kernel is
// the general form for every other such composition: x / ||x||, x - mean(x), (x - max) / sum, several reductions of
// different tensors at once, relu(reduce_sum(x) * a + b).
//
// x is viewed as [rows, r].  A row is handled by a warp (`group` = 32, eight rows per CTA) or by a CTA (`group` = 256).
// The program (ew_chain.h) is a sequence of passes.  In a pass every thread runs the element program on its vectors of
// the row: loads, elementwise steps, ROWP_ACC steps that fold a value into one of the pass's accumulators, stores of
// full-size outputs.  The accumulators are then combined across the row's threads (lanes in a fixed tree, then warps in
// order), and every thread runs the scalar program on the row's scalar registers, which the next pass reads as
// operands.  A later pass evaluates what it needs again from the inputs: the row was just read by the same threads,
// so those loads come from L1 / L2, not from HBM.
//
// The arithmetic per op is that of the chain kernels (chain_step's helpers).  Reductions combine per-thread partials
// in a tree, as every reduction kernel of this library does (sums differ from the serial order by rounding only).
// As for the chains there is an interpreting kernel and, for the programs of row_prog_static_table.inc, kernels with
// the program as template arguments.  Those come in four forms (see row_program_body): a warp, half a CTA or a CTA
// per row, the latter in two sizes; all but the single-pass ones keep the row in registers between the passes
// instead of reading it again, ask the next row into L2 meanwhile, evaluate exp / tanh / sigmoid through the
// approximate exponential, and divide by a per-row value through one reciprocal per row.
#pragma once
#include "ew_chain_body.cuh"
#include "kernel_registry.h"
#include "row_prog_prefix.h"

namespace cinn_b200 {
namespace {

struct RowInputs {
  const void* ptr[DAG_MAX_IN];
  long long mid[DAG_MAX_IN], inner[DAG_MAX_IN];
  long long row_base, row_len;  // the flat index at which the current row starts; the row's length
};
struct RowOutputs {
  void* ptr[DAG_MAX_OUT];
};

__device__ __forceinline__ float rp_identity(int kind) {
  return kind == 0 ? 0.0f : (kind == 1 ? 1.0f : (kind == 2 ? -3.402823466e38f : 3.402823466e38f));
}
__device__ __forceinline__ float rp_fold(int kind, float a, float b) {
  switch (kind) {
    case 0: return a + b;
    case 1: return a * b;
    case 2: return a > b ? a : b;  // compare + select, as the x86 path (cinn/backends/llvm/codegen_llvm.cc:310-340)
    default: return a < b ? a : b;
  }
}

template <int VEC>
__device__ __forceinline__ void rp_operand(int sel, float imm, float imm2, const float (&regs)[DAG_REGS][VEC],
                                           const float (&sregs)[ROWP_SREGS], float (&o)[VEC]) {
  if (sel < DAG_REGS) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = regs[sel][i];
  } else {
    const float v = sel >= ROWP_SREG0 ? sregs[(sel - ROWP_SREG0) & 7] : (sel == DAG_IMM ? imm : imm2);
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = v;
  }
}

// One element-program step on VEC elements at flat index i0.  acc[k] is the accumulator whose total goes to scalar
// register k.  Returns true when the step used the next word's immediate.
// FAST: exp / tanh / sigmoid through the hardware's approximate exponential and reciprocal (about 1e-6 relative):
// every result of a row program depends on a row reduction and is judged at 1e-5 relative; the specialised kernels
// use it, the interpreting kernel computes the full-precision forms.
template <int VEC, bool FAST = false>
__device__ __forceinline__ bool rp_element_step(unsigned w, float imm, float imm2, unsigned long long meta,
                                                const RowInputs& in, const RowOutputs& out, long long i0,
                                                float (&regs)[DAG_REGS][VEC], const float (&sregs)[ROWP_SREGS],
                                                float (&acc)[ROWP_SREGS], bool reread, float (*cache)[4] = nullptr,
                                                int cache_mode = 0) {
  const int op = (int)(w & 0xff), dst = (int)((w >> 8) & 15), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31),
            c = (int)((w >> 22) & 31);
  if (op == EW_NOP) return false;
  if (op == DAG_LOAD) {
    const SideSpec s = {in.ptr[a], (int)((meta >> (6 * a)) & 7), (int)((meta >> (6 * a + 3)) & 7), in.mid[a], in.inner[a], in.row_base, in.row_len};
    // cache_mode 2: this full-size input of the row is already in this thread's registers
    if (VEC == 4 && cache_mode == 2 && s.mode == EW_SIDE_FULL) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) regs[dst][i] = cache[a][i & 3];
      return false;
    }
    load_side<VEC>(s, i0, regs[dst], !reread);  // a row that a later pass reads again stays in L1
    return false;
  }
  if (op == DAG_STORE) {
    const Store2 st = {out.ptr[dst], (int)((meta >> (48 + 3 * dst)) & 7), i0, 0};
    store_second<VEC>(st, regs[a]);
    return false;
  }
  if (op == ROWP_ACC) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[dst & 7] = rp_fold(c & 3, acc[dst & 7], regs[a & 7][i]);
    return false;
  }
  const bool two = a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE;
  float x[VEC];
  rp_operand<VEC>(a, imm, imm2, regs, sregs, x);
  if (op >= EW_FIRST_UNARY) {
    apply_unary<VEC, FAST>(op, imm, x);
  } else if (op == EW_FMA) {
    float y[VEC], z[VEC];
    rp_operand<VEC>(b, imm, imm2, regs, sregs, y);
    rp_operand<VEC>(c, imm, imm2, regs, sregs, z);
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = fmaf(x[i], y[i], z[i]);
  } else if (op == EW_SELECT) {
    float y[VEC], z[VEC];
    rp_operand<VEC>(b, imm, imm2, regs, sregs, y);
    rp_operand<VEC>(c, imm, imm2, regs, sregs, z);
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = x[i] != 0.0f ? y[i] : z[i];
  } else if (op == EW_SCALE_PRE) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = imm * (x[i] + imm2);
  } else if (op == EW_DIV && b >= ROWP_SREG0) {
    // Division by a per-row value (always a function of a reduction here): one reciprocal per row, a multiplication
    // per element, as the dedicated row kernels do.  Within 1.5 ulp of the true quotient; a result that depends on
    // a reduction is compared at 1e-5 relative.
    const float rcp = 1.0f / sregs[(b - ROWP_SREG0) & 7];
#pragma unroll
    for (int i = 0; i < VEC; ++i) x[i] = x[i] * rcp;
  } else {
    float y[VEC];
    rp_operand<VEC>(b, imm, imm2, regs, sregs, y);
    apply_binary<VEC>(op, false, y, x);
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) regs[dst][i] = x[i];
  return two;
}

// One scalar-program step: the registers are the row's scalar registers; loads and stores use the row index.
__device__ __forceinline__ bool rp_scalar_step(unsigned w, float imm, float imm2, unsigned long long meta,
                                               const RowInputs& in, const RowOutputs& out, long long row, bool writer,
                                               float (&sregs)[ROWP_SREGS]) {
  const int op = (int)(w & 0xff), dst = (int)((w >> 8) & 15), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31),
            c = (int)((w >> 22) & 31);
  if (op == EW_NOP) return false;
  if (op == DAG_LOAD) {
    const SideSpec s = {in.ptr[a], (int)((meta >> (6 * a)) & 7), (int)((meta >> (6 * a + 3)) & 7), in.mid[a], in.inner[a], in.row_base, in.row_len};
    float v[1];
    load_side<1>(s, row, v);
    sregs[dst & 7] = v[0];
    return false;
  }
  if (op == DAG_STORE) {
    if (writer) {
      const Store2 st = {out.ptr[dst], (int)((meta >> (48 + 3 * dst)) & 7), row, 0};
      const float v[1] = {sregs[a & 7]};
      store_second<1>(st, v);
    }
    return false;
  }
  const bool two = a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE;
  auto pick = [&](int sel) { return sel < DAG_REGS ? sregs[sel] : (sel == DAG_IMM ? imm : imm2); };
  float x[1] = {pick(a)};
  if (op >= EW_FIRST_UNARY) {
    apply_unary<1>(op, imm, x);
  } else if (op == EW_FMA) {
    x[0] = fmaf(x[0], pick(b), pick(c));
  } else if (op == EW_SELECT) {
    x[0] = x[0] != 0.0f ? pick(b) : pick(c);
  } else if (op == EW_SCALE_PRE) {
    x[0] = imm * (x[0] + imm2);
  } else {
    const float y[1] = {pick(b)};
    apply_binary<1>(op, false, y, x);
  }
  sregs[dst & 7] = x[0];
  return two;
}

__device__ __forceinline__ float rp_imm(long long w) { return __uint_as_float((uint32_t)(w >> 32)); }

// ---- the two ways a program is known ---------------------------------------------------------------------------------
struct DynRowProgram {
  static constexpr bool kStatic = false;
  const long long* steps;
  unsigned long long counts, meta;
  __device__ __forceinline__ void run_element_cached(int, const RowInputs&, const RowOutputs&, long long,
                                                     const float (&)[ROWP_SREGS], float (&)[ROWP_SREGS], float (*)[4]) const {}
  __device__ __forceinline__ void preload(const RowInputs&, long long, float (*)[4]) const {}
  __device__ __forceinline__ void prefetch(const RowInputs&, long long) const {}
  __device__ __forceinline__ int passes() const {
    int p = 0;
    for (int k = 0; k < ROWP_MAX_PASSES; ++k)
      if (((counts >> (8 * k)) & 0xff) || ((counts >> (32 + 8 * k)) & 0xff)) p = k + 1;
    return p;
  }
  __device__ __forceinline__ int first_step(int pass, bool scalar) const {
    int at = 0;
    for (int k = 0; k < pass; ++k) at += (int)((counts >> (8 * k)) & 0xff) + (int)((counts >> (32 + 8 * k)) & 0xff);
    return at + (scalar ? (int)((counts >> (8 * pass)) & 0xff) : 0);
  }
  // which scalar registers the pass accumulates into (bit k) and the fold kind of each (2 bits per register)
  __device__ __forceinline__ void acc_plan(int pass, unsigned& mask, unsigned& kinds) const {
    mask = kinds = 0;
    const int b = first_step(pass, false), e = b + (int)((counts >> (8 * pass)) & 0xff);
    for (int k = b; k < e; ++k) {
      const unsigned w = (unsigned)steps[k];
      if ((w & 0xff) == (unsigned)ROWP_ACC) {
        const unsigned d = (w >> 8) & 7;
        mask |= 1u << d;
        kinds |= ((w >> 22) & 3u) << (2 * d);
      }
    }
  }
  template <int VEC>
  __device__ __forceinline__ void run_element(int pass, const RowInputs& in, const RowOutputs& out, long long i0,
                                              const float (&sregs)[ROWP_SREGS], float (&acc)[ROWP_SREGS]) const {
    float regs[DAG_REGS][VEC];
    const int b = first_step(pass, false), e = b + (int)((counts >> (8 * pass)) & 0xff);
    for (int k = b; k < e; ++k)
      if (rp_element_step<VEC>((unsigned)steps[k], rp_imm(steps[k]), rp_imm(steps[k + 1]), meta, in, out, i0, regs, sregs, acc, pass + 1 < passes())) ++k;
  }
  __device__ __forceinline__ void run_scalar(int pass, const RowInputs& in, const RowOutputs& out, long long row,
                                             bool writer, float (&sregs)[ROWP_SREGS]) const {
    const int b = first_step(pass, true), e = b + (int)((counts >> (32 + 8 * pass)) & 0xff);
    for (int k = b; k < e; ++k)
      if (rp_scalar_step((unsigned)steps[k], rp_imm(steps[k]), rp_imm(steps[k + 1]), meta, in, out, row, writer, sregs)) ++k;
  }
};

template <unsigned long long META, unsigned long long COUNTS, uint32_t... SIG>
struct StaticRowProgram {
  const long long* steps;
  static constexpr int kN = (int)sizeof...(SIG);
  __host__ __device__ static constexpr int count(int pass, bool scalar) { return (int)((COUNTS >> ((scalar ? 32 : 0) + 8 * pass)) & 0xff); }
  __host__ __device__ static constexpr int first(int pass, bool scalar) {
    int at = 0;
    for (int k = 0; k < pass; ++k) at += count(k, false) + count(k, true);
    return at + (scalar ? count(pass, false) : 0);
  }
  __host__ __device__ constexpr int passes() const {
    int p = 0;
    for (int k = 0; k < ROWP_MAX_PASSES; ++k)
      if (count(k, false) || count(k, true)) p = k + 1;
    return p;
  }
  __host__ __device__ static constexpr uint32_t word(int k) {
    constexpr uint32_t sig[kN > 0 ? kN : 1] = {SIG...};
    return sig[k];
  }
  __device__ __forceinline__ void acc_plan(int pass, unsigned& mask, unsigned& kinds) const {
    mask = kinds = 0;
#pragma unroll
    for (int k = 0; k < kN; ++k) {
      bool in_pass = false;
#pragma unroll
      for (int p = 0; p < ROWP_MAX_PASSES; ++p)
        in_pass = in_pass || (p == pass && k >= first(p, false) && k < first(p, false) + count(p, false));
      const unsigned w = word(k);
      if (in_pass && (w & 0xff) == (unsigned)ROWP_ACC) {
        mask |= 1u << ((w >> 8) & 7);
        kinds |= ((w >> 22) & 3u) << (2 * ((w >> 8) & 7));
      }
    }
  }
  template <int VEC, int K, int END, bool REREAD>
  __device__ __forceinline__ void element_from(const RowInputs& in, const RowOutputs& out, long long i0,
                                               float (&regs)[DAG_REGS][VEC], const float (&sregs)[ROWP_SREGS],
                                               float (&acc)[ROWP_SREGS]) const {
    if constexpr (K < END) {
      constexpr uint32_t w = word(K);
      constexpr int op = (int)(w & 0xff), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31), c = (int)((w >> 22) & 31);
      constexpr bool two = op != EW_NOP && op != DAG_LOAD && op != DAG_STORE && op != ROWP_ACC &&
                           (a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE);
      (void)rp_element_step<VEC, true>(w, rp_imm(steps[K]), rp_imm(steps[K + 1 < ROWP_MAX_STEPS ? K + 1 : K]), META, in, out, i0,
                                 regs, sregs, acc, REREAD);
      element_from<VEC, K + (two ? 2 : 1), END, REREAD>(in, out, i0, regs, sregs, acc);
    }
  }
  template <int K, int END>
  __device__ __forceinline__ void scalar_from(const RowInputs& in, const RowOutputs& out, long long row, bool writer,
                                              float (&sregs)[ROWP_SREGS]) const {
    if constexpr (K < END) {
      constexpr uint32_t w = word(K);
      constexpr int op = (int)(w & 0xff), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31), c = (int)((w >> 22) & 31);
      constexpr bool two = op != EW_NOP && op != DAG_LOAD && op != DAG_STORE &&
                           (a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE);
      (void)rp_scalar_step(w, rp_imm(steps[K]), rp_imm(steps[K + 1 < ROWP_MAX_STEPS ? K + 1 : K]), META, in, out, row, writer, sregs);
      scalar_from<K + (two ? 2 : 1), END>(in, out, row, writer, sregs);
    }
  }
  static constexpr bool kStatic = true;
  // bit k: pass 0 loads input k (so a later pass may take it from the register cache)
  __host__ __device__ static constexpr unsigned loaded_by_pass0() {
    unsigned m = 0;
    for (int k = first(0, false); k < first(0, false) + count(0, false); ++k)
      if ((word(k) & 0xff) == (unsigned)DAG_LOAD) m |= 1u << ((word(k) >> 12) & 7);
    return m;
  }
  // CTAs per SM the kernel is compiled for: a program of three passes over two or more cached inputs keeps twice the
  // row state in registers and spills at three CTAs' register budget (80), so it is built for two (128).
  __host__ __device__ static constexpr int ctas_per_sm() {
    int full = 0;
    for (int a = 0; a < DAG_MAX_IN; ++a)
      if (((loaded_by_pass0() >> a) & 1u) && ((META >> (6 * a + 3)) & 7) == (unsigned)EW_SIDE_FULL) ++full;
    return (full >= 2 && StaticRowProgram().passes() >= 3) ? 2 : 3;
  }
  __host__ __device__ static constexpr int step_words(int k) {
    const uint32_t w = word(k);
    const int op = (int)(w & 0xff), a = (int)((w >> 12) & 31), b = (int)((w >> 17) & 31), c = (int)((w >> 22) & 31);
    const bool two = op != EW_NOP && op != DAG_LOAD && op != DAG_STORE && op != ROWP_ACC &&
                     (a == DAG_IMM2 || b == DAG_IMM2 || c == DAG_IMM2 || op == EW_SCALE_PRE);
    return two ? 2 : 1;
  }
  // The loads of pass 0's full-size inputs for one vector, into its cache slot; nothing uses the values here, so the
  // loads of all of a thread's vectors are in flight together.
  template <int K, int END>
  __device__ __forceinline__ void preload_from(const RowInputs& in, long long i0, float (*cache)[4]) const {
    if constexpr (K < END) {
      constexpr uint32_t w = word(K);
      if constexpr ((w & 0xff) == (unsigned)DAG_LOAD) {
        constexpr int a = (int)((w >> 12) & 7);
        if constexpr (((META >> (6 * a + 3)) & 7) == (unsigned)EW_SIDE_FULL)
          load_vec4(in.ptr[a], (int)((META >> (6 * a)) & 7), i0, true, *reinterpret_cast<float(*)[4]>(&cache[a][0]));
      }
      preload_from<K + step_words(K), END>(in, i0, cache);
    }
  }
  template <int K, int END>
  __device__ __forceinline__ void prefetch_from(const RowInputs& in, long long i0) const {
    if constexpr (K < END) {
      constexpr uint32_t w = word(K);
      if constexpr ((w & 0xff) == (unsigned)DAG_LOAD) {
        constexpr int a = (int)((w >> 12) & 7);
        if constexpr (((META >> (6 * a + 3)) & 7) == (unsigned)EW_SIDE_FULL) {
          constexpr int dt = (int)((META >> (6 * a)) & 7);
          const char* p = static_cast<const char*>(in.ptr[a]) + i0 * (dt == EW_F32 ? 4 : (dt == EW_BOOL ? 1 : 2));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
        }
      }
      prefetch_from<K + step_words(K), END>(in, i0);
    }
  }
  // Asks the lines of pass 0's full-size inputs at flat index i0 into L2.
  __device__ __forceinline__ void prefetch(const RowInputs& in, long long i0) const {
    prefetch_from<first(0, false), first(0, false) + count(0, false)>(in, i0);
  }
  __device__ __forceinline__ void preload(const RowInputs& in, long long i0, float (*cache)[4]) const {
    preload_from<first(0, false), first(0, false) + count(0, false)>(in, i0, cache);
  }
  template <int K, int END>
  __device__ __forceinline__ void cached_from(const RowInputs& in, const RowOutputs& out, long long i0,
                                              float (&regs)[DAG_REGS][4], const float (&sregs)[ROWP_SREGS],
                                              float (&acc)[ROWP_SREGS], float (*cache)[4]) const {
    if constexpr (K < END) {
      constexpr uint32_t w = word(K);
      // only what pass 0 loaded is in the cache
      constexpr int mode = ((w & 0xff) == (unsigned)DAG_LOAD && ((loaded_by_pass0() >> ((w >> 12) & 7)) & 1u)) ? 2 : 0;
      (void)rp_element_step<4, true>(w, rp_imm(steps[K]), rp_imm(steps[K + 1 < ROWP_MAX_STEPS ? K + 1 : K]), META, in, out, i0,
                               regs, sregs, acc, false, cache, mode);
      cached_from<K + step_words(K), END>(in, out, i0, regs, sregs, acc, cache);
    }
  }
  // where the passes share their first steps (row_prog_prefix.h)
  __host__ __device__ static constexpr RowPrefixPlan prefix_plan() {
    constexpr uint32_t sig[kN > 0 ? kN : 1] = {SIG...};
    return PlanRowPrefixes(sig, COUNTS, META);
  }
  // One pass over one cached vector.  `cache` is the slot of this vector: [input][lane of the vector] for the inputs
  // pass 0 loaded.  The value at the end of the steps this pass shares with the later ones takes the place of an
  // input that nothing loads afterwards (written here after `save` words, read by the later passes, which begin
  // after those steps): no registers are added to the row's state.
  template <int PASS>
  __device__ __forceinline__ void cached_pass(const RowInputs& in, const RowOutputs& out, long long i0,
                                              const float (&sregs)[ROWP_SREGS], float (&acc)[ROWP_SREGS],
                                              float (*cache)[4]) const {
    constexpr RowPrefixPlan plan = prefix_plan();
    constexpr int b = first(PASS, false), e = b + count(PASS, false);
    constexpr int start = plan.start[PASS], save = plan.save[PASS];
    float regs[DAG_REGS][4];
    if constexpr (start > 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) regs[plan.reg[PASS]][i] = cache[plan.slot][i];
    }
    if constexpr (save > start) {
      cached_from<b + start, b + save>(in, out, i0, regs, sregs, acc, cache);
#pragma unroll
      for (int i = 0; i < 4; ++i) cache[plan.slot][i] = regs[plan.save_reg[PASS]][i];
      cached_from<b + save, e>(in, out, i0, regs, sregs, acc, cache);
    } else {
      cached_from<b + start, e>(in, out, i0, regs, sregs, acc, cache);
    }
  }
  // One vector of a row whose vectors stay in this thread's registers between the passes.
  __device__ __forceinline__ void run_element_cached(int pass, const RowInputs& in, const RowOutputs& out, long long i0,
                                                     const float (&sregs)[ROWP_SREGS], float (&acc)[ROWP_SREGS],
                                                     float (*cache)[4]) const {
    if (pass == 0) cached_pass<0>(in, out, i0, sregs, acc, cache);
    else if (pass == 1) cached_pass<1>(in, out, i0, sregs, acc, cache);
    else cached_pass<2>(in, out, i0, sregs, acc, cache);
  }
  template <int VEC>
  __device__ __forceinline__ void run_element(int pass, const RowInputs& in, const RowOutputs& out, long long i0,
                                              const float (&sregs)[ROWP_SREGS], float (&acc)[ROWP_SREGS]) const {
    float regs[DAG_REGS][VEC];
    constexpr int np = StaticRowProgram().passes();
    if (pass == 0) element_from<VEC, first(0, false), first(0, false) + count(0, false), (np > 1)>(in, out, i0, regs, sregs, acc);
    else if (pass == 1) element_from<VEC, first(1, false), first(1, false) + count(1, false), (np > 2)>(in, out, i0, regs, sregs, acc);
    else element_from<VEC, first(2, false), first(2, false) + count(2, false), false>(in, out, i0, regs, sregs, acc);
  }
  __device__ __forceinline__ void run_scalar(int pass, const RowInputs& in, const RowOutputs& out, long long row,
                                             bool writer, float (&sregs)[ROWP_SREGS]) const {
    if (pass == 0) scalar_from<first(0, true), first(0, true) + count(0, true)>(in, out, row, writer, sregs);
    else if (pass == 1) scalar_from<first(1, true), first(1, true) + count(1, true)>(in, out, row, writer, sregs);
    else scalar_from<first(2, true), first(2, true) + count(2, true)>(in, out, row, writer, sregs);
  }
};

// ---- the kernel body --------------------------------------------------------------------------------------------------
// FORM 0: warp or CTA per row by `group` at run time (the interpreting kernel); 1: a warp per row; 2: a CTA per row;
// 3: half a CTA (four warps) per row, two rows per CTA at a time, each half with a named barrier of its own; 4: a CTA
// per row with eight cached vectors per thread (rows of up to 8192 elements)
// (the specialised kernels: one instantiation each, so that the register cache below is sized for its form).
// NV > 0: every thread of the row's group holds exactly NV vectors of the row (r / 4 = NV x threads per row): no
// bounds tests, so the loads of all its vectors are issued together and their arithmetic interleaves (measured on
// B200, log_softmax over rows of 3072 elements: 0.97 of the HBM peak against 0.84 with a test per vector; standing
// in copies of the last vector for the missing ones of a shorter row, masked at the folds and stores, gave 0.83).
// NV = 0: any row, a test per vector.
template <class Prog, int FORM, int NV = 0>
__device__ __forceinline__ void row_program_body(const Prog& prog, const RowInputs& inputs, const RowOutputs& out,
                                                 long long rows, long long r, long long group, long long vec_ok) {
  RowInputs in = inputs;
  in.row_len   = r;
  __shared__ float part[8][ROWP_SREGS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = FORM == 3 ? (int)(threadIdx.x >> 7) : 0;  // FORM 3: which of the CTA's two rows
  // (FORM 2 keeps the run-time test although its rows always get a CTA: with the test folded away the compiler packs
  // the CTA form into fewer registers and no longer issues a row's loads together -- measured on B200, rms_norm over
  // 16384 x 4096 fell from 0.90 to 0.45 of the HBM peak.)
  const bool per_warp   = FORM == 1 ? true : group == 32;
  const long long first = FORM == 3 ? (long long)blockIdx.x * 2 + half : (per_warp ? (long long)blockIdx.x * 8 + warp : blockIdx.x);
  const long long step  = FORM == 3 ? (long long)gridDim.x * 2 : (per_warp ? (long long)gridDim.x * 8 : gridDim.x);
  const int t  = FORM == 3 ? (int)(threadIdx.x & 127) : (per_warp ? lane : (int)threadIdx.x);
  const int nt = FORM == 3 ? 128 : (per_warp ? 32 : 256);
  const int npass = prog.passes();
  // A specialised program of several passes keeps the row in registers between the passes instead of reading it
  // again: a CTA holds a row of up to 4096 elements in four vectors per thread, a warp one of up to 1024 in eight
  // vectors per lane.
  constexpr int kCacheVecs = FORM == 1 || FORM == 3 || FORM == 4 ? 8 : 4;
  constexpr int kStride    = FORM == 1 ? 32 : (FORM == 3 ? 128 : 256);
  const bool use_cache = Prog::kStatic && FORM != 0 && (FORM == 1 || FORM == 3 || !per_warp) && vec_ok && npass > 1 &&
                         (r >> 2) <= (long long)kCacheVecs * kStride;
  float cache[kCacheVecs][DAG_MAX_IN][4];
  const int nvec_row = use_cache ? (int)(r >> 2) : 0;
  // CTA-per-row: every thread of the CTA walks the same rows, so the barriers below are uniform.
  for (long long row = first; row < rows; row += step) {
    const long long base = row * r;
    in.row_base          = base;
    if (use_cache) {
      // this row's loads, all in flight together; the next row is asked into L2 meanwhile (no registers held for it),
      // so that the next wait is an L2 latency, not a DRAM one
#pragma unroll
      for (int j = 0; j < (NV > 0 ? NV : kCacheVecs); ++j) {
        const int v = t + j * kStride;  // (cached rows have at most 8192 elements)
        if (NV > 0 || v < nvec_row) prog.preload(in, base + (v << 2), cache[j]);
      }
      if (row + step < rows) {
#pragma unroll
        for (int j = 0; j < (NV > 0 ? NV : kCacheVecs); ++j) {
          const int v = t + j * kStride;
          if (NV > 0 || v < nvec_row) prog.prefetch(in, base + step * r + (v << 2));
        }
      }
    }
    float sregs[ROWP_SREGS];
#pragma unroll
    for (int k = 0; k < ROWP_SREGS; ++k) sregs[k] = 0.0f;
    for (int pass = 0; pass < npass; ++pass) {
      unsigned mask, kinds;
      prog.acc_plan(pass, mask, kinds);
      float acc[ROWP_SREGS];
#pragma unroll
      for (int k = 0; k < ROWP_SREGS; ++k) acc[k] = rp_identity((kinds >> (2 * k)) & 3);
      long long done = 0;
      if (use_cache) {
        // every thread's vectors of the row were loaded once, all the loads in flight together
#pragma unroll
        for (int j = 0; j < (NV > 0 ? NV : kCacheVecs); ++j) {
          const int v = t + j * kStride;
          if (NV > 0 || v < nvec_row) prog.run_element_cached(pass, in, out, base + (v << 2), sregs, acc, cache[j]);
        }
        done = r;
      } else if (vec_ok) {  // r % 4 == 0 and aligned buffers: every row starts on a vector boundary
        const long long nv = r >> 2;
        // four vectors per thread in flight (a 4096-element row is exactly that for a CTA): the loads of an unrolled
        // group are independent and are issued together
#pragma unroll 4
        for (long long v = t; v < nv; v += nt) prog.template run_element<4>(pass, in, out, base + (v << 2), sregs, acc);
        done = nv << 2;
      }
      for (long long j = done + t; j < r; j += nt) prog.template run_element<1>(pass, in, out, base + j, sregs, acc);
      // combine the accumulators over the row's threads: lanes in a tree, then (CTA per row) the warps in order
#pragma unroll
      for (int k = 0; k < ROWP_SREGS; ++k) {
        if (!(mask & (1u << k))) continue;
        const int kind = (kinds >> (2 * k)) & 3;
        float v = acc[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = rp_fold(kind, v, __shfl_xor_sync(0xffffffffu, v, o));
        acc[k] = v;
      }
      if (FORM == 3 && mask) {
        // the four warps of this half meet at a barrier of their own (ids 1 and 2): the CTA's two rows never wait
        // for each other
        asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < ROWP_SREGS; ++k)
            if (mask & (1u << k)) part[warp][k] = acc[k];
        }
        asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
#pragma unroll
        for (int k = 0; k < ROWP_SREGS; ++k) {
          if (!(mask & (1u << k))) continue;
          const int kind = (kinds >> (2 * k)) & 3;
          float v = part[4 * half][k];
#pragma unroll
          for (int w2 = 1; w2 < 4; ++w2) v = rp_fold(kind, v, part[4 * half + w2][k]);
          acc[k] = v;
        }
      } else if (!per_warp && mask) {
        __syncthreads();  // the previous pass's reads of `part` are over
        if (lane == 0) {
#pragma unroll
          for (int k = 0; k < ROWP_SREGS; ++k)
            if (mask & (1u << k)) part[warp][k] = acc[k];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < ROWP_SREGS; ++k) {
          if (!(mask & (1u << k))) continue;
          const int kind = (kinds >> (2 * k)) & 3;
          float v = part[0][k];
#pragma unroll
          for (int w2 = 1; w2 < 8; ++w2) v = rp_fold(kind, v, part[w2][k]);
          acc[k] = v;
        }
      }
#pragma unroll
      for (int k = 0; k < ROWP_SREGS; ++k)
        if (mask & (1u << k)) sregs[k] = acc[k];
      prog.run_scalar(pass, in, out, row, t == 0, sregs);
    }
  }
}

#define ROWP_PARAMS                                                                                                   \
  const void *__restrict__ i0, const void *__restrict__ i1, const void *__restrict__ i2, const void *__restrict__ i3, \
      const void *__restrict__ i4, const void *__restrict__ i5, const void *__restrict__ i6,                         \
      const void *__restrict__ i7, void *__restrict__ o0, void *__restrict__ o1, void *__restrict__ o2,              \
      void *__restrict__ o3, long long rows, long long r, long long group, long long vec_ok, long long meta,         \
      long long counts, long long m0, long long n0, long long m1, long long n1, long long m2, long long n2,         \
      long long m3, long long n3, long long m4, long long n4, long long m5, long long n5, long long m6, long long n6, \
      long long m7, long long n7, long long t0, long long t1, long long t2, long long t3, long long t4, long long t5, \
      long long t6, long long t7, long long t8, long long t9, long long t10, long long t11, long long t12,           \
      long long t13, long long t14, long long t15, long long t16, long long t17, long long t18, long long t19,       \
      long long t20, long long t21, long long t22, long long t23, long long t24, long long t25, long long t26,       \
      long long t27, long long t28, long long t29, long long t30, long long t31, long long t32, long long t33,       \
      long long t34, long long t35
#define ROWP_UNPACK                                                                                                   \
  const RowInputs in = {{i0, i1, i2, i3, i4, i5, i6, i7}, {m0, m1, m2, m3, m4, m5, m6, m7},                          \
                        {n0, n1, n2, n3, n4, n5, n6, n7}};                                                            \
  const RowOutputs out = {{o0, o1, o2, o3}};                                                                          \
  const long long steps[ROWP_MAX_STEPS + 1] = {t0,  t1,  t2,  t3,  t4,  t5,  t6,  t7,  t8,  t9,  t10, t11, t12,       \
                                               t13, t14, t15, t16, t17, t18, t19, t20, t21, t22, t23, t24, t25,       \
                                               t26, t27, t28, t29, t30, t31, t32, t33, t34, t35, 0}

__global__ void __launch_bounds__(256) k_row_program(ROWP_PARAMS) {
  grid_dependency_sync();
  ROWP_UNPACK;
  const DynRowProgram prog = {steps, (unsigned long long)counts, (unsigned long long)meta};
  row_program_body<DynRowProgram, 0>(prog, in, out, rows, r, group, vec_ok);
}

// One kernel per program, form and NV (see row_program_body).  A kernel with NV > 0 runs rows of exactly NV vectors
// per thread of the row's group in the body without bounds tests and anything else (another length -- the matcher
// does not ask for that --, buffers not aligned for vector access, which is known at launch only) in the general
// body.  Holding both bodies is deliberate: compiled alone, the straight-line body is packed into fewer registers
// (68 against 76-78 for softmax(x * s)) with its loads and arithmetic less interleaved -- measured on B200 over
// 16384 x 4096, 0.92 of the HBM peak against 0.98, fp16 rms_norm 0.68 against 0.80.
// (A CTA per row of up to 8192 elements is compiled for two CTAs per SM -- eight cached vectors per thread and the
// program's own registers do not fit 80 --, its kernels for exactly 5 or 6 vectors per thread for three: standardise
// over 16384 x 5120, 0.86 -> 0.93 of the HBM peak.)
template <int FORM, int NV, unsigned long long META, unsigned long long COUNTS, uint32_t... SIG>
__global__ void __launch_bounds__(256, (FORM == 4 && (NV == 0 || NV > 6) ? 2 : StaticRowProgram<META, COUNTS, SIG...>::ctas_per_sm()))
k_row_program_static(ROWP_PARAMS) {
  grid_dependency_sync();
  ROWP_UNPACK;
  using Prog      = StaticRowProgram<META, COUNTS, SIG...>;
  const Prog prog = {steps};
  constexpr int kPer = 4 * (FORM == 1 ? 32 : (FORM == 3 ? 128 : 256));  // elements per vector index of a thread
  if (NV > 0 && Prog().passes() > 1 && vec_ok && r == (long long)NV * kPer)
    row_program_body<Prog, FORM, NV>(prog, in, out, rows, r, group, vec_ok);
  else
    row_program_body<Prog, FORM, 0>(prog, in, out, rows, r, group, vec_ok);
}

template <uint32_t... SIG>
StaticChainKey MakeRowKey(const char* base, long long meta, long long counts) {
  // the counts word is part of the program: it goes in front of the step words
  StaticChainKey k = {base, meta, (int)sizeof...(SIG) + 2, {(uint32_t)(counts & 0xffffffff), (uint32_t)((unsigned long long)counts >> 32), SIG...}};
  return k;
}

}  // namespace
}  // namespace cinn_b200

// One specialised kernel: its name is "row_program_static_<id><suffix>", its registry key `KEY`.
#define ROWP_ONE(ID, SUFFIX, KEY, FORM, NV, META, COUNTS, ...)                                                        \
  CINN_B200_REGISTER_KERNEL_PDL("row_program_static_" #ID SUFFIX, 70, 256, k_row_program_static<FORM, NV, META##ull, COUNTS##ull, __VA_ARGS__>); \
  static int CINN_B200_CAT(cinn_b200_static_row_program_, __COUNTER__) =                                                \
      RegisterStaticChain(MakeRowKey<__VA_ARGS__>(KEY, META##ll, COUNTS##ll), "row_program_static_" #ID SUFFIX)
