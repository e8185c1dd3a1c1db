// Reductions whose operand is an elementwise chain: reduce_{sum,prod,max,min}(f(x, sides...)), one HBM pass.
//
// The reference lowers such a group as one kernel too: the producers of a reduce are computed inline or as a
// materialised stage of the same kernel (cinn/hlir/framework/op_lowering.cc:516-608, CanbeInline in
// op_lowering_util.cc:745-803) and the reduction follows (cinn/hlir/pe/reduction.cc:139-227).  Here the chain program
// of ew_chain.h is run on every loaded vector in fp32 registers and its values are folded straight into the
// accumulators: nothing but the inputs is read and nothing but the reduced result is written.  Initial values are
// those of cinn/lang/builtin.cc:123-143 (0, 1, the lowest / largest finite float); max / min are compare + select.
// The result is stored as float32, float16 or bfloat16 (a cast after the reduce, as the AutoCast pass leaves it).
//
// Two layouts, as in the other reduction kernels: rows (inner == 1: a warp or a CTA per row) and columns
// (inner > 1: a thread per four columns).  Long rows / tall columns on small grids are cut into segments whose
// float32 partials a second launch folds (reduce_generic_{row,col}_*_f32).
#include "ew_chain_body.cuh"
#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

enum { CR_SUM = 0, CR_PROD = 1, CR_MAX = 2, CR_MIN = 3 };

__device__ __forceinline__ float cr_identity(int op) {
  return op == CR_SUM ? 0.0f : (op == CR_PROD ? 1.0f : (op == CR_MAX ? -3.402823466e38f : 3.402823466e38f));
}

__device__ __forceinline__ float cr_apply(int op, float a, float b) {
  switch (op) {
    case CR_SUM: return a + b;
    case CR_PROD: return a * b;
    case CR_MAX: return a > b ? a : b;
    default: return a < b ? a : b;
  }
}

__device__ __forceinline__ void cr_store(void* out, int out_type, long long idx, float v) {
  if (out_type == EW_F16) reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  else if (out_type == EW_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[idx] = v;
}

#define CHAIN_PARAMS                                                                                                  \
  const void *__restrict__ in0, const void *__restrict__ p1, const void *__restrict__ p2, const void *__restrict__ p3, \
      void *__restrict__ out, long long n, long long vec_ok, long long meta, long long mid1, long long inner1,        \
      long long mid2, long long inner2, long long mid3, long long inner3, long long nsteps_ll, long long t0,         \
      long long t1, long long t2, long long t3, long long t4, long long t5, long long t6, long long t7, long long t8, \
      long long t9, long long t10, long long t11, long long t12, long long t13, long long t14, long long t15

// meta: as in the chain kernel (bits 0-27), plus bits 28-29 the reduce op and bits 32-35 the storage type of the result.
#define CHAIN_STEPS \
  const long long steps[EW_MAX_STEPS + 1] = {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, 0}

struct Sides {
  SideSpec sd1, sd2, sd3;
};
template <class Prog>
__device__ __forceinline__ Sides make_sides(const Prog& prog, const void* p1, const void* p2, const void* p3,
                                            long long mid1, long long inner1, long long mid2, long long inner2,
                                            long long mid3, long long inner3) {
  return Sides{{p1, prog.side_dtype(1), prog.side_mode(1), mid1, inner1},
               {p2, prog.side_dtype(2), prog.side_mode(2), mid2, inner2},
               {p3, prog.side_dtype(3), prog.side_mode(3), mid3, inner3}};
}

// The chain's values of VEC consecutive elements starting at flat input index i0.
template <int VEC, int NS, int NT, class Prog>
__device__ __forceinline__ void chain_values(const Prog& prog, const void* in0, const Sides& sd, long long i0,
                                             float (&acc)[VEC]) {
  const int in_type = prog.in_type();
  float s1[VEC], s2[VEC], s3[VEC];
  if constexpr (VEC == 4) {
    if (in_type != EW_NO_INPUT) load_vec4(in0, in_type, i0, true, *reinterpret_cast<float(*)[4]>(&acc[0]));
  } else {
    acc[0] = in_type != EW_NO_INPUT ? load_scalar(in0, in_type, i0) : 0.0f;
  }
  if (NS >= 1 && sd.sd1.mode != EW_SIDE_NONE) load_side<VEC>(sd.sd1, i0, s1);
  if (NS >= 2 && sd.sd2.mode != EW_SIDE_NONE) load_side<VEC>(sd.sd2, i0, s2);
  if (NS >= 3 && sd.sd3.mode != EW_SIDE_NONE) load_side<VEC>(sd.sd3, i0, s3);
  prog.template run<VEC, NS, NT, false>(s1, s2, s3, acc, nullptr);
}

// Two vectors whose loads are all issued before the program runs once over the eight values (kernels without
// temporaries only).
template <int NS, class Prog>
__device__ __forceinline__ void chain_values2(const Prog& prog, const void* in0, const Sides& sd, long long ia,
                                              long long ib, float (&acc)[8]) {
  const int in_type = prog.in_type();
  float s1[8], s2[8], s3[8];
  if (in_type != EW_NO_INPUT) {
    load_vec4(in0, in_type, ia, true, *reinterpret_cast<float(*)[4]>(&acc[0]));
    load_vec4(in0, in_type, ib, true, *reinterpret_cast<float(*)[4]>(&acc[4]));
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const long long i0 = j ? ib : ia;
    if (NS >= 1 && sd.sd1.mode != EW_SIDE_NONE) load_side<4>(sd.sd1, i0, *reinterpret_cast<float(*)[4]>(&s1[4 * j]));
    if (NS >= 2 && sd.sd2.mode != EW_SIDE_NONE) load_side<4>(sd.sd2, i0, *reinterpret_cast<float(*)[4]>(&s2[4 * j]));
    if (NS >= 3 && sd.sd3.mode != EW_SIDE_NONE) load_side<4>(sd.sd3, i0, *reinterpret_cast<float(*)[4]>(&s3[4 * j]));
  }
  prog.template run<8, NS, 0, false>(s1, s2, s3, acc, nullptr);
}

// Four vectors: the specialised kernels' inner step for rows (sixteen values per thread and iteration: 64 bytes of
// every full-size operand in flight per thread).
template <int NS, class Prog>
__device__ __forceinline__ void chain_values4(const Prog& prog, const void* in0, const Sides& sd, const long long (&idx)[4],
                                              float (&acc)[16]) {
  const int in_type = prog.in_type();
  float s1[16], s2[16], s3[16];
  if (in_type != EW_NO_INPUT) {
#pragma unroll
    for (int j = 0; j < 4; ++j) load_vec4(in0, in_type, idx[j], true, *reinterpret_cast<float(*)[4]>(&acc[4 * j]));
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (NS >= 1 && sd.sd1.mode != EW_SIDE_NONE) load_side<4>(sd.sd1, idx[j], *reinterpret_cast<float(*)[4]>(&s1[4 * j]));
    if (NS >= 2 && sd.sd2.mode != EW_SIDE_NONE) load_side<4>(sd.sd2, idx[j], *reinterpret_cast<float(*)[4]>(&s2[4 * j]));
    if (NS >= 3 && sd.sd3.mode != EW_SIDE_NONE) load_side<4>(sd.sd3, idx[j], *reinterpret_cast<float(*)[4]>(&s3[4 * j]));
  }
  prog.template run<16, NS, 0, false>(s1, s2, s3, acc, nullptr);
}

// ---- rows: y[row] = fold over j of f(x[row * r + j]) -----------------------------------------------------------------
// `group` = 32: a warp per row (8 rows per CTA); `group` = 256: a CTA per row.  `rows` counts segments when a row is
// cut (the matcher passes rows * S and r / S): a segment is just a shorter row of the same flat index space.
// Occupancy of the interpreting form, measured on B200 with sum(|x - y|) over 8192 x 8192 (one side operand): 4 CTAs
// per SM (64 registers, a few spilled words) 0.70 of the HBM peak; 3 CTAs (80 registers, no spills) 0.61; 5 CTAs (48
// registers) 0.57.
template <int NS, int NT, class Prog>
__device__ __forceinline__ void chain_reduce_row_body(const Prog& prog, const void* in0, const Sides& sides, void* out,
                                                      long long vec_ok, long long rows, long long r, long long group) {
  Sides sd = sides;
  sd.sd1.row_len = sd.sd2.row_len = sd.sd3.row_len = r;
  const int rop = prog.reduce_op(), out_type = prog.result_type();
  __shared__ float part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool per_warp   = group == 32;
  const long long first = per_warp ? (long long)blockIdx.x * 8 + warp : blockIdx.x;
  const long long step  = per_warp ? (long long)gridDim.x * 8 : gridDim.x;
  const int t = per_warp ? lane : (int)threadIdx.x, nt = per_warp ? 32 : 256;
  const float id = cr_identity(rop);
  for (long long row = first; row < rows; row += step) {  // uniform per CTA in the CTA-per-row form
    const long long base = row * r;
    sd.sd1.row_base = sd.sd2.row_base = sd.sd3.row_base = base;
    float a[4] = {id, id, id, id};
    long long done = 0;
    if (vec_ok) {  // r % 4 == 0 and aligned buffers: every row starts on a vector boundary
      const long long nv = r >> 2;
      long long v        = t;
      if constexpr (Prog::kStatic && NT == 0 && NS <= 1) {
        for (; v + 3 * nt < nv; v += 4 * nt) {
          float acc[16];
          const long long idx[4] = {base + (v << 2), base + ((v + nt) << 2), base + ((v + 2 * nt) << 2), base + ((v + 3 * nt) << 2)};
          chain_values4<NS>(prog, in0, sd, idx, acc);
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i & 3] = cr_apply(rop, a[i & 3], acc[i]);
        }
      }
      for (; NT == 0 && v + nt < nv; v += 2 * nt) {
        float acc[8];
        chain_values2<NS>(prog, in0, sd, base + (v << 2), base + ((v + nt) << 2), acc);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i & 3] = cr_apply(rop, a[i & 3], acc[i]);
      }
      for (; v < nv; v += nt) {
        float acc[4];
        chain_values<4, NS, NT>(prog, in0, sd, base + (v << 2), acc);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = cr_apply(rop, a[i], acc[i]);
      }
      done = nv << 2;
    }
    for (long long j = done + t; j < r; j += nt) {
      float acc[1];
      chain_values<1, NS, NT>(prog, in0, sd, base + j, acc);
      a[0] = cr_apply(rop, a[0], acc[0]);
    }
    float v = cr_apply(rop, cr_apply(rop, a[0], a[1]), cr_apply(rop, a[2], a[3]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = cr_apply(rop, v, __shfl_xor_sync(0xffffffffu, v, o));
    if (per_warp) {
      if (lane == 0) cr_store(out, out_type, row, v);
    } else {
      if (lane == 0) part[warp] = v;
      __syncthreads();
      if (threadIdx.x == 0) {
        float total = part[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) total = cr_apply(rop, total, part[w]);
        cr_store(out, out_type, row, total);
      }
      __syncthreads();
    }
  }
}

// ---- columns: y[o, c] = fold over k of f(x[(o * r + k) * inner + c]) -----------------------------------------------
// blockIdx.y = o, blockIdx.z = segment of the reduced axis (rows_per_split rows each; segment s of o writes
// out[(s * outer + o) * inner + c], so that a second launch folds the segments as rows of one matrix).
// ROWS: rows of the reduced axis whose loads a thread issues before it runs the program on them.
template <int NS, int NT, int ROWS, class Prog>
__device__ __forceinline__ void chain_reduce_col_body(const Prog& prog, const void* in0, const Sides& sd, void* out,
                                                      long long vec_ok, long long outer, long long r, long long inner,
                                                      long long rows_per_split) {
  const int rop = prog.reduce_op(), out_type = prog.result_type();
  const float id     = cr_identity(rop);
  const long long o  = blockIdx.y;
  const long long k0 = (long long)blockIdx.z * rows_per_split;
  const long long k1 = k0 + rows_per_split < r ? k0 + rows_per_split : r;
  const long long ybase = ((long long)blockIdx.z * outer + o) * inner;
  if (vec_ok) {  // inner % 4 == 0 and aligned buffers
    const long long nc = inner >> 2;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < nc; c += (long long)gridDim.x * blockDim.x) {
      float a[4] = {id, id, id, id};
      long long k = k0;
      if constexpr (NT == 0 && ROWS == 4) {
        for (; k + 4 <= k1; k += 4) {
          float acc0[8], acc1[8];
          const long long ia = (o * r + k) * inner + (c << 2);
          chain_values2<NS>(prog, in0, sd, ia, ia + inner, acc0);
          chain_values2<NS>(prog, in0, sd, ia + 2 * inner, ia + 3 * inner, acc1);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i & 3] = cr_apply(rop, a[i & 3], acc0[i]);
#pragma unroll
          for (int i = 0; i < 8; ++i) a[i & 3] = cr_apply(rop, a[i & 3], acc1[i]);
        }
      }
      for (; NT == 0 && k + 2 <= k1; k += 2) {
        float acc[8];
        const long long ia = (o * r + k) * inner + (c << 2);
        chain_values2<NS>(prog, in0, sd, ia, ia + inner, acc);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i & 3] = cr_apply(rop, a[i & 3], acc[i]);
      }
      for (; k < k1; ++k) {
        float acc[4];
        chain_values<4, NS, NT>(prog, in0, sd, (o * r + k) * inner + (c << 2), acc);
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = cr_apply(rop, a[i], acc[i]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) cr_store(out, out_type, ybase + (c << 2) + i, a[i]);
    }
  } else {
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < inner; c += (long long)gridDim.x * blockDim.x) {
      float a = id;
      for (long long k = k0; k < k1; ++k) {
        float acc[1];
        chain_values<1, NS, NT>(prog, in0, sd, (o * r + k) * inner + c, acc);
        a = cr_apply(rop, a, acc[0]);
      }
      cr_store(out, out_type, ybase + c, a);
    }
  }
}

// The interpreting kernels.
template <int NS, int NT = 0>
__global__ void __launch_bounds__(256, NS == 0 ? 5 : 4)
    k_chain_reduce_row(CHAIN_PARAMS, long long rows, long long r, long long group) {
  grid_dependency_sync();
  CHAIN_STEPS;
  const DynProgram prog = {steps, (int)nsteps_ll, meta};
  chain_reduce_row_body<NS, NT>(prog, in0, make_sides(prog, p1, p2, p3, mid1, inner1, mid2, inner2, mid3, inner3), out,
                                vec_ok, rows, r, group);
}
template <int NS, int NT = 0>
__global__ void __launch_bounds__(256, NS == 0 ? 5 : 4)
    k_chain_reduce_col(CHAIN_PARAMS, long long outer, long long r, long long inner, long long rows_per_split) {
  grid_dependency_sync();
  CHAIN_STEPS;
  const DynProgram prog = {steps, (int)nsteps_ll, meta};
  chain_reduce_col_body<NS, NT, 2>(prog, in0, make_sides(prog, p1, p2, p3, mid1, inner1, mid2, inner2, mid3, inner3),
                                   out, vec_ok, outer, r, inner, rows_per_split);
}

// The same with the program fixed at build time (see ew_static.cu for the scheme; the table of these kernels,
// chain_reduce_static_table.inc, comes from the same generator).  These kernels evaluate exp / tanh / sigmoid through
// the hardware's approximate exponential and reciprocal (relative error about 1e-6 per term): a reduction's result is
// judged at 1e-5 relative, and with the full-precision forms sum(sigmoid(..)) is issue-bound at 0.46 of the HBM peak.
template <int NS, int NT, unsigned long long META, uint32_t... SIG>
__global__ void __launch_bounds__(256, 4)
    k_chain_reduce_row_static(CHAIN_PARAMS, long long rows, long long r, long long group) {
  grid_dependency_sync();
  CHAIN_STEPS;
  const StaticProgramT<META, true, SIG...> prog = {steps};
  chain_reduce_row_body<NS, NT>(prog, in0, make_sides(prog, p1, p2, p3, mid1, inner1, mid2, inner2, mid3, inner3), out,
                                vec_ok, rows, r, group);
}
template <int NS, int NT, unsigned long long META, uint32_t... SIG>
__global__ void __launch_bounds__(256)
    k_chain_reduce_col_static(CHAIN_PARAMS, long long outer, long long r, long long inner, long long rows_per_split) {
  grid_dependency_sync();
  CHAIN_STEPS;
  const StaticProgramT<META, true, SIG...> prog = {steps};
  chain_reduce_col_body<NS, NT, 4>(prog, in0, make_sides(prog, p1, p2, p3, mid1, inner1, mid2, inner2, mid3, inner3),
                                   out, vec_ok, outer, r, inner, rows_per_split);
}

template <uint32_t... SIG>
StaticChainKey MakeKey(const char* base, long long meta) {
  StaticChainKey k = {base, meta, (int)sizeof...(SIG), {SIG...}};
  return k;
}

}  // namespace

CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_row_s0", 34, 256, k_chain_reduce_row<0>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_row_s1", 34, 256, k_chain_reduce_row<1>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_row_s3", 34, 256, k_chain_reduce_row<3>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_row_s3t", 34, 256, k_chain_reduce_row<3, 2>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_col_s0", 35, 256, k_chain_reduce_col<0>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_col_s1", 35, 256, k_chain_reduce_col<1>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_col_s3", 35, 256, k_chain_reduce_col<3>);
CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_col_s3t", 35, 256, k_chain_reduce_col<3, 2>);

}  // namespace cinn_b200

namespace cinn_b200 {
#define STATIC_CHAIN_REDUCE_ROW(ID, BASE, NS, NT, META, ...)                                                          \
  CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_static_" #ID, 34, 256, k_chain_reduce_row_static<NS, NT, META##ull, __VA_ARGS__>); \
  static int cinn_b200_static_chain_reduce_##ID = RegisterStaticChain(MakeKey<__VA_ARGS__>(BASE, META##ll), "chain_reduce_static_" #ID)
#define STATIC_CHAIN_REDUCE_COL(ID, BASE, NS, NT, META, ...)                                                          \
  CINN_B200_REGISTER_KERNEL_PDL("chain_reduce_static_" #ID, 35, 256, k_chain_reduce_col_static<NS, NT, META##ull, __VA_ARGS__>); \
  static int cinn_b200_static_chain_reduce_##ID = RegisterStaticChain(MakeKey<__VA_ARGS__>(BASE, META##ll), "chain_reduce_static_" #ID)
#include "chain_reduce_static_table.inc"
}  // namespace cinn_b200
