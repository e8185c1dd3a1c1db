// The grid-stride body shared by the interpreted chain kernel (ew_chain.cu) and the chain kernels specialised at
// build time (ew_static.cu).  `Prog` says what is known when: the interpreter's program answers from kernel
// parameters at run time, a static program answers with constants, and every test below then folds away.
//
//   prog.in_type()        storage type of the chain input (EwDType), EW_NO_INPUT when the chain starts from an operand
//   prog.side_dtype(k)    storage type of side input k (1..3)
//   prog.side_mode(k)     EwSideMode of side input k
//   prog.out2_type()      storage type of the second output (EW_STORE2)
//   prog.run<VEC, NS, NT, ST2>(s1, s2, s3, acc, st2)   applies the program to VEC values
#pragma once

#include "ew_chain_device.cuh"

namespace cinn_b200 {
namespace {

struct ChainGeometry {
  long long n, vec_ok;
  long long mid1, inner1, mid2, inner2, mid3, inner3;
};

// UNROLL: vectors (of four elements) a thread takes per iteration when the program needs no temporaries; all of
// their loads are issued before the program runs once over the UNROLL * 4 values.
template <typename OutT, int NS, int NT, bool ST2, int UNROLL, class Prog>
__device__ __forceinline__ void ew_chain_body(const Prog& prog, const void* __restrict__ in0,
                                              const void* __restrict__ p1, const void* __restrict__ p2,
                                              const void* __restrict__ p3, OutT* __restrict__ out,
                                              const ChainGeometry& geo, void* __restrict__ out2) {
  const int in_type   = prog.in_type();
  const int out2_type = prog.out2_type();
  const SideSpec sd1  = {p1, prog.side_dtype(1), prog.side_mode(1), geo.mid1, geo.inner1};
  const SideSpec sd2  = {p2, prog.side_dtype(2), prog.side_mode(2), geo.mid2, geo.inner2};
  const SideSpec sd3  = {p3, prog.side_dtype(3), prog.side_mode(3), geo.mid3, geo.inner3};
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n      = geo.n;
  long long done         = 0;
  if (geo.vec_ok) {
    const long long nvec = n >> 2;
    long long v = tid;
    if constexpr (NT == 0 && UNROLL == 2) {
      for (; v + stride < nvec; v += 2 * stride) {
        float acc[8], s1[8], s2[8], s3[8];
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (in_type != EW_NO_INPUT)
            load_vec4(in0, in_type, (v + j * stride) << 2, true, *reinterpret_cast<float(*)[4]>(&acc[4 * j]));
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const long long i0 = (v + j * stride) << 2;
          if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, *reinterpret_cast<float(*)[4]>(&s1[4 * j]));
          if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, *reinterpret_cast<float(*)[4]>(&s2[4 * j]));
          if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, *reinterpret_cast<float(*)[4]>(&s3[4 * j]));
        }
        const Store2 st2 = {out2, out2_type, v << 2, (v + stride) << 2};
        prog.template run<8, NS, 0, ST2>(s1, s2, s3, acc, ST2 ? &st2 : nullptr);
#pragma unroll
        for (int j = 0; j < 2; ++j)
          store_vec4<OutT>(out, (v + j * stride) << 2, *reinterpret_cast<float(*)[4]>(&acc[4 * j]));
      }
    }
    if constexpr (UNROLL == 4) {
      // Four independent vectors per iteration, each run through the program on its own (a static program is a
      // handful of instructions, so running it four times costs nothing and keeps four loads per operand in flight).
      for (; v + 3 * stride < nvec; v += 4 * stride) {
        float acc[4][4], s1[4][4], s2[4][4], s3[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long i0 = (v + j * stride) << 2;
          if (in_type != EW_NO_INPUT) load_vec4(in0, in_type, i0, true, acc[j]);
          if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, s1[j]);
          if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, s2[j]);
          if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, s3[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long i0 = (v + j * stride) << 2;
          const Store2 st2   = {out2, out2_type, i0, 0};
          prog.template run<4, NS, NT, ST2>(s1[j], s2[j], s3[j], acc[j], ST2 ? &st2 : nullptr);
          store_vec4<OutT>(out, i0, acc[j]);
        }
      }
    }
    for (; v < nvec; v += stride) {
      const long long i0 = v << 2;
      float acc[4], s1[4], s2[4], s3[4];
      if (in_type != EW_NO_INPUT) load_vec4(in0, in_type, i0, true, acc);
      if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<4>(sd1, i0, s1);
      if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<4>(sd2, i0, s2);
      if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<4>(sd3, i0, s3);
      const Store2 st2 = {out2, out2_type, i0, 0};
      prog.template run<4, NS, NT, ST2>(s1, s2, s3, acc, ST2 ? &st2 : nullptr);
      store_vec4<OutT>(out, i0, acc);
    }
    done = nvec << 2;
  }
  for (long long i = done + tid; i < n; i += stride) {
    float acc[1], s1[1], s2[1], s3[1];
    acc[0] = in_type != EW_NO_INPUT ? load_scalar(in0, in_type, i) : 0.0f;
    if (NS >= 1 && sd1.mode != EW_SIDE_NONE) load_side<1>(sd1, i, s1);
    if (NS >= 2 && sd2.mode != EW_SIDE_NONE) load_side<1>(sd2, i, s2);
    if (NS >= 3 && sd3.mode != EW_SIDE_NONE) load_side<1>(sd3, i, s3);
    const Store2 st2 = {out2, out2_type, i, 0};
    prog.template run<1, NS, NT, ST2>(s1, s2, s3, acc, ST2 ? &st2 : nullptr);
    store_one<OutT>(out, i, acc[0]);
  }
}

// The interpreter's program: everything comes from kernel parameters.
struct DynProgram {
  static constexpr bool kStatic = false;
  const long long* steps;
  int nsteps;
  long long meta;
  __device__ __forceinline__ int in_type() const { return (int)((meta >> 24) & 15); }
  __device__ __forceinline__ int out2_type() const { return (int)((meta >> 36) & 15); }
  // the reductions with a chain as operand (chain_reduce.cu): reduce op and storage type of the result
  __device__ __forceinline__ int reduce_op() const { return (int)((meta >> 28) & 3); }
  __device__ __forceinline__ int result_type() const { return (int)((meta >> 32) & 15); }
  __device__ __forceinline__ int side_dtype(int k) const { return (int)((meta >> (8 * (k - 1))) & 15); }
  __device__ __forceinline__ int side_mode(int k) const { return (int)((meta >> (8 * (k - 1) + 4)) & 15); }
  template <int VEC, int NS, int NT, bool ST2>
  __device__ __forceinline__ void run(const float (&s1)[VEC], const float (&s2)[VEC], const float (&s3)[VEC],
                                      float (&acc)[VEC], const Store2* st2) const {
    run_chain<VEC, NS, NT, ST2>(steps, nsteps, s1, s2, s3, acc, st2);
  }
};

// A program whose structure was fixed when the library was built: META is the kernel's `meta` word, SIG... the low
// halves of its step words.  Only the immediates (the high halves) are read from the parameters.
// FAST: see apply_unary (the specialised reductions only).
template <unsigned long long META, bool FAST, uint32_t... SIG>
struct StaticProgramT {
  static constexpr bool kStatic = true;
  const long long* steps;
  __device__ __forceinline__ constexpr int in_type() const { return (int)((META >> 24) & 15); }
  __device__ __forceinline__ constexpr int out2_type() const { return (int)((META >> 36) & 15); }
  __device__ __forceinline__ constexpr int reduce_op() const { return (int)((META >> 28) & 3); }
  __device__ __forceinline__ constexpr int result_type() const { return (int)((META >> 32) & 15); }
  __device__ __forceinline__ constexpr int side_dtype(int k) const { return (int)((META >> (8 * (k - 1))) & 15); }
  __device__ __forceinline__ constexpr int side_mode(int k) const { return (int)((META >> (8 * (k - 1) + 4)) & 15); }
  template <int VEC, int NS, int NT, bool ST2>
  __device__ __forceinline__ void run(const float (&s1)[VEC], const float (&s2)[VEC], const float (&s3)[VEC],
                                      float (&acc)[VEC], const Store2* st2) const {
    run_chain_static<VEC, NS, NT, ST2, FAST, SIG...>(steps, s1, s2, s3, acc, st2);
  }
};
template <unsigned long long META, uint32_t... SIG>
using StaticProgram = StaticProgramT<META, false, SIG...>;

}  // namespace
}  // namespace cinn_b200
