// Data-movement ops that sit either side of the fused groups: transpose, slice, concat
// (cinn/hlir/op/transform.cc, cinn/hlir/pe/transform.cc: Transpose, Slice, Concat; reshape / squeeze / expand_dims
// are aliases of their operand's memory and launch nothing).  They move bits, so the kernels are typed by element
// SIZE only (1, 2, 4 or 8 bytes) and every element type shares them.
//
//   k_transpose_vec     a permutation that collapses to [B, R, C] -> [B, C, R] (NCHW <-> NHWC, matrix transposes):
//                       64 x 64 tiles through padded shared memory, 16-byte global accesses on both sides
//   k_transpose_tiled   the same with element-sized accesses, for odd extents or unaligned buffers
//   k_strided_gather    any other permutation and every slice: out[i] = in[base + sum_d coord_d(i) * stride_d]
//   k_copy_rows         concat: each operand's rows are copied to their column offset of the output rows
#include <cstdint>

#include "kernel_registry.h"

namespace cinn_b200 {
namespace {

template <int ES>
struct UnitOf;
template <> struct UnitOf<1> { using type = uint8_t; };
template <> struct UnitOf<2> { using type = uint16_t; };
template <> struct UnitOf<4> { using type = uint32_t; };
template <> struct UnitOf<8> { using type = unsigned long long; };
template <> struct UnitOf<16> { using type = uint4; };

constexpr int kTile = 64;

// in: [B, R, C], out: [B, C, R].  Block (64, 4): thread (tx, ty) moves 16 elements of column tx per tile.
template <int ES>
__global__ void __launch_bounds__(256)
    k_transpose_tiled(const void* __restrict__ in_v, void* __restrict__ out_v, long long B, long long R, long long C) {
  using U = typename UnitOf<ES>::type;
  __shared__ U tile[kTile][kTile + 1];
  const U* in = static_cast<const U*>(in_v);
  U* out      = static_cast<U*>(out_v);
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const long long tiles_c = (C + kTile - 1) / kTile, tiles_r = (R + kTile - 1) / kTile;
  const long long total   = B * tiles_r * tiles_c;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long b  = t / (tiles_r * tiles_c);
    const long long rc = t - b * tiles_r * tiles_c;
    const long long tr = rc / tiles_c, tc = rc - tr * tiles_c;
    const long long r0 = tr * kTile, c0 = tc * kTile;
    const U* pin = in + b * R * C;
    U* pout      = out + b * R * C;
#pragma unroll
    for (int k = 0; k < kTile / 4; ++k) {
      const int r = ty + 4 * k;
      if (r0 + r < R && c0 + tx < C) tile[r][tx] = pin[(r0 + r) * C + c0 + tx];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTile / 4; ++k) {
      const int c = ty + 4 * k;
      if (c0 + c < C && r0 + tx < R) pout[(c0 + c) * R + r0 + tx] = tile[tx][c];
    }
    __syncthreads();
  }
}

// The same transposition with 16-byte global accesses on both sides (R and C multiples of 16 / ES elements, 16-byte
// aligned buffers): a thread loads a vector of a tile row, scatters its elements into the padded tile, and after the
// barrier gathers a vector of a tile COLUMN and stores it.  Consecutive lanes take consecutive vectors of a row, so
// every warp access is a run of 256 contiguous bytes (or the whole tile row).
template <int ES>
__global__ void __launch_bounds__(256)
    k_transpose_vec(const void* __restrict__ in_v, void* __restrict__ out_v, long long B, long long R, long long C) {
  using U          = typename UnitOf<ES>::type;
  constexpr int VE = 16 / ES;                       // elements per 16-byte vector
  constexpr int VR = kTile / VE;                    // vectors per tile row
  constexpr int RP = 256 / VR;                      // tile rows handled per pass of the CTA
  constexpr int STRIDE = kTile + (ES >= 4 ? 1 : 4 / ES);  // row stride: an odd number of 32-bit words
  __shared__ U tile[kTile][STRIDE];
  const U* in = static_cast<const U*>(in_v);
  U* out      = static_cast<U*>(out_v);
  const int vq = threadIdx.x % VR, rq = threadIdx.x / VR;
  const long long tiles_c = (C + kTile - 1) / kTile, tiles_r = (R + kTile - 1) / kTile;
  const long long total   = B * tiles_r * tiles_c;
  for (long long t = blockIdx.x; t < total; t += gridDim.x) {
    const long long b  = t / (tiles_r * tiles_c);
    const long long rc = t - b * tiles_r * tiles_c;
    const long long tr = rc / tiles_c, tc = rc - tr * tiles_c;
    const long long r0 = tr * kTile, c0 = tc * kTile;
    const U* pin = in + b * R * C;
    U* pout      = out + b * R * C;
    uint4 v[kTile / RP];
#pragma unroll
    for (int k = 0; k < kTile / RP; ++k) {
      const int r = rq + RP * k;
      if (r0 + r < R && c0 + vq * VE < C) v[k] = __ldcs(reinterpret_cast<const uint4*>(pin + (r0 + r) * C + c0 + vq * VE));
    }
#pragma unroll
    for (int k = 0; k < kTile / RP; ++k) {
      const int r = rq + RP * k;
      if (r0 + r < R && c0 + vq * VE < C) {
        const U* e = reinterpret_cast<const U*>(&v[k]);
#pragma unroll
        for (int i = 0; i < VE; ++i) tile[r][vq * VE + i] = e[i];
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTile / RP; ++k) {
      const int c = rq + RP * k;
      if (c0 + c < C && r0 + vq * VE < R) {
        uint4 w;
        U* e = reinterpret_cast<U*>(&w);
#pragma unroll
        for (int i = 0; i < VE; ++i) e[i] = tile[vq * VE + i][c];
        __stcs(reinterpret_cast<uint4*>(pout + (c0 + c) * R + r0 + vq * VE), w);
      }
    }
    __syncthreads();
  }
}

// out[i] = in[base + sum_d coord_d(i) * stride_d]; extents / strides of up to six output axes, innermost last.
template <int ES>
__global__ void __launch_bounds__(256)
    k_strided_gather(const void* __restrict__ in_v, void* __restrict__ out_v, long long n, long long base,
                     long long nd, long long e0, long long e1, long long e2, long long e3, long long e4, long long e5,
                     long long s0, long long s1, long long s2, long long s3, long long s4, long long s5) {
  using U = typename UnitOf<ES>::type;
  const U* in = static_cast<const U*>(in_v);
  U* out      = static_cast<U*>(out_v);
  const long long ext[6] = {e0, e1, e2, e3, e4, e5}, str[6] = {s0, s1, s2, s3, s4, s5};
  const bool small = (n >> 31) == 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long off = base;
    if (small) {
      unsigned rem = (unsigned)i;
#pragma unroll
      for (int d = 5; d >= 0; --d) {
        if (d < nd) {
          const unsigned q = rem / (unsigned)ext[d];
          off += (long long)(rem - q * (unsigned)ext[d]) * str[d];
          rem = q;
        }
      }
    } else {
      long long rem = i;
#pragma unroll
      for (int d = 5; d >= 0; --d) {
        if (d < nd) {
          const long long q = rem / ext[d];
          off += (rem - q * ext[d]) * str[d];
          rem = q;
        }
      }
    }
    out[i] = in[off];
  }
}

// out[o * out_row + offset + j] = in[o * in_row + j], j < in_row, all counted in units of UB bytes.
template <int UB>
__global__ void __launch_bounds__(256)
    k_copy_rows(const void* __restrict__ in_v, void* __restrict__ out_v, long long rows, long long in_row,
                long long out_row, long long offset) {
  using U = typename UnitOf<UB>::type;
  const U* in = static_cast<const U*>(in_v);
  U* out      = static_cast<U*>(out_v);
  const long long n = rows * in_row;
  const bool small  = (n >> 31) == 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    long long o, j;
    if (small) {
      o = (unsigned)i / (unsigned)in_row;
      j = (unsigned)i - (unsigned)o * (unsigned)in_row;
    } else {
      o = i / in_row;
      j = i - o * in_row;
    }
    out[o * out_row + offset + j] = in[i];
  }
}

}  // namespace

#define REG_TRANSFORM(ES)                                                                          \
  CINN_B200_REGISTER_KERNEL("transpose_tiled_b" #ES, 5, 256, k_transpose_tiled<ES>);             \
  CINN_B200_REGISTER_KERNEL("transpose_vec_b" #ES, 5, 256, k_transpose_vec<ES>);                 \
  CINN_B200_REGISTER_KERNEL("strided_gather_b" #ES, 17, 256, k_strided_gather<ES>)
REG_TRANSFORM(1);
REG_TRANSFORM(2);
REG_TRANSFORM(4);
REG_TRANSFORM(8);
CINN_B200_REGISTER_KERNEL("copy_rows_b1", 6, 256, k_copy_rows<1>);
CINN_B200_REGISTER_KERNEL("copy_rows_b2", 6, 256, k_copy_rows<2>);
CINN_B200_REGISTER_KERNEL("copy_rows_b4", 6, 256, k_copy_rows<4>);
CINN_B200_REGISTER_KERNEL("copy_rows_b8", 6, 256, k_copy_rows<8>);
CINN_B200_REGISTER_KERNEL("copy_rows_b16", 6, 256, k_copy_rows<16>);

}  // namespace cinn_b200
