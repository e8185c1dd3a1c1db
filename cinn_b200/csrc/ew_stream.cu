// Streaming form of cast<OutT>(tanh(scale * (x + bias[col]) + shift)): x arrives through warp-private rings of
// shared-memory buffers filled by bulk asynchronous copies (TMA), so the bytes in flight per SM are set by the ring
// depth rather than by how many loads the math-heavy threads can keep outstanding in registers.
//
// Same group, same arithmetic and same reference semantics as k_bias_scale_tanh_cast in ew_kernels.cu
// (cinn/hlir/pe/broadcast.cc:216-273, cinn/hlir/op/elementwise.cc:149-163, cinn/backends/llvm/llvm_intrin_rule.h:136-154,
// cinn/hlir/pe/elementwise.cc:213-217).  That kernel is latency-bound: its threads issue four 16-byte loads, then
// spend ~200 instructions on eight tanh evaluations before they issue the next loads.  Here each WARP owns a ring of
// S buffers of 2 KiB (512 consecutive fp32 elements); lane 0 issues one cp.async.bulk per buffer, S-1 buffers ahead
// of the one being consumed, and waits on that buffer's mbarrier (bounded); the lanes read their slices with
// conflict-free 16-byte shared loads, compute, and write 8-byte pieces that are contiguous across the warp.  A warp
// never waits for another warp: there is no CTA-wide barrier in the loop.
//
// Requirements (checked by the planner, else the register kernel is used): 16-byte aligned x / bias / out,
// cols % 4 == 0 (a lane's 4-element pieces never straddle a row end).
#include "device_math.cuh"
#include "kernel_registry.h"
#include "tma_utils.cuh"

namespace cinn_b200 {

CINN_B200_DEFINE_ASYNC_TIMEOUT_COUNTER(g_ew_stream_wait_timeouts);

namespace {

constexpr int kChunk      = 512;          // elements per warp iteration
constexpr int kChunkBytes = kChunk * 4;   // 2 KiB
constexpr int kWarps      = 8;

template <typename OutT>
__device__ __forceinline__ void store4(OutT* p, const float (&f)[4]);
template <>
__device__ __forceinline__ void store4<__half>(__half* p, const float (&f)[4]) {
  __stcs(reinterpret_cast<uint2*>(p), make_uint2(pack_h2(f[0], f[1]), pack_h2(f[2], f[3])));
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
  __stcs(reinterpret_cast<uint2*>(p), make_uint2(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3])));
}

template <typename OutT>
__global__ void __launch_bounds__(256)
    k_bias_scale_tanh_cast_stream(const float* __restrict__ x, const float* __restrict__ bias, OutT* __restrict__ y,
                                  long long n, long long cols, long long stages_ll, double scale_d, double shift_d) {
  grid_dependency_sync();
  extern __shared__ __align__(128) unsigned char ring_all[];
  __shared__ __align__(8) uint64_t full[kWarps][kMaxStages];
  const int lane           = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stages         = (int)stages_ll;
  const float scale        = (float)scale_d;
  const float shift        = (float)shift_d;
  unsigned char* ring      = ring_all + (size_t)warp * stages * kChunkBytes;
  const long long gw       = (long long)blockIdx.x * kWarps + warp;   // global warp index
  const long long nw       = (long long)gridDim.x * kWarps;
  const long long nchunks  = n / kChunk;
  const long long my       = gw < nchunks ? (nchunks - gw + nw - 1) / nw : 0;

  if (lane == 0) {
    for (int s = 0; s < stages; ++s) mbar_init(&full[warp][s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const int pre = (int)(my < stages ? my : stages);
    for (int s = 0; s < pre; ++s) {
      mbar_arrive_expect_tx(&full[warp][s], kChunkBytes);
      bulk_load_row(ring + (size_t)s * kChunkBytes, x + (gw + (long long)s * nw) * kChunk, kChunkBytes, &full[warp][s]);
    }
  }
  __syncwarp();

  // Lane l handles, in every chunk, the four 4-element pieces at element offsets (l + 32 j) * 4, j = 0..3.
  // Their columns are (chunk_start + offset) % cols.  chunk_start % cols advances by `step` per iteration;
  // when step == 0 (the planner arranges that whenever it can) the sixteen bias values stay in registers.
  const unsigned ucols     = (unsigned)cols;
  const unsigned step      = (unsigned)((nw * kChunk) % cols);
  unsigned base_col        = (unsigned)((gw * kChunk) % cols);
  float fb[4][4];
  auto load_bias = [&](unsigned start) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      unsigned c = (start + (unsigned)(lane + 32 * j) * 4u) % ucols;
      unpack4(ld_keep16(bias + c), fb[j]);
    }
  };
  if (my > 0) load_bias(base_col);

  bool gave_up = false;
  long long k  = 0;
  for (; k < my; ++k) {
    const int s           = (int)(k % stages);
    const uint32_t parity = (uint32_t)((k / stages) & 1);
    int ok = 1;
    if (lane == 0) ok = mbar_wait_bounded(&full[warp][s], parity) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();  // orders every lane's reads of the buffer after the completion lane 0 observed
    if (!ok) {
      gave_up = true;
      break;
    }
    const long long chunk = gw + k * nw;
    const uint4* src      = reinterpret_cast<const uint4*>(ring + (size_t)s * kChunkBytes);
    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) raw[j] = src[lane + 32 * j];
    __syncwarp();  // every lane has its copy of buffer s in registers
    if (lane == 0 && k + stages < my) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_expect_tx(&full[warp][s], kChunkBytes);
      bulk_load_row(ring + (size_t)s * kChunkBytes, x + (chunk + (long long)stages * nw) * kChunk, kChunkBytes,
                    &full[warp][s]);
    }
    OutT* dst = y + chunk * kChunk;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float fx[4], fy[4];
      unpack4(raw[j], fx);
#pragma unroll
      for (int i = 0; i < 4; ++i) fy[i] = x86_tanh_for_16bit_out(fmaf(scale, fx[i] + fb[j][i], shift));
      store4<OutT>(dst + (lane + 32 * j) * 4, fy);
    }
    if (step != 0) {
      base_col += step;
      if (base_col >= ucols) base_col -= ucols;
      load_bias(base_col);
    }
  }
  if (gave_up) {
    if (lane == 0) {
      atomicAdd(&g_ew_stream_wait_timeouts, 1u);
      // Drain the copies already issued into this warp's ring (bounded) before the CTA can exit.
      for (long long kk = k + 1; kk < my && kk < k + stages; ++kk)
        (void)mbar_wait_bounded(&full[warp][(int)(kk % stages)], (uint32_t)((kk / stages) & 1));
    }
    return;
  }
  // Elements past the last whole chunk: plain loads, all threads of the grid.
  const long long tid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = nchunks * kChunk + tid; i < n; i += stride)
    Io<OutT>::store1(y + i, x86_tanh_for_16bit_out(fmaf(scale, x[i] + bias[i % cols], shift)));
}

}  // namespace

CINN_B200_REGISTER_KERNEL_PDL("ew_bias_scale_tanh_cast_stream_f32_f16", 8, 256, k_bias_scale_tanh_cast_stream<__half>);
CINN_B200_REGISTER_KERNEL_PDL("ew_bias_scale_tanh_cast_stream_f32_bf16", 8, 256,
                          k_bias_scale_tanh_cast_stream<__nv_bfloat16>);

}  // namespace cinn_b200
