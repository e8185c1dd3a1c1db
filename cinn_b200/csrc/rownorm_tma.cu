// softmax / layer_norm along the last axis with the rows streamed through shared memory by the TMA engine.
//
// Same arithmetic and same reference semantics as rownorm_kernels.cu (cinn/hlir/pe/nn.cc:755-796 for softmax,
// cinn/frontend/op_mappers/paddle/layer_norm.cc:84-139 for the layer_norm composition).  What changes is how
// the bytes move: a persistent CTA owns a ring of S row buffers in shared memory; one thread issues a bulk
// asynchronous copy (cp.async.bulk, completion counted on an mbarrier) for each row S-1 rows ahead of the row
// being normalised, so the bytes in flight per SM are set by the ring depth instead of by how many registers
// the resident threads can spare.  Each thread reads its 16-byte slices of the current row from shared memory,
// the CTA reduces once (one barrier per row), the freed buffer is re-armed for the row S ahead, and the
// results go back to HBM with 16-byte streaming stores.
//
// Every wait on an mbarrier is bounded: a thread that gives up records it in a device-side counter (readable
// through cinn_b200_device_status), drains the other armed buffers with bounded waits and leaves the kernel.
#include "device_math.cuh"
#include "kernel_registry.h"
#include "tma_utils.cuh"

namespace cinn_b200 {

CINN_B200_DEFINE_ASYNC_TIMEOUT_COUNTER(g_rownorm_wait_timeouts);

namespace {

// EXACT: a row is exactly VPT vectors per thread -- no test per vector (with the tests every vector is a basic block
// of its own; without them a thread's shared-memory reads are issued together and its arithmetic interleaves).  A
// wait that ran out is then not tested per vector either: the thread reads whatever the ring buffer holds (its own
// shared memory), and the CTA leaves at the barrier of the same row before anything is stored.
template <typename T, int G, int VPT, bool LAYERNORM, bool EXACT>
__device__ __forceinline__ void rownorm_tma_body(const T* __restrict__ x, const float* __restrict__ gamma,
                                                 const float* __restrict__ beta, T* __restrict__ y, long long rows,
                                                 long long cols, long long stages_ll, double eps_d) {
  constexpr int V      = Io<T>::kVec;
  constexpr int NWARPS = G / 32;
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ __align__(8) uint64_t full[kMaxStages];
  __shared__ __align__(16) float2 partial[2][32];
  __shared__ volatile int abort_flag;  // set by a warp whose bounded wait ran out

  const int t              = threadIdx.x;
  const int lane           = t & 31, warp = t >> 5;
  const int stages         = (int)stages_ll;
  const int nvec           = (int)(cols / V);
  const uint32_t row_bytes = (uint32_t)(cols * sizeof(T));
  const float inv_n        = (float)(1.0 / (double)cols);
  const float eps          = (float)eps_d;
  // Rows of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const long long my_rows = rows > (long long)blockIdx.x ? (rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (t == 0) {
    abort_flag = 0;
    for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (t == 0) {
    const int pre = (int)(my_rows < stages ? my_rows : stages);
    for (int s = 0; s < pre; ++s) {
      mbar_arrive_expect_tx(&full[s], row_bytes);
      bulk_load_row(ring + (size_t)s * row_bytes, x + ((long long)blockIdx.x + (long long)s * gridDim.x) * cols,
                    row_bytes, &full[s]);
    }
  }

  // This thread's columns are the same for every row, so its slices of gamma / beta stay in registers.
  float g[LAYERNORM ? VPT : 1][V], b[LAYERNORM ? VPT : 1][V];
  if (LAYERNORM) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (EXACT || v < nvec) {
#pragma unroll
        for (int q = 0; q < V / 4; ++q) {
          Io<float>::unpack(ld_keep16(gamma + (long long)v * V + 4 * q), &g[j][4 * q]);
          Io<float>::unpack(ld_keep16(beta + (long long)v * V + 4 * q), &b[j][4 * q]);
        }
      }
    }
  }

  bool gave_up = false;
  long long k  = 0;
  for (; k < my_rows; ++k) {
    const int s           = (int)(k % stages);
    const uint32_t parity = (uint32_t)((k / stages) & 1);
    // One lane per warp polls the barrier (bounded).  The warp barrier after the broadcast orders the other lanes'
    // reads of the buffer after the completion that lane 0 observed (a shuffle alone orders nothing).  A warp whose
    // wait ran out raises the CTA's abort flag and still goes through this row's CTA barrier (with zero partials),
    // after which every warp sees the flag and leaves the loop together: no warp continues on unwritten partials.
    int ok = 1;
    if (lane == 0) ok = mbar_wait_bounded(&full[s], parity) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    if (!ok && lane == 0) abort_flag = 1;
    const long long row = (long long)blockIdx.x + k * gridDim.x;
    const uint4* src    = reinterpret_cast<const uint4*>(ring + (size_t)s * row_bytes);
    float f[VPT][V];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int v = t + j * G;
      if (EXACT || (v < nvec && ok)) {
        Io<T>::unpack(src[v], f[j]);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          if (LAYERNORM) {
            s1 = s1 + f[j][i];
            // 16-bit storage (1e-2 tolerance): the square is accumulated with one fused multiply-add.
            s2 = sizeof(T) == 2 ? fmaf(f[j][i], f[j][i], s2) : s2 + f[j][i] * f[j][i];
          } else {
            f[j][i] = sizeof(T) == 2 ? exp_for_16bit_out(f[j][i]) : expf(f[j][i]);
            s1      = s1 + f[j][i];
          }
        }
      }
    }
    // One CTA-wide reduction of (s1, s2) with a single barrier; the scratch is double-buffered by row parity.
    s1 = warp_allreduce<SumOp>(s1);
    if (LAYERNORM) s2 = warp_allreduce<SumOp>(s2);
    float2* scratch = partial[k & 1];
    if (lane == 0) scratch[warp] = make_float2(s1, s2);
    __syncthreads();  // also: every thread has finished reading ring buffer s
    if (abort_flag) {
      gave_up = true;
      break;
    }
    if (t == 0 && k + stages < my_rows) {
      // Order the generic-proxy reads of buffer s before the async-proxy write that refills it.
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_expect_tx(&full[s], row_bytes);
      bulk_load_row(ring + (size_t)s * row_bytes, x + (row + (long long)stages * gridDim.x) * cols, row_bytes,
                    &full[s]);
    }
    // Every thread adds the per-warp partials itself (broadcast shared-memory reads, fixed order).
    {
      const float4* pp = reinterpret_cast<const float4*>(scratch);
      float t1 = 0.0f, t2 = 0.0f;
#pragma unroll
      for (int w = 0; w < NWARPS / 2; ++w) {
        const float4 q = pp[w];
        t1             = (t1 + q.x) + q.z;
        t2             = (t2 + q.y) + q.w;
      }
      s1 = t1;
      s2 = t2;
    }

    uint4* dst = reinterpret_cast<uint4*>(y + row * cols);
    if (LAYERNORM) {
      // Reduction tolerance class (1e-5): multiply by 1/N and use the hardware reciprocal square root.
      const float mean = s1 * inv_n;
      const float var  = x86_max(s2 * inv_n - mean * mean, 0.0f);
      const float rstd = rsqrtf(var + eps);
      const float nmr  = -mean * rstd;  // 16-bit storage: (x - mean) * rstd as one fma(x, rstd, -mean * rstd)
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = t + j * G;
        if (EXACT || v < nvec) {
#pragma unroll
          for (int i = 0; i < V; ++i)
            f[j][i] = sizeof(T) == 2 ? fmaf(fmaf(f[j][i], rstd, nmr), g[j][i], b[j][i])
                                     : fmaf((f[j][i] - mean) * rstd, g[j][i], b[j][i]);
          __stcs(dst + v, Io<T>::pack(f[j]));
        }
      }
    } else {
      const float inv_s = 1.0f / s1;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = t + j * G;
        if (EXACT || v < nvec) {
#pragma unroll
          for (int i = 0; i < V; ++i) f[j][i] = f[j][i] * inv_s;
          __stcs(dst + v, Io<T>::pack(f[j]));
        }
      }
    }
  }
  if (gave_up) {
    if (t == 0) atomicAdd(&g_rownorm_wait_timeouts, 1u);
    // Copies already issued for later rows still target this CTA's shared memory: wait for them (bounded)
    // before the CTA exits.  Rows k+1 .. k+stages-1 (if they exist) are armed.
    for (long long kk = k + 1; kk < my_rows && kk < k + stages; ++kk)
      (void)mbar_wait_bounded(&full[(int)(kk % stages)], (uint32_t)((kk / stages) & 1));
  }
}

// (both bodies in one kernel, deliberately: see k_rownorm_reg)
template <typename T, int G, int VPT, bool LAYERNORM>
__global__ void __launch_bounds__(G)
    k_rownorm_tma(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                  T* __restrict__ y, long long rows, long long cols, long long stages_ll, double eps_d) {
  grid_dependency_sync();
  if (cols == (long long)G * VPT * Io<T>::kVec)
    rownorm_tma_body<T, G, VPT, LAYERNORM, true>(x, gamma, beta, y, rows, cols, stages_ll, eps_d);
  else
    rownorm_tma_body<T, G, VPT, LAYERNORM, false>(x, gamma, beta, y, rows, cols, stages_ll, eps_d);
}

}  // namespace

// Self-test of the bounded-wait path: waits on an mbarrier that nothing will ever complete, with a small poll
// limit, records the give-up in this file's counter exactly as the streaming kernels do, and returns.  It lets a
// host test check that a wait that runs out surfaces through cinn_b200_device_status without any kernel hanging.
__global__ void __launch_bounds__(32) k_selftest_bounded_wait(long long polls) {
  grid_dependency_sync();
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    bool done = false;
    for (long long i = 0; i < polls && !done; ++i) done = mbar_try_wait(&bar, 0);
    if (!done) atomicAdd(&g_rownorm_wait_timeouts, 1u);
  }
}
CINN_B200_REGISTER_KERNEL_PDL("selftest_bounded_wait", 1, 32, k_selftest_bounded_wait);

#define REG_TMA_ONE(TNAME, T, G, VPT)                                                               \
  CINN_B200_REGISTER_KERNEL_PDL("softmax_tma_" TNAME "_g" #G "_v" #VPT, 8, G, k_rownorm_tma<T, G, VPT, false>); \
  CINN_B200_REGISTER_KERNEL_PDL("layernorm_tma_" TNAME "_g" #G "_v" #VPT, 8, G, k_rownorm_tma<T, G, VPT, true>)
#define REG_TMA_G(TNAME, T, G) \
  REG_TMA_ONE(TNAME, T, G, 1); \
  REG_TMA_ONE(TNAME, T, G, 2); \
  REG_TMA_ONE(TNAME, T, G, 4)

REG_TMA_G("f32", float, 128);
REG_TMA_G("f32", float, 256);
REG_TMA_G("f32", float, 512);
REG_TMA_G("f16", __half, 128);
REG_TMA_G("f16", __half, 256);
REG_TMA_G("f16", __half, 512);
REG_TMA_G("bf16", __nv_bfloat16, 128);
REG_TMA_G("bf16", __nv_bfloat16, 256);
REG_TMA_G("bf16", __nv_bfloat16, 512);

}  // namespace cinn_b200
