// Reduction over an axis that is sharded across the GPUs of one node, fused with its cross-GPU exchange.
//
// x is [R, inner] fp32 with R split over `world` ranks (one process per GPU).  The plain path runs the local column
// reduction and then an NCCL all-reduce of the [inner] partials, which at 4 MiB is pure latency (about 40 us on 8
// GPUs against 10-20 us of kernel).  Here ONE kernel per rank does both steps over NVLink peer memory:
//
//   phase 1  every CTA reduces its column tile over the local rows (eight 16-byte row loads in flight per thread)
//            and stores the partial straight into the OWNER rank's receive area (a peer store over NVLink; the
//            owner of a column is rank = column / (inner / world)).  When a rank has written a whole band it
//            publishes a flag on the owner (system-scope release).
//   phase 2  the CTAs of the band this rank owns wait (bounded) for the flags of all ranks, combine the `world`
//            partials of their tile, and write the result to the local output and, when the full result is wanted
//            on every rank, into every peer's gather area, followed by a second flag.
//   phase 3  (full result only) all CTAs wait (bounded) for the second flags and copy the gather area to the output.
//
// Peer memory is mapped with CUDA IPC (cudaIpcGetMemHandle / cudaIpcOpenMemHandle): plain peer loads/stores, no
// multicast objects.  All CTAs of the grid are co-resident (the launcher sizes the grid from the occupancy of the
// kernel), so a waiting CTA can never keep a CTA it waits for from being scheduled; every wait has an iteration
// limit, after which the kernel records the give-up (cinn_b200_device_status) and finishes without the exchange.
// The reference has no multi-GPU execution; this is new functionality (kinds: 0 sum, 1 prod, 2 max, 3 min).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/cinn_b200.h"
#include "device_math.cuh"
#include "tma_utils.cuh"

namespace cinn_b200 {

int SetLastError(int code, const std::string& message);  // runtime.cc

CINN_B200_DEFINE_ASYNC_TIMEOUT_COUNTER(g_peer_wait_timeouts);

namespace {

constexpr int kMaxWorld       = 16;
constexpr int kHeaderBytes    = 4096;  // flags at the start of every peer buffer
constexpr unsigned kSpinLimit = 1u << 20;  // polls of a flag in local memory, ~64 ns apart: about a second

// Header of a rank's peer buffer.  Flags only ever grow (they hold the epoch of the last completed call).
struct PeerHeader {
  unsigned int partial_ready[kMaxWorld];  // [src]: src has stored its partial of MY band for epoch >= value
  unsigned int band_ready[kMaxWorld];     // [owner]: owner has stored its final band into MY gather area
  unsigned int local_count[kMaxWorld];    // per band: CTAs of this rank that finished phase 1 (local use)
  unsigned int owner_count;               // CTAs of this rank that finished phase 2 (local use)
};

struct PeerPtrs {
  unsigned char* base[kMaxWorld];
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Thread 0 waits until *flag >= epoch (bounded); the CTA learns the outcome through shared memory.
__device__ __forceinline__ bool cta_wait_flag(const unsigned int* flag, unsigned int epoch, int* smem_ok) {
  if (threadIdx.x == 0) {
    int ok = 0;
    for (unsigned i = 0; i < kSpinLimit; ++i) {
      if ((int)(ld_acquire_sys(flag) - epoch) >= 0) {
        ok = 1;
        break;
      }
      __nanosleep(64);
    }
    *smem_ok = ok;
  }
  __syncthreads();
  const bool ok = *smem_ok != 0;
  __syncthreads();
  return ok;
}

template <class Op>
__global__ void __launch_bounds__(256)
    k_col_reduce_exchange(const float* __restrict__ x, float* __restrict__ out, PeerPtrs peers, int rank, int world,
                          long long rows, long long inner, int ctas_per_band, unsigned int epoch, int all_gather) {
  __shared__ int wait_ok;
  const long long band   = inner / world;   // columns per owner (inner % (4 * world) == 0)
  const long long band_v = band >> 2;       // float4 groups per band
  const int j            = blockIdx.x % world;  // band this CTA works on in phase 1
  const int sub          = blockIdx.x / world;
  PeerHeader* my_hdr     = reinterpret_cast<PeerHeader*>(peers.base[rank]);

  // ---- phase 1: local partial of band j -> owner j's receive area, slot [rank] --------------------------------
  {
    // The receive area is double-buffered by epoch parity: a fast rank may already store the partials of the next
    // call while the owner still reads those of this one (no rank can get two calls ahead, because finishing a call
    // needs a flag that every other rank raises only after it has finished the previous call).
    float* recv = reinterpret_cast<float*>(peers.base[j] + kHeaderBytes) + (long long)(epoch & 1u) * inner +
                  (long long)rank * band;
    const uint4* px = reinterpret_cast<const uint4*>(x) + (long long)j * band_v;
    const long long inner_v = inner >> 2;
    for (long long c = (long long)sub * blockDim.x + threadIdx.x; c < band_v; c += (long long)ctas_per_band * blockDim.x) {
      float a0 = Op::identity(), a1 = a0, a2 = a0, a3 = a0;
      long long k = 0;
      for (; k + 8 <= rows; k += 8) {
        uint4 u[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) u[q] = __ldcs(px + (k + q) * inner_v + c);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          a0 = Op::accum(a0, __uint_as_float(u[q].x));
          a1 = Op::accum(a1, __uint_as_float(u[q].y));
          a2 = Op::accum(a2, __uint_as_float(u[q].z));
          a3 = Op::accum(a3, __uint_as_float(u[q].w));
        }
      }
      for (; k < rows; ++k) {
        uint4 u = __ldcs(px + k * inner_v + c);
        a0      = Op::accum(a0, __uint_as_float(u.x));
        a1      = Op::accum(a1, __uint_as_float(u.y));
        a2      = Op::accum(a2, __uint_as_float(u.z));
        a3      = Op::accum(a3, __uint_as_float(u.w));
      }
      reinterpret_cast<uint4*>(recv)[c] =
          make_uint4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3));
    }
    // Publish: every thread's peer stores are made visible system-wide, then the last CTA of the band raises the flag.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned done = atomicAdd(&my_hdr->local_count[j], 1u) + 1;
      if (done == (unsigned)ctas_per_band) {
        my_hdr->local_count[j] = 0;
        __threadfence_system();
        st_release_sys(&reinterpret_cast<PeerHeader*>(peers.base[j])->partial_ready[rank], epoch);
      }
    }
  }

  // ---- phase 2: the owner combines the partials of its band -----------------------------------------------------
  bool healthy = true;
  if (j == rank) {
    for (int src = 0; src < world && healthy; ++src) healthy = cta_wait_flag(&my_hdr->partial_ready[src], epoch, &wait_ok);
    if (healthy) {
      const float* recv = reinterpret_cast<const float*>(peers.base[rank] + kHeaderBytes) + (long long)(epoch & 1u) * inner;
      for (long long c = (long long)sub * blockDim.x + threadIdx.x; c < band_v; c += (long long)ctas_per_band * blockDim.x) {
        float a0 = Op::identity(), a1 = a0, a2 = a0, a3 = a0;
        for (int src = 0; src < world; ++src) {
          // L2-only load: peers wrote these lines over NVLink, an L1 line of an earlier call could be stale
          const uint4 u = __ldcg(reinterpret_cast<const uint4*>(recv + (long long)src * band) + c);
          a0 = Op::apply(a0, __uint_as_float(u.x));
          a1 = Op::apply(a1, __uint_as_float(u.y));
          a2 = Op::apply(a2, __uint_as_float(u.z));
          a3 = Op::apply(a3, __uint_as_float(u.w));
        }
        const uint4 r = make_uint4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(a2), __float_as_uint(a3));
        if (all_gather) {
          for (int dst = 0; dst < world; ++dst) {
            float* gather = reinterpret_cast<float*>(peers.base[dst] + kHeaderBytes) + 2 * inner;
            reinterpret_cast<uint4*>(gather + (long long)rank * band)[c] = r;
          }
        } else {
          reinterpret_cast<uint4*>(out)[c] = r;  // out holds this rank's band only
        }
      }
    }
    if (all_gather) {
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(&my_hdr->owner_count, 1u) + 1;
        if (done == (unsigned)ctas_per_band) {
          my_hdr->owner_count = 0;
          __threadfence_system();
          // Raise the flag even after a failed wait so that the peers do not wait for this rank in turn.
          for (int dst = 0; dst < world; ++dst)
            st_release_sys(&reinterpret_cast<PeerHeader*>(peers.base[dst])->band_ready[rank], epoch);
        }
      }
    }
  }

  // ---- phase 3: full result on every rank: gather area -> out --------------------------------------------------------
  if (all_gather) {
    for (int owner = 0; owner < world && healthy; ++owner) healthy = cta_wait_flag(&my_hdr->band_ready[owner], epoch, &wait_ok);
    if (healthy) {
      const uint4* gather =
          reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(peers.base[rank] + kHeaderBytes) + 2 * inner);
      const long long inner_v = inner >> 2;
      for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < inner_v; c += (long long)gridDim.x * blockDim.x)
        reinterpret_cast<uint4*>(out)[c] = __ldcg(gather + c);
    }
  }
  if (!healthy && threadIdx.x == 0) atomicAdd(&g_peer_wait_timeouts, 1u);
}

}  // namespace
}  // namespace cinn_b200

using namespace cinn_b200;

struct cinn_b200_peer_ctx {
  int rank = 0, world = 1, device = 0;
  long long capacity_floats = 0;  // per area
  unsigned char* local = nullptr;
  PeerPtrs peers;
  bool connected = false;
  unsigned int epoch = 0;
};

extern "C" {

int cinn_b200_peer_create(int rank, int world, long long max_inner, unsigned char* handle_out /* 64 bytes */,
                          cinn_b200_peer_ctx** ctx_out) {
  if (!handle_out || !ctx_out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_inner <= 0)
    return SetLastError(CINN_B200_EINVAL, "peer_create: bad argument (world must be 1..16)");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  static_assert(sizeof(PeerHeader) <= kHeaderBytes, "header fits");
  auto* c = new cinn_b200_peer_ctx();
  c->rank = rank;
  c->world = world;
  cudaGetDevice(&c->device);
  c->capacity_floats = max_inner;
  // header + two receive areas [world][band] (= inner floats each, by epoch parity) + gather area [inner].  The areas
  // are laid out with the CALL's inner, so a context serves any inner <= max_inner.
  const size_t bytes = kHeaderBytes + (size_t)max_inner * 4 * 3;
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->local), bytes);
  if (e != cudaSuccess) {
    delete c;
    return SetLastError(CINN_B200_ECUDA, std::string("peer_create: cudaMalloc: ") + cudaGetErrorString(e));
  }
  cudaMemset(c->local, 0, kHeaderBytes);
  cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, c->local);
  if (e != cudaSuccess) {
    cudaFree(c->local);
    delete c;
    return SetLastError(CINN_B200_ECUDA, std::string("peer_create: cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  memcpy(handle_out, &h, 64);
  memset(&c->peers, 0, sizeof(c->peers));
  c->peers.base[rank] = c->local;
  *ctx_out = c;
  return CINN_B200_OK;
}

int cinn_b200_peer_connect(cinn_b200_peer_ctx* c, const unsigned char* all_handles /* world * 64 bytes */) {
  if (!c || !all_handles) return SetLastError(CINN_B200_EINVAL, "peer_connect: bad argument");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, all_handles + (size_t)r * 64, 64);
    void* p       = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return SetLastError(CINN_B200_ECUDA, "peer_connect: cudaIpcOpenMemHandle of rank " + std::to_string(r) + ": " + cudaGetErrorString(e));
    c->peers.base[r] = static_cast<unsigned char*>(p);
  }
  c->connected = true;
  return CINN_B200_OK;
}

int cinn_b200_peer_destroy(cinn_b200_peer_ctx* c) {
  if (!c) return CINN_B200_OK;
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (r != c->rank && c->peers.base[r]) cudaIpcCloseMemHandle(c->peers.base[r]);
  if (c->local) cudaFree(c->local);
  delete c;
  return CINN_B200_OK;
}

int cinn_b200_col_reduce_sharded_f32(cinn_b200_peer_ctx* c, int kind, const float* x_local, long long rows_local,
                                     long long inner, float* out, int all_gather, void* stream) {
  if (!c || !x_local || !out || rows_local <= 0 || inner <= 0 || kind < 0 || kind > 3)
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: bad argument");
  if (!c->connected && c->world > 1) return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: peers are not connected");
  if (inner > c->capacity_floats)
    return SetLastError(CINN_B200_ENOSPACE, "col_reduce_sharded: inner exceeds the capacity the context was created with");
  if (inner % (4LL * c->world) != 0)
    return SetLastError(CINN_B200_ESHAPE, "col_reduce_sharded: inner must be a multiple of 4 * world");
  if ((reinterpret_cast<uintptr_t>(x_local) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: buffers must be 16-byte aligned");
  const void* fn = nullptr;
  switch (kind) {
    case 0: fn = reinterpret_cast<const void*>(&k_col_reduce_exchange<SumOp>); break;
    case 1: fn = reinterpret_cast<const void*>(&k_col_reduce_exchange<ProdOp>); break;
    case 2: fn = reinterpret_cast<const void*>(&k_col_reduce_exchange<MaxOp>); break;
    default: fn = reinterpret_cast<const void*>(&k_col_reduce_exchange<MinOp>); break;
  }
  // Every CTA must be resident at once: waiting CTAs then never occupy a slot a CTA they depend on would need.
  int per_sm = 0, sms = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, 256, 0);
  if (e != cudaSuccess || per_sm < 1) return SetLastError(CINN_B200_ECUDA, "col_reduce_sharded: occupancy query failed");
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
  const long long band_v = inner / c->world / 4;
  long long ctas_per_band = (band_v + 255) / 256;
  const long long cap     = (long long)per_sm * sms / c->world;
  if (ctas_per_band > cap) ctas_per_band = cap;
  if (ctas_per_band > 128) ctas_per_band = 128;
  if (ctas_per_band < 1) return SetLastError(CINN_B200_ECUDA, "col_reduce_sharded: the GPU cannot hold one CTA per band");
  c->epoch += 1;
  int rank = c->rank, world = c->world, cpb = (int)ctas_per_band, ag = all_gather ? 1 : 0;
  unsigned int epoch = c->epoch;
  void* params[] = {&x_local, &out, &c->peers, &rank, &world, &rows_local, &inner, &cpb, &epoch, &ag};
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim  = dim3((unsigned)(ctas_per_band * world), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream   = static_cast<cudaStream_t>(stream);
  e = cudaLaunchKernelExC(&cfg, fn, params);
  if (e != cudaSuccess) return SetLastError(CINN_B200_ECUDA, std::string("col_reduce_sharded: launch: ") + cudaGetErrorString(e));
  return CINN_B200_OK;
}

}  // extern "C"
