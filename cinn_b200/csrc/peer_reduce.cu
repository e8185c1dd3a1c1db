// Reduction over an axis that is sharded across the GPUs of one node, fused with its cross-GPU exchange.
//
// x is [R, inner] fp32 with R split over `world` ranks (one process per GPU).  The plain path runs the local column
// reduction and then an NCCL all-reduce of the [inner] partials, which at 4 MiB is pure latency (about 40 us on 8
// GPUs against 10-20 us of kernel).  Here ONE kernel per rank does both steps over NVLink peer memory:
//
//   phase 1  every CTA reduces its column tile over the local rows (eight 16-byte row loads in flight per thread)
//            and stores the partial straight into the OWNER rank's receive area (a peer store over NVLink; the
//            owner of a column is rank = column / (inner / world)).
//   phase 2  each thread of the band this rank owns waits (bounded) for the `world` partials of its four columns,
//            combines them in rank order, and writes the result to the local output and, when the full result is
//            wanted on every rank, into every peer's gather area.
//   phase 3  (full result only) the threads of the other bands wait (bounded) for their four columns in the gather
//            area and copy them to the output.
//
// There are no flags and no fences: the data is its own arrival signal.  Every receive and gather cell holds a
// sentinel bit pattern (an all-ones NaN, which senders never store: they rewrite it to the default NaN) until the
// value lands, and a waiting thread polls its own 16-byte cell until none of the four words is the sentinel.  A
// system-scope fence after the peer stores cost 12-18 us here; polling the data costs one NVLink write latency.
// The areas are used round-robin over three calls: a call reads area k % 3 and resets the cells it owns in area
// (k + 2) % 3, which the previous call consumed and which no peer can write before it has received this rank's
// data of the NEXT call (and that is sent only after this kernel has ended).
//
// Peer memory is mapped with CUDA IPC (cudaIpcGetMemHandle / cudaIpcOpenMemHandle): plain peer loads/stores, no
// multicast objects.  All CTAs of the grid are co-resident (the launcher sizes the grid from the occupancy of the
// kernel), so a waiting CTA can never keep a CTA some rank waits for from being scheduled; every thread has a poll
// budget, after which the kernel records the give-up (cinn_b200_device_status) and finishes without the exchange;
// the context is then unusable and has to be destroyed.
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

constexpr int kMaxWorld         = 16;
constexpr int kAreas            = 6;           // receive areas 0..2 and gather areas 3..5, `capacity` floats each
constexpr int kCtrlBytes        = 256;         // after the areas: [0] calls completed, [1] CTAs done in this call
constexpr unsigned kSentinel    = 0xFFFFFFFFu;  // "not arrived yet"
constexpr unsigned kDefaultNan  = 0x7FFFFFFFu;  // what a value with the sentinel's bits is sent as
constexpr unsigned kPollBudget  = 1u << 19;     // polls per thread and call, ~1 us each: about half a second

#ifdef CINN_B200_PEER_TRACE
// Development aid, compiled out by default: the latest time (globaltimer, ns) at which any CTA passed each point of
// the kernel, per call, kept in the rank's own buffer after the areas.
__device__ __forceinline__ void trace_point(unsigned long long* trace, unsigned int epoch, int slot) {
  if (threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMax(trace + (epoch & 127u) * 8 + slot, t);
  }
}
#define PEER_TRACE(slot) \
  trace_point(reinterpret_cast<unsigned long long*>(peers.base[rank] + (size_t)kAreas * capacity * 4 + kCtrlBytes), epoch, slot)
#else
#define PEER_TRACE(slot)
#endif

struct PeerPtrs {
  unsigned char* base[kMaxWorld];
};

__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_v4(uint4* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ bool arrived(const uint4& u) {
  return u.x != kSentinel && u.y != kSentinel && u.z != kSentinel && u.w != kSentinel;
}
__device__ __forceinline__ unsigned sendable(float v) {
  const unsigned b = __float_as_uint(v);
  return b == kSentinel ? kDefaultNan : b;
}
// Polls a cell of this rank's own memory until all four words have arrived or the thread's budget is spent.
__device__ __forceinline__ bool wait_cell(const uint4* p, uint4& u, unsigned& budget) {
  while (!arrived(u)) {
    if (budget == 0) return false;
    --budget;
    __nanosleep(64);
    u = ld_relaxed_sys_v4(p);
  }
  return true;
}

template <class Op>
__global__ void __launch_bounds__(256)
    k_col_reduce_exchange(const float* __restrict__ x, float* __restrict__ out, PeerPtrs peers, int rank, int world,
                          long long rows, long long inner, long long capacity, int ctas_per_band, int all_gather) {
  // The call counter lives on the device (the last CTA to finish advances it), so a launch carries no per-call
  // argument and can be replayed from a CUDA graph.
  unsigned int* ctrl = reinterpret_cast<unsigned int*>(peers.base[rank] + (size_t)kAreas * capacity * 4);
  __shared__ unsigned int epoch_s;
  if (threadIdx.x == 0) epoch_s = (*reinterpret_cast<volatile unsigned int*>(ctrl) + 1u) % 384u;  // a multiple of 3
  __syncthreads();
  const unsigned int epoch = epoch_s;
  const long long band_v  = inner / world >> 2;  // float4 groups per owner (inner % (4 * world) == 0)
  const long long inner_v = inner >> 2;
  const int j             = blockIdx.x % world;  // band this CTA works on
  const int sub           = blockIdx.x / world;  // its column tile: float4 groups sub*256 + t (+ k * ctas_per_band*256)
  const long long c0      = (long long)sub * blockDim.x + threadIdx.x;
  const long long cstep   = (long long)ctas_per_band * blockDim.x;
  const unsigned cur = epoch % 3u, stale = (epoch + 2u) % 3u;
  const uint4 sentinel4 = make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
  auto area = [&](int r, unsigned a) { return reinterpret_cast<uint4*>(peers.base[r] + (size_t)a * capacity * 4); };
  PEER_TRACE(0);

  // ---- phase 1: local partial of tile (j, sub) -> owner j's receive area, slot [rank] ---------------------------
  {
    uint4* recv     = area(j, cur) + (long long)rank * band_v;
    const uint4* px = reinterpret_cast<const uint4*>(x) + (long long)j * band_v;
    for (long long c = c0; c < band_v; c += cstep) {
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
      st_relaxed_sys_v4(recv + c, make_uint4(sendable(a0), sendable(a1), sendable(a2), sendable(a3)));
    }
    PEER_TRACE(1);
  }

  unsigned budget = kPollBudget;
  bool healthy    = true;
  if (j == rank) {
    // ---- phase 2: the owner combines the `world` partials of its columns, in rank order --------------------------
    const uint4* recv = area(rank, cur);
    uint4* recv_stale = area(rank, stale);
    for (long long c = c0; c < band_v && healthy; c += cstep) {
      float a0 = Op::identity(), a1 = a0, a2 = a0, a3 = a0;
      for (int s0 = 0; s0 < world; s0 += 4) {
        uint4 u[4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (s0 + q < world) u[q] = ld_relaxed_sys_v4(recv + (long long)(s0 + q) * band_v + c);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (s0 + q < world) {
            healthy = healthy && wait_cell(recv + (long long)(s0 + q) * band_v + c, u[q], budget);
            a0 = Op::apply(a0, __uint_as_float(u[q].x));
            a1 = Op::apply(a1, __uint_as_float(u[q].y));
            a2 = Op::apply(a2, __uint_as_float(u[q].z));
            a3 = Op::apply(a3, __uint_as_float(u[q].w));
          }
        }
      }
      if (!healthy) break;  // nothing is sent on: the peers run out of budget too, so every rank reports it
      const uint4 r = make_uint4(sendable(a0), sendable(a1), sendable(a2), sendable(a3));
      if (all_gather) {
        reinterpret_cast<uint4*>(out)[(long long)rank * band_v + c] = r;  // own band: straight to the output
        for (int d = 1; d < world; ++d) {
          const int dst = (rank + d) % world;  // every rank starts with a different peer
          st_relaxed_sys_v4(area(dst, 3 + cur) + (long long)rank * band_v + c, r);
        }
      } else {
        reinterpret_cast<uint4*>(out)[c] = r;  // out holds this rank's band only
      }
      for (int s = 0; s < world; ++s) recv_stale[(long long)s * band_v + c] = sentinel4;
    }
    PEER_TRACE(3);
  } else if (all_gather) {
    // ---- phase 3: full result on every rank: columns of band j from the gather area -> out ----------------------
    const uint4* gather = area(rank, 3 + cur) + (long long)j * band_v;
    uint4* gather_stale = area(rank, 3 + stale) + (long long)j * band_v;
    uint4* o            = reinterpret_cast<uint4*>(out) + (long long)j * band_v;
    for (long long c = c0; c < band_v; c += cstep) {
      uint4 u = ld_relaxed_sys_v4(gather + c);
      healthy = wait_cell(gather + c, u, budget);
      if (!healthy) break;
      o[c]            = u;
      gather_stale[c] = sentinel4;
    }
    PEER_TRACE(5);
  }
  const int failed = __syncthreads_or(!healthy);
  if (threadIdx.x == 0) {
    if (failed) atomicAdd(&g_peer_wait_timeouts, 1u);
    // Every CTA has read the counter before it gets here, so the last one may advance it.
    if (atomicAdd(ctrl + 1, 1u) + 1u == gridDim.x) {
      ctrl[1] = 0;
      ctrl[0] = epoch;
    }
  }
  PEER_TRACE(6);
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
  long long inner = 0;  // fixed by the first call, like the mode: the cells a call resets are those of the last one
  int all_gather = -1;
  int ctas_per_sm = 0;
};

extern "C" {

int cinn_b200_peer_create(int rank, int world, long long max_inner, unsigned char* handle_out /* 64 bytes */,
                          cinn_b200_peer_ctx** ctx_out) {
  if (!handle_out || !ctx_out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_inner <= 0)
    return SetLastError(CINN_B200_EINVAL, "peer_create: bad argument (world must be 1..16)");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  auto* c = new cinn_b200_peer_ctx();
  c->rank = rank;
  c->world = world;
  cudaGetDevice(&c->device);
  c->capacity_floats = max_inner;
  // three receive areas [world][band] and three gather areas [inner], every cell "not arrived"
  size_t bytes = (size_t)kAreas * max_inner * 4 + kCtrlBytes;
#ifdef CINN_B200_PEER_TRACE
  bytes += 128 * 8 * 8;
#endif
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&c->local), bytes);
  if (e != cudaSuccess) {
    delete c;
    return SetLastError(CINN_B200_ECUDA, std::string("peer_create: cudaMalloc: ") + cudaGetErrorString(e));
  }
  cudaMemset(c->local, 0xFF, (size_t)kAreas * max_inner * 4);
#ifdef CINN_B200_PEER_TRACE
  cudaMemset(c->local + (size_t)kAreas * max_inner * 4 + kCtrlBytes, 0, 128 * 8 * 8);
#endif
  cudaMemset(c->local + (size_t)kAreas * max_inner * 4, 0, kCtrlBytes);
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

#ifdef CINN_B200_PEER_TRACE
int cinn_b200_peer_trace_read(cinn_b200_peer_ctx* c, unsigned long long* dst /* 128 * 8 */) {
  cudaDeviceSynchronize();
  return cudaMemcpy(dst, c->local + (size_t)kAreas * c->capacity_floats * 4 + kCtrlBytes, 128 * 8 * 8, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}
#endif

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
  if (c->inner == 0) {
    c->inner      = inner;
    c->all_gather = all_gather ? 1 : 0;
  } else if (c->inner != inner || c->all_gather != (all_gather ? 1 : 0)) {
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: a context serves one inner size and one result mode");
  }
  // Every CTA must be resident at once: waiting CTAs then never occupy a slot a CTA some rank depends on would need.
  int sms = 0;
  cudaError_t e = cudaSuccess;
  if (c->ctas_per_sm == 0) {
    int per_sm = 0;  // the same for all four instantiations to within a CTA; queried for the one in use
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, 256, 0);
    if (e != cudaSuccess || per_sm < 1) return SetLastError(CINN_B200_ECUDA, "col_reduce_sharded: occupancy query failed");
    c->ctas_per_sm = per_sm;
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
  const long long band_v = inner / c->world / 4;
  long long ctas_per_band = (band_v + 255) / 256;
  const long long cap     = (long long)c->ctas_per_sm * sms / c->world;
  if (ctas_per_band > cap) ctas_per_band = cap;
  if (ctas_per_band < 1) return SetLastError(CINN_B200_ECUDA, "col_reduce_sharded: the GPU cannot hold one CTA per band");
  int rank = c->rank, world = c->world, cpb = (int)ctas_per_band, ag = all_gather ? 1 : 0;
  void* params[] = {&x_local, &out, &c->peers, &rank, &world, &rows_local, &inner, &c->capacity_floats, &cpb, &ag};
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
