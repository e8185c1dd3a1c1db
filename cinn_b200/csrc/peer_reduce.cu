// Reduction over an axis that is sharded across the GPUs of one node, fused with its cross-GPU exchange.
//
// x is [R, inner] fp32 with R split over `world` ranks (one process per GPU).  The plain path runs the local column
// reduction and then an NCCL all-reduce of the [inner] partials, which at 4 MiB is pure latency (about 40 us on 8
// GPUs against 10-20 us of kernel).  Here ONE kernel per rank does both steps over NVLink peer memory, and the
// exchange is pipelined with the local reduction tile by tile, because at 8 ranks the exchange is not latency but
// NVLink bandwidth: an all-reduce of 4 MiB moves 2 * 7/8 * 4 MiB out of (and into) every GPU, 10 us at the
// measured peer bandwidth -- as long as the local reduction itself -- when it is sent in two bursts at the end.
//
// The CTAs of a launch take one of three roles (all are resident at once; the launcher sizes the grid from the
// kernel's occupancy), and all of them walk the column tiles in the same ascending order, so that the roles follow
// each other like the stages of a pipeline:
//
//   reducers   take (tile, band) items in order: reduce a tile of 256 float4 column groups over the local rows (eight
//              16-byte row loads in flight per thread) and store the partial straight into the OWNER rank's receive
//              area (a peer store over NVLink; the owner of a column is rank = column / (inner / world)).
//   combiners  own this rank's band: each thread waits (bounded) for the `world` partials of its four columns,
//              combines them in rank order, writes the result to the local output and, when the full result is
//              wanted on every rank, stores it into every peer's gather area.
//   gatherers  (full result only) wait (bounded) for the columns of the other bands in this rank's gather area and
//              copy them to the output.
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
// multicast objects.  Every thread has a poll budget, after which the kernel records the give-up
// (cinn_b200_device_status), marks the context failed in its control block (later launches return at once,
// cinn_b200_peer_status reports it) and finishes without the exchange.  The ranks' launches therefore have to start
// within that budget of each other (about a quarter of a second).
//
// The rank is `rank0 + blockIdx.y`: a production launch has gridDim.y == 1; the emulated form runs all ranks of a
// world as ONE launch on one GPU (gridDim.y == world, every rank's buffers in that GPU's memory), so that the
// exchange protocol can be checked where only one GPU is present.
// The reference has no multi-GPU execution; this is new functionality (kinds: 0 sum, 1 prod, 2 max, 3 min).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/cinn_b200.h"
#include "device_math.cuh"
#include "tma_utils.cuh"

namespace cinn_b200 {

int SetLastError(int code, const std::string& message);  // runtime.cc
int OptPeerReducersPerSm();                                // runtime.cc: option "peer_reducers_per_sm"

CINN_B200_DEFINE_ASYNC_TIMEOUT_COUNTER(g_peer_wait_timeouts);

namespace {

constexpr int kMaxWorld         = 16;
constexpr int kAreas            = 6;           // receive areas 0..2 and gather areas 3..5, `capacity` floats each
constexpr int kCtrlBytes        = 256;         // after the areas: [0] calls completed, [1] CTAs done, [2] failed
constexpr int kTile             = 256;         // float4 column groups per tile = threads per CTA
constexpr unsigned kSentinel    = 0xFFFFFFFFu;  // "not arrived yet"
constexpr unsigned kDefaultNan  = 0x7FFFFFFFu;  // what a value with the sentinel's bits is sent as
constexpr unsigned kPollBudget  = 1u << 19;     // polls per thread and call, ~0.5 us each: about a quarter second

struct ExchangeArgs {
  const float* x[kMaxWorld];      // local rows of each rank this launch runs (production: only [rank])
  float* out[kMaxWorld];          // result buffer of each rank this launch runs
  unsigned char* base[kMaxWorld];  // exchange buffer of every rank of the world, as mapped in this process
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
    __nanosleep(96);
    u = ld_relaxed_sys_v4(p);
  }
  return true;
}

template <class Op>
__global__ void __launch_bounds__(kTile)
    k_col_reduce_exchange(ExchangeArgs args, int rank0, int world, long long rows, long long inner,
                          long long capacity, int n_red, int n_comb, int n_gath, int all_gather) {
  const int rank = rank0 + blockIdx.y;
  unsigned char* my_base = args.base[rank];
  // The call counter lives on the device (the last CTA to finish advances it), so a launch carries no per-call
  // argument and can be replayed from a CUDA graph.
  unsigned int* ctrl = reinterpret_cast<unsigned int*>(my_base + (size_t)kAreas * capacity * 4);
  __shared__ unsigned int epoch_s, failed_s;
  if (threadIdx.x == 0) {
    epoch_s  = (*reinterpret_cast<volatile unsigned int*>(ctrl) + 1u) % 384u;  // a multiple of 3
    failed_s = *reinterpret_cast<volatile unsigned int*>(ctrl + 2);
  }
  __syncthreads();
  if (failed_s) return;  // an earlier call gave up a wait: the areas' contents mean nothing any more
  const unsigned int epoch = epoch_s;
  const long long band_v   = inner / world >> 2;  // float4 groups per owner (inner % (4 * world) == 0)
  const long long inner_v  = inner >> 2;
  const long long tiles    = (band_v + kTile - 1) / kTile;  // per band
  const unsigned cur = epoch % 3u, stale = (epoch + 2u) % 3u;
  const uint4 sentinel4 = make_uint4(kSentinel, kSentinel, kSentinel, kSentinel);
  auto area = [&](int r, unsigned a) { return reinterpret_cast<uint4*>(args.base[r] + (size_t)a * capacity * 4); };

  unsigned budget = kPollBudget;
  bool healthy    = true;
  const int b     = blockIdx.x;
  if (b < n_red) {
    // ---- reducer: item q = (tile q / world, band q % world); partial -> owner's receive area, slot [rank] ---------
    const uint4* x4 = reinterpret_cast<const uint4*>(args.x[rank]);
    for (long long q = b; q < tiles * world; q += n_red) {
      const int j       = (int)(q % world);
      const long long c = (q / world) * kTile + threadIdx.x;
      if (c >= band_v) continue;
      const uint4* px = x4 + (long long)j * band_v + c;
      float a0 = Op::identity(), a1 = a0, a2 = a0, a3 = a0;
      long long k = 0;
      for (; k + 8 <= rows; k += 8) {
        uint4 u[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) u[i] = __ldcs(px + (k + i) * inner_v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          a0 = Op::accum(a0, __uint_as_float(u[i].x));
          a1 = Op::accum(a1, __uint_as_float(u[i].y));
          a2 = Op::accum(a2, __uint_as_float(u[i].z));
          a3 = Op::accum(a3, __uint_as_float(u[i].w));
        }
      }
      for (; k < rows; ++k) {
        uint4 u = __ldcs(px + k * inner_v);
        a0      = Op::accum(a0, __uint_as_float(u.x));
        a1      = Op::accum(a1, __uint_as_float(u.y));
        a2      = Op::accum(a2, __uint_as_float(u.z));
        a3      = Op::accum(a3, __uint_as_float(u.w));
      }
      st_relaxed_sys_v4(area(j, cur) + (long long)rank * band_v + c,
                        make_uint4(sendable(a0), sendable(a1), sendable(a2), sendable(a3)));
    }
  } else if (b < n_red + n_comb) {
    // ---- combiner: the owner folds the `world` partials of its columns, in rank order -----------------------------
    const uint4* recv = area(rank, cur);
    uint4* recv_stale = area(rank, stale);
    uint4* o          = reinterpret_cast<uint4*>(args.out[rank]) + (all_gather ? (long long)rank * band_v : 0);
    for (long long c = (long long)(b - n_red) * kTile + threadIdx.x; c < band_v && healthy;
         c += (long long)n_comb * kTile) {
      float a0 = Op::identity(), a1 = a0, a2 = a0, a3 = a0;
      for (int s0 = 0; s0 < world; s0 += 4) {
        uint4 u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (s0 + i < world) u[i] = ld_relaxed_sys_v4(recv + (long long)(s0 + i) * band_v + c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (s0 + i < world) {
            healthy = healthy && wait_cell(recv + (long long)(s0 + i) * band_v + c, u[i], budget);
            a0 = Op::apply(a0, __uint_as_float(u[i].x));
            a1 = Op::apply(a1, __uint_as_float(u[i].y));
            a2 = Op::apply(a2, __uint_as_float(u[i].z));
            a3 = Op::apply(a3, __uint_as_float(u[i].w));
          }
        }
      }
      if (!healthy) break;  // nothing is sent on: the peers run out of budget too, so every rank reports it
      const uint4 r = make_uint4(sendable(a0), sendable(a1), sendable(a2), sendable(a3));
      if (all_gather)
        for (int d = 1; d < world; ++d) {
          const int dst = (rank + d) % world;  // every rank starts with a different peer
          st_relaxed_sys_v4(area(dst, 3 + cur) + (long long)rank * band_v + c, r);
        }
      o[c] = r;
      for (int s = 0; s < world; ++s) recv_stale[(long long)s * band_v + c] = sentinel4;
    }
  } else {
    // ---- gatherer (full result on every rank): the other bands' columns, tile by tile, gather area -> out ----------
    const long long groups = tiles * (world - 1);  // (tile, peer) pairs, tile-major like the reducers' order
    for (long long g = b - n_red - n_comb; g < groups && healthy; g += n_gath) {
      const int j       = (rank + 1 + (int)(g % (world - 1))) % world;
      const long long c = (g / (world - 1)) * kTile + threadIdx.x;
      if (c >= band_v) continue;
      const uint4* cell = area(rank, 3 + cur) + (long long)j * band_v + c;
      uint4 u           = ld_relaxed_sys_v4(cell);
      healthy           = wait_cell(cell, u, budget);
      if (!healthy) break;
      reinterpret_cast<uint4*>(args.out[rank])[(long long)j * band_v + c] = u;
      area(rank, 3 + stale)[(long long)j * band_v + c]                    = sentinel4;
    }
  }
  const int failed = __syncthreads_or(!healthy);
  if (threadIdx.x == 0) {
    if (failed) {
      atomicAdd(&g_peer_wait_timeouts, 1u);
      atomicExch(ctrl + 2, 1u);
    }
    // Every CTA has read the counter before it gets here, so the last one may advance it.
    if (atomicAdd(ctrl + 1, 1u) + 1u == gridDim.x) {
      ctrl[1] = 0;
      ctrl[0] = epoch;
    }
  }
}

const void* KernelOfKind(int kind) {
  switch (kind) {
    case 0: return reinterpret_cast<const void*>(&k_col_reduce_exchange<SumOp>);
    case 1: return reinterpret_cast<const void*>(&k_col_reduce_exchange<ProdOp>);
    case 2: return reinterpret_cast<const void*>(&k_col_reduce_exchange<MaxOp>);
    default: return reinterpret_cast<const void*>(&k_col_reduce_exchange<MinOp>);
  }
}

size_t BufferBytes(long long capacity_floats) { return (size_t)kAreas * capacity_floats * 4 + kCtrlBytes; }

// A fresh exchange buffer: every cell "not arrived", control block zero.
cudaError_t AllocExchangeBuffer(long long capacity_floats, unsigned char** out) {
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(out), BufferBytes(capacity_floats));
  if (e != cudaSuccess) return e;
  e = cudaMemset(*out, 0xFF, (size_t)kAreas * capacity_floats * 4);
  if (e == cudaSuccess) e = cudaMemset(*out + (size_t)kAreas * capacity_floats * 4, 0, kCtrlBytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(*out);
    *out = nullptr;
  }
  return e;
}

}  // namespace
}  // namespace cinn_b200

using namespace cinn_b200;

struct cinn_b200_peer_ctx {
  int rank = 0, world = 1, device = 0;
  bool emulated = false;          // all ranks' buffers on this device, one launch runs them all
  long long capacity_floats = 0;  // per area
  unsigned char* local = nullptr;  // this rank's buffer (emulated: unused, see bases)
  ExchangeArgs args;
  bool connected = false, imports_open = false;
  long long inner = 0;  // fixed by the first call, like the mode: the cells a call resets are those of the last one
  int all_gather = -1;
  int ctas_per_sm = 0, sms = 0;
};

namespace {

// Checks the call against the context and splits the resident CTAs over the three roles.
int PlanLaunch(cinn_b200_peer_ctx* c, int kind, long long rows_local, long long inner, int all_gather, int ranks_in_launch,
               const void** fn_out, int* n_red, int* n_comb, int* n_gath) {
  if (rows_local <= 0 || inner <= 0 || kind < 0 || kind > 3)
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: bad argument");
  if (inner > c->capacity_floats)
    return SetLastError(CINN_B200_ENOSPACE, "col_reduce_sharded: inner exceeds the capacity the context was created with");
  if (inner % (4LL * c->world) != 0)
    return SetLastError(CINN_B200_ESHAPE, "col_reduce_sharded: inner must be a multiple of 4 * world");
  if (c->inner == 0) {
    c->inner      = inner;
    c->all_gather = all_gather ? 1 : 0;
  } else if (c->inner != inner || c->all_gather != (all_gather ? 1 : 0)) {
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: a context serves one inner size and one result mode");
  }
  const void* fn = KernelOfKind(kind);
  // Every CTA must be resident at once: waiting CTAs then never occupy a slot a CTA some rank depends on would need.
  if (c->ctas_per_sm == 0) {
    int per_sm = 0;  // the same for all four instantiations to within a CTA; queried for the one in use
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kTile, 0);
    if (e != cudaSuccess || per_sm < 1) return SetLastError(CINN_B200_ECUDA, "col_reduce_sharded: occupancy query failed");
    c->ctas_per_sm = per_sm;
    cudaDeviceGetAttribute(&c->sms, cudaDevAttrMultiProcessorCount, c->device);
  }
  const long long cap    = (long long)c->ctas_per_sm * c->sms / ranks_in_launch;
  const long long band_v = inner / c->world / 4;
  const long long tiles  = (band_v + kTile - 1) / kTile;
  const bool gather      = all_gather && c->world > 1;
  // Combiners and gatherers mostly wait; one CTA per SM each is plenty, the rest of the slots reduce.
  long long comb = std::min<long long>(tiles, std::max<long long>(1, std::min<long long>(c->sms, cap / 4)));
  long long gath = gather ? std::min<long long>(tiles * (c->world - 1), std::max<long long>(1, std::min<long long>(c->sms, cap / 4))) : 0;
  long long red  = std::min<long long>(tiles * c->world, cap - comb - gath);
  // Fewer reducers than fit finish their items sooner, one round after the other, so that the partials (and with them
  // the exchange) are spread over the whole reduction instead of arriving in one or two bursts.
  if (OptPeerReducersPerSm() > 0) red = std::min<long long>(red, (long long)OptPeerReducersPerSm() * c->sms / ranks_in_launch);
  if (red < 1) return SetLastError(CINN_B200_ECUDA, "col_reduce_sharded: the GPU cannot hold one CTA per role");
  // Every reducer gets the same number of items (1024 items on 316 CTAs would leave most of them idle during the
  // fourth round; 256 CTAs with four items each finish together).
  const long long rounds = (tiles * c->world + red - 1) / red;
  red                    = (tiles * c->world + rounds - 1) / rounds;
  *fn_out = fn;
  *n_red  = (int)red;
  *n_comb = (int)comb;
  *n_gath = (int)gath;
  return CINN_B200_OK;
}

int Launch(cinn_b200_peer_ctx* c, const void* fn, int rank0, int ranks_in_launch, long long rows_local, long long inner,
           int n_red, int n_comb, int n_gath, int all_gather, void* stream) {
  int world = c->world, ag = all_gather ? 1 : 0;
  void* params[] = {&c->args, &rank0, &world, &rows_local, &inner, &c->capacity_floats, &n_red, &n_comb, &n_gath, &ag};
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim  = dim3((unsigned)(n_red + n_comb + n_gath), (unsigned)ranks_in_launch, 1);
  cfg.blockDim = dim3(kTile, 1, 1);
  cfg.stream   = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaLaunchKernelExC(&cfg, fn, params);
  if (e != cudaSuccess) return SetLastError(CINN_B200_ECUDA, std::string("col_reduce_sharded: launch: ") + cudaGetErrorString(e));
  return CINN_B200_OK;
}

}  // namespace

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
  memset(&c->args, 0, sizeof(c->args));
  // three receive areas [world][band] and three gather areas [inner], every cell "not arrived"
  cudaError_t e = AllocExchangeBuffer(max_inner, &c->local);
  if (e != cudaSuccess) {
    delete c;
    return SetLastError(CINN_B200_ECUDA, std::string("peer_create: exchange buffer: ") + cudaGetErrorString(e));
  }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, c->local);
  if (e != cudaSuccess) {
    cudaFree(c->local);
    delete c;
    return SetLastError(CINN_B200_ECUDA, std::string("peer_create: cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
  }
  memcpy(handle_out, &h, 64);
  c->args.base[rank] = c->local;
  *ctx_out = c;
  return CINN_B200_OK;
}

int cinn_b200_peer_connect(cinn_b200_peer_ctx* c, const unsigned char* all_handles /* world * 64 bytes */) {
  if (!c || !all_handles || c->emulated) return SetLastError(CINN_B200_EINVAL, "peer_connect: bad argument");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, all_handles + (size_t)r * 64, 64);
    void* p       = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess)
      return SetLastError(CINN_B200_ECUDA, "peer_connect: cudaIpcOpenMemHandle of rank " + std::to_string(r) + ": " + cudaGetErrorString(e));
    c->args.base[r] = static_cast<unsigned char*>(p);
  }
  c->connected    = true;
  c->imports_open = true;
  return CINN_B200_OK;
}

int cinn_b200_peer_create_emulated(int world, long long max_inner, cinn_b200_peer_ctx** ctx_out) {
  if (!ctx_out || world < 1 || world > kMaxWorld || max_inner <= 0)
    return SetLastError(CINN_B200_EINVAL, "peer_create_emulated: bad argument (world must be 1..16)");
  auto* c = new cinn_b200_peer_ctx();
  c->world    = world;
  c->emulated = true;
  cudaGetDevice(&c->device);
  c->capacity_floats = max_inner;
  memset(&c->args, 0, sizeof(c->args));
  for (int r = 0; r < world; ++r) {
    cudaError_t e = AllocExchangeBuffer(max_inner, &c->args.base[r]);
    if (e != cudaSuccess) {
      for (int k = 0; k < r; ++k) cudaFree(c->args.base[k]);
      delete c;
      return SetLastError(CINN_B200_ECUDA, std::string("peer_create_emulated: exchange buffer: ") + cudaGetErrorString(e));
    }
  }
  c->connected = true;
  *ctx_out     = c;
  return CINN_B200_OK;
}

int cinn_b200_peer_close_imports(cinn_b200_peer_ctx* c) {
  if (!c) return CINN_B200_OK;
  cudaSetDevice(c->device);
  cudaDeviceSynchronize();
  if (c->imports_open)
    for (int r = 0; r < c->world; ++r)
      if (r != c->rank && c->args.base[r]) {
        cudaIpcCloseMemHandle(c->args.base[r]);
        c->args.base[r] = nullptr;
      }
  c->imports_open = false;
  c->connected    = c->world == 1;
  return CINN_B200_OK;
}

int cinn_b200_peer_destroy(cinn_b200_peer_ctx* c) {
  if (!c) return CINN_B200_OK;
  cinn_b200_peer_close_imports(c);
  if (c->emulated) {
    for (int r = 0; r < c->world; ++r)
      if (c->args.base[r]) cudaFree(c->args.base[r]);
  } else if (c->local) {
    cudaFree(c->local);
  }
  delete c;
  return CINN_B200_OK;
}

int cinn_b200_peer_status(cinn_b200_peer_ctx* c, int* failed_out) {
  if (!c || !failed_out) return SetLastError(CINN_B200_EINVAL, "peer_status: bad argument");
  cudaSetDevice(c->device);
  unsigned int any = 0;
  for (int r = 0; r < c->world; ++r) {
    if (!c->emulated && r != c->rank) continue;
    unsigned int word = 0;
    cudaError_t e = cudaMemcpy(&word, c->args.base[r] + (size_t)kAreas * c->capacity_floats * 4 + 8, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return SetLastError(CINN_B200_ECUDA, std::string("peer_status: ") + cudaGetErrorString(e));
    any |= word;
  }
  *failed_out = any ? 1 : 0;
  return CINN_B200_OK;
}

int cinn_b200_col_reduce_sharded_f32(cinn_b200_peer_ctx* c, int kind, const float* x_local, long long rows_local,
                                     long long inner, float* out, int all_gather, void* stream) {
  if (!c || c->emulated || !x_local || !out) return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: bad argument");
  if (!c->connected && c->world > 1) return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: peers are not connected");
  if ((reinterpret_cast<uintptr_t>(x_local) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded: buffers must be 16-byte aligned");
  const void* fn = nullptr;
  int n_red = 0, n_comb = 0, n_gath = 0;
  int rc = PlanLaunch(c, kind, rows_local, inner, all_gather, 1, &fn, &n_red, &n_comb, &n_gath);
  if (rc != CINN_B200_OK) return rc;
  c->args.x[c->rank]   = x_local;
  c->args.out[c->rank] = out;
  return Launch(c, fn, c->rank, 1, rows_local, inner, n_red, n_comb, n_gath, all_gather, stream);
}

int cinn_b200_col_reduce_sharded_f32_emulated_ranks(cinn_b200_peer_ctx* c, int kind, const float* const* x_per_rank,
                                                    long long rows_local, long long inner, float* const* out_per_rank,
                                                    int all_gather, int rank0, int nranks, void* stream) {
  if (!c || !c->emulated || !x_per_rank || !out_per_rank || rank0 < 0 || nranks < 1 || rank0 + nranks > c->world)
    return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded_emulated: bad argument");
  for (int r = rank0; r < rank0 + nranks; ++r) {
    if (!x_per_rank[r] || !out_per_rank[r] ||
        ((reinterpret_cast<uintptr_t>(x_per_rank[r]) | reinterpret_cast<uintptr_t>(out_per_rank[r])) & 15u))
      return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded_emulated: buffers must be non-null and 16-byte aligned");
    c->args.x[r]   = x_per_rank[r];
    c->args.out[r] = out_per_rank[r];
  }
  const void* fn = nullptr;
  int n_red = 0, n_comb = 0, n_gath = 0;
  int rc = PlanLaunch(c, kind, rows_local, inner, all_gather, nranks, &fn, &n_red, &n_comb, &n_gath);
  if (rc != CINN_B200_OK) return rc;
  return Launch(c, fn, rank0, nranks, rows_local, inner, n_red, n_comb, n_gath, all_gather, stream);
}

int cinn_b200_col_reduce_sharded_f32_emulated(cinn_b200_peer_ctx* c, int kind, const float* const* x_per_rank,
                                              long long rows_local, long long inner, float* const* out_per_rank,
                                              int all_gather, void* stream) {
  if (!c) return SetLastError(CINN_B200_EINVAL, "col_reduce_sharded_emulated: bad argument");
  return cinn_b200_col_reduce_sharded_f32_emulated_ranks(c, kind, x_per_rank, rows_local, inner, out_per_rank, all_gather,
                                                         0, c->world, stream);
}

}  // extern "C"
