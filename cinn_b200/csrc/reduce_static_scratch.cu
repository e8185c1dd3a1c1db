// Column reduction whose intermediate partials live in a fixed device array instead of allocated scratch.
//
// The regular path for a reduction with few output columns and many rows (x viewed as [outer, r, inner] with
// outer*inner small) splits r over many CTAs, writes one partial per split into scratch memory and finishes with
// a second launch; that scratch is obtained with cudaMalloc on the group's first run.  Some users of this
// library may not allocate at all: a host framework that owns every byte of device memory and hands kernels
// only the buffers it chose (the reference is embedded into Paddle that way), or a latency-critical loop in
// which a cudaMalloc -- which synchronises the whole device -- must never happen.  For them this file offers one
// entry point that performs the same two-step reduction with the partials in a file-scope __device__ array of
// kStaticScratchFloats floats (4 MiB).  Every GPU on which the library is used holds that array until the
// process exits.
//
// Host code must not pass the array's NAME to a kernel: in host code the name is a host-side shadow, not a
// device address.  The device address is fetched once per device with cudaGetSymbolAddress (with that device
// current) and cached; that happens on the entry point's first call on a device, which therefore should come
// before any stream capture.  All calls share the one array and it keeps whatever the last call left in it; the
// first launch overwrites every partial the second launch reads, so nothing needs clearing, but two calls that
// overlap on the GPU (different streams, or different host threads) race on it.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/cinn_b200.h"
#include "kernel_registry.h"

namespace cinn_b200 {

int SetLastError(int code, const std::string& message);  // runtime.cc

namespace {

constexpr long long kStaticScratchFloats = 1 << 20;  // 4 MiB
static __device__ __align__(256) float g_static_reduce_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mu;

// Device address of the static array on the current device (resolved once per device).
int ScratchAddress(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return SetLastError(CINN_B200_ECUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return SetLastError(CINN_B200_EINVAL, "device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    e        = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_reduce_scratch);
    if (e != cudaSuccess || !p)
      return SetLastError(CINN_B200_ECUDA, std::string("cudaGetSymbolAddress of the static scratch: ") + cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return CINN_B200_OK;
}

const KernelEntry* KernelByCName(const char* name) {
  for (const KernelEntry& k : AllKernels())
    if (!strcmp(k.name, name)) return &k;
  return nullptr;
}

int LaunchColReduce(const KernelEntry* k, const float* x, float* y, long long outer, long long r, long long inner,
                    long long rows_per_split, long long vec_ok, unsigned gx, unsigned gy, unsigned gz, unsigned block,
                    cudaStream_t stream) {
  void* params[7] = {&x, &y, &outer, &r, &inner, &rows_per_split, &vec_ok};
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim  = dim3(gx, gy, gz);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.stream   = stream;
  cudaError_t e = cudaLaunchKernelExC(&cfg, k->fn, params);
  if (e != cudaSuccess) return SetLastError(CINN_B200_ECUDA, std::string("launch of ") + k->name + ": " + cudaGetErrorString(e));
  return CINN_B200_OK;
}

}  // namespace
}  // namespace cinn_b200

using namespace cinn_b200;

extern "C" int cinn_b200_col_reduce_f32_static_scratch(int kind, const float* x, float* y, long long outer,
                                                       long long r, long long inner, void* stream) {
  static const char* const kNames[4] = {"col_reduce_sum_f32", "col_reduce_prod_f32", "col_reduce_max_f32",
                                        "col_reduce_min_f32"};
  if (kind < 0 || kind > 3) return SetLastError(CINN_B200_EINVAL, "kind must be 0 (sum), 1 (prod), 2 (max) or 3 (min)");
  if (!x || !y || outer <= 0 || r <= 0 || inner <= 0) return SetLastError(CINN_B200_EINVAL, "null buffer or non-positive extent");
  const KernelEntry* k = KernelByCName(kNames[kind]);
  if (!k) return SetLastError(CINN_B200_ENOTFOUND, "column-reduction kernel missing from the library");
  // One rule, whatever plan the shape would get: two partials of the output must fit the static array.  Larger
  // outputs are refused even where this device would not split the reduced axis at all, so that the limit does not
  // depend on the SM count or on the split heuristic.
  if (outer > kStaticScratchFloats || inner > kStaticScratchFloats || 2 * outer * inner > kStaticScratchFloats) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "reduction with %lld output elements exceeds the limit of %lld: the static scratch holds %lld floats and "
             "two partials must fit (use the regular group entry point)",
             outer * inner, kStaticScratchFloats / 2, kStaticScratchFloats);
    return SetLastError(CINN_B200_ENOSPACE, msg);
  }
  float* scratch = nullptr;
  int rc         = ScratchAddress(&scratch);
  if (rc != CINN_B200_OK) return rc;

  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sms = v;
  }
  const long long out_elems = outer * inner;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
  const long long vec = (inner % 4 == 0 && aligned) ? 1 : 0;
  const long long cols = inner % 4 == 0 ? inner / 4 : inner;
  // Split r so that about two waves of threads are busy, never more splits than the static array can hold.
  long long splits = 1;
  const long long threads = cols * outer;
  if (threads < (long long)sms * 1024 && r >= 64) {
    splits = (long long)sms * 2048 / (threads > 0 ? threads : 1);
    if (splits > r / 32) splits = r / 32;
    if (splits > 1024) splits = 1024;
    if (splits < 1) splits = 1;
  }
  if (splits * out_elems > kStaticScratchFloats) splits = kStaticScratchFloats / out_elems;  // >= 2, checked above
  long long rows_per_split = (r + splits - 1) / splits;
  splits                   = (r + rows_per_split - 1) / rows_per_split;
  const unsigned block     = cols >= 256 ? 256 : (cols >= 128 ? 128 : 64);
  const unsigned gx        = (unsigned)((cols + block - 1) / block);
  const unsigned gy        = (unsigned)(outer < 65535 ? outer : 65535);
  cudaStream_t s           = static_cast<cudaStream_t>(stream);
  if (splits == 1) return LaunchColReduce(k, x, y, outer, r, inner, rows_per_split, vec, gx, gy, 1, block, s);
  // Step 1: partial[split][outer*inner] into the static array (every element the second step reads is written).
  rc = LaunchColReduce(k, x, scratch, outer, r, inner, rows_per_split, vec, gx, gy, (unsigned)splits, block, s);
  if (rc != CINN_B200_OK) return rc;
  // Step 2: reduce the partials, viewed as [1, splits, outer*inner]; the array is 256-byte aligned.
  const long long vec2   = (out_elems % 4 == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0) ? 1 : 0;
  const long long cols2  = out_elems % 4 == 0 ? out_elems / 4 : out_elems;
  const unsigned block2  = cols2 >= 256 ? 256 : (cols2 >= 128 ? 128 : 64);
  const unsigned gx2     = (unsigned)((cols2 + block2 - 1) / block2);
  return LaunchColReduce(k, scratch, y, 1, splits, out_elems, splits, vec2, gx2, 1, 1, block2, s);
}
