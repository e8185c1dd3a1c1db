// C-ABI launch layer: kernel table, launch primitive, fused-group registry and entry points.
//
// It takes the place of cinn/runtime/cuda/cuda_util.cc:78-118 (cinn_call_cuda_kernel), of the per-group host
// stubs the reference JIT-compiles (cinn/backends/codegen_cuda_host.cc:35-170: unpack the pod array, call the
// launch primitive with the kernel handle and its grid/block) and of the name -> function lookup used to
// build Instructions (cinn/backends/llvm/execution_engine.cc:221-230).
#include <cuda_runtime.h>

#include <algorithm>
#include <array>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <unordered_map>
#include <utility>

#include "../../include/cinn_b200.h"
#include "group_desc.h"

namespace cinn_b200 {

// ---- kernel table ---------------------------------------------------------------------------------
static std::vector<KernelEntry>& Table() {
  static std::vector<KernelEntry> t;
  return t;
}
int RegisterKernel(const char* name, const void* fn, int num_params, int max_threads, bool pdl) {
  Table().push_back(KernelEntry{name, fn, num_params, max_threads, pdl});
  return (int)Table().size() - 1;
}
const KernelEntry* FindKernel(const std::string& name) {
  for (auto& e : Table())
    if (name == e.name) return &e;
  return nullptr;
}
const KernelEntry* FindKernelByFn(const void* fn) {
  for (auto& e : Table())
    if (e.fn == fn) return &e;
  return nullptr;
}
const std::vector<KernelEntry>& AllKernels() { return Table(); }

// ---- chain kernels specialised at build time -----------------------------------------------------------
struct StaticChainRecord {
  StaticChainKey key;
  std::string kernel_name;
};
static std::vector<StaticChainRecord>& StaticChains() {
  static std::vector<StaticChainRecord> t;
  return t;
}
int RegisterStaticChain(const StaticChainKey& key, const char* kernel_name) {
  StaticChains().push_back(StaticChainRecord{key, kernel_name});
  return (int)StaticChains().size();
}
const KernelEntry* FindStaticChain(const char* base, long long meta, int nsteps, const uint32_t* sig) {
  for (auto& r : StaticChains()) {
    if (r.key.meta != meta || r.key.nsteps != nsteps || strcmp(r.key.base, base) != 0) continue;
    bool same = true;
    for (int i = 0; i < nsteps && same; ++i) same = r.key.sig[i] == sig[i];
    if (same) return FindKernel(r.kernel_name);
  }
  return nullptr;
}
int NumStaticChains() { return (int)StaticChains().size(); }

// ---- errors ---------------------------------------------------------------------------------------
static thread_local std::string tls_error;

static int SetError(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  tls_error = buf;
  if (getenv("CINN_B200_VERBOSE")) fprintf(stderr, "[cinn_b200] error %d: %s\n", code, buf);
  return code;
}

int SetLastError(int code, const std::string& message) { return SetError(code, "%s", message.c_str()); }

static void FatalIfRequested() {
  if (getenv("CINN_B200_ABORT_ON_ERROR")) {
    fprintf(stderr, "[cinn_b200] fatal: %s\n", tls_error.c_str());
    abort();
  }
}

static std::atomic<long long> g_launches{0};

// ---- options ----------------------------------------------------------------------------------------
static std::mutex g_mu;
static int g_opt_sm_count = 0;  // 0: query the device, or 148 without one
static int g_opt_rownorm_rows = 0;
static int g_opt_ew_stream = 1, g_opt_ew_stream_stages = 0, g_opt_ew_stream_ctas = 0;
static int g_opt_static_chains = 1;
static int g_opt_fuse_interpreted = 0;
static int g_opt_pdl = 1;  // programmatic dependent launch for the kernels that support it
static int g_opt_peer_reducers_per_sm = 0;  // reducer CTAs per SM of the fused reduce + exchange kernel (0: automatic)
static int g_opt_ew_reg_ctas = 0;
static int g_opt_rowp_form = 0;
static int g_opt_host_chunks = 0;  // upper limit of the chunks group_run_host cuts a group into (0: up to 16)
static int g_opt_rownorm_stages = 0, g_opt_rownorm_ctas = 0, g_opt_enable_tma_rownorm = -1, g_opt_rownorm_simple = -1;

typedef unsigned int (*AsyncTimeoutReader)(int* cuda_status);
static std::vector<AsyncTimeoutReader>& TimeoutReaders() {
  static std::vector<AsyncTimeoutReader> v;
  return v;
}
int RegisterAsyncTimeoutReader(AsyncTimeoutReader reader) {
  TimeoutReaders().push_back(reader);
  return (int)TimeoutReaders().size();
}
static unsigned int ReadAndClearAsyncWaitTimeouts(int* cuda_status) {
  unsigned int total = 0;
  if (cuda_status) *cuda_status = 0;
  for (AsyncTimeoutReader r : TimeoutReaders()) {
    int st = 0;
    total += r(&st);
    if (st != 0 && cuda_status) *cuda_status = st;
  }
  return total;
}

DeviceInfo CurrentDeviceInfo() {
  DeviceInfo d;
  d.rownorm_rows_per_iter = g_opt_rownorm_rows;
  d.enable_ew_stream      = g_opt_ew_stream;
  d.ew_stream_stages      = g_opt_ew_stream_stages;
  d.ew_stream_ctas_per_sm = g_opt_ew_stream_ctas;
  d.ew_reg_ctas_per_sm    = g_opt_ew_reg_ctas;
  d.rowp_form             = g_opt_rowp_form;
  d.rownorm_stages      = g_opt_rownorm_stages;
  d.rownorm_ctas_per_sm = g_opt_rownorm_ctas;
  d.enable_tma_rownorm = g_opt_enable_tma_rownorm;
  d.rownorm_simple     = g_opt_rownorm_simple;
  d.enable_static_chains = g_opt_static_chains;
  d.fuse_interpreted_programs = g_opt_fuse_interpreted;
  if (g_opt_sm_count > 0) {
    d.sm_count = g_opt_sm_count;
    return d;
  }
  int count = 0;
  if (cudaGetDeviceCount(&count) == cudaSuccess && count > 0) {
    int dev = 0, sms = 0, smem = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
      d.sm_count = sms;
    if (cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess && smem > 0)
      d.max_smem_optin = smem;
  } else {
    (void)cudaGetLastError();  // no driver / no device: planning proceeds with the B200 defaults
  }
  return d;
}

// ---- launch primitive -------------------------------------------------------------------------------
constexpr int kMaxKernelParams = 80;  // the row-program kernels take 70
static int LaunchEntry(const KernelEntry* entry, void* v_args, int num_args, int gx, int gy, int gz, int bx, int by,
                       int bz, unsigned cluster_x, size_t dyn_smem, void* stream);

// The public launch primitive: resolves the handle in the kernel table, then launches.
static int LaunchKernel(const void* kernel_fn, void* v_args, int num_args, int gx, int gy, int gz, int bx, int by,
                        int bz, unsigned cluster_x, size_t dyn_smem, void* stream) {
  if (!kernel_fn || (!v_args && num_args > 0) || num_args < 0 || num_args > kMaxKernelParams)
    return SetError(CINN_B200_EINVAL, "cinn_call_cuda_kernel: bad kernel handle or argument array (num_args=%d)",
                    num_args);
  const KernelEntry* entry = FindKernelByFn(kernel_fn);
  if (!entry) return SetError(CINN_B200_ENOTFOUND, "cinn_call_cuda_kernel: %p is not a kernel of this library", kernel_fn);
  return LaunchEntry(entry, v_args, num_args, gx, gy, gz, bx, by, bz, cluster_x, dyn_smem, stream);
}

// Group entry points already hold the table entry and come straight here.
static int LaunchEntry(const KernelEntry* entry, void* v_args, int num_args, int gx, int gy, int gz, int bx, int by,
                       int bz, unsigned cluster_x, size_t dyn_smem, void* stream) {
  const void* kernel_fn = entry->fn;
  if (num_args != entry->num_params)
    return SetError(CINN_B200_EINVAL, "kernel %s takes %d parameters, got %d", entry->name, entry->num_params, num_args);
  if (gx <= 0 || gy <= 0 || gz <= 0 || bx <= 0 || by <= 0 || bz <= 0 ||
      (long long)bx * by * bz > entry->max_threads)
    return SetError(CINN_B200_EINVAL, "kernel %s: bad launch shape grid=(%d,%d,%d) block=(%d,%d,%d), max %d threads",
                    entry->name, gx, gy, gz, bx, by, bz, entry->max_threads);
  // cuda_util.cc:94-104: a buffer passes the address of its `memory` field, anything else its payload address.
  void* params[kMaxKernelParams];
  cinn_pod_value_t* args = static_cast<cinn_pod_value_t*>(v_args);
  for (int i = 0; i < num_args; ++i) {
    if (args[i].type_code_ == CINN_POD_BUFFERP) {
      cinn_buffer_t* b = static_cast<cinn_buffer_t*>(args[i].value_.v_handle);
      if (!b) return SetError(CINN_B200_EINVAL, "kernel %s: argument %d is a null cinn_buffer_t*", entry->name, i);
      params[i] = &b->memory;
    } else {
      params[i] = &args[i].value_;
    }
  }
  if (dyn_smem > 40 * 1024) {  // static + dynamic above 48 KiB needs the opt-in
    cudaError_t e = cudaFuncSetAttribute(kernel_fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn_smem);
    if (e != cudaSuccess)
      return SetError(CINN_B200_ECUDA, "kernel %s: cannot reserve %zu bytes of shared memory: %s", entry->name,
                      dyn_smem, cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim          = dim3(gx, gy, gz);
  cfg.blockDim         = dim3(bx, by, bz);
  cfg.dynamicSmemBytes = dyn_smem;
  cfg.stream           = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  if (cluster_x > 1) {
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = 1;
  } else if (entry->pdl && g_opt_pdl) {
    // Programmatic dependent launch: the kernel may be scheduled while the previous kernel of the stream is still
    // draining; it blocks in grid_dependency_sync() (griddepcontrol.wait) until that kernel has completed and its
    // writes are visible, so the stream's ordering is kept and only the launch latency is hidden.  Short launches
    // (a shard of a group on one of eight GPUs runs 5-15 us) gain 1-2 us each.
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = 1;
  }
  cudaError_t e = cudaLaunchKernelExC(&cfg, kernel_fn, params);
  if (e != cudaSuccess)
    return SetError(CINN_B200_ECUDA, "launch of %s grid=(%d,%d,%d) block=(%d,%d,%d) cluster=%u smem=%zu failed: %s",
                    entry->name, gx, gy, gz, bx, by, bz, cluster_x, dyn_smem, cudaGetErrorString(e));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return CINN_B200_OK;
}

// ---- group registry ---------------------------------------------------------------------------------
constexpr int kMaxGroups = 1024;

constexpr int kHostStreams = 3;

struct HostStaging {
  void* dev        = nullptr;
  size_t bytes     = 0;
  cudaStream_t s[kHostStreams] = {nullptr, nullptr, nullptr};
  cudaEvent_t replicated_ready = nullptr;
};

struct GroupSlot {
  std::unique_ptr<CompiledGroup> plan;
  GroupDesc desc;                                // what the plan was compiled from
  // run_host pipelines copies and kernels over chunks of the outer axis when the group allows it.
  bool chunk_tried = false;
  int chunk_count  = 0;                          // 0: not chunkable
  std::vector<bool> chunk_sharded;               // per argument (inputs then outputs): sliced on axis 0
  std::unique_ptr<CompiledGroup> chunk_plan;     // the group compiled for one chunk
  std::unordered_map<int, void*> scratch;        // device ordinal -> scratch buffer
  std::unordered_map<int, HostStaging> staging;  // device ordinal -> staging for run_host
  std::mutex mu;                                 // guards scratch / staging / chunk_* of this group
  ~GroupSlot();
};

// A slot holds its group through a shared_ptr: a run takes its own reference under g_mu, so compiling the same
// name again or releasing the group while another thread is inside a run cannot free the plan under it; the
// group's device memory is freed when the last reference goes.
static std::shared_ptr<GroupSlot> g_slots[kMaxGroups];
static std::unordered_map<std::string, int> g_slot_of_name;

static std::shared_ptr<GroupSlot> SlotRef(int index) {
  if (index < 0 || index >= kMaxGroups) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  return g_slots[index];
}

static int RunSlot(int slot, void* pod_args, int num_args, void* stream);

template <int I>
static void Trampoline(void* args, int32_t num_args, void* stream) {
  if (RunSlot(I, args, num_args, stream) != CINN_B200_OK) FatalIfRequested();
}

template <int... Is>
static constexpr std::array<lower_func_ptr_g, sizeof...(Is)> MakeTrampolines(std::integer_sequence<int, Is...>) {
  return {{&Trampoline<Is>...}};
}
static const std::array<lower_func_ptr_g, kMaxGroups> g_trampolines =
    MakeTrampolines(std::make_integer_sequence<int, kMaxGroups>());

static bool IsAligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int TypeMatches(const cinn_buffer_t* b, DType t) {
  const int code = (int)b->type.code, bits = b->type.bits;
  switch (t) {
    case DType::kFloat32: return code == cinn_type_float && bits == 32;
    case DType::kFloat16: return code == cinn_type_float && bits == 16;
    case DType::kBFloat16: return code == cinn_type_bfloat && bits == 16;
    case DType::kFloat64: return code == cinn_type_float && bits == 64;
    case DType::kInt32: return code == cinn_type_int && bits == 32;
    case DType::kInt64: return code == cinn_type_int && bits == 64;
    case DType::kBool: return code == cinn_type_int && bits == 1;
    case DType::kUInt8: return code == cinn_type_uint && bits == 8;
    default: return 0;
  }
}

// Checks the pod array against the compiled group and returns the buffers (inputs then outputs).
static int CheckArgs(const CompiledGroup& plan, void* pod_args, int num_args, std::vector<cinn_buffer_t*>* bufs) {
  const int n_in = (int)plan.inputs.size(), n_out = (int)plan.outputs.size();
  if (!pod_args) return SetError(CINN_B200_EINVAL, "group %s: null argument array", plan.name.c_str());
  if (num_args != n_in + n_out)
    return SetError(CINN_B200_EINVAL, "group %s takes %d inputs + %d outputs, got %d arguments", plan.name.c_str(),
                    n_in, n_out, num_args);
  cinn_pod_value_t* args = static_cast<cinn_pod_value_t*>(pod_args);
  bufs->resize(num_args);
  for (int i = 0; i < num_args; ++i) {
    const TensorDesc& t = i < n_in ? plan.inputs[i] : plan.outputs[i - n_in];
    if (args[i].type_code_ != CINN_POD_BUFFERP)
      return SetError(CINN_B200_EINVAL, "group %s: argument %d (%s) has type code %d, expected a cinn_buffer_t* (7)",
                      plan.name.c_str(), i, t.name.c_str(), args[i].type_code_);
    cinn_buffer_t* b = static_cast<cinn_buffer_t*>(args[i].value_.v_handle);
    if (!b || !b->memory)
      return SetError(CINN_B200_EINVAL, "group %s: argument %d (%s) has no memory", plan.name.c_str(), i,
                      t.name.c_str());
    if (!TypeMatches(b, t.dtype))
      return SetError(CINN_B200_ESHAPE, "group %s: argument %d (%s) has type code %d/%d bits, compiled for %s",
                      plan.name.c_str(), i, t.name.c_str(), (int)b->type.code, (int)b->type.bits, DTypeName(t.dtype));
    if (b->dimensions < 0 || b->dimensions > CINN_BUFFER_MAX_DIMS)
      return SetError(CINN_B200_ESHAPE, "group %s: argument %d (%s) has %d dimensions", plan.name.c_str(), i,
                      t.name.c_str(), b->dimensions);
    long long numel = 1;
    for (int d = 0; d < b->dimensions; ++d) numel *= b->dims[d];
    if (numel != t.numel())
      return SetError(CINN_B200_ESHAPE, "group %s: argument %d (%s) has %lld elements, compiled for %lld",
                      plan.name.c_str(), i, t.name.c_str(), numel, (long long)t.numel());
    (*bufs)[i] = b;
  }
  return CINN_B200_OK;
}

static int RunPlan(const CompiledGroup& plan, GroupSlot& slot, const std::vector<cinn_buffer_t*>& bufs, void* stream) {
  const int n_in            = (int)plan.inputs.size();
  // Device scratch (split reductions only), one buffer per device, allocated on first use.
  uint8_t* scratch = nullptr;
  if (plan.scratch_bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return SetError(CINN_B200_ECUDA, "cudaGetDevice failed");
    std::lock_guard<std::mutex> lk(slot.mu);
    auto it = slot.scratch.find(dev);
    if (it == slot.scratch.end()) {
      // First run on this device.  The buffer is zeroed (kernels that keep ticket counters in it return them to
      // zero themselves) and the zeroing is COMPLETE before this call goes on, so that a later run on any other
      // stream is ordered after it as well.  That needs a synchronisation, hence no stream capture here.
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
        return SetError(CINN_B200_EINVAL,
                        "group %s needs scratch memory: run it once outside stream capture before capturing it",
                        plan.name.c_str());
      void* p       = nullptr;
      cudaError_t e = cudaMalloc(&p, plan.scratch_bytes);
      if (e != cudaSuccess)
        return SetError(CINN_B200_ECUDA, "group %s: cudaMalloc of %zu scratch bytes failed: %s", plan.name.c_str(),
                        plan.scratch_bytes, cudaGetErrorString(e));
      e = cudaMemsetAsync(p, 0, plan.scratch_bytes, static_cast<cudaStream_t>(stream));
      if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) {
        cudaFree(p);
        return SetError(CINN_B200_ECUDA, "group %s: zeroing the scratch buffer failed: %s", plan.name.c_str(),
                        cudaGetErrorString(e));
      }
      it = slot.scratch.emplace(dev, p).first;
    }
    scratch = static_cast<uint8_t*>(it->second);
  }
  const std::vector<LaunchStep>* steps = &plan.steps;
  if (!plan.steps_unaligned.empty()) {
    bool ok = true;
    for (int i : plan.aligned_inputs) ok = ok && IsAligned16(bufs[i]->memory);
    for (int i : plan.aligned_outputs) ok = ok && IsAligned16(bufs[n_in + i]->memory);
    if (!ok) steps = &plan.steps_unaligned;
  }
  for (const LaunchStep& s : *steps) {
    cinn_pod_value_t pods[kMaxKernelParams];
    cinn_buffer_t scratch_bufs[8];
    int n_scratch = 0;
    const int n   = (int)s.args.size();
    for (int i = 0; i < n; ++i) {
      const ArgSpec& a = s.args[i];
      switch (a.kind) {
        case ArgSpec::kInput:
          pods[i].type_code_      = CINN_POD_BUFFERP;
          pods[i].value_.v_handle = bufs[a.index];
          break;
        case ArgSpec::kOutput:
          pods[i].type_code_      = CINN_POD_BUFFERP;
          pods[i].value_.v_handle = bufs[n_in + a.index];
          break;
        case ArgSpec::kScratch: {
          if (n_scratch >= 8) return SetError(CINN_B200_EINVAL, "too many scratch arguments");
          cinn_buffer_t* sb = &scratch_bufs[n_scratch++];
          memset(sb, 0, sizeof(*sb));
          sb->memory              = scratch + a.ivalue;
          pods[i].type_code_      = CINN_POD_BUFFERP;
          pods[i].value_.v_handle = sb;
          break;
        }
        case ArgSpec::kInt:
          pods[i].type_code_     = CINN_POD_INT64;
          pods[i].value_.v_int64 = a.ivalue;
          break;
        case ArgSpec::kFloat:
          pods[i].type_code_       = CINN_POD_DOUBLE;
          pods[i].value_.v_float64 = a.fvalue;
          break;
        case ArgSpec::kAligned: {
          bool ok = a.ivalue != 0;
          for (int k : a.aligned_inputs) ok = ok && IsAligned16(bufs[k]->memory);
          for (int k : a.aligned_outputs) ok = ok && IsAligned16(bufs[n_in + k]->memory);
          pods[i].type_code_     = CINN_POD_INT64;
          pods[i].value_.v_int64 = ok ? 1 : 0;
          break;
        }
      }
    }
    int rc = LaunchEntry(s.kernel, pods, n, s.grid[0], s.grid[1], s.grid[2], s.block[0], s.block[1], s.block[2],
                         s.cluster, s.dyn_smem, stream);
    if (rc != CINN_B200_OK) return rc;
  }
  return CINN_B200_OK;
}

static int RunSlot(int slot_index, void* pod_args, int num_args, void* stream) {
  std::shared_ptr<GroupSlot> slot = SlotRef(slot_index);
  if (!slot || !slot->plan) return SetError(CINN_B200_ENOTFOUND, "entry point %d is not bound to a compiled group", slot_index);
  std::vector<cinn_buffer_t*> bufs;
  int rc = CheckArgs(*slot->plan, pod_args, num_args, &bufs);
  if (rc != CINN_B200_OK) return rc;
  return RunPlan(*slot->plan, *slot, bufs, stream);
}

static int SlotOf(const char* fn_name) {
  if (!fn_name) return -1;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_slot_of_name.find(fn_name);
  return it == g_slot_of_name.end() ? -1 : it->second;
}

GroupSlot::~GroupSlot() {
  for (auto& kv : scratch) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(kv.first);
    cudaFree(kv.second);
    cudaSetDevice(prev);
  }
  for (auto& kv : staging) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(kv.first);
    if (kv.second.dev) cudaFree(kv.second.dev);
    for (int k = 0; k < kHostStreams; ++k)
      if (kv.second.s[k]) cudaStreamDestroy(kv.second.s[k]);
    if (kv.second.replicated_ready) cudaEventDestroy(kv.second.replicated_ready);
    cudaSetDevice(prev);
  }
}

static std::shared_ptr<GroupSlot> SlotByName(const char* fn_name) { return SlotRef(SlotOf(fn_name)); }

}  // namespace cinn_b200

using namespace cinn_b200;

extern "C" {

const char* cinn_b200_last_error(void) { return tls_error.c_str(); }

void cinn_call_cuda_kernel(void* kernel_fn, void* v_args, int num_args, int grid_x, int grid_y, int grid_z,
                           int block_x, int block_y, int block_z, void* stream) {
  if (LaunchKernel(kernel_fn, v_args, num_args, grid_x, grid_y, grid_z, block_x, block_y, block_z, 0, 0, stream) !=
      CINN_B200_OK)
    FatalIfRequested();
}

int cinn_b200_call_cuda_kernel_ex(void* kernel_fn, void* v_args, int num_args, int grid_x, int grid_y, int grid_z,
                                  int block_x, int block_y, int block_z, unsigned cluster_x, size_t dyn_smem,
                                  void* stream) {
  return LaunchKernel(kernel_fn, v_args, num_args, grid_x, grid_y, grid_z, block_x, block_y, block_z, cluster_x,
                      dyn_smem, stream);
}

void* cinn_b200_get_kernel(const char* kernel_name) {
  const KernelEntry* e = kernel_name ? FindKernel(kernel_name) : nullptr;
  if (!e) {
    SetError(CINN_B200_ENOTFOUND, "no kernel named '%s'", kernel_name ? kernel_name : "(null)");
    return nullptr;
  }
  return const_cast<void*>(e->fn);
}

int cinn_b200_num_kernels(void) { return (int)AllKernels().size(); }

const char* cinn_b200_kernel_name(int index) {
  if (index < 0 || index >= (int)AllKernels().size()) return nullptr;
  return AllKernels()[index].name;
}

int cinn_b200_kernel_num_params(const char* kernel_name) {
  const KernelEntry* e = kernel_name ? FindKernel(kernel_name) : nullptr;
  if (!e) return SetError(CINN_B200_ENOTFOUND, "no kernel named '%s'", kernel_name ? kernel_name : "(null)");
  return e->num_params;
}

long long cinn_b200_launch_count(void) { return g_launches.load(); }

int cinn_b200_compile_group(const char* group_desc, lower_func_ptr_g* fn_out) {
  if (!group_desc) return SetError(CINN_B200_EINVAL, "null group description");
  GroupDesc g;
  std::string err;
  if (!ParseGroupDesc(group_desc, &g, &err)) return SetError(CINN_B200_EINVAL, "%s", err.c_str());
  DeviceInfo dev = CurrentDeviceInfo();
  auto plan      = CompileGroup(g, dev, &err);
  if (!plan) return SetError(CINN_B200_ENOMATCH, "%s", err.c_str());
  auto fresh   = std::make_shared<GroupSlot>();
  fresh->plan  = std::move(plan);
  fresh->desc  = g;
  std::shared_ptr<GroupSlot> old;  // dropped after the lock is released (its destructor frees device memory)
  {
    std::lock_guard<std::mutex> lk(g_mu);
    int slot = -1;
    auto it  = g_slot_of_name.find(g.name);
    if (it != g_slot_of_name.end()) {
      slot = it->second;
    } else {
      for (int i = 0; i < kMaxGroups; ++i)
        if (!g_slots[i]) {
          slot = i;
          break;
        }
      if (slot < 0) return SetError(CINN_B200_ENOSPACE, "all %d entry points are in use; release some groups", kMaxGroups);
      g_slot_of_name[g.name] = slot;
    }
    old           = std::move(g_slots[slot]);
    g_slots[slot] = std::move(fresh);
    if (fn_out) *fn_out = g_trampolines[slot];
  }
  return CINN_B200_OK;
}

lower_func_ptr_g cinn_b200_lookup(const char* fn_name) {
  int slot = SlotOf(fn_name);
  if (slot < 0) {
    SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
    return nullptr;
  }
  return g_trampolines[slot];
}

int cinn_b200_release_group(const char* fn_name) {
  if (!fn_name) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '(null)'");
  std::shared_ptr<GroupSlot> old;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_slot_of_name.find(fn_name);
    if (it == g_slot_of_name.end()) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name);
    old = std::move(g_slots[it->second]);
    g_slots[it->second].reset();
    g_slot_of_name.erase(it);
  }
  return CINN_B200_OK;  // `old` goes here, or when the last run that still holds it returns
}

int cinn_b200_group_run(const char* fn_name, void* pod_args, int num_args, void* stream) {
  int slot = SlotOf(fn_name);
  if (slot < 0) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
  return RunSlot(slot, pod_args, num_args, stream);
}

static int CopyOut(const std::string& s, char* out, size_t len) {
  if (!out || len == 0) return CINN_B200_OK;
  if (s.size() + 1 > len) return SetError(CINN_B200_ENOSPACE, "caller buffer of %zu bytes is too small for %zu", len, s.size() + 1);
  memcpy(out, s.c_str(), s.size() + 1);
  return CINN_B200_OK;
}

int cinn_b200_group_info(const char* fn_name, char* pattern, size_t pattern_len, long long* algorithmic_bytes,
                         long long* elements, int* launches, long long* scratch_bytes) {
  std::shared_ptr<GroupSlot> ref = SlotByName(fn_name);
  if (!ref) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
  const CompiledGroup& p = *ref->plan;
  if (algorithmic_bytes) *algorithmic_bytes = p.algorithmic_bytes;
  if (elements) *elements = p.elements;
  if (launches) *launches = (int)p.steps.size();
  if (scratch_bytes) *scratch_bytes = (long long)p.scratch_bytes;
  return CopyOut(p.pattern, pattern, pattern_len);
}

int cinn_b200_group_kernel(const char* fn_name, int step, char* name, size_t name_len) {
  std::shared_ptr<GroupSlot> ref = SlotByName(fn_name);
  if (!ref) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
  const CompiledGroup& p = *ref->plan;
  if (step < 0 || step >= (int)p.steps.size()) return SetError(CINN_B200_EINVAL, "group %s has %zu launch steps", fn_name, p.steps.size());
  return CopyOut(p.steps[step].kernel->name, name, name_len);
}

long long cinn_b200_group_launch_text(const char* fn_name, char* out, size_t out_len) {
  std::shared_ptr<GroupSlot> ref = SlotByName(fn_name);
  if (!ref) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
  std::string text;
  char buf[256];
  int index = 0;
  for (const LaunchStep& s : ref->plan->steps) {
    snprintf(buf, sizeof(buf), "launch %d %s grid=%u,%u,%u block=%u,%u,%u cluster=%u smem=%zu\n", index++, s.kernel->name,
             s.grid[0], s.grid[1], s.grid[2], s.block[0], s.block[1], s.block[2], s.cluster, s.dyn_smem);
    text += buf;
    int k = 0;
    for (const ArgSpec& a : s.args) {
      switch (a.kind) {
        case ArgSpec::kInput: snprintf(buf, sizeof(buf), "arg %d input %d\n", k, a.index); break;
        case ArgSpec::kOutput: snprintf(buf, sizeof(buf), "arg %d output %d\n", k, a.index); break;
        case ArgSpec::kScratch: snprintf(buf, sizeof(buf), "arg %d scratch %lld\n", k, (long long)a.ivalue); break;
        case ArgSpec::kInt: snprintf(buf, sizeof(buf), "arg %d int %lld\n", k, (long long)a.ivalue); break;
        case ArgSpec::kFloat: snprintf(buf, sizeof(buf), "arg %d float %.17g\n", k, a.fvalue); break;
        default: snprintf(buf, sizeof(buf), "arg %d aligned %lld\n", k, (long long)a.ivalue); break;
      }
      text += buf;
      ++k;
    }
  }
  if (out && out_len > 0) {
    const size_t n = std::min(text.size(), out_len - 1);
    memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return (long long)text.size() + 1;
}

int cinn_b200_num_static_chains(void) { return NumStaticChains(); }

int cinn_b200_canonical_expr(const char* group_desc, char* out, size_t out_len) {
  if (!group_desc) return SetError(CINN_B200_EINVAL, "null group description");
  GroupDesc g;
  std::string err;
  if (!ParseGroupDesc(group_desc, &g, &err)) return SetError(CINN_B200_EINVAL, "%s", err.c_str());
  std::string e = CanonicalExpr(g, &err);
  if (e.empty()) return SetError(CINN_B200_EINVAL, "%s", err.c_str());
  return CopyOut(e, out, out_len);
}

// Decides once per group whether run_host may pipeline over chunks of the outer axis, and compiles the group for
// one chunk.  A group qualifies when its output and at least one input carry the outer extent D0 as their first
// dimension, no operand is indexed by that axis other than through its own first dimension, no reduction runs over
// it, and the chunk-sized group compiles to the same kernel family without scratch memory.
static void PrepareChunking(GroupSlot& slot) {
  slot.chunk_tried = true;
  const GroupDesc& g = slot.desc;
  const CompiledGroup& plan = *slot.plan;
  if (plan.scratch_bytes != 0 || g.outputs.size() != 1 || g.outputs[0].shape.empty()) return;
  const int64_t d0 = g.outputs[0].shape[0];
  if (d0 < 2) return;
  const size_t out_rank = g.outputs[0].shape.size();
  size_t max_rank       = out_rank;
  for (auto& t : g.inputs) max_rank = std::max(max_rank, t.shape.size());
  std::vector<bool> sharded;
  bool any = false;
  std::map<std::string, bool> sharded_input;
  for (auto& t : g.inputs) {
    bool sh = !t.shape.empty() && t.shape[0] == d0 && t.shape.size() == max_rank;
    sharded.push_back(sh);
    sharded_input[t.name] = sh;
    any = any || sh;
  }
  sharded.push_back(true);
  if (!any) return;
  auto attr = [](const OpDesc& op, const char* k) {
    auto it = op.attrs.find(k);
    return it == op.attrs.end() ? std::string() : it->second;
  };
  auto first_int = [](const std::string& text) { return text.empty() ? (int64_t)-1 : (int64_t)atoll(text.c_str()); };
  for (auto& op : g.ops) {
    if (op.type.rfind("reduce_", 0) == 0) {
      std::string dims = "," + attr(op, "dim") + ",";
      if (dims == ",," || dims.find(",0,") != std::string::npos) return;  // reduces the outer axis
    }
    for (auto& in : op.inputs) {
      auto it = sharded_input.find(in);
      if (it == sharded_input.end() || it->second) continue;
      // a replicated input: it must not be aligned to axis 0
      if (attr(op, "axis") == "0") return;
      if (op.type == "broadcast_to") {
        std::string axes = "," + attr(op, "broadcast_axes") + ",";
        if (axes.find(",0,") != std::string::npos) return;
      }
    }
  }
  size_t total = 0;
  for (auto& t : g.inputs) total += (size_t)t.numel() * DTypeBytes(t.dtype);
  total += (size_t)g.outputs[0].numel() * DTypeBytes(g.outputs[0].dtype);
  int chunks = 0;
  const int most = g_opt_host_chunks > 0 ? g_opt_host_chunks : 16;
  for (int c : {16, 8, 4, 2})
    if (c <= most && d0 % c == 0 && total / c >= (4u << 20)) {
      chunks = c;
      break;
    }
  if (!chunks) return;
  const int64_t part = d0 / chunks;
  GroupDesc sub      = g;
  sub.name           = g.name + "__chunk";
  for (size_t i = 0; i < sub.inputs.size(); ++i)
    if (sharded[i]) sub.inputs[i].shape[0] = part;
  sub.outputs[0].shape[0] = part;
  for (auto& op : sub.ops) {
    for (const char* key : {"shape", "out_shape"}) {
      auto it = op.attrs.find(key);
      if (it != op.attrs.end() && first_int(it->second) == d0) {
        auto comma = it->second.find(',');
        it->second = std::to_string(part) + (comma == std::string::npos ? "" : it->second.substr(comma));
      }
    }
  }
  std::string err;
  auto sub_plan = CompileGroup(sub, CurrentDeviceInfo(), &err);
  if (!sub_plan || sub_plan->pattern != plan.pattern || sub_plan->scratch_bytes != 0) return;
  slot.chunk_plan    = std::move(sub_plan);
  slot.chunk_sharded = sharded;
  slot.chunk_count   = chunks;
}

int cinn_b200_group_run_host(const char* fn_name, void* pod_args, int num_args, int device) {
  std::shared_ptr<GroupSlot> ref = SlotByName(fn_name);
  if (!ref) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
  GroupSlot& slot           = *ref;
  const CompiledGroup& plan = *slot.plan;
  std::vector<cinn_buffer_t*> host;
  int rc = CheckArgs(plan, pod_args, num_args, &host);
  if (rc != CINN_B200_OK) return rc;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
  // One staging allocation per (group, device): [inputs..., outputs...] each 256-byte aligned.
  const int n_in = (int)plan.inputs.size();
  std::vector<size_t> offs(num_args), sizes(num_args);
  size_t total = 0;
  for (int i = 0; i < num_args; ++i) {
    const TensorDesc& t = i < n_in ? plan.inputs[i] : plan.outputs[i - n_in];
    sizes[i]            = (size_t)t.numel() * DTypeBytes(t.dtype);
    offs[i]             = total;
    total += (sizes[i] + 255) / 256 * 256;
  }
  HostStaging* st = nullptr;
  {
    std::lock_guard<std::mutex> lk(slot.mu);
    st = &slot.staging[device];
    if (!slot.chunk_tried) PrepareChunking(slot);
  }
  if (st->bytes < total) {
    if (st->dev) cudaFree(st->dev);
    st->dev = nullptr;
    e       = cudaMalloc(&st->dev, total);
    if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "cudaMalloc of %zu staging bytes: %s", total, cudaGetErrorString(e));
    st->bytes = total;
  }
  for (int k = 0; k < kHostStreams; ++k) {
    if (st->s[k]) continue;
    e = cudaStreamCreateWithFlags(&st->s[k], cudaStreamNonBlocking);
    if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "cudaStreamCreate: %s", cudaGetErrorString(e));
  }
  if (!st->replicated_ready) {
    e = cudaEventCreateWithFlags(&st->replicated_ready, cudaEventDisableTiming);
    if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "cudaEventCreate: %s", cudaGetErrorString(e));
  }
  uint8_t* base = static_cast<uint8_t*>(st->dev);
  auto fail_copy = [&](const char* what, const std::string& name, cudaError_t err) {
    return SetError(CINN_B200_ECUDA, "%s copy of %s: %s", what, name.c_str(), cudaGetErrorString(err));
  };
  const int chunks = slot.chunk_count > 0 ? slot.chunk_count : 1;
  // Replicated (small) inputs go first on stream 0; the other streams wait for them.
  for (int i = 0; i < n_in; ++i) {
    if (chunks > 1 && slot.chunk_sharded[i]) continue;
    e = cudaMemcpyAsync(base + offs[i], host[i]->memory, sizes[i], cudaMemcpyHostToDevice, st->s[0]);
    if (e != cudaSuccess) return fail_copy("host->device", plan.inputs[i].name, e);
  }
  if (chunks == 1) {
    std::vector<cinn_buffer_t> dev_bufs(num_args);
    std::vector<cinn_buffer_t*> ptrs(num_args);
    for (int i = 0; i < num_args; ++i) {
      dev_bufs[i]        = *host[i];
      dev_bufs[i].memory = base + offs[i];
      ptrs[i]            = &dev_bufs[i];
    }
    rc = RunPlan(plan, slot, ptrs, st->s[0]);
    if (rc != CINN_B200_OK) return rc;
    for (int i = n_in; i < num_args; ++i) {
      e = cudaMemcpyAsync(host[i]->memory, base + offs[i], sizes[i], cudaMemcpyDeviceToHost, st->s[0]);
      if (e != cudaSuccess) return fail_copy("device->host", plan.outputs[i - n_in].name, e);
    }
    e = cudaStreamSynchronize(st->s[0]);
    if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "group %s: %s", plan.name.c_str(), cudaGetErrorString(e));
    return CINN_B200_OK;
  }
  // Pipelined: chunk c uses stream c % 3: copy its slices in, run the chunk-sized group, copy its slice out.  With
  // three streams the host->device copy of one chunk, the kernel of another and the device->host copy of a third
  // overlap (the two copy directions use different DMA engines).
  e = cudaEventRecord(st->replicated_ready, st->s[0]);
  if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "cudaEventRecord: %s", cudaGetErrorString(e));
  for (int k = 1; k < kHostStreams; ++k) cudaStreamWaitEvent(st->s[k], st->replicated_ready, 0);
  const CompiledGroup& sub = *slot.chunk_plan;
  std::vector<cinn_buffer_t> dev_bufs(num_args);
  std::vector<cinn_buffer_t*> ptrs(num_args);
  for (int c = 0; c < chunks; ++c) {
    cudaStream_t stream = st->s[c % kHostStreams];
    for (int i = 0; i < num_args; ++i) {
      const bool sh       = slot.chunk_sharded[i];
      const size_t part   = sh ? sizes[i] / chunks : sizes[i];
      const size_t off    = sh ? part * c : 0;
      dev_bufs[i]         = *host[i];
      dev_bufs[i].memory  = base + offs[i] + off;
      if (sh) dev_bufs[i].dims[0] = host[i]->dims[0] / chunks;
      ptrs[i]             = &dev_bufs[i];
      if (i < n_in && sh) {
        e = cudaMemcpyAsync(dev_bufs[i].memory, host[i]->memory + off, part, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return fail_copy("host->device", plan.inputs[i].name, e);
      }
    }
    rc = RunPlan(sub, slot, ptrs, stream);
    if (rc != CINN_B200_OK) return rc;
    const int o        = n_in;
    const size_t part  = sizes[o] / chunks;
    e = cudaMemcpyAsync(host[o]->memory + part * c, base + offs[o] + part * c, part, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail_copy("device->host", plan.outputs[0].name, e);
  }
  for (int k = 0; k < kHostStreams; ++k) {
    e = cudaStreamSynchronize(st->s[k]);
    if (e != cudaSuccess) return SetError(CINN_B200_ECUDA, "group %s: %s", plan.name.c_str(), cudaGetErrorString(e));
  }
  return CINN_B200_OK;
}

int cinn_b200_group_host_chunks(const char* fn_name) {
  std::shared_ptr<GroupSlot> ref = SlotByName(fn_name);
  if (!ref) return SetError(CINN_B200_ENOTFOUND, "no compiled group named '%s'", fn_name ? fn_name : "(null)");
  GroupSlot& slot = *ref;
  std::lock_guard<std::mutex> lk(slot.mu);
  if (!slot.chunk_tried) PrepareChunking(slot);
  return slot.chunk_count > 0 ? slot.chunk_count : 1;
}

int cinn_b200_device_status(unsigned int* async_wait_timeouts) {
  int st         = 0;
  unsigned int v = ReadAndClearAsyncWaitTimeouts(&st);
  if (st != 0) return SetError(CINN_B200_ECUDA, "reading the device status word: %s", cudaGetErrorString((cudaError_t)st));
  if (async_wait_timeouts) *async_wait_timeouts = v;
  return CINN_B200_OK;
}

}  // extern "C"
namespace cinn_b200 {
int OptPeerReducersPerSm() { return g_opt_peer_reducers_per_sm; }
}  // namespace cinn_b200
extern "C" {

int cinn_b200_set_option(const char* key, long long value) {
  if (!key) return SetError(CINN_B200_EINVAL, "null option key");
  if (!strcmp(key, "sm_count")) {
    g_opt_sm_count = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "peer_reducers_per_sm")) {
    g_opt_peer_reducers_per_sm = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "host_chunks")) {
    g_opt_host_chunks = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "enable_pdl")) {
    g_opt_pdl = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "fuse_interpreted_programs")) {
    g_opt_fuse_interpreted = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "enable_static_chains")) {
    g_opt_static_chains = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "enable_ew_stream")) {
    g_opt_ew_stream = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "ew_stream_stages")) {
    g_opt_ew_stream_stages = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "rowp_form")) {
    g_opt_rowp_form = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "ew_reg_ctas_per_sm")) {
    g_opt_ew_reg_ctas = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "ew_stream_ctas_per_sm")) {
    g_opt_ew_stream_ctas = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "rownorm_rows_per_iter")) {
    g_opt_rownorm_rows = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "rownorm_stages")) {
    g_opt_rownorm_stages = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "rownorm_ctas_per_sm")) {
    g_opt_rownorm_ctas = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "rownorm_simple")) {
    g_opt_rownorm_simple = (int)value;
    return CINN_B200_OK;
  }
  if (!strcmp(key, "enable_tma_rownorm")) {
    g_opt_enable_tma_rownorm = (int)value;
    return CINN_B200_OK;
  }
  return SetError(CINN_B200_ENOTFOUND, "unknown option '%s'", key);
}

}  // extern "C"
