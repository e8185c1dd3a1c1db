// Static table of the prebuilt sm_100a kernels.
//
// This replaces the reference's per-card CUmodule cache and the run-time symbol table that its JIT
// fills with "<fn>_kernel_ptr_" globals (cinn/runtime/cuda/cuda_module.cc:35-147,
// cinn/backends/compiler.cc:133-140): kernels are compiled offline into the library, and a kernel
// handle is the address of its host-side launch stub, valid on every device of the process.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace cinn_b200 {

struct KernelEntry {
  const char* name;   // unique, e.g. "row_reduce_warp_sum_f32"
  const void* fn;     // host stub address, what cinn_call_cuda_kernel receives as kernel_fn
  int num_params;     // number of kernel parameters (pointers first, then scalars)
  int max_threads;    // __launch_bounds__ of the kernel
  bool pdl;           // the kernel calls grid_dependency_sync() before it touches global memory, so it may be
                      // launched with programmatic stream serialisation (see LaunchEntry in runtime.cc)
};

// Adds an entry at static-initialisation time; returns its index.
int RegisterKernel(const char* name, const void* fn, int num_params, int max_threads, bool pdl = false);
const KernelEntry* FindKernel(const std::string& name);
const KernelEntry* FindKernelByFn(const void* fn);
const std::vector<KernelEntry>& AllKernels();

struct KernelRegistrar {
  KernelRegistrar(const char* name, const void* fn, int num_params, int max_threads, bool pdl = false) {
    RegisterKernel(name, fn, num_params, max_threads, pdl);
  }
};

// Chain kernels specialised at build time (ew_static.cu): each is registered under the interpreted kernel it
// replaces (`base`, e.g. "ew_chain_f32_s1"), the `meta` word (operand types and addressing modes) and the low
// halves of the program's step words (op, operand selectors, role).  The matcher compiles a group to the interpreted
// kernel's plan as always and then swaps in the specialised kernel when one with the same key exists: the two take
// the same parameters, immediates included.
struct StaticChainKey {
  const char* base;
  long long meta;
  int nsteps;
  uint32_t sig[40];
};
int RegisterStaticChain(const StaticChainKey& key, const char* kernel_name);
const KernelEntry* FindStaticChain(const char* base, long long meta, int nsteps, const uint32_t* sig);
int NumStaticChains();

#define CINN_B200_CAT_(a, b) a##b
#define CINN_B200_CAT(a, b) CINN_B200_CAT_(a, b)
// `fn` may contain commas (template arguments), hence the variadic tail.
#define CINN_B200_REGISTER_KERNEL(name, num_params, max_threads, ...)                                  \
  static ::cinn_b200::KernelRegistrar CINN_B200_CAT(cinn_b200_kernel_registrar_, __COUNTER__)(        \
      name, reinterpret_cast<const void*>(&__VA_ARGS__), num_params, max_threads)

// The same for a kernel whose first statement is grid_dependency_sync().
#define CINN_B200_REGISTER_KERNEL_PDL(name, num_params, max_threads, ...)                              \
  static ::cinn_b200::KernelRegistrar CINN_B200_CAT(cinn_b200_kernel_registrar_, __COUNTER__)(        \
      name, reinterpret_cast<const void*>(&__VA_ARGS__), num_params, max_threads, true)

}  // namespace cinn_b200
