// Frontend-independent description of one fused op group and of the kernel launches it compiles to.
//
// A GroupDesc carries what the reference's Graph::Group holds for lowering (cinn/hlir/framework/graph.h:58-129):
// the nodes in producer->consumer order with their attributes, and the ordered input / output tensors that
// become the entry point's arguments (inputs first, then outputs: cinn/hlir/framework/instruction.cc:81-105).
// CompileGroup() is the replacement of OpLowerer::Lower + CodeGenCUDA_Dev + NVRTC for such a group
// (cinn/hlir/framework/parallel_compiler.cc:123-199): it pattern-matches the group's expression against the
// prebuilt sm_100a kernels and returns a launch plan.  A group that matches nothing is an error: there is no
// runtime code generation and no CPU fallback.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "kernel_registry.h"

namespace cinn_b200 {

enum class DType { kFloat32, kFloat16, kBFloat16, kFloat64, kInt32, kInt64, kBool, kUInt8, kUnknown };

const char* DTypeName(DType t);
DType DTypeFromName(const std::string& s);
int DTypeBytes(DType t);

struct TensorDesc {
  std::string name;
  DType dtype = DType::kFloat32;
  std::vector<int64_t> shape;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

struct OpDesc {
  std::string type;                          // HLIR op name: elementwise_add, relu, scale, reduce_sum, ...
  std::vector<std::string> inputs;           // value names
  std::string output;                        // value name
  std::map<std::string, std::string> attrs;  // attribute name -> text (lists as "1,2,3")
};

struct GroupDesc {
  std::string name;                 // the name the entry point is looked up by, "fn_..." (graph.h:128)
  std::vector<TensorDesc> inputs;   // argument order
  std::vector<TensorDesc> outputs;  // argument order after the inputs
  std::vector<OpDesc> ops;          // topological order
};

// Text form, one item per line:
//   group <name>
//   input <name> <dtype> <d0,d1,...>
//   op <type> <out> = <in0> <in1> ... [; key=value key=value ...]
//   output <name> <dtype> <d0,d1,...>
bool ParseGroupDesc(const std::string& text, GroupDesc* out, std::string* err);
std::string PrintGroupDesc(const GroupDesc& g);

// One kernel parameter of a launch step.
struct ArgSpec {
  enum Kind { kInput, kOutput, kScratch, kInt, kFloat, kAligned } kind = kInt;
  int index         = 0;    // kInput/kOutput: position in the group's input/output list
  int64_t ivalue    = 0;    // kInt: the value; kScratch: byte offset into the group's scratch buffer;
                            // kAligned: the static part of the condition (0/1)
  double fvalue     = 0.0;  // kFloat
  std::vector<int> aligned_inputs, aligned_outputs;  // kAligned: buffers whose addresses must be 16-byte aligned
};

struct LaunchStep {
  const KernelEntry* kernel = nullptr;
  unsigned grid[3]  = {1, 1, 1};
  unsigned block[3] = {1, 1, 1};
  unsigned cluster  = 0;     // cluster size along x, 0 = no cluster launch
  size_t dyn_smem   = 0;     // dynamic shared memory in bytes
  std::vector<ArgSpec> args;
};

struct CompiledGroup {
  std::string name;
  std::string pattern;              // which kernel family matched, for logs and tests
  std::vector<TensorDesc> inputs, outputs;
  std::vector<LaunchStep> steps;
  // When non-empty: `steps` additionally require the listed buffers to be 16-byte aligned at run time, and
  // `steps_unaligned` is the plan used when one of them is not.
  std::vector<LaunchStep> steps_unaligned;
  std::vector<int> aligned_inputs, aligned_outputs;
  size_t scratch_bytes     = 0;     // device scratch the steps need (split reductions), 0 for most groups
  int64_t algorithmic_bytes = 0;    // bytes of the group's inputs + outputs
  int64_t elements          = 0;    // output elements (input elements for reductions)
};

struct DeviceInfo {
  int sm_count              = 148;
  int max_smem_optin        = 227 * 1024;
  // Tuning knobs of the row-normalisation planner (0 = automatic).
  int rownorm_stages        = 0;
  int rownorm_ctas_per_sm   = 0;
  int enable_ew_stream      = 1;   // elementwise groups streamed through shared-memory rings (0 = register kernels)
  int ew_stream_stages      = 0;
  int ew_stream_ctas_per_sm = 0;
  int rowp_form = 0;  // row programs: 0 automatic, 32 a warp per row, 128 half a CTA per row, 256 a CTA per row
  int ew_reg_ctas_per_sm = 0;  // grid of the register form of the headline elementwise kernel (0: by size)
  int rownorm_rows_per_iter = 0;  // rows a CTA of the register-resident kernels takes per iteration
  int rownorm_simple        = -1;  // plain softmax by the one-CTA-per-row kernel of softmax_safe.cu: 1 on, 0 off, -1 automatic
  int fuse_interpreted_programs = 0;  // the fusion pass also forms groups that only the INTERPRETING register / row
                                      // program kernels take (several times slower than the specialised kernels; off:
                                      // such regions are split into groups the chain and reduction kernels take)
  int enable_static_chains  = 1;   // chain programs with a kernel specialised at build time use it (0: always interpret)
  int enable_tma_rownorm    = -1;  // rows streamed through shared memory by bulk copies: 1 on, 0 off, -1 automatic
};

// The planner's view of the current device with the options of cinn_b200_set_option applied (runtime.cc); without
// a GPU, the B200 defaults.
DeviceInfo CurrentDeviceInfo();

// Returns nullptr and fills *err when no prebuilt kernel covers the group.
std::unique_ptr<CompiledGroup> CompileGroup(const GroupDesc& g, const DeviceInfo& dev, std::string* err);

// The canonical expression of the group's (single) output with inputs printed as %<index>, e.g.
// "relu(elementwise_add(%0,%1))".  Exposed for tests and for the fusion pass.
std::string CanonicalExpr(const GroupDesc& g, std::string* err);

}  // namespace cinn_b200
