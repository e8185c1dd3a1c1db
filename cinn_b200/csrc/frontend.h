// NetBuilder / Program / fusion / Computation: the host side above the fused-group kernels.
//
// Mirrors the part of the reference's frontend and HLIR framework that sits on the hot path:
//   NetBuilder          cinn/frontend/net_builder.h:125-1146 (op methods append Instructions, shapes inferred)
//   Program/Variable    cinn/frontend/syntax.h:44-196
//   fusion              cinn/hlir/pass/op_fusion_pass.cc:123-331, cinn/hlir/pass/fusion_merge_pass.cc:44-1007
//   GraphCompiler       cinn/hlir/framework/graph_compiler.cc:749-792 (+ parallel_compiler.cc:123-217)
//   Program::Execute    cinn/hlir/framework/graph_compiler.cc:212-222, instruction.cc:77-165
//   CinnComputation     cinn/frontend/computation.h:26-158
// Differences by design: groups are compiled by pattern-matching against prebuilt kernels instead of code
// generation, and the fusion pass proposes groups and keeps only those a kernel exists for.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/cinn_runtime_abi.h"
#include "group_desc.h"

namespace cinn_b200 {

// cinn/hlir/framework/op.h:46-65.
enum class OpPattern { kElementWise, kBroadcast, kInjective, kReduction, kNonFusible, kConst };

struct Variable {
  std::string id;
  DType dtype = DType::kFloat32;
  std::vector<int64_t> shape;
  bool is_input = false;
};

struct ProgramInstr {
  std::string op_type;
  std::vector<int> inputs;   // variable indices
  int output = -1;           // variable index
  std::map<std::string, std::string> attrs;
};

class NetBuilder {
 public:
  explicit NetBuilder(const std::string& name) : name_(name) {}
  // cinn/frontend/net_builder.h CreateInput: returns the variable index, or -1 with *err set.
  int CreateInput(DType dtype, const std::vector<int64_t>& shape, const std::string& id_hint, std::string* err);
  // Generic form of every op method (Add, Relu, Scale, ReduceSum, ...): appends one instruction with the HLIR
  // op name `op_type` and returns its output variable, inferring shape and dtype.  -1 with *err on failure.
  int AddOp(const std::string& op_type, const std::vector<int>& inputs,
            const std::map<std::string, std::string>& attrs, std::string* err);
  int FindVar(const std::string& id) const;
  const std::string& name() const { return name_; }
  const std::vector<Variable>& vars() const { return vars_; }
  const std::vector<ProgramInstr>& instrs() const { return instrs_; }
  // For the program passes, which rebuild the instruction list the way the reference's passes rebuild a Program
  // through a fresh builder (cinn/frontend/pass/*.cc): variables are only ever appended, so indices stay valid.
  std::vector<ProgramInstr> TakeInstrs() { return std::move(instrs_); }
  void AppendInstr(const ProgramInstr& instr) { instrs_.push_back(instr); }

 private:
  std::string NewId(const std::string& hint);
  std::string name_;
  std::vector<Variable> vars_;
  std::vector<ProgramInstr> instrs_;
  std::map<std::string, int> var_index_;
  int counter_ = 0;
};

OpPattern PatternOf(const std::string& op_type);
bool KnownOp(const std::string& op_type);
// Ops registered with the kBroadcast pattern that take two operands (cinn/hlir/op/broadcast.cc:361-441).
bool IsBinaryBroadcastOp(const std::string& op_type);

// Program passes (cinn/frontend/program_pass.h:36-105, cinn/frontend/pass/*.cc).  Known names: "AutoCast",
// "AutoBroadcast", "CastCollapsing", "TransposeCollapsing", "FillConstantRewriter", "FillConstantFolding",
// "Decomposer" (gelu, softmax of any mode but "fast", inference batch_norm), "RemoveIdentity", "DeadCodeEliminate";
// "ExpandZeroDim", the one remaining name of the reference's default list, is accepted and does nothing (tensors here
// have at least one dimension).  `fetch` lists variables that must survive.
// An unknown name fails with *err set, as the reference's registry lookup does.
bool ApplyProgramPass(NetBuilder* b, const std::string& pass, const std::vector<int>& fetch, std::string* err);
// cinn/frontend/optimize.cc:44-82 (DefaultTrainingOptimizeOptions), in its order.
const std::vector<std::string>& DefaultProgramPasses();
// One line per instruction, "op out = in, in ; attr=value ...": what a pass left, for tests and logs.
std::string PrintProgram(const NetBuilder& b);

// One fused group after the fusion pass: which instructions it holds and its interface.
struct FusedGroupInfo {
  GroupDesc desc;
  std::vector<int> instr_indices;  // into NetBuilder::instrs()
  std::vector<int> input_vars;     // variable indices, argument order
  std::vector<int> output_vars;
  std::string pattern;             // matched kernel family
  std::vector<std::string> kernels;
};

// Partitions the program into groups, each of which a prebuilt kernel exists for.  `fetch` lists variables
// that must be materialised (default: every variable no instruction consumes).  Returns false with *err when
// some instruction cannot be executed by any kernel.
bool FusePasses(const NetBuilder& b, const std::vector<int>& fetch, const DeviceInfo& dev,
                std::vector<FusedGroupInfo>* groups, std::string* err);

// A device tensor of the computation's scope (cinn/hlir/framework/tensor.h:52-108, buffer.cc).
struct ScopeTensor {
  Variable var;
  cinn_buffer_t buffer;   // memory = device pointer
  bool owned   = false;   // allocated by the computation (cudaMalloc) or bound by the caller
  size_t bytes = 0;
};

class Computation {
 public:
  // Runs the fusion pass, compiles every group and (when device >= 0) allocates the scope's tensors on that
  // device.  device < 0 plans without touching a GPU.
  static std::unique_ptr<Computation> BuildAndCompile(const NetBuilder& b, const std::vector<int>& fetch,
                                                      int device, std::string* err);
  // The compiled program as text: its tensors, its groups (descriptions, in execution order) and its aliases.  What
  // the reference's Program::Export writes into a "CINN" file for its tiny runtime
  // (cinn/hlir/framework/graph_compiler.cc:89-210, cinn/runtime/tiny_runtime.cc:40-136), re-targeted to the prebuilt
  // kernel library: instruction -> group description -> prebuilt launcher, no builder, no fusion pass, no JIT.
  std::string Export() const;
  // Rebuilds a computation from Export()'s text: every group is matched to its prebuilt kernels again.
  static std::unique_ptr<Computation> Load(const std::string& text, int device, std::string* err);
  ~Computation();
  int Execute(void* stream, std::string* err);                       // Program::Execute
  int ExecuteTest(int repeat, double* avg_ms, std::string* err, bool use_graph = false);  // Program::ExecuteTest
  // The whole program as ONE CUDA graph: captured on the first call (after one ordinary run, so that every group has
  // its scratch), replayed afterwards; re-captured when a tensor is re-bound.  `stream` must not be NULL.  No
  // counterpart in the reference (its host loop issues one launch per instruction every time).
  int ExecuteGraph(void* stream, std::string* err);
  int SetTensorData(const std::string& id, const void* host, size_t bytes, std::string* err);
  int GetTensorData(const std::string& id, void* host, size_t bytes, std::string* err);
  int BindTensor(const std::string& id, void* device_ptr, std::string* err);  // caller-owned memory
  ScopeTensor* Find(const std::string& id);
  const std::vector<FusedGroupInfo>& groups() const { return groups_; }
  const std::vector<std::string>& tensor_names() const { return names_; }
  const std::vector<std::pair<std::string, std::string>>& aliases() const { return aliases_; }
  int device() const { return device_; }

 private:
  Computation() = default;
  bool AllocateScope(std::string* err);
  void AddScopeTensor(const Variable& var);
  struct Instr {
    lower_func_ptr_g fn = nullptr;
    std::string fn_name;
    std::vector<std::string> args;  // inputs then outputs
    std::vector<cinn_pod_value_t> pods;
  };
  std::vector<FusedGroupInfo> groups_;
  std::vector<Instr> instrs_;
  std::vector<std::pair<std::string, std::string>> aliases_;  // reshape result -> operand
  std::map<std::string, std::unique_ptr<ScopeTensor>> scope_;
  std::vector<std::string> names_;
  int device_ = -1;
  bool args_cached_ = false;
  void* graph_exec_ = nullptr;  // cudaGraphExec_t
  std::string uid_;
};

}  // namespace cinn_b200
