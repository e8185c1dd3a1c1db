// Header-only C++ front end over the C ABI of cinn_b200.h, with the method names of the reference's
// frontend::NetBuilder (cinn/frontend/net_builder.h:125-1146) and frontend::CinnComputation
// (cinn/frontend/computation.h:26-158), so that C++ code written against those classes ports line by line:
//
//     cinn_b200::frontend::NetBuilder builder("net");
//     auto a = builder.CreateInput("float32", {1, 3, 224, 224}, "A");
//     auto b = builder.CreateInput("float32", {1, 3, 224, 224}, "B");
//     auto c = builder.Relu(builder.Add(a, b));
//     auto comp = cinn_b200::frontend::CinnComputation::BuildAndCompile(/*device=*/0, builder, {c});
//     comp->SetTensorData("A", host_a, bytes);  comp->Execute();  comp->GetTensorData(c.id, host_c, bytes);
//
// Failures of the C functions become std::runtime_error here (the C ABI itself never throws).
#ifndef CINN_B200_FRONTEND_HPP_
#define CINN_B200_FRONTEND_HPP_

#include <cstdint>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "cinn_b200.h"

namespace cinn_b200 {
namespace frontend {

struct Variable {
  std::string id;
  const char* c_str() const { return id.c_str(); }
};

class NetBuilder {
 public:
  explicit NetBuilder(const std::string& name) : h_(cinn_b200_builder_create(name.c_str())) {
    if (!h_) throw std::runtime_error("cinn_b200_builder_create failed");
  }
  ~NetBuilder() { cinn_b200_builder_destroy(h_); }
  NetBuilder(const NetBuilder&)            = delete;
  NetBuilder& operator=(const NetBuilder&) = delete;
  cinn_b200_builder* handle() const { return h_; }

  Variable CreateInput(const std::string& dtype, const std::vector<int64_t>& shape, const std::string& id_hint = "") {
    std::vector<long long> s(shape.begin(), shape.end());
    char id[128];
    Check(cinn_b200_builder_create_input(h_, dtype.c_str(), s.data(), (int)s.size(), id_hint.c_str(), id, sizeof(id)));
    return Variable{id};
  }
  // The generic form (NetBuilder::CustomInstr in the reference): HLIR op name, operands, "key=value ..." attributes.
  Variable CustomInstr(const std::string& op, const std::vector<Variable>& inputs, const std::string& attrs = "") {
    std::vector<const char*> ids;
    for (auto& v : inputs) ids.push_back(v.id.c_str());
    char id[128];
    Check(cinn_b200_builder_add_op(h_, op.c_str(), ids.empty() ? nullptr : ids.data(), (int)ids.size(), attrs.c_str(), id,
                                   sizeof(id)));
    return Variable{id};
  }
  std::vector<int64_t> ShapeOf(const Variable& v, std::string* dtype = nullptr) const {
    char dt[32];
    long long shape[8];
    int nd = 0;
    Check(cinn_b200_builder_var_info(h_, v.id.c_str(), dt, sizeof(dt), shape, &nd));
    if (dtype) *dtype = dt;
    return std::vector<int64_t>(shape, shape + nd);
  }

  // ---- unary (net_builder.h NETBUILDER_UNARY_OP_FOREACH) ------------------------------------------------------------
#define CINN_B200_UNARY(Name, op) \
  Variable Name(const Variable& x) { return CustomInstr(op, {x}); }
  CINN_B200_UNARY(Sqrt, "sqrt") CINN_B200_UNARY(Tanh, "tanh") CINN_B200_UNARY(Relu, "relu")
  CINN_B200_UNARY(Sigmoid, "sigmoid") CINN_B200_UNARY(Identity, "identity") CINN_B200_UNARY(Exp, "exp")
  CINN_B200_UNARY(Erf, "erf") CINN_B200_UNARY(Rsqrt, "rsqrt") CINN_B200_UNARY(Log, "log") CINN_B200_UNARY(Log2, "log2")
  CINN_B200_UNARY(Log10, "log10") CINN_B200_UNARY(Floor, "floor") CINN_B200_UNARY(Ceil, "ceil")
  CINN_B200_UNARY(Round, "round") CINN_B200_UNARY(Trunc, "trunc") CINN_B200_UNARY(Sin, "sin") CINN_B200_UNARY(Cos, "cos")
  CINN_B200_UNARY(Tan, "tan") CINN_B200_UNARY(Sinh, "sinh") CINN_B200_UNARY(Cosh, "cosh") CINN_B200_UNARY(Asin, "asin")
  CINN_B200_UNARY(Acos, "acos") CINN_B200_UNARY(Atan, "atan") CINN_B200_UNARY(Asinh, "asinh")
  CINN_B200_UNARY(Acosh, "acosh") CINN_B200_UNARY(Atanh, "atanh") CINN_B200_UNARY(Cbrt, "cbrt")
  CINN_B200_UNARY(Negative, "negative") CINN_B200_UNARY(Sign, "sign") CINN_B200_UNARY(Abs, "abs")
  CINN_B200_UNARY(Reciprocal, "reciprocal") CINN_B200_UNARY(IsNan, "isnan") CINN_B200_UNARY(IsInf, "isinf")
  CINN_B200_UNARY(IsFinite, "isfinite") CINN_B200_UNARY(LogicalNot, "logical_not")
  CINN_B200_UNARY(BitwiseNot, "bitwise_not") CINN_B200_UNARY(Clz, "clz") CINN_B200_UNARY(Popc, "popc")
#undef CINN_B200_UNARY
  Variable Relu6(const Variable& x, float threshold = 6.0f) { return CustomInstr("relu6", {x}, "threshold=" + Num(threshold)); }

  // ---- binary with the `axis` broadcast rule (net_builder.h NETBUILDER_BINARY_OP_FOREACH) ----------------------------
#define CINN_B200_BINARY(Name, op) \
  Variable Name(const Variable& x, const Variable& y, int axis = -1) { return CustomInstr(op, {x, y}, "axis=" + std::to_string(axis)); }
  CINN_B200_BINARY(Add, "elementwise_add") CINN_B200_BINARY(ElementwiseAdd, "elementwise_add")
  CINN_B200_BINARY(Multiply, "elementwise_mul") CINN_B200_BINARY(ElementwiseMul, "elementwise_mul")
  CINN_B200_BINARY(Subtract, "subtract") CINN_B200_BINARY(Divide, "divide") CINN_B200_BINARY(FloorDivide, "floor_divide")
  CINN_B200_BINARY(Mod, "mod") CINN_B200_BINARY(Remainder, "remainder") CINN_B200_BINARY(Max, "max")
  CINN_B200_BINARY(Min, "min") CINN_B200_BINARY(Pow, "pow") CINN_B200_BINARY(Atan2, "atan2")
  CINN_B200_BINARY(LogicalAnd, "logical_and") CINN_B200_BINARY(LogicalOr, "logical_or")
  CINN_B200_BINARY(LogicalXor, "logical_xor") CINN_B200_BINARY(BitwiseAnd, "bitwise_and")
  CINN_B200_BINARY(BitwiseOr, "bitwise_or") CINN_B200_BINARY(BitwiseXor, "bitwise_xor")
  CINN_B200_BINARY(LeftShift, "left_shift") CINN_B200_BINARY(RightShift, "right_shift")
  CINN_B200_BINARY(LogicalRightShift, "logical_right_shift") CINN_B200_BINARY(Equal, "equal")
  CINN_B200_BINARY(NotEqual, "not_equal") CINN_B200_BINARY(GreaterThan, "greater_than")
  CINN_B200_BINARY(LessThan, "less_than") CINN_B200_BINARY(GreaterEqual, "greater_equal")
  CINN_B200_BINARY(LessEqual, "less_equal")
#undef CINN_B200_BINARY

  // ---- the rest of the ops on this path -------------------------------------------------------------------------------
  Variable Scale(const Variable& x, float scale = 1.0f, float bias = 0.0f, bool bias_after_scale = true) {
    return CustomInstr("scale", {x}, "scale=" + Num(scale) + " bias=" + Num(bias) + " bias_after_scale=" + (bias_after_scale ? "true" : "false"));
  }
  Variable Cast(const Variable& x, const std::string& dtype) { return CustomInstr("cast", {x}, "dtype=" + dtype); }
  Variable Select(const Variable& cond, const Variable& t, const Variable& f) { return CustomInstr("select", {cond, t, f}); }
  Variable BroadcastTo(const Variable& x, const std::vector<int>& out_shape, const std::vector<int>& broadcast_axes = {}) {
    std::string a = "out_shape=" + List(out_shape);
    if (!broadcast_axes.empty()) a += " broadcast_axes=" + List(broadcast_axes);
    return CustomInstr("broadcast_to", {x}, a);
  }
  Variable FillConstant(const std::vector<int>& shape, float value, const std::string& name = "", const std::string& dtype = "float32") {
    (void)name;
    return CustomInstr("fill_constant", {}, "shape=" + List(shape) + " value=" + Num(value) + " dtype=" + dtype);
  }
  Variable Reshape(const Variable& x, const std::vector<int>& shape) { return CustomInstr("reshape", {x}, "shape=" + List(shape)); }
  Variable Squeeze(const Variable& x, const std::vector<int>& axes = {}) { return CustomInstr("squeeze", {x}, axes.empty() ? "" : "axes=" + List(axes)); }
  Variable ExpandDims(const Variable& x, const std::vector<int>& axes) { return CustomInstr("expand_dims", {x}, "axes=" + List(axes)); }
  Variable Transpose(const Variable& x, const std::vector<int>& axis) { return CustomInstr("transpose", {x}, "axis=" + List(axis)); }
  Variable Concat(const std::vector<Variable>& inputs, int axis = 0) { return CustomInstr("concat", inputs, "axis=" + std::to_string(axis)); }
  Variable Slice(const Variable& x, const std::vector<int>& axes, const std::vector<int>& starts, const std::vector<int>& ends,
                 const std::vector<int>& infer_flags = {}, const std::vector<int>& strides = {}, const std::vector<int>& decrease_axis = {}) {
    (void)infer_flags;
    std::string a = "axes=" + List(axes) + " starts=" + List(starts) + " ends=" + List(ends);
    if (!strides.empty()) a += " strides=" + List(strides);
    if (!decrease_axis.empty()) a += " decrease_axis=" + List(decrease_axis);
    return CustomInstr("slice", {x}, a);
  }
#define CINN_B200_REDUCE(Name, op)                                                                      \
  Variable Name(const Variable& x, const std::vector<int>& dim = {}, bool keep_dim = false) {             \
    return CustomInstr(op, {x}, (dim.empty() ? std::string() : "dim=" + List(dim) + " ") + "keep_dim=" + (keep_dim ? "true" : "false")); \
  }
  CINN_B200_REDUCE(ReduceSum, "reduce_sum") CINN_B200_REDUCE(ReduceProd, "reduce_prod")
  CINN_B200_REDUCE(ReduceMax, "reduce_max") CINN_B200_REDUCE(ReduceMin, "reduce_min")
  CINN_B200_REDUCE(ReduceAll, "reduce_all") CINN_B200_REDUCE(ReduceAny, "reduce_any")
#undef CINN_B200_REDUCE
  // The softmax op itself (mode "fast" of the reference: exp(x) / sum(exp(x)), cinn/hlir/pe/nn.cc:755-796).
  Variable Softmax(const Variable& x, const std::vector<int>& axes = {-1}) {
    return CustomInstr("softmax", {x}, "axis=" + std::to_string(axes.empty() ? -1 : axes[0]));
  }
  // gelu as an instruction (cinn/frontend/net_builder.h Gelu): no kernel takes it as such; compile with
  // CompileOptions::use_decomposer (or apply the "Decomposer" pass) to turn it into its primitives.
  Variable Gelu(const Variable& x) { return CustomInstr("gelu", {x}); }
  // Softmax with a mode: "fast" is the op above; any other mode subtracts the row maximum and needs the Decomposer.
  Variable Softmax(const Variable& x, const std::vector<int>& axes, const std::string& mode) {
    return CustomInstr("softmax", {x}, "axis=" + std::to_string(axes.empty() ? -1 : axes[0]) + " mode=" + mode);
  }
  // Inference batch norm (is_test = true), argument order of cinn/frontend/net_builder.cc:764-801.
  Variable BatchNorm(const Variable& x, const Variable& scale, const Variable& bias, const Variable& mean, const Variable& variance,
                     float epsilon = 1e-5f, const std::string& data_layout = "NCHW") {
    return CustomInstr("batch_norm", {x, scale, bias, mean, variance}, "epsilon=" + Num(epsilon) + " data_layout=" + data_layout);
  }
  // ProgramPass::Apply (cinn/frontend/program_pass.h:36-105): rewrites the program by the named passes, in order; an
  // empty list applies the default list of cinn/frontend/optimize.cc:44-82.  `fetch` are the variables that must survive.
  void ApplyPasses(const std::vector<Variable>& fetch, const std::vector<std::string>& passes = {}) {
    std::vector<const char*> f, p;
    for (auto& v : fetch) f.push_back(v.id.c_str());
    for (auto& n : passes) p.push_back(n.c_str());
    Check(cinn_b200_builder_apply_passes(h_, p.data(), (int)p.size(), f.data(), (int)f.size()));
  }
  // One line per instruction: "op out = in, in ; attr=value ...".
  std::string ProgramText() const {
    long long need = cinn_b200_builder_program_text(h_, nullptr, 0);
    if (need <= 0) throw std::runtime_error(std::string("cinn_b200: ") + cinn_b200_last_error());
    std::string text((size_t)need, '\0');
    cinn_b200_builder_program_text(h_, &text[0], text.size());
    text.resize((size_t)need - 1);
    return text;
  }

 private:
  static void Check(int rc) {
    if (rc != CINN_B200_OK) throw std::runtime_error(std::string("cinn_b200: ") + cinn_b200_last_error());
  }
  static std::string Num(double v) {
    std::ostringstream os;
    os.precision(9);
    os << v;
    return os.str();
  }
  static std::string List(const std::vector<int>& v) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
    return s;
  }
  cinn_b200_builder* h_;
};

// What CinnComputation::GetTensor returns: a description of a scope tensor (hlir::framework::Tensor in the reference).
struct TensorInfo {
  std::string id, dtype;
  std::vector<int64_t> shape;
  void* device_ptr = nullptr;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

// frontend::CinnComputation (cinn/frontend/computation.h:26-158).
class CinnComputation {
 public:
  // Compile is BuildAndCompile under the reference's other name (there it takes a Program already built).
  static std::shared_ptr<CinnComputation> Compile(int device, const NetBuilder& builder, const std::vector<Variable>& outputs = {}) {
    return BuildAndCompile(device, builder, outputs);
  }
  TensorInfo GetTensor(const std::string& id) const {
    TensorInfo t;
    char dt[32];
    long long shape[8];
    int nd = 0;
    Check(cinn_b200_computation_tensor_info(h_, id.c_str(), dt, sizeof(dt), shape, &nd, &t.device_ptr));
    t.id    = id;
    t.dtype = dt;
    t.shape.assign(shape, shape + nd);
    return t;
  }
  std::vector<TensorInfo> GetInputTensors() const { return TensorsOfRole(0); }
  std::vector<TensorInfo> GetOutputTensors() const { return TensorsOfRole(2); }
  // device < 0 plans without touching a GPU (fusion + kernel matching only).
  // CinnComputation::CompileOptions (cinn/frontend/computation.h:30-44).  use_decomposer runs the Decomposer program
  // pass first, as cinn/frontend/computation.cc:53-55 does; `passes` names further program passes to run after it.
  struct CompileOptions {
    bool use_decomposer = false;
    bool do_prerun = true;           // kept for source compatibility: kernels are prebuilt, there is nothing to pre-run
    bool use_default_passes = true;  // the fusion pass always runs
    std::vector<std::string> passes;
  };
  static CompileOptions DefaultCompileOptions() { return CompileOptions(); }
  static std::shared_ptr<CinnComputation> BuildAndCompile(int device, NetBuilder& builder, const CompileOptions& options,
                                                          const std::vector<Variable>& outputs = {}) {
    std::vector<std::string> names = options.passes;
    if (options.use_decomposer) names.insert(names.begin(), "Decomposer");
    if (!names.empty()) builder.ApplyPasses(outputs, names);
    return BuildAndCompile(device, builder, outputs);
  }
  static std::shared_ptr<CinnComputation> BuildAndCompile(int device, const NetBuilder& builder,
                                                          const std::vector<Variable>& outputs = {}) {
    std::vector<const char*> ids;
    for (auto& v : outputs) ids.push_back(v.id.c_str());
    cinn_b200_computation* h =
        cinn_b200_computation_build_and_compile(builder.handle(), device, ids.empty() ? nullptr : ids.data(), (int)ids.size());
    if (!h) throw std::runtime_error(std::string("cinn_b200: ") + cinn_b200_last_error());
    return std::shared_ptr<CinnComputation>(new CinnComputation(h));
  }
  // From the text written by Export(): no builder, no fusion pass (the tiny-runtime path of the reference).
  static std::shared_ptr<CinnComputation> Load(const std::string& program_text, int device) {
    cinn_b200_computation* h = cinn_b200_program_load(program_text.c_str(), device);
    if (!h) throw std::runtime_error(std::string("cinn_b200: ") + cinn_b200_last_error());
    return std::shared_ptr<CinnComputation>(new CinnComputation(h));
  }
  ~CinnComputation() { cinn_b200_computation_destroy(h_); }
  CinnComputation(const CinnComputation&)            = delete;
  CinnComputation& operator=(const CinnComputation&) = delete;

  void Execute(void* stream = nullptr) { Check(cinn_b200_computation_execute(h_, stream)); }
  // The whole program replayed as one CUDA graph (captured at the first call); `stream` must not be NULL.
  void ExecuteGraph(void* stream) { Check(cinn_b200_computation_execute_graph(h_, stream)); }
  // Program::ExecuteTest: average milliseconds per run over `repeat` runs (use_graph: replaying the CUDA graph).
  double ExecuteTest(int repeat, bool use_graph = false) {
    double ms = 0.0;
    Check(cinn_b200_computation_execute_test(h_, use_graph ? -repeat : repeat, &ms));
    return ms;
  }
  void SetTensorData(const std::string& id, const void* host, size_t bytes) {
    Check(cinn_b200_computation_set_tensor_data(h_, id.c_str(), host, bytes));
  }
  void GetTensorData(const std::string& id, void* host, size_t bytes) {
    Check(cinn_b200_computation_get_tensor_data(h_, id.c_str(), host, bytes));
  }
  void BindTensor(const std::string& id, void* device_ptr) { Check(cinn_b200_computation_bind_tensor(h_, id.c_str(), device_ptr)); }
  std::vector<std::string> GetAllTensorNames() const {
    std::vector<std::string> names;
    const int n = cinn_b200_computation_num_tensors(h_);
    for (int i = 0; i < n; ++i) names.push_back(cinn_b200_computation_tensor_name(h_, i));
    return names;
  }
  // "pattern kernel kernel ..." of every group the fusion pass produced, in execution order.
  std::vector<std::string> GroupPatterns() const {
    std::vector<std::string> out;
    const int n = cinn_b200_computation_num_groups(h_);
    for (int i = 0; i < n; ++i) {
      char buf[1024];
      Check(cinn_b200_computation_group_pattern(h_, i, buf, sizeof(buf)));
      out.push_back(buf);
    }
    return out;
  }
  std::string Export() const {
    const long long need = cinn_b200_computation_export(h_, nullptr, 0);
    if (need < 0) throw std::runtime_error(std::string("cinn_b200: ") + cinn_b200_last_error());
    std::string text((size_t)need, '\0');
    cinn_b200_computation_export(h_, &text[0], text.size());
    text.resize(text.size() - 1);
    return text;
  }
  cinn_b200_computation* handle() const { return h_; }

 private:
  explicit CinnComputation(cinn_b200_computation* h) : h_(h) {}
  std::vector<TensorInfo> TensorsOfRole(int role) const {
    std::vector<TensorInfo> out;
    for (auto& name : GetAllTensorNames())
      if (cinn_b200_computation_tensor_role(h_, name.c_str()) == role) out.push_back(GetTensor(name));
    return out;
  }
  static void Check(int rc) {
    if (rc != CINN_B200_OK) throw std::runtime_error(std::string("cinn_b200: ") + cinn_b200_last_error());
  }
  cinn_b200_computation* h_;
};

}  // namespace frontend
}  // namespace cinn_b200

#endif  // CINN_B200_FRONTEND_HPP_
