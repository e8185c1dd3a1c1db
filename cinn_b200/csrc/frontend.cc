// NetBuilder, op shape/dtype inference, the fusion pass and the Computation executor.
#include "frontend.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <set>
#include <sstream>

#include "../../include/cinn_b200.h"

namespace cinn_b200 {

// ---- op registry ------------------------------------------------------------------------------------
// Names and pattern kinds follow the op registrations of cinn/hlir/op/elementwise.cc:860-1066,
// broadcast.cc:361-441, reduction.cc:477-505 and nn.cc:2262-2433; binary "broadcast" ops take part in
// fusion as elementwise ops (cinn/hlir/pass/fusion_helper_base.h:47-59).
namespace {

const std::set<std::string>& UnaryOps() {
  static const std::set<std::string> s = {
      "sqrt", "tanh", "sigmoid", "identity", "exp", "erf", "rsqrt", "log", "log2", "log10", "floor", "ceil", "round",
      "trunc", "sin", "cos", "negative", "sign", "abs", "relu", "relu6", "reciprocal", "gelu",
      "tan", "sinh", "cosh", "asin", "acos", "atan", "asinh", "acosh", "atanh", "cbrt",
      "isnan", "isinf", "isfinite", "logical_not", "bitwise_not", "clz", "popc"};
  return s;
}
// Unary ops whose result is bool whatever the operand type (cinn/hlir/op/elementwise.cc: isnan, isfinite, isinf,
// logical_not).
const std::set<std::string>& PredicateOps() {
  static const std::set<std::string> s = {"isnan", "isinf", "isfinite", "logical_not"};
  return s;
}
const std::set<std::string>& BinaryOps() {
  static const std::set<std::string> s = {"elementwise_add", "elementwise_mul", "subtract", "divide", "max", "min",
                                          "pow", "mod", "remainder", "floor_divide", "atan2", "logical_and",
                                          "logical_or", "logical_xor", "bitwise_and", "bitwise_or", "bitwise_xor",
                                          "left_shift", "right_shift", "logical_right_shift"};
  return s;
}
const std::set<std::string>& CompareOps() {
  static const std::set<std::string> s = {"equal", "not_equal", "greater_than", "less_than", "greater_equal",
                                          "less_equal"};
  return s;
}
const std::set<std::string>& ReduceOps() {
  static const std::set<std::string> s = {"reduce_sum", "reduce_prod", "reduce_max", "reduce_min", "reduce_all",
                                          "reduce_any"};
  return s;
}

std::vector<int64_t> ParseIntList(const std::string& text) {
  std::vector<int64_t> out;
  std::string cur;
  for (char c : text + ",") {
    if (c == ',') {
      if (!cur.empty()) out.push_back(atoll(cur.c_str()));
      cur.clear();
    } else if (c != '[' && c != ']' && c != ' ' && c != '(' && c != ')') {
      cur.push_back(c);
    }
  }
  return out;
}

std::string JoinInts(const std::vector<int64_t>& v) {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) {
    if (i) s += ",";
    s += std::to_string(v[i]);
  }
  return s;
}

// cinn/hlir/pe/broadcast.cc:35-118 (GetBroadcastShape): equal shapes pass through; otherwise the
// lower-rank operand is aligned at `axis` (axis = -1: right-aligned) and extents must match or be 1.
bool BroadcastShape(const std::vector<int64_t>& a, const std::vector<int64_t>& b, int64_t axis,
                    std::vector<int64_t>* out, std::string* err) {
  if (a == b) {
    *out = a;
    return true;
  }
  const std::vector<int64_t>& big   = a.size() >= b.size() ? a : b;
  const std::vector<int64_t>& small = a.size() >= b.size() ? b : a;
  int64_t off = axis < 0 ? (int64_t)big.size() - (int64_t)small.size() : axis;
  if (off < 0 || off + small.size() > big.size()) {
    if (err) *err = "broadcast axis " + std::to_string(axis) + " does not fit the operand ranks";
    return false;
  }
  *out = big;
  for (size_t i = 0; i < small.size(); ++i) {
    int64_t x = big[off + i], y = small[i];
    if (x == y || y == 1) continue;
    if (x == 1) {
      (*out)[off + i] = y;
      continue;
    }
    if (err) *err = "operands cannot be broadcast together: extents " + std::to_string(x) + " and " + std::to_string(y);
    return false;
  }
  return true;
}

}  // namespace

bool KnownOp(const std::string& t) {
  return UnaryOps().count(t) || BinaryOps().count(t) || CompareOps().count(t) || ReduceOps().count(t) ||
         t == "scale" || t == "cast" || t == "select" || t == "broadcast_to" || t == "fill_constant" ||
         t == "softmax" || t == "batch_norm" || t == "reshape" || t == "squeeze" || t == "expand_dims" ||
         t == "transpose" || t == "slice" || t == "concat";
}

bool IsBinaryBroadcastOp(const std::string& t) { return BinaryOps().count(t) || CompareOps().count(t); }

OpPattern PatternOf(const std::string& t) {
  if (t == "fill_constant") return OpPattern::kConst;
  if (ReduceOps().count(t)) return OpPattern::kReduction;
  if (t == "broadcast_to") return OpPattern::kBroadcast;
  if (t == "reshape") return OpPattern::kNonFusible;
  // Data movement (registered kInjective in the reference, cinn/hlir/op/transform.cc): a kernel of its own here.
  if (t == "transpose" || t == "slice" || t == "concat") return OpPattern::kNonFusible;
  // softmax is registered kNonFusible in the reference (cinn/hlir/op/nn.cc:2383-2393); here the casts around
  // it may join its group, so it takes part in fusion like an elementwise op.
  return OpPattern::kElementWise;
}

// ---- NetBuilder ---------------------------------------------------------------------------------------
std::string NetBuilder::NewId(const std::string& hint) {
  if (!hint.empty() && !var_index_.count(hint)) return hint;
  std::string id;
  do {
    id = "var_" + std::to_string(counter_++);
  } while (var_index_.count(id));
  return id;
}

int NetBuilder::FindVar(const std::string& id) const {
  auto it = var_index_.find(id);
  return it == var_index_.end() ? -1 : it->second;
}

int NetBuilder::CreateInput(DType dtype, const std::vector<int64_t>& shape, const std::string& id_hint,
                            std::string* err) {
  if (dtype == DType::kUnknown) {
    if (err) *err = "create_input: unknown dtype";
    return -1;
  }
  if (shape.size() > CINN_BUFFER_MAX_DIMS) {
    if (err) *err = "create_input: at most 8 dimensions (cinn_buffer_t)";
    return -1;
  }
  for (auto d : shape)
    if (d <= 0) {
      if (err) *err = "create_input: non-positive extent";
      return -1;
    }
  Variable v;
  v.id       = NewId(id_hint);
  v.dtype    = dtype;
  v.shape    = shape;
  v.is_input = true;
  vars_.push_back(v);
  var_index_[v.id] = (int)vars_.size() - 1;
  return (int)vars_.size() - 1;
}

int NetBuilder::AddOp(const std::string& op, const std::vector<int>& inputs,
                      const std::map<std::string, std::string>& attrs_in, std::string* err) {
  auto fail = [&](const std::string& m) {
    if (err) *err = op + ": " + m;
    return -1;
  };
  if (!KnownOp(op)) return fail("op is not supported by the fused-group kernel library");
  for (int i : inputs)
    if (i < 0 || i >= (int)vars_.size()) return fail("bad input variable");
  auto attrs = attrs_in;
  auto in    = [&](int k) -> const Variable& { return vars_[inputs[k]]; };
  auto need  = [&](size_t n) { return inputs.size() == n; };
  if (op == "squeeze" || op == "expand_dims") {
    // Both only change the shape: they become a reshape, which aliases its operand's memory.
    if (!need(1)) return fail("takes 1 input");
    std::vector<int64_t> axes = ParseIntList(attrs.count("axes") ? attrs["axes"] : "");
    std::vector<int64_t> shape;
    const int nd = (int)in(0).shape.size();
    if (op == "squeeze") {
      for (auto& a : axes)
        if (a < 0) a += nd;
      for (int i = 0; i < nd; ++i) {
        const bool listed = std::find(axes.begin(), axes.end(), (int64_t)i) != axes.end();
        if (listed && in(0).shape[i] != 1) return fail("squeezed axis has extent " + std::to_string(in(0).shape[i]));
        if (!(in(0).shape[i] == 1 && (axes.empty() || listed))) shape.push_back(in(0).shape[i]);
      }
      if (shape.empty()) shape.push_back(1);
    } else {
      // cinn/hlir/op/transform.cc expand_dims: each listed position of the RESULT gets an extent-1 axis
      const int out_nd = nd + (int)axes.size();
      std::vector<bool> is_new(out_nd, false);
      for (auto a : axes) {
        if (a < 0) a += out_nd;
        if (a < 0 || a >= out_nd) return fail("axis out of range");
        is_new[a] = true;
      }
      int k = 0;
      for (int i = 0; i < out_nd; ++i) shape.push_back(is_new[i] ? 1 : in(0).shape[k++]);
    }
    return AddOp("reshape", inputs, {{"shape", JoinInts(shape)}}, err);
  }
  Variable out;
  if (UnaryOps().count(op)) {
    if (!need(1)) return fail("takes 1 input");
    out.dtype = PredicateOps().count(op) ? DType::kBool : in(0).dtype;
    out.shape = in(0).shape;
    if (op == "logical_not" && in(0).dtype != DType::kBool) return fail("operand must be bool");
    if ((op == "bitwise_not" || op == "clz" || op == "popc") && in(0).dtype != DType::kInt32 && in(0).dtype != DType::kInt64 &&
        in(0).dtype != DType::kUInt8 && !(op == "bitwise_not" && in(0).dtype == DType::kBool))
      return fail("operand must be an integer");
  } else if (BinaryOps().count(op) || CompareOps().count(op)) {
    if (!need(2)) return fail("takes 2 inputs");
    if (in(0).dtype != in(1).dtype) return fail("operand dtypes differ");
    int64_t axis = attrs.count("axis") ? atoll(attrs["axis"].c_str()) : -1;
    attrs["axis"] = std::to_string(axis);
    std::string e;
    if (!BroadcastShape(in(0).shape, in(1).shape, axis, &out.shape, &e)) return fail(e);
    out.dtype = CompareOps().count(op) ? DType::kBool : in(0).dtype;
    if (op.rfind("logical_", 0) == 0 && op != "logical_right_shift" && in(0).dtype != DType::kBool)
      return fail("operands must be bool");
  } else if (op == "scale") {
    if (!need(1)) return fail("takes 1 input");
    if (!attrs.count("scale")) attrs["scale"] = "1.0";
    if (!attrs.count("bias")) attrs["bias"] = "0.0";
    if (!attrs.count("bias_after_scale")) attrs["bias_after_scale"] = "true";
    out.dtype = in(0).dtype;
    out.shape = in(0).shape;
  } else if (op == "cast") {
    if (!need(1)) return fail("takes 1 input");
    out.dtype = DTypeFromName(attrs.count("dtype") ? attrs["dtype"] : "");
    if (out.dtype == DType::kUnknown) return fail("needs a known 'dtype' attribute");
    out.shape = in(0).shape;
  } else if (op == "select") {
    if (!need(3)) return fail("takes 3 inputs (condition, true value, false value)");
    if (in(0).dtype != DType::kBool) return fail("condition must be bool");
    if (in(1).dtype != in(2).dtype || in(1).shape != in(2).shape || in(0).shape != in(1).shape)
      return fail("operands must have one shape and the values one dtype");
    out.dtype = in(1).dtype;
    out.shape = in(1).shape;
  } else if (op == "broadcast_to") {
    if (!need(1)) return fail("takes 1 input");
    out.shape = ParseIntList(attrs.count("out_shape") ? attrs["out_shape"] : "");
    if (out.shape.empty()) return fail("needs 'out_shape'");
    std::vector<int64_t> axes = ParseIntList(attrs.count("broadcast_axes") ? attrs["broadcast_axes"] : "");
    if (axes.empty()) {  // right-aligned, cinn/hlir/pe/broadcast.cc:293-327
      for (size_t i = 0; i < in(0).shape.size(); ++i) axes.push_back(out.shape.size() - in(0).shape.size() + i);
    }
    if (axes.size() != in(0).shape.size()) return fail("'broadcast_axes' must have one entry per input dimension");
    for (size_t i = 0; i < axes.size(); ++i) {
      if (axes[i] < 0) axes[i] += out.shape.size();
      if (axes[i] < 0 || axes[i] >= (int64_t)out.shape.size()) return fail("broadcast axis out of range");
      if (in(0).shape[i] != 1 && in(0).shape[i] != out.shape[axes[i]]) return fail("input extent does not match out_shape");
    }
    attrs["out_shape"]      = JoinInts(out.shape);
    attrs["broadcast_axes"] = JoinInts(axes);
    out.dtype               = in(0).dtype;
  } else if (op == "fill_constant") {
    if (!need(0)) return fail("takes no input");
    out.shape = ParseIntList(attrs.count("shape") ? attrs["shape"] : "");
    if (out.shape.empty()) return fail("needs 'shape'");
    if (!attrs.count("value")) return fail("needs 'value'");
    out.dtype = DTypeFromName(attrs.count("dtype") ? attrs["dtype"] : "float32");
    if (out.dtype == DType::kUnknown) return fail("unknown 'dtype'");
    attrs["shape"] = JoinInts(out.shape);
    attrs["dtype"] = DTypeName(out.dtype);
  } else if (ReduceOps().count(op)) {
    if (!need(1)) return fail("takes 1 input");
    const int nd = (int)in(0).shape.size();
    std::vector<int64_t> dims = ParseIntList(attrs.count("dim") ? attrs["dim"] : "");
    // cinn/frontend/net_builder.cc:98-128: empty dim = all axes, negative axes wrap.
    if (dims.empty())
      for (int i = 0; i < nd; ++i) dims.push_back(i);
    for (auto& d : dims) {
      if (d < 0) d += nd;
      if (d < 0 || d >= nd) return fail("reduce axis out of range");
    }
    std::sort(dims.begin(), dims.end());
    dims.erase(std::unique(dims.begin(), dims.end()), dims.end());
    bool keep = attrs.count("keep_dim") && (attrs["keep_dim"] == "true" || attrs["keep_dim"] == "1" || attrs["keep_dim"] == "True");
    attrs["dim"]      = JoinInts(dims);
    attrs["keep_dim"] = keep ? "true" : "false";
    for (int i = 0; i < nd; ++i) {
      bool red = std::binary_search(dims.begin(), dims.end(), (int64_t)i);
      if (!red) out.shape.push_back(in(0).shape[i]);
      else if (keep) out.shape.push_back(1);
    }
    if (out.shape.empty()) out.shape.push_back(1);
    out.dtype = in(0).dtype;
    if ((op == "reduce_all" || op == "reduce_any") && in(0).dtype != DType::kBool) return fail("operand must be bool");
  } else if (op == "softmax") {
    if (!need(1)) return fail("takes 1 input");
    if (!attrs.count("axis")) attrs["axis"] = "-1";
    out.dtype = in(0).dtype;
    out.shape = in(0).shape;
  } else if (op == "batch_norm") {
    // argument order x, scale, bias, mean, variance: cinn/frontend/net_builder.cc:764-801
    if (!need(5)) return fail("takes 5 inputs (x, scale, bias, mean, variance)");
    if (in(0).shape.size() != 4) return fail("input must be 4-D");
    if (!attrs.count("epsilon")) attrs["epsilon"] = "1e-05";
    if (!attrs.count("data_layout")) attrs["data_layout"] = "NCHW";
    out.dtype = in(0).dtype;
    out.shape = in(0).shape;
  } else if (op == "reshape") {
    if (!need(1)) return fail("takes 1 input");
    out.shape = ParseIntList(attrs.count("shape") ? attrs["shape"] : "");
    int64_t n = 1, total = 1, unknown = -1;
    for (auto d : in(0).shape) total *= d;
    for (size_t i = 0; i < out.shape.size(); ++i) {
      if (out.shape[i] == -1) unknown = (int64_t)i;
      else n *= out.shape[i];
    }
    if (unknown >= 0) {
      if (n == 0 || total % n) return fail("cannot infer the -1 extent");
      out.shape[unknown] = total / n;
      n *= out.shape[unknown];
    }
    if (n != total) return fail("element count changes");
    attrs["shape"] = JoinInts(out.shape);
    out.dtype      = in(0).dtype;
  } else if (op == "transpose") {
    if (!need(1)) return fail("takes 1 input");
    const int nd = (int)in(0).shape.size();
    std::vector<int64_t> perm = ParseIntList(attrs.count("axis") ? attrs["axis"] : "");
    if ((int)perm.size() != nd) return fail("'axis' must list every axis once");
    std::vector<bool> seen(nd, false);
    for (auto& a : perm) {
      if (a < 0) a += nd;
      if (a < 0 || a >= nd || seen[a]) return fail("'axis' must be a permutation");
      seen[a] = true;
      out.shape.push_back(in(0).shape[a]);
    }
    attrs["axis"] = JoinInts(perm);
    out.dtype     = in(0).dtype;
  } else if (op == "concat") {
    if (inputs.empty()) return fail("takes at least 1 input");
    const int nd = (int)in(0).shape.size();
    int64_t axis = attrs.count("axis") ? atoll(attrs["axis"].c_str()) : 0;
    if (axis < 0) axis += nd;
    if (axis < 0 || axis >= nd) return fail("axis out of range");
    out.shape = in(0).shape;
    out.dtype = in(0).dtype;
    for (size_t k = 1; k < inputs.size(); ++k) {
      if (in(k).dtype != out.dtype || (int)in(k).shape.size() != nd) return fail("operands differ in type or rank");
      for (int i = 0; i < nd; ++i)
        if (i != axis && in(k).shape[i] != out.shape[i]) return fail("operands differ outside the concat axis");
      out.shape[axis] += in(k).shape[axis];
      for (size_t q = 0; q < k; ++q)
        if (inputs[q] == inputs[k]) return fail("the same variable twice has no prebuilt kernel");
    }
    attrs["axis"] = std::to_string(axis);
  } else if (op == "slice") {
    if (!need(1)) return fail("takes 1 input");
    const int nd = (int)in(0).shape.size();
    std::vector<int64_t> axes = ParseIntList(attrs.count("axes") ? attrs["axes"] : ""),
                         starts = ParseIntList(attrs.count("starts") ? attrs["starts"] : ""),
                         ends = ParseIntList(attrs.count("ends") ? attrs["ends"] : ""),
                         strides = ParseIntList(attrs.count("strides") ? attrs["strides"] : ""),
                         decrease = ParseIntList(attrs.count("decrease_axis") ? attrs["decrease_axis"] : "");
    if (starts.size() != axes.size() || ends.size() != axes.size()) return fail("axes / starts / ends differ in length");
    std::vector<int64_t> shape = in(0).shape;
    for (size_t k = 0; k < axes.size(); ++k) {
      int64_t a = axes[k] < 0 ? axes[k] + nd : axes[k];
      if (a < 0 || a >= nd) return fail("axis out of range");
      const int64_t dim = in(0).shape[a], st = k < strides.size() ? strides[k] : 1;
      int64_t b = starts[k] < 0 ? starts[k] + dim : starts[k], e = ends[k] < 0 ? ends[k] + dim : ends[k];
      if (st > 0) {
        b = std::min(std::max<int64_t>(b, 0), dim);
        e = std::min(std::max<int64_t>(e, 0), dim);
        shape[a] = e > b ? (e - b + st - 1) / st : 0;
      } else if (st < 0) {
        b = std::min(std::max<int64_t>(b, -1), dim - 1);
        e = std::min(std::max<int64_t>(e, -1), dim - 1);
        shape[a] = b > e ? (b - e + (-st) - 1) / (-st) : 0;
      } else {
        return fail("zero stride");
      }
      if (shape[a] <= 0) return fail("empty slice");
    }
    for (int i = 0; i < nd; ++i) {
      bool drop = false;
      for (auto d : decrease) drop = drop || (d < 0 ? d + nd : d) == i;
      if (drop && shape[i] != 1) return fail("decrease_axis on an axis of extent " + std::to_string(shape[i]));
      if (!drop) out.shape.push_back(shape[i]);
    }
    if (out.shape.empty()) out.shape.push_back(1);
    out.dtype = in(0).dtype;
  }
  if (out.shape.size() > CINN_BUFFER_MAX_DIMS) return fail("result has more than 8 dimensions");
  out.id = NewId("");
  vars_.push_back(out);
  var_index_[out.id] = (int)vars_.size() - 1;
  ProgramInstr ins;
  ins.op_type = op;
  ins.inputs  = inputs;
  ins.output  = (int)vars_.size() - 1;
  ins.attrs   = attrs;
  instrs_.push_back(ins);
  return ins.output;
}

// ---- fusion ---------------------------------------------------------------------------------------------
namespace {

struct FusionState {
  const NetBuilder& b;
  const DeviceInfo& dev;
  std::vector<int> producer_of_var;                // variable -> instruction (-1 for inputs)
  std::vector<std::vector<int>> consumers_of_var;  // variable -> instructions
  std::set<int> fetch;
  // Instructions that are evaluated again inside every group that reads their result (cheap elementwise producers
  // with several consumers): their result is not a group output and is never materialised.
  std::set<int> recomputed;
  int uid;

  FusionState(const NetBuilder& b_, const DeviceInfo& d, int uid_) : b(b_), dev(d), uid(uid_) {
    producer_of_var.assign(b.vars().size(), -1);
    consumers_of_var.assign(b.vars().size(), {});
    for (size_t i = 0; i < b.instrs().size(); ++i) {
      producer_of_var[b.instrs()[i].output] = (int)i;
      for (int v : b.instrs()[i].inputs) consumers_of_var[v].push_back((int)i);
    }
  }

  bool IsConst(int instr) const { return PatternOf(b.instrs()[instr].op_type) == OpPattern::kConst; }

  // Builds the description of the group formed by `members` (non-const instructions) plus the constants they
  // read.  Inputs are listed in first-encounter order walking the members producer -> consumer
  // (cinn/hlir/framework/op_lowering_util.cc:79-97); outputs are the members' results used outside or fetched.
  FusedGroupInfo Describe(const std::set<int>& members) const {
    FusedGroupInfo g;
    std::set<int> all = members;
    for (int m : members)
      for (int v : b.instrs()[m].inputs) {
        int p = producer_of_var[v];
        if (p >= 0 && IsConst(p)) all.insert(p);
      }
    std::set<int> seen_inputs;
    std::string name = "fn";
    for (int i : all) {  // std::set iterates in program (topological) order
      const ProgramInstr& ins = b.instrs()[i];
      g.instr_indices.push_back(i);
      if (!IsConst(i) && name.size() < 96) name += "_" + ins.op_type;
      OpDesc od;
      od.type   = ins.op_type;
      od.output = b.vars()[ins.output].id;
      od.attrs  = ins.attrs;
      for (int v : ins.inputs) {
        od.inputs.push_back(b.vars()[v].id);
        int p = producer_of_var[v];
        if ((p < 0 || !all.count(p)) && !seen_inputs.count(v)) {
          seen_inputs.insert(v);
          g.input_vars.push_back(v);
          TensorDesc t;
          t.name  = b.vars()[v].id;
          t.dtype = b.vars()[v].dtype;
          t.shape = b.vars()[v].shape;
          g.desc.inputs.push_back(t);
        }
      }
      g.desc.ops.push_back(od);
    }
    for (int i : members) {
      int v          = b.instrs()[i].output;
      bool external  = fetch.count(v) > 0;
      for (int c : consumers_of_var[v])
        if (!all.count(c) && !recomputed.count(i)) external = true;
      if (external) {
        g.output_vars.push_back(v);
        TensorDesc t;
        t.name  = b.vars()[v].id;
        t.dtype = b.vars()[v].dtype;
        t.shape = b.vars()[v].shape;
        g.desc.outputs.push_back(t);
      }
    }
    // The first instruction that belongs to this group alone names it (a recomputed producer sits in several groups).
    int first_own = *members.begin();
    for (int i : members)
      if (!recomputed.count(i)) {
        first_own = i;
        break;
      }
    g.desc.name = name + "_" + std::to_string(uid) + "_" + std::to_string(first_own);
    return g;
  }

  bool Compiles(const std::set<int>& members, FusedGroupInfo* out, std::string* why) const {
    FusedGroupInfo g = Describe(members);
    if (g.desc.outputs.empty()) {
      if (why) *why = "group would have no output";
      return false;
    }
    std::string err;
    auto plan = CompileGroup(g.desc, dev, &err);
    if (!plan) {
      if (why) *why = err;
      return false;
    }
    g.pattern = plan->pattern;
    for (auto& s : plan->steps) g.kernels.push_back(s.kernel->name);
    if ((g.pattern == "row_program" && g.kernels[0] == "row_program") || (g.pattern == "ew_dag" && g.kernels[0] == "ew_dag")) {
      // Measured on B200: the interpreting register-program kernel runs at 0.3 of the HBM peak and the interpreting
      // row-program kernel at 0.1, their specialised forms at 0.9 and 0.55-0.87.  A region that only an interpreter
      // takes is therefore split into groups for the chain and reduction kernels unless the caller asks otherwise.
      if (!dev.fuse_interpreted_programs) {
        if (why) *why = "only the interpreting program kernel takes this group";
        return false;
      }
    }
    if (g.pattern == "row_program" && g.kernels[0] == "row_program") {
      // The interpreting row-program kernel is worth a group of its own only where it saves a pass over a full-size
      // tensor or a launch per reduction: a per-element result that depends on a reduction (x / ||x||), or several
      // reductions.  One reduction with a per-row epilogue is better served by the dedicated reduction kernels plus
      // a tiny elementwise kernel, unless the library holds a kernel specialised for exactly this program.
      int n_reduce = 0;
      std::set<std::string> after_reduce;  // values computed from a reduction's result
      for (auto& op : g.desc.ops) {
        bool dep = op.type.rfind("reduce_", 0) == 0;
        n_reduce += dep ? 1 : 0;
        for (auto& in : op.inputs) dep = dep || after_reduce.count(in);
        if (dep) after_reduce.insert(op.output);
      }
      int64_t largest_in = 0;
      for (auto& t : g.desc.inputs) largest_in = std::max<int64_t>(largest_in, t.numel());
      bool full_result = false;
      for (auto& t : g.desc.outputs) full_result = full_result || (t.numel() == largest_in && after_reduce.count(t.name));
      if (n_reduce < 2 && !full_result) {
        if (why) *why = "one reduction with a per-row epilogue: left to the reduction kernels";
        return false;
      }
    }
    if (out) *out = std::move(g);
    return true;
  }
};

std::atomic<int> g_computation_uid{0};

}  // namespace

bool FusePasses(const NetBuilder& b, const std::vector<int>& fetch_in, const DeviceInfo& dev,
                std::vector<FusedGroupInfo>* groups, std::string* err) {
  FusionState st(b, dev, g_computation_uid.fetch_add(1));
  const int n = (int)b.instrs().size();
  if (fetch_in.empty()) {
    for (size_t v = 0; v < b.vars().size(); ++v)
      if (st.producer_of_var[v] >= 0 && st.consumers_of_var[v].empty()) st.fetch.insert((int)v);
  } else {
    for (int v : fetch_in) st.fetch.insert(v);
  }
  std::vector<int> group_of(n, -1);
  std::vector<std::set<int>> sets;
  // Instructions that no fetched variable depends on are dropped (they would form groups without an output):
  // the reference prunes them the same way when it builds the graph from the fetch list.
  {
    std::vector<bool> live(n, false);
    std::vector<int> stack;
    for (int v : st.fetch)
      if (st.producer_of_var[v] >= 0) stack.push_back(st.producer_of_var[v]);
    while (!stack.empty()) {
      int i = stack.back();
      stack.pop_back();
      if (live[i]) continue;
      live[i] = true;
      for (int v : b.instrs()[i].inputs)
        if (st.producer_of_var[v] >= 0) stack.push_back(st.producer_of_var[v]);
    }
    for (int i = 0; i < n; ++i)
      if (!live[i]) group_of[i] = -2;  // neither grouped nor available
    for (auto& cons : st.consumers_of_var)
      cons.erase(std::remove_if(cons.begin(), cons.end(), [&](int c) { return !live[c]; }), cons.end());
  }

  // Step 1: connected regions of fusible instructions, tried whole.  This is what lets a multi-reduction
  // composition (softmax, layer_norm) become ONE kernel whatever its row length, where the reference splits at
  // reduce -> broadcast edges longer than 1024 (cinn/hlir/pass/op_fusion_pass_util.h:263-265).
  {
    std::vector<int> comp(n, -1);
    int ncomp = 0;
    for (int i = 0; i < n; ++i) {
      if (comp[i] >= 0 || group_of[i] == -2 || st.IsConst(i) || PatternOf(b.instrs()[i].op_type) == OpPattern::kNonFusible) continue;
      std::vector<int> stack = {i};
      comp[i]                = ncomp;
      while (!stack.empty()) {
        int u = stack.back();
        stack.pop_back();
        auto visit = [&](int w) {
          if (w < 0 || comp[w] >= 0 || group_of[w] == -2 || st.IsConst(w) || PatternOf(b.instrs()[w].op_type) == OpPattern::kNonFusible) return;
          comp[w] = ncomp;
          stack.push_back(w);
        };
        for (int v : b.instrs()[u].inputs) visit(st.producer_of_var[v]);
        for (int c : st.consumers_of_var[b.instrs()[u].output]) visit(c);
      }
      ++ncomp;
    }
    for (int c = 0; c < ncomp; ++c) {
      std::set<int> members;
      for (int i = 0; i < n; ++i)
        if (comp[i] == c) members.insert(i);
      if (members.size() < 2) continue;
      FusedGroupInfo whole;
      const bool whole_compiles = st.Compiles(members, &whole, nullptr);
      // A region that only the interpreting row-program kernel takes as a whole is first searched for a softmax or
      // layer_norm composition inside it (below): those have dedicated kernels several times faster, and the ops
      // around them then run as chains.
      const bool interpreted_rows = whole_compiles && whole.pattern == "row_program" && whole.kernels[0] == "row_program";
      if (whole_compiles && !interpreted_rows) {
        for (int i : members) group_of[i] = (int)sets.size();
        sets.push_back(members);
        continue;
      }
      const size_t sets_before = sets.size();
      // The region as a whole has no kernel, but everything downstream of one of its values may be a composition
      // that has one (a max-subtracted softmax or a layer_norm applied to a computed tensor): such a set is closed
      // under consumers, so it can be a group of its own with that value as an input.
      std::vector<int> fork_vars;  // every value the region reads, program inputs included, in order of first use
      for (int m : members)
        for (int w : b.instrs()[m].inputs)
          if (std::find(fork_vars.begin(), fork_vars.end(), w) == fork_vars.end()) fork_vars.push_back(w);
      for (int v : fork_vars) {
        const int i = st.producer_of_var[v];  // -1: a program input
        if (i >= 0 && (st.IsConst(i) || group_of[i] == -2)) continue;
        int inside  = 0;
        for (int cns : st.consumers_of_var[v]) inside += members.count(cns) ? 1 : 0;
        if (inside < 2) continue;
        std::set<int> down;
        std::vector<int> stack(st.consumers_of_var[v].begin(), st.consumers_of_var[v].end());
        bool clean = true;
        while (!stack.empty() && clean) {
          const int d = stack.back();
          stack.pop_back();
          if (down.count(d)) continue;
          if (!members.count(d) || group_of[d] != -1) {
            clean = false;  // leaves the region, or runs into a group already formed
            break;
          }
          down.insert(d);
          for (int cns : st.consumers_of_var[b.instrs()[d].output]) stack.push_back(cns);
        }
        if (!clean || down.size() < 3) continue;
        // Candidates: everything downstream of v, or - when more follows the composition - the part of it that leads
        // to one instruction z and escapes nowhere else (largest first).
        std::vector<int> ends(down.rbegin(), down.rend());
        for (int z : ends) {
          std::set<int> part;
          std::vector<int> up = {z};
          while (!up.empty()) {
            const int d = up.back();
            up.pop_back();
            if (!down.count(d) || !part.insert(d).second) continue;
            for (int w : b.instrs()[d].inputs) {
              const int pw = st.producer_of_var[w];
              if (pw >= 0) up.push_back(pw);
            }
          }
          bool closed = part.size() >= 3;
          for (int d : part) {
            if (d == z || !closed) continue;
            closed = closed && !st.fetch.count(b.instrs()[d].output);
            for (int cns : st.consumers_of_var[b.instrs()[d].output]) closed = closed && part.count(cns);
          }
          if (!closed) continue;
          // plus what only feeds this set and hangs on nothing computed outside it (the broadcasts of gamma and beta)
          for (bool added = true; added;) {
            added = false;
            for (int q : members) {
              if (part.count(q) || group_of[q] != -1 || q == i) continue;
              bool feeds_only_part = !st.consumers_of_var[b.instrs()[q].output].empty() && !st.fetch.count(b.instrs()[q].output);
              for (int cns : st.consumers_of_var[b.instrs()[q].output]) feeds_only_part = feeds_only_part && part.count(cns);
              bool free_inputs = true;
              for (int w : b.instrs()[q].inputs) {
                const int pw = st.producer_of_var[w];
                free_inputs  = free_inputs && (pw < 0 || st.IsConst(pw) || part.count(pw));
              }
              if (feeds_only_part && free_inputs) {
                part.insert(q);
                added = true;
              }
            }
          }
          // Only the row compositions are taken here (several reductions and their consumers in one kernel); a part
          // that merely is some chain is left to the steps below, which know better where chains should end.
          FusedGroupInfo info;
          if (!st.Compiles(part, &info, nullptr)) continue;
          if (info.pattern != "softmax_row" && info.pattern != "softmax_safe_row" && info.pattern != "layernorm_row") continue;
          for (int d : part) group_of[d] = (int)sets.size();
          sets.push_back(part);
          break;
        }
      }
      if (interpreted_rows && sets.size() == sets_before) {  // no dedicated composition inside: the row program it is
        for (int i : members) group_of[i] = (int)sets.size();
        sets.push_back(members);
      }
    }
  }

  // True if some path leaves `trial` and comes back into it, with every group formed so far taken as one node: the
  // group of `trial` would then depend on a group that depends on it.
  auto leaves_and_reenters = [&](const std::set<int>& trial) {
    std::set<int> seen_instr, seen_group;
    std::vector<int> stack;
    auto push_consumers_of = [&](int i) {
      for (int c : st.consumers_of_var[b.instrs()[i].output])
        if (!trial.count(c)) stack.push_back(c);
    };
    for (int i : trial) push_consumers_of(i);
    while (!stack.empty()) {
      const int c = stack.back();
      stack.pop_back();
      if (group_of[c] == -2 || !seen_instr.insert(c).second) continue;
      std::vector<int> node = {c};
      if (group_of[c] >= 0) {
        if (!seen_group.insert(group_of[c]).second) continue;
        node.assign(sets[group_of[c]].begin(), sets[group_of[c]].end());
      }
      for (int i : node) {
        seen_instr.insert(i);
        for (int d : st.consumers_of_var[b.instrs()[i].output]) {
          if (trial.count(d)) return true;
          stack.push_back(d);
        }
      }
    }
    return false;
  };

  // Step 2: vertical fusion, consumer first (the reference walks the graph in reverse topological order,
  // cinn/hlir/pass/op_fusion_pass.cc:94-95): a producer joins its consumer's group when all of its uses are
  // inside the group and a kernel exists for the enlarged group.
  for (int root = n - 1; root >= 0; --root) {
    if (group_of[root] != -1 || st.IsConst(root)) continue;
    std::set<int> members = {root};
    bool grew             = PatternOf(b.instrs()[root].op_type) != OpPattern::kNonFusible;
    while (grew) {
      grew = false;
      for (int m : std::set<int>(members)) {
        for (int v : b.instrs()[m].inputs) {
          int p = st.producer_of_var[v];
          if (p < 0 || members.count(p) || group_of[p] >= 0 || st.IsConst(p)) continue;
          if (PatternOf(b.instrs()[p].op_type) == OpPattern::kNonFusible) continue;
          bool all_inside = !st.fetch.count(b.instrs()[p].output);
          for (int c : st.consumers_of_var[b.instrs()[p].output])
            if (!members.count(c)) all_inside = false;
          std::set<int> trial = members;
          trial.insert(p);
          if (!all_inside) {
            // The producer's result is needed outside as well (fetched, or read by another group): it may still join
            // as a second output of the group (the reference's groups keep such values as output nodes,
            // cinn/hlir/framework/op_lowering.cc:121-151) when a kernel exists for the two-output group and no other
            // group ends up both behind and in front of this one.
            if (!leaves_and_reenters(trial) && st.Compiles(trial, nullptr, nullptr)) {
              members = trial;
              grew    = true;
            }
            continue;
          }
          if (st.Compiles(trial, nullptr, nullptr)) {
            members = trial;
            grew    = true;
            continue;
          }
          // The producer alone does not give a known group; try it together with the producers that feed only
          // it (e.g. multiply(x, identity(x)) under a reduce_sum needs the identity as well).
          std::set<int> closure = trial;
          bool added            = true;
          while (added && closure.size() < trial.size() + 8) {
            added = false;
            for (int m2 : std::set<int>(closure)) {
              if (members.count(m2)) continue;
              for (int v2 : b.instrs()[m2].inputs) {
                int q = st.producer_of_var[v2];
                if (q < 0 || closure.count(q) || group_of[q] >= 0 || st.IsConst(q)) continue;
                if (PatternOf(b.instrs()[q].op_type) == OpPattern::kNonFusible) continue;
                if (st.fetch.count(b.instrs()[q].output)) continue;
                bool inside = true;
                for (int c : st.consumers_of_var[b.instrs()[q].output])
                  if (!closure.count(c)) inside = false;
                if (!inside) continue;
                closure.insert(q);
                added = true;
              }
            }
          }
          if (closure.size() > trial.size() && st.Compiles(closure, nullptr, nullptr)) {
            members = closure;
            grew    = true;
            continue;
          }
          // The same without the casts at its leaves: a cast that widens one 16-bit operand while another operand
          // (widened by a cast with further users) is still float32 gives a mixed group no kernel takes; the casts
          // join after the horizontal merge, when all of them can come in together.
          {
            std::set<int> inner = closure;
            for (int q : closure) {
              if (trial.count(q) || b.instrs()[q].op_type != "cast") continue;
              const int src = st.producer_of_var[b.instrs()[q].inputs[0]];
              if (src < 0 || !closure.count(src)) inner.erase(q);
            }
            if (inner.size() < closure.size() && inner.size() > trial.size() && st.Compiles(inner, nullptr, nullptr)) {
              members = inner;
              grew    = true;
              continue;
            }
          }
          // Last attempt: everything upstream of the whole group that is used only inside it, at once.  Some
          // compositions only have a kernel as a whole (the normalisation of batch_norm_train needs x - mean and
          // rsqrt(var + eps) together; either alone leaves too many full-size operands).
          std::set<int> big = trial;
          added             = true;
          while (added && big.size() < trial.size() + 32) {
            added = false;
            for (int m2 : std::set<int>(big)) {
              for (int v2 : b.instrs()[m2].inputs) {
                int q = st.producer_of_var[v2];
                if (q < 0 || big.count(q) || group_of[q] >= 0 || st.IsConst(q)) continue;
                if (PatternOf(b.instrs()[q].op_type) == OpPattern::kNonFusible) continue;
                if (st.fetch.count(b.instrs()[q].output)) continue;
                bool inside = true;
                for (int c : st.consumers_of_var[b.instrs()[q].output])
                  if (!big.count(c)) inside = false;
                if (!inside) continue;
                big.insert(q);
                added = true;
              }
            }
          }
          if (big.size() > closure.size() && st.Compiles(big, nullptr, nullptr)) {
            members = big;
            grew    = true;
          }
        }
      }
    }
    for (int i : members) group_of[i] = (int)sets.size();
    sets.push_back(members);
  }

  // Step 3: horizontal fusion of reduction groups that read the same tensor and do not depend on one another
  // (cinn/hlir/pass/fusion_merge_pass.cc:85-460), kept when a kernel exists for the merged, multi-output group:
  // the two channel reductions of batch_norm_train become one pass over x.
  {
    auto is_reduce_group = [&](const std::set<int>& m) {
      for (int i : m)
        if (PatternOf(b.instrs()[i].op_type) == OpPattern::kReduction) return true;
      return false;
    };
    for (size_t i = 0; i < sets.size(); ++i) {
      if (sets[i].empty() || !is_reduce_group(sets[i])) continue;
      FusedGroupInfo gi = st.Describe(sets[i]);
      // All the reduction groups that share an input with this one and are independent of it, at once (the merged
      // group may have a kernel where a pair on the way to it has none), then one by one.
      {
        std::vector<size_t> cands;
        for (size_t j = i + 1; j < sets.size(); ++j) {
          if (sets[j].empty() || !is_reduce_group(sets[j])) continue;
          const FusedGroupInfo gj = st.Describe(sets[j]);
          bool shared = false, dependent = false;
          for (int v : gj.input_vars) {
            shared = shared || std::find(gi.input_vars.begin(), gi.input_vars.end(), v) != gi.input_vars.end();
            dependent = dependent || std::find(gi.output_vars.begin(), gi.output_vars.end(), v) != gi.output_vars.end();
          }
          for (int v : gi.input_vars)
            dependent = dependent || std::find(gj.output_vars.begin(), gj.output_vars.end(), v) != gj.output_vars.end();
          if (shared && !dependent) cands.push_back(j);
        }
        if (cands.size() >= 2) {
          std::set<int> merged = sets[i];
          for (size_t j : cands) merged.insert(sets[j].begin(), sets[j].end());
          if (st.Compiles(merged, nullptr, nullptr)) {
            for (size_t j : cands) {
              for (int k : sets[j]) group_of[k] = (int)i;
              sets[j].clear();
            }
            sets[i] = merged;
            gi      = st.Describe(sets[i]);
          }
        }
      }
      for (size_t j = i + 1; j < sets.size(); ++j) {
        if (sets[j].empty() || !is_reduce_group(sets[j])) continue;
        const FusedGroupInfo gj = st.Describe(sets[j]);
        bool shared = false, dependent = false;
        for (int v : gj.input_vars) {
          shared = shared || std::find(gi.input_vars.begin(), gi.input_vars.end(), v) != gi.input_vars.end();
          dependent = dependent || std::find(gi.output_vars.begin(), gi.output_vars.end(), v) != gi.output_vars.end();
        }
        for (int v : gi.input_vars)
          dependent = dependent || std::find(gj.output_vars.begin(), gj.output_vars.end(), v) != gj.output_vars.end();
        if (!shared || dependent) continue;
        std::set<int> merged = sets[i];
        merged.insert(sets[j].begin(), sets[j].end());
        if (!st.Compiles(merged, nullptr, nullptr)) continue;
        for (int k : sets[j]) group_of[k] = (int)i;
        sets[i] = merged;
        sets[j].clear();
        // The merged group may now hold every user of a producer that vertical fusion had to leave outside (the cast
        // that widens a 16-bit x feeds both statistics): pull such single-instruction producers in.
        {
          std::vector<int> eligible;
          for (int m : sets[i]) {
            for (int v : b.instrs()[m].inputs) {
              const int p = st.producer_of_var[v];
              if (p < 0 || group_of[p] < 0 || group_of[p] == (int)i || sets[group_of[p]].size() != 1) continue;
              if (st.IsConst(p) || PatternOf(b.instrs()[p].op_type) == OpPattern::kNonFusible) continue;
              if (st.fetch.count(b.instrs()[p].output)) continue;
              bool all_inside = true;
              for (int c : st.consumers_of_var[b.instrs()[p].output])
                if (!sets[i].count(c)) all_inside = false;
              if (all_inside && std::find(eligible.begin(), eligible.end(), p) == eligible.end()) eligible.push_back(p);
            }
          }
          auto take = [&](const std::vector<int>& ps) {
            std::set<int> trial = sets[i];
            trial.insert(ps.begin(), ps.end());
            if (ps.empty() || !st.Compiles(trial, nullptr, nullptr)) return false;
            for (int p : ps) {
              sets[group_of[p]].clear();
              group_of[p] = (int)i;
            }
            sets[i] = trial;
            return true;
          };
          if (!take(eligible))  // all at once (two casts of one 16-bit type), else one by one
            for (int p : eligible) take({p});
        }
        gi = st.Describe(sets[i]);  // further reductions over the same tensors may join as well
      }
    }
  }

  // Step 4: horizontal fusion of elementwise groups that read the same tensor (the same pass of the reference): two
  // groups become one two-output group when a kernel exists for it (the chain kernel evaluates one expression,
  // stores it, and restarts for the other) and no other group ends up both behind and in front of the merged one.
  {
    auto plain_elementwise = [&](const std::set<int>& m) {
      for (int i : m) {
        const OpPattern p = PatternOf(b.instrs()[i].op_type);
        if (p == OpPattern::kReduction || p == OpPattern::kNonFusible) return false;
      }
      return !m.empty();
    };
    for (size_t i = 0; i < sets.size(); ++i) {
      if (!plain_elementwise(sets[i])) continue;
      for (size_t j = i + 1; j < sets.size(); ++j) {
        if (!plain_elementwise(sets[j])) continue;
        const FusedGroupInfo gi = st.Describe(sets[i]), gj = st.Describe(sets[j]);
        if (gi.output_vars.size() != 1 || gj.output_vars.size() != 1) continue;
        if (b.vars()[gi.output_vars[0]].shape != b.vars()[gj.output_vars[0]].shape) continue;
        bool shared = false;
        for (int v : gj.input_vars)
          shared = shared || std::find(gi.input_vars.begin(), gi.input_vars.end(), v) != gi.input_vars.end();
        if (!shared) continue;
        std::set<int> merged = sets[i];
        merged.insert(sets[j].begin(), sets[j].end());
        if (leaves_and_reenters(merged) || !st.Compiles(merged, nullptr, nullptr)) continue;
        for (int k : sets[j]) group_of[k] = (int)i;
        sets[i] = merged;
        sets[j].clear();
        break;  // a group has two outputs at most
      }
    }
  }

  // Step 5: recomputation.  A small elementwise group whose result several other groups read (bias + bias feeding
  // two sums of different shapes, x + y feeding a row and a column reduction) is evaluated again inside each of
  // them instead of being written to memory and read back, when every reader has a kernel for the enlarged group:
  // the reference's merge pass fuses such a producer into all of its consumers the same way
  // (cinn/hlir/pass/fusion_merge_pass.cc:605-700, vertical fusion with recompute).  Only producers that read nothing
  // but program inputs and constants are moved, so no ordering between groups changes.
  for (size_t si = 0; si < sets.size(); ++si) {
    const std::set<int>& S = sets[si];
    if (S.empty() || S.size() > 4) continue;
    bool movable = true;
    for (int i : S) {
      const OpPattern pat = PatternOf(b.instrs()[i].op_type);
      movable = movable && pat != OpPattern::kReduction && pat != OpPattern::kNonFusible && b.instrs()[i].op_type != "reshape";
      for (int v : b.instrs()[i].inputs) {
        const int pv = st.producer_of_var[v];
        movable      = movable && (pv < 0 || st.IsConst(pv) || S.count(pv));
      }
    }
    if (!movable) continue;
    const FusedGroupInfo gs = st.Describe(S);
    if (gs.output_vars.size() != 1 || st.fetch.count(gs.output_vars[0])) continue;
    const int v = gs.output_vars[0];
    int64_t v_numel = 1;
    for (auto d : b.vars()[v].shape) v_numel *= d;
    std::set<int> readers;
    bool ok = true;
    for (int c : st.consumers_of_var[v]) {
      if (S.count(c)) continue;
      if (group_of[c] < 0 || sets[group_of[c]].empty()) ok = false;
      else readers.insert(group_of[c]);
    }
    if (!ok || readers.size() < 2) continue;
    // tentatively: the producer's instructions count as present in every reader
    for (int i : S) st.recomputed.insert(i);
    std::vector<std::set<int>> enlarged;
    for (int r : readers) {
      std::set<int> trial = sets[r];
      trial.insert(S.begin(), S.end());
      FusedGroupInfo info;
      bool fits = st.Compiles(trial, &info, nullptr);
      // never recompute a larger tensor than the reader produces
      for (int ov : info.output_vars) {
        int64_t n_out = 1;
        for (auto d : b.vars()[ov].shape) n_out *= d;
        fits = fits && (v_numel <= n_out || PatternOf(b.instrs()[st.producer_of_var[ov]].op_type) == OpPattern::kReduction);
      }
      if (!fits) {
        ok = false;
        break;
      }
      enlarged.push_back(trial);
    }
    if (!ok) {
      for (int i : S) st.recomputed.erase(i);
      continue;
    }
    size_t k = 0;
    for (int r : readers) sets[r] = enlarged[k++];
    for (int i : S) group_of[i] = -3;  // lives in several groups
    sets[si].clear();
  }

  // Emit in a topological order of the groups (a group after the groups that produce its inputs), ties by program
  // order; every group must compile.
  std::vector<int> order;
  {
    const int ng = (int)sets.size();
    std::vector<std::set<int>> deps(ng);
    for (int gidx = 0; gidx < ng; ++gidx)
      for (int i : sets[gidx])
        for (int v : b.instrs()[i].inputs) {
          const int p = st.producer_of_var[v];
          if (p >= 0 && group_of[p] >= 0 && group_of[p] != gidx) deps[gidx].insert(group_of[p]);
        }
    std::vector<bool> done(ng, false);
    for (int emitted = 0; emitted < ng;) {
      int pick = -1;
      for (int gidx = 0; gidx < ng; ++gidx) {
        if (done[gidx]) continue;
        if (sets[gidx].empty()) {
          done[gidx] = true;
          ++emitted;
          continue;
        }
        bool ready = true;
        for (int d : deps[gidx]) ready = ready && done[d];
        if (ready && (pick < 0 || *sets[gidx].begin() < *sets[pick].begin())) pick = gidx;
      }
      if (pick < 0) {
        for (int gidx = 0; gidx < ng; ++gidx)
          if (!done[gidx] && !sets[gidx].empty()) {
            if (err) *err = "internal error: the fused groups depend on one another";
            return false;
          }
        break;  // only empty sets were left
      }
      done[pick] = true;
      ++emitted;
      order.push_back(pick);
    }
  }
  groups->clear();
  for (int gi : order) {
    FusedGroupInfo info;
    std::string why;
    if (sets[gi].size() == 1 && b.instrs()[*sets[gi].begin()].op_type == "reshape") {
      // A reshape is not a kernel: its result aliases its operand's memory (graph_compiler.cc:1017-1027).
      info         = st.Describe(sets[gi]);
      info.pattern = "reshape_alias";
      if (info.desc.outputs.empty()) {
        const ProgramInstr& ins = b.instrs()[*sets[gi].begin()];
        info.output_vars.push_back(ins.output);
      }
      groups->push_back(std::move(info));
      continue;
    }
    if (!st.Compiles(sets[gi], &info, &why)) {
      if (err) *err = "no prebuilt kernel for instruction group {" + PrintGroupDesc(st.Describe(sets[gi]).desc) + "}: " + why;
      return false;
    }
    groups->push_back(std::move(info));
  }
  return true;
}

// ---- Computation ----------------------------------------------------------------------------------------
namespace {

cinn_type_t RuntimeType(DType t) {
  cinn_type_t r;
  r.lanes         = 1;
  r.num_asterisks = 0;
  switch (t) {
    case DType::kFloat32: r.code = cinn_type_float; r.bits = 32; break;
    case DType::kFloat16: r.code = cinn_type_float; r.bits = 16; break;
    case DType::kBFloat16: r.code = cinn_type_bfloat; r.bits = 16; break;
    case DType::kFloat64: r.code = cinn_type_float; r.bits = 64; break;
    case DType::kInt32: r.code = cinn_type_int; r.bits = 32; break;
    case DType::kInt64: r.code = cinn_type_int; r.bits = 64; break;
    case DType::kBool: r.code = cinn_type_int; r.bits = 1; break;
    case DType::kUInt8: r.code = cinn_type_uint; r.bits = 8; break;
    default: r.code = cinn_type_unk; r.bits = 0; break;
  }
  return r;
}

int Fail(std::string* err, const std::string& m, int code = CINN_B200_EINVAL) {
  if (err) *err = m;
  return code;
}

}  // namespace

std::unique_ptr<Computation> Computation::BuildAndCompile(const NetBuilder& b, const std::vector<int>& fetch,
                                                          int device, std::string* err) {
  std::unique_ptr<Computation> c(new Computation());
  c->device_ = device;
  DeviceInfo dev = CurrentDeviceInfo();  // the planner options apply to the fusion pass's trial compilations too
  if (device >= 0) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
      if (err) *err = std::string("cudaSetDevice: ") + cudaGetErrorString(e);
      return nullptr;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && sms > 0) dev.sm_count = sms;
  }
  if (!FusePasses(b, fetch, dev, &c->groups_, err)) return nullptr;
  // Scope: one tensor per variable that crosses a group boundary (cinn/hlir/framework/graph_compiler.cc:1430-1451).
  auto add_tensor = [&](int v) { c->AddScopeTensor(b.vars()[v]); };
  for (auto& g : c->groups_) {
    for (int v : g.input_vars) add_tensor(v);
    for (int v : g.output_vars) add_tensor(v);
  }
  // Compile every group into the library's registry and keep the entry points (parallel_compiler.cc:201-217).
  for (auto& g : c->groups_) {
    if (g.pattern == "reshape_alias") {
      c->aliases_.push_back({b.vars()[g.output_vars[0]].id, b.vars()[g.input_vars[0]].id});
      continue;
    }
    lower_func_ptr_g fn = nullptr;
    int rc              = cinn_b200_compile_group(PrintGroupDesc(g.desc).c_str(), &fn);
    if (rc != CINN_B200_OK) {
      if (err) *err = cinn_b200_last_error();
      return nullptr;
    }
    Instr ins;
    ins.fn      = fn;
    ins.fn_name = g.desc.name;
    for (int v : g.input_vars) ins.args.push_back(b.vars()[v].id);
    for (int v : g.output_vars) ins.args.push_back(b.vars()[v].id);
    c->instrs_.push_back(std::move(ins));
  }
  if (device >= 0 && !c->AllocateScope(err)) return nullptr;
  return c;
}

void Computation::AddScopeTensor(const Variable& var) {
  if (scope_.count(var.id)) return;
  auto t    = std::make_unique<ScopeTensor>();
  t->var    = var;
  memset(&t->buffer, 0, sizeof(t->buffer));
  t->buffer.device     = cinn_unk_device;
  t->buffer.flag       = cinn_buffer_on_device;
  t->buffer.type       = RuntimeType(var.dtype);
  t->buffer.dimensions = (int32_t)var.shape.size();
  int64_t n            = 1;
  for (size_t i = 0; i < var.shape.size(); ++i) {
    t->buffer.dims[i] = (cinn_dimension_t)var.shape[i];
    n *= var.shape[i];
  }
  t->bytes              = (size_t)n * DTypeBytes(var.dtype);
  t->buffer.memory_size = t->bytes;
  names_.push_back(var.id);
  scope_[var.id] = std::move(t);
}

// cinn/hlir/framework/memory.cc:43-52: device memory from cudaMalloc, owned by the scope (alias results own none).
bool Computation::AllocateScope(std::string* err) {
  std::set<std::string> alias_outputs;
  for (auto& a : aliases_) alias_outputs.insert(a.first);
  for (auto& kv : scope_) {
    if (alias_outputs.count(kv.first)) continue;
    void* p       = nullptr;
    cudaError_t e = cudaMalloc(&p, std::max<size_t>(kv.second->bytes, 16));
    if (e != cudaSuccess) {
      if (err) *err = "cudaMalloc of tensor " + kv.first + ": " + cudaGetErrorString(e);
      return false;
    }
    kv.second->buffer.memory = static_cast<uint8_t*>(p);
    kv.second->owned         = true;
  }
  return true;
}

std::string Computation::Export() const {
  std::ostringstream os;
  os << "cinn_b200_program 1\n";
  for (auto& name : names_) {
    const Variable& v = scope_.at(name)->var;
    os << "tensor " << v.id << " " << DTypeName(v.dtype) << " ";
    for (size_t i = 0; i < v.shape.size(); ++i) os << (i ? "," : "") << v.shape[i];
    os << "\n";
  }
  for (auto& g : groups_) {
    if (g.pattern == "reshape_alias") continue;
    os << "begin_group\n" << PrintGroupDesc(g.desc) << "end_group\n";
  }
  for (auto& a : aliases_) os << "alias " << a.first << " " << a.second << "\n";
  return os.str();
}

std::unique_ptr<Computation> Computation::Load(const std::string& text, int device, std::string* err) {
  auto fail = [&](const std::string& m) {
    if (err) *err = "load: " + m;
    return nullptr;
  };
  std::unique_ptr<Computation> c(new Computation());
  c->device_ = device;
  if (device >= 0) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(std::string("cudaSetDevice: ") + cudaGetErrorString(e));
  }
  std::istringstream is(text);
  std::string line;
  if (!std::getline(is, line) || line != "cinn_b200_program 1") return fail("not a program of this library (bad first line)");
  while (std::getline(is, line)) {
    if (line.empty()) continue;
    std::istringstream ls(line);
    std::string word;
    ls >> word;
    if (word == "tensor") {
      Variable v;
      std::string dt, shape;
      ls >> v.id >> dt >> shape;
      v.dtype = DTypeFromName(dt);
      if (v.id.empty() || v.dtype == DType::kUnknown) return fail("bad tensor line: " + line);
      v.shape = ParseIntList(shape);
      c->AddScopeTensor(v);
    } else if (word == "alias") {
      std::string a, b2;
      ls >> a >> b2;
      if (!c->scope_.count(a) || !c->scope_.count(b2)) return fail("alias of an unknown tensor: " + line);
      c->aliases_.push_back({a, b2});
    } else if (word == "begin_group") {
      std::string body;
      bool closed = false;
      while (std::getline(is, line)) {
        if (line == "end_group") {
          closed = true;
          break;
        }
        body += line + "\n";
      }
      if (!closed) return fail("group without end_group");
      FusedGroupInfo g;
      std::string e;
      if (!ParseGroupDesc(body, &g.desc, &e)) return fail(e);
      for (auto& t : g.desc.inputs)
        if (!c->scope_.count(t.name)) return fail("group " + g.desc.name + " reads the unknown tensor " + t.name);
      for (auto& t : g.desc.outputs)
        if (!c->scope_.count(t.name)) return fail("group " + g.desc.name + " writes the unknown tensor " + t.name);
      // A name of its own: the computation that exported the program may still be alive in this process, and the
      // entry-point registry is keyed by name.
      g.desc.name += "_ld" + std::to_string(g_computation_uid.fetch_add(1));
      lower_func_ptr_g fn = nullptr;
      if (cinn_b200_compile_group(PrintGroupDesc(g.desc).c_str(), &fn) != CINN_B200_OK) return fail(cinn_b200_last_error());
      char pattern[128] = {0};
      long long bytes = 0, elements = 0, scratch = 0;
      int launches = 0;
      cinn_b200_group_info(g.desc.name.c_str(), pattern, sizeof(pattern), &bytes, &elements, &launches, &scratch);
      g.pattern = pattern;
      for (int k = 0; k < launches; ++k) {
        char kn[128] = {0};
        if (cinn_b200_group_kernel(g.desc.name.c_str(), k, kn, sizeof(kn)) == CINN_B200_OK) g.kernels.push_back(kn);
      }
      Instr ins;
      ins.fn      = fn;
      ins.fn_name = g.desc.name;
      for (auto& t : g.desc.inputs) ins.args.push_back(t.name);
      for (auto& t : g.desc.outputs) ins.args.push_back(t.name);
      c->instrs_.push_back(std::move(ins));
      c->groups_.push_back(std::move(g));
    } else {
      return fail("unknown line: " + line);
    }
  }
  if (device >= 0 && !c->AllocateScope(err)) return nullptr;
  return c;
}

Computation::~Computation() {
  if (graph_exec_) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec_));
  for (auto& ins : instrs_) cinn_b200_release_group(ins.fn_name.c_str());
  if (device_ >= 0) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device_);
    for (auto& kv : scope_)
      if (kv.second->owned && kv.second->buffer.memory) cudaFree(kv.second->buffer.memory);
    cudaSetDevice(prev);
  }
}

ScopeTensor* Computation::Find(const std::string& id) {
  auto it = scope_.find(id);
  return it == scope_.end() ? nullptr : it->second.get();
}

int Computation::BindTensor(const std::string& id, void* device_ptr, std::string* err) {
  ScopeTensor* t = Find(id);
  if (!t) return Fail(err, "no tensor named '" + id + "'", CINN_B200_ENOTFOUND);
  if (!device_ptr) return Fail(err, "null device pointer for tensor '" + id + "'");
  if (t->owned && t->buffer.memory) {
    cudaFree(t->buffer.memory);
    t->owned = false;
  }
  t->buffer.memory = static_cast<uint8_t*>(device_ptr);
  if (graph_exec_) {  // the captured graph holds the old address
    cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph_exec_));
    graph_exec_ = nullptr;
  }
  return CINN_B200_OK;
}

int Computation::SetTensorData(const std::string& id, const void* host, size_t bytes, std::string* err) {
  ScopeTensor* t = Find(id);
  if (!t) return Fail(err, "no tensor named '" + id + "'", CINN_B200_ENOTFOUND);
  if (bytes != t->bytes) return Fail(err, "tensor '" + id + "' holds " + std::to_string(t->bytes) + " bytes, got " + std::to_string(bytes), CINN_B200_ESHAPE);
  if (!t->buffer.memory) return Fail(err, "tensor '" + id + "' has no device memory (planned without a device)");
  cudaError_t e = cudaMemcpy(t->buffer.memory, host, bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) return Fail(err, std::string("host->device copy: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
  return CINN_B200_OK;
}

int Computation::GetTensorData(const std::string& id, void* host, size_t bytes, std::string* err) {
  ScopeTensor* t = Find(id);
  if (!t) return Fail(err, "no tensor named '" + id + "'", CINN_B200_ENOTFOUND);
  if (bytes != t->bytes) return Fail(err, "tensor '" + id + "' holds " + std::to_string(t->bytes) + " bytes, got " + std::to_string(bytes), CINN_B200_ESHAPE);
  if (!t->buffer.memory) return Fail(err, "tensor '" + id + "' has no device memory (planned without a device)");
  cudaError_t e = cudaMemcpy(host, t->buffer.memory, bytes, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return Fail(err, std::string("device->host copy: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
  return CINN_B200_OK;
}

int Computation::Execute(void* stream, std::string* err) {
  if (device_ < 0) return Fail(err, "this computation was planned without a device");
  // Instruction::UpdateArgsCache (instruction.cc:77-106): pod arrays are built once and reused.
  if (!args_cached_) {
    for (auto& ins : instrs_) {
      ins.pods.resize(ins.args.size());
      for (size_t i = 0; i < ins.args.size(); ++i) {
        ScopeTensor* t              = Find(ins.args[i]);
        ins.pods[i].type_code_      = CINN_POD_BUFFERP;
        ins.pods[i].value_.v_handle = &t->buffer;
      }
    }
    args_cached_ = true;
  }
  for (auto& a : aliases_) Find(a.first)->buffer.memory = Find(a.second)->buffer.memory;
  for (auto& ins : instrs_) {
    int rc = cinn_b200_group_run(ins.fn_name.c_str(), ins.pods.data(), (int)ins.pods.size(), stream);
    if (rc != CINN_B200_OK) return Fail(err, cinn_b200_last_error(), rc);
  }
  // Program::Execute synchronises only when no stream was given (graph_compiler.cc:216-221).
  if (stream == nullptr) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return Fail(err, std::string("cudaDeviceSynchronize: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
  }
  return CINN_B200_OK;
}

// Program::ExecuteTest (cinn/hlir/framework/graph_compiler.cc:224-244): 100 untimed runs, then `repeat` runs timed on
// the host clock up to a device synchronisation; the average per run in milliseconds.
int Computation::ExecuteGraph(void* stream_v, std::string* err) {
  if (device_ < 0) return Fail(err, "this computation was planned without a device");
  if (!stream_v) return Fail(err, "ExecuteGraph needs a stream (capture is not possible on the NULL stream)");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (!graph_exec_) {
    int rc = Execute(stream, err);  // ordinary run first: allocations (scratch) must not happen inside a capture
    if (rc != CINN_B200_OK) return rc;
    cudaError_t e = cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal);
    if (e != cudaSuccess) return Fail(err, std::string("cudaStreamBeginCapture: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
    rc = Execute(stream, err);
    cudaGraph_t graph = nullptr;
    e                 = cudaStreamEndCapture(stream, &graph);
    if (rc != CINN_B200_OK || e != cudaSuccess || !graph) {
      if (graph) cudaGraphDestroy(graph);
      return rc != CINN_B200_OK ? rc : Fail(err, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
    }
    cudaGraphExec_t exec = nullptr;
    e                    = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return Fail(err, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
    graph_exec_ = exec;
    return CINN_B200_OK;  // the capture pass did not run the kernels; the ordinary run above produced this call's results
  }
  cudaError_t e = cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph_exec_), stream);
  if (e != cudaSuccess) return Fail(err, std::string("cudaGraphLaunch: ") + cudaGetErrorString(e), CINN_B200_ECUDA);
  return CINN_B200_OK;
}

int Computation::ExecuteTest(int repeat, double* avg_ms, std::string* err, bool use_graph) {
  if (repeat <= 0) return Fail(err, "repeat must be positive");
  cudaStream_t stream = nullptr;
  if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess) return Fail(err, "cudaStreamCreate failed", CINN_B200_ECUDA);
  int rc = CINN_B200_OK;
  for (int i = 0; i < 100 && rc == CINN_B200_OK; ++i) rc = use_graph ? ExecuteGraph(stream, err) : Execute(stream, err);
  cudaStreamSynchronize(stream);
  const auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < repeat && rc == CINN_B200_OK; ++i) rc = use_graph ? ExecuteGraph(stream, err) : Execute(stream, err);
  cudaStreamSynchronize(stream);
  const auto t1 = std::chrono::steady_clock::now();
  cudaStreamDestroy(stream);
  if (rc != CINN_B200_OK) return rc;
  if (avg_ms) *avg_ms = std::chrono::duration<double, std::milli>(t1 - t0).count() / repeat;
  return CINN_B200_OK;
}

}  // namespace cinn_b200
