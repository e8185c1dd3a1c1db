// Program passes: rewrites of the instruction list between the builder and the fusion pass.
//
// What the reference does in cinn/frontend/pass/*.cc behind ProgramPass::Apply (cinn/frontend/program_pass.h:36-105),
// which frontend::Optimize runs with the list of DefaultTrainingOptimizeOptions (cinn/frontend/optimize.cc:44-82) for
// Program.apply_pass / Program.build_and_get_output (cinn/pybind/frontend.cc:157-242):
//   AutoCast          cinn/frontend/pass/auto_cast.cc:31-214     fp16 / bf16 operands of listed ops computed in fp32
//   AutoBroadcast     cinn/frontend/pass/auto_broadcast.cc:32-125 explicit broadcast_to in front of binary ops
//   CastCollapsing    cinn/frontend/pass/cast_collapsing.cc:50-301 chains of casts folded into one
//   TransposeCollapsing cinn/frontend/pass/transpose_collapsing.cc:60-340 chains of transposes folded into one
//   RemoveIdentity    cinn/frontend/pass/remove_identity.cc:23-262 ops that change nothing removed
//   Decomposer        cinn/frontend/pass/decomposer.cc + cinn/frontend/decomposer/*.cc  gelu, softmax, batch_norm into primitives
//   FillConstantRewriter / FillConstantFolding  cinn/frontend/pass/fill_constant_rewriter.cc, fill_constant_folding.cc
//   DeadCodeEliminate cinn/frontend/pass/dead_code_eliminate.cc   instructions no fetched variable depends on removed
// Each pass here rebuilds the builder's instruction list in place; the variable table only grows, so variable indices
// held by the caller (the fetch list, Python Variable objects) stay valid.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <map>
#include <functional>
#include <set>
#include <sstream>

#include "frontend.h"

namespace cinn_b200 {
namespace {

bool IsHalf(DType t) { return t == DType::kFloat16 || t == DType::kBFloat16; }

std::vector<int64_t> IntList(const std::string& text) {
  std::vector<int64_t> out;
  std::stringstream ss(text);
  std::string item;
  while (std::getline(ss, item, ','))
    if (!item.empty()) out.push_back(atoll(item.c_str()));
  return out;
}

std::string JoinList(const std::vector<int64_t>& v) {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
  return s;
}

ProgramInstr CastInto(int from, int to, DType dtype) {
  ProgramInstr c;
  c.op_type = "cast";
  c.inputs  = {from};
  c.output  = to;
  c.attrs   = {{"dtype", DTypeName(dtype)}};
  return c;
}

// ---- AutoCast ----------------------------------------------------------------------------------------
// The ops of the reference's need_cast_list that exist here (auto_cast.cc:78-108).  For batch_norm only x is cast:
// its four parameter vectors must be float32 already (auto_cast.cc:109-137).
const std::set<std::string>& NeedCastOps() {
  static const std::set<std::string> s = {"sin", "cos", "exp", "log", "log2", "log10", "sqrt", "rsqrt", "cbrt", "erf",
                                          "sinh", "cosh", "tanh", "asin", "acos", "atan", "asinh", "acosh", "atanh",
                                          "remainder", "pow", "reduce_sum", "reduce_prod", "sigmoid", "softmax", "gelu",
                                          "batch_norm"};
  return s;
}

bool AutoCast(NetBuilder* b, std::string* err) {
  const std::vector<ProgramInstr> old = b->TakeInstrs();
  for (const ProgramInstr& ins : old) {
    bool half_in = false;
    for (int v : ins.inputs) half_in = half_in || IsHalf(b->vars()[v].dtype);
    if (!NeedCastOps().count(ins.op_type) || !half_in) {
      b->AppendInstr(ins);
      continue;
    }
    std::vector<int> casted = ins.inputs;
    if (ins.op_type == "batch_norm") {
      for (size_t k = 1; k < ins.inputs.size(); ++k)
        if (b->vars()[ins.inputs[k]].dtype != DType::kFloat32) {
          if (err) *err = "AutoCast: batch_norm's scale, bias, mean and variance must be float32";
          return false;
        }
    }
    for (size_t k = 0; k < casted.size(); ++k) {
      if (!IsHalf(b->vars()[casted[k]].dtype) || (ins.op_type == "batch_norm" && k > 0)) continue;
      casted[k] = b->AddOp("cast", {casted[k]}, {{"dtype", "float32"}}, err);
      if (casted[k] < 0) return false;
    }
    const int wide = b->AddOp(ins.op_type, casted, ins.attrs, err);
    if (wide < 0) return false;
    const DType narrow = b->vars()[ins.output].dtype;
    if (b->vars()[wide].dtype == DType::kFloat32) {
      b->AppendInstr(CastInto(wide, ins.output, narrow));
    } else {
      ProgramInstr keep;
      keep.op_type = "identity";
      keep.inputs  = {wide};
      keep.output  = ins.output;
      b->AppendInstr(keep);
    }
  }
  return true;
}

// ---- AutoBroadcast -----------------------------------------------------------------------------------
bool AutoBroadcast(NetBuilder* b, std::string* err) {
  const std::vector<ProgramInstr> old = b->TakeInstrs();
  for (ProgramInstr ins : old) {
    if (!IsBinaryBroadcastOp(ins.op_type) || ins.inputs.size() <= 1) {
      b->AppendInstr(ins);
      continue;
    }
    const std::vector<int64_t> out_shape = b->vars()[ins.output].shape;
    int64_t axis = ins.attrs.count("axis") ? atoll(ins.attrs.at("axis").c_str()) : -1;
    bool inserted = false;
    for (int& v : ins.inputs) {
      const std::vector<int64_t> shape = b->vars()[v].shape;
      if (shape == out_shape) continue;
      // auto_broadcast.cc:37-58: same rank => every axis in place, otherwise `axis` (or right-aligned) onwards
      std::vector<int64_t> axes;
      if (shape.size() == out_shape.size()) {
        for (size_t i = 0; i < shape.size(); ++i) axes.push_back((int64_t)i);
      } else {
        int64_t a = axis == -1 ? (int64_t)out_shape.size() - (int64_t)shape.size() : axis;
        if (a < 0 || a + shape.size() > out_shape.size()) {
          if (err) *err = "AutoBroadcast: cannot broadcast [" + JoinList(shape) + "] to [" + JoinList(out_shape) + "] with axis=" + std::to_string(axis);
          return false;
        }
        for (size_t i = 0; i < shape.size(); ++i) axes.push_back(a++);
      }
      v = b->AddOp("broadcast_to", {v}, {{"out_shape", JoinList(out_shape)}, {"broadcast_axes", JoinList(axes)}}, err);
      if (v < 0) return false;
      inserted = true;
    }
    if (inserted) ins.attrs["axis"] = "-1";
    b->AppendInstr(ins);
  }
  return true;
}

// ---- CastCollapsing / TransposeCollapsing -------------------------------------------------------------
// cast_collapsing.cc:111-248 and transpose_collapsing.cc:119-290, which share one algorithm: every chain of casts
// (transposes) is walked from its first one; an op all of whose users are of the same kind hands its operand to them
// and disappears (a transpose composes its permutation into theirs), an op that changes nothing - a cast to its
// operand's own type, an identity permutation - disappears (or, when fetched, becomes an identity), an op nothing
// uses and nobody fetches disappears.  As in the reference a program with a single such op is left alone, and the
// user lists are those of the program before the pass.
struct Collapser {
  NetBuilder* b;
  std::string kind;  // "cast" or "transpose"
  std::vector<ProgramInstr> ins;
  std::set<int> fetch;
  std::vector<std::vector<int>> users;  // per variable: instructions reading it (before the pass)
  std::vector<int> producer;            // per variable
  std::set<int> removed, visited;

  bool ChangesNothing(const ProgramInstr& c) const {
    if (kind == "cast") return b->vars()[c.inputs[0]].dtype == b->vars()[c.output].dtype;
    const std::vector<int64_t> perm = IntList(c.attrs.count("axis") ? c.attrs.at("axis") : "");
    for (size_t i = 0; i < perm.size(); ++i)
      if (perm[i] != (int64_t)i) return false;
    return true;
  }

  // `first` then `second`, as one op written into `second`.
  void Compose(const ProgramInstr& first, ProgramInstr* second) const {
    second->inputs[0] = first.inputs[0];
    if (kind == "cast") return;  // the second cast keeps its own target type
    const std::vector<int64_t> p1 = IntList(first.attrs.at("axis")), p2 = IntList(second->attrs.at("axis"));
    std::vector<int64_t> fused(p2.size());
    for (size_t i = 0; i < p2.size(); ++i) fused[i] = p1[p2[i]];  // out[i] = mid[p2[i]] and mid[j] = in[p1[j]]
    second->attrs["axis"] = JoinList(fused);
  }

  void Fuse(int i) {
    visited.insert(i);
    ProgramInstr& c    = ins[i];
    const int in       = c.inputs[0], out = c.output;
    const bool fetched = fetch.count(out) > 0;
    const bool useless = ChangesNothing(c);
    const std::vector<int>& next = users[out];
    if (next.empty()) {
      if (!fetched) removed.insert(i);
      else if (useless) ToIdentity(&c);
      return;
    }
    if (useless) {
      if (fetched) {
        ToIdentity(&c);
        return;
      }
      for (int u : next)
        for (int& v : ins[u].inputs)
          if (v == out) v = in;
      removed.insert(i);
      for (int u : next)
        if (ins[u].op_type == kind) Fuse(u);
      return;
    }
    bool any_same = false;
    for (int u : next) any_same = any_same || ins[u].op_type == kind;
    if (!any_same) return;
    bool can_remove = !fetched;
    std::vector<int> fused;
    for (int u : next) {
      if (ins[u].op_type != kind) {
        can_remove = false;
        continue;
      }
      Compose(c, &ins[u]);
      fused.push_back(u);
    }
    if (can_remove) removed.insert(i);
    for (int u : fused) Fuse(u);
  }

  static void ToIdentity(ProgramInstr* c) {
    c->op_type = "identity";
    c->attrs.clear();
  }

  void Run() {
    users.assign(b->vars().size(), {});
    producer.assign(b->vars().size(), -1);
    int count = 0;
    for (size_t i = 0; i < ins.size(); ++i) {
      producer[ins[i].output] = (int)i;
      std::set<int> seen;
      for (int v : ins[i].inputs)
        if (seen.insert(v).second) users[v].push_back((int)i);
      count += ins[i].op_type == kind;
    }
    if (count <= 1) return;
    for (size_t i = 0; i < ins.size(); ++i) {
      if (ins[i].op_type != kind || visited.count((int)i)) continue;
      int first = (int)i;
      for (int p = producer[ins[first].inputs[0]]; p >= 0 && ins[p].op_type == kind; p = producer[ins[p].inputs[0]]) first = p;
      if (!visited.count(first)) Fuse(first);
    }
  }
};

bool Collapse(NetBuilder* b, const std::string& kind, const std::vector<int>& fetch) {
  Collapser c;
  c.b    = b;
  c.kind = kind;
  c.ins  = b->TakeInstrs();
  c.fetch.insert(fetch.begin(), fetch.end());
  c.Run();
  for (size_t i = 0; i < c.ins.size(); ++i) {
    if (c.removed.count((int)i)) continue;
    b->AppendInstr(c.ins[i]);
  }
  return true;
}

// ---- RemoveIdentity ----------------------------------------------------------------------------------
// remove_identity.cc:36-75: which instructions change nothing.
bool ChangesNothing(const NetBuilder& b, const ProgramInstr& ins) {
  const std::string& t = ins.op_type;
  auto attr = [&](const char* k, const char* d) { return ins.attrs.count(k) ? ins.attrs.at(k) : std::string(d); };
  if (t == "identity") return true;
  if (t == "scale") return atof(attr("scale", "1").c_str()) == 1.0 && atof(attr("bias", "0").c_str()) == 0.0;
  if (t == "cast") return b.vars()[ins.inputs[0]].dtype == b.vars()[ins.output].dtype;
  if (t == "transpose") {
    std::vector<int64_t> perm = IntList(attr("axis", ""));
    if (perm.size() != b.vars()[ins.inputs[0]].shape.size()) return false;
    for (size_t i = 0; i < perm.size(); ++i)
      if (perm[i] != (int64_t)i) return false;
    return true;
  }
  if (t == "concat") return ins.inputs.size() == 1;
  if (t == "broadcast_to" || t == "slice" || t == "reshape" || t.rfind("reduce_", 0) == 0)
    return b.vars()[ins.inputs[0]].shape == b.vars()[ins.output].shape;
  return false;
}

bool RemoveIdentity(NetBuilder* b, const std::vector<int>& fetch_list) {
  std::vector<ProgramInstr> ins = b->TakeInstrs();
  std::set<int> fetch(fetch_list.begin(), fetch_list.end());
  const int nv = (int)b->vars().size();
  std::vector<int> producer(nv, -1), repl(nv);
  for (int v = 0; v < nv; ++v) repl[v] = v;
  for (size_t i = 0; i < ins.size(); ++i) producer[ins[i].output] = (int)i;
  std::function<int(int)> find = [&](int v) { return repl[v] == v ? v : repl[v] = find(repl[v]); };
  std::vector<bool> gone(ins.size(), false);
  for (size_t i = 0; i < ins.size(); ++i) {
    if (!ChangesNothing(*b, ins[i])) continue;
    const int in = find(ins[i].inputs[0]), out = ins[i].output;
    if (!fetch.count(out)) {
      repl[out] = in;  // users of the result read the operand
      gone[i]   = true;
    } else if (!b->vars()[in].is_input && !fetch.count(in) && producer[in] >= 0 &&
               b->vars()[in].shape == b->vars()[out].shape && b->vars()[in].dtype == b->vars()[out].dtype) {
      ins[producer[in]].output = out;  // the operand's producer writes the fetched result directly
      producer[out]            = producer[in];
      repl[in]                 = out;
      gone[i]                  = true;
    } else if (ins[i].op_type != "reshape") {
      ins[i].op_type = "identity";  // both ends must survive (remove_identity.cc:222-224)
      ins[i].attrs.clear();
    }
  }
  for (size_t i = 0; i < ins.size(); ++i) {
    if (gone[i]) continue;
    for (int& v : ins[i].inputs) v = find(v);
    b->AppendInstr(ins[i]);
  }
  return true;
}

// ---- FillConstantRewriter / FillConstantFolding ----------------------------------------------------------
std::string FormatConstant(double v, DType t) {
  char buf[64];
  if (t == DType::kInt32 || t == DType::kInt64 || t == DType::kBool) snprintf(buf, sizeof(buf), "%lld", (long long)v);
  else if (t == DType::kFloat64) snprintf(buf, sizeof(buf), "%.17g", v);
  else snprintf(buf, sizeof(buf), "%.9g", (double)(float)v);
  return buf;
}

// fill_constant_rewriter.cc:54-142: an op that reads a constant and whose result is a constant again becomes a
// fill_constant itself (reshape, scale, cast, broadcast_to, slice, abs, log, log2, log10, tanh); a constant all of
// whose users were rewritten, and that nobody fetches, disappears.  float32 constants are computed in float, as the
// reference's variant holding a `float` does.
bool FillConstantRewriter(NetBuilder* b, const std::vector<int>& fetch_list) {
  std::vector<ProgramInstr> ins = b->TakeInstrs();
  const std::set<int> fetch(fetch_list.begin(), fetch_list.end());
  std::vector<std::vector<int>> users(b->vars().size());
  for (size_t i = 0; i < ins.size(); ++i) {
    std::set<int> seen;
    for (int v : ins[i].inputs)
      if (seen.insert(v).second) users[v].push_back((int)i);
  }
  std::set<int> removed;
  static const std::set<std::string> math = {"abs", "log", "log2", "log10", "tanh"};
  std::function<void(int)> rewrite = [&](int ci) {
    const ProgramInstr constant = ins[ci];  // a copy: users are rewritten in place
    const int out               = constant.output;
    if (users[out].empty()) return;
    bool can_remove = true;
    for (int u : users[out]) {
      ProgramInstr& op     = ins[u];
      const std::string t  = op.op_type;
      const DType out_type = b->vars()[op.output].dtype;
      const DType in_type  = b->vars()[out].dtype;
      const bool is_float  = in_type == DType::kFloat32 || in_type == DType::kFloat16 || in_type == DType::kBFloat16;
      auto attr = [&](const char* k, const char* d) { return op.attrs.count(k) ? op.attrs.at(k) : std::string(d); };
      std::map<std::string, std::string> attrs = constant.attrs;
      const double v = atof(constant.attrs.count("value") ? constant.attrs.at("value").c_str() : "0");
      if (t == "reshape" || t == "broadcast_to" || t == "slice") {
        attrs["shape"] = JoinList(b->vars()[op.output].shape);
      } else if (t == "scale") {
        const std::string bas = attr("bias_after_scale", "true");
        const bool after      = bas == "true" || bas == "1" || bas == "True";
        double r;
        if (is_float) {
          const float x = (float)v, sc = (float)atof(attr("scale", "1").c_str()), bi = (float)atof(attr("bias", "0").c_str());
          volatile float prod = after ? x * sc : x + bi;  // two roundings, as two float operations
          r                   = after ? (float)(prod + bi) : (float)(prod * sc);
        } else {
          const double sc = atof(attr("scale", "1").c_str()), bi = atof(attr("bias", "0").c_str());
          r = after ? v * sc + bi : (v + bi) * sc;
          if (in_type == DType::kInt32 || in_type == DType::kInt64) r = (double)(long long)r;
        }
        attrs["value"] = FormatConstant(r, in_type);
      } else if (t == "cast") {
        attrs["dtype"] = DTypeName(out_type);
        double r = v;
        if (out_type == DType::kInt32 || out_type == DType::kInt64) r = (double)(long long)v;  // toward zero
        if (out_type == DType::kBool) r = v != 0.0;
        attrs["value"] = FormatConstant(r, out_type);
      } else if (math.count(t) && (is_float || in_type == DType::kFloat64)) {
        double r;
        if (is_float) {
          const float x = (float)v;
          r = t == "abs" ? fabsf(x) : t == "log" ? logf(x) : t == "log2" ? log2f(x) : t == "log10" ? log10f(x) : tanhf(x);
        } else {
          r = t == "abs" ? fabs(v) : t == "log" ? log(v) : t == "log2" ? log2(v) : t == "log10" ? log10(v) : tanh(v);
        }
        attrs["value"] = FormatConstant(r, in_type);
      } else {
        can_remove = false;
        continue;
      }
      op.op_type = "fill_constant";
      op.inputs.clear();
      op.attrs = attrs;
      if (!op.attrs.count("dtype")) op.attrs["dtype"] = DTypeName(out_type);
      rewrite(u);
    }
    if (can_remove && !fetch.count(out)) removed.insert(ci);
  };
  for (size_t i = 0; i < ins.size(); ++i)
    if (ins[i].op_type == "fill_constant" && !removed.count((int)i)) rewrite((int)i);
  for (size_t i = 0; i < ins.size(); ++i)
    if (!removed.count((int)i)) b->AppendInstr(ins[i]);
  return true;
}

// fill_constant_folding.cc: constants with the same shape, value and type are one constant; the later ones, unless
// fetched, disappear and their users read the first.
bool FillConstantFolding(NetBuilder* b, const std::vector<int>& fetch_list) {
  std::vector<ProgramInstr> ins = b->TakeInstrs();
  const std::set<int> fetch(fetch_list.begin(), fetch_list.end());
  std::map<std::string, int> first;  // key -> variable
  std::map<int, int> repl;
  for (size_t i = 0; i < ins.size(); ++i) {
    ProgramInstr& op = ins[i];
    for (int& v : op.inputs)
      if (repl.count(v)) v = repl[v];
    if (op.op_type != "fill_constant") {
      b->AppendInstr(op);
      continue;
    }
    std::string key;
    for (auto& kv : op.attrs) key += kv.first + "=" + kv.second + ";";
    auto it = first.find(key);
    if (it == first.end() || fetch.count(op.output)) {
      if (it == first.end()) first[key] = op.output;
      b->AppendInstr(op);
    } else {
      repl[op.output] = it->second;
    }
  }
  return true;
}

// ---- Decomposer -------------------------------------------------------------------------------------------
// cinn/frontend/pass/decomposer.cc with the decomposers of cinn/frontend/decomposer/activation.cc:54-118 (gelu,
// softmax) and batch_norm.cc:246-280 (inference batch_norm): the instruction is replaced by the primitives that
// compute it, the last of which writes the original result variable.  relu is left alone: its decomposed form
// max(x, 0) is what the kernels compute for it anyway.  The training-mode batch norms are decomposed by the
// builder's own methods (they have several results).
bool Decomposer(NetBuilder* b, std::string* err) {
  const std::vector<ProgramInstr> old = b->TakeInstrs();
  bool ok = true;
  auto op = [&](const std::string& type, const std::vector<int>& ins, const std::map<std::string, std::string>& attrs) {
    const int v = ok ? b->AddOp(type, ins, attrs, err) : -1;
    ok = ok && v >= 0;
    return v;
  };
  // the instruction that produced `v` (the last one appended) writes `into` instead
  auto retarget = [&](int v, int into) {
    if (!ok) return;
    std::vector<ProgramInstr> all = b->TakeInstrs();
    if (!all.empty() && all.back().output == v) all.back().output = into;
    for (auto& i : all) b->AppendInstr(i);
  };
  for (const ProgramInstr& ins : old) {
    const Variable x = ins.inputs.empty() ? Variable() : b->vars()[ins.inputs[0]];
    const std::string shape = JoinList(x.shape), dt = DTypeName(x.dtype);
    auto attr = [&](const char* k, const char* d) { return ins.attrs.count(k) ? ins.attrs.at(k) : std::string(d); };
    auto constant = [&](const std::string& value) { return op("fill_constant", {}, {{"shape", shape}, {"value", value}, {"dtype", dt}}); };
    if (ins.op_type == "gelu") {
      // x * (0.5 + 0.5 * erf(sqrt(0.5) * x))
      const int p5 = constant("0.5"), p7 = constant("0.7071067811865476");
      const int e  = op("erf", {op("elementwise_mul", {ins.inputs[0], p7}, {})}, {});
      const int cdf = op("elementwise_add", {p5, op("elementwise_mul", {p5, e}, {})}, {});
      retarget(op("elementwise_mul", {ins.inputs[0], cdf}, {}), ins.output);
    } else if (ins.op_type == "softmax" && attr("mode", "fast") != "fast") {
      // exp(x - max) / sum(exp(x - max)) along the axis
      const int nd = (int)x.shape.size();
      int axis     = atoi(attr("axis", "-1").c_str());
      if (axis < 0) axis += nd;
      std::vector<int64_t> kept;
      for (int i = 0; i < nd; ++i)
        if (i != axis) kept.push_back(i);
      if (kept.empty()) kept.push_back(-1);
      const std::map<std::string, std::string> red = {{"dim", std::to_string(axis)}, {"keep_dim", "false"}};
      const std::map<std::string, std::string> bc  = {{"out_shape", shape}, {"broadcast_axes", JoinList(kept)}};
      const int m4 = op("broadcast_to", {op("reduce_max", {ins.inputs[0]}, red)}, bc);
      const int e1 = op("exp", {op("subtract", {ins.inputs[0], m4}, {})}, {});
      const int s4 = op("broadcast_to", {op("reduce_sum", {e1}, red)}, bc);
      const int e2 = op("exp", {op("subtract", {ins.inputs[0], m4}, {})}, {});
      retarget(op("divide", {e2, s4}, {}), ins.output);
    } else if (ins.op_type == "batch_norm" && ins.inputs.size() == 5 && x.shape.size() == 4 && attr("data_layout", "NCHW") == "NCHW") {
      // ((x - mean) * rsqrt(variance + epsilon)) * scale + bias with the per-channel operands broadcast along axis 1
      const std::map<std::string, std::string> bc = {{"out_shape", shape}, {"broadcast_axes", "1"}};
      const int mean4 = op("broadcast_to", {ins.inputs[3]}, bc);
      const int var4  = op("broadcast_to", {ins.inputs[4]}, bc);
      const int inv   = op("rsqrt", {op("elementwise_add", {var4, constant(attr("epsilon", "1e-05"))}, {})}, {});
      const int sc4 = op("broadcast_to", {ins.inputs[1]}, bc), bi4 = op("broadcast_to", {ins.inputs[2]}, bc);
      const int normalized = op("elementwise_mul", {op("subtract", {ins.inputs[0], mean4}, {}), inv}, {});
      retarget(op("elementwise_add", {op("elementwise_mul", {normalized, sc4}, {}), bi4}, {}), ins.output);
    } else {
      b->AppendInstr(ins);
    }
    if (!ok) return false;
  }
  return true;
}

// ---- DeadCodeEliminate -------------------------------------------------------------------------------
bool DeadCodeEliminate(NetBuilder* b, const std::vector<int>& fetch) {
  if (fetch.empty()) return true;  // nothing named: every unread result counts as an output
  std::vector<ProgramInstr> ins = b->TakeInstrs();
  std::vector<int> producer(b->vars().size(), -1);
  for (size_t i = 0; i < ins.size(); ++i) producer[ins[i].output] = (int)i;
  std::vector<bool> live(ins.size(), false);
  std::vector<int> stack;
  for (int v : fetch)
    if (producer[v] >= 0) stack.push_back(producer[v]);
  while (!stack.empty()) {
    int i = stack.back();
    stack.pop_back();
    if (live[i]) continue;
    live[i] = true;
    for (int v : ins[i].inputs)
      if (producer[v] >= 0) stack.push_back(producer[v]);
  }
  for (size_t i = 0; i < ins.size(); ++i)
    if (live[i]) b->AppendInstr(ins[i]);
  return true;
}

}  // namespace

const std::vector<std::string>& DefaultProgramPasses() {
  static const std::vector<std::string> s = {"ExpandZeroDim", "AutoCast", "Decomposer", "RemoveIdentity",
                                             "CastCollapsing", "TransposeCollapsing", "RemoveIdentity",
                                             "AutoBroadcast", "FillConstantRewriter", "FillConstantFolding",
                                             "RemoveIdentity", "DeadCodeEliminate"};
  return s;
}

bool ApplyProgramPass(NetBuilder* b, const std::string& pass, const std::vector<int>& fetch, std::string* err) {
  if (!b) return false;
  for (int v : fetch)
    if (v < 0 || v >= (int)b->vars().size()) {
      if (err) *err = "apply_pass: bad fetch variable";
      return false;
    }
  if (pass == "AutoCast") return AutoCast(b, err);
  if (pass == "AutoBroadcast") return AutoBroadcast(b, err);
  if (pass == "CastCollapsing") return Collapse(b, "cast", fetch);
  if (pass == "TransposeCollapsing") return Collapse(b, "transpose", fetch);
  if (pass == "RemoveIdentity") return RemoveIdentity(b, fetch);
  if (pass == "DeadCodeEliminate") return DeadCodeEliminate(b, fetch);
  if (pass == "FillConstantRewriter") return FillConstantRewriter(b, fetch);
  if (pass == "FillConstantFolding") return FillConstantFolding(b, fetch);
  if (pass == "Decomposer") return Decomposer(b, err);
  if (pass == "ExpandZeroDim")
    return true;
  if (err) *err = "apply_pass: no program pass named '" + pass + "'";
  return false;
}

std::string PrintProgram(const NetBuilder& b) {
  std::string s;
  for (const ProgramInstr& ins : b.instrs()) {
    s += ins.op_type + " " + b.vars()[ins.output].id + " =";
    for (size_t k = 0; k < ins.inputs.size(); ++k) s += (k ? ", " : " ") + b.vars()[ins.inputs[k]].id;
    if (!ins.attrs.empty()) {
      s += " ;";
      for (auto& kv : ins.attrs) s += " " + kv.first + "=" + kv.second;
    }
    s += "\n";
  }
  return s;
}

}  // namespace cinn_b200
