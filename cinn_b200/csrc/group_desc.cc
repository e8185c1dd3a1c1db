// Parsing / printing of group descriptions and the canonical expression used by the pattern matcher.
#include "group_desc.h"

#include <algorithm>
#include <functional>
#include <set>
#include <sstream>

namespace cinn_b200 {

const char* DTypeName(DType t) {
  switch (t) {
    case DType::kFloat32: return "float32";
    case DType::kFloat16: return "float16";
    case DType::kBFloat16: return "bfloat16";
    case DType::kFloat64: return "float64";
    case DType::kInt32: return "int32";
    case DType::kInt64: return "int64";
    case DType::kBool: return "bool";
    case DType::kUInt8: return "uint8";
    default: return "unknown";
  }
}

DType DTypeFromName(const std::string& s) {
  if (s == "float32" || s == "float" || s == "fp32") return DType::kFloat32;
  if (s == "float16" || s == "fp16" || s == "half") return DType::kFloat16;
  if (s == "bfloat16" || s == "bf16") return DType::kBFloat16;
  if (s == "float64" || s == "double") return DType::kFloat64;
  if (s == "int32" || s == "int") return DType::kInt32;
  if (s == "int64") return DType::kInt64;
  if (s == "bool") return DType::kBool;
  if (s == "uint8") return DType::kUInt8;
  return DType::kUnknown;
}

int DTypeBytes(DType t) {
  switch (t) {
    case DType::kFloat32: case DType::kInt32: return 4;
    case DType::kFloat16: case DType::kBFloat16: return 2;
    case DType::kFloat64: case DType::kInt64: return 8;
    case DType::kBool: case DType::kUInt8: return 1;
    default: return 0;
  }
}

static std::vector<std::string> SplitWs(const std::string& s) {
  std::istringstream is(s);
  std::vector<std::string> out;
  std::string w;
  while (is >> w) out.push_back(w);
  return out;
}

static bool ParseShape(const std::string& s, std::vector<int64_t>* shape) {
  shape->clear();
  if (s == "scalar" || s.empty()) return true;
  std::string cur;
  for (size_t i = 0; i <= s.size(); ++i) {
    if (i == s.size() || s[i] == ',') {
      if (cur.empty()) return false;
      char* end = nullptr;
      long long v = strtoll(cur.c_str(), &end, 10);
      if (*end != 0 || v < 0) return false;
      shape->push_back(v);
      cur.clear();
    } else {
      cur.push_back(s[i]);
    }
  }
  return true;
}

static std::string ShapeText(const std::vector<int64_t>& shape) {
  if (shape.empty()) return "scalar";
  std::string s;
  for (size_t i = 0; i < shape.size(); ++i) {
    if (i) s += ",";
    s += std::to_string(shape[i]);
  }
  return s;
}

bool ParseGroupDesc(const std::string& text, GroupDesc* out, std::string* err) {
  *out = GroupDesc();
  std::istringstream is(text);
  std::string line;
  int lineno = 0;
  auto fail  = [&](const std::string& m) {
    if (err) *err = "group description line " + std::to_string(lineno) + ": " + m;
    return false;
  };
  while (std::getline(is, line)) {
    ++lineno;
    auto hash = line.find('#');
    if (hash != std::string::npos) line = line.substr(0, hash);
    std::string attrs_part;
    auto semi = line.find(';');
    if (semi != std::string::npos) {
      attrs_part = line.substr(semi + 1);
      line       = line.substr(0, semi);
    }
    auto w = SplitWs(line);
    if (w.empty()) continue;
    if (w[0] == "group") {
      if (w.size() != 2) return fail("expected: group <name>");
      out->name = w[1];
    } else if (w[0] == "input" || w[0] == "output") {
      if (w.size() != 4) return fail("expected: " + w[0] + " <name> <dtype> <shape>");
      TensorDesc t;
      t.name  = w[1];
      t.dtype = DTypeFromName(w[2]);
      if (t.dtype == DType::kUnknown) return fail("unknown dtype '" + w[2] + "'");
      if (!ParseShape(w[3], &t.shape)) return fail("bad shape '" + w[3] + "'");
      (w[0] == "input" ? out->inputs : out->outputs).push_back(t);
    } else if (w[0] == "op") {
      if (w.size() < 4 || w[3] != "=") return fail("expected: op <type> <out> = <inputs...> [; attrs]");
      OpDesc op;
      op.type   = w[1];
      op.output = w[2];
      for (size_t i = 4; i < w.size(); ++i) op.inputs.push_back(w[i]);
      for (auto& kv : SplitWs(attrs_part)) {
        auto eq = kv.find('=');
        if (eq == std::string::npos) return fail("attribute '" + kv + "' is not key=value");
        op.attrs[kv.substr(0, eq)] = kv.substr(eq + 1);
      }
      out->ops.push_back(op);
    } else {
      return fail("unknown item '" + w[0] + "'");
    }
  }
  if (out->name.empty()) {
    lineno = 0;
    return fail("missing 'group <name>'");
  }
  if (out->outputs.empty()) {
    lineno = 0;
    return fail("group has no output");
  }
  return true;
}

std::string PrintGroupDesc(const GroupDesc& g) {
  std::ostringstream os;
  os << "group " << g.name << "\n";
  for (auto& t : g.inputs) os << "input " << t.name << " " << DTypeName(t.dtype) << " " << ShapeText(t.shape) << "\n";
  for (auto& op : g.ops) {
    os << "op " << op.type << " " << op.output << " =";
    for (auto& i : op.inputs) os << " " << i;
    if (!op.attrs.empty()) {
      os << " ;";
      for (auto& kv : op.attrs) os << " " << kv.first << "=" << kv.second;
    }
    os << "\n";
  }
  for (auto& t : g.outputs) os << "output " << t.name << " " << DTypeName(t.dtype) << " " << ShapeText(t.shape) << "\n";
  return os.str();
}

std::string CanonicalExpr(const GroupDesc& g, std::string* err) {
  std::map<std::string, int> input_index;
  for (size_t i = 0; i < g.inputs.size(); ++i) input_index[g.inputs[i].name] = (int)i;
  std::map<std::string, const OpDesc*> producer;
  for (auto& op : g.ops) producer[op.output] = &op;
  if (g.outputs.empty()) {
    if (err) *err = "group has no output";
    return "";
  }
  bool ok = true;
  std::function<std::string(const std::string&, int)> print = [&](const std::string& v, int depth) -> std::string {
    if (depth > 64) {
      ok = false;
      if (err) *err = "expression too deep (cycle?) at '" + v + "'";
      return "?";
    }
    auto in = input_index.find(v);
    if (in != input_index.end()) return "%" + std::to_string(in->second);
    auto p = producer.find(v);
    if (p == producer.end()) {
      ok = false;
      if (err) *err = "value '" + v + "' is neither a group input nor produced by an op of the group";
      return "?";
    }
    std::string s = p->second->type + "(";
    for (size_t i = 0; i < p->second->inputs.size(); ++i) {
      if (i) s += ",";
      s += print(p->second->inputs[i], depth + 1);
    }
    return s + ")";
  };
  // Several outputs: their expressions in output order, separated by ';'.
  std::string s;
  for (size_t i = 0; i < g.outputs.size(); ++i) s += (i ? ";" : "") + print(g.outputs[i].name, 0);
  return ok ? s : "";
}

}  // namespace cinn_b200
