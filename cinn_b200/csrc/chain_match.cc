// Linearises an elementwise / broadcast group into a program for the generic chain kernel (ew_chain.cu).
//
// What a group computes follows the reference's lowering of elementwise groups: every producer is inlined into
// the single output expression (cinn/hlir/framework/op_lowering.cc:247-310), binary ops index their smaller
// operand with the broadcast rule (cinn/hlir/pe/broadcast.cc:35-273), an Add fed by an inlined Mul becomes a
// fused multiply-add (cinn/optim/lower_intrin.cc:41-59), and values of 16-bit float type are rounded to that
// type after every op.  A group is accepted when its expression is a chain: walking back from the output, every
// op has exactly one operand computed inside the group; all other operands are group inputs (possibly through
// broadcast_to), constants, or the chain value itself (x * identity(x)).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <map>
#include <set>
#include <sstream>

#include "ew_chain.h"
#include "row_prog_prefix.h"
#include "group_desc.h"

namespace cinn_b200 {
namespace {

struct Value {
  DType dtype = DType::kFloat32;
  std::vector<int64_t> shape;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return n;
  }
};

int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

std::vector<int64_t> IntList(const std::string& text) {
  std::vector<int64_t> out;
  std::string cur;
  for (char c : text + ",") {
    if (c == ',') {
      if (!cur.empty()) out.push_back(atoll(cur.c_str()));
      cur.clear();
    } else if (c != '[' && c != ']' && c != ' ') {
      cur.push_back(c);
    }
  }
  return out;
}

const std::map<std::string, int>& UnaryCodes() {
  static const std::map<std::string, int> m = {
      {"exp", EW_EXP},     {"tanh", EW_TANH},   {"sigmoid", EW_SIGMOID}, {"rsqrt", EW_RSQRT}, {"sqrt", EW_SQRT},
      {"relu", EW_RELU},   {"negative", EW_NEG}, {"abs", EW_ABS},        {"log", EW_LOG},     {"floor", EW_FLOOR},
      {"ceil", EW_CEIL},   {"erf", EW_ERF},     {"sin", EW_SIN},         {"cos", EW_COS},     {"reciprocal", EW_RECIP},
      {"round", EW_ROUND}, {"trunc", EW_TRUNC}, {"sign", EW_SIGN},       {"relu6", EW_RELU6}, {"log2", EW_LOG2},
      {"log10", EW_LOG10}, {"identity", EW_IDENTITY}, {"tan", EW_TAN},       {"sinh", EW_SINH},   {"cosh", EW_COSH},
      {"asin", EW_ASIN},   {"acos", EW_ACOS},   {"atan", EW_ATAN},       {"asinh", EW_ASINH}, {"acosh", EW_ACOSH},
      {"atanh", EW_ATANH}, {"cbrt", EW_CBRT},   {"isnan", EW_ISNAN},     {"isinf", EW_ISINF}, {"isfinite", EW_ISFINITE},
      {"logical_not", EW_LNOT}};
  return m;
}
const std::map<std::string, int>& IntUnaryCodes() {
  static const std::map<std::string, int> m = {
      {"negative", EW_NEG}, {"abs", EW_ABS}, {"identity", EW_IDENTITY}, {"relu", EW_RELU}, {"logical_not", EW_LNOT},
      {"bitwise_not", EW_BNOT}, {"clz", EW_CLZ}, {"popc", EW_POPC}};
  return m;
}
const std::map<std::string, int>& IntBinaryCodes() {
  static const std::map<std::string, int> m = {
      {"elementwise_add", EW_ADD}, {"subtract", EW_SUB}, {"elementwise_mul", EW_MUL}, {"divide", EW_DIV},
      {"max", EW_MAX}, {"min", EW_MIN}, {"pow", EW_POW}, {"equal", EW_EQ}, {"not_equal", EW_NE}, {"greater_than", EW_GT},
      {"less_than", EW_LT}, {"greater_equal", EW_GE}, {"less_equal", EW_LE}, {"mod", EW_MOD}, {"remainder", EW_MOD},
      {"floor_divide", EW_FLOOR_DIV}, {"logical_and", EW_LAND}, {"logical_or", EW_LOR}, {"logical_xor", EW_LXOR},
      {"bitwise_and", EW_BAND}, {"bitwise_or", EW_BOR}, {"bitwise_xor", EW_BXOR}, {"left_shift", EW_SHL},
      {"right_shift", EW_SHR}, {"logical_right_shift", EW_LSHR}};
  return m;
}
const std::map<std::string, int>& BinaryCodes() {
  static const std::map<std::string, int> m = {
      {"elementwise_add", EW_ADD}, {"subtract", EW_SUB},   {"elementwise_mul", EW_MUL}, {"divide", EW_DIV},
      {"max", EW_MAX},             {"min", EW_MIN},        {"pow", EW_POW},             {"equal", EW_EQ},
      {"not_equal", EW_NE},        {"greater_than", EW_GT}, {"less_than", EW_LT},       {"greater_equal", EW_GE},
      {"less_equal", EW_LE},       {"mod", EW_MOD},        {"remainder", EW_MOD},       {"floor_divide", EW_FLOOR_DIV},
      {"atan2", EW_ATAN2},         {"logical_and", EW_LAND}, {"logical_or", EW_LOR},    {"logical_xor", EW_LXOR}};
  return m;
}

uint64_t Word(int op, int asel, int bsel, int role, float imm) {
  uint32_t bits;
  memcpy(&bits, &imm, 4);
  return (uint64_t)(op & 0xff) | ((uint64_t)(asel & 0xff) << 8) | ((uint64_t)(bsel & 0xff) << 16) |
         ((uint64_t)(role & 3) << 24) | ((uint64_t)bits << 32);
}

bool IsFloatType(DType t) { return t == DType::kFloat32 || t == DType::kFloat16 || t == DType::kBFloat16; }
bool IsIntType(DType t) { return t == DType::kInt32 || t == DType::kInt64 || t == DType::kUInt8; }
bool IsAnyOp(const std::string& t) {
  return UnaryCodes().count(t) || BinaryCodes().count(t) || IntUnaryCodes().count(t) || IntBinaryCodes().count(t);
}
bool YieldsBool(int code) {
  return (code >= EW_EQ && code <= EW_LE) || code == EW_LAND || code == EW_LOR || code == EW_LXOR || code == EW_ISNAN ||
         code == EW_ISINF || code == EW_ISFINITE || code == EW_LNOT;
}

struct Side {
  int input = -1;  // group input index
  int mode  = EW_SIDE_NONE;
  int64_t mid = 1, inner = 1;
  bool operator==(const Side& o) const { return input == o.input && mode == o.mode && mid == o.mid && inner == o.inner; }
};

// A primitive step before encoding.
struct Step {
  int op     = EW_NOP;
  int asel   = 0;      // 0 imm, 1..3 side, 4 the chain value itself
  bool swap  = false;
  float imm  = 0.0f;
  bool f32   = true;   // result type is float32 (contraction only applies to fp32 arithmetic)
  bool single_use = true;  // EW_MUL: the product has one user in the group (the reference inlines, hence contracts, only then)
  // EW_SELECT only: second operand and the role of the chain value (see ew_chain.h)
  int bsel   = 0;
  float imm2 = 0.0f;
  int role   = 0;
};

struct ChainBuilder {
  const GroupDesc& g;
  std::string* why;
  std::map<std::string, Value> values;
  std::map<std::string, const OpDesc*> producer;
  std::map<std::string, int> input_index;
  std::vector<Side> sides;
  int64_t n = 0;
  std::vector<int64_t> out_shape;
  // The float form carries float32 / float16 / bfloat16 / bool values in fp32 registers; the integer form carries
  // values of ONE integer type (`compute`) and bool in registers of that type.
  bool int_class = false;
  bool dbl_class = false;  // float64 values and bool in double registers; immediates through a table of doubles
  bool allow_reduce = false;  // Infer() also accepts reduce ops (the row programs)
  DType compute  = DType::kFloat32;
  std::vector<double> dimms;

  ChainBuilder(const GroupDesc& g_, std::string* w) : g(g_), why(w) {}

  bool Ok(DType t) const {
    if (t == DType::kBool) return true;
    if (dbl_class) return t == DType::kFloat64;
    return int_class ? t == compute : IsFloatType(t);
  }
  // The type whose Mul + Add pairs contract into a fused multiply-add.
  bool Arith(DType t) const { return dbl_class ? t == DType::kFloat64 : (!int_class && t == DType::kFloat32); }
  const std::map<std::string, int>& Unary() const { return int_class ? IntUnaryCodes() : UnaryCodes(); }
  const std::map<std::string, int>& Binary() const { return int_class ? IntBinaryCodes() : BinaryCodes(); }
  // A constant as the immediate field of a program word: an fp32 value, or (integer form) the bits of an int32.
  bool Imm(const std::string& text, float* out) {
    if (dbl_class) {
      const double d = atof(text.c_str());
      int32_t idx    = -1;
      for (size_t i = 0; i < dimms.size(); ++i)
        if (memcmp(&dimms[i], &d, 8) == 0) idx = (int32_t)i;
      if (idx < 0) {
        if (dimms.size() >= 8) return false;
        dimms.push_back(d);
        idx = (int32_t)dimms.size() - 1;
      }
      memcpy(out, &idx, 4);
      return true;
    }
    if (!int_class) {
      *out = (float)atof(text.c_str());
      return true;
    }
    const double d = atof(text.c_str());
    if (d != std::floor(d) || d < -2147483648.0 || d > 2147483647.0) return false;
    const int32_t v = (int32_t)d;
    memcpy(out, &v, 4);
    return true;
  }

  bool Fail(const std::string& m) {
    if (why) *why = m;
    return false;
  }

  static std::string Attr(const OpDesc& op, const char* k, const std::string& d) {
    auto it = op.attrs.find(k);
    return it == op.attrs.end() ? d : it->second;
  }

  // dtype / shape of every value of the group, by the same rules the frontend uses.
  bool Infer() {
    for (size_t i = 0; i < g.inputs.size(); ++i) {
      Value v;
      v.dtype                  = g.inputs[i].dtype;
      v.shape                  = g.inputs[i].shape;
      values[g.inputs[i].name] = v;
      input_index[g.inputs[i].name] = (int)i;
    }
    for (auto& op : g.ops) {
      producer[op.output] = &op;
      for (auto& in : op.inputs)
        if (!values.count(in)) return Fail("value '" + in + "' is used before it is defined");
      Value v;
      if (op.type == "fill_constant") {
        v.dtype = DTypeFromName(Attr(op, "dtype", "float32"));
        v.shape = IntList(Attr(op, "shape", "1"));
      } else if (op.type == "cast") {
        v       = values[op.inputs[0]];
        v.dtype = DTypeFromName(Attr(op, "dtype", ""));
        if (v.dtype == DType::kUnknown) return Fail("cast without a known dtype");
      } else if (op.type == "broadcast_to") {
        v.dtype = values[op.inputs[0]].dtype;
        v.shape = IntList(Attr(op, "out_shape", ""));
      } else if (BinaryCodes().count(op.type) || IntBinaryCodes().count(op.type)) {
        if (op.inputs.size() != 2) return Fail(op.type + " needs two operands");
        const Value &a = values[op.inputs[0]], &b = values[op.inputs[1]];
        v       = a.numel() >= b.numel() ? a : b;
        if (a.shape.size() != b.shape.size() && a.numel() == b.numel()) v = a.shape.size() >= b.shape.size() ? a : b;
        const int code = BinaryCodes().count(op.type) ? BinaryCodes().at(op.type) : IntBinaryCodes().at(op.type);
        v.dtype        = YieldsBool(code) ? DType::kBool : a.dtype;
      } else if (UnaryCodes().count(op.type) || IntUnaryCodes().count(op.type) || op.type == "scale") {
        if (op.inputs.size() != 1) return Fail(op.type + " needs one operand");
        v = values[op.inputs[0]];
        if (UnaryCodes().count(op.type) && YieldsBool(UnaryCodes().at(op.type))) v.dtype = DType::kBool;
      } else if (op.type == "select") {
        if (op.inputs.size() != 3) return Fail("select needs three operands");
        v = values[op.inputs[1]];
        for (int k = 0; k < 3; ++k)
          if (values[op.inputs[k]].numel() > v.numel()) v.shape = values[op.inputs[k]].shape;
      } else if (allow_reduce && op.type.rfind("reduce_", 0) == 0 && op.inputs.size() == 1) {
        // cinn/hlir/op/reduction.cc:49-158: `dim` (empty: all axes), `keep_dim`
        const Value& x = values[op.inputs[0]];
        std::vector<int64_t> dims = IntList(Attr(op, "dim", ""));
        const int nd = (int)x.shape.size();
        if (dims.empty())
          for (int i = 0; i < nd; ++i) dims.push_back(i);
        std::vector<bool> red(nd, false);
        for (auto d : dims) {
          if (d < 0) d += nd;
          if (d < 0 || d >= nd) return Fail("reduce dim out of range");
          red[d] = true;
        }
        const std::string keep = Attr(op, "keep_dim", "false");
        const bool keep_dim    = keep == "true" || keep == "1" || keep == "True";
        v.dtype = x.dtype;
        for (int i = 0; i < nd; ++i) {
          if (!red[i]) v.shape.push_back(x.shape[i]);
          else if (keep_dim) v.shape.push_back(1);
        }
        if (v.shape.empty()) v.shape.push_back(1);
      } else {
        return Fail("op '" + op.type + "' is not an elementwise op");
      }
      values[op.output] = v;
    }
    return true;
  }

  // The (mid, inner) addressing of an operand of shape `s` placed at output axes [off, off + rank).
  bool SideSpec(const std::vector<int64_t>& s, const std::vector<int64_t>& axes, int input, Side* out) {
    out->input = input;
    int64_t sn = 1;
    for (auto d : s) sn *= d;
    if (sn == 1) {
      out->mode = EW_SIDE_SCALAR;
      return true;
    }
    if (sn == n) {
      // Same element count: must cover the output axes in order.
      out->mode = EW_SIDE_FULL;
      out->mid  = n;
      return true;
    }
    // Non-unit dims must sit on consecutive output axes and match their extents.
    int lo = -1, hi = -1;
    for (size_t i = 0; i < s.size(); ++i) {
      if (s[i] == 1) continue;
      const int ax = (int)axes[i];
      if (ax < 0 || ax >= (int)out_shape.size() || out_shape[ax] != s[i]) return false;
      if (lo < 0) lo = ax;
      else if (ax != hi + 1) {
        // allow skipped output axes of extent 1 between them
        for (int k = hi + 1; k < ax; ++k)
          if (out_shape[k] != 1) return false;
      }
      hi = ax;
    }
    int64_t mid = 1, inner = 1;
    for (int k = lo; k <= hi; ++k) mid *= out_shape[k];
    if (mid != sn) return false;
    for (int k = hi + 1; k < (int)out_shape.size(); ++k) inner *= out_shape[k];
    out->mid   = mid;
    out->inner = inner;
    if (inner % 4 == 0) out->mode = EW_SIDE_ONE_PER_VEC;
    else if (inner == 1 && mid % 4 == 0) out->mode = EW_SIDE_PERIODIC_VEC;
    else out->mode = EW_SIDE_GENERIC;
    return true;
  }

  int AddSide(const Side& s) {
    for (size_t i = 0; i < sides.size(); ++i)
      if (sides[i] == s) return (int)i + 1;
    if (sides.size() >= 3) return -1;
    sides.push_back(s);
    return (int)sides.size();
  }

  // Resolves a non-chain operand `name` of binary op `op`: an immediate, or a side input.  Returns false if it
  // is something else (computed in the group).
  bool ResolveOperand(const std::string& name, const OpDesc& op, int* asel, float* imm) {
    const OpDesc* p = producer.count(name) ? producer[name] : nullptr;
    if (p && p->type == "fill_constant") {
      *asel = 0;
      return Imm(Attr(*p, "value", "0"), imm);
    }
    std::string src = name;
    std::vector<int64_t> axes;
    const Value* sv = &values[name];
    if (p && IsLoadCast(*p)) {
      // cast(group input): the conversion happens in the load
      src = p->inputs[0];
      sv  = &values[src];
      int64_t axis = atoll(Attr(op, "axis", "-1").c_str());
      int64_t off  = (axis < 0 || sv->shape.size() == out_shape.size()) ? (int64_t)out_shape.size() - (int64_t)sv->shape.size() : axis;
      for (size_t i = 0; i < sv->shape.size(); ++i) axes.push_back(off + (int64_t)i);
    } else if (p && p->type == "broadcast_to") {
      src = p->inputs[0];
      if (!input_index.count(src)) return false;
      axes = IntList(Attr(*p, "broadcast_axes", ""));
      sv   = &values[src];
      if (axes.size() != sv->shape.size()) {
        axes.clear();
        for (size_t i = 0; i < sv->shape.size(); ++i) axes.push_back(out_shape.size() - sv->shape.size() + i);
      }
    } else if (p) {
      return false;
    } else {
      if (!input_index.count(name)) return false;
      // cinn/hlir/pe/broadcast.cc:35-118: the lower-rank operand is aligned at `axis` (-1: right-aligned).
      int64_t axis = atoll(Attr(op, "axis", "-1").c_str());
      int64_t off  = (axis < 0 || sv->shape.size() == out_shape.size()) ? (int64_t)out_shape.size() - (int64_t)sv->shape.size() : axis;
      for (size_t i = 0; i < sv->shape.size(); ++i) axes.push_back(off + (int64_t)i);
    }
    if (!Ok(sv->dtype) && !((IsIntType(sv->dtype) || (dbl_class && sv->dtype == DType::kFloat32)) && src != name)) return false;
    Side s;
    if (!SideSpec(sv->shape, axes, input_index[src], &s)) return false;
    int sel = AddSide(s);
    if (sel < 0) return false;
    *asel = sel;
    return true;
  }

  // A cast whose source is a group input and whose conversion the kernel's load performs exactly as the cast op
  // would: integer -> float32 (one rounding to nearest even), bool -> any float, float16/bfloat16 -> float32.
  bool IsLoadCast(const OpDesc& p) {
    if (p.type != "cast" || !input_index.count(p.inputs[0])) return false;
    const DType from = values[p.inputs[0]].dtype, to = values[p.output].dtype;
    if (int_class) return (IsIntType(from) || from == DType::kBool) && to == compute;  // widen / truncate / 0-1
    if (dbl_class) return (from == DType::kFloat32 || IsIntType(from) || from == DType::kBool) && to == DType::kFloat64;
    if (IsIntType(from)) return to == DType::kFloat32;
    if (from == DType::kBool) return IsFloatType(to);
    if (from == DType::kFloat16 || from == DType::kBFloat16) return to == DType::kFloat32;
    return false;
  }

  // True if `name` is the chain value `chain` possibly through identity ops.
  bool IsSameAs(std::string name, const std::string& chain) {
    while (name != chain) {
      const OpDesc* p = producer.count(name) ? producer[name] : nullptr;
      if (!p || p->type != "identity") return false;
      name = p->inputs[0];
    }
    return true;
  }

  bool InGroupComputed(const std::string& name) {
    const OpDesc* p = producer.count(name) ? producer[name] : nullptr;
    if (!p) return false;
    if (p->type == "fill_constant") return false;
    if (p->type == "broadcast_to" && input_index.count(p->inputs[0])) return false;
    if (IsLoadCast(*p)) return false;
    return true;
  }
};

int DTypeKernelCode(DType t) {
  switch (t) {
    case DType::kFloat32: return EW_F32;
    case DType::kFloat16: return EW_F16;
    case DType::kBFloat16: return EW_BF16;
    case DType::kBool: return EW_BOOL;
    case DType::kInt32: return EW_I32;
    case DType::kInt64: return EW_I64;
    case DType::kFloat64: return EW_F64;
    case DType::kUInt8: return EW_U8;
    default: return -1;
  }
}
const char* DTypeKernelName(DType t) {
  switch (t) {
    case DType::kFloat32: return "f32";
    case DType::kFloat16: return "f16";
    case DType::kBFloat16: return "bf16";
    case DType::kBool: return "bool";
    case DType::kInt32: return "i32";
    case DType::kInt64: return "i64";
    case DType::kFloat64: return "f64";
    case DType::kUInt8: return "u8";
    default: return nullptr;
  }
}

}  // namespace

enum ChainClass { kFloatChain, kIntChain, kDoubleChain };
bool Ok2(const ChainBuilder& cb, DType t) { return cb.Ok(t); }

// `final_idx`: which output the chain ends at.  A second output (float form only) must be a value on the way to it:
// it is stored by an EW_STORE2 step right after the op that produces it.
std::unique_ptr<CompiledGroup> MatchChainOfClass(const GroupDesc& g, const DeviceInfo& dev, ChainClass klass,
                                                 std::string* why, int final_idx = 0, bool allow_sibling = false) {
  ChainBuilder cb(g, why);
  const bool int_class = klass == kIntChain, dbl_class = klass == kDoubleChain;
  cb.int_class = int_class;
  cb.dbl_class = dbl_class;
  if (dbl_class) cb.compute = DType::kFloat64;
  if (g.outputs.size() != 1 && !(g.outputs.size() == 2 && klass == kFloatChain)) {
    cb.Fail("a chain has one output (two in the float form)");
    return nullptr;
  }
  if (!cb.Infer()) return nullptr;
  const TensorDesc& out    = g.outputs[final_idx];
  const TensorDesc* second = g.outputs.size() == 2 ? &g.outputs[1 - final_idx] : nullptr;
  int second_stores        = 0;
  if (second) {
    const DType t = second->dtype;
    if (!cb.values.count(second->name) || cb.values[second->name].dtype != t || second->numel() != out.numel() ||
        !(t == DType::kFloat32 || t == DType::kFloat16 || t == DType::kBFloat16 || t == DType::kBool)) {
      cb.Fail("the second output must be a float or bool value of the output's size");
      return nullptr;
    }
  }
  if (!cb.values.count(out.name)) {
    cb.Fail("output is not produced by the group");
    return nullptr;
  }
  cb.n         = out.numel();
  cb.out_shape = out.shape;
  if (!DTypeKernelName(out.dtype)) {
    cb.Fail(std::string("output dtype ") + DTypeName(out.dtype) + " is not supported by the chain kernel");
    return nullptr;
  }
  if (dbl_class && out.dtype != DType::kFloat64 && out.dtype != DType::kFloat32 && out.dtype != DType::kBool) {
    cb.Fail(std::string("a float64 chain cannot store ") + DTypeName(out.dtype));
    return nullptr;
  }
  if (int_class) {
    // The integer type the chain computes in: that of the last value that is not a cast or a bool, walking back
    // from the output.
    std::string v = out.name;
    cb.compute    = DType::kUnknown;
    for (int guard = 0; guard < 64 && cb.compute == DType::kUnknown; ++guard) {
      const DType t   = cb.values[v].dtype;
      const OpDesc* p = cb.producer.count(v) ? cb.producer[v] : nullptr;
      if (IsIntType(t) && !(p && p->type == "cast")) cb.compute = t;
      else if (p && !p->inputs.empty()) v = p->inputs[p->type == "select" ? 1 : 0];
      else break;
    }
    if (cb.compute == DType::kUnknown) {
      cb.Fail("no integer arithmetic in the group");
      return nullptr;
    }
    if (!IsIntType(out.dtype) && out.dtype != DType::kBool && out.dtype != DType::kFloat32) {
      cb.Fail(std::string("an integer chain cannot store ") + DTypeName(out.dtype));
      return nullptr;
    }
    if (cb.compute == DType::kUInt8)
      for (auto& op : g.ops)
        if (op.type == "pow" || op.type == "clz") {
          cb.Fail("'" + op.type + "' is not offered for uint8 (the reference's host intrinsics define it for int32 / int64 only)");
          return nullptr;
        }
  }

  // Walk back from a value collecting primitive steps in reverse order.  A segment is one such walk: the main one
  // starts at the output; a binary op whose operands are BOTH computed in the group (a tree) makes the walk of one
  // operand a segment of its own, which runs first and leaves its value in a temporary (float form only, at most
  // two temporaries per group).
  struct Segment {
    std::vector<Step> rev;
    bool starts_from_operand = false;
    std::string end;  // the value the walk stopped at (a group input unless starts_from_operand)
  };
  std::vector<Segment> segments;  // finished sub-segments, in program order
  int temps_used = 0;
  std::map<std::string, int> uses;
  for (auto& o : g.ops)
    for (auto& in : o.inputs) ++uses[in];
  if (second) ++uses[second->name];  // a group output is materialised: its product is not contracted into a later add
  auto single_use_mul = [&](const std::string& v) {
    const OpDesc* q = cb.producer.count(v) ? cb.producer[v] : nullptr;
    return q && q->type == "elementwise_mul" && uses[v] == 1 && cb.Arith(cb.values[v].dtype);
  };
  // Where a segment starts: a broadcast operand / constant (EW_COPY already pushed), a smaller group input that
  // broadcasts by the binary ops' own rule, or a full-size group input.  Only the first segment of the program finds
  // its full-size input preloaded in the chain value; the others copy it from a side operand.
  auto finish_start = [&](Segment* seg, bool first) -> bool {
    const std::string& cur = seg->end;
    if (!seg->starts_from_operand && cb.input_index.count(cur) && (cb.values[cur].numel() != cb.n || !first) && Ok2(cb, cb.values[cur].dtype)) {
      Step s;
      s.op  = EW_COPY;
      s.f32 = false;
      OpDesc fake;
      fake.type = "elementwise_add";
      if (cb.ResolveOperand(cur, fake, &s.asel, &s.imm)) {
        seg->rev.push_back(s);
        seg->starts_from_operand = true;
      }
    }
    if (!seg->starts_from_operand && (!cb.input_index.count(cur) || cb.values[cur].numel() != cb.n)) {
      cb.Fail("the chain does not start at a full-size group input");
      return false;
    }
    if (!seg->starts_from_operand && !first) {
      cb.Fail("too many operands for a second branch of the expression");
      return false;
    }
    return true;
  };
  std::function<bool(std::string, Segment*)> walk = [&](std::string cur, Segment* seg) -> bool {
    std::vector<Step>& rev    = seg->rev;
    bool& starts_from_operand = seg->starts_from_operand;
    while (cb.producer.count(cur)) {
      const OpDesc& op = *cb.producer[cur];
      const Value& ov  = cb.values[cur];
      if (second && cur == second->name) {
        Step st;
        st.op  = EW_STORE2;
        st.f32 = false;
        rev.push_back(st);  // runs right after the op (and the rounding) that produces this value
        ++second_stores;
      }
      if (ov.numel() != cb.n) {
        cb.Fail("value '" + cur + "' on the chain has " + std::to_string(ov.numel()) + " elements, the output " + std::to_string(cb.n));
        return false;
      }
      // 16-bit float results are rounded to their type after the op.
      auto round_after = [&]() {
        if (ov.dtype == DType::kFloat16 || ov.dtype == DType::kBFloat16) {
          Step r;
          r.op  = ov.dtype == DType::kFloat16 ? EW_ROUND_F16 : EW_ROUND_BF16;
          r.f32 = false;
          rev.push_back(r);
        }
      };
      const bool f32 = cb.Arith(ov.dtype);
      if (op.type == "cast") {
        const Value& iv = cb.values[op.inputs[0]];
        bool ok = false;
        if (dbl_class) {
          if (iv.dtype == DType::kFloat64 && ov.dtype == DType::kBool) {
            ok = true;
            Step r;
            r.op  = EW_TO_BOOL;
            r.f32 = false;
            rev.push_back(r);
          } else if (cb.Ok(iv.dtype) && cb.Ok(ov.dtype)) {
            ok = true;  // bool -> float64 (0 / 1) or the same type
          } else if (iv.dtype == DType::kFloat64 && ov.dtype == DType::kFloat32) {
            ok = cur == out.name;  // the store rounds to float32
          } else if ((iv.dtype == DType::kFloat32 || IsIntType(iv.dtype)) && ov.dtype == DType::kFloat64) {
            ok = cb.input_index.count(op.inputs[0]) != 0;  // the load of the chain's input converts
          }
        } else if (int_class) {
          if (cb.Ok(iv.dtype) && ov.dtype == DType::kBool && iv.dtype != DType::kBool) {
            ok = true;
            Step r;
            r.op = EW_TO_BOOL;
            rev.push_back(r);
          } else if (cb.Ok(iv.dtype) && cb.Ok(ov.dtype)) {
            ok = true;  // bool -> integer (0 / 1) or the same type
          } else if (cb.Ok(iv.dtype) && cur == out.name && (IsIntType(ov.dtype) || ov.dtype == DType::kFloat32)) {
            ok = true;  // the store converts: other integer width, or float32 (to nearest even)
          } else if ((IsIntType(iv.dtype) || iv.dtype == DType::kBool) && ov.dtype == cb.compute) {
            ok = cb.input_index.count(op.inputs[0]) != 0;  // the load of the chain's input converts
          }
        } else if (IsFloatType(iv.dtype) && IsFloatType(ov.dtype)) {
          ok = true;
          round_after();  // widening casts are exact and need no step
        } else if (iv.dtype == DType::kBool && (IsFloatType(ov.dtype) || ov.dtype == DType::kBool)) {
          ok = true;      // 0 / 1 are exact in every float type
        } else if (cb.Ok(iv.dtype) && ov.dtype == DType::kBool) {
          ok = true;
          Step r;
          r.op = EW_TO_BOOL;
          r.f32 = false;
          rev.push_back(r);
        } else if (cb.Ok(iv.dtype) && IsIntType(ov.dtype)) {
          ok = cur == out.name;  // float -> integer only as the last op: the store converts (toward zero)
        } else if (IsIntType(iv.dtype) && IsFloatType(ov.dtype)) {
          // integer -> float only on the chain's input: the load converts to float32 (to nearest even).  A 16-bit
          // target is then rounded from that float32, which is what the reference's 16-bit classes do (they are
          // constructed from float: cinn/common/float16.h:95-122, bfloat16.h); for float16 the result equals the direct
          // conversion (every integer the first rounding touches overflows float16 anyway).
          ok = cb.input_index.count(op.inputs[0]) != 0;
          if (ok) round_after();
        }
        if (!ok) {
          cb.Fail("cast from " + std::string(DTypeName(iv.dtype)) + " to " + DTypeName(ov.dtype) + " is not supported at this place of a chain");
          return false;
        }
        cur = op.inputs[0];
      } else if (op.type == "scale" && int_class) {
        cb.Fail("scale on integers has no prebuilt kernel");
        return false;
      } else if (op.type == "scale") {
        float s = 0.0f, b = 0.0f;
        if (!cb.Imm(ChainBuilder::Attr(op, "scale", "1"), &s) || !cb.Imm(ChainBuilder::Attr(op, "bias", "0"), &b)) {
          cb.Fail("too many distinct constants for one chain");
          return false;
        }
        const std::string bas = ChainBuilder::Attr(op, "bias_after_scale", "true");
        const bool after      = bas == "true" || bas == "1" || bas == "True";
        round_after();
        Step mul, add;
        mul.op = EW_MUL; mul.imm = s; mul.f32 = f32;
        add.op = EW_ADD; add.imm = b; add.f32 = f32;
        // reverse order: the step executed last is pushed first
        if (after) { rev.push_back(add); rev.push_back(mul); }
        else { rev.push_back(mul); rev.push_back(add); }
        cur = op.inputs[0];
      } else if (cb.Unary().count(op.type)) {
        if (!cb.Ok(cb.values[op.inputs[0]].dtype)) {
          cb.Fail("op '" + op.type + "' on a " + DTypeName(cb.values[op.inputs[0]].dtype) + " value does not fit this form of chain");
          return false;
        }
        round_after();
        if (op.type != "identity") {
          Step s;
          s.op  = cb.Unary().at(op.type);
          s.f32 = f32;
          if (op.type == "relu6") cb.Imm(ChainBuilder::Attr(op, "threshold", "6"), &s.imm);
          if (s.op == EW_RELU && int_class) {  // max(x, 0) with an integer zero
            s.op = EW_MAX;
            cb.Imm("0", &s.imm);
          }
          rev.push_back(s);
        }
        cur = op.inputs[0];
      } else if (cb.Binary().count(op.type)) {
        const std::string &a = op.inputs[0], &b = op.inputs[1];
        const bool ca = cb.InGroupComputed(a), cbb = cb.InGroupComputed(b);
        Step s;
        s.op  = cb.Binary().at(op.type);
        s.f32 = cb.Arith(cb.values[a].dtype);
        std::string next;
        if (ca && cbb) {
          // Both computed in the group: only the "value with itself" form is a chain.
          if (cb.IsSameAs(b, a)) { next = a; s.asel = 4; }
          else if (cb.IsSameAs(a, b)) { next = b; s.asel = 4; s.swap = true; }
          else if (temps_used < 2 && cb.values[a].numel() == cb.n && cb.values[b].numel() == cb.n) {
            // A tree: one operand is walked as a segment of its own, which runs first and is stashed in a temporary;
            // the other continues this walk.  For a float32 add the operand that continues is the product the
            // reference contracts into a fused multiply-add (the right one first, cinn/optim/lower_intrin.cc:45-50),
            // so that the Mul and the Add end up adjacent.
            bool chain_is_a = true;
            if (s.op == EW_ADD && s.f32) {
              if (single_use_mul(b)) chain_is_a = false;
              else if (single_use_mul(a)) chain_is_a = true;
            }
            const std::string sub = chain_is_a ? b : a;
            const int t           = temps_used++;
            Segment sg;
            if (!walk(sub, &sg)) return false;
            if (!finish_start(&sg, segments.empty())) return false;
            Step st;
            st.op   = EW_STASH;
            st.asel = 5 + t;
            st.f32  = false;
            sg.rev.insert(sg.rev.begin(), st);  // executed last in its segment
            segments.push_back(sg);
            next   = chain_is_a ? a : b;
            s.asel = 5 + t;
            s.swap = !chain_is_a;
          } else {
            cb.Fail("op '" + op.type + "' combines two values computed in the group (a tree, not a chain)");
            return false;
          }
        } else {
          bool chain_is_a;
          if (ca) chain_is_a = true;
          else if (cbb) chain_is_a = false;
          else {
            // Neither operand is computed in the group: the chain starts at the full-size group input.
            // (a group input itself, or a cast of one that the load performs: the walk continues through that cast)
            auto full_input = [&](const std::string& v) {
              if (cb.values[v].numel() != cb.n) return false;
              if (cb.input_index.count(v)) return true;
              const OpDesc* q = cb.producer.count(v) ? cb.producer[v] : nullptr;
              return q && cb.IsLoadCast(*q);
            };
            const bool a_full = full_input(a), b_full = full_input(b);
            // two constants (or a constant and a broadcast operand): the chain starts from a full-size constant
            auto full_constant = [&](const std::string& v) {
              const OpDesc* q = cb.producer.count(v) ? cb.producer[v] : nullptr;
              return q && q->type == "fill_constant" && cb.values[v].numel() == cb.n;
            };
            if (!a_full && !b_full && !full_constant(a) && !full_constant(b)) {
              cb.Fail("op '" + op.type + "' has no full-size operand to start the chain from");
              return false;
            }
            chain_is_a = a_full || (!b_full && full_constant(a));
          }
          next                     = chain_is_a ? a : b;
          const std::string& other = chain_is_a ? b : a;
          if (cb.IsSameAs(other, next)) {
            s.asel = 4;
          } else if (!cb.ResolveOperand(other, op, &s.asel, &s.imm)) {
            cb.Fail("operand '" + other + "' of '" + op.type + "' is neither a broadcastable group input nor a constant");
            return false;
          }
          s.swap = !chain_is_a;  // the side operand is the LEFT operand
        }
        if (!cb.Ok(cb.values[a].dtype) || !cb.Ok(cb.values[b].dtype)) {
          cb.Fail("op '" + op.type + "' on " + DTypeName(cb.values[a].dtype) + " operands does not fit this form of chain");
          return false;
        }
        s.single_use = uses[op.output] <= 1;
        round_after();
        rev.push_back(s);
        cur = next;
      } else if (op.type == "select") {
        // One of the three operands continues the chain; the other two are inputs, constants or the chain value.
        int chain_pos = -1;
        for (int k = 0; k < 3 && chain_pos < 0; ++k)
          if (cb.InGroupComputed(op.inputs[k])) chain_pos = k;
        for (int k = 0; k < 3; ++k)
          if (cb.InGroupComputed(op.inputs[k]) && k != chain_pos && !cb.IsSameAs(op.inputs[k], op.inputs[chain_pos])) {
            cb.Fail("select combines two values computed in the group (a tree, not a chain)");
            return false;
          }
        if (chain_pos < 0) {
          for (int k : {1, 2, 0})
            if (chain_pos < 0 && cb.input_index.count(op.inputs[k]) && cb.values[op.inputs[k]].numel() == cb.n &&
                cb.Ok(cb.values[op.inputs[k]].dtype))
              chain_pos = k;
          if (chain_pos < 0) {
            cb.Fail("select has no full-size operand to start the chain from");
            return false;
          }
        }
        Step s;
        s.op   = EW_SELECT;
        s.role = chain_pos;
        s.f32  = false;
        // operand A / B by role: role 0 -> (true, false); role 1 -> (cond, false); role 2 -> (cond, true)
        const int a_pos = chain_pos == 0 ? 1 : 0, b_pos = chain_pos == 2 ? 1 : 2;
        const std::string& chain = op.inputs[chain_pos];
        auto resolve = [&](int pos, int* sel, float* imm) {
          const std::string& nm = op.inputs[pos];
          if (!cb.Ok(cb.values[nm].dtype)) return false;
          if (cb.IsSameAs(nm, chain)) { *sel = 4; return true; }
          return cb.ResolveOperand(nm, op, sel, imm);
        };
        if (!cb.Ok(cb.values[chain].dtype) || !resolve(a_pos, &s.asel, &s.imm) || !resolve(b_pos, &s.bsel, &s.imm2)) {
          cb.Fail("an operand of select is neither a broadcastable group input nor a constant");
          return false;
        }
        round_after();
        rev.push_back(s);
        cur = chain;
      } else if (op.type == "fill_constant") {
        // The chain starts from a constant (EW_COPY of an immediate): no operand at all at this end.
        Step s;
        s.op   = EW_COPY;
        s.asel = 0;
        s.f32  = false;
        if (!cb.Imm(ChainBuilder::Attr(op, "value", "0"), &s.imm)) {
          cb.Fail("constant does not fit an immediate");
          return false;
        }
        rev.push_back(s);
        starts_from_operand = true;
        break;
      } else if (op.type == "broadcast_to" && cb.input_index.count(op.inputs[0])) {
        // No operand has the output's size: the chain starts from this broadcast operand (EW_COPY).
        Step s;
        s.op  = EW_COPY;
        s.f32 = false;
        if (!cb.ResolveOperand(cur, op, &s.asel, &s.imm)) {
          cb.Fail("the broadcast of '" + op.inputs[0] + "' cannot be addressed as a chain operand");
          return false;
        }
        rev.push_back(s);
        starts_from_operand = true;
        break;
      } else {
        cb.Fail("op '" + op.type + "' cannot be part of an elementwise chain");
        return false;
      }
    }
    seg->end = cur;
    return true;
  };
  Segment main_seg;
  if (!walk(out.name, &main_seg)) return nullptr;
  if (second && second_stores == 0 && allow_sibling) {
    // The second output is not on the way to the first: a sibling (two expressions over shared inputs, the
    // reference's horizontal fusion, cinn/hlir/pass/fusion_merge_pass.cc:85-460).  It is evaluated first as a segment
    // of its own that ends in the store; the main walk then restarts from its own input.
    Segment sg;
    if (!walk(second->name, &sg)) return nullptr;
    if (!finish_start(&sg, segments.empty())) return nullptr;
    segments.push_back(sg);
  }
  if (second && second_stores != 1) {
    cb.Fail("output '" + second->name + (second_stores ? "' would have to be stored more than once" : "' is not a value on the way to the other output"));
    return nullptr;
  }
  if (!finish_start(&main_seg, segments.empty())) return nullptr;
  // Program order: sub-segments (innermost first), then the main walk.
  std::vector<Step> rev;  // the whole program, reversed
  rev = main_seg.rev;
  for (auto it = segments.rbegin(); it != segments.rend(); ++it) rev.insert(rev.end(), it->rev.begin(), it->rev.end());
  const Segment& first_seg       = segments.empty() ? main_seg : segments.front();
  const bool starts_from_operand = first_seg.starts_from_operand;
  std::string cur                = first_seg.end;
  // in0 < 0: no pointer operand at all (a chain of constants); the output pointer fills the unused slots.
  const int in0       = starts_from_operand ? (cb.sides.empty() ? -1 : cb.sides[0].input) : cb.input_index[cur];
  const DType in_type = in0 >= 0 ? g.inputs[in0].dtype
                                 : (int_class ? cb.compute : (dbl_class ? DType::kFloat64 : DType::kFloat32));
  if (int_class && !IsIntType(in_type) && in_type != DType::kBool) {
    cb.Fail("an integer chain starts at an integer or bool input");
    return nullptr;
  }
  if (!dbl_class && !int_class && in_type == DType::kFloat64) {
    cb.Fail("float64 input");
    return nullptr;
  }
  if (DTypeKernelCode(in_type) < 0) {
    cb.Fail(std::string("input dtype ") + DTypeName(in_type) + " is not supported by the chain kernel");
    return nullptr;
  }
  // Every group input must be used (as the chain start or as a side operand).
  for (size_t i = 0; i < g.inputs.size(); ++i) {
    bool used = !starts_from_operand && (int)i == in0;
    for (auto& s : cb.sides) used = used || s.input == (int)i;
    if (!used) {
      cb.Fail("group input '" + g.inputs[i].name + "' is not reachable as a chain operand");
      return nullptr;
    }
  }

  // Forward order, then the Mul -> Add contraction (fp32 only), then encoding.
  std::vector<Step> steps(rev.rbegin(), rev.rend());
  std::vector<uint64_t> words;
  for (size_t i = 0; i < steps.size(); ++i) {
    const Step& s = steps[i];
    if (!int_class && s.op == EW_MUL && s.f32 && s.single_use && i + 1 < steps.size() && steps[i + 1].op == EW_ADD && steps[i + 1].f32 &&
        steps[i + 1].asel != 4) {
      const Step& a = steps[i + 1];
      words.push_back(Word(EW_FMA, s.asel, a.asel, 0, s.imm));
      if (a.asel == 0) words.push_back(Word(EW_NOP, 0, 0, 0, a.imm));
      ++i;
      continue;
    }
    if (s.op >= EW_FIRST_UNARY) {
      words.push_back(Word(s.op, 0, 0, 0, s.imm));
    } else if (s.op == EW_SELECT) {
      words.push_back(Word(EW_SELECT, s.asel, s.bsel, s.role, s.imm));
      if (s.bsel == 0) words.push_back(Word(EW_NOP, 0, 0, 0, s.imm2));
    } else {
      words.push_back(Word(s.op, s.asel, 0, s.swap ? 1 : 0, s.imm));
    }
  }
  if (words.size() > (size_t)EW_MAX_STEPS) {
    cb.Fail("chain of " + std::to_string(words.size()) + " steps exceeds the limit of " + std::to_string(EW_MAX_STEPS));
    return nullptr;
  }

  auto p      = std::make_unique<CompiledGroup>();
  p->name     = g.name;
  p->pattern  = "ew_chain";
  p->inputs   = g.inputs;
  p->outputs  = g.outputs;
  p->elements = cb.n;
  for (auto& t : g.inputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
  p->algorithmic_bytes += out.numel() * DTypeBytes(out.dtype);
  if (second) p->algorithmic_bytes += second->numel() * DTypeBytes(second->dtype);
  LaunchStep st;
  // _s3t: temporaries (and a second output); _s1o / _s3o: a second output without temporaries; else by operand count
  const std::string ns = temps_used > 0 ? "_s3t" : second ? (cb.sides.size() <= 1 ? "_s1o" : "_s3o") : std::string("_s") + (cb.sides.empty() ? "0" : (cb.sides.size() == 1 ? "1" : "3"));
  st.kernel = FindKernel(int_class ? std::string("ew_chain_int_") + DTypeKernelName(cb.compute) + "_" + DTypeKernelName(out.dtype) + ns
                         : dbl_class ? std::string("ew_chain_f64_") + DTypeKernelName(out.dtype) + ns
                                     : std::string("ew_chain_") + DTypeKernelName(out.dtype) + ns);
  if (!st.kernel) {
    cb.Fail("chain kernel for these dtypes is not in the library");
    return nullptr;
  }
  st.block[0] = 256;
  st.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(CeilDiv(cb.n, 8), 256), (int64_t)dev.sm_count * 16));
  auto in_arg = [](int i) {
    ArgSpec a;
    a.kind  = i >= 0 ? ArgSpec::kInput : ArgSpec::kOutput;
    a.index = i >= 0 ? i : 0;
    return a;
  };
  auto int_arg = [](int64_t v) { ArgSpec a; a.kind = ArgSpec::kInt; a.ivalue = v; return a; };
  st.args.push_back(in_arg(in0));
  int64_t meta = (int64_t)(starts_from_operand ? (int)EW_NO_INPUT : DTypeKernelCode(in_type)) << 24;
  ArgSpec aligned;
  aligned.kind   = ArgSpec::kAligned;
  aligned.ivalue = 1;
  if (in0 >= 0) aligned.aligned_inputs.push_back(in0);
  aligned.aligned_outputs.push_back(0);
  if (second) aligned.aligned_outputs.push_back(1);
  if (second) meta |= (int64_t)DTypeKernelCode(second->dtype) << 36;
  for (int k = 0; k < 3; ++k) {
    if (k < (int)cb.sides.size()) {
      const Side& s = cb.sides[k];
      st.args.push_back(in_arg(s.input));
      meta |= (int64_t)(DTypeKernelCode(g.inputs[s.input].dtype) | (s.mode << 4)) << (8 * k);
      if (s.mode == EW_SIDE_FULL || s.mode == EW_SIDE_PERIODIC_VEC) aligned.aligned_inputs.push_back(s.input);
    } else {
      st.args.push_back(in_arg(in0));  // unused pointer slot
    }
  }
  ArgSpec out_arg;
  out_arg.kind  = ArgSpec::kOutput;
  out_arg.index = final_idx;
  st.args.push_back(out_arg);
  st.args.push_back(int_arg(cb.n));
  st.args.push_back(aligned);
  st.args.push_back(int_arg(meta));
  for (int k = 0; k < 3; ++k) {
    st.args.push_back(int_arg(k < (int)cb.sides.size() ? cb.sides[k].mid : 1));
    st.args.push_back(int_arg(k < (int)cb.sides.size() ? cb.sides[k].inner : 1));
  }
  st.args.push_back(int_arg((int64_t)words.size()));
  for (int k = 0; k < EW_MAX_STEPS; ++k) st.args.push_back(int_arg(k < (int)words.size() ? (int64_t)words[k] : 0));
  if (dbl_class) {
    for (int k = 0; k < 8; ++k) {
      ArgSpec a;
      a.kind   = ArgSpec::kFloat;
      a.fvalue = k < (int)cb.dimms.size() ? cb.dimms[k] : 0.0;
      st.args.push_back(a);
    }
  }
  if (!int_class && !dbl_class) {  // the float kernels' last parameter: the second output (the first one when there is none)
    ArgSpec o2;
    o2.kind  = ArgSpec::kOutput;
    o2.index = second ? 1 - final_idx : final_idx;
    st.args.push_back(o2);
  }
  if (dev.enable_static_chains) {
    // A kernel specialised at build time for exactly this program (same operand types and addressing modes, same
    // ops and operand selectors; the immediates stay parameters) takes the interpreter's place: same parameters.
    uint32_t sig[EW_MAX_STEPS] = {0};
    for (size_t k = 0; k < words.size(); ++k) sig[k] = (uint32_t)(words[k] & 0xffffffffu);
    if (const KernelEntry* fixed = FindStaticChain(st.kernel->name, meta, (int)words.size(), sig)) st.kernel = fixed;
  }
  p->steps.push_back(st);
  return p;
}

namespace {

// x of `shape` reduced over `dims` seen as [outer, r, inner] (extent-1 axes ignored): the reduced axes must be adjacent.
bool AdjacentReduceView(const std::vector<int64_t>& shape, std::vector<int64_t> dims, int64_t* outer, int64_t* r, int64_t* inner) {
  const int nd = (int)shape.size();
  if (dims.empty())
    for (int i = 0; i < nd; ++i) dims.push_back(i);
  for (auto& d : dims) {
    if (d < 0) d += nd;
    if (d < 0 || d >= nd) return false;
  }
  *outer = *r = *inner = 1;
  int state            = 0;  // 0 outer, 1 reduce, 2 inner
  for (int i = 0; i < nd; ++i) {
    if (shape[i] == 1) continue;
    if (std::find(dims.begin(), dims.end(), (int64_t)i) != dims.end()) {
      if (state == 2) return false;
      state = 1;
      *r *= shape[i];
    } else {
      if (state == 1) state = 2;
      (state == 0 ? *outer : *inner) *= shape[i];
    }
  }
  return true;
}

std::vector<int64_t> DimList(const std::string& text) {
  std::vector<int64_t> v;
  std::stringstream ss(text);
  std::string item;
  while (std::getline(ss, item, ','))
    if (!item.empty()) v.push_back(atoll(item.c_str()));
  return v;
}

}  // namespace

// reduce_{sum,prod,max,min}(chain(inputs)) [-> cast to a 16-bit float]: the chain is matched as for the plain chain
// kernel (float form), then run as the first stage of the reduction kernels of chain_reduce.cu.  Returns nullptr
// without a reason when the group is not of this form at all.
std::unique_ptr<CompiledGroup> MatchChainReduce(const GroupDesc& g, const DeviceInfo& dev, std::string* why) {
  if (g.outputs.size() != 1 || g.ops.size() < 2) return nullptr;
  const TensorDesc& out = g.outputs[0];
  std::map<std::string, const OpDesc*> producer;
  std::map<std::string, int> uses;
  for (auto& op : g.ops) {
    producer[op.output] = &op;
    for (auto& in : op.inputs) ++uses[in];
  }
  if (!producer.count(out.name)) return nullptr;
  const OpDesc* top = producer[out.name];
  const OpDesc* red = top;
  if (top->type == "cast") {
    if (out.dtype != DType::kFloat16 && out.dtype != DType::kBFloat16) return nullptr;
    if (top->inputs.empty() || !producer.count(top->inputs[0])) return nullptr;
    red = producer[top->inputs[0]];
    if (uses[red->output] != 1) return nullptr;
  } else if (out.dtype != DType::kFloat32) {
    return nullptr;
  }
  static const std::map<std::string, int> kinds = {{"reduce_sum", 0}, {"reduce_prod", 1}, {"reduce_max", 2}, {"reduce_min", 3}};
  auto kind = kinds.find(red->type);
  if (kind == kinds.end() || red->inputs.size() != 1) return nullptr;
  const std::string t = red->inputs[0];
  if (!producer.count(t) || uses[t] != 1) return nullptr;  // a bare input is the plain reductions' business
  // The chain alone, as a group of its own whose output is the reduce's operand.
  GroupDesc chain = g;
  chain.ops.clear();
  for (auto& op : g.ops)
    if (&op != red && &op != top) chain.ops.push_back(op);
  std::string w;
  std::vector<int64_t> shape;
  {
    ChainBuilder probe(chain, &w);
    if (!probe.Infer() || !probe.values.count(t)) return nullptr;
    if (probe.values[t].dtype != DType::kFloat32) {
      if (why) *why = "a reduction fused with its producers is prebuilt for a float32 operand only";
      return nullptr;
    }
    shape = probe.values[t].shape;
  }
  chain.outputs.resize(1);
  chain.outputs[0].name  = t;
  chain.outputs[0].dtype = DType::kFloat32;
  chain.outputs[0].shape = shape;
  DeviceInfo interp = dev;
  interp.enable_static_chains = 0;  // the plan is re-targeted below; the reductions have their own static table
  auto plan = MatchChainOfClass(chain, interp, kFloatChain, &w);
  if (!plan) {
    if (why) *why = "the reduce's operand is not an elementwise chain: " + w;
    return nullptr;
  }
  int64_t outer, r, inner;
  auto it_dim = red->attrs.find("dim");
  if (!AdjacentReduceView(shape, DimList(it_dim == red->attrs.end() ? "" : it_dim->second), &outer, &r, &inner)) {
    if (why) *why = "reduce over non-adjacent axes has no prebuilt kernel";
    return nullptr;
  }
  if (out.numel() != outer * inner) {
    if (why) *why = "reduce output has " + std::to_string(out.numel()) + " elements, expected " + std::to_string(outer * inner);
    return nullptr;
  }
  // Re-target the chain's launch: same 31 parameters (the program, the side operands), reduce geometry appended.
  LaunchStep st    = plan->steps[0];
  st.args.resize(31);  // the chain kernel's own last parameter (its second output) is not one of these kernels'
  const std::string kname = st.kernel->name;
  const std::string ns    = kname.substr(kname.rfind('_'));  // "_s0" / "_s1" / "_s3" / "_s3t"
  auto int_arg = [](int64_t v) { ArgSpec a; a.kind = ArgSpec::kInt; a.ivalue = v; return a; };
  const int kOut = 4, kAligned = 6, kMeta = 7;
  const int64_t out_code = out.dtype == DType::kFloat16 ? EW_F16 : (out.dtype == DType::kBFloat16 ? EW_BF16 : EW_F32);
  st.args[kMeta].ivalue |= ((int64_t)kind->second << 28) | (out_code << 32);
  const int sms  = dev.sm_count;
  const bool f32 = out.dtype == DType::kFloat32;
  auto p         = std::make_unique<CompiledGroup>();
  p->name        = g.name;
  p->pattern     = inner == 1 ? "chain_row_reduce" : "chain_col_reduce";
  p->inputs      = g.inputs;
  p->outputs     = g.outputs;
  p->elements    = outer * r * inner;
  for (auto& x : g.inputs) p->algorithmic_bytes += x.numel() * DTypeBytes(x.dtype);
  p->algorithmic_bytes += out.numel() * DTypeBytes(out.dtype);
  // vectors of four: rows must start on a vector boundary / columns must come in fours; the chain's own side-operand
  // modes were chosen for the flat index, which both layouts keep.
  st.args[kAligned].ivalue = ((inner == 1 ? r : inner) % 4 == 0) ? 1 : 0;
  st.args[kAligned].aligned_outputs.clear();
  const char* opname = kind->second == 0 ? "sum" : (kind->second == 1 ? "prod" : (kind->second == 2 ? "max" : "min"));
  auto scratch_arg = [&](int64_t off) { ArgSpec a; a.kind = ArgSpec::kScratch; a.ivalue = off; return a; };
  // The kernel specialised at build time for this program and reduce op, when the library has one.
  auto specialised = [&](const KernelEntry* base) {
    if (!dev.enable_static_chains || !base) return base;
    const int nsteps = (int)st.args[14].ivalue;
    uint32_t sig[EW_MAX_STEPS] = {0};
    for (int k = 0; k < nsteps && k < EW_MAX_STEPS; ++k) sig[k] = (uint32_t)(st.args[15 + k].ivalue & 0xffffffff);
    const KernelEntry* fixed = FindStaticChain(base->name, st.args[kMeta].ivalue, nsteps, sig);
    return fixed ? fixed : base;
  };
  ArgSpec out_arg;
  out_arg.kind  = ArgSpec::kOutput;
  out_arg.index = 0;
  if (inner == 1) {
    int64_t S = 1;  // few long rows: segments of a row, folded by a second launch
    if (f32 && outer < (int64_t)sms * 2 && r >= 65536)
      while (S < 1024 && r % (S * 2) == 0 && (r / (S * 2)) % 4 == 0 && r / (S * 2) >= 4096 && outer * S < (int64_t)sms * 8) S *= 2;
    const int64_t rows = outer * S, len = r / S;
    st.kernel = specialised(FindKernel("chain_reduce_row" + ns));
    if (!st.kernel) return nullptr;
    const int64_t group = len > 2048 ? 256 : 32;
    st.block[0] = 256;
    st.grid[0]  = (unsigned)std::max<int64_t>(
        1, group == 32 ? std::min<int64_t>(CeilDiv(rows, 8), (int64_t)sms * 32) : std::min<int64_t>(rows, (int64_t)sms * 16));
    if (S > 1) {
      p->scratch_bytes = (size_t)(rows * 4 + 255) / 256 * 256;
      st.args[kOut]    = scratch_arg(0);
    }
    st.args.push_back(int_arg(rows));
    st.args.push_back(int_arg(len));
    st.args.push_back(int_arg(group));
    p->steps.push_back(st);
    if (S > 1) {
      LaunchStep f;
      f.kernel = FindKernel(std::string("reduce_generic_row_") + opname + "_f32");
      if (!f.kernel) return nullptr;
      f.block[0] = 256;
      f.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(outer, 8), (int64_t)sms * 32));
      f.args     = {scratch_arg(0), out_arg, int_arg(outer), int_arg(S), int_arg(32), int_arg(S % 4 == 0 ? 1 : 0)};
      p->steps.push_back(f);
    }
  } else {
    const int64_t cols = st.args[kAligned].ivalue ? inner / 4 : inner;
    const int64_t gx   = std::max<int64_t>(1, CeilDiv(cols, 256));
    int64_t S = 1;  // few columns: the reduced axis in segments, folded by a second launch
    if (f32 && outer * r * inner * 4 >= (4 << 20))
      while (gx * outer * S < (int64_t)sms * 4 && r / (S * 2) >= 16 && S < 64) S *= 2;
    const int64_t rows_per_split = CeilDiv(r, S);
    S                            = CeilDiv(r, rows_per_split);
    st.kernel = specialised(FindKernel("chain_reduce_col" + ns));
    if (!st.kernel) return nullptr;
    if (outer > 65535) {
      if (why) *why = "more than 65535 outer slices in a column reduction";
      return nullptr;
    }
    st.block[0] = 256;
    st.grid[0]  = (unsigned)gx;
    st.grid[1]  = (unsigned)outer;
    st.grid[2]  = (unsigned)S;
    if (S > 1) {
      p->scratch_bytes = (size_t)(S * outer * inner * 4 + 255) / 256 * 256;
      st.args[kOut]    = scratch_arg(0);
    }
    st.args.push_back(int_arg(outer));
    st.args.push_back(int_arg(r));
    st.args.push_back(int_arg(inner));
    st.args.push_back(int_arg(rows_per_split));
    p->steps.push_back(st);
    if (S > 1 && (outer * inner) % 4 == 0) {
      // few columns, S rows of partials: the rows over the warps of a CTA (reduce_generic.cu)
      LaunchStep f;
      f.kernel = FindKernel(std::string("reduce_generic_col_fold_") + opname + "_f32");
      if (!f.kernel) return nullptr;
      f.block[0] = 256;
      f.grid[0]  = (unsigned)CeilDiv(outer * inner / 4, 32);
      f.args     = {scratch_arg(0), out_arg, int_arg(S), int_arg(outer * inner)};
      p->steps.push_back(f);
    } else if (S > 1) {
      LaunchStep f;
      f.kernel = FindKernel(std::string("reduce_generic_col_") + opname + "_f32");
      if (!f.kernel) return nullptr;
      const int64_t total = outer * inner;
      ArgSpec al;
      al.kind   = ArgSpec::kAligned;
      al.ivalue = total % 4 == 0 ? 1 : 0;
      al.aligned_outputs.push_back(0);
      f.block[0] = 256;
      f.grid[0]  = (unsigned)std::max<int64_t>(1, CeilDiv(total % 4 == 0 ? total / 4 : total, 256));
      f.args     = {scratch_arg(0), out_arg, int_arg(1), int_arg(S), int_arg(total), int_arg(S), al};
      p->steps.push_back(f);
    }
  }
  return p;
}

std::unique_ptr<CompiledGroup> MatchGenericChain(const GroupDesc& g, const DeviceInfo& dev, std::string* why) {
  std::string why_float, why_other;
  if (auto p = MatchChainOfClass(g, dev, kFloatChain, &why_float)) return p;
  if (g.outputs.size() == 2) {
    // first the forms where one output lies on the way to the other (nothing is computed twice), then siblings
    std::string w;
    if (auto p = MatchChainOfClass(g, dev, kFloatChain, &w, 1)) return p;
    if (auto p = MatchChainOfClass(g, dev, kFloatChain, &w, 0, true)) return p;
    if (auto p = MatchChainOfClass(g, dev, kFloatChain, &w, 1, true)) return p;
  }
  bool has_int = false, has_f64 = false;
  for (auto& t : g.inputs) has_int = has_int || IsIntType(t.dtype), has_f64 = has_f64 || t.dtype == DType::kFloat64;
  for (auto& t : g.outputs) has_int = has_int || IsIntType(t.dtype), has_f64 = has_f64 || t.dtype == DType::kFloat64;
  if (why) *why = why_float;
  if (has_f64) {
    if (auto p = MatchChainOfClass(g, dev, kDoubleChain, &why_other)) return p;
    if (why) *why += "; as a float64 chain: " + why_other;
  }
  if (has_int) {
    if (auto p = MatchChainOfClass(g, dev, kIntChain, &why_other)) return p;
    if (why) *why += "; as an integer chain: " + why_other;
  }
  return nullptr;
}

}  // namespace cinn_b200

// ---- register programs ------------------------------------------------------------------------------------------------
// Elementwise groups that are not chains (ew_dag.cu) and groups with reductions over the trailing axes (row_prog.cu)
// are compiled into register programs: the ops are taken in their topological order and each live value holds one of
// DAG_REGS registers until its last use.  RegProgramBuilder emits one program segment at a time: the whole program of
// an elementwise group, or one element / scalar program of a row program.
namespace cinn_b200 {
namespace {

uint64_t DagWord(int op, int dst, int a, int b, int c, float imm) {
  uint32_t bits;
  memcpy(&bits, &imm, 4);
  return (uint64_t)(op & 0xff) | ((uint64_t)(dst & 15) << 8) | ((uint64_t)(a & 31) << 12) | ((uint64_t)(b & 31) << 17) |
         ((uint64_t)(c & 31) << 22) | ((uint64_t)bits << 32);
}

struct RegOperand {
  enum Kind { kReg, kImm } kind = kReg;
  int sel   = -1;  // register 0-7, or ROWP_SREG0 + k for a row scalar seen from an element program
  float imm = 0.0f;
};

// What happens to a value once its op has been emitted.
struct ValueAction {
  enum Kind { kNone, kStore, kAccumulate } kind = kNone;
  int index = 0;      // kStore: output index; kAccumulate: scalar register that receives the row's total
  int fold  = 0;      // kAccumulate: 0 sum, 1 prod, 2 max, 3 min
};

// What happens to values once computed: a value may be stored and folded into several accumulators (reduce_min and
// reduce_max of the same operand).
using ActionMap = std::multimap<std::string, ValueAction>;

struct RegProgramBuilder {
  ChainBuilder& cb;
  const GroupDesc& g;
  // Set by the caller -------------------------------------------------------------------------------------------
  std::map<std::string, std::string> alias;           // value -> the value it merely renames (no-op ops)
  std::map<std::string, int> uses;                    // uses of every value inside the whole group
  std::set<std::string> group_outputs;
  // Addressing of group input k in the index space of the segment being emitted (fills *side), false if impossible.
  std::function<bool(const std::string&, int, Side*)> address_input;
  // Selector of a value that lives outside the segment's register file (a row scalar seen from an element program),
  // or -1.
  std::function<int(const std::string&)> outside_selector = [](const std::string&) { return -1; };
  // State ---------------------------------------------------------------------------------------------------------
  std::vector<uint64_t> words;
  std::vector<bool> reg_busy = std::vector<bool>(DAG_REGS, false);
  std::map<std::string, int> reg_of;     // root value -> register
  std::map<std::string, int> remaining;  // root value -> uses still to come in this segment
  std::vector<Side> in_side;
  std::vector<bool> in_used;
  bool failed = false;

  RegProgramBuilder(ChainBuilder& c) : cb(c), g(c.g), in_side(c.g.inputs.size()), in_used(c.g.inputs.size(), false) {}

  void Fail(const std::string& m) {
    if (!failed) cb.Fail(m);
    failed = true;
  }
  std::string Root(const std::string& v) const {
    auto it = alias.find(v);
    return it == alias.end() ? v : Root(it->second);
  }
  bool ExactCast(const OpDesc& op) const {
    const DType from = cb.values.at(op.inputs[0]).dtype, to = cb.values.at(op.output).dtype;
    if (from == to) return true;
    if (to == DType::kFloat32) return from == DType::kFloat16 || from == DType::kBFloat16 || from == DType::kBool;
    if (from == DType::kBool) return IsFloatType(to);  // 0 / 1 are exact in every float type
    return false;
  }
  // Values that are only another value seen through a no-op (broadcast_to, identity, exact casts) are aliases, unless
  // they are group outputs (those need a register of their own to be stored from).
  void FindAliases(const std::function<bool(const OpDesc&)>& live) {
    for (auto& op : g.ops) {
      if (!live(op)) continue;
      const bool noop = op.type == "broadcast_to" || op.type == "identity" || (op.type == "cast" && ExactCast(op));
      if (noop && !group_outputs.count(op.output)) alias[op.output] = op.inputs[0];
    }
  }
  int Alloc() {
    for (int r = 0; r < DAG_REGS; ++r)
      if (!reg_busy[r]) {
        reg_busy[r] = true;
        return r;
      }
    Fail("more than eight values are live at once");
    return -1;
  }
  bool ConstantOf(const std::string& v, float* imm) const {
    const std::string r = Root(v);
    auto p = cb.producer.find(r);
    if (p == cb.producer.end() || p->second->type != "fill_constant") return false;
    *imm = (float)atof(ChainBuilder::Attr(*p->second, "value", "0").c_str());
    return true;
  }
  // The register, outside selector or immediate holding `v`; a group input is loaded on its first use.
  RegOperand Operand(const std::string& v) {
    RegOperand o;
    if (ConstantOf(v, &o.imm)) {
      o.kind = RegOperand::kImm;
      return o;
    }
    const std::string r = Root(v);
    const int outside   = outside_selector(r);
    if (outside >= 0) {
      o.sel = outside;
      return o;
    }
    auto it = reg_of.find(r);
    if (it != reg_of.end()) {
      o.sel = it->second;
      return o;
    }
    auto in = cb.input_index.find(r);
    if (in == cb.input_index.end()) {
      Fail("value '" + v + "' is used before it is computed");
      return o;
    }
    const int k = in->second;
    Side side;
    if (!address_input(r, k, &side)) {
      Fail("input '" + r + "' cannot be addressed from the index this part of the group runs over");
      return o;
    }
    if (in_used[k] && !(in_side[k] == side)) {
      Fail("input '" + r + "' is read at two different alignments");
      return o;
    }
    in_side[k] = side;
    in_used[k] = true;
    const int reg = Alloc();
    if (reg < 0) return o;
    words.push_back(DagWord(DAG_LOAD, reg, k, 0, 0, 0.0f));
    reg_of[r] = reg;
    o.sel     = reg;
    return o;
  }
  // One use of `v` has been emitted: its register is free after the last one.
  void Release(const std::string& v) {
    const std::string r = Root(v);
    auto it = remaining.find(r);
    if (it == remaining.end()) return;
    if (--it->second <= 0) {
      auto rg = reg_of.find(r);
      if (rg != reg_of.end()) {
        reg_busy[rg->second] = false;
        reg_of.erase(rg);
      }
    }
  }
  // The value will not be read again (by any segment): its register is free.
  void ForceFree(const std::string& v) {
    const std::string r = Root(v);
    remaining.erase(r);
    auto rg = reg_of.find(r);
    if (rg != reg_of.end()) {
      reg_busy[rg->second] = false;
      reg_of.erase(rg);
    }
  }
  // A Mul whose single consumer, a float32 Add, absorbs it as a fused multiply-add (cinn/optim/lower_intrin.cc:41-59).
  const OpDesc* ContractibleMul(const std::string& v, const std::set<std::string>& never) const {
    if (alias.count(v) || never.count(v)) return nullptr;  // the reference contracts the Mul node itself
    auto p = cb.producer.find(v);
    if (p == cb.producer.end() || p->second->type != "elementwise_mul") return nullptr;
    auto u = uses.find(v);
    if (u == uses.end() || u->second != 1 || group_outputs.count(v) || cb.values.at(v).dtype != DType::kFloat32) return nullptr;
    return p->second;
  }

  int Emit(int opc, const std::string& out, const std::vector<RegOperand>& ops, float imm_for_op, bool has_op_imm) {
    // immediates: at most two per step (the word's own and the next word's)
    float imms[2] = {0.0f, 0.0f};
    int n_imm     = 0;
    if (has_op_imm) imms[n_imm++] = imm_for_op;
    int sel[3] = {0, 0, 0};
    for (size_t i = 0; i < ops.size(); ++i) {
      if (ops[i].kind == RegOperand::kReg) {
        sel[i] = ops[i].sel;
        continue;
      }
      int found = -1;
      for (int q = has_op_imm ? 1 : 0; q < n_imm; ++q)
        if (memcmp(&imms[q], &ops[i].imm, 4) == 0) found = q;
      if (found < 0) {
        if (n_imm >= 2) {
          Fail("an op needs more than two constants");
          return -1;
        }
        imms[n_imm] = ops[i].imm;
        found       = n_imm++;
      }
      sel[i] = found == 0 ? DAG_IMM : DAG_IMM2;
    }
    const int dst = Alloc();
    if (dst < 0) return -1;
    words.push_back(DagWord(opc, dst, sel[0], sel[1], sel[2], imms[0]));
    if (n_imm == 2 || opc == EW_SCALE_PRE) words.push_back(DagWord(EW_NOP, 0, 0, 0, 0, imms[1]));
    reg_of[out] = dst;
    return dst;
  }

  // Emits `ops` (a topologically ordered subset of the group's ops, all of one index space).  `actions` says which
  // values are stored or accumulated once computed; `extra_uses` are uses of values outside this segment that must
  // keep their registers (scalar programs: values a later pass reads).  Values in `keep_mul` are never contracted
  // (they are reduce operands: materialised in the reference).
  bool EmitSegment(const std::vector<const OpDesc*>& ops, const ActionMap& actions,
                   const std::map<std::string, int>& extra_uses, const std::set<std::string>& keep_mul) {
    std::set<const OpDesc*> in_segment(ops.begin(), ops.end());
    for (const OpDesc* op : ops) {
      if (alias.count(op->output)) continue;
      for (auto& in : op->inputs) ++remaining[Root(in)];
    }
    for (auto& kv : actions) ++remaining[Root(kv.first)];
    for (auto& kv : extra_uses) remaining[Root(kv.first)] += kv.second;
    std::map<const OpDesc*, const OpDesc*> absorbed_by;  // mul -> add
    for (const OpDesc* op : ops) {
      if (op->type != "elementwise_add" || cb.values.at(op->output).dtype != DType::kFloat32) continue;
      for (int k : {1, 0}) {  // the right operand is tried first
        const OpDesc* m = ContractibleMul(op->inputs[k], keep_mul);
        if (m && in_segment.count(m)) {
          absorbed_by[m] = op;
          break;
        }
      }
    }
    for (const OpDesc* opp : ops) {
      const OpDesc& op = *opp;
      if (failed) return false;
      if (op.type == "fill_constant" || alias.count(op.output) || absorbed_by.count(opp)) continue;
      const DType out_t = cb.values.at(op.output).dtype;
      int dst = -1;
      const OpDesc* mul = nullptr;
      int mul_side      = -1;
      if (op.type == "elementwise_add" && out_t == DType::kFloat32)
        for (int k : {1, 0}) {
          const OpDesc* m = ContractibleMul(op.inputs[k], keep_mul);
          if (m && absorbed_by.count(m) && absorbed_by[m] == opp) {
            mul      = m;
            mul_side = k;
            break;
          }
        }
      if (mul) {
        std::vector<RegOperand> o = {Operand(mul->inputs[0]), Operand(mul->inputs[1]), Operand(op.inputs[1 - mul_side])};
        if (failed) return false;
        Release(mul->inputs[0]);
        Release(mul->inputs[1]);
        Release(op.inputs[1 - mul_side]);
        // the absorbed Mul's own result was counted as a use of the Add: it never gets a register
        remaining.erase(Root(op.inputs[mul_side]));
        dst = Emit(EW_FMA, op.output, o, 0.0f, false);
      } else if (op.type == "scale") {
        const float sc = (float)atof(ChainBuilder::Attr(op, "scale", "1").c_str());
        const float bi = (float)atof(ChainBuilder::Attr(op, "bias", "0").c_str());
        const std::string after = ChainBuilder::Attr(op, "bias_after_scale", "true");
        RegOperand x = Operand(op.inputs[0]);
        if (failed) return false;
        if (x.kind != RegOperand::kReg) {
          Fail("scale of a constant");
          return false;
        }
        Release(op.inputs[0]);
        if (after == "true" || after == "1" || after == "True") {
          RegOperand s2, b2;
          s2.kind = b2.kind = RegOperand::kImm;
          s2.imm  = sc;
          b2.imm  = bi;
          dst = Emit(EW_FMA, op.output, {x, s2, b2}, 0.0f, false);  // fma(x, scale, bias)
        } else {
          dst = Alloc();
          if (dst < 0) return false;
          words.push_back(DagWord(EW_SCALE_PRE, dst, x.sel, 0, 0, sc));  // scale * (x + bias)
          words.push_back(DagWord(EW_NOP, 0, 0, 0, 0, bi));
          reg_of[op.output] = dst;
        }
      } else if (op.type == "cast") {
        RegOperand x = Operand(op.inputs[0]);
        if (failed) return false;
        Release(op.inputs[0]);
        const int code = out_t == DType::kBool ? EW_TO_BOOL
                                               : (out_t == DType::kFloat16 ? EW_ROUND_F16
                                                                           : (out_t == DType::kBFloat16 ? EW_ROUND_BF16 : EW_IDENTITY));
        dst = Emit(code, op.output, {x}, 0.0f, false);
      } else if (op.type == "identity" || op.type == "broadcast_to") {  // a no-op that is a group output: a copy
        RegOperand x = Operand(op.inputs[0]);
        if (failed) return false;
        Release(op.inputs[0]);
        dst = Emit(EW_IDENTITY, op.output, {x}, 0.0f, false);
      } else if (op.type == "select") {
        std::vector<RegOperand> o = {Operand(op.inputs[0]), Operand(op.inputs[1]), Operand(op.inputs[2])};
        if (failed) return false;
        for (auto& in : op.inputs) Release(in);
        dst = Emit(EW_SELECT, op.output, o, 0.0f, false);
      } else if (UnaryCodes().count(op.type)) {
        RegOperand x = Operand(op.inputs[0]);
        if (failed) return false;
        Release(op.inputs[0]);
        if (op.type == "relu6")
          dst = Emit(EW_RELU6, op.output, {x}, (float)atof(ChainBuilder::Attr(op, "threshold", "6").c_str()), true);
        else
          dst = Emit(UnaryCodes().at(op.type), op.output, {x}, 0.0f, false);
      } else if (BinaryCodes().count(op.type)) {
        std::vector<RegOperand> o = {Operand(op.inputs[0]), Operand(op.inputs[1])};
        if (failed) return false;
        Release(op.inputs[0]);
        Release(op.inputs[1]);
        dst = Emit(BinaryCodes().at(op.type), op.output, o, 0.0f, false);
      } else {
        Fail("op '" + op.type + "' is not an elementwise op");
        return false;
      }
      if (failed || dst < 0) return false;
      // 16-bit values are rounded to their type after every op (a cast to that type IS the rounding)
      if (op.type != "cast" && (out_t == DType::kFloat16 || out_t == DType::kBFloat16))
        words.push_back(DagWord(out_t == DType::kFloat16 ? EW_ROUND_F16 : EW_ROUND_BF16, dst, dst, 0, 0, 0.0f));
      auto acts = actions.equal_range(op.output);
      for (auto act = acts.first; act != acts.second; ++act) {
        if (act->second.kind == ValueAction::kStore) words.push_back(DagWord(DAG_STORE, act->second.index, dst, 0, 0, 0.0f));
        if (act->second.kind == ValueAction::kAccumulate)
          words.push_back(DagWord(ROWP_ACC, act->second.index, dst, 0, act->second.fold, 0.0f));
        Release(op.output);
      }
      if (remaining.count(op.output) == 0 || remaining[op.output] <= 0) {  // nothing else reads it
        auto rg = reg_of.find(op.output);
        if (rg != reg_of.end()) {
          reg_busy[rg->second] = false;
          reg_of.erase(rg);
        }
      }
    }
    // targets that are not computed by an op of this segment: a group input (or a value held elsewhere) taken as is
    for (auto& kv : actions) {
      const std::string r = Root(kv.first);
      auto p = cb.producer.find(kv.first);
      const bool computed_here = p != cb.producer.end() && in_segment.count(p->second) && !alias.count(kv.first);
      if (computed_here) continue;
      RegOperand x = Operand(kv.first);
      if (failed) return false;
      if (x.kind != RegOperand::kReg || x.sel >= DAG_REGS) {
        Fail("value '" + kv.first + "' cannot be stored or reduced as it is");
        return false;
      }
      if (kv.second.kind == ValueAction::kStore) words.push_back(DagWord(DAG_STORE, kv.second.index, x.sel, 0, 0, 0.0f));
      if (kv.second.kind == ValueAction::kAccumulate) words.push_back(DagWord(ROWP_ACC, kv.second.index, x.sel, 0, kv.second.fold, 0.0f));
      Release(kv.first);
      (void)r;
    }
    return !failed;
  }
};

// Which output axis every dimension of every value sits on, walked back from `seeds` (value -> axes) through the ops
// `take` accepts.  Returns false (with the reason set) on an impossible or contradictory placement.
bool PlaceAxes(ChainBuilder& cb, const std::function<bool(const OpDesc&)>& take,
               std::map<std::string, std::vector<int64_t>>* axes) {
  bool conflict = false;
  auto place    = [&](const std::string& name, const std::vector<int64_t>& ax) {
    auto it = axes->find(name);
    if (it == axes->end()) (*axes)[name] = ax;
    else if (it->second != ax) conflict = true;
  };
  for (auto it = cb.g.ops.rbegin(); it != cb.g.ops.rend(); ++it) {
    const OpDesc& op = *it;
    if (!axes->count(op.output) || !take(op) || op.type == "fill_constant") continue;
    const std::vector<int64_t> oa = (*axes)[op.output];
    const Value& ov               = cb.values[op.output];
    if (op.type == "broadcast_to") {
      const Value& sv = cb.values[op.inputs[0]];
      std::vector<int64_t> bax = IntList(ChainBuilder::Attr(op, "broadcast_axes", ""));
      if (bax.size() != sv.shape.size()) {
        bax.clear();
        for (size_t i = 0; i < sv.shape.size(); ++i) bax.push_back((int64_t)(ov.shape.size() - sv.shape.size() + i));
      }
      std::vector<int64_t> ax;
      for (auto d : bax) {
        if (d < 0 || d >= (int64_t)oa.size()) return cb.Fail("broadcast_axes out of range");
        ax.push_back(oa[d]);
      }
      place(op.inputs[0], ax);
      continue;
    }
    const int64_t axis = atoll(ChainBuilder::Attr(op, "axis", "-1").c_str());
    for (auto& in : op.inputs) {
      const Value& sv = cb.values[in];
      if (sv.shape.size() == ov.shape.size()) {
        place(in, oa);
      } else if (sv.shape.size() < ov.shape.size()) {
        // cinn/hlir/pe/broadcast.cc:35-118: the lower-rank operand is aligned at `axis` (-1: right-aligned)
        const int64_t off = axis < 0 ? (int64_t)ov.shape.size() - (int64_t)sv.shape.size() : axis;
        std::vector<int64_t> ax;
        for (size_t i = 0; i < sv.shape.size(); ++i) {
          if (off + (int64_t)i >= (int64_t)oa.size()) return cb.Fail("operand of '" + op.type + "' does not fit at axis " + std::to_string(axis));
          ax.push_back(oa[off + i]);
        }
        place(in, ax);
      } else {
        return cb.Fail("operand of '" + op.type + "' has a higher rank than its result");
      }
    }
  }
  if (conflict) return cb.Fail("a value is used at two different alignments");
  return true;
}

bool StorableInFloatRegisters(ChainBuilder& cb) {
  for (auto& kv : cb.values)
    if (!IsFloatType(kv.second.dtype) && kv.second.dtype != DType::kBool)
      return cb.Fail(std::string("value of type ") + DTypeName(kv.second.dtype) + " in a float register program");
  return true;
}

ArgSpec IntArg(int64_t v) {
  ArgSpec a;
  a.kind   = ArgSpec::kInt;
  a.ivalue = v;
  return a;
}

// The pointer parameters (eight inputs, four outputs; unused slots repeat the first) and the meta word shared by the
// register-program kernels; `aligned` collects the buffers the vector path needs 16-byte aligned.
int64_t PushPointerArgs(const GroupDesc& g, const std::vector<Side>& in_side, LaunchStep* st, ArgSpec* aligned) {
  int64_t meta = 0;
  for (int k = 0; k < DAG_MAX_IN; ++k) {
    ArgSpec a;
    a.kind  = ArgSpec::kInput;
    a.index = k < (int)g.inputs.size() ? k : 0;
    st->args.push_back(a);
    if (k < (int)g.inputs.size()) {
      meta |= (int64_t)(DTypeKernelCode(g.inputs[k].dtype) | (in_side[k].mode << 3)) << (6 * k);
      if (in_side[k].mode == EW_SIDE_FULL || in_side[k].mode == EW_SIDE_PERIODIC_VEC) aligned->aligned_inputs.push_back(k);
    }
  }
  for (int k = 0; k < DAG_MAX_OUT; ++k) {
    ArgSpec a;
    a.kind  = ArgSpec::kOutput;
    a.index = k < (int)g.outputs.size() ? k : 0;
    st->args.push_back(a);
    if (k < (int)g.outputs.size()) meta |= (int64_t)DTypeKernelCode(g.outputs[k].dtype) << (48 + 3 * k);
  }
  return meta;
}

}  // namespace

std::unique_ptr<CompiledGroup> MatchDag(const GroupDesc& g, const DeviceInfo& dev, std::string* why) {
  ChainBuilder cb(g, why);
  if (g.outputs.empty() || g.outputs.size() > (size_t)DAG_MAX_OUT) {
    cb.Fail("a register program has one to four outputs");
    return nullptr;
  }
  if (g.inputs.size() > (size_t)DAG_MAX_IN) {
    cb.Fail("a register program reads at most eight tensors");
    return nullptr;
  }
  if (!cb.Infer() || !StorableInFloatRegisters(cb)) return nullptr;
  cb.out_shape = g.outputs[0].shape;
  cb.n         = g.outputs[0].numel();
  std::map<std::string, std::vector<int64_t>> axes;
  ActionMap actions;
  RegProgramBuilder rb(cb);
  for (size_t k = 0; k < g.outputs.size(); ++k) {
    const TensorDesc& o = g.outputs[k];
    if (o.shape != cb.out_shape) {
      cb.Fail("the outputs of a register program have one shape");
      return nullptr;
    }
    if (!cb.values.count(o.name) || cb.values[o.name].dtype != o.dtype || cb.values[o.name].shape != cb.out_shape ||
        !cb.producer.count(o.name) || cb.producer[o.name]->type == "fill_constant") {
      cb.Fail("output '" + o.name + "' is not a value of that type and shape computed in the group");
      return nullptr;
    }
    std::vector<int64_t> id;
    for (size_t i = 0; i < cb.out_shape.size(); ++i) id.push_back((int64_t)i);
    axes[o.name] = id;
    ValueAction act;
    act.kind  = ValueAction::kStore;
    act.index = (int)k;
    actions.insert({o.name, act});
    rb.group_outputs.insert(o.name);
  }
  if (!PlaceAxes(cb, [](const OpDesc&) { return true; }, &axes)) return nullptr;
  auto live = [&](const OpDesc& op) { return axes.count(op.output) > 0; };
  std::vector<const OpDesc*> ops;
  for (auto& op : g.ops)
    if (live(op)) {
      ops.push_back(&op);
      for (auto& in : op.inputs) ++rb.uses[in];
    }
  rb.FindAliases(live);
  rb.address_input = [&](const std::string& name, int k, Side* side) {
    auto ax = axes.find(name);
    return ax != axes.end() && cb.SideSpec(cb.values[name].shape, ax->second, k, side);
  };
  if (!rb.EmitSegment(ops, actions, {}, {})) return nullptr;
  if (rb.words.size() > (size_t)DAG_MAX_STEPS) {
    cb.Fail("register program of " + std::to_string(rb.words.size()) + " steps exceeds the limit of " + std::to_string(DAG_MAX_STEPS));
    return nullptr;
  }
  for (size_t i = 0; i < g.inputs.size(); ++i)
    if (!rb.in_used[i]) {
      cb.Fail("group input '" + g.inputs[i].name + "' is not used");
      return nullptr;
    }

  auto p      = std::make_unique<CompiledGroup>();
  p->name     = g.name;
  p->pattern  = "ew_dag";
  p->inputs   = g.inputs;
  p->outputs  = g.outputs;
  p->elements = cb.n;
  for (auto& t : g.inputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
  for (auto& t : g.outputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
  LaunchStep st;
  st.kernel = FindKernel("ew_dag");
  if (!st.kernel) {
    cb.Fail("the register-program kernel is not in the library");
    return nullptr;
  }
  st.block[0] = 256;
  st.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(CeilDiv(cb.n, 8), 256), (int64_t)dev.sm_count * 16));
  ArgSpec aligned;
  aligned.kind   = ArgSpec::kAligned;
  aligned.ivalue = 1;
  const int64_t meta = PushPointerArgs(g, rb.in_side, &st, &aligned);
  for (size_t k = 0; k < g.outputs.size(); ++k) aligned.aligned_outputs.push_back((int)k);
  st.args.push_back(IntArg(cb.n));
  st.args.push_back(aligned);
  st.args.push_back(IntArg(meta));
  for (int k = 0; k < DAG_MAX_IN; ++k) {
    st.args.push_back(IntArg(k < (int)g.inputs.size() ? rb.in_side[k].mid : 1));
    st.args.push_back(IntArg(k < (int)g.inputs.size() ? rb.in_side[k].inner : 1));
  }
  st.args.push_back(IntArg((int64_t)rb.words.size()));
  for (int k = 0; k < DAG_MAX_STEPS; ++k) st.args.push_back(IntArg(k < (int)rb.words.size() ? (int64_t)rb.words[k] : 0));
  if (dev.enable_static_chains) {
    uint32_t sig[40] = {0};
    for (size_t k = 0; k < rb.words.size(); ++k) sig[k] = (uint32_t)(rb.words[k] & 0xffffffffu);
    if (const KernelEntry* fixed = FindStaticChain("ew_dag", meta, (int)rb.words.size(), sig)) st.kernel = fixed;
  }
  p->steps.push_back(st);
  return p;
}

}  // namespace cinn_b200

// ---- row programs: reductions over the trailing axes with elementwise ops either side (row_prog.cu) -------------------
namespace cinn_b200 {

std::unique_ptr<CompiledGroup> MatchRowProgram(const GroupDesc& g, const DeviceInfo& dev, std::string* why) {
  ChainBuilder cb(g, why);
  cb.allow_reduce = true;
  if (g.outputs.empty() || g.outputs.size() > (size_t)DAG_MAX_OUT || g.inputs.size() > (size_t)DAG_MAX_IN) {
    cb.Fail("a row program has one to four outputs and reads at most eight tensors");
    return nullptr;
  }
  if (!cb.Infer() || !StorableInFloatRegisters(cb)) return nullptr;
  static const std::map<std::string, int> folds = {{"reduce_sum", 0}, {"reduce_prod", 1}, {"reduce_max", 2}, {"reduce_min", 3}};
  // ---- geometry: every reduce folds the same trailing axes of one full shape ----
  std::vector<int64_t> full;
  int lead = -1;
  std::vector<const OpDesc*> reduces;
  for (auto& op : g.ops) {
    if (op.type.rfind("reduce_", 0) != 0) continue;
    if (!folds.count(op.type)) {
      cb.Fail("'" + op.type + "' has no row-program form");
      return nullptr;
    }
    const Value& x = cb.values[op.inputs[0]];
    if (x.dtype != DType::kFloat32) {
      cb.Fail("a row program reduces float32 values");
      return nullptr;
    }
    std::vector<int64_t> dims = IntList(ChainBuilder::Attr(op, "dim", ""));
    const int nd = (int)x.shape.size();
    if (dims.empty())
      for (int i = 0; i < nd; ++i) dims.push_back(i);
    std::vector<bool> red(nd, false);
    for (auto d : dims) red[(d % nd + nd) % nd] = true;
    int first_red = nd;
    for (int i = nd - 1; i >= 0 && red[i]; --i) first_red = i;
    int count = 0;
    for (bool b2 : red) count += b2 ? 1 : 0;
    if (count != nd - first_red) {
      cb.Fail("a row program reduces trailing axes");
      return nullptr;
    }
    if (reduces.empty()) {
      full = x.shape;
      lead = first_red;
    } else if (x.shape != full || first_red != lead) {
      cb.Fail("the reductions of a row program fold the same axes of one shape");
      return nullptr;
    }
    reduces.push_back(&op);
  }
  if (reduces.empty()) {
    cb.Fail("no reduction in the group");
    return nullptr;
  }
  int64_t rows = 1, r = 1;
  for (int i = 0; i < (int)full.size(); ++i) (i < lead ? rows : r) *= full[i];
  const int64_t n = rows * r;
  if (r < 2 || r > 16384) {
    cb.Fail("a row program keeps rows of 2 to 16384 elements");
    return nullptr;
  }
  std::vector<int64_t> row_shape(full.begin(), full.begin() + lead);
  if (row_shape.empty()) row_shape.push_back(1);

  // ---- which values depend on a reduction, and where they live ----
  std::map<std::string, bool> dep_red;
  for (auto& t : g.inputs) dep_red[t.name] = false;
  for (auto& op : g.ops) {
    bool d = op.type.rfind("reduce_", 0) == 0;
    for (auto& in : op.inputs) d = d || dep_red[in];
    dep_red[op.output] = d;
  }
  auto is_row  = [&](const std::string& v) { return dep_red[v] && cb.values[v].numel() == rows; };
  auto is_full = [&](const std::string& v) { return cb.values[v].numel() == n && cb.values[v].shape.size() == full.size() && !is_row(v); };
  for (auto& op : g.ops)
    if (dep_red[op.output] && !is_row(op.output) && cb.values[op.output].numel() != n) {
      cb.Fail("value '" + op.output + "' is neither one per row nor one per element");
      return nullptr;
    }
  // avail: the pass after whose reduction a per-row value exists; need: the first pass that can evaluate a
  // per-element value (one after the last per-row value it reads)
  std::map<std::string, int> avail, need, pass_of_reduce;
  for (auto& t : g.inputs) need[t.name] = 0;
  for (auto& op : g.ops) {
    const std::string& o = op.output;
    if (!dep_red[o]) {
      need[o] = 0;
    } else if (op.type.rfind("reduce_", 0) == 0) {
      pass_of_reduce[o] = need[op.inputs[0]];
      avail[o]          = pass_of_reduce[o];
    } else if (is_row(o)) {
      int a = 0;
      for (auto& in : op.inputs)
        if (dep_red[in]) {
          if (!is_row(in)) {
            cb.Fail("a per-row value computed from a per-element one without a reduction");
            return nullptr;
          }
          a = std::max(a, avail[in]);
        }
      avail[o] = a;
    } else {
      int q = 0;
      for (auto& in : op.inputs) q = std::max(q, dep_red[in] && is_row(in) ? avail[in] + 1 : need[in]);
      need[o] = q;
    }
  }
  int npass = 0;
  for (auto& kv : pass_of_reduce) npass = std::max(npass, kv.second + 1);
  std::map<std::string, int> output_index;
  for (size_t k = 0; k < g.outputs.size(); ++k) {
    const TensorDesc& o = g.outputs[k];
    if (!cb.producer.count(o.name) || cb.values[o.name].dtype != o.dtype || cb.values[o.name].shape != o.shape) {
      cb.Fail("output '" + o.name + "' is not a value of that type and shape computed in the group");
      return nullptr;
    }
    if (is_row(o.name)) {
    } else if (is_full(o.name) && o.shape == full) {
      npass = std::max(npass, need[o.name] + 1);
    } else {
      cb.Fail("output '" + o.name + "' is neither one value per row nor a tensor of the reduced shape");
      return nullptr;
    }
    output_index[o.name] = (int)k;
  }
  if (npass > ROWP_MAX_PASSES) {
    cb.Fail("the reductions depend on one another more than three deep");
    return nullptr;
  }

  // ---- axes: per-element values against the full shape, per-row values against the row shape ----
  auto identity_axes = [](size_t rank) {
    std::vector<int64_t> id;
    for (size_t i = 0; i < rank; ++i) id.push_back((int64_t)i);
    return id;
  };
  std::map<std::string, std::vector<int64_t>> full_axes, row_axes;
  for (const OpDesc* red : reduces) full_axes[red->inputs[0]] = identity_axes(full.size());
  for (auto& o : g.outputs)
    if (!is_row(o.name)) full_axes[o.name] = identity_axes(full.size());
  auto element_op = [&](const OpDesc& op) { return op.type.rfind("reduce_", 0) != 0 && !is_row(op.output); };
  if (!PlaceAxes(cb, element_op, &full_axes)) return nullptr;
  // a per-row value read by a per-element op must lie along the leading axes
  for (auto& kv : full_axes) {
    if (!dep_red[kv.first] || !is_row(kv.first)) continue;
    const auto& shape = cb.values[kv.first].shape;
    int next = 0;
    for (size_t i = 0; i < shape.size(); ++i) {
      if (shape[i] == 1) continue;
      while (next < lead && full[next] == 1) ++next;
      if (next >= lead || kv.second[i] != next) {
        cb.Fail("per-row value '" + kv.first + "' is broadcast along an axis that is not reduced");
        return nullptr;
      }
      ++next;
    }
  }
  auto row_value_axes = [&](const std::string& v) {
    const auto& shape = cb.values[v].shape;
    std::vector<int64_t> ax;
    int next = 0;
    for (size_t i = 0; i < shape.size(); ++i) {
      if (shape[i] == 1 && !(next < lead && full[next] == 1)) {
        ax.push_back(0);  // an extent-1 axis kept by keep_dim: addressing ignores it
        continue;
      }
      ax.push_back(std::min<int64_t>(next, (int64_t)row_shape.size() - 1));
      ++next;
    }
    return ax;
  };
  for (auto& op : g.ops)
    if (dep_red[op.output] && is_row(op.output)) row_axes[op.output] = row_value_axes(op.output);
  auto scalar_op = [&](const OpDesc& op) { return op.type.rfind("reduce_", 0) != 0 && (is_row(op.output) || !dep_red[op.output]); };
  {
    // placements in the row space only matter below per-row values: walk from them
    ChainBuilder& c2 = cb;
    c2.out_shape     = row_shape;
    c2.n             = rows;
    if (!PlaceAxes(cb, scalar_op, &row_axes)) return nullptr;
  }

  // ---- uses and last uses ----
  std::map<std::string, int> uses;
  for (auto& op : g.ops)
    for (auto& in : op.inputs) ++uses[in];
  // what a set of targets needs, within one index space: ops in program order
  auto needed_ops = [&](const std::vector<std::string>& targets, bool scalar_space, int pass) {
    std::set<const OpDesc*> take;
    std::vector<std::string> stack = targets;
    while (!stack.empty()) {
      const std::string v = stack.back();
      stack.pop_back();
      auto p = cb.producer.find(v);
      if (p == cb.producer.end()) continue;  // a group input
      const OpDesc* op = p->second;
      if (op->type.rfind("reduce_", 0) == 0) continue;       // its total sits in a scalar register
      if (!scalar_space && dep_red[v] && is_row(v)) continue;  // a per-row value: read from its scalar register
      if (scalar_space && dep_red[v] && avail[v] < pass) continue;  // computed by an earlier scalar program
      if (!take.insert(op).second) continue;
      for (auto& in : op->inputs) stack.push_back(in);
    }
    std::vector<const OpDesc*> ordered;
    for (auto& op : g.ops)
      if (take.count(&op)) ordered.push_back(&op);
    return ordered;
  };
  // segment index 2p (element program of pass p) / 2p + 1 (scalar program) of the last read of every per-row value
  std::map<std::string, int> last_read;
  std::vector<std::vector<const OpDesc*>> seg_ops(2 * npass);
  std::vector<ActionMap> seg_actions(2 * npass);
  for (int p = 0; p < npass; ++p) {
    std::vector<std::string> et, st2;
    for (const OpDesc* red : reduces)
      if (pass_of_reduce[red->output] == p) et.push_back(red->inputs[0]);
    for (auto& o : g.outputs) {
      if (!is_row(o.name) && need[o.name] == p) {
        et.push_back(o.name);
        ValueAction a;
        a.kind  = ValueAction::kStore;
        a.index = output_index[o.name];
        seg_actions[2 * p].insert({o.name, a});
      }
      if (is_row(o.name) && avail[o.name] == p) {
        ValueAction a;
        a.kind  = ValueAction::kStore;
        a.index = output_index[o.name];
        seg_actions[2 * p + 1].insert({o.name, a});
      }
    }
    for (auto& op : g.ops)
      if (dep_red[op.output] && is_row(op.output) && op.type.rfind("reduce_", 0) != 0 && avail[op.output] == p) st2.push_back(op.output);
    seg_ops[2 * p]     = needed_ops(et, false, p);
    seg_ops[2 * p + 1] = needed_ops(st2, true, p);
    for (int s2 = 2 * p; s2 <= 2 * p + 1; ++s2)
      for (const OpDesc* op : seg_ops[s2])
        for (auto& in : op->inputs)
          if (dep_red[in] && is_row(in)) last_read[in] = s2;
    for (auto& kv : seg_actions[2 * p + 1]) last_read[kv.first] = std::max(last_read[kv.first], 2 * p + 1);
  }

  // ---- emission ----
  std::vector<Side> in_side(g.inputs.size());
  std::vector<int> in_space(g.inputs.size(), -1);  // 0 element space, 1 row space
  auto merge_sides = [&](const RegProgramBuilder& b2, int space) {
    for (size_t k = 0; k < g.inputs.size(); ++k) {
      if (!b2.in_used[k]) continue;
      if (in_space[k] >= 0 && (in_space[k] != space || !(in_side[k] == b2.in_side[k]))) {
        cb.Fail("input '" + g.inputs[k].name + "' is read both per element and per row");
        return false;
      }
      in_space[k] = space;
      in_side[k]  = b2.in_side[k];
    }
    return true;
  };
  std::set<std::string> reduce_operands;
  for (const OpDesc* red : reduces) reduce_operands.insert(red->inputs[0]);
  RegProgramBuilder sb(cb);  // the scalar registers persist over the passes
  sb.uses = uses;
  for (auto& o : g.outputs) sb.group_outputs.insert(o.name);
  auto live_all = [](const OpDesc&) { return true; };
  sb.FindAliases(live_all);
  // a broadcast of a per-row value to the full shape is the value itself, seen from an element program; every other
  // alias must stay inside one index space
  sb.address_input = [&](const std::string& name, int k, Side* side) {
    auto ax = row_axes.find(name);
    cb.out_shape = row_shape;
    cb.n         = rows;
    return ax != row_axes.end() && cb.SideSpec(cb.values[name].shape, ax->second, k, side);
  };
  std::vector<uint64_t> words;
  unsigned long long counts = 0;
  for (int p = 0; p < npass; ++p) {
    // element program
    RegProgramBuilder eb(cb);
    eb.uses          = uses;
    eb.group_outputs = sb.group_outputs;
    eb.alias         = sb.alias;
    eb.address_input = [&](const std::string& name, int k, Side* side) {
      auto ax = full_axes.find(name);
      cb.out_shape = full;
      cb.n         = n;
      return ax != full_axes.end() && cb.SideSpec(cb.values[name].shape, ax->second, k, side);
    };
    eb.outside_selector = [&](const std::string& root) {
      if (!(dep_red[root] && is_row(root))) return -1;
      auto it = sb.reg_of.find(root);
      return it == sb.reg_of.end() ? -1 : ROWP_SREG0 + it->second;
    };
    ActionMap actions = seg_actions[2 * p];
    for (const OpDesc* red : reduces) {
      if (pass_of_reduce[red->output] != p) continue;
      const int sreg = sb.Alloc();
      if (sreg < 0) return nullptr;
      sb.reg_of[red->output]    = sreg;
      sb.remaining[red->output] = 1;  // held until its last read (freed below)
      ValueAction a;
      a.kind  = ValueAction::kAccumulate;
      a.index = sreg;
      a.fold  = folds.at(red->type);
      actions.insert({red->inputs[0], a});
    }
    if (!eb.EmitSegment(seg_ops[2 * p], actions, {}, reduce_operands) || !merge_sides(eb, 0)) return nullptr;
    counts |= (unsigned long long)eb.words.size() << (8 * p);
    words.insert(words.end(), eb.words.begin(), eb.words.end());
    for (auto& kv : last_read)
      if (kv.second == 2 * p) sb.ForceFree(kv.first);
    // scalar program
    std::map<std::string, int> later;
    for (auto& kv : last_read)
      if (kv.second > 2 * p + 1) later[kv.first] = 1;
    const size_t before = sb.words.size();
    if (!sb.EmitSegment(seg_ops[2 * p + 1], seg_actions[2 * p + 1], later, {})) return nullptr;
    counts |= (unsigned long long)(sb.words.size() - before) << (32 + 8 * p);
    words.insert(words.end(), sb.words.begin() + before, sb.words.end());
    for (auto& kv : last_read)
      if (kv.second == 2 * p + 1) sb.ForceFree(kv.first);
    // values the scalar program loaded or computed for itself only are dead now
    for (auto it = sb.reg_of.begin(); it != sb.reg_of.end();) {
      if (!last_read.count(it->first) || last_read[it->first] <= 2 * p + 1) {
        sb.reg_busy[it->second] = false;
        sb.remaining.erase(it->first);
        it = sb.reg_of.erase(it);
      } else {
        ++it;
      }
    }
  }
  if (!merge_sides(sb, 1)) return nullptr;
  if (words.size() > (size_t)ROWP_MAX_STEPS) {
    cb.Fail("row program of " + std::to_string(words.size()) + " steps exceeds the limit of " + std::to_string(ROWP_MAX_STEPS));
    return nullptr;
  }
  for (size_t k = 0; k < g.inputs.size(); ++k)
    if (in_space[k] < 0) {
      cb.Fail("group input '" + g.inputs[k].name + "' is not used");
      return nullptr;
    }

  auto p      = std::make_unique<CompiledGroup>();
  p->name     = g.name;
  p->pattern  = "row_program";
  p->inputs   = g.inputs;
  p->outputs  = g.outputs;
  p->elements = n;
  for (auto& t : g.inputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
  for (auto& t : g.outputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
  LaunchStep st;
  st.kernel = FindKernel("row_program");
  if (!st.kernel) {
    cb.Fail("the row-program kernel is not in the library");
    return nullptr;
  }
  // A warp per row while a row's re-reads fit L1 with every warp of the SM on a row of its own (one pass: rows of
  // up to 16 KiB, read once; more passes: 4 KiB); else a CTA per row.
  int64_t group = r > (npass > 1 ? 1024 : 4096) ? 256 : 32;
  if (dev.rowp_form == 32 || dev.rowp_form == 256) group = dev.rowp_form;
  st.block[0] = 256;
  st.grid[0]  = (unsigned)std::max<int64_t>(1, group == 32 ? std::min<int64_t>(CeilDiv(rows, 8), (int64_t)dev.sm_count * 16)
                                                            : std::min<int64_t>(rows, (int64_t)dev.sm_count * 8));
  ArgSpec aligned;
  aligned.kind   = ArgSpec::kAligned;
  aligned.ivalue = r % 4 == 0 ? 1 : 0;
  const int64_t meta = PushPointerArgs(g, in_side, &st, &aligned);
  for (size_t k = 0; k < g.outputs.size(); ++k)
    if (!is_row(g.outputs[k].name)) aligned.aligned_outputs.push_back((int)k);
  st.args.push_back(IntArg(rows));
  st.args.push_back(IntArg(r));
  st.args.push_back(IntArg(group));
  st.args.push_back(aligned);
  st.args.push_back(IntArg(meta));
  st.args.push_back(IntArg((int64_t)counts));
  for (int k = 0; k < DAG_MAX_IN; ++k) {
    st.args.push_back(IntArg(k < (int)g.inputs.size() ? in_side[k].mid : 1));
    st.args.push_back(IntArg(k < (int)g.inputs.size() ? in_side[k].inner : 1));
  }
  for (int k = 0; k < ROWP_MAX_STEPS; ++k) st.args.push_back(IntArg(k < (int)words.size() ? (int64_t)words[k] : 0));
  if (dev.enable_static_chains) {
    uint32_t sig[40] = {(uint32_t)(counts & 0xffffffffu), (uint32_t)(counts >> 32)};
    for (size_t k = 0; k < words.size(); ++k) sig[k + 2] = (uint32_t)(words[k] & 0xffffffffu);
    // Half a CTA per row (two rows per CTA, a named barrier per half): only the specialised kernels have this form.
    // Taken for programs of several passes over rows of 1025 to 4096 elements (or on request).  Measured on B200,
    // 16384 x 4096, against a CTA per row: standardise (three passes) 0.94 of the HBM peak against 0.79, log_softmax
    // 0.91 against 0.72, l2_normalise 0.99 against 0.96, rms_norm 0.92 against 0.90.
    const bool half_ok = r % 4 == 0 && r <= 4096 && npass > 1;
    const bool half    = half_ok && (dev.rowp_form == 128 || (dev.rowp_form == 0 && group == 256));
    // Every form has, besides the kernel for any row, kernels for rows of exactly 2 ... 8 vectors per thread of the
    // row's group (no bounds tests: see row_program_body; a warp per row: 2 / 4 / 6 / 8 only); they are taken when
    // the row length is such a multiple.
    auto find = [&](const std::string& key, int64_t per_vector) -> const KernelEntry* {
      const KernelEntry* k = nullptr;
      if (npass > 1 && r % (4 * per_vector) == 0 && r / (4 * per_vector) >= (per_vector == 256 ? 5 : 2) && r / (4 * per_vector) <= 8)
        k = FindStaticChain((key + std::to_string(r / (4 * per_vector))).c_str(), meta, (int)words.size() + 2, sig);
      return k ? k : FindStaticChain(key.c_str(), meta, (int)words.size() + 2, sig);
    };
    const KernelEntry* fixed = nullptr;
    if (half) fixed = find("row_program_h", 128);
    if (fixed) {
      st.grid[0] = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(rows, 2), (int64_t)dev.sm_count * 8));
    } else if (r % 4 == 0 && r > 4096 && r <= 8192 && npass > 1 && group == 256 &&
               (fixed = find("row_program_c8", 256)) != nullptr) {
      // rows of 4097 to 8192 elements: a CTA per row with eight vectors per thread in registers between the passes
    } else {
      fixed = group == 32 ? find("row_program_w", 32) : FindStaticChain("row_program", meta, (int)words.size() + 2, sig);
    }
    // The specialised kernels evaluate the steps that a pass shares with the passes after it once per row
    // (row_prog_prefix.h), which is only the same arithmetic when those steps carry the same constants.  The builder
    // emits them from the same graph nodes, so they do; a program where they differ keeps the interpreting kernel.
    if (fixed) {
      const RowPrefixPlan plan = PlanRowPrefixes(sig + 2, counts, (unsigned long long)meta);
      for (int q = 1; q < npass && fixed; ++q)
        for (int k = 0; k < plan.start[q] && fixed; ++k)
          if ((words[row_prefix::ElementFirst(counts, q) + k] >> 32) != (words[row_prefix::ElementFirst(counts, q - 1) + k] >> 32))
            fixed = nullptr;
    }
    if (fixed) st.kernel = fixed;
  }
  p->steps.push_back(st);
  return p;
}

}  // namespace cinn_b200
