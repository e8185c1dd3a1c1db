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

#include "ew_chain.h"
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
      {"log10", EW_LOG10}, {"identity", EW_IDENTITY}};
  return m;
}
const std::map<std::string, int>& BinaryCodes() {
  static const std::map<std::string, int> m = {
      {"elementwise_add", EW_ADD}, {"subtract", EW_SUB},   {"elementwise_mul", EW_MUL}, {"divide", EW_DIV},
      {"max", EW_MAX},             {"min", EW_MIN},        {"pow", EW_POW},             {"equal", EW_EQ},
      {"not_equal", EW_NE},        {"greater_than", EW_GT}, {"less_than", EW_LT},       {"greater_equal", EW_GE},
      {"less_equal", EW_LE}};
  return m;
}

uint64_t Word(int op, int asel, int bsel, bool swap, float imm) {
  uint32_t bits;
  memcpy(&bits, &imm, 4);
  return (uint64_t)(op & 0xff) | ((uint64_t)(asel & 0xff) << 8) | ((uint64_t)(bsel & 0xff) << 16) |
         ((uint64_t)(swap ? 1 : 0) << 24) | ((uint64_t)bits << 32);
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

  ChainBuilder(const GroupDesc& g_, std::string* w) : g(g_), why(w) {}

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
      } else if (BinaryCodes().count(op.type)) {
        if (op.inputs.size() != 2) return Fail(op.type + " needs two operands");
        const Value &a = values[op.inputs[0]], &b = values[op.inputs[1]];
        v       = a.numel() >= b.numel() ? a : b;
        if (a.shape.size() != b.shape.size() && a.numel() == b.numel()) v = a.shape.size() >= b.shape.size() ? a : b;
        v.dtype = BinaryCodes().at(op.type) >= EW_EQ && BinaryCodes().at(op.type) <= EW_LE ? DType::kBool : a.dtype;
      } else if (UnaryCodes().count(op.type) || op.type == "scale") {
        if (op.inputs.size() != 1) return Fail(op.type + " needs one operand");
        v = values[op.inputs[0]];
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
      *imm  = (float)atof(Attr(*p, "value", "0").c_str());
      return true;
    }
    std::string src = name;
    std::vector<int64_t> axes;
    const Value* sv = &values[name];
    if (p && p->type == "broadcast_to") {
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
    if (sv->dtype != DType::kFloat32 && sv->dtype != DType::kFloat16 && sv->dtype != DType::kBFloat16) return false;
    Side s;
    if (!SideSpec(sv->shape, axes, input_index[src], &s)) return false;
    int sel = AddSide(s);
    if (sel < 0) return false;
    *asel = sel;
    return true;
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
    return true;
  }
};

int DTypeKernelCode(DType t) { return t == DType::kFloat32 ? 0 : (t == DType::kFloat16 ? 1 : (t == DType::kBFloat16 ? 2 : -1)); }
const char* DTypeKernelName(DType t) {
  switch (t) {
    case DType::kFloat32: return "f32";
    case DType::kFloat16: return "f16";
    case DType::kBFloat16: return "bf16";
    case DType::kBool: return "bool";
    default: return nullptr;
  }
}

}  // namespace

std::unique_ptr<CompiledGroup> MatchGenericChain(const GroupDesc& g, const DeviceInfo& dev, std::string* why) {
  ChainBuilder cb(g, why);
  if (g.outputs.size() != 1) {
    cb.Fail("a chain has exactly one output");
    return nullptr;
  }
  if (!cb.Infer()) return nullptr;
  const TensorDesc& out = g.outputs[0];
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

  // Walk back from the output collecting primitive steps in reverse order.
  std::vector<Step> rev;
  std::string cur = out.name;
  while (cb.producer.count(cur)) {
    const OpDesc& op = *cb.producer[cur];
    const Value& ov  = cb.values[cur];
    if (ov.numel() != cb.n) {
      cb.Fail("value '" + cur + "' on the chain has " + std::to_string(ov.numel()) + " elements, the output " + std::to_string(cb.n));
      return nullptr;
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
    const bool f32 = ov.dtype == DType::kFloat32;
    if (op.type == "cast") {
      const Value& iv = cb.values[op.inputs[0]];
      const bool in_float  = iv.dtype == DType::kFloat32 || iv.dtype == DType::kFloat16 || iv.dtype == DType::kBFloat16;
      const bool out_float = ov.dtype == DType::kFloat32 || ov.dtype == DType::kFloat16 || ov.dtype == DType::kBFloat16;
      if (!in_float || !out_float) {
        cb.Fail("cast between " + std::string(DTypeName(iv.dtype)) + " and " + DTypeName(ov.dtype) + " is not supported in a chain");
        return nullptr;
      }
      round_after();  // widening casts are exact and need no step
      cur = op.inputs[0];
    } else if (op.type == "scale") {
      const float s = (float)atof(ChainBuilder::Attr(op, "scale", "1").c_str());
      const float b = (float)atof(ChainBuilder::Attr(op, "bias", "0").c_str());
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
    } else if (UnaryCodes().count(op.type)) {
      round_after();
      if (op.type != "identity") {
        Step s;
        s.op  = UnaryCodes().at(op.type);
        s.f32 = f32;
        if (op.type == "relu6") s.imm = (float)atof(ChainBuilder::Attr(op, "threshold", "6").c_str());
        rev.push_back(s);
      }
      cur = op.inputs[0];
    } else if (BinaryCodes().count(op.type)) {
      const std::string &a = op.inputs[0], &b = op.inputs[1];
      const bool ca = cb.InGroupComputed(a), cbb = cb.InGroupComputed(b);
      Step s;
      s.op  = BinaryCodes().at(op.type);
      s.f32 = cb.values[a].dtype == DType::kFloat32;
      std::string next;
      if (ca && cbb) {
        // Both computed in the group: only the "value with itself" form is a chain.
        if (cb.IsSameAs(b, a)) { next = a; s.asel = 4; }
        else if (cb.IsSameAs(a, b)) { next = b; s.asel = 4; s.swap = true; }
        else {
          cb.Fail("op '" + op.type + "' combines two values computed in the group (a tree, not a chain)");
          return nullptr;
        }
      } else {
        bool chain_is_a;
        if (ca) chain_is_a = true;
        else if (cbb) chain_is_a = false;
        else {
          // Neither operand is computed in the group: the chain starts at the full-size group input.
          const bool a_full = cb.input_index.count(a) && cb.values[a].numel() == cb.n;
          const bool b_full = cb.input_index.count(b) && cb.values[b].numel() == cb.n;
          if (!a_full && !b_full) {
            cb.Fail("op '" + op.type + "' has no full-size operand to start the chain from");
            return nullptr;
          }
          chain_is_a = a_full;
        }
        next                     = chain_is_a ? a : b;
        const std::string& other = chain_is_a ? b : a;
        if (cb.IsSameAs(other, next)) {
          s.asel = 4;
        } else if (!cb.ResolveOperand(other, op, &s.asel, &s.imm)) {
          cb.Fail("operand '" + other + "' of '" + op.type + "' is neither a broadcastable group input nor a constant");
          return nullptr;
        }
        s.swap = !chain_is_a;  // the side operand is the LEFT operand
      }
      if (s.op >= EW_EQ && s.op <= EW_LE && cur != out.name) {
        cb.Fail("a comparison must be the last op of a chain");
        return nullptr;
      }
      round_after();
      rev.push_back(s);
      cur = next;
    } else {
      cb.Fail("op '" + op.type + "' cannot be part of an elementwise chain");
      return nullptr;
    }
  }
  if (!cb.input_index.count(cur) || cb.values[cur].numel() != cb.n) {
    cb.Fail("the chain does not start at a full-size group input");
    return nullptr;
  }
  const int in0       = cb.input_index[cur];
  const DType in_type = g.inputs[in0].dtype;
  if (DTypeKernelCode(in_type) < 0) {
    cb.Fail(std::string("input dtype ") + DTypeName(in_type) + " is not supported by the chain kernel");
    return nullptr;
  }
  // Every group input must be used (as the chain start or as a side operand).
  for (size_t i = 0; i < g.inputs.size(); ++i) {
    bool used = (int)i == in0;
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
    if (s.op == EW_MUL && s.f32 && i + 1 < steps.size() && steps[i + 1].op == EW_ADD && steps[i + 1].f32 &&
        steps[i + 1].asel != 4) {
      const Step& a = steps[i + 1];
      words.push_back(Word(EW_FMA, s.asel, a.asel, false, s.imm));
      if (a.asel == 0) words.push_back(Word(EW_NOP, 0, 0, false, a.imm));
      ++i;
      continue;
    }
    if (s.op >= EW_FIRST_UNARY)
      words.push_back(Word(s.op, 0, 0, false, s.imm));
    else
      words.push_back(Word(s.op, s.asel, 0, s.swap, s.imm));
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
  LaunchStep st;
  st.kernel = FindKernel(std::string("ew_chain_") + DTypeKernelName(in_type) + "_" + DTypeKernelName(out.dtype));
  if (!st.kernel) {
    cb.Fail("chain kernel for these dtypes is not in the library");
    return nullptr;
  }
  st.block[0] = 256;
  st.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(CeilDiv(cb.n, 8), 256), (int64_t)dev.sm_count * 16));
  auto in_arg = [](int i) { ArgSpec a; a.kind = ArgSpec::kInput; a.index = i; return a; };
  auto int_arg = [](int64_t v) { ArgSpec a; a.kind = ArgSpec::kInt; a.ivalue = v; return a; };
  st.args.push_back(in_arg(in0));
  int64_t meta = 0;
  ArgSpec aligned;
  aligned.kind   = ArgSpec::kAligned;
  aligned.ivalue = 1;
  aligned.aligned_inputs.push_back(in0);
  aligned.aligned_outputs.push_back(0);
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
  out_arg.index = 0;
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
  p->steps.push_back(st);
  return p;
}

}  // namespace cinn_b200
