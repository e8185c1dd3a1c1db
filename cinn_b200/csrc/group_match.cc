// Pattern matcher: fused group -> launch plan over the prebuilt kernels.
//
// This is "dispatch point #1": where the reference turns a Graph::Group into generated CUDA through
// OpLowerer::Lower (cinn/hlir/framework/op_lowering.cc:48-162) and CodegenAndJit
// (cinn/hlir/framework/parallel_compiler.cc:151-199), this file recognises the group's expression and picks a
// hand-written kernel plus its launch shape.  What each recognised expression computes is defined by the op
// semantics cited next to each matcher.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <functional>
#include <regex>
#include <set>
#include <sstream>

#include "group_desc.h"

namespace cinn_b200 {

std::unique_ptr<CompiledGroup> MatchGenericChain(const GroupDesc& g, const DeviceInfo& dev, std::string* why);  // chain_match.cc
std::unique_ptr<CompiledGroup> MatchChainReduce(const GroupDesc& g, const DeviceInfo& dev, std::string* why);   // chain_match.cc
std::unique_ptr<CompiledGroup> MatchDag(const GroupDesc& g, const DeviceInfo& dev, std::string* why);           // chain_match.cc
std::unique_ptr<CompiledGroup> MatchRowProgram(const GroupDesc& g, const DeviceInfo& dev, std::string* why);    // chain_match.cc

namespace {

int64_t CeilDiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
int64_t RoundUp(int64_t a, int64_t b) { return CeilDiv(a, b) * b; }

struct Matcher {
  const GroupDesc& g;
  const DeviceInfo& dev;
  std::string* err;
  std::map<std::string, const OpDesc*> producer;
  std::map<std::string, int> input_index;
  std::map<std::string, TensorDesc> values;  // every value with inferred dtype/shape

  Matcher(const GroupDesc& g_, const DeviceInfo& d, std::string* e) : g(g_), dev(d), err(e) {
    for (size_t i = 0; i < g.inputs.size(); ++i) {
      input_index[g.inputs[i].name] = (int)i;
      values[g.inputs[i].name]      = g.inputs[i];
    }
    for (auto& op : g.ops) producer[op.output] = &op;
  }

  bool Fail(const std::string& m) {
    if (err) *err = "group '" + g.name + "': " + m;
    return false;
  }

  // ---- attribute access ----------------------------------------------------------------------
  static bool HasAttr(const OpDesc& op, const char* k) { return op.attrs.count(k) != 0; }
  static std::string AttrS(const OpDesc& op, const char* k, const std::string& dflt) {
    auto it = op.attrs.find(k);
    return it == op.attrs.end() ? dflt : it->second;
  }
  static double AttrF(const OpDesc& op, const char* k, double dflt) {
    auto it = op.attrs.find(k);
    return it == op.attrs.end() ? dflt : atof(it->second.c_str());
  }
  static int64_t AttrI(const OpDesc& op, const char* k, int64_t dflt) {
    auto it = op.attrs.find(k);
    return it == op.attrs.end() ? dflt : atoll(it->second.c_str());
  }
  static bool AttrB(const OpDesc& op, const char* k, bool dflt) {
    auto it = op.attrs.find(k);
    if (it == op.attrs.end()) return dflt;
    return it->second == "1" || it->second == "true" || it->second == "True";
  }
  static std::vector<int64_t> AttrList(const OpDesc& op, const char* k) {
    std::vector<int64_t> out;
    auto it = op.attrs.find(k);
    if (it == op.attrs.end()) return out;
    std::string cur;
    for (char c : it->second + ",") {
      if (c == ',') {
        if (!cur.empty()) out.push_back(atoll(cur.c_str()));
        cur.clear();
      } else if (c != '[' && c != ']' && c != ' ') {
        cur.push_back(c);
      }
    }
    return out;
  }

  const OpDesc* Producer(const std::string& v) const {
    auto it = producer.find(v);
    return it == producer.end() ? nullptr : it->second;
  }
  // The op producing `v` if it has the given type, else nullptr.
  const OpDesc* ProducerOfType(const std::string& v, const char* type) const {
    const OpDesc* p = Producer(v);
    return (p && p->type == type) ? p : nullptr;
  }
  int InputIndex(const std::string& v) const {
    auto it = input_index.find(v);
    return it == input_index.end() ? -1 : it->second;
  }

  // ---- common pieces of a plan ---------------------------------------------------------------
  std::unique_ptr<CompiledGroup> NewPlan(const char* pattern) {
    auto p     = std::make_unique<CompiledGroup>();
    p->name    = g.name;
    p->pattern = pattern;
    p->inputs  = g.inputs;
    p->outputs = g.outputs;
    for (auto& t : g.inputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
    for (auto& t : g.outputs) p->algorithmic_bytes += t.numel() * DTypeBytes(t.dtype);
    p->elements = g.outputs[0].numel();
    return p;
  }
  static ArgSpec In(int i) {
    ArgSpec a;
    a.kind  = ArgSpec::kInput;
    a.index = i;
    return a;
  }
  static ArgSpec Out(int i) {
    ArgSpec a;
    a.kind  = ArgSpec::kOutput;
    a.index = i;
    return a;
  }
  static ArgSpec Scratch(int64_t offset) {
    ArgSpec a;
    a.kind   = ArgSpec::kScratch;
    a.ivalue = offset;
    return a;
  }
  static ArgSpec I(int64_t v) {
    ArgSpec a;
    a.kind   = ArgSpec::kInt;
    a.ivalue = v;
    return a;
  }
  static ArgSpec F(double v) {
    ArgSpec a;
    a.kind   = ArgSpec::kFloat;
    a.fvalue = v;
    return a;
  }
  // 16-bit storage of a group computed in fp32: float16 or bfloat16, the same on both sides.
  const char* half_name_ = "f16";
  bool SetHalfType(DType in, DType out) {
    if (in != out || (in != DType::kFloat16 && in != DType::kBFloat16)) return false;
    half_name_ = in == DType::kFloat16 ? "f16" : "bf16";
    return true;
  }
  // What the AutoCast pass leaves around a 16-bit batch norm (cinn/frontend/pass/auto_cast.cc:109-214): 16-bit inputs
  // widened to float32 by a cast at the load, the result narrowed by a cast at the end.  Returns the expression with
  // those casts removed ("cast(%2)" -> "%2", an outer "cast(...)" dropped) and sets *wide to the 16-bit type
  // (kFloat32 if there is none).  The kernels do the same conversions in their loads and stores.
  std::string StripHalfCasts(const std::string& expr, DType* wide) {
    *wide = DType::kFloat32;
    auto is_half = [](DType t) { return t == DType::kFloat16 || t == DType::kBFloat16; };
    std::string e = expr;
    for (size_t i = 0; i < g.inputs.size(); ++i) {
      if (!is_half(g.inputs[i].dtype)) continue;
      if (*wide != DType::kFloat32 && *wide != g.inputs[i].dtype) return expr;  // two different 16-bit types
      for (auto& op : g.ops)
        if (op.type == "cast" && op.inputs[0] == g.inputs[i].name && DTypeFromName(AttrS(op, "dtype", "")) != DType::kFloat32) return expr;
      *wide = g.inputs[i].dtype;
      const std::string from = "cast(%" + std::to_string(i) + ")", to = "%" + std::to_string(i);
      for (size_t pos = e.find(from); pos != std::string::npos; pos = e.find(from, pos + to.size())) e.replace(pos, from.size(), to);
    }
    if (*wide == DType::kFloat32) return expr;
    if (g.outputs.size() == 1 && is_half(g.outputs[0].dtype)) {
      const OpDesc* top = Producer(g.outputs[0].name);
      if (top && top->type == "relu" && g.outputs[0].dtype == *wide && e.rfind("relu(cast(", 0) == 0 && e.size() > 12 &&
          e.compare(e.size() - 2, 2, "))") == 0) {
        // relu after the narrowing cast (what AutoCast leaves of relu(batch_norm(x)) on 16-bit storage): rounding is
        // monotonic and keeps zero, so relu(cast(v)) and cast(relu(v)) are the same bits
        e = "relu(" + e.substr(10, e.size() - 12) + ")";
      } else {
        if (!top || top->type != "cast" || g.outputs[0].dtype != *wide || e.rfind("cast(", 0) != 0 || e.back() != ')') return expr;
        e = e.substr(5, e.size() - 6);
      }
    }
    half_name_ = *wide == DType::kFloat16 ? "f16" : "bf16";
    return e;
  }
  static ArgSpec Aligned(bool static_ok, std::vector<int> ins, std::vector<int> outs) {
    ArgSpec a;
    a.kind            = ArgSpec::kAligned;
    a.ivalue          = static_ok ? 1 : 0;
    a.aligned_inputs  = std::move(ins);
    a.aligned_outputs = std::move(outs);
    return a;
  }
  bool Kernel(LaunchStep* s, const std::string& name) {
    s->kernel = FindKernel(name);
    if (!s->kernel) return Fail("kernel '" + name + "' is not in the library");
    return true;
  }

  // ---- relu(elementwise_add(%0,%1)), fp32, equal shapes --------------------------------------
  // cinn/hlir/pe/broadcast.cc:216-273, cinn/hlir/pe/nn.cc:61-64.
  std::unique_ptr<CompiledGroup> MatchAddRelu(const std::string& expr) {
    if (expr != "relu(elementwise_add(%0,%1))" && expr != "relu(elementwise_add(%1,%0))") return nullptr;
    if (g.inputs.size() != 2) return nullptr;
    const auto &a = g.inputs[0], &b = g.inputs[1], &o = g.outputs[0];
    if (a.dtype != DType::kFloat32 || b.dtype != DType::kFloat32 || o.dtype != DType::kFloat32) return nullptr;
    if (a.shape != b.shape || a.numel() != o.numel()) return nullptr;
    auto p    = NewPlan("ew_add_relu");
    int64_t n = o.numel();
    LaunchStep s;
    if (!Kernel(&s, "ew_add_relu_f32")) return nullptr;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(CeilDiv(n, 4), 256), dev.sm_count * 32));
    s.args     = {In(0), In(1), Out(0), I(n), Aligned(true, {0, 1}, {0})};
    p->steps.push_back(s);
    return p;
  }

  // ---- cast(tanh(scale(elementwise_add(%0,%1)))) with %1 a vector on the last axis ------------
  // cinn/hlir/pe/broadcast.cc:35-273 (axis = -1 or ndim-1), cinn/hlir/op/elementwise.cc:149-163,
  // cinn/backends/llvm/llvm_intrin_rule.h:136-154, cinn/hlir/pe/elementwise.cc:213-217.
  std::unique_ptr<CompiledGroup> MatchBiasScaleTanhCast(const std::string& expr) {
    // The bias arrives either through the add's `axis` rule or, after the AutoBroadcast program pass, through an
    // explicit broadcast_to along the last axis (cinn/frontend/pass/auto_broadcast.cc:60-110), which then comes first
    // in the group and makes the bias input 0.
    int xi = 0, bi = 1;
    bool explicit_bc = false, with_cast = false, found = false;
    for (int form = 0; form < 3 && !found; ++form) {
      const std::string operands = form == 0 ? "%0,%1" : form == 1 ? "%0,broadcast_to(%1)" : "%1,broadcast_to(%0)";
      const std::string core     = "tanh(scale(elementwise_add(" + operands + ")))";
      if (expr != core && expr != "cast(" + core + ")") continue;
      found       = true;
      with_cast   = expr != core;
      explicit_bc = form > 0;
      if (form == 2) xi = 1, bi = 0;
    }
    if (!found || g.inputs.size() != 2) return nullptr;
    const auto &x = g.inputs[xi], &bias = g.inputs[bi], &o = g.outputs[0];
    if (x.dtype != DType::kFloat32 || bias.dtype != DType::kFloat32) return nullptr;
    if (x.shape.empty() || o.numel() != x.numel()) return nullptr;
    const int64_t cols = x.shape.back();
    if (!(bias.shape.size() == 1 && bias.shape[0] == cols)) return nullptr;
    const OpDesc* top   = Producer(o.name);
    const OpDesc* tanh  = with_cast ? Producer(top->inputs[0]) : top;
    const OpDesc* scale = Producer(tanh->inputs[0]);
    const OpDesc* add   = Producer(scale->inputs[0]);
    int64_t axis        = AttrI(*add, "axis", -1);
    if (explicit_bc) {
      const OpDesc* bc = Producer(add->inputs[1]);
      if (!bc || AttrList(*bc, "broadcast_axes") != std::vector<int64_t>{(int64_t)x.shape.size() - 1}) return nullptr;
    } else if (!(axis == -1 || axis == (int64_t)x.shape.size() - 1)) {
      return nullptr;
    }
    if (!AttrB(*scale, "bias_after_scale", true)) return nullptr;
    const char* suffix = nullptr;
    if (with_cast) {
      DType want = DTypeFromName(AttrS(*top, "dtype", "float32"));
      if (want != o.dtype) {
        Fail("cast dtype attribute does not match the output tensor's dtype");
        return nullptr;
      }
    }
    switch (o.dtype) {
      case DType::kFloat16: suffix = "f16"; break;
      case DType::kBFloat16: suffix = "bf16"; break;
      case DType::kFloat32: suffix = "f32"; break;
      default: return nullptr;
    }
    auto p    = NewPlan("ew_bias_scale_tanh_cast");
    int64_t n = x.numel();
    LaunchStep s;
    if (!Kernel(&s, std::string("ew_bias_scale_tanh_cast_f32_") + suffix)) return nullptr;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(CeilDiv(n, 8), 512), dev.sm_count * 32));
    if (dev.ew_reg_ctas_per_sm > 0) s.grid[0] = (unsigned)std::min<int64_t>(s.grid[0] * 2, (int64_t)dev.sm_count * dev.ew_reg_ctas_per_sm);
    s.args     = {In(xi), In(bi), Out(0), I(n), I(cols), Aligned(cols % 8 == 0, {0, 1}, {0}),
                  F((float)AttrF(*scale, "scale", 1.0)), F((float)AttrF(*scale, "bias", 0.0))};
    // Large 16-bit-output launches stream x through warp-private shared-memory rings filled by bulk copies
    // (ew_stream.cu); the register kernel above stays as the plan for unaligned buffers and small sizes.
    // Below some 32 M elements the register kernel is the faster one: measured on an 8.4 M-element slice (what one
    // of eight GPUs gets of 64x1024x1024) 11.1 us against 12.9 us for the rings, whose prologue and two waves of
    // CTAs do not amortise over one or two chunks per warp; at 67 M elements the rings win, 61.6 us against 64.6 us.
    const bool stream_ok = (o.dtype == DType::kFloat16 || o.dtype == DType::kBFloat16) && cols % 4 == 0 &&
                           (dev.enable_ew_stream > 1 ? n >= (int64_t)dev.sm_count * 8 * 512 * 8 : n >= (int64_t(1) << 25)) &&
                           dev.enable_ew_stream != 0;
    if (stream_ok) {
      LaunchStep t;
      if (!Kernel(&t, std::string("ew_bias_scale_tanh_cast_stream_f32_") + suffix)) return nullptr;
      // Measured on B200 (64x1024x1024): a ring of 2 buffers and a grid of 8 CTAs per SM (four resident at a time,
      // two waves) gives 0.975 of the HBM peak against 0.945 for the register kernel; deeper rings are slower.
      const int64_t stages = dev.ew_stream_stages > 0 ? std::min(dev.ew_stream_stages, 8) : 2;
      const int64_t smem   = 8 * stages * 2048;
      int64_t per_sm       = dev.ew_stream_ctas_per_sm > 0 ? dev.ew_stream_ctas_per_sm : 8;
      int64_t grid         = (int64_t)dev.sm_count * per_sm;
      // Prefer a warp count whose stride (warps * 512 elements) is a multiple of the row length: the bias values
      // of a lane are then the same for every chunk it handles.
      {
        int64_t a = 4096, b = cols;
        while (b) {
          int64_t r = a % b;
          a         = b;
          b         = r;
        }
        const int64_t need = cols / a;  // grid must be a multiple of this
        if (need <= grid) grid = grid / need * need;
      }
      t.block[0] = 256;
      t.grid[0]  = (unsigned)grid;
      t.dyn_smem = (size_t)smem;
      t.args     = {In(xi), In(bi), Out(0), I(n), I(cols), I(stages), F((float)AttrF(*scale, "scale", 1.0)),
                    F((float)AttrF(*scale, "bias", 0.0))};
      p->steps.push_back(t);
      p->steps_unaligned.push_back(s);
      p->aligned_inputs  = {0, 1};
      p->aligned_outputs = {0};
      return p;
    }
    p->steps.push_back(s);
    return p;
  }

  // ---- [cast(] [relu(] batch_norm(x, scale, bias, mean, variance) [)] [)] on NCHW ---------------
  // cinn/hlir/pe/nn.cc:700-721; argument order cinn/frontend/net_builder.cc:764-801.  The op itself is fp32
  // only (cinn/hlir/op/nn.cc:1078-1082); 16-bit storage is expressed as cast(..(cast(%0),..)).
  std::unique_ptr<CompiledGroup> MatchBatchNorm(const std::string& expr) {
    bool relu = false, half = false;
    if (expr == "relu(batch_norm(%0,%1,%2,%3,%4))") {
      relu = true;
    } else if (expr == "batch_norm(%0,%1,%2,%3,%4)") {
    } else if (expr == "cast(relu(batch_norm(cast(%0),%1,%2,%3,%4)))") {
      relu = half = true;
    } else if (expr == "cast(batch_norm(cast(%0),%1,%2,%3,%4))") {
      half = true;
    } else {
      return nullptr;
    }
    if (g.inputs.size() != 5) return nullptr;
    const auto &x = g.inputs[0], &o = g.outputs[0];
    if (x.shape.size() != 4 || o.shape != x.shape) return nullptr;
    if (half ? !SetHalfType(x.dtype, o.dtype)
             : (x.dtype != DType::kFloat32 || o.dtype != DType::kFloat32))
      return nullptr;
    const int64_t N = x.shape[0], C = x.shape[1], HW = x.shape[2] * x.shape[3];
    for (int i = 1; i < 5; ++i) {
      if (g.inputs[i].dtype != DType::kFloat32 || g.inputs[i].shape != std::vector<int64_t>{C}) {
        Fail("batch_norm parameters must be float32 vectors of length C");
        return nullptr;
      }
    }
    const OpDesc* bn = nullptr;
    for (auto& op : g.ops)
      if (op.type == "batch_norm") bn = &op;
    std::string layout = AttrS(*bn, "data_layout", "NCHW");
    if (layout != "NCHW") {
      Fail("batch_norm layout '" + layout + "' has no prebuilt kernel (NCHW only)");
      return nullptr;
    }
    const double eps = (float)AttrF(*bn, "epsilon", 1e-5);
    auto p           = NewPlan(relu ? "ew_bn_relu_nchw" : "ew_bn_nchw");
    const int V      = half ? 8 : 4;
    const int64_t planes = N * C;
    // A CTA takes about 1024 vectors of one plane; small problems get more, smaller chunks to fill the SMs.
    const int64_t units = HW % V == 0 ? HW / V : HW;
    int64_t chunks      = std::max<int64_t>(1, (units + 512) / 1024);
    while (planes * chunks < (int64_t)dev.sm_count * 4 && units / (chunks * 2) >= 256) chunks *= 2;
    LaunchStep s;
    if (!Kernel(&s, std::string(relu ? "ew_bn_relu_nchw_" : "ew_bn_nchw_") + (half ? half_name_ : "f32"))) return nullptr;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(planes * chunks, (int64_t)dev.sm_count * 64));
    s.args     = {In(0), In(1), In(2), In(3), In(4), Out(0), I(planes), I(C), I(HW), I(chunks),
                  Aligned(HW % V == 0, {0}, {0}), F(eps)};
    p->steps.push_back(s);
    return p;
  }

  // The normalisation group of the decomposed batch_norm_train (cinn/frontend/decomposer/batch_norm.cc:155-166):
  // add(mul(mul(sub(x, bc(mean)), rsqrt(add(bc(var), eps))), bc(scale)), bc(bias)), optionally under a relu.
  // Whatever the numbering of the inputs, the five operands are picked out of the expression.
  std::unique_ptr<CompiledGroup> MatchBnTrainApply(const std::string& expr) {
    static const std::regex form(
        R"(^(relu\()?elementwise_add\(elementwise_mul\(elementwise_mul\(subtract\(%(\d),broadcast_to\(%(\d)\)\),)"
        R"(rsqrt\(elementwise_add\(broadcast_to\(%(\d)\),fill_constant\(\)\)\)\),broadcast_to\(%(\d)\)\),broadcast_to\(%(\d)\)\)(\))?$)");
    std::smatch m;
    DType wide;
    const std::string stripped = StripHalfCasts(expr, &wide);
    if (!std::regex_match(stripped, m, form) || g.inputs.size() != 5) return nullptr;
    const bool relu = m[1].matched;
    if (relu != m[7].matched) return nullptr;
    const int ix = atoi(m[2].str().c_str()), im = atoi(m[3].str().c_str()), iv = atoi(m[4].str().c_str()),
              is = atoi(m[5].str().c_str()), ib = atoi(m[6].str().c_str());
    const std::set<int> distinct = {ix, im, iv, is, ib};
    if (distinct.size() != 5 || *distinct.rbegin() > 4) return nullptr;
    const auto &x = g.inputs[ix], &o = g.outputs[0];
    if (x.shape.size() != 4 || o.shape != x.shape || x.dtype != wide || o.dtype != wide) return nullptr;
    const int V = wide == DType::kFloat32 ? 4 : 8;
    const std::string tname = wide == DType::kFloat32 ? "f32" : half_name_;
    const int64_t N = x.shape[0], C = x.shape[1], HW = x.shape[2] * x.shape[3];
    for (int i : {im, iv, is, ib})
      if (g.inputs[i].dtype != DType::kFloat32 || g.inputs[i].numel() != C) return nullptr;
    double eps = 0.0;
    bool have_eps = false;
    for (auto& op : g.ops) {
      if (op.type == "broadcast_to") {
        const std::vector<int64_t> axes = AttrList(op, "broadcast_axes");
        if (axes != std::vector<int64_t>{1}) {
          Fail("batch_norm_train parameters must be broadcast along axis 1 (NCHW)");
          return nullptr;
        }
      } else if (op.type == "rsqrt") {
        const OpDesc* add = Producer(op.inputs[0]);
        for (auto& in : add->inputs)
          if (const OpDesc* fc = ProducerOfType(in, "fill_constant")) {
            eps      = (float)AttrF(*fc, "value", 1e-5);
            have_eps = true;
          }
      }
    }
    if (!have_eps) return nullptr;
    auto p = NewPlan(relu ? "ew_bn_train_apply_relu_nchw" : "ew_bn_train_apply_nchw");
    const int64_t planes = N * C;
    const int64_t units  = HW % V == 0 ? HW / V : HW;
    int64_t chunks       = std::max<int64_t>(1, (units + 512) / 1024);
    while (planes * chunks < (int64_t)dev.sm_count * 4 && units / (chunks * 2) >= 256) chunks *= 2;
    LaunchStep s;
    if (!Kernel(&s, std::string(relu ? "ew_bn_train_apply_relu_nchw_" : "ew_bn_train_apply_nchw_") + tname)) return nullptr;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(planes * chunks, (int64_t)dev.sm_count * 64));
    s.args     = {In(ix), In(is), In(ib), In(im), In(iv), Out(0), I(planes), I(C), I(HW), I(chunks),
                  Aligned(HW % V == 0, {ix}, {0}), F(eps)};
    p->steps.push_back(s);
    return p;
  }

  // x_grad of the decomposed batch_norm_grad (cinn/frontend/decomposer/batch_norm.cc:212-238):
  //   mul(tmp0, sub(sub(mul(dy, nhw), bc(bias_grad)), div(mul(sub(x, bc(mean)), bc(S)), bc(var + eps))))
  // tmp0 is broadcast(%t) or broadcast((scale * rsqrt(var + eps)) / nhw); var + eps is broadcast(%v) or computed.
  std::unique_ptr<CompiledGroup> MatchBnGradApply(const std::string& expr) {
    static const std::string t0 =
        R"(broadcast_to\((?:%(\d)|divide\(elementwise_mul\(%(\d),rsqrt\(elementwise_add\(%(\d),fill_constant\(\)\)\)\),fill_constant\(\)\))\))";
    static const std::string vae = R"(broadcast_to\((?:%(\d)|elementwise_add\(%(\d),fill_constant\(\)\))\))";
    static const std::regex form("^elementwise_mul\\(" + t0 +
                                 R"(,subtract\(subtract\(elementwise_mul\(%(\d),fill_constant\(\)\),broadcast_to\(%(\d)\)\),)"
                                 R"(divide\(elementwise_mul\(subtract\(%(\d),broadcast_to\(%(\d)\)\),broadcast_to\(%(\d)\)\),)" +
                                 vae + R"(\)\)\)$)");
    std::smatch m;
    DType wide;
    const std::string stripped = StripHalfCasts(expr, &wide);
    if (!std::regex_match(stripped, m, form)) return nullptr;
    auto idx = [&](int k) { return m[k].matched ? atoi(m[k].str().c_str()) : -1; };
    const int t0_in = idx(1), scale = idx(2), var0 = idx(3), dy = idx(4), db = idx(5), x = idx(6), mean = idx(7),
              S = idx(8), vae_in = idx(9), var1 = idx(10);
    const bool t0_form = t0_in < 0, vae_form = vae_in < 0;
    const auto& xt = g.inputs[x];
    const auto& o  = g.outputs[0];
    if (xt.shape.size() != 4 || g.inputs[dy].shape != xt.shape || o.shape != xt.shape || xt.dtype != wide ||
        g.inputs[dy].dtype != wide || o.dtype != wide || x == dy)
      return nullptr;
    const int V = wide == DType::kFloat32 ? 4 : 8;
    const int64_t N = xt.shape[0], C = xt.shape[1], HW = xt.shape[2] * xt.shape[3];
    for (int i : {t0_form ? scale : t0_in, t0_form ? var0 : mean, db, mean, S, vae_form ? var1 : vae_in})
      if (i < 0 || i >= (int)g.inputs.size() || g.inputs[i].dtype != DType::kFloat32 || g.inputs[i].numel() != C) return nullptr;
    double count = 0.0, eps = 0.0;
    for (auto& op : g.ops) {
      if (op.type == "broadcast_to" && AttrList(op, "broadcast_axes") != std::vector<int64_t>{1}) {
        Fail("batch_norm_grad operands must be broadcast along axis 1 (NCHW)");
        return nullptr;
      }
      const OpDesc* fc = nullptr;
      for (auto& in : op.inputs)
        if (const OpDesc* q = ProducerOfType(in, "fill_constant")) fc = q;
      if (!fc) continue;
      const double v = (float)AttrF(*fc, "value", 0.0);
      if (op.type == "elementwise_add") eps = v;
      else if (op.type == "elementwise_mul" || op.type == "divide") count = v;
    }
    if (count != (double)(N * HW)) {
      Fail("batch_norm_grad: the element count constant does not match the tensor");
      return nullptr;
    }
    auto p               = NewPlan("ew_bn_grad_apply_nchw");
    const int64_t planes = N * C;
    const int64_t units  = HW % V == 0 ? HW / V : HW;
    int64_t chunks       = std::max<int64_t>(1, (units + 256) / 512);
    while (planes * chunks < (int64_t)dev.sm_count * 4 && units / (chunks * 2) >= 256) chunks *= 2;
    LaunchStep s;
    if (!Kernel(&s, std::string("ew_bn_grad_apply_nchw_") + (wide == DType::kFloat32 ? "f32" : half_name_))) return nullptr;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(planes * chunks, (int64_t)dev.sm_count * 64));
    s.args     = {In(x), In(dy), In(mean), In(S), In(db), In(vae_form ? var1 : vae_in), In(t0_form ? scale : t0_in),
                  In(t0_form ? var0 : mean), Out(0), I(planes), I(C), I(HW), I(chunks), Aligned(HW % V == 0, {x, dy}, {0}),
                  I(t0_form ? 1 : 0), I(vae_form ? 1 : 0), F(count), F(eps)};
    p->steps.push_back(s);
    return p;
  }

  // ---- transpose / slice / concat (cinn/hlir/op/transform.cc): data movement, typed by element size ----------
  static std::vector<int64_t> StridesOf(const std::vector<int64_t>& shape) {
    std::vector<int64_t> st(shape.size(), 1);
    for (int i = (int)shape.size() - 2; i >= 0; --i) st[i] = st[i + 1] * shape[i + 1];
    return st;
  }

  bool GatherStep(CompiledGroup* p, int es, const std::vector<int64_t>& ext, const std::vector<int64_t>& str, int64_t base,
                  int64_t n) {
    if (ext.size() > 6) return Fail("more than six axes after merging have no prebuilt kernel");
    LaunchStep s;
    if (!Kernel(&s, "strided_gather_b" + std::to_string(es))) return false;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(n, 256), (int64_t)dev.sm_count * 32));
    s.args     = {In(0), Out(0), I(n), I(base), I((int64_t)ext.size())};
    for (int d = 0; d < 6; ++d) s.args.push_back(I(d < (int)ext.size() ? ext[d] : 1));
    for (int d = 0; d < 6; ++d) s.args.push_back(I(d < (int)str.size() ? str[d] : 0));
    p->steps.push_back(s);
    return true;
  }

  std::unique_ptr<CompiledGroup> MatchTransform(const std::string& expr) {
    static const std::regex concat_form(R"(^concat\((%\d+)(,%\d+)*\)$)");
    const bool is_concat = std::regex_match(expr, concat_form);
    if (expr != "transpose(%0)" && expr != "slice(%0)" && !is_concat) return nullptr;
    const auto& o     = g.outputs[0];
    const OpDesc& op  = g.ops.back();
    const int es      = DTypeBytes(o.dtype);
    for (auto& t : g.inputs)
      if (t.dtype != o.dtype) {
        Fail("operands and result must have one element type");
        return nullptr;
      }
    if (es != 1 && es != 2 && es != 4 && es != 8) return nullptr;
    if (is_concat) {
      const int nd = (int)o.shape.size();
      int64_t axis = AttrI(op, "axis", 0);
      if (axis < 0) axis += nd;
      if (axis < 0 || axis >= nd || g.inputs.size() != op.inputs.size()) {
        Fail("concat: bad axis or repeated operand");
        return nullptr;
      }
      int64_t outer = 1, inner = 1, total = 0;
      for (int i = 0; i < axis; ++i) outer *= o.shape[i];
      for (int i = axis + 1; i < nd; ++i) inner *= o.shape[i];
      for (auto& t : g.inputs) total += t.shape[axis];
      if (total != o.shape[axis]) {
        Fail("concat: operand extents do not add up to the output extent");
        return nullptr;
      }
      auto p      = NewPlan("concat_rows");
      p->elements = o.numel();
      for (int pass = 0; pass < 2; ++pass) {  // 0: widest unit (needs 16-byte aligned buffers), 1: element-sized units
        int ub = pass == 0 ? 16 : es;
        if (pass == 0) {
          int64_t all = o.shape[axis] * inner * es;
          int64_t off = 0;
          for (auto& t : g.inputs) {
            all |= t.shape[axis] * inner * es | off;
            off += t.shape[axis] * inner * es;
          }
          while (ub > es && all % ub != 0) ub /= 2;
        }
        std::vector<LaunchStep>& dst = pass == 0 ? p->steps : p->steps_unaligned;
        int64_t off_elems            = 0;
        for (size_t k = 0; k < g.inputs.size(); ++k) {
          // operands are bound in the order the op lists them
          int idx = -1;
          for (size_t q = 0; q < g.inputs.size(); ++q)
            if (g.inputs[q].name == op.inputs[k]) idx = (int)q;
          const int64_t w = g.inputs[idx].shape[axis] * inner;
          LaunchStep s;
          if (!Kernel(&s, "copy_rows_b" + std::to_string(ub))) return nullptr;
          const int64_t units = outer * w * es / ub;
          s.block[0] = 256;
          s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(units, 256), (int64_t)dev.sm_count * 32));
          s.args     = {In(idx), Out(0), I(outer), I(w * es / ub), I(o.shape[axis] * inner * es / ub), I(off_elems * es / ub)};
          if (units > 0) dst.push_back(s);
          off_elems += w;
        }
      }
      for (size_t q = 0; q < g.inputs.size(); ++q) p->aligned_inputs.push_back((int)q);
      p->aligned_outputs = {0};
      return p;
    }
    const auto& x = g.inputs[0];
    const int nd  = (int)x.shape.size();
    const std::vector<int64_t> in_str = StridesOf(x.shape);
    if (expr == "slice(%0)") {
      std::vector<int64_t> axes = AttrList(op, "axes"), starts = AttrList(op, "starts"), ends = AttrList(op, "ends"),
                           strides = AttrList(op, "strides");
      std::vector<int64_t> start(nd, 0), step(nd, 1), ext = x.shape;
      if (starts.size() != axes.size() || ends.size() != axes.size()) {
        Fail("slice: axes / starts / ends differ in length");
        return nullptr;
      }
      for (size_t k = 0; k < axes.size(); ++k) {
        int64_t a = axes[k] < 0 ? axes[k] + nd : axes[k];
        if (a < 0 || a >= nd) {
          Fail("slice: axis out of range");
          return nullptr;
        }
        // cinn/hlir/pe/transform.cc Slice: negative positions count from the end, positions are clamped
        const int64_t dim = x.shape[a], st = k < strides.size() ? strides[k] : 1;
        int64_t b = starts[k] < 0 ? starts[k] + dim : starts[k], e = ends[k] < 0 ? ends[k] + dim : ends[k];
        if (st > 0) {
          b = std::min(std::max<int64_t>(b, 0), dim);
          e = std::min(std::max<int64_t>(e, 0), dim);
          ext[a] = e > b ? CeilDiv(e - b, st) : 0;
        } else if (st < 0) {
          b = std::min(std::max<int64_t>(b, -1), dim - 1);
          e = std::min(std::max<int64_t>(e, -1), dim - 1);
          ext[a] = b > e ? CeilDiv(b - e, -st) : 0;
        } else {
          Fail("slice: zero stride");
          return nullptr;
        }
        start[a] = b;
        step[a]  = st;
      }
      int64_t n = 1, base = 0;
      std::vector<int64_t> e2, s2;
      for (int a = 0; a < nd; ++a) {
        n *= ext[a];
        base += start[a] * in_str[a];
        if (ext[a] != 1) {
          e2.push_back(ext[a]);
          s2.push_back(step[a] * in_str[a]);
        }
      }
      if (n != o.numel() || n == 0) {
        Fail("slice: the output has " + std::to_string(o.numel()) + " elements, the slice " + std::to_string(n));
        return nullptr;
      }
      auto p      = NewPlan("slice_gather");
      p->elements = n;
      if (!GatherStep(p.get(), es, e2, s2, base, n)) return nullptr;
      return p;
    }
    // transpose: out axis k is in axis perm[k]
    std::vector<int64_t> perm = AttrList(op, "axis");
    if ((int)perm.size() != nd) {
      Fail("transpose: 'axis' must list every axis");
      return nullptr;
    }
    std::vector<int64_t> ext, str, first;  // merged output axes: extent, input stride, first input axis of the run
    int64_t prev = -2;
    for (int k = 0; k < nd; ++k) {
      int64_t a = perm[k] < 0 ? perm[k] + nd : perm[k];
      if (a < 0 || a >= nd) {
        Fail("transpose: axis out of range");
        return nullptr;
      }
      if (x.shape[a] == 1) continue;
      // the next non-unit input axis after `prev`?
      int64_t nxt = prev + 1;
      while (prev >= 0 && nxt < nd && x.shape[nxt] == 1) ++nxt;
      if (prev >= 0 && a == nxt) {
        ext.back() *= x.shape[a];
        str.back() = in_str[a];
      } else {
        ext.push_back(x.shape[a]);
        str.push_back(in_str[a]);
        first.push_back(a);
      }
      prev = a;
    }
    const int m = (int)ext.size();
    const int64_t n = x.numel();
    if (n != o.numel()) {
      Fail("transpose: element counts differ");
      return nullptr;
    }
    bool tiled = m >= 2 && str[m - 2] == 1;  // the input's innermost run becomes the output's second-to-last
    for (int d = 0; tiled && d + 1 < m - 2; ++d) tiled = first[d] < first[d + 1];
    if (tiled && m >= 3) tiled = first[m - 3] < first[m - 1];
    if (tiled) tiled = first[m - 1] < first[m - 2];
    auto p      = NewPlan(tiled ? "transpose_tiled" : "transpose_gather");
    p->elements = n;
    if (tiled) {
      int64_t B = 1;
      for (int d = 0; d < m - 2; ++d) B *= ext[d];
      const int64_t C = ext[m - 2], R = ext[m - 1];
      LaunchStep s;
      if (!Kernel(&s, "transpose_tiled_b" + std::to_string(es))) return nullptr;
      s.block[0] = 256;
      const int64_t tiles = B * CeilDiv(R, 64) * CeilDiv(C, 64);
      s.grid[0] = (unsigned)std::max<int64_t>(1, std::min<int64_t>(tiles, (int64_t)dev.sm_count * 64));
      s.args    = {In(0), Out(0), I(B), I(R), I(C)};
      const int ve = 16 / es;
      if (R % ve == 0 && C % ve == 0) {
        // 16-byte accesses on both sides when the buffers are aligned; the element-wise tiles otherwise.
        LaunchStep v = s;
        if (!Kernel(&v, "transpose_vec_b" + std::to_string(es))) return nullptr;
        p->steps.push_back(v);
        p->steps_unaligned.push_back(s);
        p->aligned_inputs  = {0};
        p->aligned_outputs = {0};
      } else {
        p->steps.push_back(s);
      }
      return p;
    }
    if (!GatherStep(p.get(), es, ext, str, 0, n)) return nullptr;
    return p;
  }

  // ---- reduce_{sum,prod,max,min}(%0) -----------------------------------------------------------
  // cinn/hlir/op/reduction.cc:49-158 (dim normalisation: negative dims wrap, empty = all), cinn/hlir/pe/reduction.cc.
  static bool ReduceView(const std::vector<int64_t>& shape, std::vector<int64_t> dims, int64_t* outer, int64_t* r,
                         int64_t* inner) {
    const int nd = (int)shape.size();
    if (dims.empty())
      for (int i = 0; i < nd; ++i) dims.push_back(i);
    for (auto& d : dims)
      if (d < 0) d += nd;
    std::sort(dims.begin(), dims.end());
    dims.erase(std::unique(dims.begin(), dims.end()), dims.end());
    for (auto d : dims)
      if (d < 0 || d >= nd) return false;
    // Drop extent-1 axes from consideration, then the reduced axes must be contiguous.
    std::vector<int> kind;  // 0 keep, 1 reduce, per non-unit axis
    std::vector<int64_t> ext;
    for (int i = 0; i < nd; ++i) {
      if (shape[i] == 1) continue;
      kind.push_back(std::binary_search(dims.begin(), dims.end(), (int64_t)i) ? 1 : 0);
      ext.push_back(shape[i]);
    }
    *outer = *r = *inner = 1;
    int state            = 0;  // 0 outer, 1 reduce, 2 inner
    for (size_t i = 0; i < kind.size(); ++i) {
      if (kind[i] == 1) {
        if (state == 2) return false;
        state = 1;
        *r *= ext[i];
      } else {
        if (state == 1) state = 2;
        if (state == 0) *outer *= ext[i];
        else *inner *= ext[i];
      }
    }
    return true;
  }

  // x viewed as [A, B, I] with the axes of A and I reduced and those of B kept (extent-1 axes ignored): the
  // reduced axes form a leading and a trailing block, e.g. dims {0, 2, 3} of an NCHW tensor.
  static bool MidKeepView(const std::vector<int64_t>& shape, std::vector<int64_t> dims, int64_t* A, int64_t* B,
                          int64_t* I) {
    const int nd = (int)shape.size();
    for (auto& d : dims)
      if (d < 0) d += nd;
    std::sort(dims.begin(), dims.end());
    *A = *B = *I = 1;
    int state    = 0;  // 0 leading reduced block, 1 kept block, 2 trailing reduced block
    for (int i = 0; i < nd; ++i) {
      if (shape[i] == 1) continue;
      const bool red = std::binary_search(dims.begin(), dims.end(), (int64_t)i);
      if (state == 0 && !red) state = 1;
      else if (state == 1 && red) state = 2;
      else if (state == 2 && !red) return false;
      (state == 0 ? *A : (state == 1 ? *B : *I)) *= shape[i];
    }
    return state == 2 && *A > 1;
  }

  // First pass of a middle-axis-keeping reduction into scratch partials [splits][B] (per accumulation), then a
  // column reduction over the splits.  opname2 != nullptr: the dual kernel (sum and sum of squares).
  bool PlanMidKeep(CompiledGroup* p, const char* opname, bool dual, int64_t A, int64_t B, int64_t I, ArgSpec dst,
                   ArgSpec dst2, int x_in = 0, int x2_in = -1, int mean_in = -1, DType storage = DType::kFloat32) {
    const int sms        = dev.sm_count;
    const int V          = storage == DType::kFloat32 ? 4 : 8;  // elements per 16-byte vector
    const char* tname    = storage == DType::kFloat32 ? "f32" : (storage == DType::kFloat16 ? "f16" : "bf16");
    const bool vec       = I % V == 0;
    const int64_t units  = vec ? I / V : I;
    const int64_t chunks = std::max<int64_t>(1, (units + 2048) / 4096);  // about 4096 vectors per work item
    const int64_t items  = A * chunks;
    if (items >= (int64_t)1 << 31) return Fail("reduction with more than 2^31 work items");
    // Several waves of small CTAs (5 are resident per SM) balance better than one wave of large ones (measured).
    int64_t splits       = std::max<int64_t>(1, std::min<int64_t>(items, CeilDiv((int64_t)sms * 32, B)));
    const int64_t off1   = p->scratch_bytes;
    p->scratch_bytes += (size_t)RoundUp(splits * B * 4, 256);
    const int64_t off2 = p->scratch_bytes;
    if (dual) p->scratch_bytes += (size_t)RoundUp(splits * B * 4, 256);
    const int64_t off_tickets = p->scratch_bytes;  // one counter per kept element; scratch starts zeroed
    p->scratch_bytes += (size_t)RoundUp(B * 4, 256);
    LaunchStep s;
    const bool grad = x2_in >= 0;
    if (storage != DType::kFloat32 && !grad && !dual) return Fail("16-bit channel reductions are prebuilt for the statistics pair only");
    if (!Kernel(&s, grad ? std::string("bn_grad_stats_") + tname
                         : (dual ? std::string("mid_keep_reduce_sum_sumsq_") + tname : std::string("mid_keep_reduce_") + opname + "_f32")))
      return false;
    s.block[0] = 256;
    s.grid[0]  = (unsigned)(B * splits);
    std::vector<int> aligned_in = {x_in};
    if (grad) aligned_in.push_back(x2_in);
    s.args = {In(x_in), In(grad ? x2_in : x_in), In(grad ? mean_in : x_in), Scratch(off1), Scratch(dual ? off2 : off1),
              Scratch(off_tickets), dst, dual ? dst2 : dst, this->I(A), this->I(B), this->I(I), this->I(chunks),
              this->I(splits), Aligned(vec, aligned_in, {})};
    p->steps.push_back(s);
    return true;
  }

  bool PlanReduce(CompiledGroup* p, const char* opname, int64_t outer, int64_t r, int64_t inner, ArgSpec src,
                  ArgSpec dst, std::vector<int> src_in_for_align) {
    const int sms = dev.sm_count;
    if (inner == 1) {
      const int64_t rows = outer;
      const bool vec     = r % 4 == 0;
      if (r <= 2048) {
        int iters = 1;
        while (iters * 128 < r) iters *= 2;
        LaunchStep s;
        if (!Kernel(&s, "row_reduce_warp" + std::to_string(iters) + "_" + opname + "_f32")) return false;
        s.block[0] = 256;
        s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(rows, 8), (int64_t)sms * 64));
        s.args     = {src, dst, I(rows), I(r), Aligned(vec, src_in_for_align, {})};
        p->steps.push_back(s);
        return true;
      }
      const unsigned block = r >= 16384 ? 512 : 256;
      if (rows >= (int64_t)sms * 2 || r < 32768) {
        LaunchStep s;
        if (!Kernel(&s, std::string("row_reduce_cta_") + opname + "_f32")) return false;
        s.block[0] = block;
        s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(rows, (int64_t)sms * 32));
        s.args     = {src, dst, I(rows), I(r), I(1), I(RoundUp(r, 4)), Aligned(vec, src_in_for_align, {})};
        p->steps.push_back(s);
        return true;
      }
      if (rows * 8 >= sms) {
        // A cluster of 8 CTAs per row merges partials through distributed shared memory: one launch.
        const int64_t csize = 8;
        LaunchStep s;
        if (!Kernel(&s, std::string("row_reduce_cluster_") + opname + "_f32")) return false;
        s.block[0] = 512;
        s.cluster  = (unsigned)csize;
        s.grid[0]  = (unsigned)(std::min<int64_t>(rows, std::max<int64_t>(1, (int64_t)sms * 2 / csize)) * csize);
        s.args     = {src, dst, I(rows), I(r), I(RoundUp(CeilDiv(r, csize), 4)), Aligned(vec, src_in_for_align, {})};
        p->steps.push_back(s);
        return true;
      }
      // Few, very long rows: split every row over many CTAs into scratch partials, then finish.
      int64_t splits = std::min<int64_t>(CeilDiv((int64_t)sms * 4, rows), std::max<int64_t>(1, r / 8192));
      splits         = std::min<int64_t>(splits, 2048);
      const int64_t seg = RoundUp(CeilDiv(r, splits), 4);
      splits            = CeilDiv(r, seg);
      const int64_t scratch_off = p->scratch_bytes;
      p->scratch_bytes += (size_t)RoundUp(rows * splits * 4, 256);
      LaunchStep s1;
      if (!Kernel(&s1, std::string("row_reduce_cta_") + opname + "_f32")) return false;
      s1.block[0] = 512;
      s1.grid[0]  = (unsigned)(rows * splits);
      s1.args = {src, Scratch(scratch_off), I(rows), I(r), I(splits), I(seg), Aligned(vec, src_in_for_align, {})};
      p->steps.push_back(s1);
      // The partials of a sum are summed; of max/min/prod combined with the same op.
      return PlanReduceFinishRows(p, BaseReduceOp(opname), rows, splits, Scratch(scratch_off), dst);
    }
    // inner > 1: column reduction.
    const bool vec       = inner % 4 == 0;
    const int64_t cols   = vec ? inner / 4 : inner;
    const int64_t thr    = cols * outer;
    int64_t splits       = 1;
    if (thr < (int64_t)sms * 1024 && r >= 64) {
      splits = std::min<int64_t>(r / 32, CeilDiv((int64_t)sms * 2048, thr));
      splits = std::max<int64_t>(1, std::min<int64_t>(splits, 1024));
    }
    const int64_t rows_per_split = CeilDiv(r, splits);
    splits                       = CeilDiv(r, rows_per_split);
    const unsigned block         = cols >= 256 ? 256 : (cols >= 128 ? 128 : 64);
    LaunchStep s;
    if (!Kernel(&s, std::string("col_reduce_") + opname + "_f32")) return false;
    s.block[0] = block;
    s.grid[0]  = (unsigned)CeilDiv(cols, block);
    s.grid[1]  = (unsigned)std::min<int64_t>(outer, 65535);
    s.grid[2]  = (unsigned)splits;
    if (splits == 1) {
      std::vector<int> outs;
      ArgSpec al = Aligned(vec, src_in_for_align, {});
      if (dst.kind == ArgSpec::kOutput) al.aligned_outputs.push_back(dst.index);
      s.args = {src, dst, I(outer), I(r), I(inner), I(rows_per_split), al};
      p->steps.push_back(s);
      return true;
    }
    const int64_t scratch_off = p->scratch_bytes;
    p->scratch_bytes += (size_t)RoundUp(splits * outer * inner * 4, 256);
    // Scratch is 256-byte aligned; the partial of split k starts at k*outer*inner floats, which keeps 16-byte
    // alignment only when outer*inner % 4 == 0 (true when inner % 4 == 0).
    s.args = {src, Scratch(scratch_off), I(outer), I(r), I(inner), I(rows_per_split),
              Aligned(vec, src_in_for_align, {})};
    p->steps.push_back(s);
    const int64_t oi = outer * inner;
    if (oi % 4 == 0 && FindKernel(std::string("reduce_generic_col_fold_") + BaseReduceOp(opname) + "_f32")) {
      // the partials are few columns and `splits` rows: the rows over the warps of a CTA (reduce_generic.cu)
      LaunchStep f;
      if (!Kernel(&f, std::string("reduce_generic_col_fold_") + BaseReduceOp(opname) + "_f32")) return false;
      f.block[0] = 256;
      f.grid[0]  = (unsigned)CeilDiv(oi / 4, 32);
      f.args     = {Scratch(scratch_off), dst, I(splits), I(oi)};
      p->steps.push_back(f);
      return true;
    }
    return PlanReduce(p, BaseReduceOp(opname), 1, splits, oi, Scratch(scratch_off), dst, {});
  }

  bool PlanReduceFinishRows(CompiledGroup* p, const char* opname, int64_t rows, int64_t splits, ArgSpec src,
                            ArgSpec dst) {
    return PlanReduce(p, opname, rows, splits, 1, src, dst, {});
  }

  // Second passes over partial results use the plain op of a reduction that has a producer folded in.
  static const char* BaseReduceOp(const char* opname) {
    const std::string s = opname;
    if (s == "sumsq" || s == "sumabs" || s == "sumexp") return "sum";
    if (s == "maxabs") return "max";
    return opname;
  }

  // reduce_{sum,prod,max,min}(%0), and the forms with one elementwise producer folded into the reduction's first
  // pass: sum of squares, of absolute values, of exponentials, and max of absolute values.  (The reference keeps a
  // reduce's producer as a separate, materialised stage of the same kernel; here it costs no extra pass over HBM.)
  std::unique_ptr<CompiledGroup> MatchReduce(const std::string& expr) {
    static const std::map<std::string, const char*> kinds = {
        {"reduce_sum(%0)", "sum"}, {"reduce_prod(%0)", "prod"}, {"reduce_max(%0)", "max"}, {"reduce_min(%0)", "min"},
        {"reduce_sum(elementwise_mul(%0,%0))", "sumsq"}, {"reduce_sum(elementwise_mul(%0,identity(%0)))", "sumsq"},
        {"reduce_sum(elementwise_mul(identity(%0),%0))", "sumsq"}, {"reduce_sum(abs(%0))", "sumabs"},
        {"reduce_sum(exp(%0))", "sumexp"}, {"reduce_max(abs(%0))", "maxabs"}};
    // What the AutoCast program pass makes of a 16-bit reduction (cinn/frontend/pass/auto_cast.cc:50-76): widen, reduce
    // in float32, narrow.  The 16-bit reduction kernels do exactly that in registers.
    static const std::regex widened(R"(^cast\((reduce_(?:sum|prod|max|min))\(cast\(%0\)\)\)$)");
    std::smatch wm;
    if (std::regex_match(expr, wm, widened)) {
      const auto &x = g.inputs[0], &o = g.outputs[0];
      const OpDesc* red = Producer(Producer(o.name)->inputs[0]);
      const OpDesc* in  = red ? Producer(red->inputs[0]) : nullptr;
      const bool half   = x.dtype == DType::kFloat16 || x.dtype == DType::kBFloat16;
      if (!half || o.dtype != x.dtype || !in || DTypeFromName(AttrS(*in, "dtype", "")) != DType::kFloat32) return nullptr;
      return MatchGenericReduce(wm[1].str() + "(%0)");
    }
    auto it = kinds.find(expr);
    const bool all_any = expr == "reduce_all(%0)" || expr == "reduce_any(%0)";
    if (it == kinds.end() && !all_any) return nullptr;
    const auto &x = g.inputs[0], &o = g.outputs[0];
    if (x.dtype != DType::kFloat32 || o.dtype != DType::kFloat32 || all_any) return MatchGenericReduce(expr);
    const OpDesc* op = Producer(o.name);
    int64_t outer, r, inner;
    if (!ReduceView(x.shape, AttrList(*op, "dim"), &outer, &r, &inner)) {
      int64_t A, B, I;
      if (MidKeepView(x.shape, AttrList(*op, "dim"), &A, &B, &I) && o.numel() == B &&
          FindKernel(std::string("mid_keep_reduce_") + it->second + "_f32")) {
        auto p      = NewPlan("mid_keep_reduce");
        p->elements = x.numel();
        if (!PlanMidKeep(p.get(), it->second, false, A, B, I, Out(0), Out(0))) return nullptr;
        return p;
      }
      // Any other set of axes (cinn/hlir/pe/reduction.cc:139-227 takes every set): the runs of adjacent reduced axes
      // are folded one at a time, the last run first, each as an [outer, r, inner] reduction of what the previous
      // step left in scratch memory.  Every step shrinks the data by its run's extent, so the first step carries
      // nearly all of the traffic; the result differs from the serial order by rounding only (sum, prod) or not at
      // all (max, min).
      std::vector<int64_t> dims = AttrList(*op, "dim");
      const int nd = (int)x.shape.size();
      std::vector<bool> red(nd, false);
      for (auto d : dims) {
        if (d < 0) d += nd;
        if (d < 0 || d >= nd) return nullptr;
        red[d] = true;
      }
      std::vector<int64_t> ext;   // non-unit extents, and whether each is reduced
      std::vector<bool> is_red;
      for (int i = 0; i < nd; ++i)
        if (x.shape[i] != 1) {
          ext.push_back(x.shape[i]);
          is_red.push_back(red[i]);
        }
      int64_t kept = 1;
      for (size_t i = 0; i < ext.size(); ++i) kept *= is_red[i] ? 1 : ext[i];
      if (o.numel() != kept) {
        Fail("reduce output has " + std::to_string(o.numel()) + " elements, expected " + std::to_string(kept));
        return nullptr;
      }
      auto p      = NewPlan("multi_axis_reduce");
      p->elements = x.numel();
      ArgSpec src = In(0);
      std::vector<int> align = {0};
      const char* kind = it->second;
      while (true) {
        int hi = (int)ext.size() - 1;
        while (hi >= 0 && !is_red[hi]) --hi;
        if (hi < 0) break;
        int lo = hi;
        while (lo > 0 && is_red[lo - 1]) --lo;
        int64_t so = 1, sr = 1, si = 1;
        for (int i = 0; i < lo; ++i) so *= ext[i];
        for (int i = lo; i <= hi; ++i) sr *= ext[i];
        for (int i = hi + 1; i < (int)ext.size(); ++i) si *= ext[i];
        bool last = true;
        for (int i = 0; i < lo; ++i) last = last && !is_red[i];
        ArgSpec dst = Out(0);
        if (!last) {
          const int64_t off = p->scratch_bytes;
          p->scratch_bytes += (size_t)RoundUp(so * si * 4, 256);
          dst = Scratch(off);
        }
        if (!PlanReduce(p.get(), kind, so, sr, si, src, dst, align)) return nullptr;
        ext.erase(ext.begin() + lo, ext.begin() + hi + 1);
        is_red.erase(is_red.begin() + lo, is_red.begin() + hi + 1);
        src  = dst;
        align.clear();
        kind = BaseReduceOp(kind);  // a folded producer (x * x, |x|, exp x) belongs to the first step only
        if (last) break;
      }
      return p;
    }
    if (o.numel() != outer * inner) {
      Fail("reduce output has " + std::to_string(o.numel()) + " elements, expected " + std::to_string(outer * inner));
      return nullptr;
    }
    auto p      = NewPlan(inner == 1 ? "row_reduce" : "col_reduce");
    p->elements = x.numel();
    if (!PlanReduce(p.get(), it->second, outer, r, inner, In(0), Out(0), {0})) return nullptr;
    return p;
  }

  // The two-output group {reduce_sum(x), reduce_sum(x * x)} over the same leading + trailing axes: the statistics
  // pass of batch_norm_train (cinn/frontend/decomposer/batch_norm.cc:60-92), one read of x.
  // The statistics of the decomposed batch_norm_grad (cinn/frontend/decomposer/batch_norm.cc:62-72):
  // {reduce_sum(dy), reduce_sum(dy * (x - broadcast(mean)))} over N, H, W, or the second one alone.
  std::unique_ptr<CompiledGroup> MatchBnGradStats(const std::string& expr_in) {
    static const std::regex both(R"(^reduce_sum\(%(\d)\);reduce_sum\(elementwise_mul\(%(\d),subtract\(%(\d),broadcast_to\(%(\d)\)\)\)\)$)");
    static const std::regex one(R"(^reduce_sum\(elementwise_mul\(%(\d),subtract\(%(\d),broadcast_to\(%(\d)\)\)\)\)$)");
    std::smatch m;
    int idy, ix, im;
    bool dual;
    DType wide;
    const std::string stripped = StripHalfCasts(expr_in, &wide);
    const std::string& expr    = stripped;
    if (std::regex_match(expr, m, both) && g.outputs.size() == 2) {
      if (m[1].str() != m[2].str()) return nullptr;
      idy = atoi(m[2].str().c_str()), ix = atoi(m[3].str().c_str()), im = atoi(m[4].str().c_str());
      dual = true;
    } else if (std::regex_match(expr, m, one) && g.outputs.size() == 1) {
      idy = atoi(m[1].str().c_str()), ix = atoi(m[2].str().c_str()), im = atoi(m[3].str().c_str());
      dual = false;
    } else {
      return nullptr;
    }
    if (g.inputs.size() != 3 || idy == ix || idy == im || ix == im) return nullptr;
    const auto &dy = g.inputs[idy], &x = g.inputs[ix], &mean = g.inputs[im];
    if (dy.dtype != wide || x.dtype != wide || mean.dtype != DType::kFloat32 || dy.shape != x.shape) {
      Fail("batch_norm_grad statistics are prebuilt for float32 (or, between casts, 16-bit) tensors of one shape");
      return nullptr;
    }
    int64_t A = 0, B = 0, I = 0;
    for (auto& op : g.ops) {
      if (op.type == "reduce_sum") {
        int64_t a2, b2, i2;
        if (!MidKeepView(x.shape, AttrList(op, "dim"), &a2, &b2, &i2) || (A && (a2 != A || b2 != B || i2 != I))) {
          Fail("the reductions must keep the same middle axes");
          return nullptr;
        }
        A = a2, B = b2, I = i2;
      }
    }
    if (!A || mean.numel() != B) return nullptr;
    for (auto& o : g.outputs)
      if (o.numel() != B || o.dtype != DType::kFloat32) return nullptr;
    auto p      = NewPlan("bn_grad_stats");
    p->elements = x.numel();
    if (dual) {
      if (!PlanMidKeep(p.get(), "sum", true, A, B, I, Out(0), Out(1), idy, ix, im, wide)) return nullptr;
    } else {
      // the kernel always keeps both sums; the first one lands in scratch
      const int64_t off = p->scratch_bytes;
      p->scratch_bytes += (size_t)RoundUp(B * 4, 256);
      if (!PlanMidKeep(p.get(), "sum", true, A, B, I, Scratch(off), Out(0), idy, ix, im, wide)) return nullptr;
    }
    return p;
  }

  std::unique_ptr<CompiledGroup> MatchChannelStats(const std::string& expr) {
    static const std::set<std::string> forms = {
        "reduce_sum(%0);reduce_sum(elementwise_mul(%0,identity(%0)))", "reduce_sum(%0);reduce_sum(elementwise_mul(%0,%0))",
        "reduce_sum(%0);reduce_sum(elementwise_mul(identity(%0),%0))"};
    DType wide;
    const std::string stripped = StripHalfCasts(expr, &wide);
    if (!forms.count(stripped) || g.inputs.size() != 1 || g.outputs.size() != 2) return nullptr;
    const auto& x = g.inputs[0];
    if (x.dtype != wide || g.outputs[0].dtype != DType::kFloat32 || g.outputs[1].dtype != DType::kFloat32) {
      Fail("channel statistics are prebuilt for float32 results only");
      return nullptr;
    }
    const OpDesc *r0 = Producer(g.outputs[0].name), *r1 = Producer(g.outputs[1].name);
    int64_t A, B, I, A2, B2, I2;
    if (!MidKeepView(x.shape, AttrList(*r0, "dim"), &A, &B, &I) || !MidKeepView(x.shape, AttrList(*r1, "dim"), &A2, &B2, &I2) ||
        A != A2 || B != B2 || I != I2 || g.outputs[0].numel() != B || g.outputs[1].numel() != B) {
      Fail("the two reductions must keep the same middle axes");
      return nullptr;
    }
    auto p      = NewPlan("channel_stats");
    p->elements = x.numel();
    if (!PlanMidKeep(p.get(), "sum", true, A, B, I, Out(0), Out(1), 0, -1, -1, wide)) return nullptr;
    return p;
  }

  // Reductions of the other element types (reduce_generic.cu): float16 / bfloat16 / float64 / int32 / int64 with
  // sum, prod, max, min; bool with all, any (cinn/hlir/op/reduction.cc:477-505).
  std::unique_ptr<CompiledGroup> MatchGenericReduce(const std::string& expr) {
    static const std::map<std::string, const char*> kinds = {
        {"reduce_sum(%0)", "sum"}, {"reduce_prod(%0)", "prod"}, {"reduce_max(%0)", "max"},
        {"reduce_min(%0)", "min"}, {"reduce_all(%0)", "all"},   {"reduce_any(%0)", "any"}};
    auto it = kinds.find(expr);
    const auto &x = g.inputs[0], &o = g.outputs[0];
    if (it == kinds.end()) {
      Fail("reductions with a folded producer are prebuilt for float32 only");
      return nullptr;
    }
    const char* tname = nullptr;
    switch (x.dtype) {
      case DType::kFloat16: tname = "f16"; break;
      case DType::kBFloat16: tname = "bf16"; break;
      case DType::kFloat64: tname = "f64"; break;
      case DType::kInt32: tname = "i32"; break;
      case DType::kInt64: tname = "i64"; break;
      case DType::kBool: tname = "bool"; break;
      default: break;
    }
    const bool logical = std::string(it->second) == "all" || std::string(it->second) == "any";
    if (!tname || o.dtype != x.dtype || logical != (x.dtype == DType::kBool)) {
      Fail(std::string("no prebuilt ") + it->second + " reduction from " + DTypeName(x.dtype) + " to " + DTypeName(o.dtype));
      return nullptr;
    }
    const OpDesc* op = Producer(o.name);
    if (op->type == "cast") op = Producer(op->inputs[0]);  // the widened form, see MatchReduce
    const int64_t esize = DTypeBytes(x.dtype), V = 16 / esize;
    const int sms       = dev.sm_count;
    const std::string suffix = std::string(it->second) + "_" + tname;
    std::unique_ptr<CompiledGroup> p;
    auto row_step = [&](ArgSpec src, ArgSpec dst, int64_t rows, int64_t len, std::vector<int> align_in) -> bool {
      LaunchStep s;
      if (!Kernel(&s, "reduce_generic_row_" + suffix)) return false;
      const int64_t group = len * esize > 8192 ? 256 : 32;
      s.block[0] = 256;
      s.grid[0]  = (unsigned)std::max<int64_t>(
          1, group == 32 ? std::min<int64_t>(CeilDiv(rows, 8), (int64_t)sms * 32) : std::min<int64_t>(rows, (int64_t)sms * 16));
      ArgSpec al = Aligned(len % V == 0, align_in, {});
      s.args     = {src, dst, I(rows), I(len), I(group), al};
      p->steps.push_back(s);
      return true;
    };
    // Columns: a thread per 16 bytes of columns.  With few columns the reduced axis is split over blockIdx.z into
    // partial results in scratch, which a second launch of the same kernel folds.
    auto col_step = [&](ArgSpec src, ArgSpec dst, int64_t o2, int64_t len, int64_t in, int64_t splits,
                        std::vector<int> align_in, bool dst_is_out) -> bool {
      LaunchStep s;
      if (!Kernel(&s, "reduce_generic_col_" + suffix)) return false;
      const bool vec     = in % V == 0;
      const int64_t cols = vec ? in / V : in;
      s.block[0] = cols >= 256 ? 256 : (cols >= 128 ? 128 : 64);
      s.grid[0]  = (unsigned)std::max<int64_t>(1, vec ? CeilDiv(cols, s.block[0]) : std::min<int64_t>(CeilDiv(cols, s.block[0]), (int64_t)sms * 8));
      s.grid[1]  = (unsigned)std::min<int64_t>(o2, 65535);
      s.grid[2]  = (unsigned)splits;
      ArgSpec al = Aligned(vec, align_in, dst_is_out ? std::vector<int>{0} : std::vector<int>{});
      s.args     = {src, dst, I(o2), I(len), I(in), I(CeilDiv(len, splits)), al};
      p->steps.push_back(s);
      return true;
    };
    // One [outer, r, inner] reduction from `src` to `dst` (either may be scratch memory of an earlier / for a later step).
    auto plan_one = [&](ArgSpec src, ArgSpec dst, int64_t outer, int64_t r, int64_t inner, std::vector<int> align_in,
                        bool dst_is_out) -> bool {
      if (inner == 1) {
        // Few very long rows: cut each row into S equal segments (partials in scratch), then fold the S partials.
        int64_t S = 1;
        if (outer < (int64_t)sms * 2 && r >= 65536) {
          while (S < 1024 && r % (S * 2) == 0 && r / (S * 2) >= 4096 && outer * S < (int64_t)sms * 8) S *= 2;
        }
        if (S > 1) {
          const int64_t off = p->scratch_bytes;
          p->scratch_bytes += (size_t)RoundUp(outer * S * esize, 256);
          return row_step(src, Scratch(off), outer * S, r / S, align_in) && row_step(Scratch(off), dst, outer, S, {});
        }
        return row_step(src, dst, outer, r, align_in);
      }
      const bool vec     = inner % V == 0;
      const int64_t thr  = (vec ? inner / V : inner) * outer;
      int64_t splits     = 1;
      if (thr < (int64_t)sms * 512 && r >= 64 && outer * r * inner * esize >= (4 << 20)) {  // a second launch only pays on large inputs
        splits = std::min<int64_t>(r / 16, CeilDiv((int64_t)sms * 1024, thr));
        splits = std::max<int64_t>(1, std::min<int64_t>(splits, 512));
      }
      // whole groups of eight rows per split: the kernel keeps eight row loads in flight and takes a remainder one
      // row (one DRAM latency) at a time
      const int64_t rps = splits > 1 ? RoundUp(CeilDiv(r, splits), 8) : r;
      splits            = CeilDiv(r, rps);
      if (splits == 1) return col_step(src, dst, outer, r, inner, 1, align_in, dst_is_out);
      const int64_t off = p->scratch_bytes;
      p->scratch_bytes += (size_t)RoundUp(splits * outer * inner * esize, 256);
      if (!col_step(src, Scratch(off), outer, r, inner, splits, align_in, false)) return false;
      if ((outer * inner) % V == 0) {  // the partials are few columns and many rows: rows over the warps of a CTA
        LaunchStep f;
        if (!Kernel(&f, "reduce_generic_col_fold_" + suffix)) return false;
        f.block[0] = 256;
        f.grid[0]  = (unsigned)CeilDiv(outer * inner / V, 32);
        f.args     = {Scratch(off), dst, I(splits), I(outer * inner)};
        p->steps.push_back(f);
        return true;
      }
      return col_step(Scratch(off), dst, 1, splits, outer * inner, 1, {}, dst_is_out);
    };
    int64_t outer, r, inner;
    if (!ReduceView(x.shape, AttrList(*op, "dim"), &outer, &r, &inner)) {
      // Any other set of axes: the runs of adjacent reduced axes are folded one at a time, the last run first, each
      // as an [outer, r, inner] reduction of what the previous step left in scratch memory (see MatchReduce; the
      // intermediates have the tensor's own type, so a 16-bit sum is rounded to 16 bits between the steps, as the
      // reference's accumulation in the tensor's type is at every step).
      std::vector<int64_t> dims = AttrList(*op, "dim");
      const int nd = (int)x.shape.size();
      std::vector<bool> red(nd, false);
      for (auto d : dims) {
        if (d < 0) d += nd;
        if (d < 0 || d >= nd) return nullptr;
        red[d] = true;
      }
      std::vector<int64_t> ext;
      std::vector<bool> is_red;
      for (int i = 0; i < nd; ++i)
        if (x.shape[i] != 1) {
          ext.push_back(x.shape[i]);
          is_red.push_back(red[i]);
        }
      int64_t kept = 1;
      for (size_t i = 0; i < ext.size(); ++i) kept *= is_red[i] ? 1 : ext[i];
      if (o.numel() != kept) {
        Fail("reduce output has " + std::to_string(o.numel()) + " elements, expected " + std::to_string(kept));
        return nullptr;
      }
      p           = NewPlan("multi_axis_reduce");
      p->elements = x.numel();
      ArgSpec src = In(0);
      std::vector<int> align = {0};
      while (true) {
        int hi = (int)ext.size() - 1;
        while (hi >= 0 && !is_red[hi]) --hi;
        if (hi < 0) break;
        int lo = hi;
        while (lo > 0 && is_red[lo - 1]) --lo;
        int64_t so = 1, sr = 1, si = 1;
        for (int i = 0; i < lo; ++i) so *= ext[i];
        for (int i = lo; i <= hi; ++i) sr *= ext[i];
        for (int i = hi + 1; i < (int)ext.size(); ++i) si *= ext[i];
        bool last = true;
        for (int i = 0; i < lo; ++i) last = last && !is_red[i];
        ArgSpec dst = Out(0);
        if (!last) {
          const int64_t off = p->scratch_bytes;
          p->scratch_bytes += (size_t)RoundUp(so * si * esize, 256);
          dst = Scratch(off);
        }
        if (!plan_one(src, dst, so, sr, si, align, last)) return nullptr;
        ext.erase(ext.begin() + lo, ext.begin() + hi + 1);
        is_red.erase(is_red.begin() + lo, is_red.begin() + hi + 1);
        src = dst;
        align.clear();
        if (last) break;
      }
      return p;
    }
    if (o.numel() != outer * inner) {
      Fail("reduce output has " + std::to_string(o.numel()) + " elements, expected " + std::to_string(outer * inner));
      return nullptr;
    }
    p           = NewPlan(inner == 1 ? "row_reduce" : "col_reduce");
    p->elements = x.numel();
    if (!plan_one(In(0), Out(0), outer, r, inner, {0}, true)) return nullptr;
    return p;
  }

  // ---- row normalisation ---------------------------------------------------------------------
  bool PlanRowNorm(CompiledGroup* p, bool layernorm, bool half, int64_t rows, int64_t cols, double eps, int x_in,
                   int gamma_in, int beta_in) {
    const int V        = half ? 8 : 4;
    const char* tname  = half ? half_name_ : "f32";
    const int sms      = dev.sm_count;
    const int64_t nvec = cols / V;
    auto cluster_step  = [&](LaunchStep* s) -> bool {
      const int64_t cap = 48 * 1024;  // floats of dynamic shared memory per CTA (192 KiB)
      int64_t csize     = 1;
      while (csize < 8 && CeilDiv(cols, csize) > cap) csize *= 2;
      if (CeilDiv(cols, csize) > cap)
        return Fail("row of " + std::to_string(cols) + " elements exceeds the cluster capacity of " +
                    std::to_string(8 * cap));
      const int64_t seg = CeilDiv(cols, csize);
      if (!Kernel(s, std::string("rownorm_cluster_") + tname)) return false;
      s->block[0] = 512;
      s->cluster  = (unsigned)csize;
      s->dyn_smem = (size_t)seg * 4;
      const int64_t per_sm = std::max<int64_t>(1, std::min<int64_t>(4, (200 * 1024) / (seg * 4 + 1024)));
      const int64_t ncl    = std::max<int64_t>(1, std::min<int64_t>(rows, (int64_t)sms * per_sm / csize));
      s->grid[0]           = (unsigned)(ncl * csize);
      s->args = {In(x_in), layernorm ? In(gamma_in) : In(x_in), layernorm ? In(beta_in) : In(x_in), Out(0), I(rows),
                 I(cols), I(seg), I(layernorm ? 1 : 0), F(eps)};
      return true;
    };
    LaunchStep slow;
    if (!cluster_step(&slow)) return false;
    // Rows of 2 KiB .. 32 KiB: stream them through a shared-memory ring filled by bulk asynchronous copies.
    const int64_t row_bytes = cols * (half ? 2 : 4);
    const int vpt_max       = half ? 2 : 4;  // at most 16 elements (and 16+16 gamma/beta values) per thread
    // Measured on B200 (16384 x 4096): the streamed kernel wins for fp16 layer_norm (0.84 of the HBM peak
    // against 0.72 with register-resident rows: gamma/beta stay in registers instead of going through L1 for
    // every row); elsewhere the register-resident kernels are as fast or faster, so "automatic" picks it only there.
    const bool use_tma = dev.enable_tma_rownorm > 0 || (dev.enable_tma_rownorm < 0 && layernorm && half);
    if (cols % V == 0 && nvec >= 128 && nvec <= 512 * vpt_max && use_tma) {
      int G = 128;
      while (G * vpt_max < nvec) G *= 2;
      int vpt = 1;
      while (G * vpt < nvec) vpt *= 2;
      int64_t stages = dev.rownorm_stages > 0 ? dev.rownorm_stages
                                              : std::max<int64_t>(3, std::min<int64_t>(8, 24576 / row_bytes));
      stages         = std::min<int64_t>(stages, 8);
      const int64_t smem = stages * row_bytes;
      int64_t per_sm     = std::min<int64_t>((224 * 1024) / (smem + 2048), 768 / G);
      per_sm             = std::min<int64_t>(per_sm, 65536 / (G * 64));
      if (dev.rownorm_ctas_per_sm > 0) per_sm = dev.rownorm_ctas_per_sm;
      per_sm = std::max<int64_t>(1, per_sm);
      // A CTA that gets only a handful of rows (a shard of the tensor on one of several GPUs) never fills a deep
      // ring: two buffers then start sooner (2048 x 4096 fp16: 8.8 us against 9.1 us with three).
      if (dev.rownorm_stages <= 0 && rows < (int64_t)sms * per_sm * 8) stages = 2;
      const int64_t smem2 = stages * row_bytes;
      LaunchStep s;
      std::string name = std::string(layernorm ? "layernorm_tma_" : "softmax_tma_") + tname + "_g" +
                         std::to_string(G) + "_v" + std::to_string(vpt);
      if (!Kernel(&s, name)) return false;
      s.block[0] = G;
      s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(rows, (int64_t)sms * per_sm));
      s.dyn_smem = (size_t)smem2;
      s.args     = {In(x_in), layernorm ? In(gamma_in) : In(x_in), layernorm ? In(beta_in) : In(x_in), Out(0), I(rows),
                    I(cols), I(stages), F(eps)};
      p->steps.push_back(s);
      p->aligned_inputs  = layernorm ? std::vector<int>{x_in, gamma_in, beta_in} : std::vector<int>{x_in};
      p->aligned_outputs = {0};
      p->steps_unaligned.push_back(slow);
      return true;
    }
    if (cols % V == 0 && nvec <= 4096) {
      // At most 16 elements per thread where the row length allows it (fp16 vectors hold 8 elements).
      const int vmax = half ? 2 : 4;
      int G = 32;
      if (nvec > 32 * vmax) G = 128;
      if (nvec > 128 * vmax) G = 256;
      if (nvec > 256 * vmax) G = 512;
      if (nvec > 512 * vmax) G = 1024;
      int vpt = 1;
      while (G * vpt < nvec) vpt *= 2;
      // Rows per iteration: more for short rows so that a CTA keeps >= 16 KiB in flight and (layer_norm) reads
      // gamma/beta once for several rows.
      int R = 1;
      if (G >= 128 && G <= 512) {
        const int64_t row_b = cols * (half ? 2 : 4);
        // Measured on B200: one row per iteration is best except for fp16 layer_norm, where two rows share one
        // read of gamma/beta through L1.
        if (dev.rownorm_rows_per_iter > 0) R = dev.rownorm_rows_per_iter;
        else if (layernorm && half && row_b <= 8192 && vpt <= 2) R = 2;
        if (R == 4 && vpt > 2) R = 2;
        if (rows < (int64_t)sms * R) R = 1;
      }
      LaunchStep s;
      std::string name = std::string(layernorm ? "layernorm_row_" : "softmax_row_") + tname + "_g" +
                         std::to_string(G) + "_v" + std::to_string(vpt) + "_r" + std::to_string(R);
      if (!Kernel(&s, name)) return false;
      const int64_t groups = CeilDiv(rows, R);
      if (G == 32) {
        s.block[0] = 256;
        s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(CeilDiv(rows, 8), (int64_t)sms * 16));
      } else {
        s.block[0] = G;
        s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(groups, (int64_t)sms * (2048 / G) * 2));
      }
      s.args = {In(x_in), layernorm ? In(gamma_in) : In(x_in), layernorm ? In(beta_in) : In(x_in), Out(0), I(rows),
                I(cols), F(eps), F(1.0 / (double)cols)};
      p->steps.push_back(s);
      // Register-resident rows need 16-byte aligned buffers; otherwise the cluster kernel takes over.
      p->aligned_inputs  = layernorm ? std::vector<int>{x_in, gamma_in, beta_in} : std::vector<int>{x_in};
      p->aligned_outputs = {0};
      p->steps_unaligned.push_back(slow);
    } else {
      p->steps.push_back(slow);
    }
    return true;
  }

  // softmax op along the last axis: cinn/hlir/pe/nn.cc:755-796 (exp(x)/sum exp(x)); 16-bit storage as
  // cast(softmax(cast(%0))).  Also the decomposed "fast" form of cinn/frontend/decomposer/activation.cc:70-118:
  // divide(exp(x), broadcast_to(reduce_sum(exp(x)))).
  std::unique_ptr<CompiledGroup> MatchSoftmax(const std::string& expr) {
    bool half = false, safe = false;
    // The decomposed form with the row maximum subtracted (cinn/frontend/decomposer/activation.cc:104-116).
    auto safe_form = [](const std::string& x) {
      const std::string d = "exp(subtract(" + x + ",broadcast_to(reduce_max(" + x + "))))";
      return "divide(" + d + ",broadcast_to(reduce_sum(" + d + ")))";
    };
    if (expr == "softmax(%0)" || expr == "divide(exp(%0),broadcast_to(reduce_sum(exp(%0))))") {
    } else if (expr == "cast(softmax(cast(%0)))" ||
               expr == "cast(divide(exp(cast(%0)),broadcast_to(reduce_sum(exp(cast(%0))))))") {
      half = true;
    } else if (expr == safe_form("%0")) {
      safe = true;
    } else if (expr == "cast(" + safe_form("cast(%0)") + ")") {
      safe = half = true;
    } else {
      return nullptr;
    }
    const auto &x = g.inputs[0], &o = g.outputs[0];
    if (x.shape.empty() || o.shape != x.shape) return nullptr;
    if (half ? !SetHalfType(x.dtype, o.dtype)
             : (x.dtype != DType::kFloat32 || o.dtype != DType::kFloat32))
      return nullptr;
    const int nd = (int)x.shape.size();
    for (auto& op : g.ops) {
      if (op.type == "softmax") {
        int64_t axis = AttrI(op, "axis", -1);
        auto axes    = AttrList(op, "axes");
        if (!axes.empty()) axis = axes[0];
        if (axes.size() > 1 || !(axis == -1 || axis == nd - 1)) {
          Fail("softmax is prebuilt for the last axis only");
          return nullptr;
        }
      } else if (op.type == "reduce_sum" || op.type == "reduce_max") {
        auto dims = AttrList(op, "dim");
        if (dims.size() != 1 || !(dims[0] == -1 || dims[0] == nd - 1)) {
          Fail("decomposed softmax must reduce the last axis");
          return nullptr;
        }
      }
    }
    const int64_t cols = x.shape.back(), rows = x.numel() / std::max<int64_t>(cols, 1);
    const bool simple  = !safe && dev.rownorm_simple > 0 && CeilDiv(cols, half ? 8 : 4) <= 4096;
    if (safe || simple) {
      // One CTA per row, the row in registers: at most 512 threads x 8 vectors.
      const int V        = half ? 8 : 4;
      const int64_t nvec = CeilDiv(cols, V);
      if (nvec > 4096) {
        Fail("max-subtracted softmax is prebuilt for rows of up to " + std::to_string(4096 * V) + " elements");
        return nullptr;
      }
      // 4 vectors per thread for fp32, 2 for 16-bit storage (measured: 128-thread CTAs with 4 are slower there),
      // between 128 and 512 threads; as many again of the next row are on their way.
      const int target = half ? 2 : 4;
      int G            = 128;
      while (G < 512 && G * target < nvec) G *= 2;
      int vpt = 1;
      while (G * vpt < nvec) vpt *= 2;
      auto p = NewPlan(safe ? "softmax_safe_row" : "softmax_row");
      LaunchStep s;
      if (!Kernel(&s, std::string(safe ? "softmax_safe_" : "softmax_plain_") + (half ? half_name_ : "f32") + "_v" + std::to_string(vpt)))
        return nullptr;
      s.block[0] = G;
      s.grid[0]  = (unsigned)std::max<int64_t>(1, std::min<int64_t>(rows, (int64_t)dev.sm_count * (2048 / G) * 4));
      s.args     = {In(0), Out(0), I(rows), I(cols), Aligned(cols % V == 0, {0}, {0})};
      p->steps.push_back(s);
      return p;
    }
    auto p = NewPlan("softmax_row");
    if (!PlanRowNorm(p.get(), false, half, rows, cols, 0.0, 0, 0, 0)) return nullptr;
    return p;
  }

  // layer_norm composition over [rows, cols] (cinn/frontend/op_mappers/paddle/layer_norm.cc:84-139 with
  // rsqrt+multiply): inputs x, gamma, beta.  The expression below is what LayerNormExpr() prints for the op
  // sequence built by the frontend helper; constants are checked against the shapes.
  static std::string LayerNormExpr(bool half) {
    const std::string x    = half ? "cast(%0)" : "%0";
    const std::string n    = "fill_constant()";
    const std::string mean = "divide(reduce_sum(" + x + ")," + n + ")";
    const std::string m2   = "divide(reduce_sum(elementwise_mul(" + x + ",identity(" + x + ")))," + n + ")";
    const std::string var  = "max(subtract(" + m2 + ",elementwise_mul(" + mean + ",identity(" + mean + "))),fill_constant())";
    const std::string rstd = "rsqrt(elementwise_add(" + var + ",fill_constant()))";
    const std::string xn   = "elementwise_mul(subtract(" + x + ",broadcast_to(" + mean + ")),broadcast_to(" + rstd + "))";
    const std::string y    = "elementwise_add(elementwise_mul(" + xn + ",broadcast_to(%1)),broadcast_to(%2))";
    return half ? "cast(" + y + ")" : y;
  }

  std::unique_ptr<CompiledGroup> MatchLayerNorm(const std::string& expr) {
    bool half = false;
    if (expr == LayerNormExpr(false)) {
    } else if (expr == LayerNormExpr(true)) {
      half = true;
    } else {
      return nullptr;
    }
    if (g.inputs.size() != 3) return nullptr;
    const auto &x = g.inputs[0], &gamma = g.inputs[1], &beta = g.inputs[2], &o = g.outputs[0];
    if (x.shape.size() != 2 || o.shape != x.shape) return nullptr;
    if (half ? !SetHalfType(x.dtype, o.dtype)
             : (x.dtype != DType::kFloat32 || o.dtype != DType::kFloat32))
      return nullptr;
    const int64_t rows = x.shape[0], cols = x.shape[1];
    if (gamma.dtype != DType::kFloat32 || beta.dtype != DType::kFloat32 || gamma.shape != std::vector<int64_t>{cols} ||
        beta.shape != std::vector<int64_t>{cols}) {
      Fail("layer_norm gamma/beta must be float32 vectors of the row length");
      return nullptr;
    }
    // Constants: the element count, zero and epsilon, identified by the op that consumes them.
    double eps = -1.0;
    for (auto& op : g.ops) {
      if (op.type == "divide") {
        const OpDesc* c = ProducerOfType(op.inputs[1], "fill_constant");
        if (!c || AttrF(*c, "value", 0) != (double)cols) {
          Fail("layer_norm divisor constant is not the row length");
          return nullptr;
        }
      } else if (op.type == "max") {
        const OpDesc* c = ProducerOfType(op.inputs[1], "fill_constant");
        if (!c || AttrF(*c, "value", 1) != 0.0) {
          Fail("layer_norm variance clamp constant is not 0");
          return nullptr;
        }
      } else if (op.type == "elementwise_add") {
        const OpDesc* c = ProducerOfType(op.inputs[1], "fill_constant");
        if (c) eps = (float)AttrF(*c, "value", 0);
      } else if (op.type == "reduce_sum") {
        auto dims = AttrList(op, "dim");
        if (dims.size() != 1 || !(dims[0] == 1 || dims[0] == -1)) {
          Fail("layer_norm reductions must be over axis 1");
          return nullptr;
        }
      }
    }
    if (eps < 0) {
      Fail("layer_norm epsilon constant not found");
      return nullptr;
    }
    auto p = NewPlan("layernorm_row");
    if (!PlanRowNorm(p.get(), true, half, rows, cols, eps, 0, 1, 2)) return nullptr;
    return p;
  }

  bool HasReduce() const {
    for (auto& op : g.ops)
      if (op.type.rfind("reduce_", 0) == 0) return true;
    return false;
  }

  std::unique_ptr<CompiledGroup> Run() {
    std::string e;
    std::string expr = CanonicalExpr(g, &e);
    if (expr.empty()) {
      Fail(e);
      return nullptr;
    }
    if (err) err->clear();
    if (g.outputs.size() != 1) {
      // The only multi-output family: the fused channel statistics.
      if (auto p = MatchChannelStats(expr)) return p;
      if (err && !err->empty()) return nullptr;
      if (auto p = MatchBnGradStats(expr)) return p;
      if (err && !err->empty()) return nullptr;
      // An elementwise chain one of whose intermediate values is an output too.
      std::string why2;
      if (g.outputs.size() == 2)
        if (auto p = MatchGenericChain(g, dev, &why2)) return p;
      // Any other elementwise group with up to four outputs of one shape: a register program.
      std::string why3;
      if (auto p = MatchDag(g, dev, &why3)) return p;
      // Reductions over the trailing axes with elementwise ops around them, several results: a row program.
      std::string why4;
      if (HasReduce())
        if (auto p = MatchRowProgram(g, dev, &why4)) return p;
      if (!why4.empty()) why3 += "; as a row program: " + why4;
      Fail("groups with " + std::to_string(g.outputs.size()) + " outputs have no prebuilt kernel (" + expr +
           (why2.empty() ? std::string("") : "; as a chain with a second output: " + why2) +
           "; as a register program: " + why3 + ")");
      return nullptr;
    }
    typedef std::unique_ptr<CompiledGroup> (Matcher::*Fn)(const std::string&);
    const Fn fns[] = {&Matcher::MatchAddRelu, &Matcher::MatchBiasScaleTanhCast, &Matcher::MatchBatchNorm,
                      &Matcher::MatchBnTrainApply, &Matcher::MatchBnGradApply,  &Matcher::MatchTransform,
                      &Matcher::MatchBnGradStats,
                      &Matcher::MatchReduce,
                      &Matcher::MatchSoftmax,      &Matcher::MatchLayerNorm};
    for (Fn f : fns) {
      auto p = (this->*f)(expr);
      if (p) return p;
      if (err && !err->empty()) return nullptr;  // a matcher recognised the form but rejected its details
    }
    // A reduction whose operand is an elementwise chain: the chain runs inside the reduction kernel.
    std::string why_reduce;
    if (auto p = MatchChainReduce(g, dev, &why_reduce)) return p;
    if (HasReduce()) {
      // Anything else with reductions over the trailing axes: a row program (elementwise ops before, between and
      // after the reductions, one kernel).
      std::string why_row;
      if (auto p = MatchRowProgram(g, dev, &why_row)) return p;
      if (!why_reduce.empty() || !why_row.empty()) {
        Fail("no prebuilt sm_100a kernel matches expression " + expr + " (" + why_reduce +
             (why_row.empty() ? std::string("") : "; as a row program: " + why_row) + ")");
        return nullptr;
      }
    }
    if (!why_reduce.empty()) {
      Fail("no prebuilt sm_100a kernel matches expression " + expr + " (" + why_reduce + ")");
      return nullptr;
    }
    // Last resort for elementwise / broadcast groups: a linear chain run by the generic kernel.
    std::string why;
    if (auto p = MatchGenericChain(g, dev, &why)) return p;
    // An elementwise group that is not a chain (a value used twice, more operands): a register program.
    std::string why_dag;
    if (auto p = MatchDag(g, dev, &why_dag)) return p;
    Fail("no prebuilt sm_100a kernel matches expression " + expr + " (as an elementwise chain: " + why +
         "; as a register program: " + why_dag + ")");
    return nullptr;
  }
};

}  // namespace

std::unique_ptr<CompiledGroup> CompileGroup(const GroupDesc& g, const DeviceInfo& dev, std::string* err) {
  std::string local;
  Matcher m(g, dev, err ? err : &local);
  return m.Run();
}

}  // namespace cinn_b200
