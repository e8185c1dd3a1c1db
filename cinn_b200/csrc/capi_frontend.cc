// C ABI of the NetBuilder / Computation layer (see include/cinn_b200.h for the contract of each function).
#include <cstring>
#include <sstream>

#include "../../include/cinn_b200.h"
#include "frontend.h"

using namespace cinn_b200;

namespace cinn_b200 {
int SetLastError(int code, const std::string& message);  // runtime.cc
}

struct cinn_b200_builder {
  NetBuilder builder;
  explicit cinn_b200_builder(const char* name) : builder(name ? name : "net") {}
};
struct cinn_b200_computation {
  std::unique_ptr<Computation> impl;
};

static int CopyText(const std::string& s, char* out, size_t len) {
  if (!out || len == 0) return CINN_B200_OK;
  if (s.size() + 1 > len) return SetLastError(CINN_B200_ENOSPACE, "caller buffer too small for '" + s + "'");
  memcpy(out, s.c_str(), s.size() + 1);
  return CINN_B200_OK;
}

static std::map<std::string, std::string> ParseAttrs(const char* attrs) {
  std::map<std::string, std::string> m;
  if (!attrs) return m;
  std::istringstream is(attrs);
  std::string kv;
  while (is >> kv) {
    auto eq = kv.find('=');
    if (eq != std::string::npos) m[kv.substr(0, eq)] = kv.substr(eq + 1);
  }
  return m;
}

extern "C" {

cinn_b200_builder* cinn_b200_builder_create(const char* name) { return new cinn_b200_builder(name); }
void cinn_b200_builder_destroy(cinn_b200_builder* b) { delete b; }

int cinn_b200_builder_create_input(cinn_b200_builder* b, const char* dtype, const long long* shape, int ndim,
                                   const char* id_hint, char* id_out, size_t id_len) {
  if (!b || !dtype || (!shape && ndim > 0) || ndim < 0) return SetLastError(CINN_B200_EINVAL, "create_input: bad argument");
  std::vector<int64_t> sh(shape, shape + ndim);
  std::string err;
  int v = b->builder.CreateInput(DTypeFromName(dtype), sh, id_hint ? id_hint : "", &err);
  if (v < 0) return SetLastError(CINN_B200_EINVAL, err);
  return CopyText(b->builder.vars()[v].id, id_out, id_len);
}

int cinn_b200_builder_add_op(cinn_b200_builder* b, const char* op_type, const char* const* input_ids, int num_inputs,
                             const char* attrs, char* id_out, size_t id_len) {
  if (!b || !op_type || (num_inputs > 0 && !input_ids) || num_inputs < 0) return SetLastError(CINN_B200_EINVAL, "add_op: bad argument");
  std::vector<int> ins;
  for (int i = 0; i < num_inputs; ++i) {
    int v = input_ids[i] ? b->builder.FindVar(input_ids[i]) : -1;
    if (v < 0) return SetLastError(CINN_B200_ENOTFOUND, std::string(op_type) + ": unknown variable '" + (input_ids[i] ? input_ids[i] : "(null)") + "'");
    ins.push_back(v);
  }
  std::string err;
  int v = b->builder.AddOp(op_type, ins, ParseAttrs(attrs), &err);
  if (v < 0) return SetLastError(CINN_B200_EINVAL, err);
  return CopyText(b->builder.vars()[v].id, id_out, id_len);
}

int cinn_b200_builder_var_info(cinn_b200_builder* b, const char* id, char* dtype, size_t dtype_len, long long* shape,
                               int* ndim) {
  if (!b || !id) return SetLastError(CINN_B200_EINVAL, "var_info: bad argument");
  int v = b->builder.FindVar(id);
  if (v < 0) return SetLastError(CINN_B200_ENOTFOUND, std::string("unknown variable '") + id + "'");
  const Variable& var = b->builder.vars()[v];
  if (ndim) *ndim = (int)var.shape.size();
  if (shape)
    for (size_t i = 0; i < var.shape.size(); ++i) shape[i] = var.shape[i];
  return CopyText(DTypeName(var.dtype), dtype, dtype_len);
}

int cinn_b200_builder_apply_passes(cinn_b200_builder* b, const char* const* passes, int num_passes,
                                   const char* const* fetch_ids, int num_fetch) {
  if (!b || num_passes < 0 || num_fetch < 0 || (num_passes > 0 && !passes) || (num_fetch > 0 && !fetch_ids))
    return SetLastError(CINN_B200_EINVAL, "apply_passes: bad argument");
  std::vector<int> fetch;
  for (int i = 0; i < num_fetch; ++i) {
    int v = fetch_ids[i] ? b->builder.FindVar(fetch_ids[i]) : -1;
    if (v < 0) return SetLastError(CINN_B200_ENOTFOUND, "apply_passes: unknown fetch variable");
    fetch.push_back(v);
  }
  std::vector<std::string> names;
  for (int i = 0; i < num_passes; ++i) names.push_back(passes[i] ? passes[i] : "");
  if (names.empty()) names = DefaultProgramPasses();
  for (auto& name : names) {
    std::string err;
    if (!ApplyProgramPass(&b->builder, name, fetch, &err)) return SetLastError(CINN_B200_EINVAL, err);
  }
  return CINN_B200_OK;
}

long long cinn_b200_builder_program_text(cinn_b200_builder* b, char* out, size_t out_len) {
  if (!b) return SetLastError(CINN_B200_EINVAL, "program_text: null builder");
  const std::string text = PrintProgram(b->builder);
  if (out && out_len > 0) {
    const size_t n = std::min(out_len - 1, text.size());
    memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return (long long)text.size() + 1;
}

cinn_b200_computation* cinn_b200_computation_build_and_compile(cinn_b200_builder* b, int device,
                                                               const char* const* fetch_ids, int num_fetch) {
  if (!b) {
    SetLastError(CINN_B200_EINVAL, "build_and_compile: null builder");
    return nullptr;
  }
  std::vector<int> fetch;
  for (int i = 0; i < num_fetch; ++i) {
    int v = fetch_ids && fetch_ids[i] ? b->builder.FindVar(fetch_ids[i]) : -1;
    if (v < 0) {
      SetLastError(CINN_B200_ENOTFOUND, "build_and_compile: unknown fetch variable");
      return nullptr;
    }
    fetch.push_back(v);
  }
  std::string err;
  auto impl = Computation::BuildAndCompile(b->builder, fetch, device, &err);
  if (!impl) {
    SetLastError(CINN_B200_ENOMATCH, err);
    return nullptr;
  }
  auto* c = new cinn_b200_computation();
  c->impl = std::move(impl);
  return c;
}

void cinn_b200_computation_destroy(cinn_b200_computation* c) { delete c; }

long long cinn_b200_computation_export(cinn_b200_computation* c, char* out, size_t out_len) {
  if (!c) return SetLastError(CINN_B200_EINVAL, "export: null computation");
  const std::string text = c->impl->Export();
  if (out && out_len > 0) {
    const size_t n = std::min(out_len - 1, text.size());
    memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return (long long)text.size() + 1;
}

cinn_b200_computation* cinn_b200_program_load(const char* text, int device) {
  if (!text) {
    SetLastError(CINN_B200_EINVAL, "program_load: null text");
    return nullptr;
  }
  std::string err;
  auto impl = Computation::Load(text, device, &err);
  if (!impl) {
    SetLastError(CINN_B200_ENOMATCH, err);
    return nullptr;
  }
  auto* c = new cinn_b200_computation();
  c->impl = std::move(impl);
  return c;
}

int cinn_b200_computation_execute_graph(cinn_b200_computation* c, void* stream) {
  if (!c) return SetLastError(CINN_B200_EINVAL, "execute_graph: null computation");
  std::string err;
  int rc = c->impl->ExecuteGraph(stream, &err);
  if (rc != CINN_B200_OK) return SetLastError(rc, err);
  return CINN_B200_OK;
}

int cinn_b200_computation_execute_test(cinn_b200_computation* c, int repeat, double* avg_ms) {
  if (!c) return SetLastError(CINN_B200_EINVAL, "execute_test: null computation");
  std::string err;
  // repeat < 0: the same measurement with the program replayed from its CUDA graph
  int rc = c->impl->ExecuteTest(repeat < 0 ? -repeat : repeat, avg_ms, &err, repeat < 0);
  if (rc != CINN_B200_OK) return SetLastError(rc, err);
  return CINN_B200_OK;
}

int cinn_b200_computation_execute(cinn_b200_computation* c, void* stream) {
  if (!c) return SetLastError(CINN_B200_EINVAL, "execute: null computation");
  std::string err;
  int rc = c->impl->Execute(stream, &err);
  return rc == CINN_B200_OK ? rc : SetLastError(rc, err);
}

int cinn_b200_computation_set_tensor_data(cinn_b200_computation* c, const char* id, const void* host, size_t bytes) {
  if (!c || !id || !host) return SetLastError(CINN_B200_EINVAL, "set_tensor_data: bad argument");
  std::string err;
  int rc = c->impl->SetTensorData(id, host, bytes, &err);
  return rc == CINN_B200_OK ? rc : SetLastError(rc, err);
}

int cinn_b200_computation_get_tensor_data(cinn_b200_computation* c, const char* id, void* host, size_t bytes) {
  if (!c || !id || !host) return SetLastError(CINN_B200_EINVAL, "get_tensor_data: bad argument");
  std::string err;
  int rc = c->impl->GetTensorData(id, host, bytes, &err);
  return rc == CINN_B200_OK ? rc : SetLastError(rc, err);
}

int cinn_b200_computation_bind_tensor(cinn_b200_computation* c, const char* id, void* device_ptr) {
  if (!c || !id) return SetLastError(CINN_B200_EINVAL, "bind_tensor: bad argument");
  std::string err;
  int rc = c->impl->BindTensor(id, device_ptr, &err);
  return rc == CINN_B200_OK ? rc : SetLastError(rc, err);
}

int cinn_b200_computation_num_tensors(cinn_b200_computation* c) { return c ? (int)c->impl->tensor_names().size() : 0; }

const char* cinn_b200_computation_tensor_name(cinn_b200_computation* c, int index) {
  if (!c || index < 0 || index >= (int)c->impl->tensor_names().size()) return nullptr;
  return c->impl->tensor_names()[index].c_str();
}

int cinn_b200_computation_tensor_info(cinn_b200_computation* c, const char* id, char* dtype, size_t dtype_len,
                                      long long* shape, int* ndim, void** device_ptr) {
  if (!c || !id) return SetLastError(CINN_B200_EINVAL, "tensor_info: bad argument");
  ScopeTensor* t = c->impl->Find(id);
  if (!t) return SetLastError(CINN_B200_ENOTFOUND, std::string("no tensor named '") + id + "'");
  if (ndim) *ndim = (int)t->var.shape.size();
  if (shape)
    for (size_t i = 0; i < t->var.shape.size(); ++i) shape[i] = t->var.shape[i];
  if (device_ptr) *device_ptr = t->buffer.memory;
  return CopyText(DTypeName(t->var.dtype), dtype, dtype_len);
}

int cinn_b200_computation_tensor_role(cinn_b200_computation* c, const char* id) {
  if (!c || !id) return SetLastError(CINN_B200_EINVAL, "tensor_role: bad argument");
  if (!c->impl->Find(id)) return SetLastError(CINN_B200_ENOTFOUND, std::string("no tensor named '") + id + "'");
  bool written = false, read = false;
  for (auto& g : c->impl->groups()) {
    if (g.pattern == "reshape_alias") {
      // an alias group reads its operand and defines its result
      for (auto& op : g.desc.ops) {
        written = written || op.output == id;
        for (auto& in : op.inputs) read = read || in == id;
      }
      continue;
    }
    for (auto& t : g.desc.outputs) written = written || t.name == id;
    for (auto& t : g.desc.inputs) read = read || t.name == id;
  }
  for (auto& a : c->impl->aliases()) {
    written = written || a.first == id;
    read    = read || a.second == id;
  }
  return !written ? 0 : (read ? 1 : 2);
}

int cinn_b200_computation_num_groups(cinn_b200_computation* c) { return c ? (int)c->impl->groups().size() : 0; }

int cinn_b200_computation_group_desc(cinn_b200_computation* c, int index, char* out, size_t len) {
  if (!c || index < 0 || index >= (int)c->impl->groups().size()) return SetLastError(CINN_B200_EINVAL, "group_desc: bad index");
  return CopyText(PrintGroupDesc(c->impl->groups()[index].desc), out, len);
}

int cinn_b200_computation_group_pattern(cinn_b200_computation* c, int index, char* out, size_t len) {
  if (!c || index < 0 || index >= (int)c->impl->groups().size()) return SetLastError(CINN_B200_EINVAL, "group_pattern: bad index");
  const FusedGroupInfo& g = c->impl->groups()[index];
  std::string s           = g.pattern;
  for (auto& k : g.kernels) s += " " + k;
  return CopyText(s, out, len);
}

}  // extern "C"
