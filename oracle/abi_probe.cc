// Prints, as JSON, the layout facts of the reference's runtime ABI as its OWN header and its OWN
// cinn_runtime.cc define them.  Test infrastructure: compiled against a CINN checkout (make ref) and
// used to (re)generate tests/golden/abi_layout.json; the product never includes the reference header.
#include <cstddef>
#include <cstdio>
#include <cstring>

#include "cinn/runtime/cinn_runtime.h"

#pragma GCC diagnostic ignored "-Winvalid-offsetof"

template <typename T>
static void dump_pod(const char* name, T v, bool last = false) {
  cinn_pod_value_t p(v);
  unsigned char raw[16];
  std::memcpy(raw, &p, 16);
  std::printf("    \"%s\": {\"type_code\": %d, \"data_addr_offset\": %d, \"bytes\": \"", name, p.type_code(),
              static_cast<int>(static_cast<char*>(p.data_addr()) - reinterpret_cast<char*>(&p)));
  for (int i = 8; i < 16; ++i) std::printf("%02x", raw[i]);
  std::printf("\"}%s\n", last ? "" : ",");
}

int main() {
  std::printf("{\n");
  std::printf("  \"sizeof_cinn_type_t\": %zu,\n", sizeof(cinn_type_t));
  std::printf("  \"sizeof_cinn_buffer_t\": %zu,\n", sizeof(cinn_buffer_t));
  std::printf("  \"sizeof_cinn_pod_value_t\": %zu,\n", sizeof(cinn_pod_value_t));
  std::printf("  \"type_offsets\": {\"code\": %zu, \"bits\": %zu, \"lanes\": %zu, \"num_asterisks\": %zu},\n",
              offsetof(cinn_type_t, code), offsetof(cinn_type_t, bits), offsetof(cinn_type_t, lanes),
              offsetof(cinn_type_t, num_asterisks));
  std::printf(
      "  \"buffer_offsets\": {\"device\": %zu, \"device_interface\": %zu, \"memory\": %zu, \"flag\": %zu, "
      "\"type\": %zu, \"dimensions\": %zu, \"dims\": %zu, \"lazy\": %zu, \"memory_size\": %zu, \"align\": %zu, "
      "\"external_malloc\": %zu, \"external_free\": %zu},\n",
      offsetof(cinn_buffer_t, device), offsetof(cinn_buffer_t, device_interface), offsetof(cinn_buffer_t, memory),
      offsetof(cinn_buffer_t, flag), offsetof(cinn_buffer_t, type), offsetof(cinn_buffer_t, dimensions),
      offsetof(cinn_buffer_t, dims), offsetof(cinn_buffer_t, lazy), offsetof(cinn_buffer_t, memory_size),
      offsetof(cinn_buffer_t, align), offsetof(cinn_buffer_t, external_malloc),
      offsetof(cinn_buffer_t, external_free));
  std::printf("  \"buffer_max_dims\": %d,\n", CINN_BUFFER_MAX_DIMS);
  std::printf("  \"buffer_kind\": {\"on_host\": %d, \"on_device\": %d},\n", cinn_buffer_on_host, cinn_buffer_on_device);
  cinn_type_t f32 = cinn_float32_t(), f16 = cinn_float16_t(), bf16 = cinn_bfloat16_t(), i32 = cinn_int32_t(),
              b1 = cinn_bool_t(), f64 = cinn_float64_t(), i64 = cinn_int64_t(), u8 = cinn_uint8_t();
  std::printf(
      "  \"types\": {\"float32\": [%d, %d], \"float16\": [%d, %d], \"bfloat16\": [%d, %d], \"int32\": [%d, %d], "
      "\"bool\": [%d, %d], \"float64\": [%d, %d], \"int64\": [%d, %d], \"uint8\": [%d, %d]},\n",
      f32.code, f32.bits, f16.code, f16.bits, bf16.code, bf16.bits, i32.code, i32.bits, b1.code, b1.bits, f64.code,
      f64.bits, i64.code, i64.bits, u8.code, u8.bits);
  std::printf("  \"pods\": {\n");
  cinn_buffer_t* buf = reinterpret_cast<cinn_buffer_t*>(0x1122334455667788ULL);
  dump_pod("buffer", buf);
  dump_pod("int32_minus7", static_cast<int32_t>(-7));
  dump_pod("int64_big", static_cast<int64_t>(0x0102030405060708LL));
  dump_pod("float_1p5", 1.5f);
  dump_pod("double_pi", 3.141592653589793);
  dump_pod("bool_true", true);
  dump_pod("uint32_max", static_cast<uint32_t>(0xffffffffu));
  dump_pod("voidp", reinterpret_cast<void*>(0xdeadbeefULL), true);
  std::printf("  }\n}\n");
  return 0;
}
