/*
 * Argument and buffer model of the CINN runtime, restated layout-for-layout.
 *
 * The structures here are what a fused-group entry point receives from the
 * reference executor: an array of 16-byte tagged values, most of which point
 * at 120-byte buffer descriptors.  They follow cinn/runtime/cinn_runtime.h
 * (type tag :51-93, device kind :147-160, buffer :186-292, tagged value
 * :390-498).  Field names, order, widths and offsets are identical so that a
 * pointer produced by the reference can be read through these declarations
 * and vice versa; the static assertions at the end pin every offset.
 *
 * When this header is compiled inside the reference tree (its own header has
 * already been included) nothing is declared twice: the reference's
 * definitions are used as they are.
 */
#ifndef CINN_B200_RUNTIME_ABI_H_
#define CINN_B200_RUNTIME_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifndef CINN_RUNTIME_CINN_RUNTIME_H_

#ifdef __cplusplus
extern "C" {
#endif

/* cinn_runtime.h:51-58 — scalar class of an element type. */
typedef enum cinn_type_code_t {
  cinn_type_unk    = -1,
  cinn_type_int    = 0,
  cinn_type_uint   = 1,
  cinn_type_float  = 2,
  cinn_type_handle = 3,
  cinn_type_bfloat = 4
} cinn_type_code_t;

/* cinn_runtime.h:67-93 — 12 bytes: code@0 (int), bits@4, lanes@6, num_asterisks@8. */
typedef struct cinn_type_t {
  cinn_type_code_t code;
  uint8_t bits;
  uint16_t lanes;
  uint8_t num_asterisks;
} cinn_type_t;

/* cinn_runtime.h:147-153 — where a buffer lives. */
typedef enum cinn_device_kind_t {
  cinn_unk_device    = -1,
  cinn_x86_device    = 0,
  cinn_opencl_device = 1,
  cinn_arm_device    = 2
} cinn_device_kind_t;

/* cinn_runtime.h:166-171 — bits of cinn_buffer_t::flag. */
typedef enum cinn_buffer_kind_t {
  cinn_buffer_on_host   = 0,
  cinn_buffer_on_device = 1 << 1
} cinn_buffer_kind_t;

typedef int cinn_dimension_t;

#define CINN_BUFFER_MAX_DIMS 8

struct cinn_device_interface_t;

/*
 * cinn_runtime.h:186-292 — buffer descriptor, 120 bytes.
 * `memory` is a host pointer for the x86 target and a device pointer for the
 * GPU target; kernels receive `&memory` from the launch primitive.
 * The last two fields are pointers to std::function objects in the reference;
 * they are opaque here and never dereferenced by this library.
 */
typedef struct cinn_buffer_t {
  cinn_device_kind_t device;                             /* @0   */
  const struct cinn_device_interface_t* device_interface; /* @8   */
  uint8_t* memory;                                       /* @16  */
  uint64_t flag;                                         /* @24  */
  cinn_type_t type;                                      /* @32  */
  int32_t dimensions;                                    /* @44  */
  cinn_dimension_t dims[CINN_BUFFER_MAX_DIMS];           /* @48  */
  char lazy;                                             /* @80  */
  uint64_t memory_size;                                  /* @88  */
  uint16_t align;                                        /* @96  */
  void* external_malloc;                                 /* @104 */
  void* external_free;                                   /* @112 */
} cinn_buffer_t;

/* cinn_runtime.h:390-395 — payload of a tagged value. */
union cinn_value_t {
  int64_t v_int64;
  double v_float64;
  void* v_handle;
  char* v_str;
};

/* cinn_runtime.h:397-460 — 16 bytes: type_code_@0, value_@8. */
typedef struct cinn_pod_value_t {
  int type_code_;
  union cinn_value_t value_;
} cinn_pod_value_t;

/* cinn_runtime.h:497-499 — entry-point types stored in an Instruction. */
typedef void (*lower_func_ptr_t)(void*, int32_t);
typedef void (*lower_func_ptr_g)(void*, int32_t, void*);

#ifdef __cplusplus
}
static_assert(sizeof(cinn_buffer_t) == 120, "cinn_buffer_t is 120 bytes");
static_assert(offsetof(cinn_buffer_t, memory) == 16 && offsetof(cinn_buffer_t, flag) == 24 &&
                  offsetof(cinn_buffer_t, type) == 32 && offsetof(cinn_buffer_t, dimensions) == 44 &&
                  offsetof(cinn_buffer_t, dims) == 48 && offsetof(cinn_buffer_t, lazy) == 80 &&
                  offsetof(cinn_buffer_t, memory_size) == 88 && offsetof(cinn_buffer_t, align) == 96 &&
                  offsetof(cinn_buffer_t, external_malloc) == 104 && offsetof(cinn_buffer_t, external_free) == 112,
              "cinn_buffer_t field offsets");
#endif

#endif /* !CINN_RUNTIME_CINN_RUNTIME_H_ */

/*
 * cinn_runtime.h:467-488 — the numeric tag stored in cinn_pod_value_t::type_code_
 * for each C type.  Floats travel as double (cinn_runtime.cc:274-281).
 */
enum cinn_b200_pod_code {
  CINN_POD_INT32   = 0,
  CINN_POD_INT64   = 1,
  CINN_POD_FLOAT   = 2,
  CINN_POD_DOUBLE  = 3,
  CINN_POD_VOIDP   = 4,
  CINN_POD_CHARP   = 5,
  CINN_POD_CCHARP  = 6,
  CINN_POD_BUFFERP = 7,
  CINN_POD_INT8    = 8,
  CINN_POD_BOOL    = 9,
  CINN_POD_FLOAT16 = 10,
  CINN_POD_INT16   = 11,
  CINN_POD_UINT8   = 12,
  CINN_POD_UINT16  = 13,
  CINN_POD_UINT32  = 14,
  CINN_POD_UINT64  = 15,
  CINN_POD_BFLOAT16 = 16
};

#ifdef __cplusplus
static_assert(sizeof(cinn_type_t) == 12, "cinn_type_t is 12 bytes");
static_assert(offsetof(cinn_type_t, bits) == 4 && offsetof(cinn_type_t, lanes) == 6 &&
                  offsetof(cinn_type_t, num_asterisks) == 8,
              "cinn_type_t field offsets");
static_assert(sizeof(cinn_pod_value_t) == 16 && offsetof(cinn_pod_value_t, value_) == 8, "tagged value layout");
#endif

#endif /* CINN_B200_RUNTIME_ABI_H_ */
