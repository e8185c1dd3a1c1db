// Row programs: of the specialised kernels of row_prog_static_table.inc, half a CTA per row for rows of exactly
// 7 / 5 / 3 vectors per thread (3584 / 2560 / 1536 elements; keys "row_program_h7" ...), and a CTA per row of up to
// 8192 elements (key "row_program_c8"; "row_program_c88" ... "_c85" for exactly 8192 / 7168 / 6144 / 5120 elements).
// The kernels' code is in row_prog_body.cuh.
#include "row_prog_body.cuh"

namespace cinn_b200 {

#define STATIC_ROW_PROGRAM(ID, META, COUNTS, ...) \
  ROWP_ONE(ID, "_h7", "row_program_h7", 3, 7, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_h5", "row_program_h5", 3, 5, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_h3", "row_program_h3", 3, 3, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_c8", "row_program_c8", 4, 0, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_c88", "row_program_c88", 4, 8, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_c87", "row_program_c87", 4, 7, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_c86", "row_program_c86", 4, 6, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_c85", "row_program_c85", 4, 5, META, COUNTS, __VA_ARGS__)

#include "row_prog_static_table.inc"

}  // namespace cinn_b200
