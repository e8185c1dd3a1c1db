// Row programs: of the specialised kernels of row_prog_static_table.inc, the form with half a CTA per row (key
// "row_program_h") and its kernels for rows of exactly 8 / 6 / 4 / 2 vectors per thread (4096 / 3072 / 2048 / 1024
// elements; keys "row_program_h8" ...).  The kernels' code is in row_prog_body.cuh.
#include "row_prog_body.cuh"

namespace cinn_b200 {

#define STATIC_ROW_PROGRAM(ID, META, COUNTS, ...) \
  ROWP_ONE(ID, "_h", "row_program_h", 3, 0, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_h8", "row_program_h8", 3, 8, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_h6", "row_program_h6", 3, 6, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_h4", "row_program_h4", 3, 4, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_h2", "row_program_h2", 3, 2, META, COUNTS, __VA_ARGS__)

#include "row_prog_static_table.inc"

}  // namespace cinn_b200
