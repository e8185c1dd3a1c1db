// Row programs: the interpreting kernel and, of the specialised kernels of row_prog_static_table.inc, the forms with
// a CTA per row of up to 4096 elements (key "row_program") and a warp per row (key "row_program_w"; "row_program_w2",
// "_w4", "_w6", "_w8" for rows of exactly 2 / 4 / 6 / 8 vectors per lane: 256 / 512 / 768 / 1024 elements).  The
// other forms are compiled in row_prog_half.cu and row_prog_half_b.cu, side by side with this file; the kernels'
// code is in row_prog_body.cuh.
#include "row_prog_body.cuh"

namespace cinn_b200 {

CINN_B200_REGISTER_KERNEL_PDL("row_program", 70, 256, k_row_program);

#define STATIC_ROW_PROGRAM(ID, META, COUNTS, ...) \
  ROWP_ONE(ID, "", "row_program", 2, 0, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_w", "row_program_w", 1, 0, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_w8", "row_program_w8", 1, 8, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_w6", "row_program_w6", 1, 6, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_w4", "row_program_w4", 1, 4, META, COUNTS, __VA_ARGS__); \
  ROWP_ONE(ID, "_w2", "row_program_w2", 1, 2, META, COUNTS, __VA_ARGS__)

#include "row_prog_static_table.inc"

}  // namespace cinn_b200
