// Program encoding of the generic elementwise-chain kernel, shared by the kernel and the matcher.
//
// A step is one 64-bit word: bits 0-7 opcode, 8-15 operand A selector (0 = the immediate, 1..3 = side input,
// 4 = the chain value itself),
// 16-23 operand B selector (EW_FMA and EW_SELECT only: 0 = the immediate of the NEXT word, which is then skipped),
// bits 24-25 "swap" for a binary op (1: the side operand is the LEFT operand) or, for EW_SELECT, the role of the
// chain value (0: the condition, A = value if true, B = value if false; 1: the value if true, A = condition,
// B = value if false; 2: the value if false, A = condition, B = value if true), bits 32-63 an fp32 immediate.
// Operand selectors 5 and 6 name two temporaries (float form only): EW_STASH copies the chain value into the
// temporary its A selector names, so that an expression tree runs as: first branch, stash, second branch, join.
// Values of type bool travel as 0.0f / 1.0f.  The integer form of the kernel (ew_chain_int.cu) uses the same words
// with a signed 32-bit integer in bits 32-63; bool travels as 0 / 1.  The float64 form (ew_chain_f64.cu) keeps in
// bits 32-63 an index into a table of eight double immediates.
#pragma once

namespace cinn_b200 {

constexpr int EW_MAX_STEPS = 16;

enum EwOp {
  EW_NOP = 0,
  // binary: acc = acc (op) operand, or operand (op) acc when swapped
  EW_ADD = 1, EW_SUB, EW_MUL, EW_DIV, EW_MAX, EW_MIN, EW_POW,
  EW_EQ, EW_NE, EW_GT, EW_LT, EW_GE, EW_LE,
  EW_MOD = 14, EW_FLOOR_DIV, EW_ATAN2, EW_LAND, EW_LOR, EW_LXOR,
  // integer chains only
  EW_BAND = 23, EW_BOR, EW_BXOR, EW_SHL, EW_SHR, EW_LSHR,
  EW_COPY = 29,  // acc = operand: how a chain starts from a broadcast operand when no input has the output's size
  EW_STASH = 30, // temporary[A - 5] = acc (kernels with temporaries only)
  EW_STORE2 = 31, // second output[i] = acc: a value on the way that is a group output too (same kernels)
  EW_FMA = 20,        // acc = fma(acc, A, B)
  EW_SCALE_PRE = 21,  // acc = imm * (acc + imm_next)
  EW_SELECT = 22,     // acc = cond ? t : f, see the role bits above
  // unary
  EW_FIRST_UNARY = 32,
  EW_EXP = 32, EW_TANH, EW_SIGMOID, EW_RSQRT, EW_SQRT, EW_RELU, EW_NEG, EW_ABS, EW_LOG, EW_FLOOR, EW_CEIL, EW_ERF,
  EW_SIN, EW_COS, EW_RECIP, EW_ROUND, EW_TRUNC, EW_SIGN, EW_RELU6, EW_LOG2, EW_LOG10,
  EW_ROUND_F16, EW_ROUND_BF16, EW_IDENTITY,
  EW_TAN, EW_SINH, EW_COSH, EW_ASIN, EW_ACOS, EW_ATAN, EW_ASINH, EW_ACOSH, EW_ATANH, EW_CBRT,
  EW_ISNAN, EW_ISINF, EW_ISFINITE, EW_LNOT,
  EW_TO_BOOL,  // x != 0 ? 1 : 0 (cast to bool in the middle of a chain)
  EW_BNOT, EW_CLZ, EW_POPC  // integer chains only
};

// ---- register programs (ew_dag.cu) --------------------------------------------------------------------------------
// An elementwise group that is not a chain (a value used twice, several outputs, more operands) runs as a register
// program: up to DAG_MAX_IN inputs, DAG_MAX_OUT outputs of one shape, DAG_REGS vector registers.  A step word holds
// bits 0-7 the op (an EwOp, or DAG_LOAD / DAG_STORE), 8-11 the destination register (DAG_STORE: the output index),
// 12-16 / 17-21 / 22-26 operands A / B / C (0-7 a register, DAG_IMM the word's immediate, DAG_IMM2 the immediate of the
// NEXT word, which is then skipped; DAG_LOAD: A is the input index), bits 32-63 an fp32 immediate.
// Unary ops: dst = op(A).  Binary ops: dst = A op B.  EW_FMA: dst = fma(A, B, C).  EW_SELECT: dst = A != 0 ? B : C.
// EW_SCALE_PRE: dst = imm * (A + imm2).  The kernel's meta word packs, per input k, bits 6k..6k+2 the storage type
// and 6k+3..6k+5 the addressing mode, and per output j bits 48+3j..50+3j the storage type.
constexpr int DAG_MAX_IN = 8, DAG_MAX_OUT = 4, DAG_MAX_STEPS = 30, DAG_REGS = 8;
constexpr int DAG_LOAD = 200, DAG_STORE = 201;
constexpr int DAG_IMM = 8, DAG_IMM2 = 9;

// ---- row programs (row_prog.cu) ------------------------------------------------------------------------------------
// A group with reductions over the trailing axes and elementwise ops either side of them runs as a row program over
// x viewed as [rows, r]: up to ROWP_MAX_PASSES passes over a row, each an element program (register-program steps
// run on every vector of the row, with ROWP_ACC steps that fold a register into a row accumulator) followed, after
// the accumulators have been combined across the row's threads, by a scalar program run once per row on the row's
// ROWP_SREGS scalar registers.  Step words are those of the register programs with three additions: operand selectors
// 16-23 name scalar register 0-7 (its value for every element); ROWP_ACC: scalar register `dst` receives the fold,
// by reduce kind C (0 sum, 1 prod, 2 max, 3 min), of register A over the row; in a scalar program the registers ARE
// the scalar registers, DAG_LOAD reads an input at the row index and DAG_STORE writes a per-row output.
// counts word: bits 8p..8p+7 = element steps of pass p, bits 32+8p.. = scalar steps of pass p (steps are laid out
// pass by pass, element program then scalar program).
constexpr int ROWP_MAX_PASSES = 3, ROWP_MAX_STEPS = 36, ROWP_SREGS = 8, ROWP_MAX_ACC = 4;
constexpr int ROWP_ACC = 202;
constexpr int ROWP_SREG0 = 16;

// Storage types of the chain kernel's operands (runtime codes; the output type is a template parameter).
// EW_NO_INPUT as the type of the chain input: there is none, the program starts with EW_COPY.
enum EwDType { EW_NO_INPUT = 15, EW_F32 = 0, EW_F16 = 1, EW_BF16 = 2, EW_BOOL = 3, EW_I32 = 4, EW_I64 = 5, EW_F64 = 6, EW_U8 = 7 };

// How a side input is addressed for the flat output index i: value = side[(i / inner) % mid].
enum EwSideMode {
  EW_SIDE_NONE = 0,
  EW_SIDE_FULL,          // same element count as the output: vector load at i
  EW_SIDE_ONE_PER_VEC,   // inner % 4 == 0: one value serves a whole 4-element vector
  EW_SIDE_PERIODIC_VEC,  // inner == 1 and mid % 4 == 0: vector load at i % mid
  EW_SIDE_GENERIC,       // one index computation per element
  EW_SIDE_SCALAR         // a single element
};

}  // namespace cinn_b200
