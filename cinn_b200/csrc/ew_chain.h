// Program encoding of the generic elementwise-chain kernel, shared by the kernel and the matcher.
//
// A step is one 64-bit word: bits 0-7 opcode, 8-15 operand A selector (0 = the immediate, 1..3 = side input,
// 4 = the chain value itself),
// 16-23 operand B selector (EW_FMA only: 0 = the immediate of the NEXT word, which is then skipped),
// bit 24 "swap" (the side operand is the LEFT operand of a binary op), bits 32-63 an fp32 immediate.
#pragma once

namespace cinn_b200 {

constexpr int EW_MAX_STEPS = 16;

enum EwOp {
  EW_NOP = 0,
  // binary: acc = acc (op) operand, or operand (op) acc when swapped
  EW_ADD = 1, EW_SUB, EW_MUL, EW_DIV, EW_MAX, EW_MIN, EW_POW,
  EW_EQ, EW_NE, EW_GT, EW_LT, EW_GE, EW_LE,
  EW_FMA = 20,        // acc = fma(acc, A, B)
  EW_SCALE_PRE = 21,  // acc = imm * (acc + imm_next)
  // unary
  EW_FIRST_UNARY = 32,
  EW_EXP = 32, EW_TANH, EW_SIGMOID, EW_RSQRT, EW_SQRT, EW_RELU, EW_NEG, EW_ABS, EW_LOG, EW_FLOOR, EW_CEIL, EW_ERF,
  EW_SIN, EW_COS, EW_RECIP, EW_ROUND, EW_TRUNC, EW_SIGN, EW_RELU6, EW_LOG2, EW_LOG10,
  EW_ROUND_F16, EW_ROUND_BF16, EW_IDENTITY
};

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
