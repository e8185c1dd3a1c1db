// Shared starts of a row program's passes.
//
// A later pass of a row program evaluates what it needs again from the inputs: softmax's second pass computes
// x * scale - max once more, its third pass exp(...) once more.  Where the element programs of passes p .. last begin
// with the same steps, and only ONE register of that shared start is read by what follows in the later passes, the
// specialised kernels keep that register's value per cached vector at the end of the shared start in pass p (in
// place of a cached input that nothing loads afterwards), and the later passes begin after it.  This file finds those points from the step words alone (constexpr: the kernels
// evaluate it on their template arguments, the matcher on the program it built, which also compares the immediates
// of the shared steps, the one thing the kernels cannot know at build time).
#pragma once
#include <cstdint>

#include "ew_chain.h"

namespace cinn_b200 {

struct RowPrefixPlan {
  int start[ROWP_MAX_PASSES];  // words of pass p's element program that are skipped (its value comes from the slot)
  int save[ROWP_MAX_PASSES];   // after this many words pass p writes register save_reg[p] into the slot (0: never)
  int reg[ROWP_MAX_PASSES];    // the register pass p starts from (start > 0) -- the one the saving pass kept
  int save_reg[ROWP_MAX_PASSES];
  int slot;  // the input whose cached copy the kept value replaces
};

namespace row_prefix {
constexpr int Op(uint32_t w) { return (int)(w & 0xff); }
constexpr int Dst(uint32_t w) { return (int)((w >> 8) & 15); }
constexpr int SelA(uint32_t w) { return (int)((w >> 12) & 31); }
constexpr int SelB(uint32_t w) { return (int)((w >> 17) & 31); }
constexpr int SelC(uint32_t w) { return (int)((w >> 22) & 31); }
constexpr bool IsPlain(uint32_t w) {  // an arithmetic step (not a load, store, fold or filler)
  return Op(w) != EW_NOP && Op(w) != DAG_LOAD && Op(w) != DAG_STORE && Op(w) != ROWP_ACC;
}
constexpr int Words(uint32_t w) {
  return IsPlain(w) && (SelA(w) == DAG_IMM2 || SelB(w) == DAG_IMM2 || SelC(w) == DAG_IMM2 || Op(w) == EW_SCALE_PRE) ? 2 : 1;
}
// how many operand selectors the step reads: unary ops and the pre-scaled form one, fma / select three, others two
constexpr int Operands(uint32_t w) {
  if (!IsPlain(w)) return 0;
  if (Op(w) >= EW_FIRST_UNARY || Op(w) == EW_SCALE_PRE) return 1;
  return (Op(w) == EW_FMA || Op(w) == EW_SELECT) ? 3 : 2;
}
constexpr int Sel(uint32_t w, int k) { return k == 0 ? SelA(w) : (k == 1 ? SelB(w) : SelC(w)); }
// bit r: vector register r is read by the step
constexpr unsigned RegReads(uint32_t w) {
  if (Op(w) == DAG_STORE) return 1u << (SelA(w) & 7);
  if (Op(w) == ROWP_ACC) return 1u << (SelA(w) & 7);
  unsigned m = 0;
  for (int k = 0; k < Operands(w); ++k)
    if (Sel(w, k) < DAG_REGS) m |= 1u << Sel(w, k);
  return m;
}
// bit s: scalar register s is read by the (element) step
constexpr unsigned ScalarReads(uint32_t w) {
  unsigned m = 0;
  for (int k = 0; k < Operands(w); ++k)
    if (Sel(w, k) >= ROWP_SREG0) m |= 1u << ((Sel(w, k) - ROWP_SREG0) & 7);
  return m;
}
constexpr int RegWritten(uint32_t w) { return (Op(w) == DAG_LOAD || IsPlain(w)) ? (Dst(w) & 7) : -1; }

constexpr int ElementCount(unsigned long long counts, int pass) { return (int)((counts >> (8 * pass)) & 0xff); }
constexpr int ScalarCount(unsigned long long counts, int pass) { return (int)((counts >> (32 + 8 * pass)) & 0xff); }
constexpr int ElementFirst(unsigned long long counts, int pass) {
  int at = 0;
  for (int k = 0; k < pass; ++k) at += ElementCount(counts, k) + ScalarCount(counts, k);
  return at;
}
constexpr int Passes(unsigned long long counts) {
  int p = 0;
  for (int k = 0; k < ROWP_MAX_PASSES; ++k)
    if (ElementCount(counts, k) || ScalarCount(counts, k)) p = k + 1;
  return p;
}
// the scalar registers that change from the end of pass `from` on: its accumulators and those of the later passes,
// and what their scalar programs write
constexpr unsigned ScalarsWrittenFrom(const uint32_t* words, unsigned long long counts, int from) {
  unsigned m = 0;
  for (int p = from; p < Passes(counts); ++p) {
    const int b = ElementFirst(counts, p), e = b + ElementCount(counts, p), se = e + ScalarCount(counts, p);
    for (int k = b; k < e; k += Words(words[k]))
      if (Op(words[k]) == ROWP_ACC) m |= 1u << (Dst(words[k]) & 7);
    for (int k = e; k < se; k += Words(words[k]))
      if (Op(words[k]) == DAG_LOAD || IsPlain(words[k])) m |= 1u << (Dst(words[k]) & 7);
  }
  return m;
}
// the vector registers the element program of `pass` reads from word `at` on before it writes them
constexpr unsigned LiveIn(const uint32_t* words, unsigned long long counts, int pass, int at) {
  const int b = ElementFirst(counts, pass), e = b + ElementCount(counts, pass);
  unsigned live = 0, written = 0;
  for (int k = b + at; k < e; k += Words(words[k])) {
    live |= RegReads(words[k]) & ~written;
    if (RegWritten(words[k]) >= 0) written |= 1u << RegWritten(words[k]);
  }
  return live;
}
// input `a` is loaded by pass `p` at or after word `at`, or by a later pass at or after word `at`
constexpr bool LoadedLater(const uint32_t* words, unsigned long long counts, int a, int p, int at) {
  for (int q = p; q < Passes(counts); ++q) {
    const int b = ElementFirst(counts, q), e = b + ElementCount(counts, q);
    for (int k = b; k < e; k += Words(words[k]))
      if (k - b >= at && Op(words[k]) == DAG_LOAD && (SelA(words[k]) & 7) == a) return true;
  }
  return false;
}
// input `a` is full-size and loaded by pass 0: the kernels hold it in registers from the row's start on
constexpr bool CachedInput(const uint32_t* words, unsigned long long counts, unsigned long long meta, int a) {
  if (((meta >> (6 * a + 3)) & 7) != (unsigned)EW_SIDE_FULL) return false;
  for (int k = 0; k < ElementCount(counts, 0); k += Words(words[k]))
    if (Op(words[k]) == DAG_LOAD && (SelA(words[k]) & 7) == a) return true;
  return false;
}
}  // namespace row_prefix

// The plan for a program.  Every start is 0 when no pass shares a start worth keeping (a lone load is not: the
// kernels keep loaded inputs in registers anyway).
constexpr RowPrefixPlan PlanRowPrefixes(const uint32_t* words, unsigned long long counts, unsigned long long meta) {
  using namespace row_prefix;
  RowPrefixPlan plan = {};
  const int np = Passes(counts);
  int kept = 0, kept_reg = 0;  // the slot holds register kept_reg after `kept` words of the shared start
  int slot = -1;
  for (int p = 0; p < np; ++p) {
    plan.start[p] = kept;
    plan.reg[p]   = kept_reg;
    plan.save[p] = plan.save_reg[p] = 0;
    if (p + 1 >= np) break;
    const int b = ElementFirst(counts, p), n = ElementCount(counts, p);
    const unsigned changing = ScalarsWrittenFrom(words, counts, p);
    // the longest start of pass p that every later pass repeats word for word, made of loads and arithmetic that
    // reads no scalar register which changes later
    int len = 0;
    while (len < n) {
      const uint32_t w = words[b + len];
      const int nw     = Words(w);
      if (len + nw > n) break;
      if (Op(w) != DAG_LOAD && !IsPlain(w)) break;
      if (ScalarReads(w) & changing) break;
      bool same = true;
      for (int q = p + 1; q < np && same; ++q) {
        if (len + nw > ElementCount(counts, q)) same = false;
        for (int j = 0; j < nw && same; ++j) same = words[ElementFirst(counts, q) + len + j] == words[b + len + j];
      }
      if (!same) break;
      len += nw;
    }
    // walk back to a step after which the later passes read one register only, the one that step wrote
    int best = 0, best_reg = 0;
    for (int at = 0, last = -1; at <= len;) {
      if (at > kept && last >= 0) {
        bool one = true;
        for (int q = p + 1; q < np; ++q) one = one && (LiveIn(words, counts, q, at) & ~(1u << last)) == 0;
        if (one) best = at, best_reg = last;
      }
      if (at >= len) break;
      last = RegWritten(words[b + at]);
      at += Words(words[b + at]);
    }
    // worth keeping: more than a lone load since the previous point
    int plain = 0;
    for (int k = kept; k < best; k += Words(words[b + k]))
      if (IsPlain(words[b + k]) || (k > 0 && Op(words[b + k]) == DAG_LOAD)) ++plain;
    if (best > kept && plain > 0 && slot < 0) {
      for (int a = 0; a < DAG_MAX_IN && slot < 0; ++a)
        if (CachedInput(words, counts, meta, a) && !LoadedLater(words, counts, a, p, best)) slot = a;
    }
    if (best > kept && plain > 0 && slot >= 0) {
      plan.slot        = slot;
      plan.save[p]     = best;
      plan.save_reg[p] = best_reg;
      kept             = best;
      kept_reg         = best_reg;
    }
  }
  return plan;
}

}  // namespace cinn_b200
