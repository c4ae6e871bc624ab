// Host-side layout services: validation, constant folding of a staged layout
// into digit strides, strength-reduced divisors, and the compact programs the
// device kernels take as launch parameters.
#pragma once

#include <cstdint>
#include <vector>

#include "../../include/lego_b200.h"

namespace lego {

// ---- strength-reduced division ------------------------------------------------
// Unsigned division of n < 2^31 by a constant 1 <= d < 2^31.
//   power of two : q = n >> shr                       (mul == 0)
//   otherwise    : q = umulhi(n, mul) >> shr, mul = ceil(2^(31+s) / d), shr = s - 1,
//                  s = ceil(log2 d)  (round-up method, exact for every n < 2^31)
struct FastDiv {
  uint32_t d;
  uint32_t mul;
  uint32_t shr;
};
FastDiv make_fastdiv(uint64_t d);

// One term of a digit-sum program: out[dst] += ((x[src] / a) % m) * b.
// m == 0 means "no wrap" (the digit is the most significant one of its source).
struct DigitTerm {
  int32_t src;
  int32_t dst;
  FastDiv a;
  FastDiv m;
  uint64_t a64;
  uint64_t m64;
  uint64_t b;
};

struct DigitProgram {
  int32_t n_terms;
  int32_t n_src;
  int32_t n_dst;
  int32_t wide;  // 1: values may reach 2^31, use the 64-bit fields
  DigitTerm t[LEGO_MAX_TERMS];
};

// One stage of the staged interpreter.  For RegP blocks the whole OrderBy is one
// gather of the stage's components followed by a row-major flatten.
struct DevStage {
  int32_t rank;
  int32_t n_blocks;
  int64_t dims[LEGO_MAX_RANK];   // stage dims, in index order
  int64_t pdims[LEGO_MAX_RANK];  // dims after the gather
  int8_t gperm[LEGO_MAX_RANK];   // gathered[i] = idx[gperm[i]]
  int8_t blk_start[LEGO_MAX_BLOCKS];
  int8_t blk_rank[LEGO_MAX_BLOCKS];
  int8_t blk_kind[LEGO_MAX_BLOCKS];
  const int64_t* lut_apply[LEGO_MAX_BLOCKS];  // device tables of LEGO_BLOCK_LUT blocks, else null
  const int64_t* lut_inv[LEGO_MAX_BLOCKS];
};

struct StagedProgram {
  int32_t rank;
  int32_t n_stages;
  int64_t dims[LEGO_MAX_RANK];
  DevStage stages[LEGO_MAX_STAGES];
};

// A folded digit of the logical flat id L: value = (L / pos) % radix, placed at
// `stride` in the layout's flat output.  `src`/`div` keep its origin.
struct Digit {
  int32_t src;
  int64_t div;
  int64_t mod;
  int64_t pos;     // suffix product of the logical dims times div
  int64_t stride;  // weight in the folded flat index
};

int32_t check_layout(const lego_layout_t* L, int64_t* size_out);
// Returns LEGO_OK and fills `digits` (most significant output digit first) when
// the layout folds; LEGO_ERR_UNSUPPORTED when only the staged form applies.
int32_t fold_layout(const lego_layout_t* L, std::vector<Digit>* digits);
int32_t build_staged(const lego_layout_t* L, StagedProgram* out);

// out[dst] += ((x[src] / a) % m) * b; m == 0: no wrap.
void set_term(DigitTerm* t, int src, int dst, int64_t a, int64_t m, int64_t b);

// Digit-sum programs over a folded layout.
void program_range(const std::vector<Digit>& dg, int64_t size, DigitProgram* p);   // L -> flat
void program_apply(const std::vector<Digit>& dg, int rank, int64_t size, DigitProgram* p);  // idx[] -> flat
void program_inv(const std::vector<Digit>& dg, int rank, int64_t size, DigitProgram* p);    // flat -> idx[]

// Common refinement of two folded layouts over the same logical domain: digits
// of L with a stride on the `a` side and one on the `b` side, least significant
// (in L) first, unmerged.  Returns false when the two digit sets do not nest.
struct PairDigit {
  int64_t pos;
  int64_t radix;
  int64_t sa;
  int64_t sb;
};
bool refine_pair(const std::vector<Digit>& a, const std::vector<Digit>& b, std::vector<PairDigit>* out);
// Fuse digits that behave as one in the map a-flat -> b-flat (sa and sb both
// continue the previous digit), whatever their position in L; result sorted by sa.
void merge_pairs(std::vector<PairDigit>* v);

}  // namespace lego
