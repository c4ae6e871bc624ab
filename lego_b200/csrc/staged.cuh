// Staged interpreter: evaluates any layout by walking its stages, re-cutting and
// permuting the flat id in 64-bit arithmetic as lego/lego.py:388-433 does.
#pragma once

#include "common.cuh"

namespace lego {

// ---- staged interpreter --------------------------------------------------------

__device__ __forceinline__ int64_t antidiag_apply(int64_t n, int64_t i, int64_t j) {
  const int64_t k = i + j + 1;
  if (k <= n) return k * (k - 1) / 2 + i;
  const int64_t m = 2 * n - k;
  return n * n - n + i - m * (m - 1) / 2;
}

__device__ __forceinline__ void antidiag_inv(int64_t n, int64_t f, int64_t* i, int64_t* j) {
  // Diagonal k (= i + j + 1) holding flat id f, found from a floating-point
  // guess corrected by exact integer comparisons.
  const int64_t tri = n * (n + 1) / 2;
  int64_t k;
  if (f < tri) {
    k = (int64_t)((sqrt(8.0 * (double)f + 1.0) - 1.0) * 0.5) + 1;
    while (k > 1 && k * (k - 1) / 2 > f) --k;
    while ((k + 1) * k / 2 <= f) ++k;
    *i = f - k * (k - 1) / 2;
  } else {
    const int64_t g = n * n - 1 - f;  // mirrored id counts from the far corner
    int64_t kk = (int64_t)((sqrt(8.0 * (double)g + 1.0) - 1.0) * 0.5) + 1;
    while (kk > 1 && kk * (kk - 1) / 2 > g) --kk;
    while ((kk + 1) * kk / 2 <= g) ++kk;
    const int64_t im = g - kk * (kk - 1) / 2;  // mirrored i
    *i = n - 1 - im;
    k = 2 * n - kk;
    *j = k - 1 - *i;
    return;
  }
  *j = k - 1 - *i;
}

__device__ inline int64_t staged_apply(const StagedProgram& sp, int64_t flat) {
  for (int s = sp.n_stages - 1; s >= 0; --s) {
    const DevStage& st = sp.stages[s];
    int64_t idx[LEGO_MAX_RANK];
    for (int k = st.rank - 1; k > 0; --k) {
      idx[k] = flat % st.dims[k];
      flat /= st.dims[k];
    }
    idx[0] = flat;
    int64_t acc = 0;
    for (int b = 0; b < st.n_blocks; ++b) {
      const int at = st.blk_start[b];
      if (st.blk_kind[b] == LEGO_BLOCK_REGP) {
        for (int i = 0; i < st.blk_rank[b]; ++i) acc = acc * st.pdims[at + i] + idx[st.gperm[at + i]];
      } else if (st.blk_kind[b] == LEGO_BLOCK_ANTIDIAG) {
        acc = acc * (st.dims[at] * st.dims[at]) + antidiag_apply(st.dims[at], idx[at], idx[at + 1]);
      } else if (st.blk_kind[b] == LEGO_BLOCK_LUT) {
        int64_t r = 0, bsz = 1;
        for (int i = 0; i < st.blk_rank[b]; ++i) {
          r = r * st.dims[at + i] + idx[at + i];
          bsz *= st.dims[at + i];
        }
        acc = acc * bsz + __ldg(st.lut_apply[b] + r);
      } else {
        acc = acc * (st.dims[at] * st.dims[at + 1]) +
              ((st.dims[at] - 1 - idx[at]) * st.dims[at + 1] + st.dims[at + 1] - 1 - idx[at + 1]);
      }
    }
    flat = acc;
  }
  return flat;
}

__device__ inline int64_t staged_inv(const StagedProgram& sp, int64_t flat) {
  for (int s = 0; s < sp.n_stages; ++s) {
    const DevStage& st = sp.stages[s];
    int64_t idx[LEGO_MAX_RANK];
    for (int b = st.n_blocks - 1; b >= 0; --b) {
      const int at = st.blk_start[b];
      const int r = st.blk_rank[b];
      int64_t bsz = 1;
      for (int i = 0; i < r; ++i) bsz *= st.dims[at + i];
      int64_t v = flat % bsz;  // OrderBy.inv peels every block with %, lego/lego.py:341
      flat /= bsz;
      if (st.blk_kind[b] == LEGO_BLOCK_REGP) {
        for (int i = r - 1; i > 0; --i) {
          idx[st.gperm[at + i]] = v % st.pdims[at + i];
          v /= st.pdims[at + i];
        }
        idx[st.gperm[at]] = v;
      } else {
        if (st.blk_kind[b] == LEGO_BLOCK_ANTIDIAG) {
          antidiag_inv(st.dims[at], v, &idx[at], &idx[at + 1]);
        } else if (st.blk_kind[b] == LEGO_BLOCK_LUT) {
          int64_t w = __ldg(st.lut_inv[b] + v);
          for (int i = r - 1; i > 0; --i) {
            idx[at + i] = w % st.dims[at + i];
            w /= st.dims[at + i];
          }
          idx[at] = w;
        } else {
          const int64_t w = bsz - 1 - v;
          idx[at] = w / st.dims[at + 1];
          idx[at + 1] = w % st.dims[at + 1];
        }
      }
    }
    int64_t acc = 0;
    for (int k = 0; k < st.rank; ++k) acc = acc * st.dims[k] + idx[k];
    flat = acc;
  }
  return flat;
}

}  // namespace lego
