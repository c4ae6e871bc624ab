// LayerNorm backward: dx per row, dgamma / dbeta by a deterministic two-stage
// column reduction.
//
// Stage one: persistent CTAs keep a row of x, dy in registers, compute dx, and
// accumulate dy * xhat and dy for their rows in registers; each CTA then writes
// one partial row.  Stage two sums the partial rows per column in a fixed order.
// The reference instead funnels rows into GROUP_SIZE_M buffers guarded by a spin
// lock (triton_generated/layernorm/layernorm.py:195-215); a fixed-order reduction
// needs no lock and gives the same bits on every run.
#include <cuda_fp16.h>

#include "common.cuh"
#include "rowwise.cuh"

namespace lego {
namespace {

constexpr int kMaxPartialRows = 592;  // 4 CTAs on each of 148 SMs

struct BwdParams {
  const __half* dy;
  const __half* x;
  const __half* gamma;
  const float* mean;
  const float* rstd;
  __half* dx;
  float* partial;  // [2][partial_rows][cols]
  int64_t rows;
  int32_t cols;
  int32_t partial_rows;
};

template <int TPR, int EPT, bool VECTOR>
__global__ void __launch_bounds__(TPR)
ln_bwd_dx_kernel(const __grid_constant__ BwdParams P) {
  __shared__ float slots[2][32];
  const int t = threadIdx.x;
  const int cols = P.cols;
  float acc_w[EPT], acc_b[EPT];
#pragma unroll
  for (int k = 0; k < EPT; ++k) acc_w[k] = acc_b[k] = 0.f;
  float g[EPT];
  load_row<__half, TPR, EPT, VECTOR>(P.gamma, cols, t, 0.f, g);

  for (int64_t row = blockIdx.x; row < P.rows; row += gridDim.x) {
    float xh[EPT], wdy[EPT];
    load_row<__half, TPR, EPT, VECTOR>(P.x + row * cols, cols, t, 0.f, xh);
    load_row<__half, TPR, EPT, VECTOR>(P.dy + row * cols, cols, t, 0.f, wdy);
    const float mean = P.mean[row], rstd = P.rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const bool in = col_of<__half, TPR, VECTOR>(k, t) < cols;
      const float h = in ? (xh[k] - mean) * rstd : 0.f;
      const float d = wdy[k];
      acc_w[k] = fmaf(d, h, acc_w[k]);
      acc_b[k] += d;
      xh[k] = h;
      wdy[k] = d * g[k];
      s1 = fmaf(h, wdy[k], s1);
      s2 += wdy[k];
    }
    s1 = row_reduce<TPR, false>(s1, slots[0]);
    s2 = row_reduce<TPR, false>(s2, slots[1]);
    const float c1 = s1 / (float)cols, c2 = s2 / (float)cols;
#pragma unroll
    for (int k = 0; k < EPT; ++k) xh[k] = (wdy[k] - fmaf(xh[k], c1, c2)) * rstd;
    store_row<__half, TPR, EPT, VECTOR>(P.dx + row * cols, cols, t, xh);
  }
  if ((int)blockIdx.x < P.partial_rows) {
    float* pw = P.partial + (size_t)blockIdx.x * cols;
    float* pb = P.partial + ((size_t)P.partial_rows + blockIdx.x) * cols;
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const int c = col_of<__half, TPR, VECTOR>(k, t);
      if (c < cols) {
        pw[c] = acc_w[k];
        pb[c] = acc_b[k];
      }
    }
  }
}

__global__ void __launch_bounds__(256)
ln_bwd_reduce_kernel(const float* __restrict__ partial, __half* __restrict__ dgamma, __half* __restrict__ dbeta,
                     int cols, int partial_rows) {
  // 32 columns x 8 row-lanes per CTA; each row-lane sums every 8th partial row.
  __shared__ float sw[8][33], sb[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float w = 0.f, b = 0.f;
  if (c < cols) {
    for (int r = ry; r < partial_rows; r += 8) {
      w += partial[(size_t)r * cols + c];
      b += partial[((size_t)partial_rows + r) * cols + c];
    }
  }
  sw[ry][cx] = w;
  sb[ry][cx] = b;
  __syncthreads();
  if (ry == 0 && c < cols) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      tw += sw[r][cx];
      tb += sb[r][cx];
    }
    dgamma[c] = __float2half_rn(tw);
    dbeta[c] = __float2half_rn(tb);
  }
}

template <int TPR, int EPT, bool VECTOR>
int32_t launch_dx(const BwdParams& P, cudaStream_t s) {
  ln_bwd_dx_kernel<TPR, EPT, VECTOR><<<P.partial_rows, TPR, 0, s>>>(P);
  return cuda_status(cudaGetLastError());
}

template <bool VECTOR>
int32_t launch_dx_by_cols(const BwdParams& P, cudaStream_t s) {
  if (P.cols <= 256 * 8) return launch_dx<256, 8, VECTOR>(P, s);
  if (P.cols <= 256 * 32) return launch_dx<256, 32, VECTOR>(P, s);
  if (P.cols <= 1024 * 32) return launch_dx<1024, 32, VECTOR>(P, s);
  return LEGO_ERR_UNSUPPORTED;
}

int64_t partial_rows_for(int64_t rows) { return rows < kMaxPartialRows ? rows : kMaxPartialRows; }

}  // namespace
}  // namespace lego

using namespace lego;

extern "C" {

int64_t lego_layernorm_bwd_partial_rows(int64_t rows, int64_t cols) {
  (void)cols;
  return rows < 1 ? 0 : partial_rows_for(rows);
}

int32_t lego_layernorm_bwd_f16(const void* dy, const void* x, const void* gamma, const float* mean,
                               const float* rstd, void* dx, void* dgamma, void* dbeta,
                               float* partial, int64_t rows, int64_t cols, void* stream) {
  if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || !partial) return LEGO_ERR_NULL;
  if (rows < 1 || cols < 1) return LEGO_ERR_SIZE;
  if (cols > 1024 * 32) return LEGO_ERR_UNSUPPORTED;
  BwdParams P{};
  P.dy = (const __half*)dy; P.x = (const __half*)x; P.gamma = (const __half*)gamma;
  P.mean = mean; P.rstd = rstd; P.dx = (__half*)dx; P.partial = partial;
  P.rows = rows; P.cols = (int32_t)cols; P.partial_rows = (int32_t)partial_rows_for(rows);
  cudaStream_t s = (cudaStream_t)stream;
  auto a16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = cols % 8 == 0 && a16(dy) && a16(x) && a16(gamma) && a16(dx);
  int32_t st = vec ? launch_dx_by_cols<true>(P, s) : launch_dx_by_cols<false>(P, s);
  if (st != LEGO_OK) return st;
  ln_bwd_reduce_kernel<<<(unsigned)((cols + 31) / 32), 256, 0, s>>>(partial, (__half*)dgamma, (__half*)dbeta,
                                                                 (int)cols, P.partial_rows);
  return cuda_status(cudaGetLastError());
}

}  // extern "C"
