// Row-wise softmax and LayerNorm forward: one pass over HBM per row.
//
// A row lives in registers (up to 32 fp32 values per thread) spread over a warp,
// a 256-thread CTA or a 1024-thread CTA depending on its length, so each element
// is read once and written once.  Reductions are warp shuffles plus one shared-
// memory hop.  CTAs are persistent: work item w (a logical id of the row map)
// belongs to CTA w mod grid, and row_map.apply(w) names the row it processes.
#include <cuda_fp16.h>

#include "common.cuh"
#include "rowwise.cuh"

namespace lego {
namespace {

enum { OP_SOFTMAX = 0, OP_LAYERNORM = 1 };

struct RowParams {
  const void* x;
  void* y;
  const void* gamma;
  const void* beta;
  float* mean;
  float* rstd;
  int64_t rows;
  int32_t cols;
  float eps;
  int32_t has_map;
  DigitProgram map;  // logical id -> row
};

__device__ __forceinline__ uint64_t map_eval(const DigitProgram& p, uint64_t x) {
  uint64_t acc = 0;
  for (int j = 0; j < p.n_terms; ++j) {
    const DigitTerm& t = p.t[j];
    if (p.wide) {
      uint64_t q = t.a64 > 1 ? x / t.a64 : x;
      if (t.m64) q %= t.m64;
      acc += q * t.b;
    } else {
      uint32_t q = fd_div((uint32_t)x, t.a);
      if (t.m.d) q -= fd_div(q, t.m) * t.m.d;
      acc += (uint64_t)q * t.b;
    }
  }
  return acc;
}

// ---- the kernel ---------------------------------------------------------------------

template <int OP, typename T, int TPR, int EPT, bool VECTOR>
__global__ void __launch_bounds__(TPR < 256 ? 256 : TPR)
row_kernel(const __grid_constant__ RowParams P) {
  constexpr int BLOCK = TPR < 256 ? 256 : TPR;
  constexpr int RPC = BLOCK / TPR;  // rows in flight per CTA
  __shared__ float slots[3][32];
  const int t = threadIdx.x % TPR;
  const int sub = threadIdx.x / TPR;
  const int cols = P.cols;
  const T* __restrict__ x = reinterpret_cast<const T*>(P.x);
  T* __restrict__ y = reinterpret_cast<T*>(P.y);
  const int64_t n_groups = (P.rows + RPC - 1) / RPC;

  for (int64_t grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
    const int64_t w = grp * RPC + sub;
    const bool live = w < P.rows;
    int64_t row = w;
    if (live && P.has_map) row = (int64_t)map_eval(P.map, (uint64_t)w);
    float v[EPT];
    if (OP == OP_SOFTMAX) {
      if (live) load_row<T, TPR, EPT, VECTOR>(x + row * cols, cols, t, -INFINITY, v);
      else {
#pragma unroll
        for (int k = 0; k < EPT; ++k) v[k] = -INFINITY;
      }
      float m = v[0];
#pragma unroll
      for (int k = 1; k < EPT; ++k) m = fmaxf(m, v[k]);
      m = row_reduce<TPR, true>(m, slots[0]);
      const float ms = m * 1.4426950408889634f;
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        v[k] = exp2f(fmaf(v[k], 1.4426950408889634f, -ms));
        s += v[k];
      }
      s = row_reduce<TPR, false>(s, slots[1]);
      const float inv = 1.0f / s;
#pragma unroll
      for (int k = 0; k < EPT; ++k) v[k] *= inv;
      if (live) store_row<T, TPR, EPT, VECTOR>(y + row * cols, cols, t, v);
    } else {
      if (live) load_row<T, TPR, EPT, VECTOR>(x + row * cols, cols, t, 0.f, v);
      else {
#pragma unroll
        for (int k = 0; k < EPT; ++k) v[k] = 0.f;
      }
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < EPT; ++k) s += v[k];
      s = row_reduce<TPR, false>(s, slots[0]);
      const float mean = s / (float)cols;
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        const float d = col_of<T, TPR, VECTOR>(k, t) < cols ? v[k] - mean : 0.f;
        v[k] = d;
        q = fmaf(d, d, q);
      }
      q = row_reduce<TPR, false>(q, slots[1]);
      const float rstd = 1.0f / sqrtf(q / (float)cols + P.eps);
      if (live && t == 0) {
        P.mean[row] = mean;
        P.rstd[row] = rstd;
      }
      // gamma / beta are the same for every row: default-cached loads keep them in L1
      const T* __restrict__ gam = reinterpret_cast<const T*>(P.gamma);
      const T* __restrict__ bet = reinterpret_cast<const T*>(P.beta);
      T* __restrict__ yrow = y + row * cols;
      if (VECTOR) {
        constexpr int VEC = Elem<T>::VEC;
#pragma unroll
        for (int k = 0; k < EPT / VEC; ++k) {
          const int c = (k * TPR + t) * VEC;
          if (c < cols) {
            float g[VEC], b[VEC];
            Elem<T>::unpack(__ldg(reinterpret_cast<const uint4*>(gam + c)), g);
            Elem<T>::unpack(__ldg(reinterpret_cast<const uint4*>(bet + c)), b);
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[k * VEC + e] = fmaf(v[k * VEC + e] * rstd, g[e], b[e]);
            if (live) __stcs(reinterpret_cast<uint4*>(yrow + c), Elem<T>::pack(v + k * VEC));
          }
        }
      } else {
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
          const int c = k * TPR + t;
          if (c < cols && live)
            yrow[c] = Elem<T>::from_float(fmaf(v[k] * rstd, Elem<T>::to_float(gam[c]), Elem<T>::to_float(bet[c])));
        }
      }
    }
  }
}

template <int OP, typename T, int TPR, int EPT, bool VECTOR>
int32_t launch_cfg(const RowParams& P, DeviceCtx* ctx, cudaStream_t s) {
  constexpr int BLOCK = TPR < 256 ? 256 : TPR;
  constexpr int RPC = BLOCK / TPR;
  auto kern = row_kernel<OP, T, TPR, EPT, VECTOR>;
  int per_sm = 0;
  LEGO_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, BLOCK, 0));
  if (per_sm < 1) per_sm = 1;
  const int64_t groups = (P.rows + RPC - 1) / RPC;
  int64_t grid = (int64_t)ctx->sm_count * per_sm;
  if (grid > groups) grid = groups;
  kern<<<(unsigned)grid, BLOCK, 0, s>>>(P);
  return cuda_status(cudaGetLastError());
}

template <int OP, typename T, bool VECTOR>
int32_t launch_vec(const RowParams& P, DeviceCtx* ctx, cudaStream_t s) {
  const int c = P.cols;
  if (c <= 32 * 8) return launch_cfg<OP, T, 32, 8, VECTOR>(P, ctx, s);
  if (c <= 32 * 32) return launch_cfg<OP, T, 32, 32, VECTOR>(P, ctx, s);
  if (c <= 256 * 8) return launch_cfg<OP, T, 256, 8, VECTOR>(P, ctx, s);
  if (c <= 256 * 16) return launch_cfg<OP, T, 256, 16, VECTOR>(P, ctx, s);
  if (c <= 256 * 32) return launch_cfg<OP, T, 256, 32, VECTOR>(P, ctx, s);
  if (c <= 1024 * 32) return launch_cfg<OP, T, 1024, 32, VECTOR>(P, ctx, s);
  return LEGO_ERR_UNSUPPORTED;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <int OP, typename T>
int32_t run_rows(RowParams& P, const lego_layout_t* row_map, void* stream) {
  if (P.rows < 0 || P.cols < 1) return LEGO_ERR_SIZE;
  if (P.rows > 0 && (!P.x || !P.y)) return LEGO_ERR_NULL;  // empty buffers may be NULL
  if (P.rows > 0 && OP == OP_LAYERNORM && (!P.gamma || !P.beta || !P.mean || !P.rstd)) return LEGO_ERR_NULL;
  if (((uintptr_t)P.x % sizeof(T)) || ((uintptr_t)P.y % sizeof(T))) return LEGO_ERR_ALIGN;
  P.has_map = 0;
  if (row_map) {
    int64_t size = 0;
    int32_t st = check_layout(row_map, &size);
    if (st != LEGO_OK) return st;
    if (size != P.rows) return LEGO_ERR_DOMAIN;
    std::vector<Digit> dg;
    st = fold_layout(row_map, &dg);
    if (st == LEGO_ERR_UNSUPPORTED) return LEGO_ERR_UNSUPPORTED;  // row maps must fold to digit strides
    if (st != LEGO_OK) return st;
    program_range(dg, size, &P.map);
    // an identity map needs no evaluation
    P.has_map = !(P.map.n_terms == 1 && P.map.t[0].a64 == 1 && P.map.t[0].b == 1 && P.map.t[0].m64 == 0);
    if (size <= 1) P.has_map = 0;
  }
  if (P.rows == 0) return LEGO_OK;
  int32_t err = LEGO_OK;
  DeviceCtx* ctx = device_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = (cudaStream_t)stream;
  constexpr int VEC = Elem<T>::VEC;
  bool vec = (P.cols % VEC == 0) && aligned16(P.x) && aligned16(P.y);
  if (OP == OP_LAYERNORM) vec = vec && aligned16(P.gamma) && aligned16(P.beta);
  return vec ? launch_vec<OP, T, true>(P, ctx, s) : launch_vec<OP, T, false>(P, ctx, s);
}

}  // namespace
}  // namespace lego

using namespace lego;

extern "C" {

int32_t lego_softmax_f16(const void* x, void* y, int64_t rows, int64_t cols,
                         const lego_layout_t* row_map, void* stream) {
  if (cols > 0x7fffffff) return LEGO_ERR_UNSUPPORTED;
  RowParams P{};
  P.x = x; P.y = y; P.rows = rows; P.cols = (int32_t)cols;
  return run_rows<OP_SOFTMAX, __half>(P, row_map, stream);
}

int32_t lego_softmax_f32(const void* x, void* y, int64_t rows, int64_t cols,
                         const lego_layout_t* row_map, void* stream) {
  if (cols > 0x7fffffff) return LEGO_ERR_UNSUPPORTED;
  RowParams P{};
  P.x = x; P.y = y; P.rows = rows; P.cols = (int32_t)cols;
  return run_rows<OP_SOFTMAX, float>(P, row_map, stream);
}

int32_t lego_layernorm_fwd_f16(const void* x, const void* gamma, const void* beta, void* y,
                               float* mean, float* rstd, int64_t rows, int64_t cols, float eps,
                               const lego_layout_t* row_map, void* stream) {
  if (cols > 0x7fffffff) return LEGO_ERR_UNSUPPORTED;
  RowParams P{};
  P.x = x; P.y = y; P.gamma = gamma; P.beta = beta; P.mean = mean; P.rstd = rstd;
  P.rows = rows; P.cols = (int32_t)cols; P.eps = eps;
  return run_rows<OP_LAYERNORM, __half>(P, row_map, stream);
}

}  // extern "C"
