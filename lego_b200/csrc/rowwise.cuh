// Register-resident row helpers shared by the row-wise kernels: a row of up to
// 32 values per thread spread over TPR threads, vector or scalar loads/stores,
// and reductions over the threads of a row.
#pragma once

#include <cuda_fp16.h>

#include "common.cuh"

namespace lego {

// ---- loads / stores of EPT elements per thread -----------------------------------

template <typename T> struct Elem;
template <> struct Elem<__half> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(h[i]);
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return r;
  }
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct Elem<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x);
    f[1] = __uint_as_float(r.y);
    f[2] = __uint_as_float(r.z);
    f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                      __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ float to_float(float v) { return v; }
  static __device__ __forceinline__ float from_float(float v) { return v; }
};

template <typename T, int TPR, int EPT, bool VECTOR>
__device__ __forceinline__ void load_row(const T* __restrict__ row, int cols, int t, float fill, float* v) {
  if (VECTOR) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int NV = EPT / VEC;
    uint4 raw[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * TPR + t) * VEC;
      if (c < cols) raw[k] = __ldcs(reinterpret_cast<const uint4*>(row + c));
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * TPR + t) * VEC;
      if (c < cols) {
        Elem<T>::unpack(raw[k], v + k * VEC);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[k * VEC + e] = fill;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const int c = k * TPR + t;
      v[k] = c < cols ? Elem<T>::to_float(row[c]) : fill;
    }
  }
}

template <typename T, int TPR, int EPT, bool VECTOR>
__device__ __forceinline__ void store_row(T* __restrict__ row, int cols, int t, const float* v) {
  if (VECTOR) {
    constexpr int VEC = Elem<T>::VEC;
    constexpr int NV = EPT / VEC;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * TPR + t) * VEC;
      if (c < cols) __stcs(reinterpret_cast<uint4*>(row + c), Elem<T>::pack(v + k * VEC));
    }
  } else {
#pragma unroll
    for (int k = 0; k < EPT; ++k) {
      const int c = k * TPR + t;
      if (c < cols) row[c] = Elem<T>::from_float(v[k]);
    }
  }
}

// column of register slot k of thread t
template <typename T, int TPR, bool VECTOR>
__device__ __forceinline__ int col_of(int k, int t) {
  if (VECTOR) {
    constexpr int VEC = Elem<T>::VEC;
    return ((k / VEC) * TPR + t) * VEC + (k % VEC);
  }
  return k * TPR + t;
}

// ---- reductions over the TPR threads of a row -------------------------------------

template <bool IS_MAX>
__device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, w) : v + w;
  }
  return v;
}

// BAR == 0 synchronises the whole CTA; BAR > 0 uses that named barrier over TPR threads
// (for kernels whose CTA has extra warps that do not take part).
template <int TPR, bool IS_MAX, int BAR = 0>
__device__ __forceinline__ float row_reduce(float v, float* slots) {
  v = warp_reduce<IS_MAX>(v);
  if (TPR == 32) return v;
  constexpr int NW = TPR / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) slots[warp] = v;
  if (BAR == 0) __syncthreads();
  else asm volatile("bar.sync %0, %1;" ::"n"(BAR), "n"(TPR) : "memory");
  if (NW <= 8) {
    float r = slots[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) r = IS_MAX ? fmaxf(r, slots[w]) : r + slots[w];
    return r;
  }
  float r = lane < NW ? slots[lane] : (IS_MAX ? -INFINITY : 0.f);
  return warp_reduce<IS_MAX>(r);
}

}  // namespace lego
