// Host-side creation of TMA tensor maps through the driver entry point, so the
// library does not link against libcuda.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"

namespace lego {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn(int32_t* err) {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  static int32_t status = LEGO_OK;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess) { (void)cudaGetLastError(); status = cuda_status(e); return; }
    if (q != cudaDriverEntryPointSuccess || !p) { status = LEGO_ERR_UNSUPPORTED; return; }
    fn = (EncodeFn)p;
  });
  if (err) *err = status;
  return fn;
}

// 2-D map, 128-byte swizzle: `inner` contiguous elements per row, `outer` rows,
// rows `pitch_bytes` apart; the box is box_inner x box_outer elements.
inline int32_t make_tmap_2d(EncodeFn enc, CUtensorMap* out, CUtensorMapDataType dt, const void* base,
                            uint64_t inner, uint64_t outer, uint64_t pitch_bytes, uint32_t box_inner,
                            uint32_t box_outer) {
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LEGO_OK : LEGO_ERR_UNSUPPORTED;
}

// 3-D map, 128-byte swizzle, over a row-major matrix whose rows are taken `group`
// apart: coordinate (x, k, g) is element x of row g * group + k.  A box
// {box_inner, 1, box_groups} therefore gathers rows k, k + group, k + 2 group, ...
inline int32_t make_tmap_row_groups(EncodeFn enc, CUtensorMap* out, CUtensorMapDataType dt, const void* base,
                                    uint64_t inner, uint64_t rows, uint64_t pitch_bytes, uint32_t group,
                                    uint32_t box_inner, uint32_t box_groups) {
  const cuuint64_t dims[3] = {inner, group, rows / group};
  const cuuint64_t strides[2] = {pitch_bytes, pitch_bytes * group};
  const cuuint32_t box[3] = {box_inner, 1, box_groups};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  const CUresult r = enc(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LEGO_OK : LEGO_ERR_UNSUPPORTED;
}

// The same rows seen as (x, g, k): the group index before the row-in-group index, so that
// one box {box_inner, box_groups, group} lands in shared memory as `group` blocks of
// box_groups rows each: block k holds rows k, k + group, k + 2 group, ...  The stride of
// the last dimension (one row) is smaller than that of the middle one (one group); the
// driver may refuse such a map, in which case the caller gathers with one load per k.
inline int32_t make_tmap_group_major(EncodeFn enc, CUtensorMap* out, CUtensorMapDataType dt, const void* base,
                                     uint64_t inner, uint64_t rows, uint64_t pitch_bytes, uint32_t group,
                                     uint32_t box_inner, uint32_t box_groups) {
  const cuuint64_t dims[3] = {inner, rows / group, group};
  const cuuint64_t strides[2] = {pitch_bytes * group, pitch_bytes};
  const cuuint32_t box[3] = {box_inner, box_groups, group};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LEGO_OK : LEGO_ERR_UNSUPPORTED;
}

}  // namespace lego
