// Housekeeping entry points of the C ABI: per-device workspace, status words,
// and the host-only layout services.
#include <mutex>
#include <vector>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace lego {

int32_t static_status_take(cudaStream_t s, uint32_t* word);  // gemm_sm100.cu

namespace {
std::mutex g_mu;
std::vector<DeviceCtx*> g_ctx;  // indexed by device ordinal
}  // namespace

DeviceCtx* device_ctx(int32_t* err) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    if (err) *err = cuda_status(e);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if ((int)g_ctx.size() <= dev) g_ctx.resize(dev + 1, nullptr);
  if (g_ctx[dev]) return g_ctx[dev];
  DeviceCtx* c = new DeviceCtx();
  c->device = dev;
  e = cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&c->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (e == cudaSuccess) e = cudaMalloc(&c->status_word, 256);
  if (e == cudaSuccess) e = cudaMemset(c->status_word, 0, 256);
  c->tmap_table_bytes = (size_t)LEGO_MAX_GROUPS * 640;  // one 640-byte problem record per group
  if (e == cudaSuccess) e = cudaMalloc(&c->tmap_table, c->tmap_table_bytes);
  if (e != cudaSuccess) {
    if (err) *err = cuda_status(e);
    if (c->status_word) cudaFree(c->status_word);
    delete c;
    return nullptr;
  }
  g_ctx[dev] = c;
  return c;
}

DeviceCtx* device_ctx_if_any() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  return dev < (int)g_ctx.size() ? g_ctx[dev] : nullptr;
}

namespace {
// The give-up path of a bounded wait, run for real: one CTA initialises an mbarrier that
// nothing ever arrives on, waits on it with the same helper the kernels use, and on expiry
// records its code in the status word exactly as they do.  It neither faults nor hangs;
// the context stays usable.
__global__ void bounded_wait_selftest_kernel(long long limit_cycles, uint32_t* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_barrier_init();
    if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bar), 0, &abort_flag, limit_cycles))
      atomicCAS(status, 0u, 0x7e570000u);
  }
}
}  // namespace

void release_all_ctx() {
  std::lock_guard<std::mutex> lock(g_mu);
  int cur = 0;
  const bool have_cur = cudaGetDevice(&cur) == cudaSuccess;
  for (DeviceCtx* c : g_ctx) {
    if (!c) continue;
    if (cudaSetDevice(c->device) == cudaSuccess) {
      cudaFree(c->status_word);
      cudaFree(c->tmap_table);
    }
    delete c;
  }
  g_ctx.clear();
  if (have_cur) cudaSetDevice(cur);
}

}  // namespace lego

using namespace lego;

extern "C" {

int32_t lego_layout_check(const lego_layout_t* layout) { return check_layout(layout, nullptr); }

int32_t lego_layout_fold(const lego_layout_t* layout, lego_folded_t* out) {
  if (!layout || !out) return LEGO_ERR_NULL;
  int64_t size = 0;
  int32_t st = check_layout(layout, &size);
  if (st != LEGO_OK) return st;
  out->size = size;
  out->n_terms = 0;
  out->foldable = 0;
  std::vector<Digit> dg;
  st = fold_layout(layout, &dg);
  if (st == LEGO_ERR_UNSUPPORTED) return LEGO_OK;  // valid layout, staged form only
  if (st != LEGO_OK) return st;
  out->foldable = 1;
  out->n_terms = (int32_t)dg.size();
  for (size_t j = 0; j < dg.size(); ++j) {
    out->terms[j].src = dg[j].src;
    out->terms[j].reserved = 0;
    out->terms[j].div = dg[j].div;
    out->terms[j].mod = dg[j].mod;
    out->terms[j].stride = dg[j].stride;
  }
  return LEGO_OK;
}

int32_t lego_device_status(void* stream, uint32_t* detail) {
  // Reads what exists and creates nothing: a process that only ever used the non-allocating
  // entry point must not get a workspace allocated by asking for its status.
  cudaStream_t s = (cudaStream_t)stream;
  uint32_t word = 0;
  if (DeviceCtx* c = device_ctx_if_any()) {
    LEGO_CUDA_TRY(cudaMemcpyAsync(&word, c->status_word, sizeof(word), cudaMemcpyDeviceToHost, s));
    LEGO_CUDA_TRY(cudaStreamSynchronize(s));
    if (word) {
      LEGO_CUDA_TRY(cudaMemsetAsync(c->status_word, 0, sizeof(word), s));
      LEGO_CUDA_TRY(cudaStreamSynchronize(s));
    }
  } else {
    LEGO_CUDA_TRY(cudaStreamSynchronize(s));
  }
  uint32_t static_word = 0;
  const int32_t st = static_status_take(s, &static_word);
  if (st != LEGO_OK) return st;
  if (!word) word = static_word;
  if (detail) *detail = word;
  return word ? (int32_t)LEGO_ERR_DEVICE_TIMEOUT : (int32_t)LEGO_OK;
}

int32_t lego_copy_2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t width_bytes,
                     int64_t height, void* stream) {
  if (!dst || !src) return LEGO_ERR_NULL;
  if (width_bytes < 0 || height < 0 || dst_pitch < width_bytes || src_pitch < width_bytes) return LEGO_ERR_SIZE;
  if (width_bytes == 0 || height == 0) return LEGO_OK;
  LEGO_CUDA_TRY(cudaMemcpy2DAsync(dst, (size_t)dst_pitch, src, (size_t)src_pitch, (size_t)width_bytes, (size_t)height,
                                  cudaMemcpyDefault, (cudaStream_t)stream));
  return LEGO_OK;
}

int32_t lego_selftest_bounded_wait(int64_t limit_cycles, void* stream) {
  if (limit_cycles < 1 || limit_cycles > 2000000000LL) return LEGO_ERR_SIZE;
  int32_t err = LEGO_OK;
  DeviceCtx* c = device_ctx(&err);
  if (!c) return err;
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((long long)limit_cycles, c->status_word);
  return cuda_status(cudaGetLastError());
}

const char* lego_status_string(int32_t status) {
  switch (status) {
    case LEGO_OK: return "ok";
    case LEGO_ERR_NULL: return "a required pointer is NULL";
    case LEGO_ERR_RANK: return "rank or count outside the supported limits, or mismatched";
    case LEGO_ERR_PERM: return "perm is not a permutation";
    case LEGO_ERR_DIM: return "a dimension is smaller than 1 or invalid for the block kind";
    case LEGO_ERR_NOT_BIJECTIVE: return "a stage does not cover the logical index space exactly (layout is not a bijection)";
    case LEGO_ERR_SIZE: return "sizes are inconsistent with the operation";
    case LEGO_ERR_ALIGN: return "pointer or leading dimension is not aligned as required";
    case LEGO_ERR_UNSUPPORTED: return "valid request this build has no kernel for";
    case LEGO_ERR_DOMAIN: return "layouts disagree on the logical domain";
    case LEGO_ERR_OVERFLOW: return "index space does not fit in 63 bits";
    case LEGO_ERR_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    default: break;
  }
  if (status >= LEGO_ERR_CUDA_BASE && status < LEGO_ERR_DEVICE_TIMEOUT)
    return cudaGetErrorString((cudaError_t)(status - LEGO_ERR_CUDA_BASE));
  return "unknown status";
}

int32_t lego_shutdown(void) {
  release_all_ctx();
  return LEGO_OK;
}

}  // extern "C"
