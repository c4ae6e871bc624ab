// Row-wise softmax and LayerNorm forward: one pass over HBM per row.
//
// A row lives in registers (up to 32 fp32 values per thread) spread over a warp,
// a 256-thread CTA or a 1024-thread CTA depending on its length, so each element
// is read once and written once.  Reductions are warp shuffles plus one shared-
// memory hop.  CTAs are persistent: work item w (a logical id of the row map)
// belongs to CTA w mod grid, and row_map.apply(w) names the row it processes.
#include <cuda_fp16.h>

#include "common.cuh"
#include "ptx_sm100.cuh"
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


// ---- bulk-copy pipelined kernel ------------------------------------------------------
//
// For rows of at least 2 KiB (softmax: 4 KiB) whose bytes are a multiple of 16.  One CTA per SM: a producer
// warp streams whole rows into a shared-memory ring with 1-D bulk copies (cp.async.bulk,
// completion on mbarriers; lane l owns ring slot l and the lanes work in lock step, so the
// per-row latencies of barrier polls and copy issue overlap); several groups of consumer
// threads each take every groups-th row: pull it into registers with 128-bit
// shared-memory loads (32 values per thread, so a group has cols / 32 threads: 32 .. 512),
// free the slot at once, reduce within the group (named barrier) and write the result
// with 128-bit streaming stores.  One CTA with several consumer groups instead of several
// CTAs per SM because the memory system prefers few row streams per SM: a plain copy
// through this ring ran at 0.955 of the copy peak with one CTA per SM, 0.915 with two and
// 0.89 with three.  The row a slot holds is named by the producer next to the data.
// gamma / beta of LayerNorm are staged in shared memory once per CTA.

constexpr int kRing = 32;         // most ring slots a CTA may use (one producer lane each)
constexpr int kRingEpt = 32;      // values per consumer thread
constexpr int kMaxGroups = 15;    // named barriers 1 .. 15
constexpr int kMaxConsumers = 768;
constexpr long long kWaitLimit = 2000000000LL;  // SM cycles, about a second

struct RingCtl {
  uint64_t full[kRing];
  uint64_t empty[kRing];
  int64_t row[kRing];
  uint32_t abort_flag;               // any role gave up: polled inside every bounded wait
  uint32_t group_abort[kMaxGroups];  // written only by the group's own threads, read after its barrier
};

// Reduction over the `gsize` threads (nw warps) of one consumer group (named barrier `bar`).
// `slots` holds 16 partials; entries of warps the group does not have were set to the
// operation's identity once, so the fold is a fixed tree over two or four 128-bit loads
// whatever the group size.
template <bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float* slots, int bar, int gsize, int nw, int warp_in_group) {
  v = warp_reduce<IS_MAX>(v);
  if (nw == 1) return v;
  if ((threadIdx.x & 31) == 0) slots[warp_in_group] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(gsize) : "memory");
  const float4* q = reinterpret_cast<const float4*>(slots);
  const float4 a = q[0], b = q[1];
  float r;
  if (IS_MAX) r = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
  else r = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
  if (nw > 8) {
    const float4 c = q[2], d = q[3];
    if (IS_MAX) r = fmaxf(r, fmaxf(fmaxf(fmaxf(c.x, c.y), fmaxf(c.z, c.w)), fmaxf(fmaxf(d.x, d.y), fmaxf(d.z, d.w))));
    else r += ((c.x + c.y) + (c.z + c.w)) + ((d.x + d.y) + (d.z + d.w));
  }
  return r;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// G: threads per consumer group when it is one of the common sizes (constants for the
// address arithmetic and the barrier), 0 = taken from `gsize_rt`.
// EPT: values per consumer thread, 32, or 64 for rows beyond 8 Ki values so that such a row is
// still handled by a group of 256 and a CTA keeps two rows in flight.
template <int OP, typename T, int G, int EPT = kRingEpt>
__global__ void __launch_bounds__(EPT > kRingEpt ? 512 + 32 : kMaxConsumers + 32, 1)
row_ring_kernel(const __grid_constant__ RowParams P, int stages, int groups, int gsize_rt, uint32_t* status) {
  const int gsize = G > 0 ? G : gsize_rt;
  constexpr int VEC = Elem<T>::VEC;
  constexpr int NV = EPT / VEC;
  extern __shared__ __align__(128) uint8_t ring_smem[];
  const int cols = P.cols;
  const uint32_t row_bytes = (uint32_t)cols * sizeof(T);
  const uint32_t slot_bytes = (row_bytes + 127u) & ~127u;
  uint8_t* params_smem = ring_smem + (size_t)stages * slot_bytes;  // gamma | beta (LayerNorm)
  RingCtl* ctl = reinterpret_cast<RingCtl*>(params_smem + (OP == OP_LAYERNORM ? 2 * slot_bytes : 0));
  __shared__ __align__(16) float slots_all[kMaxGroups][2][16];
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  const int tid = threadIdx.x;
  const int n_consumers = groups * gsize;
  const int nw = gsize >> 5;  // warps per group
  const int64_t my_rows = P.rows > blockIdx.x ? (P.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), nw);
    }
    ctl->abort_flag = 0;
    for (int g = 0; g < kMaxGroups; ++g) ctl->group_abort[g] = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  // partials of warps a group does not have: the identity of the reduction that uses the array
  for (int i = tid; i < kMaxGroups * 2 * 16; i += blockDim.x)
    (&slots_all[0][0][0])[i] = (OP == OP_SOFTMAX && ((i >> 4) & 1) == 0) ? -INFINITY : 0.f;
  // The next grid of the stream may set itself up now; global memory is touched only once
  // the previous grid is complete (programmatic dependent launch).
  ptx::launch_dependents();
  ptx::grid_dependency_wait();
  if (OP == OP_LAYERNORM) {
    const uint4* g = reinterpret_cast<const uint4*>(P.gamma);
    const uint4* b = reinterpret_cast<const uint4*>(P.beta);
    uint4* sg = reinterpret_cast<uint4*>(params_smem);
    uint4* sb = reinterpret_cast<uint4*>(params_smem + slot_bytes);
    for (int i = tid; i < (int)(row_bytes / 16); i += blockDim.x) {
      sg[i] = __ldg(g + i);
      sb[i] = __ldg(b + i);
    }
  }
  __syncthreads();

  if (tid >= n_consumers) {
    // ---------------- producer warp ----------------
    // Rows are requested in order, `chunk` at a time by as many lanes in lock step (their
    // barrier polls and copy issues overlap).  With many small groups a round feeds one row
    // to every group: it only waits for slots that the groups free at about the same time,
    // so the ring never drains while a round waits.  With few large groups (long rows) one
    // lane does it all: the per-row cost is negligible there and a round of three would hold
    // back the first copy until the third slot is free.
    // (16384 x 8192 fp16, same box: one lane / lock-step rounds: softmax 6450 / 6470 GB/s,
    // LayerNorm 6480 / 6300.)
    // (Fetching a round of `groups` consecutive rows by ONE copy into adjacent slots, which is what
    // lifted the narrow rows of LayerNorm backward, loses here: LayerNorm 16384 x 1024 / 2048 / 4096
    // 4369 / 5595 / 6291 -> 3732 / 4877 / 5597 GB/s -- all groups then wait for the same barrier and
    // the producer for all of their slots, instead of each group drifting at its own pace.)
    const int chunk = groups > 4 ? groups : 1;
    const int lane = tid & 31;
    const T* __restrict__ x = reinterpret_cast<const T*>(P.x);
    int slot0 = 0;       // first slot of this round (the slot count is a multiple of the group count)
    uint32_t lap = 0;    // how often the ring has wrapped
    int64_t issued = 0;  // rows requested so far
    bool failed = false;
    for (int64_t base = 0; base < my_rows; base += chunk) {
      const int64_t n = base + lane;
      const int sl = slot0 + lane;
      if (lane < chunk && n < my_rows) {
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[sl]), (lap & 1) ^ 1, abort_flag, kWaitLimit)) {
          *abort_flag = 1;
          atomicCAS(status, 0u, 0x40000u | (uint32_t)sl);
          failed = true;
        } else {
          const int64_t w = blockIdx.x + n * (int64_t)gridDim.x;
          const int64_t row = P.has_map ? (int64_t)map_eval(P.map, (uint64_t)w) : w;
          ctl->row[sl] = row;
          const uint32_t full = ptx::smem_u32(&ctl->full[sl]);
          ptx::mbar_arrive_expect_tx(full, row_bytes);
          ptx::bulk_load(ptx::smem_u32(ring_smem + (size_t)sl * slot_bytes), x + row * cols, row_bytes, full);
        }
      }
      if (__any_sync(0xffffffffu, failed)) break;
      issued = base + chunk < my_rows ? base + chunk : my_rows;
      slot0 += chunk;
      if (slot0 == stages) {
        slot0 = 0;
        ++lap;
      }
    }
    if (*abort_flag && lane == 0) {
      // leave no copy of ours in flight: the last request into every slot
      uint32_t never = 0;
      for (int sl = 0; sl < stages; ++sl) {
        const int64_t uses = issued > sl ? (issued - sl + stages - 1) / stages : 0;
        if (uses) ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[sl]), (uint32_t)((uses - 1) & 1), &never, kWaitLimit);
      }
    }
    return;
  }

  // ---------------- consumers: group g takes rows g, g + groups, ... of this CTA ----------------
  // The slot count is a multiple of the group count, so a slot is always drained by the same
  // group (a waiter two uses ahead of an mbarrier could not tell its phase from the one two back).
  T* __restrict__ y = reinterpret_cast<T*>(P.y);
  const int group = tid / gsize;
  const int gtid = tid - group * gsize;  // thread within the group
  const int lane = tid & 31;
  const int warp_in_group = gtid >> 5;
  const int bar = 1 + group;
  float (*slots)[16] = slots_all[group];
  volatile uint32_t* group_abort = &ctl->group_abort[group];
  int s = group;       // this group walks slots group, group + groups, ...
  uint32_t use = 0;    // laps of the ring
  for (int64_t n = group; n < my_rows; n += groups, s += groups) {
    if (s >= stages) {
      s -= stages;
      ++use;
    }
    const bool ok = ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), use & 1, abort_flag, kWaitLimit);
    if (!ok) {
      *abort_flag = 1;
      *group_abort = 1;
      atomicCAS(status, 0u, 0x50000u | (uint32_t)s);
    }
    const int64_t row = ok ? ctl->row[s] : 0;
    const uint4* slot = reinterpret_cast<const uint4*>(ring_smem + (size_t)s * slot_bytes);
    float v[EPT];
    const float fill = OP == OP_SOFTMAX ? -INFINITY : 0.f;
    // (An instance without the `c < cols` predicates for rows of exactly gsize x EPT values was
    // slower, same box, 16384 x 8192 fp16: softmax 6501 -> 5879 GB/s, LayerNorm 6276-6544 -> 5700.)
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * gsize + gtid) * VEC;
      if (ok && c < cols) {
        Elem<T>::unpack(slot[k * gsize + gtid], v + k * VEC);
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) v[k * VEC + e] = fill;
      }
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[s]));  // slot may be refilled now

    if (OP == OP_SOFTMAX) {
      float m = v[0];
#pragma unroll
      for (int k = 1; k < EPT; ++k) m = fmaxf(m, v[k]);
      m = group_reduce<true>(m, slots[0], bar, gsize, nw, warp_in_group);
      if (*group_abort) break;  // uniform: the group's own flag writes of this row precede the barrier above
      const float ms = m * 1.4426950408889634f;
      float sum = 0.f;
#pragma unroll
      for (int k = 0; k < EPT; ++k) {
        v[k] = fast_exp2(fmaf(v[k], 1.4426950408889634f, -ms));
        sum += v[k];
      }
      sum = group_reduce<false>(sum, slots[1], bar, gsize, nw, warp_in_group);
      const float inv = 1.0f / sum;
      T* __restrict__ yrow = y + row * cols;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * gsize + gtid) * VEC;
        if (c < cols) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) v[k * VEC + e] *= inv;
          __stcs(reinterpret_cast<uint4*>(yrow + c), Elem<T>::pack(v + k * VEC));
        }
      }
    } else {
      float sum = 0.f;
#pragma unroll
      for (int k = 0; k < EPT; ++k) sum += v[k];
      sum = group_reduce<false>(sum, slots[0], bar, gsize, nw, warp_in_group);
      if (*group_abort) break;
      const float mean = sum / (float)cols;
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const bool in = (k * gsize + gtid) * VEC < cols;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float d = in ? v[k * VEC + e] - mean : 0.f;
          v[k * VEC + e] = d;
          q = fmaf(d, d, q);
        }
      }
      q = group_reduce<false>(q, slots[1], bar, gsize, nw, warp_in_group);
      const float rstd = 1.0f / sqrtf(q / (float)cols + P.eps);
      if (gtid == 0) {
        P.mean[row] = mean;
        P.rstd[row] = rstd;
      }
      const uint4* sg = reinterpret_cast<const uint4*>(params_smem);
      const uint4* sb = reinterpret_cast<const uint4*>(params_smem + slot_bytes);
      T* __restrict__ yrow = y + row * cols;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * gsize + gtid) * VEC;
        if (c < cols) {
          float g[VEC], b[VEC];
          Elem<T>::unpack(sg[k * gsize + gtid], g);
          Elem<T>::unpack(sb[k * gsize + gtid], b);
#pragma unroll
          for (int e = 0; e < VEC; ++e) v[k * VEC + e] = fmaf(v[k * VEC + e] * rstd, g[e], b[e]);
          __stcs(reinterpret_cast<uint4*>(yrow + c), Elem<T>::pack(v + k * VEC));
        }
      }
    }
  }
}

template <int OP, typename T, int G, int EPT = kRingEpt>
int32_t launch_ring_g(const RowParams& P, DeviceCtx* ctx, cudaStream_t s, int stages, int groups, int gsize, size_t smem) {
  auto kern = row_ring_kernel<OP, T, G, EPT>;
  static PerDeviceFlag configured;
  if (!configured.test(ctx->device)) {
    LEGO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->smem_optin - 4096));  // static part: reduction slots
    configured.set(ctx->device);
  }
  int64_t grid = ctx->sm_count;
  if (grid > P.rows) grid = P.rows;
  const cudaError_t e = launch_overlapped(kern, dim3((unsigned)grid), dim3(groups * gsize + 32), smem, s, P, stages,
                                          groups, gsize, ctx->status_word);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return cuda_status(e);
}

template <int OP, typename T>
int32_t launch_ring(const RowParams& P, DeviceCtx* ctx, cudaStream_t s) {
  constexpr int VEC = Elem<T>::VEC;
  const size_t row_bytes = (size_t)P.cols * sizeof(T);
  const size_t slot = (row_bytes + 127) & ~(size_t)127;
  const size_t fixed = (OP == OP_LAYERNORM ? 2 * slot : 0) + sizeof(RingCtl) + 128;
  // threads per row: 32 values each, whole warps; 64 each once that would need more than 256 threads
  // (one group of 512 turns one row around at a time: 16384-wide fp16 rows ran at 0.76 of the copy peak)
  int per_thread = kRingEpt / VEC;  // vectors per thread
  const int vectors = P.cols / VEC;
  int gsize = ((vectors + per_thread - 1) / per_thread + 31) & ~31;
  const bool wide = gsize > 256;
  if (wide) {
    per_thread *= 2;
    gsize = ((vectors + per_thread - 1) / per_thread + 31) & ~31;
  }
  if (gsize > 512) return LEGO_ERR_UNSUPPORTED;
  // Measured on B200 (16384 x 8192 fp16, 256 threads per row), same box, GB/s: one group turns
  // a row around in about 2500 cycles, so two groups (softmax: 6260; three: 5580, they fight
  // over the special-function pipe) or three (LayerNorm: 6390; two: 5410) keep up with HBM;
  // other widths keep the same number of consumer threads (512 / 768).  About 96 KiB of rows in
  // flight is the sweet spot (softmax 64 / 96 / 128 KiB: 6170 / 6260 / 6260; LayerNorm 48 / 96 /
  // 144 / 192 KiB: 5930 / 6390 / 6060 / 5930).
  int groups = (OP == OP_SOFTMAX || wide ? 512 : kMaxConsumers) / gsize;
  if (groups < 1) groups = 1;
  if (groups > kMaxGroups) groups = kMaxGroups;
  const size_t budget = (size_t)ctx->smem_optin - 4096 - fixed;
  int stages = (int)((96 * 1024 + slot / 2) / slot);
  if (stages < 2 * groups) stages = 2 * groups;
  if (stages > kRing) stages = kRing;
  if ((size_t)stages > budget / slot) stages = (int)(budget / slot);
  stages -= stages % groups;  // a slot always belongs to one group
  if (stages < groups) return LEGO_ERR_UNSUPPORTED;
  const size_t smem = (size_t)stages * slot + fixed;
  if (wide) {
    if (gsize == 256) return launch_ring_g<OP, T, 256, 2 * kRingEpt>(P, ctx, s, stages, groups, gsize, smem);
    return launch_ring_g<OP, T, 0, 2 * kRingEpt>(P, ctx, s, stages, groups, gsize, smem);
  }
  switch (gsize) {
    case 64: return launch_ring_g<OP, T, 64>(P, ctx, s, stages, groups, gsize, smem);
    case 128: return launch_ring_g<OP, T, 128>(P, ctx, s, stages, groups, gsize, smem);
    case 256: return launch_ring_g<OP, T, 256>(P, ctx, s, stages, groups, gsize, smem);
    default: return launch_ring_g<OP, T, 0>(P, ctx, s, stages, groups, gsize, smem);
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
  if (c <= 32 * 16) return launch_cfg<OP, T, 32, 16, VECTOR>(P, ctx, s);
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
  // long aligned rows, enough of them to fill the machine: the bulk-copy pipeline
  // (2 KiB rows: LayerNorm gains from the ring, 3.9 -> 4.4 TB/s; softmax loses, 5.9 -> 5.2 -- a warp per
  // row suits 1024 fp16 values exactly -- and takes the ring from there on: 16384 x 1280 / 1536 27.9 / 28.8
  // -> 19.9 / 20.1 us.  Several consecutive rows per ring slot, fetched by one copy, and three to six
  // slots per group instead of two were tried for these narrow rows: no gain, or a loss.)
  const size_t ring_from = OP == OP_SOFTMAX ? 2049 : 2048;
  if (vec && (size_t)P.cols * sizeof(T) >= ring_from && P.rows >= 2 * (int64_t)ctx->sm_count) {
    const int32_t st = launch_ring<OP, T>(P, ctx, s);
    if (st != LEGO_ERR_UNSUPPORTED) return st;
  }
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
