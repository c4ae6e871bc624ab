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
#include "ptx_sm100.cuh"
#include "rowwise.cuh"

namespace lego {
// lego_tune(LEGO_TUNE_LNBWD_LANES): producer of the grouped ring kernel.  0 = one thread; 1 = a lane
// per group in lock step where a slot holds one row; 2 = the same, and never the block form.
// most consumer groups for which the grouped ring kernel runs a folding warp per group (0: never)
std::atomic<int> g_lnbwd_foldw_groups{3};
// fewest rows the ring-fed kernels take; below, the register kernel
std::atomic<int> g_lnbwd_min_rows{1};
std::atomic<int> g_lnbwd_lanes{1};
// 8 added to the knob's value: every group writes its own partial row (no fold inside the CTA)
std::atomic<int> g_lnbwd_fold{1};
namespace {

constexpr int kMaxPartialRows = 1184;  // 8 partial rows (one per consumer group) on each of 148 SMs

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

// ---- bulk-copy pipelined dx kernel, one group (rows of more than 3 Ki columns) -------
//
// One CTA per SM.  A producer thread streams the rows of x and dy (and the 16-byte
// chunks holding the row's mean and rstd) into a shared-memory ring with 1-D bulk
// copies; 512 consumer threads own 8 or 16 fixed columns each: gamma and the two
// column accumulators of those columns stay in registers for the whole kernel, a row
// costs one two-value reduction over the CTA, and dx leaves in 128-bit streaming
// stores.  Memory-level parallelism comes from the ring (as many rows of x and dy in
// flight per SM as fit, up to 12), not from occupancy.

// The statistics of a row whose 16-byte chunk would reach past the arrays (the last rows & 3 rows of
// a row count that is no multiple of four): the producer reads the two floats itself and stores
// them where the chunk's copy would have put them (mean chunk at `stats`, rstd chunk `rstd_off`
// bytes behind), before its arrive on the slot's barrier, which publishes them to the consumers.
__device__ __forceinline__ void stats_by_hand(unsigned char* stats, uint32_t rstd_off, const BwdParams& P, int64_t row) {
  reinterpret_cast<float*>(stats)[row & 3] = P.mean[row];
  reinterpret_cast<float*>(stats + rstd_off)[row & 3] = P.rstd[row];
}

constexpr int kBwd1Consumers = 512;
constexpr int kBwd1Ring = 12;  // two slots are held by the rows in phase 1 and phase 2, the rest are loads in flight
constexpr long long kBwd1WaitLimit = 2000000000LL;  // SM cycles, about a second

struct BwdRing1Ctl {
  uint64_t full[kBwd1Ring];
  uint64_t empty[kBwd1Ring];
  uint64_t rowbar[2];  // row n's warp totals are all in red[]: 16 arrivals (one per consumer warp)
  uint64_t totbar[2];  // row n's totals are in tot[]: one arrival (the folding warp)
  int64_t row[kBwd1Ring];
  float2 tot[4];       // [row & 3] -> the row's (s1, s2)
  uint32_t abort_flag;
};

// FULLW (EPT 16, 24 or 32): the row is exactly 512 x EPT columns wide, so no vector of a thread
// lies past its end: no bounds predicates and no zero fill of the vectors.
// EPT: columns per consumer thread, 8 or 16 with gamma in registers; 24 or 32 (rows of 8 Ki .. 16 Ki
// columns) with gamma staged once per CTA in shared memory as fp16, because 64 accumulator
// registers leave no room for it: three ring slots of 64 KiB then.
template <int EPT, bool FULLW>
__global__ void __launch_bounds__(kBwd1Consumers + (EPT <= 24 ? 64 : 32), 1)
ln_bwd_ring1_kernel(const __grid_constant__ BwdParams P, int stages, uint32_t* status) {
  constexpr bool fold_warp = EPT <= 24;  // a second helper warp sums the rows' totals (see there)
  constexpr int NV = EPT / 8;
  constexpr int NW = kBwd1Consumers / 32;
  constexpr bool GSMEM = EPT > 16;
  extern __shared__ __align__(128) uint8_t bwd1_smem[];
  __shared__ __align__(16) float red[4][NW][2];  // [row & 3][warp] -> (s1, s2)
  __shared__ __align__(16) float2 part[fold_warp ? 2 : 1][fold_warp ? kBwd1Consumers : 1];  // [row & 1][thread] -> (s1, s2)
  const int cols = P.cols;
  const uint32_t row_bytes = (uint32_t)cols * 2u;
  const uint32_t half_slot = (row_bytes + 127u) & ~127u;
  const uint32_t slot_bytes = 2u * half_slot + 128u;  // x | dy | mean chunk, rstd chunk
  const uint4* gsm = reinterpret_cast<const uint4*>(bwd1_smem + (size_t)stages * slot_bytes);  // gamma (GSMEM)
  BwdRing1Ctl* ctl = reinterpret_cast<BwdRing1Ctl*>(bwd1_smem + (size_t)stages * slot_bytes + (GSMEM ? half_slot : 0u));
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const int tid = threadIdx.x;
  const int64_t my_rows = P.rows > blockIdx.x ? (P.rows - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), NW);
    }
    ptx::mbar_init(ptx::smem_u32(&ctl->rowbar[0]), NW);
    ptx::mbar_init(ptx::smem_u32(&ctl->rowbar[1]), NW);
    ptx::mbar_init(ptx::smem_u32(&ctl->totbar[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&ctl->totbar[1]), 1);
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
  ptx::launch_dependents();     // the column reduction (or the next op) may set itself up now
  ptx::grid_dependency_wait();  // global memory only once the previous grid is complete

  if (tid >= kBwd1Consumers + 32) {
    // ---------------- folding warp ----------------
    // Sums a row's 512 pairs of per-thread sums once for the whole CTA and publishes the totals
    // through totbar.  The consumers' phase 1 then ends with one shared-memory store instead of
    // six dependent shuffle levels, and their phase 2 starts with one load instead of four more.
    // Same box, 16384 x 8192: folding the 16 warp totals here 152 -> 135 us, the threads' sums
    // too 135 -> 129 us (6.25 TB/s); 8192 x 10240: 125 -> 104 -> 100 us.  The instances with 32
    // columns per thread have three ring slots and no room for part[]; folding only the warp
    // totals here made them 3 % slower, so they keep the fold in the consumers.
    const int lane = tid & 31;
    for (int64_t n = 0; fold_warp && n < my_rows; ++n) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->rowbar[n & 1]), (uint32_t)((n >> 1) & 1), abort_flag,
                                  kBwd1WaitLimit)) {
        *abort_flag = 1;
        atomicCAS(status, 0u, 0x78000u | (uint32_t)(n & 0xfff));
        break;
      }
      // lane l adds the sums of threads l, l + 32, ... (a fixed tree), then five shuffle levels
      float2 q[kBwd1Consumers / 32];
#pragma unroll
      for (int i = 0; i < kBwd1Consumers / 32; ++i) q[i] = part[fold_warp ? (n & 1) : 0][fold_warp ? lane + 32 * i : 0];
#pragma unroll
      for (int w = kBwd1Consumers / 64; w > 0; w >>= 1)
#pragma unroll
        for (int i = 0; i < w; ++i) q[i] = ptx::add2(q[i], q[i + w]);
      float2 ss = q[0];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ss.x += __shfl_xor_sync(0xffffffffu, ss.x, o);
        ss.y += __shfl_xor_sync(0xffffffffu, ss.y, o);
      }
      if (lane == 0) {
        ctl->tot[n & 3] = ss;
        ptx::mbar_arrive(ptx::smem_u32(&ctl->totbar[n & 1]));  // release: the store above is visible to the waiters
      }
      __syncwarp();
    }
    return;
  }
  if (tid >= kBwd1Consumers) {
    // ---------------- producer ----------------
    if (tid == kBwd1Consumers) {
      int64_t issued = 0;
      // s walks the ring, use counts the laps (no 64-bit division per row)
      int s = 0;
      uint32_t use = 0;
      for (int64_t n = 0; n < my_rows; ++n, s = (s + 1 == stages ? 0 : s + 1), use += (s == 0)) {
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[s]), (use & 1) ^ 1, abort_flag, kBwd1WaitLimit)) {
          *abort_flag = 1;
          atomicCAS(status, 0u, 0x60000u | (uint32_t)s);
          break;
        }
        const int64_t row = blockIdx.x + n * (int64_t)gridDim.x;
        ctl->row[s] = row;
        const uint32_t full = ptx::smem_u32(&ctl->full[s]);
        const uint32_t dst = ptx::smem_u32(bwd1_smem + (size_t)s * slot_bytes);
        const bool whole = (row | 3) < P.rows;  // else by plain loads: see stats_by_hand
        if (!whole) stats_by_hand(bwd1_smem + (size_t)s * slot_bytes + 2u * half_slot, 16u, P, row);
        ptx::mbar_arrive_expect_tx(full, 2u * row_bytes + (whole ? 32u : 0u));
        ptx::bulk_load(dst, P.x + row * cols, row_bytes, full);
        ptx::bulk_load(dst + half_slot, P.dy + row * cols, row_bytes, full);
        if (whole) {
          ptx::bulk_load(dst + 2u * half_slot, P.mean + (row & ~3LL), 16u, full);
          ptx::bulk_load(dst + 2u * half_slot + 16u, P.rstd + (row & ~3LL), 16u, full);
        }
        ++issued;
      }
      if (*abort_flag) {
        // leave no copy of ours in flight
        uint32_t never = 0;
        for (int s = 0; s < stages; ++s) {
          const int64_t uses = issued > s ? (issued - s + stages - 1) / stages : 0;
          if (uses) ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), (uint32_t)((uses - 1) & 1), &never, kBwd1WaitLimit);
        }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  // All element-wise fp32 work runs as packed pairs (f32x2).  A row is handled in two
  // phases with the next row's first phase in between, so that the CTA-wide reduction of a
  // row (shuffles, a hop through shared memory, an mbarrier) is in flight while the thread
  // does useful work instead of waiting at a barrier:
  //   phase 1 (row n)  column accumulators, the row's two sums -> part[n & 1] (or, without a
  //                    folding warp, warp totals -> red[n & 3]), arrive on rowbar[n & 1];
  //   phase 2 (row n)  wait for the row's totals (totbar; or rowbar and fold the 16 warp
  //                    totals oneself), re-read x and dy from the
  //                    ring slot, recompute xhat and dy * gamma (cheaper than keeping 32
  //                    registers alive across phase 1 of the next row), write dx, free the slot.
  // Four red[] buffers: a warp in phase 1 of row n + 2 has passed the barrier of row n, so
  // every warp has finished phase 1 of row n, which follows its phase 2 of row n - 2.
  constexpr int P2 = EPT / 2;
  const int lane = tid & 31, warp = tid >> 5;
  float2 g[GSMEM ? 1 : P2], acc_w[P2], acc_b[P2];
  if (GSMEM) {
    uint4* gw = reinterpret_cast<uint4*>(bwd1_smem + (size_t)stages * slot_bytes);
    for (int v = tid; v < (int)(half_slot / 16u); v += kBwd1Consumers)
      gw[v] = (FULLW || v * 8 < cols) ? __ldg(reinterpret_cast<const uint4*>(P.gamma) + v) : make_uint4(0u, 0u, 0u, 0u);
    ptx::named_barrier<1, kBwd1Consumers>();  // consumers only: the producer is already streaming rows
  } else {
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * kBwd1Consumers + tid) * 8;
      uint4 raw = make_uint4(0u, 0u, 0u, 0u);
      if ((FULLW || c < cols)) raw = __ldg(reinterpret_cast<const uint4*>(P.gamma + c));
      const __half2* hp = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) g[k * 4 + e] = __half22float2(hp[e]);
    }
  }
  // gamma of this thread's e-th pair of its k-th vector
  auto gamma_of = [&](const uint4& gv, int k, int e) -> float2 {
    return GSMEM ? __half22float2(reinterpret_cast<const __half2*>(&gv)[e]) : g[GSMEM ? 0 : k * 4 + e];
  };
#pragma unroll
  for (int k = 0; k < P2; ++k) acc_w[k] = acc_b[k] = make_float2(0.f, 0.f);
  const float inv_cols = 1.0f / (float)cols;

  bool alive = true;
  auto phase1 = [&](int64_t n, int s, uint32_t use) {
    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), use & 1, abort_flag, kBwd1WaitLimit)) {
      *abort_flag = 1;
      atomicCAS(status, 0u, 0x70000u | (uint32_t)s);
      alive = false;
      return;
    }
    const uint8_t* slot = bwd1_smem + (size_t)s * slot_bytes;
    const int64_t row = ctl->row[s];
    const float mean = reinterpret_cast<const float*>(slot + 2u * half_slot)[row & 3];
    const float rstd = reinterpret_cast<const float*>(slot + 2u * half_slot + 16u)[row & 3];
    // xhat = x * rstd - mean * rstd; columns past the end hold dy = 0 and gamma = 0, so they add nothing
    const float2 rstd2 = make_float2(rstd, rstd), shift2 = make_float2(-mean * rstd, -mean * rstd);
    float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int v = k * kBwd1Consumers + tid;
      uint4 xr = make_uint4(0u, 0u, 0u, 0u), dr = make_uint4(0u, 0u, 0u, 0u), gv = make_uint4(0u, 0u, 0u, 0u);
      if ((FULLW || v * 8 < cols)) {
        xr = reinterpret_cast<const uint4*>(slot)[v];
        dr = reinterpret_cast<const uint4*>(slot + half_slot)[v];
        if (GSMEM) gv = gsm[v];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 d = __half22float2(reinterpret_cast<const __half2*>(&dr)[e]);
        const float2 h = ptx::fma2(__half22float2(reinterpret_cast<const __half2*>(&xr)[e]), rstd2, shift2);
        acc_w[k * 4 + e] = ptx::fma2(d, h, acc_w[k * 4 + e]);
        acc_b[k * 4 + e] = ptx::add2(acc_b[k * 4 + e], d);
        const float2 w = ptx::mul2(d, gamma_of(gv, k, e));
        s1 = ptx::fma2(h, w, s1);
        s2 = ptx::add2(s2, w);
      }
    }
    // Even lanes fold the first sum, odd lanes the second: one shuffle per level instead of
    // two; lanes 0 and 1 end with the warp's two totals.
    const float a = s1.x + s1.y, bsum = s2.x + s2.y;
    if (fold_warp) {
      part[fold_warp ? (n & 1) : 0][fold_warp ? tid : 0] = make_float2(a, bsum);  // the folding warp adds them up
    } else {
      const bool odd = (lane & 1) != 0;
      float keep = odd ? bsum : a;
      keep += __shfl_xor_sync(0xffffffffu, odd ? a : bsum, 1);
#pragma unroll
      for (int o = 2; o <= 16; o <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
      if (lane < 2) red[n & 3][warp][lane] = keep;
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->rowbar[n & 1]));
  };
  auto phase2 = [&](int64_t n, int s) {
    if (!ptx::mbar_wait_bounded(ptx::smem_u32(fold_warp ? &ctl->totbar[n & 1] : &ctl->rowbar[n & 1]),
                                (uint32_t)((n >> 1) & 1), abort_flag, kBwd1WaitLimit)) {
      *abort_flag = 1;
      atomicCAS(status, 0u, (fold_warp ? 0x7c000u : 0x78000u) | (uint32_t)s);
      alive = false;
      return;
    }
    float2 ss;
    if (fold_warp) {
      ss = ctl->tot[n & 3];  // the row's totals, folded once for the CTA
    } else {
      // Both half-warps fold the same 16 warp totals, so every lane ends with the row's totals
      // after four shuffle levels.
      ss = *reinterpret_cast<const float2*>(&red[n & 3][lane & (NW - 1)][0]);
#pragma unroll
      for (int o = NW / 2; o > 0; o >>= 1) {
        ss.x += __shfl_xor_sync(0xffffffffu, ss.x, o);
        ss.y += __shfl_xor_sync(0xffffffffu, ss.y, o);
      }
    }
    const uint8_t* slot = bwd1_smem + (size_t)s * slot_bytes;
    const int64_t row = ctl->row[s];
    const float mean = reinterpret_cast<const float*>(slot + 2u * half_slot)[row & 3];
    const float rstd = reinterpret_cast<const float*>(slot + 2u * half_slot + 16u)[row & 3];
    const float2 rstd2 = make_float2(rstd, rstd), shift2 = make_float2(-mean * rstd, -mean * rstd);
    // dx = (wdy - (xhat * c1 + c2)) * rstd, as two fused steps per pair
    const float c1r = ss.x * inv_cols * rstd, c2r = ss.y * inv_cols * rstd;
    const float2 nc1 = make_float2(-c1r, -c1r), nc2 = make_float2(-c2r, -c2r);
    __half* __restrict__ dx = P.dx + row * cols;
    uint4 outv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int v = k * kBwd1Consumers + tid;
      uint4 xr = make_uint4(0u, 0u, 0u, 0u), dr = make_uint4(0u, 0u, 0u, 0u), gv = make_uint4(0u, 0u, 0u, 0u);
      if ((FULLW || v * 8 < cols)) {
        xr = reinterpret_cast<const uint4*>(slot)[v];
        dr = reinterpret_cast<const uint4*>(slot + half_slot)[v];
        if (GSMEM) gv = gsm[v];
      }
      __half2* o2 = reinterpret_cast<__half2*>(&outv[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 d = __half22float2(reinterpret_cast<const __half2*>(&dr)[e]);
        const float2 h = ptx::fma2(__half22float2(reinterpret_cast<const __half2*>(&xr)[e]), rstd2, shift2);
        const float2 w = ptx::mul2(d, gamma_of(gv, k, e));
        const float2 t = ptx::fma2(h, nc1, ptx::fma2(w, rstd2, nc2));
        o2[e] = __floats2half2_rn(t.x, t.y);
      }
      // with 32 columns per thread the results leave at once: no registers to park four vectors in
      if (GSMEM && (FULLW || v * 8 < cols)) __stcs(reinterpret_cast<uint4*>(dx + v * 8), outv[k]);
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[s]));  // slot may be refilled now
    if (!GSMEM) {
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * kBwd1Consumers + tid) * 8;
        if ((FULLW || c < cols)) __stcs(reinterpret_cast<uint4*>(dx + c), outv[k]);
      }
    }
  };

  // ring cursors of the row in phase 1 (s1, use1) and of the row in phase 2 (s2)
  int s1 = 0, s2 = 0;
  uint32_t use1 = 0;
  auto advance = [&](int& s) { s = (s + 1 == stages) ? 0 : s + 1; };
  if (my_rows > 0) phase1(0, s1, use1);
  for (int64_t n = 0; alive && n < my_rows; ++n) {
    if (n + 1 < my_rows) {
      advance(s1);
      use1 += (s1 == 0);
      phase1(n + 1, s1, use1);
      if (!alive) break;
    }
    phase2(n, s2);
    advance(s2);
  }
  if (*abort_flag) return;
  float* pw = P.partial + (size_t)blockIdx.x * cols;
  float* pb = P.partial + ((size_t)P.partial_rows + blockIdx.x) * cols;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = (k * kBwd1Consumers + tid) * 8;
    if ((FULLW || c < cols)) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = k * 4 + 2 * e;
        *reinterpret_cast<float4*>(pw + c + 4 * e) = make_float4(acc_w[j].x, acc_w[j].y, acc_w[j + 1].x, acc_w[j + 1].y);
        *reinterpret_cast<float4*>(pb + c + 4 * e) = make_float4(acc_b[j].x, acc_b[j].y, acc_b[j + 1].x, acc_b[j + 1].y);
      }
    }
  }
}

// Launches the ring kernel when the shape suits it; LEGO_ERR_UNSUPPORTED otherwise.
template <int EPT>
int32_t launch_ring1_dx(BwdParams& P, DeviceCtx* ctx, cudaStream_t s) {
  // Without the bounds predicates, same box: 8192 x 12288 (24 columns per thread) 135.7 -> 119 us,
  // 8192 x 16384 (32) 176 -> 164 us; 16384 x 8192 (16): 150 -> 154 us while the consumers still
  // folded the row sums by shuffles, 135.5 -> 130.5 us since the folding warp does.
  const bool fullw = EPT >= 16 && P.cols == EPT * kBwd1Consumers;
  auto kern = fullw ? ln_bwd_ring1_kernel<EPT, (EPT >= 16)> : ln_bwd_ring1_kernel<EPT, false>;
  const size_t half_slot = ((size_t)P.cols * 2 + 127) & ~(size_t)127;
  const size_t slot = 2 * half_slot + 128;
  const size_t part_bytes = EPT <= 24 ? 2 * kBwd1Consumers * sizeof(float2) : 0;  // static: the threads' row sums
  static PerDeviceFlag configured[2];  // one per kernel
  if (!configured[fullw].test(ctx->device)) {
    LEGO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->smem_optin - 1024 - part_bytes));
    configured[fullw].set(ctx->device);
  }
  const size_t gamma_bytes = EPT > 16 ? half_slot : 0;  // gamma staged in shared memory
  const size_t budget = (size_t)ctx->smem_optin - 1024 - sizeof(BwdRing1Ctl) - 128 - gamma_bytes - part_bytes;
  int stages = (int)(budget / slot);
  if (stages > kBwd1Ring) stages = kBwd1Ring;
  if (stages < 3) return LEGO_ERR_UNSUPPORTED;  // the rows in phase 1 and phase 2 hold two slots; one more for the load in flight
  const size_t smem = (size_t)stages * slot + gamma_bytes + sizeof(BwdRing1Ctl) + 128;
  const int grid = (int)(P.rows < ctx->sm_count ? P.rows : ctx->sm_count);
  P.partial_rows = grid;
  const cudaError_t e = launch_overlapped(kern, dim3(grid), dim3(kBwd1Consumers + (EPT <= 24 ? 64 : 32)), smem, s, P, stages,
                                          ctx->status_word);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return cuda_status(e);
}

// ---- rows of 16 Ki .. 32 Ki columns: a CTA pair per row ------------------------------
//
// The 64 accumulator registers of 32 columns per thread are all a thread can hold, so rows wider
// than 512 x 32 columns are split between the two CTAs of a cluster: each runs the ring scheme of
// ln_bwd_ring1_kernel<32> on its half of the columns of the SAME rows (gamma of its half in shared
// memory, three ring slots), and the two halves of a row's sums meet in both CTAs: every warp
// writes its two totals into its slot of red[] in its own and in the peer's shared memory and
// arrives on both row barriers (32 arrivals: 16 warps of each CTA).  Everything else -- two phases
// per row with the next row's first phase in between, fixed columns per thread, one partial row per
// pair -- is as there.  No thread leaves before the final cluster barrier: the peer may still
// store into this CTA's shared memory.

struct BwdPairCtl {
  uint64_t full[kBwd1Ring];
  uint64_t empty[kBwd1Ring];
  uint64_t rowbar[2];   // 16 arrivals: this CTA's consumer warps have left their totals of the row in red[]
  uint64_t peerbar[2];  // one arrival, from the peer's liaison warp: the peer's half of the row sums is in peer_tot[]
  uint64_t totbar[2];   // one arrival, from this CTA's liaison warp: the whole row's sums are in tot[]
  int64_t row[kBwd1Ring];
  float2 peer_tot[4];   // [row & 3], written by the peer
  float2 tot[4];        // [row & 3]
  uint32_t abort_flag;
};

template <bool FULLW>  // FULLW: 32768 columns, both halves exactly 512 x 32: no bounds predicates
__global__ void __launch_bounds__(kBwd1Consumers + 64, 1)
ln_bwd_pair_kernel(const __grid_constant__ BwdParams P, int stages, int col_half, uint32_t* status) {
  constexpr int EPT = 32;
  constexpr int NV = EPT / 8;
  constexpr int NW = kBwd1Consumers / 32;
  constexpr int P2 = EPT / 2;
  extern __shared__ __align__(128) uint8_t pair_smem[];
  __shared__ __align__(16) float red[4][NW][2];  // [row & 3][warp] -> (s1, s2) of this CTA's half of the row
  const uint32_t rank = ptx::cluster_ctarank();
  const uint32_t peer = rank ^ 1u;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int cols_full = P.cols;
  const int col0 = (int)rank * col_half;
  const int cols = cols_full - col0 < col_half ? cols_full - col0 : col_half;  // this CTA's columns
  const uint32_t row_bytes = (uint32_t)cols * 2u;
  const uint32_t half_slot = ((uint32_t)col_half * 2u + 127u) & ~127u;
  const uint32_t slot_bytes = 2u * half_slot + 128u;  // x | dy | mean chunk, rstd chunk
  uint4* gsm = reinterpret_cast<uint4*>(pair_smem + (size_t)stages * slot_bytes);  // gamma of this half
  BwdPairCtl* ctl = reinterpret_cast<BwdPairCtl*>(pair_smem + (size_t)stages * slot_bytes + half_slot);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const int tid = threadIdx.x;
  const int64_t my_rows = P.rows > pair ? (P.rows - pair + n_pairs - 1) / n_pairs : 0;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), NW);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(ptx::smem_u32(&ctl->rowbar[i]), NW);
      ptx::mbar_init(ptx::smem_u32(&ctl->peerbar[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->totbar[i]), 1);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers exist before anything arrives on them
  ptx::launch_dependents();
  ptx::grid_dependency_wait();

  auto fail = [&](uint32_t code) {
    *abort_flag = 1;
    ptx::st_cluster_u32(ptx::mapa(ptx::smem_u32(const_cast<uint32_t*>(abort_flag)), peer), 1u);
    atomicCAS(status, 0u, code);
  };

  if (tid >= kBwd1Consumers + 32) {
    // ---------------- liaison warp ----------------
    // The only role that talks to the peer CTA.  Per row: wait for this CTA's 16 warp totals, fold
    // them, store the pair of sums into the peer's peer_tot[] and arrive on its peerbar (release at
    // cluster scope), wait for the peer's pair (acquire at cluster scope), add the two halves in
    // rank order (the same bits in both CTAs) and publish the row's sums to the consumers through
    // totbar.  The consumers themselves synchronise at CTA scope only: when every consumer warp
    // stored to the peer and arrived with a cluster-scope release, each such arrive first waited
    // for the warp's outstanding dx stores (stall_membar 2.8 per issue, the top stall; 4096 x 32768:
    // 216 us with that form).
    const int lane = tid & 31;
    const uint32_t peer_tot_remote = ptx::mapa(ptx::smem_u32(&ctl->peer_tot[0]), peer);
    const uint32_t peerbar_remote = ptx::mapa(ptx::smem_u32(&ctl->peerbar[0]), peer);
    for (int64_t n = 0; n < my_rows; ++n) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->rowbar[n & 1]), (uint32_t)((n >> 1) & 1), abort_flag,
                                  kBwd1WaitLimit)) {
        if (lane == 0) fail(0x78000u | 0x2000u);
        break;
      }
      float2 mine = *reinterpret_cast<const float2*>(&red[n & 3][lane & (NW - 1)][0]);
#pragma unroll
      for (int o = NW / 2; o > 0; o >>= 1) {
        mine.x += __shfl_xor_sync(0xffffffffu, mine.x, o);
        mine.y += __shfl_xor_sync(0xffffffffu, mine.y, o);
      }
      int ok = 1;
      if (lane == 0) {
        ptx::st_cluster_f32x2(peer_tot_remote + (uint32_t)(n & 3) * 8u, mine.x, mine.y);
        ptx::mbar_arrive_cluster(peerbar_remote + (uint32_t)(n & 1) * 8u);
        ok = ptx::mbar_wait_bounded_cluster(ptx::smem_u32(&ctl->peerbar[n & 1]), (uint32_t)((n >> 1) & 1), abort_flag,
                                            kBwd1WaitLimit) ? 1 : 0;
        if (ok) {
          const volatile float* pt = reinterpret_cast<const volatile float*>(&ctl->peer_tot[n & 3]);
          const float2 theirs = make_float2(pt[0], pt[1]);
          const float2 r0 = rank == 0 ? mine : theirs, r1 = rank == 0 ? theirs : mine;
          ctl->tot[n & 3] = make_float2(r0.x + r1.x, r0.y + r1.y);
          ptx::mbar_arrive(ptx::smem_u32(&ctl->totbar[n & 1]));  // release: the store above is visible to the waiters
        } else {
          fail(0x78000u | 0x1000u);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
    }
  } else if (tid >= kBwd1Consumers) {
    // ---------------- producer ----------------
    if (tid == kBwd1Consumers) {
      int64_t issued = 0;
      int s = 0;
      uint32_t use = 0;
      for (int64_t n = 0; n < my_rows; ++n, s = (s + 1 == stages ? 0 : s + 1), use += (s == 0)) {
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[s]), (use & 1) ^ 1, abort_flag, kBwd1WaitLimit)) {
          fail(0x60000u | 0x8000u | (uint32_t)s);
          break;
        }
        const int64_t row = pair + n * (int64_t)n_pairs;
        ctl->row[s] = row;
        const uint32_t full = ptx::smem_u32(&ctl->full[s]);
        const uint32_t dst = ptx::smem_u32(pair_smem + (size_t)s * slot_bytes);
        const bool whole = (row | 3) < P.rows;
        if (!whole) stats_by_hand(pair_smem + (size_t)s * slot_bytes + 2u * half_slot, 64u, P, row);
        ptx::mbar_arrive_expect_tx(full, 2u * row_bytes + (whole ? 32u : 0u));
        ptx::bulk_load(dst, P.x + row * cols_full + col0, row_bytes, full);
        ptx::bulk_load(dst + half_slot, P.dy + row * cols_full + col0, row_bytes, full);
        if (whole) {
          ptx::bulk_load(dst + 2u * half_slot, P.mean + (row & ~3LL), 16u, full);
          ptx::bulk_load(dst + 2u * half_slot + 64u, P.rstd + (row & ~3LL), 16u, full);
        }
        ++issued;
      }
      if (*abort_flag) {
        uint32_t never = 0;
        for (int sl = 0; sl < stages; ++sl) {
          const int64_t uses = issued > sl ? (issued - sl + stages - 1) / stages : 0;
          if (uses) ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[sl]), (uint32_t)((uses - 1) & 1), &never, kBwd1WaitLimit);
        }
      }
    }
  } else {
    // ---------------- consumers ----------------
    const int lane = tid & 31, warp = tid >> 5;
    for (int v = tid; v < (int)(half_slot / 16u); v += kBwd1Consumers)
      gsm[v] = (FULLW || v * 8 < cols) ? __ldg(reinterpret_cast<const uint4*>(P.gamma + col0) + v) : make_uint4(0u, 0u, 0u, 0u);
    ptx::named_barrier<1, kBwd1Consumers>();
    float2 acc_w[P2], acc_b[P2];
#pragma unroll
    for (int k = 0; k < P2; ++k) acc_w[k] = acc_b[k] = make_float2(0.f, 0.f);
    const float inv_cols = 1.0f / (float)cols_full;

    bool alive = true;
    auto phase1 = [&](int64_t n, int s, uint32_t use) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), use & 1, abort_flag, kBwd1WaitLimit)) {
        fail(0x70000u | 0x8000u | (uint32_t)s);
        alive = false;
        return;
      }
      const uint8_t* slot = pair_smem + (size_t)s * slot_bytes;
      const int64_t row = ctl->row[s];
      const float mean = reinterpret_cast<const float*>(slot + 2u * half_slot)[row & 3];
      const float rstd = reinterpret_cast<const float*>(slot + 2u * half_slot + 64u)[row & 3];
      const float2 rstd2 = make_float2(rstd, rstd), shift2 = make_float2(-mean * rstd, -mean * rstd);
      float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int v = k * kBwd1Consumers + tid;
        uint4 xr = make_uint4(0u, 0u, 0u, 0u), dr = make_uint4(0u, 0u, 0u, 0u), gv = make_uint4(0u, 0u, 0u, 0u);
        if ((FULLW || v * 8 < cols)) {
          xr = reinterpret_cast<const uint4*>(slot)[v];
          dr = reinterpret_cast<const uint4*>(slot + half_slot)[v];
          gv = gsm[v];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 d = __half22float2(reinterpret_cast<const __half2*>(&dr)[e]);
          const float2 h = ptx::fma2(__half22float2(reinterpret_cast<const __half2*>(&xr)[e]), rstd2, shift2);
          acc_w[k * 4 + e] = ptx::fma2(d, h, acc_w[k * 4 + e]);
          acc_b[k * 4 + e] = ptx::add2(acc_b[k * 4 + e], d);
          const float2 w = ptx::mul2(d, __half22float2(reinterpret_cast<const __half2*>(&gv)[e]));
          s1 = ptx::fma2(h, w, s1);
          s2 = ptx::add2(s2, w);
        }
      }
      float a = s1.x + s1.y, bsum = s2.x + s2.y;
#pragma unroll
      for (int o = 1; o <= 16; o <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        bsum += __shfl_xor_sync(0xffffffffu, bsum, o);
      }
      if (lane == 0) {
        // this warp's totals for the liaison warp; CTA scope only
        red[n & 3][warp][0] = a;
        red[n & 3][warp][1] = bsum;
        ptx::mbar_arrive(ptx::smem_u32(&ctl->rowbar[n & 1]));
      }
    };
    auto phase2 = [&](int64_t n, int s) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->totbar[n & 1]), (uint32_t)((n >> 1) & 1), abort_flag, kBwd1WaitLimit)) {
        fail(0x78000u | 0x4000u | (uint32_t)s);
        alive = false;
        return;
      }
      const float2 ss = ctl->tot[n & 3];  // both halves of the row, added up by the liaison warp
      const uint8_t* slot = pair_smem + (size_t)s * slot_bytes;
      const int64_t row = ctl->row[s];
      const float mean = reinterpret_cast<const float*>(slot + 2u * half_slot)[row & 3];
      const float rstd = reinterpret_cast<const float*>(slot + 2u * half_slot + 64u)[row & 3];
      const float2 rstd2 = make_float2(rstd, rstd), shift2 = make_float2(-mean * rstd, -mean * rstd);
      const float c1r = ss.x * inv_cols * rstd, c2r = ss.y * inv_cols * rstd;
      const float2 nc1 = make_float2(-c1r, -c1r), nc2 = make_float2(-c2r, -c2r);
      __half* __restrict__ dx = P.dx + row * cols_full + col0;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int v = k * kBwd1Consumers + tid;
        if ((FULLW || v * 8 < cols)) {
          const uint4 xr = reinterpret_cast<const uint4*>(slot)[v];
          const uint4 dr = reinterpret_cast<const uint4*>(slot + half_slot)[v];
          const uint4 gv = gsm[v];
          uint4 outv;
          __half2* o2 = reinterpret_cast<__half2*>(&outv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 d = __half22float2(reinterpret_cast<const __half2*>(&dr)[e]);
            const float2 h = ptx::fma2(__half22float2(reinterpret_cast<const __half2*>(&xr)[e]), rstd2, shift2);
            const float2 w = ptx::mul2(d, __half22float2(reinterpret_cast<const __half2*>(&gv)[e]));
            const float2 t = ptx::fma2(h, nc1, ptx::fma2(w, rstd2, nc2));
            o2[e] = __floats2half2_rn(t.x, t.y);
          }
          __stcs(reinterpret_cast<uint4*>(dx + v * 8), outv);
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[s]));  // slot may be refilled now
    };

    int s1 = 0, s2 = 0;
    uint32_t use1 = 0;
    auto advance = [&](int& s) { s = (s + 1 == stages) ? 0 : s + 1; };
    if (my_rows > 0) phase1(0, s1, use1);
    for (int64_t n = 0; alive && n < my_rows; ++n) {
      if (n + 1 < my_rows) {
        advance(s1);
        use1 += (s1 == 0);
        phase1(n + 1, s1, use1);
        if (!alive) break;
      }
      phase2(n, s2);
      advance(s2);
    }
    if (!*abort_flag) {
      float* pw = P.partial + (size_t)pair * cols_full + col0;
      float* pb = P.partial + ((size_t)P.partial_rows + pair) * cols_full + col0;
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const int c = (k * kBwd1Consumers + tid) * 8;
        if ((FULLW || c < cols)) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = k * 4 + 2 * e;
            *reinterpret_cast<float4*>(pw + c + 4 * e) = make_float4(acc_w[j].x, acc_w[j].y, acc_w[j + 1].x, acc_w[j + 1].y);
            *reinterpret_cast<float4*>(pb + c + 4 * e) = make_float4(acc_b[j].x, acc_b[j].y, acc_b[j + 1].x, acc_b[j + 1].y);
          }
        }
      }
    }
  }
  __syncthreads();
  ptx::cluster_sync();  // neither CTA leaves while the other may still store into its shared memory
}

// The pair kernel for rows of more than 16 Ki columns; LEGO_ERR_UNSUPPORTED when the device cannot
// schedule the clusters or the shape does not suit it.
int32_t launch_pair_dx(BwdParams& P, DeviceCtx* ctx, cudaStream_t s) {
  const int col_half = (int)((((int64_t)P.cols + 1) / 2 + 7) & ~7LL);  // columns of the first CTA, a multiple of 8
  if (col_half > kBwd1Consumers * 32 || P.cols - col_half < 8) return LEGO_ERR_UNSUPPORTED;
  const size_t half_slot = ((size_t)col_half * 2 + 127) & ~(size_t)127;
  const size_t slot = 2 * half_slot + 128;
  const bool fullw = P.cols == 2 * kBwd1Consumers * 32;
  auto kern = fullw ? ln_bwd_pair_kernel<true> : ln_bwd_pair_kernel<false>;
  static PerDeviceFlag configured[2];  // one per kernel
  if (!configured[fullw].test(ctx->device)) {
    LEGO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->smem_optin - 1024));
    configured[fullw].set(ctx->device);
  }
  const size_t budget = (size_t)ctx->smem_optin - 1024 - sizeof(BwdPairCtl) - 128 - half_slot;
  int stages = (int)(budget / slot);
  if (stages > kBwd1Ring) stages = kBwd1Ring;
  if (stages < 3) return LEGO_ERR_UNSUPPORTED;
  const size_t smem = (size_t)stages * slot + half_slot + sizeof(BwdPairCtl) + 128;
  int pairs = ctx->sm_count / 2;
  if (pairs > P.rows) pairs = (int)P.rows;
  if (pairs < 1) return LEGO_ERR_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kBwd1Consumers + 64);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters < 1) {
    (void)cudaGetLastError();
    return LEGO_ERR_UNSUPPORTED;
  }
  if (pairs > max_clusters) {  // every pair must be resident: the grid is persistent
    pairs = max_clusters;
    cfg.gridDim = dim3(2 * pairs);
  }
  P.partial_rows = pairs;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, P, stages, col_half, ctx->status_word);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return cuda_status(e);
}

// ---- bulk-copy pipelined dx kernel, several groups (rows of up to 3 Ki columns) ------
//
// One CTA per SM.  A producer thread streams x and dy into a shared-memory ring with 1-D
// bulk copies, `groups` CONSECUTIVE rows per ring slot: one copy of x, one of dy and two
// small ones for the rows' mean and rstd per slot, whatever the number of groups.  (With
// one slot per row the lone producer thread was the limit for narrow rows: four copies per
// row cost it about 0.4 us, which is what a row of 1 Ki columns took per SM.)  Up to 512
// consumer threads in 1 .. 8 groups: a group of cols / 16 threads (cols / 8 for the
// narrowest rows) takes one row of every slot, each of its threads owning 16 (8) fixed columns:
// (BLOCKS = false: one row per slot, group g takes rows g, g + groups, ... of the CTA, and the
// producer warp feeds the groups with one lane each, in lock step.  Groups that do not share a
// slot drift apart instead of waiting for the same barrier: rows of 3 Ki .. 5 Ki columns lost
// 6 - 10 % in the block form; it pays only for the narrowest rows, where even a lane per group
// cannot issue four copies per row fast enough.) gamma and the two column accumulators of those
// columns stay in registers for the whole kernel, a row costs one two-value reduction
// over the group (named barrier), and dx leaves in 128-bit streaming stores.  Every
// group ends with its own partial row of column sums.  All element-wise fp32 work is
// packed (f32x2).  Memory-level parallelism comes from the ring, not from occupancy.

constexpr int kBwdConsumers = 512;
constexpr int kBwdMaxGroups = 8;   // partial rows: 8 per SM (kMaxPartialRows)
constexpr int kBwdRing = 16;
constexpr long long kBwdWaitLimit = 2000000000LL;  // SM cycles, about a second

struct BwdRingCtl {
  uint64_t full[kBwdRing];
  uint64_t empty[kBwdRing];
  int64_t row[kBwdRing];
  uint64_t rowbar[kBwdMaxGroups][2];    // [group][row & 1]: the row's warp totals are all in red_all (or the threads' sums in part[])
  uint64_t totbar[kBwdMaxGroups][2];    // [group][row & 1]: the row's totals are in tot[] (one arrival: the group's folding warp)
  float2 tot[kBwdMaxGroups][4];         // [group][row & 3] -> the row's (s1, s2)
  uint32_t abort_flag;                  // any role gave up: polled inside every bounded wait
  uint32_t group_abort[kBwdMaxGroups];  // set by a thread of the group that gave up
};

// (ONE folding warp for all groups was slower than none, whether it served the groups in turn or
// polled their barriers and served whichever had a row ready; same box: 16384 x 4096 72.6 -> 77 us
// with two groups, 16384 x 2048 38.5 -> 57-60 us with four, 4096 x 1024 12.7 -> 18.6 us with eight.
// A folding warp per group: 16384 x 4096 72.7 -> 67.7 us (5.54 -> 5.95 TB/s), 16384 x 3072 63 ->
// 59.2 us, 4096 x 4096 23.1 -> 22.3 us; possible for up to three groups, see FOLDW.  Two folding
// warps for four groups, each serving two: 16384 x 2048 38.4 -> 41.7 us.)
// G: threads per group when known at compile time, 0 = taken from `gsize_rt`.
// FOLDW: one folding warp PER GROUP (after the producer's warp; up to three groups, so that no
// scheduler holds more than five warps) adds up the row sums the group's threads leave in part[],
// as in ln_bwd_ring1_kernel; without it every consumer folds its group's warp totals itself.
template <int EPT, int G, bool BLOCKS, bool FOLDW>
__global__ void __launch_bounds__(FOLDW ? 640 : kBwdConsumers + 32, 1)
ln_bwd_ring_kernel(const __grid_constant__ BwdParams P, int stages, int groups_rt, int gsize_rt, int lanes, int fold,
                   uint32_t* status) {
  constexpr int NV = EPT / 8;
  const int gsize = G > 0 ? G : gsize_rt;
  const int groups = G == kBwdConsumers ? 1 : groups_rt;
  constexpr int P2 = EPT / 2;  // packed pairs per thread and row
  extern __shared__ __align__(128) uint8_t bwd_smem[];
  __shared__ __align__(16) float2 red_all[kBwdMaxGroups][4][16];  // [group][row & 3][warp] -> (s1, s2)
  __shared__ __align__(16) float2 part[FOLDW ? 2 : 1][FOLDW ? kBwdConsumers : 1];  // [row & 1][thread] -> (s1, s2)
  const int cols = P.cols;
  const uint32_t row_bytes = (uint32_t)cols * 2u;
  const uint32_t half_slot = ((BLOCKS ? (uint32_t)groups : 1u) * row_bytes + 127u) & ~127u;  // the slot's rows of x (or of dy)
  const uint32_t slot_bytes = 2u * half_slot + 128u;  // x rows | dy rows | mean chunk (32 bytes), rstd chunk
  BwdRingCtl* ctl = reinterpret_cast<BwdRingCtl*>(bwd_smem + (size_t)stages * slot_bytes);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const int tid = threadIdx.x;
  const int n_consumers = groups * gsize;
  const int nw = gsize >> 5;  // warps per group
  // slot fills (blocks of `groups` consecutive rows, or single rows) are dealt to the CTAs round-robin
  const int per_fill = BLOCKS ? groups : 1;
  const int64_t n_blocks = (P.rows + per_fill - 1) / per_fill;
  const int64_t my_blocks = n_blocks > blockIdx.x ? (n_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), BLOCKS ? n_consumers >> 5 : nw);  // the warps that read a slot
    }
    ctl->abort_flag = 0;
    for (int g = 0; g < kBwdMaxGroups; ++g) {
      ctl->group_abort[g] = 0;
      ptx::mbar_init(ptx::smem_u32(&ctl->rowbar[g][0]), nw);
      ptx::mbar_init(ptx::smem_u32(&ctl->rowbar[g][1]), nw);
      ptx::mbar_init(ptx::smem_u32(&ctl->totbar[g][0]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->totbar[g][1]), 1);
    }
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  // partials of warps a group does not have: zero, so the fold below is a fixed tree
  for (int i = tid; i < kBwdMaxGroups * 4 * 16; i += blockDim.x) (&red_all[0][0][0])[i] = make_float2(0.f, 0.f);
  __syncthreads();
  ptx::launch_dependents();     // the column reduction (or the next op) may set itself up now
  ptx::grid_dependency_wait();  // global memory only once the previous grid is complete

  if (FOLDW && tid >= n_consumers + 32) {
    // ---------------- folding warps: warp g serves group g ----------------
    const int lane = tid & 31;
    const int g = (tid - n_consumers - 32) >> 5;
    const int64_t g_rows = BLOCKS ? my_blocks : (my_blocks > g ? (my_blocks - g + groups - 1) / groups : 0);
    for (int64_t j = 0; j < g_rows; ++j) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->rowbar[g][j & 1]), (uint32_t)((j >> 1) & 1), abort_flag,
                                  kBwdWaitLimit)) {
        *abort_flag = 1;
        atomicCAS(status, 0u, 0x7a000u | (uint32_t)g);
        return;
      }
      // lane l adds the sums of the group's threads l, l + 32, ... in order, then five shuffle levels
      float2 ss = make_float2(0.f, 0.f);
      for (int i = 0; i < nw; ++i) ss = ptx::add2(ss, part[FOLDW ? (j & 1) : 0][FOLDW ? g * gsize + 32 * i + lane : 0]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ss.x += __shfl_xor_sync(0xffffffffu, ss.x, o);
        ss.y += __shfl_xor_sync(0xffffffffu, ss.y, o);
      }
      if (lane == 0) {
        ctl->tot[g][j & 3] = ss;
        ptx::mbar_arrive(ptx::smem_u32(&ctl->totbar[g][j & 1]));  // release: the store above is visible to the waiters
      }
      __syncwarp();
    }
    return;
  }
  if (tid >= n_consumers) {
    // ---------------- producer: blocks in order, block n of this CTA into slot n mod stages ----------------
    if (!BLOCKS && lanes > 1) {
      // One row per slot, several groups: `lanes` (= groups) lanes in lock step, lane l feeding
      // group l -- their barrier polls and copy issues overlap instead of adding up in one thread.
      const int lane = tid - n_consumers;
      int slot0 = 0;
      uint32_t lap = 0;
      int64_t issued = 0;
      bool failed = false;
      for (int64_t base = 0; base < my_blocks; base += lanes) {
        const int64_t n = base + lane;
        const int sl = slot0 + lane;
        if (lane < lanes && n < my_blocks) {
          if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[sl]), (lap & 1) ^ 1, abort_flag, kBwdWaitLimit)) {
            *abort_flag = 1;
            atomicCAS(status, 0u, 0x60000u | (uint32_t)sl);
            failed = true;
          } else {
            const int64_t row = blockIdx.x + n * (int64_t)gridDim.x;
            ctl->row[sl] = row;
            const uint32_t full = ptx::smem_u32(&ctl->full[sl]);
            const uint32_t dst = ptx::smem_u32(bwd_smem + (size_t)sl * slot_bytes);
            const bool whole = (row | 3) < P.rows;
            if (!whole) stats_by_hand(bwd_smem + (size_t)sl * slot_bytes + 2u * half_slot, 64u, P, row);
            ptx::mbar_arrive_expect_tx(full, 2u * row_bytes + (whole ? 32u : 0u));
            ptx::bulk_load(dst, P.x + row * cols, row_bytes, full);
            ptx::bulk_load(dst + half_slot, P.dy + row * cols, row_bytes, full);
            if (whole) {
              ptx::bulk_load(dst + 2u * half_slot, P.mean + (row & ~3LL), 16u, full);
              ptx::bulk_load(dst + 2u * half_slot + 64u, P.rstd + (row & ~3LL), 16u, full);
            }
          }
        }
        if (__any_sync(0xffffffffu, failed)) break;
        issued = base + lanes < my_blocks ? base + lanes : my_blocks;
        slot0 += lanes;
        if (slot0 == stages) {
          slot0 = 0;
          ++lap;
        }
      }
      if (*abort_flag && lane == 0) {
        // leave no copy of ours in flight
        uint32_t never = 0;
        for (int sl = 0; sl < stages; ++sl) {
          const int64_t uses = issued > sl ? (issued - sl + stages - 1) / stages : 0;
          if (uses) ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[sl]), (uint32_t)((uses - 1) & 1), &never, kBwdWaitLimit);
        }
      }
      return;
    }
    if (tid == n_consumers) {
      int64_t issued = 0;
      int s = 0;
      uint32_t use = 0;
      for (int64_t n = 0; n < my_blocks; ++n, s = (s + 1 == stages ? 0 : s + 1), use += (s == 0)) {
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[s]), (use & 1) ^ 1, abort_flag, kBwdWaitLimit)) {
          *abort_flag = 1;
          atomicCAS(status, 0u, 0x60000u | (uint32_t)s);
          break;
        }
        const int64_t row0 = (blockIdx.x + n * (int64_t)gridDim.x) * per_fill;
        const int64_t left = P.rows - row0;
        const uint32_t bytes = (uint32_t)(left < per_fill ? left : per_fill) * row_bytes;
        // the rows' statistics: the whole 16-byte chunks that hold rows row0 .. end - 1; the rows of a
        // last chunk that would reach past the arrays by plain loads
        const int64_t end = row0 + (left < per_fill ? left : per_fill);
        const int64_t chunk0 = row0 & ~3LL;
        const int64_t chunk_end = ((end + 3) & ~3LL) <= P.rows ? ((end + 3) & ~3LL) : (P.rows & ~3LL);
        const uint32_t stat_bytes = (uint32_t)(chunk_end - chunk0) * 4u;
        for (int64_t r = chunk_end > row0 ? chunk_end : row0; r < end; ++r) {
          float* st = reinterpret_cast<float*>(bwd_smem + (size_t)s * slot_bytes + 2u * half_slot);
          st[r - chunk0] = P.mean[r];
          st[16 + (r - chunk0)] = P.rstd[r];
        }
        ctl->row[s] = row0;
        const uint32_t full = ptx::smem_u32(&ctl->full[s]);
        const uint32_t dst = ptx::smem_u32(bwd_smem + (size_t)s * slot_bytes);
        ptx::mbar_arrive_expect_tx(full, 2u * bytes + 2u * stat_bytes);
        ptx::bulk_load(dst, P.x + row0 * cols, bytes, full);
        ptx::bulk_load(dst + half_slot, P.dy + row0 * cols, bytes, full);
        if (stat_bytes) {
          ptx::bulk_load(dst + 2u * half_slot, P.mean + chunk0, stat_bytes, full);
          ptx::bulk_load(dst + 2u * half_slot + 64u, P.rstd + chunk0, stat_bytes, full);
        }
        ++issued;
      }
      if (*abort_flag) {
        // leave no copy of ours in flight
        uint32_t never = 0;
        for (int sl = 0; sl < stages; ++sl) {
          const int64_t uses = issued > sl ? (issued - sl + stages - 1) / stages : 0;
          if (uses) ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[sl]), (uint32_t)((uses - 1) & 1), &never, kBwdWaitLimit);
        }
      }
    }
    return;
  }

  // ---------------- consumers: group g takes row g of every block of this CTA ----------------
  const int group = tid / gsize;
  const int gtid = tid - group * gsize;
  const int lane = tid & 31, warp_in_group = gtid >> 5;
  volatile uint32_t* group_abort = &ctl->group_abort[group];
  float2 g[P2], acc_w[P2], acc_b[P2];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = (k * gsize + gtid) * 8;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (c < cols) raw = __ldg(reinterpret_cast<const uint4*>(P.gamma + c));
    const __half2* hp = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) g[k * 4 + e] = __half22float2(hp[e]);
  }
#pragma unroll
  for (int k = 0; k < P2; ++k) acc_w[k] = acc_b[k] = make_float2(0.f, 0.f);
  const float inv_cols = 1.0f / (float)cols;

  // A row is handled in two phases with the group's next row's first phase in between (see
  // ln_bwd_ring1_kernel): the group-wide reduction of a row is in flight while its threads work
  // on the next row, and x and dy are read from the ring slot again for phase 2.
  float2 (*red)[16] = red_all[group];           // [row & 3][warp]
  uint64_t* rowbar = ctl->rowbar[group];        // [row & 1], nw arrivals
  bool alive = true;
  auto phase1 = [&](int64_t j, int s, uint32_t use) {   // j: this group's j-th row
    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), use & 1, abort_flag, kBwdWaitLimit)) {
      *abort_flag = 1;
      atomicCAS(status, 0u, 0x70000u | (uint32_t)s);
      alive = false;
      return;
    }
    const uint8_t* slot = bwd_smem + (size_t)s * slot_bytes;
    const int64_t row0 = ctl->row[s];
    const int64_t row = BLOCKS ? row0 + group : row0;
    const bool exists = !BLOCKS || row < P.rows;  // the last block of the matrix may hold fewer rows than groups
    const int at = (int)(row - (row0 & ~3LL));
    const float mean = exists ? reinterpret_cast<const float*>(slot + 2u * half_slot)[at] : 0.f;
    const float rstd = exists ? reinterpret_cast<const float*>(slot + 2u * half_slot + 64u)[at] : 0.f;
    const uint8_t* xrow = BLOCKS ? slot + (size_t)group * row_bytes : slot;
    // xhat = x * rstd - mean * rstd; columns past the end hold dy = 0 and gamma = 0, so they add nothing
    const float2 rstd2 = make_float2(rstd, rstd), shift2 = make_float2(-mean * rstd, -mean * rstd);
    float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int v = k * gsize + gtid;
      uint4 xr = make_uint4(0u, 0u, 0u, 0u), dr = make_uint4(0u, 0u, 0u, 0u);
      if (exists && v * 8 < cols) {
        xr = reinterpret_cast<const uint4*>(xrow)[v];
        dr = reinterpret_cast<const uint4*>(xrow + half_slot)[v];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 d = __half22float2(reinterpret_cast<const __half2*>(&dr)[e]);
        const float2 h = ptx::fma2(__half22float2(reinterpret_cast<const __half2*>(&xr)[e]), rstd2, shift2);
        acc_w[k * 4 + e] = ptx::fma2(d, h, acc_w[k * 4 + e]);
        acc_b[k * 4 + e] = ptx::add2(acc_b[k * 4 + e], d);
        const float2 w = ptx::mul2(d, g[k * 4 + e]);
        s1 = ptx::fma2(h, w, s1);
        s2 = ptx::add2(s2, w);
      }
    }
    // even lanes fold the first sum, odd lanes the second: one shuffle per level instead of two
    const float a = s1.x + s1.y, bsum = s2.x + s2.y;
    if (FOLDW) {
      part[FOLDW ? (j & 1) : 0][FOLDW ? tid : 0] = make_float2(a, bsum);  // the group's folding warp adds them up
    } else {
      const bool odd = (lane & 1) != 0;
      float keep = odd ? bsum : a;
      keep += __shfl_xor_sync(0xffffffffu, odd ? a : bsum, 1);
#pragma unroll
      for (int o = 2; o <= 16; o <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
      if (lane < 2) reinterpret_cast<float*>(&red[j & 3][warp_in_group])[lane] = keep;
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&rowbar[j & 1]));
  };
  auto phase2 = [&](int64_t j, int s) {
    if (!ptx::mbar_wait_bounded(ptx::smem_u32(FOLDW ? &ctl->totbar[group][j & 1] : &rowbar[j & 1]), (uint32_t)((j >> 1) & 1),
                                abort_flag, kBwdWaitLimit)) {
      *abort_flag = 1;
      atomicCAS(status, 0u, (FOLDW ? 0x7c000u : 0x78000u) | (uint32_t)s);
      alive = false;
      return;
    }
    float2 ss;
    const float2* r = red[j & 3];
    if (FOLDW) {
      ss = ctl->tot[group][j & 3];  // folded once for the group by its folding warp
    } else if (nw > 8) {
      // 16 partials: both half-warps fold the same 16 values by shuffles (few registers)
      ss = r[lane & 15];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        ss.x += __shfl_xor_sync(0xffffffffu, ss.x, o);
        ss.y += __shfl_xor_sync(0xffffffffu, ss.y, o);
      }
    } else {
      // up to 8 partials (absent warps hold zeros): a fixed tree over four 128-bit loads
      const float4* q = reinterpret_cast<const float4*>(r);
      const float4 a0 = q[0], a1 = q[1], a2 = q[2], a3 = q[3];
      ss.x = ((a0.x + a0.z) + (a1.x + a1.z)) + ((a2.x + a2.z) + (a3.x + a3.z));
      ss.y = ((a0.y + a0.w) + (a1.y + a1.w)) + ((a2.y + a2.w) + (a3.y + a3.w));
    }
    const uint8_t* slot = bwd_smem + (size_t)s * slot_bytes;
    const int64_t row0 = ctl->row[s];
    const int64_t row = BLOCKS ? row0 + group : row0;
    const bool exists = !BLOCKS || row < P.rows;
    const int at = (int)(row - (row0 & ~3LL));
    const float mean = exists ? reinterpret_cast<const float*>(slot + 2u * half_slot)[at] : 0.f;
    const float rstd = exists ? reinterpret_cast<const float*>(slot + 2u * half_slot + 64u)[at] : 0.f;
    const uint8_t* xrow = BLOCKS ? slot + (size_t)group * row_bytes : slot;
    const float2 rstd2 = make_float2(rstd, rstd), shift2 = make_float2(-mean * rstd, -mean * rstd);
    // dx = (wdy - (xhat * c1 + c2)) * rstd, as two fused steps per pair
    const float c1r = ss.x * inv_cols * rstd, c2r = ss.y * inv_cols * rstd;
    const float2 nc1 = make_float2(-c1r, -c1r), nc2 = make_float2(-c2r, -c2r);
    __half* __restrict__ dx = P.dx + row * cols;
    uint4 outv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int v = k * gsize + gtid;
      uint4 xr = make_uint4(0u, 0u, 0u, 0u), dr = make_uint4(0u, 0u, 0u, 0u);
      if (exists && v * 8 < cols) {
        xr = reinterpret_cast<const uint4*>(xrow)[v];
        dr = reinterpret_cast<const uint4*>(xrow + half_slot)[v];
      }
      __half2* o2 = reinterpret_cast<__half2*>(&outv[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 d = __half22float2(reinterpret_cast<const __half2*>(&dr)[e]);
        const float2 h = ptx::fma2(__half22float2(reinterpret_cast<const __half2*>(&xr)[e]), rstd2, shift2);
        const float2 w = ptx::mul2(d, g[k * 4 + e]);
        const float2 t = ptx::fma2(h, nc1, ptx::fma2(w, rstd2, nc2));
        o2[e] = __floats2half2_rn(t.x, t.y);
      }
    }
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[s]));  // slot may be refilled now
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * gsize + gtid) * 8;
      if (exists && c < cols) __stcs(reinterpret_cast<uint4*>(dx + c), outv[k]);
    }
  };

  // Ring cursors of the group's row in phase 1 (s1, use1) and in phase 2 (s2).  BLOCKS: every
  // group walks every slot (at least three slots).  Else group g walks slots g, g + groups, ...;
  // the slot count is a multiple of the group count and at least twice it.  Either way the two
  // rows sit in different slots.
  const int step = BLOCKS ? 1 : groups;
  const int64_t group_rows = BLOCKS ? my_blocks : (my_blocks > group ? (my_blocks - group + groups - 1) / groups : 0);
  int s1 = BLOCKS ? 0 : group, s2 = s1;
  uint32_t use1 = 0;
  if (group_rows > 0) phase1(0, s1, use1);
  for (int64_t j = 0; alive && j < group_rows; ++j) {
    if (j + 1 < group_rows) {
      s1 += step;
      if (s1 >= stages) { s1 -= stages; ++use1; }
      phase1(j + 1, s1, use1);
      if (!alive) break;
    }
    phase2(j, s2);
    s2 += step;
    if (s2 >= stages) s2 -= stages;
  }
  if (!alive) *group_abort = 1;
  if (fold) {
    // The groups' column sums are added up inside the CTA, in group order, and ONE partial row per
    // CTA goes to global memory: with eight groups their own rows were a third of the kernel's
    // traffic.  The sums are parked in the ring's memory, which is free once EVERY group has left
    // its loop (first barrier: every copy has landed and every slot has been read by then); every
    // consumer thread reaches the barriers, also those of a group that gave up.
    asm volatile("bar.sync 1, %0;" ::"r"(n_consumers) : "memory");
    float* fw = reinterpret_cast<float*>(bwd_smem) + (size_t)group * 2 * cols;
    float* fb = fw + cols;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = (k * gsize + gtid) * 8;
      if (c < cols) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = k * 4 + 2 * e;
          *reinterpret_cast<float4*>(fw + c + 4 * e) = make_float4(acc_w[j].x, acc_w[j].y, acc_w[j + 1].x, acc_w[j + 1].y);
          *reinterpret_cast<float4*>(fb + c + 4 * e) = make_float4(acc_b[j].x, acc_b[j].y, acc_b[j + 1].x, acc_b[j + 1].y);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"r"(n_consumers) : "memory");
    if (*abort_flag) return;
    const float4* all = reinterpret_cast<const float4*>(bwd_smem);
    const int quads = cols >> 2;  // float4 columns of one array
    float* pw = P.partial + (size_t)blockIdx.x * cols;
    float* pb = P.partial + ((size_t)P.partial_rows + blockIdx.x) * cols;
    for (int i = tid; i < 2 * quads; i += n_consumers) {
      const int arr = i >= quads ? 1 : 0, q = i - arr * quads;
      float4 acc = all[(size_t)arr * quads + q];
      for (int g2 = 1; g2 < groups; ++g2) {
        const float4 v = all[((size_t)g2 * 2 + arr) * quads + q];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      *reinterpret_cast<float4*>((arr ? pb : pw) + 4 * q) = acc;
    }
    return;
  }
  if (*group_abort) return;
  // this group's partial row of column sums
  const size_t prow = (size_t)blockIdx.x * groups + group;
  float* pw = P.partial + prow * cols;
  float* pb = P.partial + ((size_t)P.partial_rows + prow) * cols;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = (k * gsize + gtid) * 8;
    if (c < cols) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int j = k * 4 + 2 * e;
        *reinterpret_cast<float4*>(pw + c + 4 * e) = make_float4(acc_w[j].x, acc_w[j].y, acc_w[j + 1].x, acc_w[j + 1].y);
        *reinterpret_cast<float4*>(pb + c + 4 * e) = make_float4(acc_b[j].x, acc_b[j].y, acc_b[j + 1].x, acc_b[j + 1].y);
      }
    }
  }
}

// Launches the ring kernel when the shape suits it; LEGO_ERR_UNSUPPORTED otherwise.
template <int EPT, int G, bool BLOCKS, bool FOLDW>
int32_t launch_ring_dx_g(const BwdParams& P, DeviceCtx* ctx, cudaStream_t s, int grid, int stages, int groups, int gsize,
                         size_t smem, int fold) {
  auto kern = ln_bwd_ring_kernel<EPT, G, BLOCKS, FOLDW>;
  static PerDeviceFlag configured;
  if (!configured.test(ctx->device)) {
    // static part: 4 KiB of reduction slots, with folding warps 8 KiB of row sums too
    LEGO_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ctx->smem_optin - (FOLDW ? 16384 : 8192)));
    configured.set(ctx->device);
  }
  const cudaError_t e = launch_overlapped(kern, dim3(grid), dim3(groups * gsize + 32 + (FOLDW ? 32 * groups : 0)), smem, s, P, stages,
                                          groups, gsize, g_lnbwd_lanes.load() && !BLOCKS && groups > 1 ? groups : 1, fold,
                                          ctx->status_word);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return cuda_status(e);
}

template <int EPT>
int32_t launch_ring_dx(BwdParams& P, DeviceCtx* ctx, cudaStream_t s) {
  // threads per row: EPT columns each, whole warps; as many groups as fit into 512 threads
  int gsize = (((P.cols + EPT - 1) / EPT) + 31) & ~31;
  if (gsize > kBwdConsumers) return LEGO_ERR_UNSUPPORTED;
  int groups = kBwdConsumers / gsize;
  if (groups > kBwdMaxGroups) groups = kBwdMaxGroups;
  const int64_t rows_cap = P.rows < ctx->sm_count ? P.rows : ctx->sm_count;
  // one partial row per group and CTA: no more than the caller's scratch holds
  const int64_t room = (P.rows < kMaxPartialRows ? P.rows : kMaxPartialRows) / rows_cap;
  if (groups > room) groups = (int)room;
  if (groups < 1) return LEGO_ERR_UNSUPPORTED;
  // How the producer keeps up with narrow rows (16384 rows, same box, us per launch: one thread and
  // a slot per row / a block of `groups` rows per slot / a producer lane per group, slot per row):
  // N = 1024 (8 groups) 43.2 / 28.4 / 36.1; N = 2048 (4 groups) 47.9 / 43.5 / 40.8; N = 1536 (5) - /
  // 35.4 / 35.8; 4096 rows: N = 1024 17.1 / 16.3 / 15.4, N = 2048 18.6 / - / 16.3.  So: blocks for
  // eight groups when a CTA has many rows to go through, lanes otherwise.
  const bool blocks = g_lnbwd_lanes.load() < 2 && groups >= 8 && P.rows >= 64 * (int64_t)ctx->sm_count;
  const int per_fill = blocks ? groups : 1;
  const int64_t fills = (P.rows + per_fill - 1) / per_fill;
  const int grid = (int)(fills < ctx->sm_count ? fills : ctx->sm_count);
  const size_t half_slot = ((size_t)per_fill * P.cols * 2 + 127) & ~(size_t)127;
  const size_t slot = 2 * half_slot + 128;
  // a folding warp per group while consumers, producer and folding warps make 20 warps or fewer (five
  // per scheduler, 96 registers); their 8 KiB of row sums come out of the ring's memory
  const bool foldw = !blocks && groups <= g_lnbwd_foldw_groups.load() && groups * gsize + 32 + 32 * groups <= 640;
  const size_t budget = (size_t)ctx->smem_optin - (foldw ? 16384 : 8192) - sizeof(BwdRingCtl) - 128;
  int stages = (int)((192 * 1024 + slot / 2) / slot);  // about 192 KiB of x and dy in flight
  const int least = blocks ? 3 : 2 * groups;  // the rows in phase 1 and phase 2 hold a slot each (per group)
  if (stages < least) stages = least;
  if (stages > kBwdRing) stages = kBwdRing;
  if ((size_t)stages > budget / slot) stages = (int)(budget / slot);
  if (!blocks) stages -= stages % groups;  // a slot always belongs to one group
  if (stages < least) return LEGO_ERR_UNSUPPORTED;
  const size_t smem = (size_t)stages * slot + sizeof(BwdRingCtl) + 128;
  // several groups: their column sums are folded in the ring's memory at the end, one partial row per CTA
  const int fold = (groups > 1 && P.cols % 4 == 0 && (size_t)groups * 2 * P.cols * 4 <= (size_t)stages * slot &&
                    g_lnbwd_fold.load()) ? 1 : 0;
  P.partial_rows = fold ? grid : grid * groups;  // every group writes its row, all zeros if it saw no row of x
  if (blocks) return launch_ring_dx_g<EPT, 0, true, false>(P, ctx, s, grid, stages, groups, gsize, smem, fold);
  return foldw ? launch_ring_dx_g<EPT, 0, false, true>(P, ctx, s, grid, stages, groups, gsize, smem, fold)
               : launch_ring_dx_g<EPT, 0, false, false>(P, ctx, s, grid, stages, groups, gsize, smem, fold);
}

// Column reduction for widths that are a multiple of 4: a CTA of 32 warps sums 32 columns;
// lane (q, r) of warp w reads the 16 bytes of column quad q in partial rows r + 4 w,
// + 128, ... (a warp reads four whole 128-byte lines per step, and with the usual 148
// partial rows no thread waits for more than two loads in a row), the 128 row lanes are
// folded by shuffles and one pass through shared memory, always in the same order.
__global__ void __launch_bounds__(1024)
ln_bwd_reduce4_kernel(const float* __restrict__ partial, __half* __restrict__ dgamma, __half* __restrict__ dbeta,
                      int cols, int partial_rows) {
  __shared__ float4 sw[32][8], sb[32][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q = lane & 7, rl = (lane >> 3) + 4 * warp;
  const int c = blockIdx.x * 32 + q * 4;
  float4 w = make_float4(0.f, 0.f, 0.f, 0.f), b = w;
  ptx::launch_dependents();
  ptx::grid_dependency_wait();  // the partial rows are complete and visible after this
  if (c < cols) {
#pragma unroll 2
    for (int r = rl; r < partial_rows; r += 128) {
      const float4 pw = __ldcs(reinterpret_cast<const float4*>(partial + (size_t)r * cols + c));
      const float4 pb = __ldcs(reinterpret_cast<const float4*>(partial + ((size_t)partial_rows + r) * cols + c));
      w.x += pw.x; w.y += pw.y; w.z += pw.z; w.w += pw.w;
      b.x += pb.x; b.y += pb.y; b.z += pb.z; b.w += pb.w;
    }
  }
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
    w.x += __shfl_xor_sync(0xffffffffu, w.x, o); w.y += __shfl_xor_sync(0xffffffffu, w.y, o);
    w.z += __shfl_xor_sync(0xffffffffu, w.z, o); w.w += __shfl_xor_sync(0xffffffffu, w.w, o);
    b.x += __shfl_xor_sync(0xffffffffu, b.x, o); b.y += __shfl_xor_sync(0xffffffffu, b.y, o);
    b.z += __shfl_xor_sync(0xffffffffu, b.z, o); b.w += __shfl_xor_sync(0xffffffffu, b.w, o);
  }
  if (lane < 8) {
    sw[warp][q] = w;
    sb[warp][q] = b;
  }
  __syncthreads();
  if (warp == 0 && lane < 8 && c < cols) {
    float4 tw = sw[0][q], tb = sb[0][q];
#pragma unroll
    for (int k = 1; k < 32; ++k) {
      tw.x += sw[k][q].x; tw.y += sw[k][q].y; tw.z += sw[k][q].z; tw.w += sw[k][q].w;
      tb.x += sb[k][q].x; tb.y += sb[k][q].y; tb.z += sb[k][q].z; tb.w += sb[k][q].w;
    }
    __half2* dg = reinterpret_cast<__half2*>(dgamma + c);
    __half2* dbp = reinterpret_cast<__half2*>(dbeta + c);
    dg[0] = __floats2half2_rn(tw.x, tw.y);
    dg[1] = __floats2half2_rn(tw.z, tw.w);
    dbp[0] = __floats2half2_rn(tb.x, tb.y);
    dbp[1] = __floats2half2_rn(tb.z, tb.w);
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
  if (P.cols <= 1024 * 16) return launch_dx<1024, 16, VECTOR>(P, s);  // half the registers of the next one
  if (P.cols <= 1024 * 32) return launch_dx<1024, 32, VECTOR>(P, s);
  return LEGO_ERR_UNSUPPORTED;
}

int64_t partial_rows_for(int64_t rows) { return rows < kMaxPartialRows ? rows : kMaxPartialRows; }

}  // namespace
extern std::atomic<int> g_lnbwd_split;
namespace {

}  // namespace
}  // namespace lego

namespace lego {
std::atomic<int> g_lnbwd_split{4096};  // rows wider than this take the one-group kernel
}

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
  int32_t st = LEGO_ERR_UNSUPPORTED;
  int32_t err = LEGO_OK;
  DeviceCtx* ctx = device_ctx(&err);
  if (!ctx) return err;
  // Ring-fed kernels: 16-byte aligned rows of 1 Ki .. 32 Ki columns, any number of rows (the rows'
  // statistics travel in 16-byte chunks; the last rows & 3 rows, whose chunk would reach past the
  // arrays, get theirs by plain loads -- the reference's own test shape has 1151 rows).
  // (Rows of 8 Ki .. 16 Ki columns, 8192 rows, same box: 24 / 32 columns per thread with gamma in
  // shared memory 3.2 - 4.9 TB/s; the register kernel they ran on before 1.1; the library kernel 2.1.
  // Few rows, us per call, ring kernels / register kernel / library: 256 x 4096 7.3 / 16.4 / 7.7,
  // 100 x 8192 9.1 / 17.2 / 11.2, 64 x 4096 5.9 / 9.0 / 6.3, 12 x 1024 3.9 / 5.2 / 4.4.)
  if (vec && cols >= 1024 && cols <= kBwdConsumers * 64 && rows >= g_lnbwd_min_rows.load() && a16(mean) && a16(rstd) &&
      a16(partial)) {
    const int32_t room = P.partial_rows;
    // Same box, GB/s, 16384 rows, both kernels with rows in two phases: one group of 512 threads /
    // groups of cols/16 threads: N = 2048: 2010 / 4180, N = 4096: 3850 / 5350, N = 6144: 4160 / 4670,
    // N = 8192: 5500 / 5250.
    // (The pair kernel with 16 columns per thread for rows of 12 Ki .. 16 Ki columns, six ring slots
    // instead of three: 8192 x 16384 157 -> 233 us, same box.  A pair turns one row around in about
    // 2.1 us whatever its width -- the round trip of the row sums between the two CTAs, of which only
    // one first phase is covered -- so it pays only where one CTA cannot hold the row.)
    if (cols > kBwd1Consumers * 32) st = launch_pair_dx(P, ctx, s);
    else if (cols > kBwd1Consumers * 16) st = cols <= kBwd1Consumers * 24 ? launch_ring1_dx<24>(P, ctx, s) : launch_ring1_dx<32>(P, ctx, s);
    else if (cols > g_lnbwd_split.load()) st = cols <= kBwd1Consumers * 8 ? launch_ring1_dx<8>(P, ctx, s) : launch_ring1_dx<16>(P, ctx, s);
    else st = launch_ring_dx<16>(P, ctx, s);
    if (st == LEGO_ERR_UNSUPPORTED) P.partial_rows = room;
  }
  if (st == LEGO_ERR_UNSUPPORTED) st = vec ? launch_dx_by_cols<true>(P, s) : launch_dx_by_cols<false>(P, s);
  if (st != LEGO_OK) return st;
  if (cols % 4 == 0 && a16(partial) && ((uintptr_t)dgamma & 3) == 0 && ((uintptr_t)dbeta & 3) == 0) {
    const cudaError_t e = launch_overlapped(ln_bwd_reduce4_kernel, dim3((unsigned)((cols + 31) / 32)), dim3(1024), 0, s,
                                            (const float*)partial, (__half*)dgamma, (__half*)dbeta, (int)cols,
                                            (int)P.partial_rows);
    if (e != cudaSuccess) (void)cudaGetLastError();
    return cuda_status(e);
  }
  ln_bwd_reduce_kernel<<<(unsigned)((cols + 31) / 32), 256, 0, s>>>(partial, (__half*)dgamma, (__half*)dbeta,
                                                                 (int)cols, P.partial_rows);
  return cuda_status(cudaGetLastError());
}

}  // extern "C"
