// Index-map evaluator: GroupBy.apply / GroupBy.inv over arrays of indices and
// over ranges of logical ids, as device-side integer arithmetic.
//
// A layout that folds runs as a digit-sum program (a handful of strength-reduced
// divide / wrap / multiply-add terms, 32-bit when the index space allows); any
// other layout runs the staged interpreter, which re-cuts and permutes the flat
// id stage by stage in 64-bit arithmetic exactly as lego/lego.py:388-433 does.
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "staged.cuh"

namespace lego {

enum { MODE_RANGE = 0, MODE_APPLY = 1, MODE_INV = 2 };

template <bool WIDE>
__device__ __forceinline__ uint64_t term_value(const DigitTerm& t, uint64_t x) {
  if (WIDE) {
    uint64_t q = t.a64 > 1 ? x / t.a64 : x;
    if (t.m64) q %= t.m64;
    return q * t.b;
  } else {
    uint32_t q = fd_div((uint32_t)x, t.a);
    if (t.m.d) q -= fd_div(q, t.m) * t.m.d;
    return (uint64_t)(q * (uint32_t)t.b);
  }
}

template <bool WIDE, int MODE>
__global__ void __launch_bounds__(256)
digit_eval_kernel(const __grid_constant__ DigitProgram p, const int64_t* __restrict__ in,
                  int64_t* __restrict__ out, int64_t begin, int64_t n) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    if (MODE == MODE_INV) {
      const uint64_t x = (uint64_t)in[i];
      uint64_t acc[LEGO_MAX_RANK];
#pragma unroll
      for (int k = 0; k < LEGO_MAX_RANK; ++k) acc[k] = 0;
      for (int j = 0; j < p.n_terms; ++j) {
        const uint64_t v = term_value<WIDE>(p.t[j], x);
        const int dst = p.t[j].dst;
#pragma unroll
        for (int k = 0; k < LEGO_MAX_RANK; ++k)
          if (k == dst) acc[k] += v;
      }
#pragma unroll
      for (int k = 0; k < LEGO_MAX_RANK; ++k)
        if (k < p.n_dst) out[i * p.n_dst + k] = (int64_t)acc[k];
    } else {
      uint64_t acc = 0;
      if (MODE == MODE_RANGE) {
        const uint64_t x = (uint64_t)(begin + i);
        for (int j = 0; j < p.n_terms; ++j) acc += term_value<WIDE>(p.t[j], x);
      } else {
        const int64_t* row = in + i * p.n_src;
        for (int j = 0; j < p.n_terms; ++j) acc += term_value<WIDE>(p.t[j], (uint64_t)row[p.t[j].src]);
      }
      out[i] = (int64_t)acc;
    }
  }
}

// Range evaluation for the common case (32-bit index space, at most kFastTerms digits):
// the terms live in registers, every thread produces two consecutive ids and writes them
// as one 16-byte store, so the kernel is bound by the int64 output stream, not by
// fetching term fields from the parameter bank for every index.
constexpr int kFastTerms = 6;

__global__ void __launch_bounds__(256)
digit_range_fast_kernel(const __grid_constant__ DigitProgram p, int64_t* __restrict__ out, int64_t begin, int64_t n) {
  uint32_t a_mul[kFastTerms], a_shr[kFastTerms], m_mul[kFastTerms], m_shr[kFastTerms], m_d[kFastTerms], b[kFastTerms];
#pragma unroll
  for (int j = 0; j < kFastTerms; ++j) {
    const bool on = j < p.n_terms;
    a_mul[j] = on ? p.t[j].a.mul : 0u;
    a_shr[j] = on ? p.t[j].a.shr : 0u;
    m_mul[j] = on ? p.t[j].m.mul : 0u;
    m_shr[j] = on ? p.t[j].m.shr : 0u;
    m_d[j] = on ? p.t[j].m.d : 0u;
    b[j] = on ? (uint32_t)p.t[j].b : 0u;   // a disabled term multiplies by zero
  }
  auto eval = [&](uint32_t x) {
    uint32_t acc = 0;
#pragma unroll
    for (int j = 0; j < kFastTerms; ++j) {
      uint32_t q = a_mul[j] ? (__umulhi(x, a_mul[j]) >> a_shr[j]) : (x >> a_shr[j]);
      if (m_d[j]) {
        const uint32_t w = m_mul[j] ? (__umulhi(q, m_mul[j]) >> m_shr[j]) : (q >> m_shr[j]);
        q -= w * m_d[j];
      }
      acc += q * b[j];
    }
    return (int64_t)acc;
  };
  const int64_t pairs = n >> 1;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += step) {
    const uint32_t x = (uint32_t)(begin + 2 * i);
    const int64_t v0 = eval(x), v1 = eval(x + 1);
    if (aligned) {
      *reinterpret_cast<longlong2*>(out + 2 * i) = make_longlong2(v0, v1);
    } else {
      out[2 * i] = v0;
      out[2 * i + 1] = v1;
    }
  }
  if ((n & 1) && blockIdx.x == 0 && threadIdx.x == 0) out[n - 1] = eval((uint32_t)(begin + n - 1));
}

// Range evaluation, one warp per 1024 consecutive ids.  Terms whose divisor is a multiple
// of 32 ("slow" terms) are constant over a 32-aligned run of ids: lane L evaluates their
// sum once for run L of the warp's 32 runs, and the sums travel by shuffle.  Only the
// remaining "fast" terms (normally just the innermost digit) are evaluated per id.  Each
// store instruction writes 64 consecutive int64 (512 contiguous bytes per warp).
constexpr int kWarpFast = 2;
constexpr int kWarpSlow = 6;

struct TermRegs {
  uint32_t a_mul, a_shr, m_mul, m_shr, m_d, b;
};

__device__ __forceinline__ TermRegs load_term(const DigitProgram& p, int j, bool on) {
  TermRegs r;
  r.a_mul = on ? p.t[j].a.mul : 0u;
  r.a_shr = on ? p.t[j].a.shr : 0u;
  r.m_mul = on ? p.t[j].m.mul : 0u;
  r.m_shr = on ? p.t[j].m.shr : 0u;
  r.m_d = on ? p.t[j].m.d : 0u;
  r.b = on ? (uint32_t)p.t[j].b : 0u;  // a disabled term multiplies by zero
  return r;
}

__device__ __forceinline__ uint32_t eval_term(const TermRegs& r, uint32_t x) {
  uint32_t q = r.a_mul ? (__umulhi(x, r.a_mul) >> r.a_shr) : (x >> r.a_shr);
  if (r.m_d) {
    const uint32_t w = r.m_mul ? (__umulhi(q, r.m_mul) >> r.m_shr) : (q >> r.m_shr);
    q -= w * r.m_d;
  }
  return q * r.b;
}

// `p` holds the fast terms first (n_fast of them), then the slow ones.
__global__ void __launch_bounds__(256)
digit_range_warp_kernel(const __grid_constant__ DigitProgram p, int n_fast, int64_t* __restrict__ out, int64_t begin,
                        int64_t n, int vec, int trigger_early, int resident_ctas) {
  TermRegs fast[kWarpFast], slow[kWarpSlow];
#pragma unroll
  for (int j = 0; j < kWarpFast; ++j) fast[j] = load_term(p, j, j < n_fast);
#pragma unroll
  for (int j = 0; j < kWarpSlow; ++j) slow[j] = load_term(p, n_fast + j, n_fast + j < p.n_terms);
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t block_end = (begin + n + 1023) >> 10;
  // Programmatic dependent launch.  A grid of a few waves triggers only after this CTA's last
  // store has been issued: triggering at the start lets the next grids of the stream (each of
  // which triggers at once, too) become resident on the SM slots this grid's own later CTAs
  // need -- 16 MiB of ids took 11.3 us that way against 4.4 us.  From about ten waves on the
  // early trigger wins (128 MiB: 21.9 against 22.8 us).
  // resident_ctas > 0 selects the other rule: only the CTAs of the grid's last wave trigger
  // early, and only after their own wait has returned -- the next grid then becomes resident
  // on the slots this grid frees as it drains, and at most one grid waits behind the running one.
  const bool last_wave = resident_ctas > 0 && (int64_t)blockIdx.x + resident_ctas >= (int64_t)gridDim.x;
  if (trigger_early && resident_ctas == 0) ptx::launch_dependents();
  ptx::grid_dependency_wait();  // stores only once the previous grid is complete
  if (last_wave) ptx::launch_dependents();
  for (int64_t blk = (begin >> 10) + warp; blk < block_end; blk += n_warps) {
    const uint32_t base = (uint32_t)(blk << 10);
    uint32_t run_sum = 0;
#pragma unroll
    for (int j = 0; j < kWarpSlow; ++j) run_sum += eval_term(slow[j], base + 32u * lane);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const uint32_t s = __shfl_sync(0xffffffffu, run_sum, 2 * k + (lane >> 4));
      const uint32_t x = base + 64u * k + 2u * lane;
      uint32_t v0 = s, v1 = s;
#pragma unroll
      for (int j = 0; j < kWarpFast; ++j) {
        v0 += eval_term(fast[j], x);
        v1 += eval_term(fast[j], x + 1);
      }
      const int64_t i = (int64_t)x - begin;
      if (vec && i >= 0 && i + 1 < n) {
        *reinterpret_cast<longlong2*>(out + i) = make_longlong2((int64_t)v0, (int64_t)v1);
      } else {
        if (i >= 0 && i < n) out[i] = (int64_t)v0;
        if (i + 1 >= 0 && i + 1 < n) out[i + 1] = (int64_t)v1;
      }
    }
  }
  if (resident_ctas > 0 ? !last_wave : !trigger_early) ptx::launch_dependents();
}

// inv over an array of flat positions, one thread per POSITION: a thread evaluates every term
// once (terms sorted by coordinate, in shared memory, read at warp-uniform addresses) and the
// warp turns its 32 x RANK coordinates through shared memory so that they leave as whole
// 16-byte words, 512 contiguous bytes per store instruction.  About a quarter of the
// instructions per position of the per-output-word form below, which is issue-bound
// (0.57 of the copy rate on 2^24 positions of a rank-4 layout).
// (Handing each warp's 256 x RANK contiguous bytes to the copy engine instead -- coordinates parked
// in output order, one cp.async.bulk shared -> global per 32 positions -- was slower: rank 4
// 126 against 115 us for 2^24 positions, rank 2 88 against 77.)
template <int RANK>
__global__ void __launch_bounds__(256)
digit_inv_rows_kernel(const __grid_constant__ DigitProgram p, const int64_t* __restrict__ in,
                      int64_t* __restrict__ out, int64_t n, int resident_ctas) {
  __shared__ __align__(16) int64_t turn[8][32 * RANK];
  // Term ranges per coordinate; the terms themselves are read from the parameter bank at
  // warp-uniform indices (no shared-memory or L1 traffic for them).
  int lo[RANK + 1];
  {
    int t = 0;
#pragma unroll
    for (int k = 0; k <= RANK; ++k) {
      while (t < p.n_terms && p.t[t].dst < k) ++t;
      lo[k] = t;
    }
  }
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  int64_t* mine = turn[wib];
  const bool last_wave = resident_ctas > 0 && (int64_t)blockIdx.x + resident_ctas >= (int64_t)gridDim.x;
  ptx::grid_dependency_wait();
  if (last_wave) ptx::launch_dependents();  // see digit_range_warp_kernel
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t runs = (n + 31) >> 5;
  constexpr int CHUNKS = RANK * 16;  // 16-byte words a full warp's coordinates make
  // Even ranks park whole 16-byte words; word w sits at w ^ ((w >> 3) & 1), which spreads a
  // quarter-warp's words (32 bytes apart for rank 4) over all eight 16-byte bank groups.
  constexpr bool PAIRS = RANK % 2 == 0;
  int64_t run = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  uint32_t x_next = 0;
  if (run < runs && run * 32 + lane < n) x_next = (uint32_t)in[run * 32 + lane];
  for (; run < runs; run += n_warps) {
    const uint32_t x = x_next;
    const int64_t nxt = (run + n_warps) * 32 + lane;
    if (nxt < n) x_next = (uint32_t)in[nxt];  // the next run's position is in flight while this one is decoded
    int64_t c[RANK];
#pragma unroll
    for (int k = 0; k < RANK; ++k) {
      uint32_t acc = 0;
      for (int t = lo[k]; t < lo[k + 1]; ++t) acc += eval_term(load_term(p, t, true), x);
      c[k] = (int64_t)acc;
    }
    const int64_t word0 = run * 32 * RANK;             // first output word of this run
    const int64_t words = (n - run * 32 < 32 ? n - run * 32 : 32) * RANK;
    if (PAIRS) {
#pragma unroll
      for (int h = 0; h < RANK / 2; ++h) {
        const int w = lane * (RANK / 2) + h;
        *reinterpret_cast<longlong2*>(mine + 2 * (w ^ ((w >> 3) & 1))) = make_longlong2(c[2 * h], c[2 * h + 1]);
      }
    } else {
#pragma unroll
      for (int k = 0; k < RANK; ++k) mine[lane * RANK + k] = c[k];
    }
    __syncwarp();
#pragma unroll
    for (int w = lane; w < CHUNKS; w += 32) {
      const int at = PAIRS ? 2 * (w ^ ((w >> 3) & 1)) : 2 * w;
      if (2 * w + 1 < words) {
        *reinterpret_cast<longlong2*>(out + word0 + 2 * w) = *reinterpret_cast<const longlong2*>(mine + at);
      } else if (2 * w < words) {
        out[word0 + 2 * w] = mine[at];
      }
    }
    __syncwarp();
  }
  if (!last_wave) ptx::launch_dependents();  // only now: see digit_range_warp_kernel
}

// inv over an array of flat positions, one thread per pair of OUTPUT words: output word e
// is coordinate e % rank of index e / rank, so a warp writes 512 contiguous bytes per store
// and a thread only evaluates the terms of its own coordinate (the terms arrive sorted by
// coordinate and sit in shared memory, because neighbouring lanes need different ones).
// The thread-per-index form writes rank words per thread at a stride of rank * 8 bytes and
// evaluates every term: 2.2 - 3.8 TB/s against this form's store-stream rate.
__global__ void __launch_bounds__(256)
digit_inv_flat_kernel(const __grid_constant__ DigitProgram p, FastDiv rank_div, const int64_t* __restrict__ in,
                      int64_t* __restrict__ out, int64_t n_out, int vec) {
  __shared__ TermRegs st[LEGO_MAX_TERMS];
  __shared__ int first[LEGO_MAX_RANK + 1];
  if (threadIdx.x < p.n_terms) st[threadIdx.x] = load_term(p, threadIdx.x, true);
  if (threadIdx.x == 0) {
    int t = 0;
    for (int k = 0; k <= p.n_dst; ++k) {
      while (t < p.n_terms && p.t[t].dst < k) ++t;
      first[k] = t;
    }
  }
  __syncthreads();
  const uint32_t rank = (uint32_t)p.n_dst;
  auto coord = [&](uint32_t k, uint32_t x) {
    uint32_t acc = 0;
    for (int t = first[k]; t < first[k + 1]; ++t) acc += eval_term(st[t], x);
    return (int64_t)acc;
  };
  ptx::grid_dependency_wait();
  const int64_t pairs = (n_out + 1) >> 1;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  // Four pairs per thread and step: their flat ids are loaded before the first is decoded, so a
  // thread has four independent chains in flight (one pair at a time ran at 0.62 of the copy peak).
  constexpr int U = 4;
  for (int64_t j0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j0 < pairs; j0 += U * step) {
    uint32_t e[U], i0[U], k0[U], x0[U], x1[U];
    bool wrap[U], live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t j = j0 + u * step;
      live[u] = j < pairs;
      e[u] = (uint32_t)(2 * (live[u] ? j : 0));
      i0[u] = fd_div(e[u], rank_div);
      k0[u] = e[u] - i0[u] * rank;
      wrap[u] = k0[u] + 1 == rank;
      x0[u] = live[u] ? (uint32_t)in[i0[u]] : 0u;
      x1[u] = (live[u] && wrap[u] && (int64_t)e[u] + 1 < n_out) ? (uint32_t)in[i0[u] + 1] : x0[u];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      const int64_t v0 = coord(k0[u], x0[u]);
      if ((int64_t)e[u] + 1 < n_out) {
        const int64_t v1 = coord(wrap[u] ? 0u : k0[u] + 1, x1[u]);
        if (vec) {
          *reinterpret_cast<longlong2*>(out + e[u]) = make_longlong2(v0, v1);
        } else {
          out[e[u]] = v0;
          out[e[u] + 1] = v1;
        }
      } else {
        out[e[u]] = v0;
      }
    }
  }
  ptx::launch_dependents();  // only now: see digit_range_warp_kernel
}

template <int MODE>
__global__ void __launch_bounds__(256)
staged_eval_kernel(const __grid_constant__ StagedProgram sp, const int64_t* __restrict__ in,
                   int64_t* __restrict__ out, int64_t begin, int64_t n) {
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    if (MODE == MODE_INV) {
      int64_t flat = staged_inv(sp, in[i]);
      for (int k = sp.rank - 1; k > 0; --k) {
        out[i * sp.rank + k] = flat % sp.dims[k];
        flat /= sp.dims[k];
      }
      out[i * sp.rank] = flat;
    } else {
      int64_t flat;
      if (MODE == MODE_RANGE) {
        flat = begin + i;
      } else {
        flat = 0;
        for (int k = 0; k < sp.rank; ++k) flat = flat * sp.dims[k] + in[i * sp.rank + k];
      }
      out[i] = staged_apply(sp, flat);
    }
  }
}

// lego_tune(LEGO_TUNE_PDL_LAST_WAVE): 1 = a grid of the index kernels that fills at most half of
// the machine lets the next grid of the stream become resident beside it (trigger after its own
// dependency wait), 0 = the grid-depth rule alone.  Same box, graph of 100 launches, us per launch
// of lego_eval_range without / with: 2^18 ids 3.18 / 2.89, 2^21 4.89 / 4.32, 2^22 7.93 / 7.36; a
// grid that nearly fills the machine must not do it (2^23 ids, 1024 CTAs on 1184 slots: 12.66 /
// 13.37 -- the waiting CTAs take the slots as they free up and end up unevenly spread).
std::atomic<int> g_pdl_last_wave{1};

// CTAs of `kernel` (256 threads, no dynamic shared memory) the current device holds at once, if a
// grid of `grid` CTAs leaves room for the next grid beside it; else 0 (the grid-depth rule applies).
template <typename K>
static int resident_ctas_of(K kernel, const DeviceCtx* ctx, int64_t grid) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  const int64_t resident = (int64_t)per_sm * ctx->sm_count;
  return 2 * grid <= resident ? (int)resident : 0;
}

template <int MODE>
static int32_t run_eval(const lego_layout_t* layout, const int64_t* in, int64_t* out, int64_t begin,
                        int64_t n, void* stream) {
  int64_t size = 0;
  int32_t st = check_layout(layout, &size);
  if (st != LEGO_OK) return st;
  if (n < 0) return LEGO_ERR_SIZE;
  if (MODE == MODE_RANGE && (begin < 0 || begin + n > size)) return LEGO_ERR_SIZE;
  if (n == 0) return LEGO_OK;  // nothing to do; empty buffers may be NULL
  if (!out || (MODE != MODE_RANGE && !in)) return LEGO_ERR_NULL;
  int32_t err = LEGO_OK;
  DeviceCtx* ctx = device_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  int64_t blocks64 = (n + threads - 1) / threads;
  const int64_t cap = (int64_t)ctx->sm_count * 16;
  const int blocks = (int)(blocks64 < cap ? blocks64 : cap);

  std::vector<Digit> dg;
  st = fold_layout(layout, &dg);
  if (st == LEGO_OK) {
    DigitProgram p;
    if (MODE == MODE_RANGE) program_range(dg, size, &p);
    if (MODE == MODE_APPLY) program_apply(dg, layout->rank, size, &p);
    if (MODE == MODE_INV) program_inv(dg, layout->rank, size, &p);
    if (MODE == MODE_RANGE && !p.wide && n >= 4096) {
      // fast terms first; a term is slow when its divisor is a multiple of 32
      DigitProgram w = p;
      int n_fast = 0, k = 0;
      for (int j = 0; j < p.n_terms; ++j)
        if (p.t[j].a.d % 32 != 0) w.t[k++] = p.t[j];
      n_fast = k;
      for (int j = 0; j < p.n_terms; ++j)
        if (p.t[j].a.d % 32 == 0) w.t[k++] = p.t[j];
      if (n_fast <= kWarpFast && p.n_terms - n_fast <= kWarpSlow) {
        const int64_t id_blocks = ((begin + n + 1023) >> 10) - (begin >> 10);
        const int64_t want = (id_blocks + 7) / 8, most = (int64_t)ctx->sm_count * 64;
        const int vec = (begin % 2 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) ? 1 : 0;
        const int early = want >= (int64_t)ctx->sm_count * 12 ? 1 : 0;
        const int resident =
            g_pdl_last_wave.load() ? resident_ctas_of(digit_range_warp_kernel, ctx, want < most ? want : most) : 0;
        const cudaError_t e = launch_overlapped(digit_range_warp_kernel, dim3((unsigned)(want < most ? want : most)),
                                                dim3(threads), 0, s, w, n_fast, out, begin, n, vec, early, resident);
        if (e != cudaSuccess) (void)cudaGetLastError();
        return cuda_status(e);
      }
    }
    if (MODE == MODE_INV && !p.wide && n * p.n_dst < ((int64_t)1 << 31) && n >= 4096) {
      // terms sorted by the coordinate they feed (stable: the sum order within a coordinate is kept)
      DigitProgram w = p;
      int k = 0;
      for (int d = 0; d < p.n_dst; ++d)
        for (int j = 0; j < p.n_terms; ++j)
          if (p.t[j].dst == d) w.t[k++] = p.t[j];
      const bool aligned16 = reinterpret_cast<uintptr_t>(out) % 16 == 0;
      if (k == p.n_terms && aligned16 && p.n_dst >= 2 && p.n_dst <= 4) {
        const int64_t want = (n + threads - 1) / threads, most = (int64_t)ctx->sm_count * 16;
        const dim3 grid((unsigned)(want < most ? want : most));
        cudaError_t e;
        const bool lw = g_pdl_last_wave.load() != 0;
        auto go = [&](auto kernel) {
          return launch_overlapped(kernel, grid, dim3(threads), 0, s, w, in, out, n,
                                   lw ? resident_ctas_of(kernel, ctx, (int64_t)grid.x) : 0);
        };
        if (p.n_dst == 2) e = go(digit_inv_rows_kernel<2>);
        else if (p.n_dst == 3) e = go(digit_inv_rows_kernel<3>);
        else e = go(digit_inv_rows_kernel<4>);
        if (e != cudaSuccess) (void)cudaGetLastError();
        return cuda_status(e);
      }
      if (k == p.n_terms) {
        const int64_t n_out = n * p.n_dst;
        const int64_t want = ((n_out + 1) / 2 + threads - 1) / threads, most = (int64_t)ctx->sm_count * 32;
        const int vec = reinterpret_cast<uintptr_t>(out) % 16 == 0 ? 1 : 0;
        const cudaError_t e = launch_overlapped(digit_inv_flat_kernel, dim3((unsigned)(want < most ? want : most)),
                                                dim3(threads), 0, s, w, make_fastdiv((uint64_t)p.n_dst), in, out, n_out, vec);
        if (e != cudaSuccess) (void)cudaGetLastError();
        return cuda_status(e);
      }
    }
    if (MODE == MODE_RANGE && !p.wide && p.n_terms <= kFastTerms)
      digit_range_fast_kernel<<<blocks, threads, 0, s>>>(p, out, begin, n);
    else if (p.wide)
      digit_eval_kernel<true, MODE><<<blocks, threads, 0, s>>>(p, in, out, begin, n);
    else
      digit_eval_kernel<false, MODE><<<blocks, threads, 0, s>>>(p, in, out, begin, n);
  } else if (st == LEGO_ERR_UNSUPPORTED) {
    StagedProgram sp;
    st = build_staged(layout, &sp);
    if (st != LEGO_OK) return st;
    staged_eval_kernel<MODE><<<blocks, threads, 0, s>>>(sp, in, out, begin, n);
  } else {
    return st;
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace lego

using namespace lego;

extern "C" {

int32_t lego_eval_apply(const lego_layout_t* layout, const int64_t* idx, int64_t* flat, int64_t n,
                        void* stream) {
  return run_eval<MODE_APPLY>(layout, idx, flat, 0, n, stream);
}

int32_t lego_eval_inv(const lego_layout_t* layout, const int64_t* flat, int64_t* idx, int64_t n,
                      void* stream) {
  return run_eval<MODE_INV>(layout, flat, idx, 0, n, stream);
}

int32_t lego_eval_range(const lego_layout_t* layout, int64_t begin, int64_t n, int64_t* flat_out,
                        void* stream) {
  return run_eval<MODE_RANGE>(layout, nullptr, flat_out, begin, n, stream);
}

}  // extern "C"
