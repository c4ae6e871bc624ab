// fp16 GEMM and grouped GEMM on tcgen05 tensor cores (sm_100a).
//
// One persistent CTA per SM walks a flat tile index; a LEGO layout's inverse maps
// that index to (tile_m, tile_n) -- the grouped swizzle of the reference's
// matmul_kernel -- and, for the grouped GEMM, a prefix table maps it to the
// problem first.  Inside a CTA the warps are specialised:
//   warp 0      TMA producer: 128x64 A and 256x64 B fp16 tiles, 128-byte swizzle,
//               4-stage ring in shared memory, completion on mbarriers;
//   warp 1      MMA issuer: tcgen05.mma kind::f16, M128 N256 K16, fp32
//               accumulators in TMEM, two 256-column buffers so the epilogue of
//               tile i overlaps the main loop of tile i+1;
//   warps 2..5  epilogue: tcgen05.ld -> activation -> fp16 -> global stores.
// Edges are handled by TMA zero fill on the loads and masks on the stores.
// Every wait is bounded: on expiry the CTA records a code in the status word,
// raises a CTA-wide abort flag, drains its own TMA loads, frees TMEM and returns.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstring>
#include <mutex>

#include "common.cuh"
#include "ptx_sm100.cuh"
#include "tma_host.cuh"

namespace lego {
namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SUB_BYTES = 64 * BK * 2;  // one 64 x 64 box of an MN-major fp16 operand

// A stage always holds 128 bytes of K per row: 64 fp16 or 128 fp8 values.  What depends
// on the element width: K values per stage, elements per 128-byte line of an MN-major
// box, the size of such a box (k rows x 128 bytes), and the descriptor step from one MMA
// to the next in an MN-major operand (MMA K rows x 128 bytes; 32 bytes when K-major).
struct Geometry {
  int bk, mn_box, sub_bytes;
  uint32_t mn_kstep;
};
__host__ __device__ __forceinline__ Geometry geometry_of(int elem8) {
  Geometry g;
  g.bk = elem8 ? 2 * BK : BK;
  g.mn_box = elem8 ? 128 : 64;
  g.sub_bytes = g.bk * 128;
  g.mn_kstep = (elem8 ? 4096u : 2048u) >> 4;
  return g;
}
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int EPI_STAGE_TOTAL = 4 * 2 * 32 * 64 * 2;  // epilogue staging, see EPI_BYTES
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_TOTAL + 1024 + 256;
constexpr long long WAIT_LIMIT = 2000000000LL;  // SM cycles, about a second

constexpr int kMaxOrderTerms = 8;
struct TileTerm { uint32_t a, m, b, dst; };  // coord[dst] += ((t / a) % m) * b; m == 0: no wrap
struct TileOrder { int32_t n_terms; int32_t reserved; TileTerm t[kMaxOrderTerms]; };

// Tensor maps that TMA reads from global memory must sit on 128-byte boundaries: with a
// 64-byte aligned record the maps of every second problem were fetched from the wrong
// line (results depended on the neighbouring record).  Hence the alignment and size.
struct alignas(128) Problem {
  CUtensorMap tma_a;
  CUtensorMap tma_b;
  CUtensorMap tma_c;    // C as [M rows][N contiguous], box 64 columns x 32 rows
  __half* c;
  int32_t m, n, k;
  int32_t tiles_m, tiles_n;
  int32_t tile_start;   // first flat tile id of this problem
  int32_t a_mn_major;   // 1: A stored [K, M] row-major
  int32_t b_mn_major;   // 1: B stored [K, N] row-major
  int32_t elem8;        // 1: A and B hold 8-bit floats (e5m2), 0: fp16
  TileOrder order;
};
static_assert(sizeof(Problem) == 640, "Problem must stay 640 bytes: the device tables are sized for it");

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

__device__ __forceinline__ void fail(uint32_t* status, volatile uint32_t* abort_flag, uint32_t code) {
  *abort_flag = 1;
  atomicCAS(status, 0u, code);
}

__host__ __device__ __forceinline__ void tile_coords(const Problem& p, int local, int* tm, int* tn) {
  if (p.order.n_terms == 0) {
    *tm = local / p.tiles_n;
    *tn = local % p.tiles_n;
    return;
  }
  uint32_t c0 = 0, c1 = 0;
  for (int j = 0; j < p.order.n_terms; ++j) {
    const TileTerm t = p.order.t[j];
    uint32_t q = (uint32_t)local / t.a;
    if (t.m) q %= t.m;
    q *= t.b;
    if (t.dst == 0) c0 += q; else c1 += q;
  }
  *tm = (int)c0;
  *tn = (int)c1;
}

// Epilogue staging: each of the four epilogue warps owns two 4 KiB buffers (32 rows x
// 128 bytes, 128-byte swizzle) and writes C with TMA stores, 64 columns at a time.
constexpr int EPI_CHUNK_COLS = 64;
constexpr int EPI_BUF_BYTES = 32 * EPI_CHUNK_COLS * 2;   // 4 KiB
constexpr int EPI_BYTES = 4 * 2 * EPI_BUF_BYTES;          // 32 KiB per CTA
static_assert(EPI_BYTES == EPI_STAGE_TOTAL, "staging size");

// One accumulator tile (this warp's 32 rows x 256 columns) -> activation -> fp16 ->
// swizzled shared memory -> TMA store.  Thread `lane` holds row q * 32 + lane; its eight
// 16-byte pieces of a 64-column chunk go to positions j ^ (lane & 7) of its row, so a
// quarter-warp writes eight distinct bank groups.  Full 128-byte lines reach L2, where the
// direct per-thread stores this replaces wrote 16-byte pieces of 32 different rows per
// instruction and cost about 40 us per 8192 x 8192 output.  `chunk_no` counts the chunks
// this warp has stored so far (selects the buffer; lane 0 keeps at most one store pending
// before a buffer is rewritten).
__device__ __forceinline__ void epilogue_store_tile(const Problem* p, int tm, int tn, int q, int lane,
                                                    uint32_t tmem_tile, uint8_t* warp_stage, int activation,
                                                    uint32_t* chunk_no, const Problem** fenced) {
  const int row0 = tm * BM + q * 32;
  if (row0 >= p->m) return;  // nothing of this warp's rows exists (warp-uniform)
  if (fenced && *fenced != p) {  // table-resident map: acquire once per problem
    if (lane == 0) ptx::tensormap_acquire(&p->tma_c);
    *fenced = p;
  }
#pragma unroll 1
  for (int c = 0; c < BN / EPI_CHUNK_COLS; ++c) {
    // Chunks past the last column are not staged at all: every staged chunk commits
    // exactly one bulk group, which is what the "at most one pending" wait below counts.
    const int col0 = tn * BN + c * EPI_CHUNK_COLS;
    if (col0 >= p->n) break;
    uint32_t r[64];
    ptx::tmem_ld_32x32(tmem_tile + c * EPI_CHUNK_COLS, r);
    ptx::tmem_ld_32x32(tmem_tile + c * EPI_CHUNK_COLS + 32, r + 32);
    uint8_t* buf = warp_stage + ((*chunk_no) & 1u) * EPI_BUF_BYTES;
    if (lane == 0) ptx::bulk_wait_group_read<1>();  // the store that last read this buffer is done with it
    __syncwarp();
    ptx::tmem_ld_wait();
    uint4* dst = reinterpret_cast<uint4*>(buf + lane * 128);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x0 = __uint_as_float(r[j * 8 + 2 * e]);
        float x1 = __uint_as_float(r[j * 8 + 2 * e + 1]);
        if (activation == LEGO_ACT_LEAKY_RELU) {
          x0 = x0 >= 0.f ? x0 : 0.01f * x0;
          x1 = x1 >= 0.f ? x1 : 0.01f * x1;
        }
        const __half2 hh = __floats2half2_rn(x0, x1);
        h[e] = *reinterpret_cast<const uint32_t*>(&hh);
      }
      dst[j ^ (lane & 7)] = make_uint4(h[0], h[1], h[2], h[3]);
    }
    ptx::fence_proxy_async();  // generic-proxy writes above -> visible to the TMA engine
    __syncwarp();
    if (lane == 0) {
      ptx::tma_store_2d(&p->tma_c, col0, row0, ptx::smem_u32(buf));
      ptx::bulk_commit_group();
    }
    ++(*chunk_no);
  }
}

template <bool GROUPED>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ Problem single, const Problem* __restrict__ table, int n_problems,
            int total_tiles, int activation, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(epi_stage + EPI_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&bars->tmem_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->tmem_empty[a]), 128);
    }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  auto problem_of = [&](int tile, int* cursor) -> const Problem* {
    if (!GROUPED) return &single;
    int g = *cursor;
    while (g + 1 < n_problems && tile >= table[g + 1].tile_start) ++g;
    *cursor = g;
    return &table[g];
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued[STAGES] = {0, 0, 0, 0};
      int cursor = 0;
      const Problem* fenced = nullptr;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const Problem* p = problem_of(tile, &cursor);
        if (GROUPED && p != fenced) {  // once per problem this CTA meets, not per tile
          ptx::tensormap_acquire(&p->tma_a);
          ptx::tensormap_acquire(&p->tma_b);
          fenced = p;
        }
        int tm, tn;
        tile_coords(*p, tile - p->tile_start, &tm, &tn);
        const Geometry geo = geometry_of(p->elem8);
        const int kblocks = (p->k + geo.bk - 1) / geo.bk;
        const bool a_mn = p->a_mn_major != 0, b_mn = p->b_mn_major != 0;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, WAIT_LIMIT)) {
            fail(status, abort_flag, 0x10000u | stage);
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&bars->full[stage]);
          const uint32_t a_dst = ptx::smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t b_dst = a_dst + A_BYTES;
          ptx::mbar_arrive_expect_tx(full, STAGE_BYTES);
          if (a_mn) {
            for (int j = 0; j < BM / geo.mn_box; ++j)
              ptx::tma_load_2d(a_dst + j * geo.sub_bytes, &p->tma_a, tm * BM + j * geo.mn_box, kb * geo.bk, full);
          } else {
            ptx::tma_load_2d(a_dst, &p->tma_a, kb * geo.bk, tm * BM, full);
          }
          if (b_mn) {
            for (int j = 0; j < BN / geo.mn_box; ++j)
              ptx::tma_load_2d(b_dst + j * geo.sub_bytes, &p->tma_b, tn * BN + j * geo.mn_box, kb * geo.bk, full);
          } else {
            ptx::tma_load_2d(b_dst, &p->tma_b, kb * geo.bk, tn * BN, full);
          }
          ++issued[stage];
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag) {
        // Leave no copy of ours in flight: wait (bounded) for the last load of each stage.
        uint32_t never = 0;
#pragma unroll
        for (int s = 0; s < STAGES; ++s)
          if (issued[s])
            ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->full[s]), (issued[s] - 1) & 1, &never, WAIT_LIMIT);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      int cursor = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
        const Problem* p = problem_of(tile, &cursor);
        const Geometry geo = geometry_of(p->elem8);
        const bool f8 = p->elem8 != 0;
        const int kblocks = (p->k + geo.bk - 1) / geo.bk;
        const uint32_t a_mn = p->a_mn_major != 0, b_mn = p->b_mn_major != 0;
        const uint32_t idesc = f8 ? ptx::idesc_f8(BM, BN, a_mn, b_mn, 1u) : ptx::idesc_f16(BM, BN, a_mn, b_mn);
        // K-major: the K values of one MMA (16 fp16 / 32 fp8) are 32 bytes inside the 128-byte
        // swizzled row.  MN-major: they are that many rows of 128 bytes; the next box of 128
        // bytes of MN follows at sub_bytes.
        const uint64_t da_fixed = ptx::smem_desc_sw128(0, a_mn ? geo.sub_bytes : 16, 1024);
        const uint64_t db_fixed = ptx::smem_desc_sw128(0, b_mn ? geo.sub_bytes : 16, 1024);
        const uint32_t a_kstep = a_mn ? geo.mn_kstep : (32 >> 4), b_kstep = b_mn ? geo.mn_kstep : (32 >> 4);
        const uint32_t smem_enc = ptx::smem_u32(smem) >> 4;
        const uint32_t acc = it & 1, aphase = (it >> 1) & 1;
        if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_empty[acc]), aphase ^ 1, abort_flag, WAIT_LIMIT)) {
          fail(status, abort_flag, 0x20000u | 0x100u | acc);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->full[stage]), phase, abort_flag, WAIT_LIMIT)) {
            fail(status, abort_flag, 0x20000u | stage);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          // Only the 14-bit start-address field of a descriptor changes from MMA to MMA.
          const uint32_t a_enc = smem_enc + stage * (STAGE_BYTES >> 4);
          const uint32_t b_enc = a_enc + (A_BYTES >> 4);
          if (f8) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              ptx::mma_f8_ss(d_tmem, da_fixed | (uint64_t)(a_enc + kk * a_kstep), db_fixed | (uint64_t)(b_enc + kk * b_kstep),
                             idesc, (kb | kk) != 0 ? 1u : 0u);
          } else {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              ptx::mma_f16_ss(d_tmem, da_fixed | (uint64_t)(a_enc + kk * a_kstep), db_fixed | (uint64_t)(b_enc + kk * b_kstep),
                              idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          ptx::mma_commit(ptx::smem_u32(&bars->empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) ptx::mma_commit(ptx::smem_u32(&bars->tmem_full[acc]));
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t chunk_no = 0;
    const Problem* epi_fenced = nullptr;
    int cursor = 0;
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const Problem* p = problem_of(tile, &cursor);
      int tm, tn;
      tile_coords(*p, tile - p->tile_start, &tm, &tn);
      const uint32_t acc = it & 1, aphase = (it >> 1) & 1;
      bool ok = true;
      if (lane == 0)
        ok = ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_full[acc]), aphase, abort_flag, WAIT_LIMIT);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) fail(status, abort_flag, 0x30000u | acc);
        break;
      }
      ptx::tc_fence_after();
      epilogue_store_tile(p, tm, tn, q, lane, tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN,
                          epi_stage + q * 2 * EPI_BUF_BYTES, activation, &chunk_no, GROUPED ? &epi_fenced : nullptr);
      ptx::tc_fence_before();
      ptx::mbar_arrive(ptx::smem_u32(&bars->tmem_empty[acc]));
    }
    if (lane == 0) ptx::bulk_wait_group_read<0>();  // staging must outlive the stores that read it
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- CTA-pair kernel ---------------------------------------------------------------------
//
// Two CTAs on neighbouring SMs (a cluster of two) compute a 256 x 256 block of C with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own 128
// columns of B, so an SM pulls 32 KiB per 64-deep k-step from L2 instead of 48 KiB
// and the ring holds 5 stages next to the epilogue staging.  CTA r of pair p works on flat tile id 2p + r; the host
// only selects this kernel when the tile order puts ids 2p and 2p + 1 on vertically
// adjacent tiles of the same tile column.  The leader (rank 0) issues the MMAs; TMA
// loads of both CTAs complete on the leader's "full" barrier, MMA completion is
// committed to the "empty" / "accumulator full" barriers of both CTAs, and both
// epilogues report to the leader's "accumulator empty" barrier.  No load is multicast.

constexpr int P_STAGES = 5;
constexpr int P_BN_HALF = BN / 2;                    // B columns staged per CTA
constexpr int P_A_BYTES = BM * BK * 2;
constexpr int P_B_BYTES = P_BN_HALF * BK * 2;
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;  // 32 KiB
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + EPI_STAGE_TOTAL + 1024 + 256;

struct PairBarriers {
  uint64_t full[P_STAGES];
  uint64_t empty[P_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

template <bool GROUPED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ Problem prob, const Problem* __restrict__ table, int n_problems,
                 int total_pairs, int activation, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* epi_stage = smem + P_STAGES * P_STAGE_BYTES;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(epi_stage + EPI_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int n_pairs_grid = gridDim.x >> 1;
  const int first_pair = blockIdx.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&bars->tmem_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->tmem_empty[a]), 256);  // 128 epilogue threads of each CTA
    }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&bars->tmem_base), TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers exist before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // problem owning flat tile id `tile` (ids of one pair always belong to one problem)
  auto problem_of = [&](int tile, int* cursor) -> const Problem* {
    if (!GROUPED) return &prob;
    int g = *cursor;
    while (g + 1 < n_problems && tile >= table[g + 1].tile_start) ++g;
    *cursor = g;
    return &table[g];
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued[P_STAGES] = {};
      bool ok = true;
      const Problem* fenced = nullptr;
      // One k-step of this CTA's share of the pair's tile: the boxes of A and B to fetch.
      struct Step {
        int pair, kb, kblocks, cursor, tm, n0;
        const Problem* pr;
      };
      auto enter = [&](Step& st) {  // position `st` on the first k-step of st.pair
        if (st.pair >= total_pairs) return;
        st.pr = problem_of(2 * st.pair, &st.cursor);
        st.kblocks = (st.pr->k + geometry_of(st.pr->elem8).bk - 1) / geometry_of(st.pr->elem8).bk;
        st.kb = 0;
        int tn;
        tile_coords(*st.pr, 2 * st.pair + (int)rank - st.pr->tile_start, &st.tm, &tn);
        st.n0 = tn * BN + (int)rank * P_BN_HALF;
      };
      auto advance = [&](Step& st) {
        if (++st.kb == st.kblocks) {
          st.pair += n_pairs_grid;
          enter(st);
        }
      };
      auto acquire = [&](const Problem* pr) {  // once per problem this CTA meets, not per tile
        if (GROUPED && pr != fenced) {
          ptx::tensormap_acquire(&pr->tma_a);
          ptx::tensormap_acquire(&pr->tma_b);
          fenced = pr;
        }
      };
      Step ld = {first_pair, 0, 0, 0, 0, 0, nullptr};
      enter(ld);
      while (ld.pair < total_pairs) {
        const Problem* pr = ld.pr;
        acquire(pr);
        if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, WAIT_LIMIT)) {
          fail(status, abort_flag, 0x110000u | stage);
          ok = false;
          break;
        }
        const uint32_t full_local = ptx::smem_u32(&bars->full[stage]);
        const uint32_t full_leader = ptx::mapa(full_local, 0);
        const uint32_t a_dst = ptx::smem_u32(smem + stage * P_STAGE_BYTES);
        const uint32_t b_dst = a_dst + P_A_BYTES;
        if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * P_STAGE_BYTES);  // both CTAs' bytes
        const Geometry geo = geometry_of(pr->elem8);
        if (pr->a_mn_major) {
          for (int j = 0; j < BM / geo.mn_box; ++j)
            ptx::tma_load_2d_pair(a_dst + j * geo.sub_bytes, &pr->tma_a, ld.tm * BM + j * geo.mn_box, ld.kb * geo.bk,
                                  full_leader);
        } else {
          ptx::tma_load_2d_pair(a_dst, &pr->tma_a, ld.kb * geo.bk, ld.tm * BM, full_leader);
        }
        if (pr->b_mn_major) {
          for (int j = 0; j < P_BN_HALF / geo.mn_box; ++j)
            ptx::tma_load_2d_pair(b_dst + j * geo.sub_bytes, &pr->tma_b, ld.n0 + j * geo.mn_box, ld.kb * geo.bk,
                                  full_leader);
        } else {
          ptx::tma_load_2d_pair(b_dst, &pr->tma_b, ld.kb * geo.bk, ld.n0, full_leader);
        }
        ++issued[stage];
        if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        advance(ld);
      }
      (void)ok;
      if (*abort_flag && rank == 0) {
        // Leave no copy in flight on the barrier we own: wait (bounded) for each stage's last load.
        uint32_t never = 0;
#pragma unroll
        for (int s = 0; s < P_STAGES; ++s)
          if (issued[s])
            ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->full[s]), (issued[s] - 1) & 1, &never, WAIT_LIMIT);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t it = 0;
      bool ok = true;
      int cursor = 0;
      const uint32_t smem_enc = ptx::smem_u32(smem) >> 4;
      for (int pair = first_pair; ok && pair < total_pairs; pair += n_pairs_grid, ++it) {
        const Problem* pr = problem_of(2 * pair, &cursor);
        const Geometry geo = geometry_of(pr->elem8);
        const bool f8 = pr->elem8 != 0;
        const int kblocks = (pr->k + geo.bk - 1) / geo.bk;
        const bool a_mn = pr->a_mn_major != 0, b_mn = pr->b_mn_major != 0;
        const uint32_t idesc = f8 ? ptx::idesc_f8(2 * BM, BN, a_mn ? 1u : 0u, b_mn ? 1u : 0u, 1u)
                                  : ptx::idesc_f16(2 * BM, BN, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
        // Only the 14-bit start-address field of a descriptor changes from MMA to MMA.
        const uint64_t da_fixed = ptx::smem_desc_sw128(0, a_mn ? geo.sub_bytes : 16, 1024);
        const uint64_t db_fixed = ptx::smem_desc_sw128(0, b_mn ? geo.sub_bytes : 16, 1024);
        const uint32_t a_kstep = a_mn ? geo.mn_kstep : (32 >> 4), b_kstep = b_mn ? geo.mn_kstep : (32 >> 4);
        const uint32_t acc = it & 1, aphase = (it >> 1) & 1;
        if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_empty[acc]), aphase ^ 1, abort_flag, WAIT_LIMIT)) {
          fail(status, abort_flag, 0x120000u | 0x100u | acc);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->full[stage]), phase, abort_flag, WAIT_LIMIT)) {
            fail(status, abort_flag, 0x120000u | stage);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_enc = smem_enc + stage * (P_STAGE_BYTES >> 4);
          const uint32_t b_enc = a_enc + (P_A_BYTES >> 4);
          if (f8) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              ptx::mma_f8_ss_pair(d_tmem, da_fixed | (uint64_t)(a_enc + kk * a_kstep),
                                  db_fixed | (uint64_t)(b_enc + kk * b_kstep), idesc, (kb | kk) != 0 ? 1u : 0u);
          } else {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              ptx::mma_f16_ss_pair(d_tmem, da_fixed | (uint64_t)(a_enc + kk * a_kstep),
                                   db_fixed | (uint64_t)(b_enc + kk * b_kstep), idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          ptx::mma_commit_pair(ptx::smem_u32(&bars->empty[stage]), 3);  // frees the slot in both CTAs
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) ptx::mma_commit_pair(ptx::smem_u32(&bars->tmem_full[acc]), 3);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows) ----------------
    const int q = warp & 3;
    uint32_t chunk_no = 0;
    const Problem* epi_fenced = nullptr;
    uint32_t it = 0;
    int cursor = 0;
    for (int pair = first_pair; pair < total_pairs; pair += n_pairs_grid, ++it) {
      const Problem* pr = problem_of(2 * pair, &cursor);
      int tm, tn;
      tile_coords(*pr, 2 * pair + (int)rank - pr->tile_start, &tm, &tn);
      const uint32_t acc = it & 1, aphase = (it >> 1) & 1;
      bool ok = true;
      if (lane == 0)
        ok = ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_full[acc]), aphase, abort_flag, WAIT_LIMIT);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) fail(status, abort_flag, 0x130000u | acc);
        break;
      }
      ptx::tc_fence_after();
      epilogue_store_tile(pr, tm, tn, q, lane, tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN,
                          epi_stage + q * 2 * EPI_BUF_BYTES, activation, &chunk_no, GROUPED ? &epi_fenced : nullptr);
      ptx::tc_fence_before();
      ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&bars->tmem_empty[acc]), 0));
    }
    if (lane == 0) ptx::bulk_wait_group_read<0>();  // staging must outlive the stores that read it
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // neither CTA leaves while the other may still touch its shared memory
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- host side ---------------------------------------------------------------------------

// 2-D tensor map of fp16 (elem_bytes 2) or 8-bit (elem_bytes 1) elements: `inner`
// contiguous elements per row, `outer` rows.
int32_t make_tmap(EncodeFn enc, CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                  uint32_t box_inner, uint32_t box_outer, int elem_bytes = 2) {
  return make_tmap_2d(enc, out, elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, base,
                      inner, outer, inner * (uint64_t)elem_bytes, box_inner, box_outer);
}

int32_t fill_order(const lego_layout_t* order, int tiles_m, int tiles_n, TileOrder* out) {
  std::memset(out, 0, sizeof(*out));
  if (!order) return LEGO_OK;
  int64_t size = 0;
  int32_t st = check_layout(order, &size);
  if (st != LEGO_OK) return st;
  if (order->rank != 2 || order->dims[0] != tiles_m || order->dims[1] != tiles_n) return LEGO_ERR_DOMAIN;
  std::vector<Digit> dg;
  st = fold_layout(order, &dg);
  if (st != LEGO_OK) return st;  // tile orders must fold to digit strides
  // identity order (row-major over tiles) needs no terms
  if ((int)dg.size() > kMaxOrderTerms) return LEGO_ERR_UNSUPPORTED;
  for (const Digit& d : dg) {
    TileTerm& t = out->t[out->n_terms++];
    t.a = (uint32_t)d.stride;
    t.m = (d.stride * d.mod == size) ? 0u : (uint32_t)d.mod;
    t.b = (uint32_t)d.div;
    t.dst = (uint32_t)d.src;
  }
  return LEGO_OK;
}

int32_t fill_problem(EncodeFn enc, Problem* p, const void* A, const void* B, void* C, int64_t M, int64_t N,
                     int64_t K, int trans_a, int trans_b, const lego_layout_t* order, int tile_start,
                     int b_box_rows = BN, int elem8 = 0) {
  if (!A || !B || !C) return LEGO_ERR_NULL;
  if (M < 1 || N < 1 || K < 1 || M > 0x3fffffff || N > 0x3fffffff || K > 0x3fffffff) return LEGO_ERR_SIZE;
  // 16-byte global strides for TMA (8 fp16 or 16 fp8 values) and 16-byte rows of the fp16 C
  const int per16 = elem8 ? 16 : 8;
  if (N % 8 || K % per16 || (trans_a && M % per16) || (!trans_b && N % per16)) return LEGO_ERR_SIZE;
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return LEGO_ERR_ALIGN;
  std::memset(p, 0, sizeof(*p));
  p->c = (__half*)C;
  p->m = (int32_t)M;
  p->n = (int32_t)N;
  p->k = (int32_t)K;
  p->tiles_m = (int32_t)((M + BM - 1) / BM);
  p->tiles_n = (int32_t)((N + BN - 1) / BN);
  p->tile_start = tile_start;
  p->a_mn_major = trans_a ? 1 : 0;
  p->b_mn_major = trans_b ? 0 : 1;
  p->elem8 = elem8 ? 1 : 0;
  const Geometry geo = geometry_of(p->elem8);
  const int eb = elem8 ? 1 : 2;
  int32_t st;
  if (trans_a) st = make_tmap(enc, &p->tma_a, A, (uint64_t)M, (uint64_t)K, geo.mn_box, geo.bk, eb);   // [K, M], M contiguous
  else         st = make_tmap(enc, &p->tma_a, A, (uint64_t)K, (uint64_t)M, geo.bk, BM, eb);           // [M, K], K contiguous
  if (st != LEGO_OK) return st;
  if (trans_b) st = make_tmap(enc, &p->tma_b, B, (uint64_t)K, (uint64_t)N, geo.bk, b_box_rows, eb);   // [N, K], K contiguous
  else         st = make_tmap(enc, &p->tma_b, B, (uint64_t)N, (uint64_t)K, geo.mn_box, geo.bk, eb);   // [K, N], N contiguous
  if (st != LEGO_OK) return st;
  st = make_tmap(enc, &p->tma_c, C, (uint64_t)N, (uint64_t)M, EPI_CHUNK_COLS, 32);      // [M, N], N contiguous
  if (st != LEGO_OK) return st;
  return fill_order(order, p->tiles_m, p->tiles_n, &p->order);
}

// Scratch of lego_grouped_gemm_f16_static: a 256-byte status area followed by the
// problem table.  Lives in the library's device image: every GPU that loads the
// library holds these 40.25 KiB until the process exits.
constexpr int kStaticGroups = 64;
constexpr size_t kStaticStatusBytes = 256;
constexpr size_t kStaticScratchBytes = kStaticStatusBytes + (size_t)kStaticGroups * sizeof(Problem);
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct StaticScratch {
  unsigned char* dev;  // device address of g_static_scratch on this device
  int sm_count;
  bool ready;
};
constexpr int kMaxDevices = 64;
StaticScratch g_static[kMaxDevices];
std::mutex g_static_mu;

// In host code `g_static_scratch` is only a stand-in for the symbol; the address a
// kernel may use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
int32_t static_scratch(StaticScratch** out) {
  int dev = 0;
  LEGO_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return LEGO_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticScratch& sc = g_static[dev];
  if (!sc.ready) {
    void* p = nullptr;
    LEGO_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    LEGO_CUDA_TRY(cudaDeviceGetAttribute(&sc.sm_count, cudaDevAttrMultiProcessorCount, dev));
    sc.dev = (unsigned char*)p;
    sc.ready = true;
  }
  *out = &sc;
  return LEGO_OK;
}

template <bool GROUPED>
int32_t configure() {
  static std::once_flag once;
  static cudaError_t result = cudaSuccess;
  std::call_once(once, [] {
    result = cudaFuncSetAttribute(gemm_kernel<GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  });
  return cuda_status(result);
}

// One-time set-up of the CTA-pair kernel: shared-memory limit and how many pairs
// the device can hold at once.
template <bool GROUPED>
int32_t configure_pair(int* max_clusters) {
  static std::once_flag once;
  static int32_t result = LEGO_OK;
  static int clusters = 0;
  std::call_once(once, [] {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES);
    if (e == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(NUM_THREADS, 1, 1);
      cfg.dynamicSmemBytes = P_SMEM_BYTES;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      e = cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<GROUPED>, &cfg);
    }
    if (e != cudaSuccess) { (void)cudaGetLastError(); result = cuda_status(e); }
  });
  *max_clusters = clusters;
  return result;
}

// Do tile ids 2p and 2p + 1 of this problem share a tile column (they would share B)?
bool pairs_share_columns(const Problem& p) {
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n;
  if (total % 2 || total > (1 << 22)) return false;
  for (int64_t t = 0; t < total; t += 2) {
    int m0, n0, m1, n1;
    tile_coords(p, (int)t, &m0, &n0);
    tile_coords(p, (int)t + 1, &m1, &n1);
    if (n0 != n1) return false;
  }
  return true;
}

// Build the problem records of a grouped GEMM into `table` (host), copy them to
// `dev_table` and launch on `s`.  A group without a tile order gets the reference's
// in-group order, row-major tiles (tile_m = t / tiles_n, tile_n = t % tiles_n), which the
// single-CTA kernel runs; CTA pairs are used when every group's order puts tiles 2p and
// 2p + 1 in one tile column.  (Sustained A/B on one box, 16 groups: row-major / single CTA
// 1 050-1 090 TFLOP/s, column-major / pairs 1 010-1 050; isolated launches tie.)  Allocates nothing.
int32_t run_grouped(EncodeFn enc, Problem* table, const void* const* A, const void* const* B, void* const* C,
                    const int64_t* mnk, int32_t G, const lego_layout_t* const* tile_orders, Problem* dev_table,
                    uint32_t* status, int sm_count, cudaStream_t s) {
  int64_t total = 0;
  bool pairs = true;
  for (int g = 0; g < G; ++g) {
    const lego_layout_t* order = tile_orders ? tile_orders[g] : nullptr;
    const int32_t st = fill_problem(enc, &table[g], A[g], B[g], C[g], mnk[3 * g], mnk[3 * g + 1], mnk[3 * g + 2],
                                    0, 0, order, (int)total);
    if (st != LEGO_OK) return st;
    Problem& p = table[g];
    pairs = pairs && pairs_share_columns(p);
    total += (int64_t)p.tiles_m * p.tiles_n;
    if (total > 0x7fffffff) return LEGO_ERR_SIZE;
  }
  LEGO_CUDA_TRY(cudaMemcpyAsync(dev_table, table, (size_t)G * sizeof(Problem), cudaMemcpyHostToDevice, s));
  if (pairs) {
    int max_clusters = 0;
    if (configure_pair<true>(&max_clusters) == LEGO_OK && max_clusters >= 1) {
      const int64_t n_pairs = total / 2;
      const int clusters = (int)(n_pairs < max_clusters ? n_pairs : max_clusters);
      gemm_pair_kernel<true><<<2 * clusters, NUM_THREADS, P_SMEM_BYTES, s>>>(table[0], dev_table, G, (int)n_pairs,
                                                                            LEGO_ACT_NONE, status);
      return cuda_status(cudaGetLastError());
    }
  }
  const int32_t st = configure<true>();
  if (st != LEGO_OK) return st;
  const int grid = (int)(total < sm_count ? total : sm_count);
  gemm_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(table[0], dev_table, G, (int)total, LEGO_ACT_NONE, status);
  return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace lego

using namespace lego;

extern "C" {

// One GEMM, fp16 or e5m2 operands: CTA pairs when the tile order allows, else one CTA per tile.
static int32_t run_gemm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int32_t trans_a,
                        int32_t trans_b, int32_t activation, const lego_layout_t* tile_order, int elem8,
                        void* stream) {
  if (activation != LEGO_ACT_NONE && activation != LEGO_ACT_LEAKY_RELU) return LEGO_ERR_UNSUPPORTED;
  int32_t err = LEGO_OK;
  DeviceCtx* ctx = device_ctx(&err);
  if (!ctx) return err;
  EncodeFn enc = encode_fn(&err);
  if (!enc) return err;
  Problem p;
  int32_t st = fill_problem(enc, &p, A, B, C, M, N, K, trans_a, trans_b, tile_order, 0, BN, elem8);
  if (st != LEGO_OK) return st;
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n;
  if (total > 0x7fffffff) return LEGO_ERR_SIZE;
  // CTA pairs: tile ids 2p and 2p + 1 must share their tile column (they share B).
  bool pairs = total >= 2 && total % 2 == 0 && total <= (1 << 22);
  for (int64_t t = 0; pairs && t < total; t += 2) {
    int m0, n0, m1, n1;
    tile_coords(p, (int)t, &m0, &n0);
    tile_coords(p, (int)t + 1, &m1, &n1);
    pairs = (n0 == n1);
  }
  if (pairs) {
    st = fill_problem(enc, &p, A, B, C, M, N, K, trans_a, trans_b, tile_order, 0, P_BN_HALF, elem8);
    if (st != LEGO_OK) return st;
    int max_clusters = 0;
    st = configure_pair<false>(&max_clusters);
    if (st == LEGO_OK && max_clusters >= 1) {
      const int64_t n_pairs = total / 2;
      const int clusters = (int)(n_pairs < max_clusters ? n_pairs : max_clusters);
      gemm_pair_kernel<false><<<2 * clusters, NUM_THREADS, P_SMEM_BYTES, (cudaStream_t)stream>>>(p, nullptr, 1, (int)n_pairs, activation,
                                                                                   ctx->status_word);
      return cuda_status(cudaGetLastError());
    }
    st = fill_problem(enc, &p, A, B, C, M, N, K, trans_a, trans_b, tile_order, 0, BN, elem8);
    if (st != LEGO_OK) return st;
  }
  st = configure<false>();
  if (st != LEGO_OK) return st;
  const int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
  gemm_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(p, nullptr, 1, (int)total, activation,
                                                                         ctx->status_word);
  return cuda_status(cudaGetLastError());
}

int32_t lego_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                      int32_t trans_a, int32_t trans_b, int32_t activation,
                      const lego_layout_t* tile_order, void* stream) {
  return run_gemm(A, B, C, M, N, K, trans_a, trans_b, activation, tile_order, 0, stream);
}

int32_t lego_gemm_e5m2(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                       int32_t trans_a, int32_t trans_b, int32_t activation,
                       const lego_layout_t* tile_order, void* stream) {
  return run_gemm(A, B, C, M, N, K, trans_a, trans_b, activation, tile_order, 1, stream);
}

int32_t lego_grouped_gemm_f16(const void* const* A, const void* const* B, void* const* C,
                              const int64_t* mnk, int32_t G,
                              const lego_layout_t* const* tile_orders, void* stream) {
  if (!A || !B || !C || !mnk) return LEGO_ERR_NULL;
  if (G < 0 || G > LEGO_MAX_GROUPS) return LEGO_ERR_RANK;
  if (G == 0) return LEGO_OK;
  int32_t err = LEGO_OK;
  DeviceCtx* ctx = device_ctx(&err);
  if (!ctx) return err;
  EncodeFn enc = encode_fn(&err);
  if (!enc) return err;
  if ((size_t)G * sizeof(Problem) > ctx->tmap_table_bytes) return LEGO_ERR_RANK;
  std::vector<Problem> table(G);
  // The device table is per device and reused by every call: calls on one stream are
  // ordered; callers overlapping grouped GEMMs on different streams must serialise.
  return run_grouped(enc, table.data(), A, B, C, mnk, G, tile_orders, (Problem*)ctx->tmap_table, ctx->status_word,
                     ctx->sm_count, (cudaStream_t)stream);
}

int32_t lego_grouped_gemm_f16_static(const void* const* A, const void* const* B, void* const* C,
                                     const int64_t* mnk, int32_t G,
                                     const lego_layout_t* const* tile_orders, uint32_t* dev_status,
                                     void* stream) {
  if (!A || !B || !C || !mnk) return LEGO_ERR_NULL;
  if (G < 0) return LEGO_ERR_RANK;
  if (G > kStaticGroups) return LEGO_ERR_SIZE;  // the built-in table holds LEGO_STATIC_MAX_GROUPS records
  if (G == 0) return LEGO_OK;
  int32_t err = LEGO_OK;
  StaticScratch* sc = nullptr;
  err = static_scratch(&sc);
  if (err != LEGO_OK) return err;
  EncodeFn enc = encode_fn(&err);
  if (!enc) return err;
  Problem table[kStaticGroups];  // host stack: no heap, no device allocation anywhere in this call
  cudaStream_t s = (cudaStream_t)stream;
  uint32_t* status = dev_status;
  if (!status) {
    // the array keeps whatever the previous call left: the status word must start at zero
    status = reinterpret_cast<uint32_t*>(sc->dev);
    LEGO_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(uint32_t), s));
  }
  Problem* dev_table = reinterpret_cast<Problem*>(sc->dev + kStaticStatusBytes);
  return run_grouped(enc, table, A, B, C, mnk, G, tile_orders, dev_table, status, sc->sm_count, s);
}

}  // extern "C"
