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

#include <atomic>
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
// A wait that spans a whole k-loop (accumulator full / empty) gets this much more per k-step,
// about a hundred times what a step takes, so that a very deep K cannot trip a false timeout.
constexpr long long WAIT_PER_KSTEP = 65536LL;
__device__ __forceinline__ long long loop_wait_limit(int kblocks) { return WAIT_LIMIT + WAIT_PER_KSTEP * kblocks; }

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
        if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_empty[acc]), aphase ^ 1, abort_flag,
                                          loop_wait_limit(kblocks))) {
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
        ok = ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_full[acc]), aphase, abort_flag,
                                          loop_wait_limit((p->k + geometry_of(p->elem8).bk - 1) / geometry_of(p->elem8).bk));
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
// Two CTAs on neighbouring SMs (a cluster of two) compute MT blocks of 256 x 256 of C with
// tcgen05.mma.cta_group::2.  A "pair tile" is 2 * MT consecutive flat tile ids that share a
// tile column: id 2 * MT * t + 2 * j + r is the 128 x 256 tile whose rows CTA r contributes
// to block j.  Each CTA stages its own MT x 128 rows of A and its own 128 columns of B per
// 64-deep k-step, so an SM pulls 32 KiB (MT = 1) or 48 KiB for twice the flops (MT = 2) from
// L2 where one CTA per tile pulls 48 KiB.  MT = 1 alternates two 256-column accumulators so
// the epilogue of one pair tile overlaps the main loop of the next; MT = 2 fills all 512
// TMEM columns with one pair tile (block 0 is drained while block 1's last MMAs retire).
// The leader (rank 0) issues the MMAs; TMA loads of both CTAs complete on the leader's
// "full" barrier, MMA completion is committed to the "empty" / "accumulator full" barriers
// of both CTAs, and both epilogues report to the leader's "accumulator empty" barrier.  No
// load is multicast.
//
// Work split (single problem only): pair tiles [0, dp_tiles) are walked data-parallel,
// worker w taking w, w + W, ...; the remaining sk_tiles -- the partial last wave -- are cut
// along K into W equal runs of k-steps (stream-K), so every pair of SMs gets the same number
// of k-steps.  A run may start inside a tile: that worker is not the tile's owner and writes
// its fp32 accumulator to its slot of the workspace; the owner (the worker whose run holds
// k-step 0 of the tile) adds the slots of the workers that follow it and stores C.  Runs are
// processed before the data-parallel tiles and in increasing k order, so an owner's own part
// finishes after its peers' parts: the flag waits are there for correctness and are bounded
// like every other wait.

constexpr int P_BN_HALF = BN / 2;                    // B columns staged per CTA
constexpr int P_A_BYTES = BM * BK * 2;               // one 128-row block of A
constexpr int P_B_BYTES = P_BN_HALF * BK * 2;
__host__ __device__ constexpr int pair_stage_bytes(int mt) { return mt * P_A_BYTES + P_B_BYTES; }
__host__ __device__ constexpr int pair_stages(int mt) { return mt == 1 ? 5 : 4; }
__host__ __device__ constexpr int pair_smem_bytes(int mt) {
  return pair_stages(mt) * pair_stage_bytes(mt) + EPI_STAGE_TOTAL + 1024 + 256;
}
constexpr int P_MAX_STAGES = 5;

struct PairBarriers {
  uint64_t full[P_MAX_STAGES];
  uint64_t empty[P_MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// Stream-K workspace: kSkFlagBytes of flags (one word per worker, CTA rank and epilogue warp;
// zero before the first call, every call that completes leaves them zero) followed by one
// fp32 accumulator slot per worker: [rank][block j][column 0..255][row 0..127].
constexpr int kSkFlagBytes = 8192;
constexpr int kSkMaxWorkers = kSkFlagBytes / (2 * 8 * 4);  // a word per CTA rank and epilogue warp
// The pair kernel has eight epilogue warps: two per TMEM lane quarter, each taking half of
// the 256 columns of an accumulator block.  One warp per quarter (four in all) needed about
// 3 300 cycles per block, more than the 2 048 the MMA schedule hides, and ran a 74-tile wave
// of one-k-step tiles in 6.7 us where the output stream alone takes 3 us.
constexpr int P_EPI_WARPS = 8;
constexpr int P_THREADS = 64 + 32 * P_EPI_WARPS;
constexpr int kSkBlockFloats = BM * BN;  // one CTA's 128 x 256 accumulator

struct Sched {
  int32_t total_tiles;  // pair tiles
  int32_t dp_tiles;     // walked whole, round-robin
  int32_t sk_tiles;     // cut along K (ids dp_tiles .. total_tiles - 1)
  int32_t sk_run;       // k-steps per worker in the stream-K part
  int32_t kblocks;      // k-steps per tile (uniform: the stream-K part exists for one problem only)
  int32_t lag;          // MT = 2: k-steps block 0 runs ahead of block 1 at both ends of a tile
  float* workspace;     // nullable when sk_tiles == 0
};

struct WorkItem {
  int tile;       // pair tile
  int kb0, kb1;   // k-steps [kb0, kb1); kb1 < 0: all of the tile's
  int n_peers;    // > 0: add the slots of workers w + 1 .. w + n_peers before storing C
  bool partial;   // true: write the accumulator to this worker's slot instead of C
};

struct WorkIter {
  int u, u_end;  // stream-K k-steps left, as offsets into the stream-K part
  int tile;      // next data-parallel pair tile
};

__device__ __forceinline__ WorkIter work_begin(const Sched& sc, int w) {
  WorkIter it;
  const long long total = (long long)sc.sk_tiles * sc.kblocks;
  const long long u0 = (long long)w * sc.sk_run;
  it.u = (int)(u0 < total ? u0 : total);
  it.u_end = (int)(u0 + sc.sk_run < total ? u0 + sc.sk_run : total);
  it.tile = w;
  return it;
}

__device__ __forceinline__ bool work_next(WorkIter& it, const Sched& sc, int w, int n_workers, WorkItem* out) {
  if (it.u < it.u_end) {
    const int j = it.u / sc.kblocks;
    const int kb0 = it.u - j * sc.kblocks;
    const int tile_end = (j + 1) * sc.kblocks;
    const int seg_end = it.u_end < tile_end ? it.u_end : tile_end;
    out->tile = sc.dp_tiles + j;
    out->kb0 = kb0;
    out->kb1 = kb0 + (seg_end - it.u);
    out->partial = kb0 > 0;
    out->n_peers = (kb0 == 0 && seg_end < tile_end) ? (tile_end - 1) / sc.sk_run - w : 0;
    it.u = seg_end;
    return true;
  }
  if (it.tile < sc.dp_tiles) {
    out->tile = it.tile;
    out->kb0 = 0;
    out->kb1 = -1;
    out->partial = false;
    out->n_peers = 0;
    it.tile += n_workers;
    return true;
  }
  return false;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// What the pair kernel's epilogue does besides storing C.
struct EpiSplit {
  float* partial_out;       // non-null: dump this warp's accumulator rows here, store no C
  const float* partial_in;  // first peer's block (same rank and j); further peers follow at `stride`
  int n_in;
  size_t stride;
};

// This warp is done reading its rows of an accumulator block: every lane's tcgen05.ld has
// completed (wait::ld before the call); one arrival per warp on the leader CTA's barrier.
__device__ __forceinline__ void release_accumulator(uint32_t empty_bar, int lane) {
  ptx::tc_fence_before();
  __syncwarp();
  if (lane == 0) ptx::mbar_arrive_cluster(empty_bar);
}

// 64 fp32 accumulator columns of one row -> activation -> 32 packed fp16 pairs.
template <int ACT>
__device__ __forceinline__ void convert_chunk(const uint32_t* r, uint32_t* h) {
#pragma unroll
  for (int e = 0; e < 32; ++e) {
    float x0 = __uint_as_float(r[2 * e]);
    float x1 = __uint_as_float(r[2 * e + 1]);
    if (ACT == LEGO_ACT_LEAKY_RELU) {
      x0 = x0 >= 0.f ? x0 : 0.01f * x0;
      x1 = x1 >= 0.f ? x1 : 0.01f * x1;
    }
    const __half2 hh = __floats2half2_rn(x0, x1);
    h[e] = *reinterpret_cast<const uint32_t*>(&hh);
  }
}

// This warp's 32 rows x 64 fp16 columns -> its 4 KiB staging buffer (128-byte swizzle) -> TMA
// store at (row0, col0) of C.  The buffer is reused: first wait until the store that last read
// it has done so.
__device__ __forceinline__ void stage_and_store(const Problem* p, uint8_t* buf, int lane, const uint32_t* h,
                                                int col0, int row0) {
  if (lane == 0) ptx::bulk_wait_group_read<0>();
  __syncwarp();
  uint4* dst = reinterpret_cast<uint4*>(buf + lane * 128);
#pragma unroll
  for (int j = 0; j < 8; ++j) dst[j ^ (lane & 7)] = make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
  ptx::fence_proxy_async();  // generic-proxy writes above -> visible to the TMA engine
  __syncwarp();
  if (lane == 0) {
    ptx::tma_store_2d(&p->tma_c, col0, row0, ptx::smem_u32(buf));
    ptx::bulk_commit_group();
  }
}

// One accumulator block, this warp's share (32 rows x the 128 columns of half `half`) ->
// [+ peers' partial sums] -> activation -> fp16 -> swizzled shared memory -> TMA store; or ->
// fp32 partial slot.  A warp has one 4 KiB staging buffer: the wait for the previous store to
// have read it sits after the TMEM load and the conversion of the next chunk.  (Reading the
// staged chunk back and writing it with plain 128-bit stores, whole lines per instruction, was
// slower: 8192^3 1 130 against 1 210 TFLOP/s sustained.  Reading block 1 into registers before
// block 0's second half is stored, so that both blocks leave TMEM within a few hundred cycles
// of each other, needs 128 + 32 live registers per thread; ten warps leave 168 and the spills
// cost more than the earlier release gains: 1 229 against 1 291.)
template <int ACT>
__device__ __forceinline__ void epilogue_pair_block(const Problem* p, int tm, int tn, int q, int half, int lane,
                                                    uint32_t tmem_tile, uint8_t* buf,
                                                    const Problem** fenced, const EpiSplit& sp,
                                                    uint32_t empty_bar) {
  const int row0 = tm * BM + q * 32;
  const int row = q * 32 + lane;
  if (sp.partial_out) {
#pragma unroll 1
    for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
      uint32_t r[32];
      ptx::tmem_ld_32x32(tmem_tile + c * 32, r);
      ptx::tmem_ld_wait();
      float* dst = sp.partial_out + (size_t)(c * 32) * BM + row;
#pragma unroll
      for (int i = 0; i < 32; ++i) __stcg(dst + (size_t)i * BM, __uint_as_float(r[i]));
    }
    release_accumulator(empty_bar, lane);
    return;
  }
  if (row0 >= p->m) {  // nothing of this warp's rows exists (warp-uniform)
    release_accumulator(empty_bar, lane);
    return;
  }
  if (fenced && *fenced != p) {  // table-resident map: acquire once per problem
    if (lane == 0) ptx::tensormap_acquire(&p->tma_c);
    *fenced = p;
  }
  constexpr int CHUNKS = BN / EPI_CHUNK_COLS / 2;  // per warp: two chunks of 64 columns
  static_assert(CHUNKS == 2, "the loads of both chunks are issued up front");
  // TMEM -> registers takes about a thousand cycles for 64 columns (measured), whatever follows:
  // both chunks' loads are issued before the first is converted, so the second one's latency
  // is hidden behind the first one's conversion, staging and store.
  uint32_t r[2][64];
  const int c_first = half * CHUNKS;
  ptx::tmem_ld_32x32(tmem_tile + c_first * EPI_CHUNK_COLS, r[0]);
  ptx::tmem_ld_32x32(tmem_tile + c_first * EPI_CHUNK_COLS + 32, r[0] + 32);
  ptx::tmem_ld_32x32(tmem_tile + (c_first + 1) * EPI_CHUNK_COLS, r[1]);
  ptx::tmem_ld_32x32(tmem_tile + (c_first + 1) * EPI_CHUNK_COLS + 32, r[1] + 32);
  ptx::tmem_ld_wait();
  release_accumulator(empty_bar, lane);  // the block is in registers: the next tile's MMAs may overwrite it
#pragma unroll
  for (int k = 0; k < CHUNKS; ++k) {
    const int c = c_first + k;
    const int col0 = tn * BN + c * EPI_CHUNK_COLS;
    if (col0 >= p->n) break;  // chunks past the last column are not staged at all
    for (int peer = 0; peer < sp.n_in; ++peer) {
      const float* src = sp.partial_in + peer * sp.stride + (size_t)(c * EPI_CHUNK_COLS) * BM + row;
#pragma unroll
      for (int i = 0; i < 64; ++i) r[k][i] = __float_as_uint(__uint_as_float(r[k][i]) + __ldcg(src + (size_t)i * BM));
    }
    uint32_t h[32];
    convert_chunk<ACT>(r[k], h);
    stage_and_store(p, buf, lane, h, col0, row0);
  }
}

// Raise the abort flag of this CTA and of its peer: the peer's waits then give up at their
// next check instead of running out one after another.
__device__ __forceinline__ void fail_pair(uint32_t* status, volatile uint32_t* abort_flag, uint32_t peer_rank,
                                          uint32_t code) {
  *abort_flag = 1;
  ptx::st_cluster_u32(ptx::mapa(ptx::smem_u32(const_cast<uint32_t*>(abort_flag)), peer_rank), 1u);
  atomicCAS(status, 0u, code);
}

template <bool GROUPED, int MT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ Problem prob, const Problem* __restrict__ table, int n_problems,
                 const __grid_constant__ Sched sched, int activation, uint32_t* status) {
  constexpr int NSTAGE = pair_stages(MT);
  constexpr int STAGE = pair_stage_bytes(MT);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* epi_stage = smem + NSTAGE * STAGE;
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(epi_stage + EPI_BYTES);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int n_workers = gridDim.x >> 1;
  const int worker = blockIdx.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bars->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(ptx::smem_u32(&bars->tmem_full[a]), 1);
      ptx::mbar_init(ptx::smem_u32(&bars->tmem_empty[a]), 2 * P_EPI_WARPS);  // one arrival per epilogue warp of both CTAs
    }
    bars->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  if (warp == 1) {  // warp 1 of both CTAs: the pair's allocation is collective
    ptx::tmem_alloc_pair(ptx::smem_u32(&bars->tmem_base), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // the peer's barriers exist before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  // problem owning pair tile `tile` (the ids of one pair tile always belong to one problem)
  auto problem_of = [&](int tile, int* cursor) -> const Problem* {
    if (!GROUPED) return &prob;
    int g = *cursor;
    while (g + 1 < n_problems && 2 * MT * tile >= table[g + 1].tile_start) ++g;
    *cursor = g;
    return &table[g];
  };
  auto kblocks_of = [](const Problem* pr) {
    const int bk = geometry_of(pr->elem8).bk;
    return (pr->k + bk - 1) / bk;
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      uint32_t issued[NSTAGE] = {};
      const Problem* fenced = nullptr;
      int cursor = 0;
      WorkIter iter = work_begin(sched, worker);
      WorkItem item;
      bool ok = true;
      while (ok && work_next(iter, sched, worker, n_workers, &item)) {
        const Problem* pr = problem_of(item.tile, &cursor);
        if (GROUPED && pr != fenced) {  // once per problem this CTA meets, not per tile
          ptx::tensormap_acquire(&pr->tma_a);
          ptx::tensormap_acquire(&pr->tma_b);
          fenced = pr;
        }
        const Geometry geo = geometry_of(pr->elem8);
        const int kb1 = item.kb1 < 0 ? kblocks_of(pr) : item.kb1;
        int tm[MT], tn = 0;
#pragma unroll
        for (int j = 0; j < MT; ++j)
          tile_coords(*pr, 2 * MT * item.tile + 2 * j + (int)rank - pr->tile_start, &tm[j], &tn);
        const int n0 = tn * BN + (int)rank * P_BN_HALF;
        for (int kb = item.kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->empty[stage]), phase ^ 1, abort_flag, WAIT_LIMIT)) {
            fail_pair(status, abort_flag, rank ^ 1u, 0x110000u | stage);
            ok = false;
            break;
          }
          const uint32_t full_local = ptx::smem_u32(&bars->full[stage]);
          const uint32_t full_leader = ptx::mapa(full_local, 0);
          const uint32_t a_dst = ptx::smem_u32(smem + stage * STAGE);
          const uint32_t b_dst = a_dst + MT * P_A_BYTES;
          if (rank == 0) ptx::mbar_arrive_expect_tx(full_local, 2 * STAGE);  // both CTAs' bytes
#pragma unroll
          for (int j = 0; j < MT; ++j) {
            if (pr->a_mn_major) {
              for (int b = 0; b < BM / geo.mn_box; ++b)
                ptx::tma_load_2d_pair(a_dst + j * P_A_BYTES + b * geo.sub_bytes, &pr->tma_a,
                                      tm[j] * BM + b * geo.mn_box, kb * geo.bk, full_leader);
            } else {
              ptx::tma_load_2d_pair(a_dst + j * P_A_BYTES, &pr->tma_a, kb * geo.bk, tm[j] * BM, full_leader);
            }
          }
          if (pr->b_mn_major) {
            for (int b = 0; b < P_BN_HALF / geo.mn_box; ++b)
              ptx::tma_load_2d_pair(b_dst + b * geo.sub_bytes, &pr->tma_b, n0 + b * geo.mn_box, kb * geo.bk,
                                    full_leader);
          } else {
            ptx::tma_load_2d_pair(b_dst, &pr->tma_b, kb * geo.bk, n0, full_leader);
          }
          ++issued[stage];
          if (++stage == NSTAGE) { stage = 0; phase ^= 1; }
        }
      }
      if (*abort_flag && rank == 0) {
        // Leave no copy in flight on the barrier we own: wait (bounded) for each stage's last load.
        uint32_t never = 0;
#pragma unroll
        for (int s = 0; s < NSTAGE; ++s)
          if (issued[s])
            ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->full[s]), (issued[s] - 1) & 1, &never, WAIT_LIMIT);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t kcount = 0;  // k-steps consumed so far: ring slot kcount % NSTAGE, parity (kcount / NSTAGE) & 1
      uint32_t acc_it = 0;
      bool ok = true;
      int cursor = 0;
      const uint32_t smem_enc = ptx::smem_u32(smem) >> 4;
      WorkIter iter = work_begin(sched, worker);
      WorkItem item;
      while (ok && work_next(iter, sched, worker, n_workers, &item)) {
        const Problem* pr = problem_of(item.tile, &cursor);
        const Geometry geo = geometry_of(pr->elem8);
        const bool f8 = pr->elem8 != 0;
        const int kblocks = kblocks_of(pr);
        const int n_steps = (item.kb1 < 0 ? kblocks : item.kb1) - item.kb0;
        const bool a_mn = pr->a_mn_major != 0, b_mn = pr->b_mn_major != 0;
        const uint32_t idesc = f8 ? ptx::idesc_f8(2 * BM, BN, a_mn ? 1u : 0u, b_mn ? 1u : 0u, 1u)
                                  : ptx::idesc_f16(2 * BM, BN, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
        // Only the 14-bit start-address field of a descriptor changes from MMA to MMA.
        const uint64_t da_fixed = ptx::smem_desc_sw128(0, a_mn ? geo.sub_bytes : 16, 1024);
        const uint64_t db_fixed = ptx::smem_desc_sw128(0, b_mn ? geo.sub_bytes : 16, 1024);
        const uint32_t a_kstep = a_mn ? geo.mn_kstep : (32 >> 4), b_kstep = b_mn ? geo.mn_kstep : (32 >> 4);

        // the MMAs of k-step t (relative to the item) into accumulator block j
        auto issue = [&](int j, int t) {
          const uint32_t slot = (kcount + (uint32_t)t) % NSTAGE;
          const uint32_t a_enc = smem_enc + slot * (STAGE >> 4) + j * (P_A_BYTES >> 4);
          const uint32_t b_enc = smem_enc + slot * (STAGE >> 4) + MT * (P_A_BYTES >> 4);
          const uint32_t d = tmem_base + ((acc_it + j) & 1) * BN;
          if (f8) {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              ptx::mma_f8_ss_pair(d, da_fixed | (uint64_t)(a_enc + kk * a_kstep),
                                  db_fixed | (uint64_t)(b_enc + kk * b_kstep), idesc, (t > 0 || kk != 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              ptx::mma_f16_ss_pair(d, da_fixed | (uint64_t)(a_enc + kk * a_kstep),
                                   db_fixed | (uint64_t)(b_enc + kk * b_kstep), idesc, (t > 0 || kk != 0) ? 1u : 0u);
          }
        };
        auto wait_loaded = [&](int t) {
          const uint32_t c = kcount + (uint32_t)t;
          if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->full[c % NSTAGE]), (c / NSTAGE) & 1u, abort_flag,
                                            WAIT_LIMIT)) {
            fail_pair(status, abort_flag, 1u, 0x120000u | (c % NSTAGE));
            ok = false;
            return false;
          }
          ptx::tc_fence_after();
          return true;
        };
        auto release = [&](int t) {  // frees the ring slot of k-step t in both CTAs once the MMAs so far are done
          ptx::mma_commit_pair(ptx::smem_u32(&bars->empty[(kcount + (uint32_t)t) % NSTAGE]), 3);
        };
        auto wait_drained = [&](int j) {
          const uint32_t acc = (acc_it + j) & 1, aphase = ((acc_it + j) >> 1) & 1;
          if (!ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_empty[acc]), aphase ^ 1, abort_flag,
                                            loop_wait_limit(kblocks))) {
            fail_pair(status, abort_flag, 1u, 0x120000u | 0x100u | acc);
            ok = false;
            return false;
          }
          ptx::tc_fence_after();
          return true;
        };
        auto publish = [&](int j) {
          ptx::mma_commit_pair(ptx::smem_u32(&bars->tmem_full[(acc_it + j) & 1]), 3);
        };

        if (MT == 1) {
          if (!wait_drained(0)) break;
          for (int t = 0; t < n_steps; ++t) {
            if (!wait_loaded(t)) break;
            issue(0, t);
            release(t);
          }
          if (ok) publish(0);
        } else {
          // Two accumulator blocks fill all of TMEM, so there is no spare buffer to hide the
          // epilogue behind: when a tile's MMAs end, both blocks are read out of TMEM at once
          // (the epilogue warps hold them in registers and store afterwards).  Block 0 of the
          // next tile starts as soon as block 0 has left TMEM and runs `lag` k-steps on its own
          // while block 1 is still being read; block 1 then catches up on the same ring slots
          // and from there the two alternate on every k-step, ending together.  (Staggering the
          // end of the tile as well starves the tensor pipe: the ring has four slots, block 0's
          // last steps would need all four, and they are released only every two blocks' worth
          // of MMA time.)
          int lag = sched.lag < n_steps / 2 ? sched.lag : n_steps / 2;
          if (lag > NSTAGE) lag = NSTAGE;
          if (!wait_drained(0)) break;
          for (int t = 0; ok && t < lag; ++t)
            if (wait_loaded(t)) issue(0, t);
          if (!ok || !wait_drained(1)) break;
          for (int t = 0; t < lag; ++t) {
            issue(1, t);
            release(t);
          }
          for (int t = lag; ok && t < n_steps; ++t) {
            if (!wait_loaded(t)) break;
            issue(0, t);
            issue(1, t);
            release(t);
          }
          if (!ok) break;
          publish(0);
          publish(1);
        }
        kcount += (uint32_t)n_steps;
        acc_it += MT;
      }
    }
  } else {
    // ---------------- epilogue (both CTAs, own rows) ----------------
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;    // which 128 of the 256 columns it drains
    const int fslot = q * 2 + half;      // its flag word within a (worker, rank)
    uint8_t* stage_buf = epi_stage + (warp - 2) * EPI_BUF_BYTES;
    const Problem* epi_fenced = nullptr;
    uint32_t acc_it = 0;
    int cursor = 0;
    uint32_t* flags = reinterpret_cast<uint32_t*>(sched.workspace);
    float* slots = sched.workspace ? sched.workspace + kSkFlagBytes / 4 : nullptr;
    const size_t worker_stride = (size_t)2 * MT * kSkBlockFloats;
    WorkIter iter = work_begin(sched, worker);
    WorkItem item;
    bool ok = true;
    while (ok && work_next(iter, sched, worker, n_workers, &item)) {
      const Problem* pr = problem_of(item.tile, &cursor);
      const int kblocks = kblocks_of(pr);
      if (item.n_peers > 0) {
        // the peers' parts were computed before ours; make sure their slots are complete
        if (lane == 0) {
          const long long t0 = clock64();
          for (int peer = 1; ok && peer <= item.n_peers; ++peer) {
            const uint32_t* f = flags + ((worker + peer) * 2 + (int)rank) * 8 + fslot;
            while (ld_acquire_gpu(f) == 0u) {
              if (*abort_flag || clock64() - t0 > loop_wait_limit(kblocks)) { ok = false; break; }
              __nanosleep(200);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) {
          if (lane == 0) fail_pair(status, abort_flag, rank ^ 1u, 0x140000u | (uint32_t)fslot);
          break;
        }
      }
#pragma unroll
      for (int j = 0; j < MT; ++j) {
        int tm, tn;
        tile_coords(*pr, 2 * MT * item.tile + 2 * j + (int)rank - pr->tile_start, &tm, &tn);
        const uint32_t acc = (acc_it + j) & 1, aphase = ((acc_it + j) >> 1) & 1;
        if (lane == 0)
          ok = ptx::mbar_wait_bounded<true>(ptx::smem_u32(&bars->tmem_full[acc]), aphase, abort_flag,
                                            loop_wait_limit(kblocks));
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) {
          if (lane == 0) fail_pair(status, abort_flag, rank ^ 1u, 0x130000u | acc);
          break;
        }
        ptx::tc_fence_after();
        EpiSplit sp;
        sp.partial_out = item.partial ? slots + (size_t)worker * worker_stride + ((size_t)rank * MT + j) * kSkBlockFloats
                                      : nullptr;
        sp.n_in = item.n_peers;
        sp.partial_in = item.n_peers > 0
                            ? slots + (size_t)(worker + 1) * worker_stride + ((size_t)rank * MT + j) * kSkBlockFloats
                            : nullptr;
        sp.stride = worker_stride;
        const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
        // the function arrives on this barrier as soon as the block has left TMEM
        const uint32_t empty_bar = ptx::mapa(ptx::smem_u32(&bars->tmem_empty[acc]), 0);
        if (activation == LEGO_ACT_LEAKY_RELU)
          epilogue_pair_block<LEGO_ACT_LEAKY_RELU>(pr, tm, tn, q, half, lane, t_acc, stage_buf,
                                                   GROUPED ? &epi_fenced : nullptr, sp, empty_bar);
        else
          epilogue_pair_block<LEGO_ACT_NONE>(pr, tm, tn, q, half, lane, t_acc, stage_buf,
                                             GROUPED ? &epi_fenced : nullptr, sp, empty_bar);
      }
      if (!ok) break;
      if (item.partial) {
        // publish this warp's rows of the slot: every lane's stores, then the flag
        __threadfence();
        __syncwarp();
        if (lane == 0) st_release_gpu(flags + (worker * 2 + (int)rank) * 8 + fslot, 1u);
      } else if (item.n_peers > 0) {
        __syncwarp();  // every lane has read the peers' slots
        if (lane == 0)
          for (int peer = 1; peer <= item.n_peers; ++peer) flags[((worker + peer) * 2 + (int)rank) * 8 + fslot] = 0u;
      }
      acc_it += MT;
    }
    if (lane == 0) ptx::bulk_wait_group_read<0>();  // staging must outlive the stores that read it
  }

  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_sync();  // neither CTA leaves while the other may still touch its shared memory
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
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
  int device;
  bool ready;
};
StaticScratch g_static[64];
std::mutex g_static_mu;

// In host code `g_static_scratch` is only a stand-in for the symbol; the address a
// kernel may use comes from cudaGetSymbolAddress, asked once per device with that
// device current.
int32_t static_scratch(StaticScratch** out) {
  int dev = 0;
  LEGO_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return LEGO_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticScratch& sc = g_static[dev];
  if (!sc.ready) {
    void* p = nullptr;
    LEGO_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    LEGO_CUDA_TRY(cudaDeviceGetAttribute(&sc.sm_count, cudaDevAttrMultiProcessorCount, dev));
    sc.dev = (unsigned char*)p;
    sc.device = dev;
    sc.ready = true;
  }
  *out = &sc;
  return LEGO_OK;
}

template <bool GROUPED>
int32_t configure(int dev) {
  static PerDeviceFlag done;
  if (done.test(dev)) return LEGO_OK;
  LEGO_CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<GROUPED>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  done.set(dev);
  return LEGO_OK;
}

// Set-up of one CTA-pair kernel on the current device: shared-memory limit and how many
// pairs the device can hold at once.  Both belong to the device, so they are kept per
// device ordinal.
constexpr int kMaxDevices = 64;
template <bool GROUPED, int MT>
int32_t configure_pair(int dev, int* max_clusters) {
  static PerDeviceFlag done;
  static int clusters[kMaxDevices];
  static std::mutex mu;
  if (dev < 0 || dev >= kMaxDevices) return LEGO_ERR_UNSUPPORTED;
  if (!done.test(dev)) {
    std::lock_guard<std::mutex> lock(mu);
    if (!done.test(dev)) {
      LEGO_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<GROUPED, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         pair_smem_bytes(MT)));
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(P_THREADS, 1, 1);
      cfg.dynamicSmemBytes = pair_smem_bytes(MT);
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      LEGO_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<GROUPED, MT>, &cfg));
      clusters[dev] = n;
      done.set(dev);
    }
  }
  *max_clusters = clusters[dev];
  return LEGO_OK;
}

// Do the flat tile ids g * n .. g * n + n - 1 of this problem share a tile column (they
// would share B) for every g?
bool ids_share_columns(const Problem& p, int n) {
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n;
  if (total < n || total % n || total > (1 << 22)) return false;
  for (int64_t t = 0; t < total; t += n) {
    int m0, n0;
    tile_coords(p, (int)t, &m0, &n0);
    for (int i = 1; i < n; ++i) {
      int m1, n1;
      tile_coords(p, (int)t + i, &m1, &n1);
      if (n1 != n0) return false;
    }
  }
  return true;
}

}  // namespace
extern std::atomic<int> g_lnbwd_split;      // layernorm_bwd.cu
extern std::atomic<int> g_lnbwd_lanes;      // layernorm_bwd.cu
extern std::atomic<int> g_lnbwd_fold;       // layernorm_bwd.cu
extern std::atomic<int> g_lnbwd_min_rows;   // layernorm_bwd.cu
extern std::atomic<int> g_lnbwd_foldw_groups;  // layernorm_bwd.cu
extern std::atomic<int> g_chunk_tile_vecs;  // permute.cu
extern std::atomic<int> g_dma_tile_bytes;   // permute.cu
extern std::atomic<int> g_dma_ctas_per_sm;  // permute.cu
extern std::atomic<int> g_dma_long_runs;    // permute.cu
extern std::atomic<int> g_pdl_last_wave;    // eval.cu
namespace {
// Tuning knobs (lego_tune), process-wide.
std::atomic<int> g_tune_blocks{0};   // 0: choose, 1: 256 x 256 pair tiles, 2: 512 x 256
std::atomic<int> g_tune_streamk{0};  // see make_sched
std::atomic<int> g_tune_lag{4};      // see Sched::lag

// Data-parallel over `tiles` pair tiles, or with the partial last wave cut along K.
Sched make_sched(int64_t tiles, int workers, int kblocks, int mt, void* workspace, int64_t workspace_bytes) {
  Sched sc = {};
  sc.total_tiles = (int32_t)tiles;
  sc.dp_tiles = (int32_t)tiles;
  sc.kblocks = kblocks;
  sc.lag = g_tune_lag.load();
  const int64_t need = kSkFlagBytes + (int64_t)workers * 2 * mt * kSkBlockFloats * 4;
  const int64_t rest = tiles % workers;
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15) || workers > kSkMaxWorkers ||
      g_tune_streamk.load() == 0 || rest == 0 || kblocks > (1 << 20))
    return sc;
  // Off unless asked for (LEGO_TUNE_GEMM_STREAMK).  The split balances the k-steps exactly but
  // it also takes the workers out of step: CTAs that share a B column block no longer walk K
  // together, so B is fetched from DRAM once per worker instead of once per wave.  Measured
  // on one box, sustained TFLOP/s with / without: 8192^3 1 175 / 1 200; 1024 x 8192 x 8192 (1.73
  // waves of 256 x 256 tiles, the case it was built for) 1 030 / 1 051, and 982 against 1 134
  // for 512 x 256 tiles that fit one wave.  Mode 1 splits only a poorly filled last wave.
  const int64_t waves = (tiles + workers - 1) / workers;
  if (g_tune_streamk.load() == 1 && (waves * workers - tiles) * 25 < waves * workers) return sc;
  const int64_t units = rest * kblocks;
  const int64_t run = (units + workers - 1) / workers;
  if (run < 4) return sc;  // a handful of k-steps per worker is not worth a fix-up
  sc.dp_tiles = (int32_t)(tiles - rest);
  sc.sk_tiles = (int32_t)rest;
  sc.sk_run = (int32_t)run;
  sc.workspace = reinterpret_cast<float*>(workspace);
  return sc;
}

template <bool GROUPED, int MT>
int32_t launch_pair(const Problem& p, const Problem* dev_table, int n_problems, int64_t tiles, int kblocks,
                    int activation, void* workspace, int64_t workspace_bytes, int dev, uint32_t* status,
                    cudaStream_t s, bool* launched) {
  *launched = false;
  int max_clusters = 0;
  const int32_t st = configure_pair<GROUPED, MT>(dev, &max_clusters);
  if (st != LEGO_OK || max_clusters < 1) return LEGO_OK;  // the caller falls back to one CTA per tile
  const int64_t n_pair_tiles = tiles / (2 * MT);
  Sched sc = make_sched(n_pair_tiles, max_clusters, kblocks, MT, GROUPED ? nullptr : workspace, workspace_bytes);
  const int workers = sc.sk_tiles ? max_clusters : (int)(n_pair_tiles < max_clusters ? n_pair_tiles : max_clusters);
  gemm_pair_kernel<GROUPED, MT><<<2 * workers, P_THREADS, pair_smem_bytes(MT), s>>>(p, dev_table, n_problems, sc,
                                                                                     activation, status);
  *launched = true;
  return cuda_status(cudaGetLastError());
}

// Build the problem records of a grouped GEMM into `table` (host), copy them to
// `dev_table` and launch on `s`.  A group without a tile order gets the reference's
// in-group order, row-major tiles (tile_m = t / tiles_n, tile_n = t % tiles_n), which the
// single-CTA kernel runs; CTA pairs are used when every group's order puts tiles 2p and
// 2p + 1 in one tile column, with 512 x 256 per pair when that holds for 4p .. 4p + 3
// (column-major in-group orders over a multiple of four tile rows).  Allocates nothing.
// The host table dies with the caller's frame, so the upload cannot be part of a stream
// capture: a captured copy node would read a dead frame on every replay.
int32_t run_grouped(EncodeFn enc, Problem* table, const void* const* A, const void* const* B, void* const* C,
                    const int64_t* mnk, int32_t G, const lego_layout_t* const* tile_orders, Problem* dev_table,
                    uint32_t* status, int sm_count, int dev, cudaStream_t s) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  LEGO_CUDA_TRY(cudaStreamIsCapturing(s, &cap));
  if (cap != cudaStreamCaptureStatusNone) return LEGO_ERR_UNSUPPORTED;
  int64_t total = 0;
  bool pairs = true, quads = true;
  for (int g = 0; g < G; ++g) {
    const lego_layout_t* order = tile_orders ? tile_orders[g] : nullptr;
    const int32_t st = fill_problem(enc, &table[g], A[g], B[g], C[g], mnk[3 * g], mnk[3 * g + 1], mnk[3 * g + 2],
                                    0, 0, order, (int)total);
    if (st != LEGO_OK) return st;
    Problem& p = table[g];
    pairs = pairs && ids_share_columns(p, 2);
    quads = quads && pairs && ids_share_columns(p, 4);
    total += (int64_t)p.tiles_m * p.tiles_n;
    if (total > 0x7fffffff) return LEGO_ERR_SIZE;
  }
  LEGO_CUDA_TRY(cudaMemcpyAsync(dev_table, table, (size_t)G * sizeof(Problem), cudaMemcpyHostToDevice, s));
  bool launched = false;
  const int blocks = g_tune_blocks.load();
  if (quads && blocks != 1) {  // 512 x 256 per SM pair whenever every group's order allows it
    const int32_t st = launch_pair<true, 2>(table[0], dev_table, G, total, 0, LEGO_ACT_NONE, nullptr, 0, dev, status, s,
                                            &launched);
    if (launched) return st;
  }
  if (pairs) {
    const int32_t st = launch_pair<true, 1>(table[0], dev_table, G, total, 0, LEGO_ACT_NONE, nullptr, 0, dev, status, s,
                                            &launched);
    if (launched) return st;
  }
  const int32_t st = configure<true>(dev);
  if (st != LEGO_OK) return st;
  const int grid = (int)(total < sm_count ? total : sm_count);
  gemm_kernel<true><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(table[0], dev_table, G, (int)total, LEGO_ACT_NONE, status);
  return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace lego

using namespace lego;

// Read (and clear, when set) the status word inside the static scratch of the current
// device, if lego_grouped_gemm_f16_static has been used there.  Allocates nothing.
namespace lego {
int32_t static_status_take(cudaStream_t s, uint32_t* word) {
  *word = 0;
  int dev = 0;
  LEGO_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return LEGO_OK;
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static[dev].ready) return LEGO_OK;
    base = g_static[dev].dev;
  }
  LEGO_CUDA_TRY(cudaMemcpyAsync(word, base, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
  LEGO_CUDA_TRY(cudaStreamSynchronize(s));
  if (*word) {
    LEGO_CUDA_TRY(cudaMemsetAsync(base, 0, sizeof(uint32_t), s));
    LEGO_CUDA_TRY(cudaStreamSynchronize(s));
  }
  return LEGO_OK;
}
}  // namespace lego

extern "C" {

// One GEMM, fp16 or e5m2 operands: CTA pairs when the tile order allows, else one CTA per tile.
static int32_t run_gemm(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int32_t trans_a,
                        int32_t trans_b, int32_t activation, const lego_layout_t* tile_order, int elem8,
                        void* workspace, int64_t workspace_bytes, void* stream) {
  if (activation != LEGO_ACT_NONE && activation != LEGO_ACT_LEAKY_RELU) return LEGO_ERR_UNSUPPORTED;
  if (workspace_bytes < 0) return LEGO_ERR_SIZE;
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
  const Geometry geo = geometry_of(p.elem8);
  const int kblocks = (int)((K + geo.bk - 1) / geo.bk);
  cudaStream_t s = (cudaStream_t)stream;
  // CTA pairs: the tile ids of a pair tile must share their tile column (they share B).
  const bool pairs = ids_share_columns(p, 2);
  if (pairs) {
    st = fill_problem(enc, &p, A, B, C, M, N, K, trans_a, trans_b, tile_order, 0, P_BN_HALF, elem8);
    if (st != LEGO_OK) return st;
    bool launched = false;
    // 512 x 256 per SM pair moves a quarter less operand data per flop (sustained on one box,
    // TFLOP/s: 8192^3 1 200 against 1 100; a 1024-row slab of it, 64 tall tiles on 74 pairs,
    // 1 134 against 1 051) but halves the number of work items: it is the choice from half a
    // wave of them.
    int max_tall = 0;
    const int blocks = g_tune_blocks.load();
    const bool tall_ok = blocks != 1 && ids_share_columns(p, 4) &&
                         configure_pair<false, 2>(ctx->device, &max_tall) == LEGO_OK && max_tall >= 1;
    if (tall_ok && (blocks == 2 || total / 4 >= max_tall / 2)) {
      st = launch_pair<false, 2>(p, nullptr, 1, total, kblocks, activation, workspace, workspace_bytes, ctx->device,
                                 ctx->status_word, s, &launched);
      if (launched) return st;
    }
    st = launch_pair<false, 1>(p, nullptr, 1, total, kblocks, activation, workspace, workspace_bytes, ctx->device,
                               ctx->status_word, s, &launched);
    if (launched) return st;
    st = fill_problem(enc, &p, A, B, C, M, N, K, trans_a, trans_b, tile_order, 0, BN, elem8);
    if (st != LEGO_OK) return st;
  }
  st = configure<false>(ctx->device);
  if (st != LEGO_OK) return st;
  const int grid = (int)(total < ctx->sm_count ? total : ctx->sm_count);
  gemm_kernel<false><<<grid, NUM_THREADS, SMEM_BYTES, s>>>(p, nullptr, 1, (int)total, activation, ctx->status_word);
  return cuda_status(cudaGetLastError());
}

int32_t lego_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                      int32_t trans_a, int32_t trans_b, int32_t activation,
                      const lego_layout_t* tile_order, void* stream) {
  return run_gemm(A, B, C, M, N, K, trans_a, trans_b, activation, tile_order, 0, nullptr, 0, stream);
}

int32_t lego_gemm_e5m2(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                       int32_t trans_a, int32_t trans_b, int32_t activation,
                       const lego_layout_t* tile_order, void* stream) {
  return run_gemm(A, B, C, M, N, K, trans_a, trans_b, activation, tile_order, 1, nullptr, 0, stream);
}

int64_t lego_gemm_workspace_bytes(void) {
  int32_t err = LEGO_OK;
  DeviceCtx* ctx = device_ctx(&err);
  if (!ctx) return 0;
  const int64_t workers = ctx->sm_count / 2;
  return kSkFlagBytes + workers * 2 * 2 * (int64_t)kSkBlockFloats * 4;
}

int32_t lego_gemm_f16_ws(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                         int32_t trans_a, int32_t trans_b, int32_t activation,
                         const lego_layout_t* tile_order, void* workspace, int64_t workspace_bytes, void* stream) {
  return run_gemm(A, B, C, M, N, K, trans_a, trans_b, activation, tile_order, 0, workspace, workspace_bytes, stream);
}

int32_t lego_gemm_e5m2_ws(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                          int32_t trans_a, int32_t trans_b, int32_t activation,
                          const lego_layout_t* tile_order, void* workspace, int64_t workspace_bytes, void* stream) {
  return run_gemm(A, B, C, M, N, K, trans_a, trans_b, activation, tile_order, 1, workspace, workspace_bytes, stream);
}


int32_t lego_tune(int32_t knob, int32_t value) {
  switch (knob) {
    case LEGO_TUNE_GEMM_BLOCKS:
      if (value < 0 || value > 2) return LEGO_ERR_SIZE;
      g_tune_blocks.store(value);
      return LEGO_OK;
    case LEGO_TUNE_GEMM_STREAMK:
      if (value < 0 || value > 2) return LEGO_ERR_SIZE;
      g_tune_streamk.store(value);
      return LEGO_OK;
    case LEGO_TUNE_PERMUTE_TILE_VECS:
      if (value < 64 || value > 6144) return LEGO_ERR_SIZE;
      g_chunk_tile_vecs.store(value);
      return LEGO_OK;
    case LEGO_TUNE_PERMUTE_DMA_TILE:
      if (value != 0 && (value < 2048 || value > 49152)) return LEGO_ERR_SIZE;
      g_dma_tile_bytes.store(value);
      return LEGO_OK;
    case LEGO_TUNE_PERMUTE_DMA_CTAS:
      if (value < 1 || value > 4) return LEGO_ERR_SIZE;
      g_dma_ctas_per_sm.store(value);
      return LEGO_OK;
    case LEGO_TUNE_PERMUTE_DMA_LONG:
      if (value < 0 || value > 1) return LEGO_ERR_SIZE;
      g_dma_long_runs.store(value);
      return LEGO_OK;
    case LEGO_TUNE_LNBWD_LANES:
      if (value < 0 || (value & 7) > 2 || value > 10) return LEGO_ERR_SIZE;
      g_lnbwd_lanes.store(value & 7);
      g_lnbwd_fold.store(value & 8 ? 0 : 1);
      return LEGO_OK;
    case LEGO_TUNE_LNBWD_FOLD_WARP:
      if (value < 0 || value > 3) return LEGO_ERR_SIZE;
      g_lnbwd_foldw_groups.store(value);
      return LEGO_OK;
    case LEGO_TUNE_LNBWD_MIN_ROWS:
      if (value < 1) return LEGO_ERR_SIZE;
      g_lnbwd_min_rows.store(value);
      return LEGO_OK;
    case LEGO_TUNE_PDL_LAST_WAVE:
      if (value < 0 || value > 1) return LEGO_ERR_SIZE;
      g_pdl_last_wave.store(value);
      return LEGO_OK;
    case LEGO_TUNE_LNBWD_SPLIT:
      if (value < 0) return LEGO_ERR_SIZE;
      g_lnbwd_split.store(value);
      return LEGO_OK;
    case LEGO_TUNE_GEMM_LAG:
      if (value < 0 || value > 4) return LEGO_ERR_SIZE;
      g_tune_lag.store(value);
      return LEGO_OK;
    default:
      return LEGO_ERR_UNSUPPORTED;
  }
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
                     ctx->sm_count, ctx->device, (cudaStream_t)stream);
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
  cudaStream_t s = (cudaStream_t)stream;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  LEGO_CUDA_TRY(cudaStreamIsCapturing(s, &cap));
  if (cap != cudaStreamCaptureStatusNone) return LEGO_ERR_UNSUPPORTED;  // before anything is enqueued
  Problem table[kStaticGroups];  // host stack: no heap, no device allocation anywhere in this call
  uint32_t* status = dev_status;
  if (!status) {
    // The word inside the array is read and cleared by lego_device_status; a code a previous
    // call left there stays until then (a kernel only records the first failure).
    status = reinterpret_cast<uint32_t*>(sc->dev);
  }
  Problem* dev_table = reinterpret_cast<Problem*>(sc->dev + kStaticStatusBytes);
  return run_grouped(enc, table, A, B, C, mnk, G, tile_orders, dev_table, status, sc->sm_count, sc->device, s);
}

}  // extern "C"
