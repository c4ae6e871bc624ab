// Layout reorganisation: out_flat[dst(idx)] = in_flat[src(idx)].
//
// Both layouts are folded to digit strides on the host and refined to a common
// digit set, which turns the pair into a digit permutation of the flat index.
// Three kernels cover it:
//   tiled  : the unit-stride digit differs between input and output; tiles go
//            through XOR-swizzled shared memory with 128-bit accesses to HBM on
//            both sides and conflict-free shared-memory phases;
//   gather : output-order copy with the widest vector the common unit-stride run
//            allows (also the fallback for digit sets the tiled kernel rejects);
//   staged : any layout pair, element by element through the staged interpreter.
// The tile a CTA moves is named by tile_order.inv(cta) when that layout is given.
#include <algorithm>
#include <cstring>

#include "common.cuh"
#include "ptx_sm100.cuh"
#include "staged.cuh"
#include "tma_host.cuh"

namespace lego {

namespace {

enum { KIND_STAGED = 0, KIND_GATHER = 1, KIND_TILED = 2, KIND_TMA = 3, KIND_CHUNK = 4, KIND_DMA = 5 };

constexpr int kThreads = 256;
constexpr int kVecPerThread = 4;
constexpr int kCtaVectors = kThreads * kVecPerThread;  // 16 KiB of 16-byte vectors per CTA
constexpr int kMaxTilesPerCta = 16;

struct TiledParams {
  DigitProgram p1;  // tile id -> tile coordinates
  DigitProgram p2;  // tile coordinates -> (input base, output base), in elements
  int64_t n_tiles;  // tiles this launch moves: ids tile_begin .. tile_begin + n_tiles - 1
  int64_t tile_begin;
  int64_t s_in_o;   // input stride of the output-fast digit (elements)
  int64_t s_out_i;  // output stride of the input-fast digit (elements)
  int32_t tiles_per_cta;
  int32_t log_ti;   // tile extent along the input-fast digit, log2 elements
  int32_t log_to;   // tile extent along the output-fast digit, log2 elements
  int32_t reserved;
};

struct GatherParams {
  DigitProgram g;   // output element offset -> input element offset
  int64_t n_vec;
  int32_t elems_per_vec;
  int32_t reserved;
};

struct TmaParams {
  DigitProgram p1;  // tile id -> tile coordinates
  DigitProgram p2;  // tile coordinates -> (input base, output base), in elements
  int64_t n_tiles;  // tiles this launch moves: ids tile_begin .. tile_begin + n_tiles - 1
  int64_t tile_begin;
  int64_t pitch;    // elements between consecutive rows of the input tensor map
  int64_t s_out_i;  // output stride of the input-contiguous digit (elements)
  int32_t stages;   // ring slots per CTA
  int32_t one_load; // 1: the tensor map is group-major, one TMA load fetches a whole tile
};

// Chunk-tiled permute: both sides share a contiguous run of rv 16-byte vectors (the
// innermost digit is the same on both sides), and a tile is made of the digits that
// continue that run on the input side plus the digits that continue it on the output
// side, so that a tile is read in long contiguous pieces, parked in shared memory, and
// written in long contiguous pieces.  Example: a 384^3 volume from row-major order into
// 8^3 bricks (benchmarks/cuda/bricks_f3d.py:10-13) -- the run is a brick row of 8 floats,
// the input continues with the brick index along z (48 bricks = 1536 contiguous bytes),
// the output with the rows and planes of the brick (2 KiB contiguous).
constexpr int kChunkMaxInner = 4;
constexpr int kChunkMaxVecs = 6144;  // most 16-byte vectors per tile (96 KiB of shared memory)
struct ChunkDigit {
  uint32_t radix;
  uint32_t w_smem;   // weight in the tile's input-order run index (position in shared memory / rv)
  uint32_t w_out;    // weight in the tile's output-order run index
  uint32_t reserved;
  FastDiv fd;
  uint32_t s_in;     // strides in 16-byte vectors (a tile spans less than 2^31 of them on either side)
  uint32_t s_out;
};
struct ChunkParams {
  DigitProgram p1;  // tile id -> outer coordinates
  DigitProgram p2;  // outer coordinates -> (input base, output base), in 16-byte vectors
  int64_t n_tiles;
  int32_t n_inner;
  int32_t rv;         // vectors per run
  int32_t tile_runs;  // runs per tile
  int32_t swizzle;    // 1: XOR the low bits of the shared-memory position with the output-order run index
  ChunkDigit by_in[kChunkMaxInner];   // inner digits, input-fastest first
  ChunkDigit by_out[kChunkMaxInner];  // the same digits, output-fastest first
};

// DMA permute: the same pairs of layouts as the chunk-tiled kernel (a common contiguous run
// shorter than a line), moved by the copy engine alone.  A tile is a box of digits; ONE tensor
// map per side describes the whole buffer with those digits as dimensions, in the same order on
// both sides (the order of the box in shared memory), each with its own stride on that side.  A
// tile is then one tiled TMA load (rows as long as the input allows) and one tiled TMA store
// from the same bytes: no thread touches the data.  Example, the 384^3 volume into 8^3 bricks:
// the box is [z 8][y 8][bx 8][x 8] floats = 16 KiB; the load map sees it as (x + bx merged: 64
// contiguous floats, y, z), the store map as (x, bx, y + z merged, by + bz merged).
constexpr int kDmaMaxOuter = 8;
struct DmaOuter {   // a digit of the tile id
  FastDiv fd;
  uint32_t radix;
  int32_t ld_dim, ld_mul;  // tensor-map dimension it moves on the load side, coordinate units per step
  int32_t st_dim, st_mul;  // the same on the store side
};
struct DmaParams {
  int64_t n_tiles;
  int32_t n_outer;
  int32_t ld_rank, st_rank;
  int32_t stages;
  uint32_t tile_bytes;  // bytes of one box
  uint32_t slot_bytes;  // pitch of the ring slots (tile_bytes rounded up to 128)
  DmaOuter o[kDmaMaxOuter];
};
struct DmaMapSpec {     // host side: the arguments of the tensor-map encoder, in elements
  int rank;
  uint64_t size[5];
  uint64_t stride[5];
  uint32_t box[5];
};

struct Plan {
  int kind;
  bool by_order;  // tile ids are the ids of the caller's tile_order layout
  int elem_bytes;
  int vec_bytes;
  int64_t size;
  int64_t tile_in, tile_out;
  TiledParams tiled;
  TmaParams tma;
  GatherParams gather;
  ChunkParams chunk;
  DmaParams dma;
  DmaMapSpec dma_ld, dma_st;
  int dma_elem_bytes;  // element size the maps are written in (16-byte elements count as two of 8)
  StagedProgram staged_src, staged_dst;
};

template <bool WIDE>
__device__ __forceinline__ uint64_t term_eval(const DigitTerm& t, uint64_t x) {
  if (WIDE) {
    uint64_t q = t.a64 > 1 ? x / t.a64 : x;
    if (t.m64) q %= t.m64;
    return q * t.b;
  } else {
    uint32_t q = fd_div((uint32_t)x, t.a);
    if (t.m.d) q -= fd_div(q, t.m) * t.m.d;
    return (uint64_t)q * t.b;
  }
}

template <int BYTES> struct VecT;
template <> struct VecT<1> { using type = uint8_t; };
template <> struct VecT<2> { using type = uint16_t; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<8> { using type = uint2; };
template <> struct VecT<16> { using type = uint4; };

// ---- chunk-tiled permute ---------------------------------------------------------

template <bool WIDE>
__global__ void __launch_bounds__(kThreads, 3)
chunk_permute_kernel(const __grid_constant__ ChunkParams P, const uint4* __restrict__ in, uint4* __restrict__ out) {
  extern __shared__ uint4 chunk_tile[];
  __shared__ int64_t base[2];
  if (threadIdx.x == 0) {
    const uint64_t t = blockIdx.x;
    uint64_t coord[LEGO_MAX_RANK];
    for (int k = 0; k < LEGO_MAX_RANK; ++k) coord[k] = 0;
    for (int j = 0; j < P.p1.n_terms; ++j) coord[P.p1.t[j].dst] += term_eval<WIDE>(P.p1.t[j], t);
    uint64_t b0 = 0, b1 = 0;
    for (int j = 0; j < P.p2.n_terms; ++j) {
      const uint64_t v = term_eval<WIDE>(P.p2.t[j], coord[P.p2.t[j].src]);
      if (P.p2.t[j].dst == 0) b0 += v; else b1 += v;
    }
    base[0] = (int64_t)b0;
    base[1] = (int64_t)b1;
  }
  __syncthreads();
  const uint4* src = in + base[0];
  uint4* dst = out + base[1];
  const int rv = P.rv, n = P.n_inner;
  const uint32_t mask = P.swizzle ? 7u : 0u;
  // phase 1: runs in input order (contiguous global reads); position in shared memory = run index * rv.
  // Four runs per thread and step: all their loads are issued before the first is parked.
  constexpr int UNROLL = 4;
  for (uint32_t r0 = threadIdx.x; r0 < (uint32_t)P.tile_runs; r0 += UNROLL * kThreads) {
    uint32_t off[UNROLL];
    uint32_t tw[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      uint32_t rest = r0 + u * kThreads, w = 0;
      off[u] = 0;
#pragma unroll
      for (int k = 0; k < kChunkMaxInner; ++k) {
        if (k < n) {
          const ChunkDigit& d = P.by_in[k];
          const uint32_t q = (k + 1 < n) ? fd_div(rest, d.fd) : 0u;
          const uint32_t v = (k + 1 < n) ? rest - q * d.radix : rest;
          rest = q;
          off[u] += v * d.s_in;
          w += v * d.w_out;
        }
      }
      tw[u] = (w * (uint32_t)rv) & mask;
    }
    if (rv == 2) {
      uint4 v[UNROLL][2];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (r0 + u * kThreads < (uint32_t)P.tile_runs) {
          v[u][0] = __ldcs(src + off[u]);
          v[u][1] = __ldcs(src + off[u] + 1);
        }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (r0 + u * kThreads < (uint32_t)P.tile_runs) {
          const uint32_t pos = (r0 + u * kThreads) * 2u;
          chunk_tile[pos ^ tw[u]] = v[u][0];
          chunk_tile[(pos + 1) ^ tw[u]] = v[u][1];
        }
    } else {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
        if (r0 + u * kThreads < (uint32_t)P.tile_runs) {
          const uint32_t pos = (r0 + u * kThreads) * (uint32_t)rv;
          for (int x = 0; x < rv; ++x) chunk_tile[(pos + x) ^ tw[u]] = __ldcs(src + off[u] + x);
        }
    }
  }
  __syncthreads();
  // phase 2: runs in output order (contiguous global writes)
  for (uint32_t q0 = threadIdx.x; q0 < (uint32_t)P.tile_runs; q0 += kThreads) {
    uint32_t rest = q0, r = 0, off = 0;
#pragma unroll
    for (int k = 0; k < kChunkMaxInner; ++k) {
      if (k < n) {
        const ChunkDigit& d = P.by_out[k];
        const uint32_t q = (k + 1 < n) ? fd_div(rest, d.fd) : 0u;
        const uint32_t v = (k + 1 < n) ? rest - q * d.radix : rest;
        rest = q;
        off += v * d.s_out;
        r += v * d.w_smem;
      }
    }
    const uint32_t pos = r * (uint32_t)rv, tw = (q0 * (uint32_t)rv) & mask;
    for (int x = 0; x < rv; ++x) __stcs(dst + off + x, chunk_tile[(pos + x) ^ tw]);
  }
}

// ---- DMA permute: tiled TMA load -> shared memory -> tiled TMA store ------------------
//
// Two threads per CTA do everything.  The loader walks this CTA's tiles (dealt round-robin),
// waits for a free ring slot and issues one TMA load per tile; the storer waits for the
// bytes, issues one TMA store from the same slot, and hands the slot back once the store has
// read it (at most kDmaStoresInFlight stores are reading at a time, the rest of the ring is
// loads in flight).  Several CTAs share an SM, so that issue latencies overlap.

constexpr int kDmaThreads = 64;
constexpr int kDmaMaxStages = 12;
constexpr int kDmaStoresInFlight = 2;
constexpr long long kDmaWaitLimit = 2000000000LL;  // SM cycles, about a second

struct DmaCtl {
  uint64_t full[kDmaMaxStages];
  uint64_t empty[kDmaMaxStages];
  uint32_t abort_flag;
};

template <bool STORE>
__device__ __forceinline__ void dma_coords(const DmaParams& P, uint32_t t, int32_t (&c)[5]) {
#pragma unroll
  for (int k = 0; k < 5; ++k) c[k] = 0;
  uint32_t rest = t;
#pragma unroll
  for (int j = 0; j < kDmaMaxOuter; ++j) {
    if (j < P.n_outer) {
      const DmaOuter& o = P.o[j];
      const uint32_t q = (j + 1 < P.n_outer) ? fd_div(rest, o.fd) : 0u;
      const uint32_t v = rest - q * o.radix;
      rest = q;
      const int dim = STORE ? o.st_dim : o.ld_dim;
      const int32_t add = (int32_t)v * (STORE ? o.st_mul : o.ld_mul);
#pragma unroll
      for (int k = 0; k < 5; ++k) c[k] += (k == dim) ? add : 0;
    }
  }
}

__global__ void __launch_bounds__(kDmaThreads)
dma_permute_kernel(const __grid_constant__ CUtensorMap ld_map, const __grid_constant__ CUtensorMap st_map,
                   const __grid_constant__ DmaParams P, uint32_t* status) {
  extern __shared__ uint8_t dsm_raw[];
  const uint32_t raw = ptx::smem_u32(dsm_raw);
  uint8_t* slots = dsm_raw + (((raw + 127u) & ~127u) - raw);
  DmaCtl* ctl = reinterpret_cast<DmaCtl*>(slots + (size_t)P.stages * P.slot_bytes);
  volatile uint32_t* abort_flag = &ctl->abort_flag;
  const int stages = P.stages;
  const int64_t my_tiles =
      P.n_tiles > blockIdx.x ? (P.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 1);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
  ptx::launch_dependents();
  ptx::grid_dependency_wait();

  if (threadIdx.x == 0) {
    // ---------------- loader ----------------
    int s = 0;
    uint32_t use = 0;  // times the ring has wrapped
    uint32_t t = blockIdx.x;
    int64_t issued = 0;
    for (int64_t n = 0; n < my_tiles; ++n, t += gridDim.x) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[s]), (use & 1) ^ 1, abort_flag, kDmaWaitLimit)) {
        *abort_flag = 1;
        atomicCAS(status, 0u, 0xA0000u | (uint32_t)s);
        break;
      }
      int32_t c[5];
      dma_coords<false>(P, t, c);
      const uint32_t full = ptx::smem_u32(&ctl->full[s]);
      ptx::mbar_arrive_expect_tx(full, P.tile_bytes);
      ptx::tma_load_nd(P.ld_rank, ptx::smem_u32(slots + (size_t)s * P.slot_bytes), &ld_map, c, full);
      ++issued;
      if (++s == stages) { s = 0; ++use; }
    }
    if (*abort_flag) {
      // leave no load of ours in flight: the last one issued into every slot
      uint32_t never = 0;
      for (int k = 0; k < stages && k < issued; ++k) {
        const int64_t last = issued - 1 - k;  // the k-th most recent load
        ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[last % stages]), (uint32_t)((last / stages) & 1), &never,
                               kDmaWaitLimit);
      }
    }
  } else if (threadIdx.x == 32) {
    // ---------------- storer ----------------
    int s = 0, s_free = 0;
    uint32_t use = 0;
    uint32_t t = blockIdx.x;
    for (int64_t n = 0; n < my_tiles; ++n, t += gridDim.x) {
      if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), use & 1, abort_flag, kDmaWaitLimit)) {
        *abort_flag = 1;
        atomicCAS(status, 0u, 0xB0000u | (uint32_t)s);
        break;
      }
      int32_t c[5];
      dma_coords<true>(P, t, c);
      ptx::tma_store_nd(P.st_rank, &st_map, c, ptx::smem_u32(slots + (size_t)s * P.slot_bytes));
      ptx::bulk_commit_group();
      ptx::bulk_wait_group_read<kDmaStoresInFlight>();
      if (n >= kDmaStoresInFlight) {  // the store of tile n - kDmaStoresInFlight has read its slot
        ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[s_free]));
        if (++s_free == stages) s_free = 0;
      }
      if (++s == stages) { s = 0; ++use; }
    }
    ptx::bulk_wait_group<0>();  // shared memory must outlive the stores, and the writes end with the grid
  }
}

// ---- gather: thread per output vector ------------------------------------------

template <int VB, bool WIDE>
__global__ void __launch_bounds__(kThreads)
gather_kernel(const __grid_constant__ GatherParams P, const uint8_t* __restrict__ in,
              uint8_t* __restrict__ out) {
  using V = typename VecT<VB>::type;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < P.n_vec; v += step) {
    const uint64_t x = (uint64_t)v * (uint32_t)P.elems_per_vec;
    uint64_t src = 0;
    for (int j = 0; j < P.g.n_terms; ++j) src += term_eval<WIDE>(P.g.t[j], x);
    const V val = reinterpret_cast<const V*>(in)[src / (uint32_t)P.elems_per_vec];
    reinterpret_cast<V*>(out)[v] = val;
  }
}

// ---- staged: any pair of layouts -----------------------------------------------

template <int EB>
__global__ void __launch_bounds__(kThreads)
staged_permute_kernel(const __grid_constant__ StagedProgram src, const __grid_constant__ StagedProgram dst,
                      const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int64_t n) {
  using V = typename VecT<EB>::type;
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const int64_t s = staged_apply(src, i);
    const int64_t d = staged_apply(dst, i);
    reinterpret_cast<V*>(out)[d] = reinterpret_cast<const V*>(in)[s];
  }
}

// ---- tiled transpose -------------------------------------------------------------
//
// A tile is TI elements along the digit that is contiguous in the input times TO
// elements along the digit that is contiguous in the output.  Shared memory holds
// it output-major: row i (TO contiguous elements), the 16-byte column c of row i
// stored at column c ^ f(i), f(i) = (i / VE) mod min(8, TO / VE).  Phase one
// (global -> shared) has each group of 8 lanes read 128 contiguous bytes of one
// input row and scatter elements down a shared-memory column: the XOR puts the 8
// lanes of a group on distinct 16-byte bank groups and the 4 rows of a warp on the
// 4 words inside a bank group.  Phase two reads whole 16-byte columns of a row.

template <int EB, bool WIDE>
__global__ void __launch_bounds__(kThreads)
tiled_transpose_kernel(const __grid_constant__ TiledParams P, const uint8_t* __restrict__ in,
                       uint8_t* __restrict__ out) {
  using E = typename VecT<EB>::type;
  constexpr int VE = 16 / EB;
  constexpr int LOG_VE = (VE == 1) ? 0 : (VE == 2) ? 1 : (VE == 4) ? 2 : (VE == 8) ? 3 : 4;
  __shared__ uint4 tile_mem[kCtaVectors];
  __shared__ int64_t base_in[kMaxTilesPerCta];
  __shared__ int64_t base_out[kMaxTilesPerCta];

  const int tid = threadIdx.x;
  const int log_ti = P.log_ti, log_to = P.log_to;
  const int log_nvi = log_ti - LOG_VE;                 // vectors per input row of a tile
  const int log_nvo = log_to - LOG_VE;                 // vectors per output row of a tile
  const int log_vpt = log_ti + log_to - LOG_VE;        // vectors per tile
  const int log_ci = log_nvi < 3 ? log_nvi : 3;        // lanes that walk one input row
  const int fmask = (log_nvo < 3 ? (1 << log_nvo) : 8) - 1;
  const int G = P.tiles_per_cta;

  if (tid < G) {
    const int64_t t = (int64_t)blockIdx.x * G + tid;
    int64_t bi = -1, bo = -1;
    if (t < P.n_tiles) {
      uint64_t coord[LEGO_MAX_RANK];
      for (int k = 0; k < LEGO_MAX_RANK; ++k) coord[k] = 0;
      for (int j = 0; j < P.p1.n_terms; ++j)
        coord[P.p1.t[j].dst] += term_eval<WIDE>(P.p1.t[j], (uint64_t)(t + P.tile_begin));
      uint64_t b0 = 0, b1 = 0;
      for (int j = 0; j < P.p2.n_terms; ++j) {
        const uint64_t v = term_eval<WIDE>(P.p2.t[j], coord[P.p2.t[j].src]);
        if (P.p2.t[j].dst == 0) b0 += v; else b1 += v;
      }
      bi = (int64_t)b0;
      bo = (int64_t)b1;
    }
    base_in[tid] = bi;
    base_out[tid] = bo;
  }
  __syncthreads();

  uint4 reg[kVecPerThread];
  bool ok[kVecPerThread];
#pragma unroll
  for (int k = 0; k < kVecPerThread; ++k) {
    const int gv = k * kThreads + tid;
    const int g = gv >> log_vpt;
    const int vi = gv & ((1 << log_vpt) - 1);
    ok[k] = (g < G) && (base_in[g < kMaxTilesPerCta ? g : 0] >= 0);
    if (ok[k]) {
      const int a = vi & ((1 << log_ci) - 1);
      const int o = (vi >> log_ci) & ((1 << log_to) - 1);
      const int c = vi >> (log_ci + log_to);
      const int iv = (c << log_ci) + a;
      const int64_t off = base_in[g] + (int64_t)o * P.s_in_o + ((int64_t)iv << LOG_VE);
      reg[k] = *reinterpret_cast<const uint4*>(in + off * EB);
    }
  }
#pragma unroll
  for (int k = 0; k < kVecPerThread; ++k) {
    if (!ok[k]) continue;
    const int gv = k * kThreads + tid;
    const int g = gv >> log_vpt;
    const int vi = gv & ((1 << log_vpt) - 1);
    const int a = vi & ((1 << log_ci) - 1);
    const int o = (vi >> log_ci) & ((1 << log_to) - 1);
    const int c = vi >> (log_ci + log_to);
    const int iv = (c << log_ci) + a;
    E* tile = reinterpret_cast<E*>(tile_mem + ((size_t)g << log_vpt));
    const E* src = reinterpret_cast<const E*>(&reg[k]);
    const int f = iv & fmask;  // (i / VE) mod fm is the same for the VE elements of this vector
    const int col = (((o >> LOG_VE) ^ f) << LOG_VE) + (o & (VE - 1));
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int i = (iv << LOG_VE) + e;
      tile[(i << log_to) + col] = src[e];
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < kVecPerThread; ++k) {
    const int gv = k * kThreads + tid;
    const int g = gv >> log_vpt;
    const int vi = gv & ((1 << log_vpt) - 1);
    if (g >= G || base_out[g < kMaxTilesPerCta ? g : 0] < 0) continue;
    const int ov = vi & ((1 << log_nvo) - 1);
    const int i = vi >> log_nvo;
    const int f = (i >> LOG_VE) & fmask;
    const uint4 w = tile_mem[((size_t)g << log_vpt) + ((size_t)i << log_nvo) + (ov ^ f)];
    const int64_t off = base_out[g] + (int64_t)i * P.s_out_i + ((int64_t)ov << LOG_VE);
    *reinterpret_cast<uint4*>(out + off * EB) = w;
  }
}


// ---- TMA-fed transpose ---------------------------------------------------------------
//
// Persistent CTAs of ten warps.  A tile is 128 bytes along the input-contiguous digit
// times 8 * (16 / EB) rows (32 x 32 fp32, 64 x 64 fp16, 16 x 16 fp64).
//   planner   (1 warp)  evaluates tile_order.inv and both layouts' strides for 32
//             tiles at a time, one tile per lane, fully converged, into a queue;
//   producer  (1 warp, lane l owns ring slot l, lanes in lock step)  takes queue entries
//             a round of slots at a time: waits for the slot, publishes the tile's output
//             offset and issues one TMA load (128-byte swizzle) through a 3-D map whose
//             box gathers every (16/EB)-th row into one 8-row block of the slot (or
//             16/EB loads through the row-group map if the driver refuses that map);
//   consumers (8 warps, in pairs)  read a (16/EB) x (16/EB) block per thread with
//             conflict-free 128-bit shared-memory loads, transpose it in registers
//             and write 128-bit vectors; a quarter-warp fills one whole output line.
// Tiles are dealt to CTAs round-robin in tile-order sequence.

constexpr int kTmaStages = 32;   // one producer lane per slot
constexpr int kTmaConsumerWarps = 8;
constexpr int kTmaThreads = 32 * (2 + kTmaConsumerWarps);
constexpr int kPlanBatch = 32;
constexpr long long kTmaWaitLimit = 2000000000LL;  // SM cycles, about a second

struct PlanEntry {
  int64_t out_base;
  int32_t cx, cy;   // tensor-map coordinates of the tile; cx < 0: no tile (ragged end)
};

struct TmaCtl {
  uint64_t full[kTmaStages];
  uint64_t empty[kTmaStages];
  uint64_t plan_full[2];
  uint64_t plan_empty[2];
  int64_t out_base[kTmaStages];
  PlanEntry plan[2][kPlanBatch];
  uint32_t abort_flag;
};

template <int EB, bool WIDE>
__global__ void __launch_bounds__(kTmaThreads)
tma_transpose_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ TmaParams P,
                     uint8_t* __restrict__ out, uint32_t* status) {
  constexpr int VE = 16 / EB;            // elements per 16-byte vector
  constexpr int ROWS = 8 * VE;           // tile rows (along the output-contiguous digit)
  constexpr int TILE_BYTES = ROWS * 128;
  extern __shared__ uint8_t tsm_raw[];
  const uint32_t raw = ptx::smem_u32(tsm_raw);
  uint8_t* tiles = tsm_raw + (((raw + 1023u) & ~1023u) - raw);
  TmaCtl* ctl = reinterpret_cast<TmaCtl*>(tiles + P.stages * TILE_BYTES);
  volatile uint32_t* abort_flag = &ctl->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = P.stages;  // ring slots in use (<= kTmaStages)
  // tiles are dealt round-robin: the n-th tile of this CTA has id blockIdx.x + n * gridDim.x
  const int64_t my_tiles =
      P.n_tiles > blockIdx.x ? (P.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  auto tile_id = [&](int64_t n) { return blockIdx.x + n * (int64_t)gridDim.x; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&ctl->full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->empty[s]), 2);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(ptx::smem_u32(&ctl->plan_full[b]), 1);
      ptx::mbar_init(ptx::smem_u32(&ctl->plan_empty[b]), 1);
    }
    ctl->abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async();
  }
  __syncthreads();
  // Let the next grid of the stream start its own set-up now; and touch global memory only
  // once the previous grid is complete.  The planner warp works from kernel parameters and
  // shared memory alone, so it runs ahead of that wait.
  ptx::launch_dependents();
  if (warp != kTmaConsumerWarps + 1) ptx::grid_dependency_wait();

  if (warp == kTmaConsumerWarps + 1) {
    // ---------------- planner: one tile per lane, 32 tiles per batch ----------------
    const int64_t batches = (my_tiles + kPlanBatch - 1) / kPlanBatch;
    for (int64_t k = 0; k < batches; ++k) {
      const int b = (int)(k & 1);
      bool ok = true;
      if (lane == 0)
        ok = ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->plan_empty[b]), (uint32_t)(((k >> 1) & 1) ^ 1), abort_flag,
                                    kTmaWaitLimit);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) {
        if (lane == 0) { *abort_flag = 1; atomicCAS(status, 0u, 0x80000u | (uint32_t)b); }
        break;
      }
      const int64_t n = k * kPlanBatch + lane;
      PlanEntry e;
      e.out_base = 0;
      e.cx = -1;
      e.cy = 0;
      const int64_t t = tile_id(n);
      if (n < my_tiles && t < P.n_tiles) {
        uint64_t coord[LEGO_MAX_RANK];
#pragma unroll
        for (int c = 0; c < LEGO_MAX_RANK; ++c) coord[c] = 0;
        for (int j = 0; j < P.p1.n_terms; ++j) {
          const uint64_t v = term_eval<WIDE>(P.p1.t[j], (uint64_t)(t + P.tile_begin));
          const int dst = P.p1.t[j].dst;
#pragma unroll
          for (int c = 0; c < LEGO_MAX_RANK; ++c)
            if (c == dst) coord[c] += v;
        }
        uint64_t b_in = 0, b_out = 0;
        for (int j = 0; j < P.p2.n_terms; ++j) {
          const int src = P.p2.t[j].src;
          uint64_t x = 0;
#pragma unroll
          for (int c = 0; c < LEGO_MAX_RANK; ++c)
            if (c == src) x = coord[c];
          const uint64_t v = term_eval<WIDE>(P.p2.t[j], x);
          if (P.p2.t[j].dst == 0) b_in += v; else b_out += v;
        }
        e.out_base = (int64_t)b_out;
        if (WIDE) {
          e.cx = (int32_t)(b_in % (uint64_t)P.pitch);
          e.cy = (int32_t)(b_in / (uint64_t)P.pitch);
        } else {
          e.cy = (int32_t)((uint32_t)b_in / (uint32_t)P.pitch);
          e.cx = (int32_t)((uint32_t)b_in - (uint32_t)e.cy * (uint32_t)P.pitch);
        }
      }
      ctl->plan[b][lane] = e;
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->plan_full[b]));
    }
    return;
  }

  if (warp == kTmaConsumerWarps) {
    // ---------------- producer: lane l owns ring slot l ----------------
    // The lanes work in lock step, one round of `stages` tiles at a time, so the latencies of
    // the plan read, the barrier polls and the TMA issue overlap across up to 32 tiles
    // instead of adding up in one thread; no per-tile division is needed either.
    uint32_t uses = 0;       // loads this lane has issued into its slot
    bool failed = false;
    for (int64_t base = 0; base < my_tiles; base += stages) {
      const int64_t n = base + lane;
      const bool active = lane < stages && n < my_tiles;
      const int64_t k = n / kPlanBatch;
      const int b = (int)(k & 1), q = (int)(n % kPlanBatch);
      if (active) {
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->plan_full[b]), (uint32_t)((k >> 1) & 1), abort_flag,
                                    kTmaWaitLimit)) {
          *abort_flag = 1;
          atomicCAS(status, 0u, 0x90000u | (uint32_t)b);
          failed = true;
        }
      }
      if (__any_sync(0xffffffffu, failed)) break;
      if (active) {
        const PlanEntry e = ctl->plan[b][q];
        if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->empty[lane]), (uses & 1) ^ 1, abort_flag, kTmaWaitLimit)) {
          *abort_flag = 1;
          atomicCAS(status, 0u, 0x60000u | (uint32_t)lane);
          failed = true;
        } else {
          ctl->out_base[lane] = e.out_base;
          const uint32_t full = ptx::smem_u32(&ctl->full[lane]);
          ptx::mbar_arrive_expect_tx(full, TILE_BYTES);
          // rows k, k + VE, k + 2 VE, ... of the tile go to the k-th 8-row group of the slot
          if (P.one_load) {
            ptx::tma_load_3d(ptx::smem_u32(tiles + lane * TILE_BYTES), &tmap, e.cx, e.cy / VE, 0, full);
          } else {
#pragma unroll
            for (int kk = 0; kk < VE; ++kk)
              ptx::tma_load_3d(ptx::smem_u32(tiles + lane * TILE_BYTES + kk * 1024), &tmap, e.cx, kk, e.cy / VE, full);
          }
          ++uses;
        }
      }
      __syncwarp();  // every lane has read its plan entry before a batch is handed back
      if (active && (q == kPlanBatch - 1 || n + 1 == my_tiles)) ptx::mbar_arrive(ptx::smem_u32(&ctl->plan_empty[b]));
      if (__any_sync(0xffffffffu, failed)) break;
    }
    if (*abort_flag && uses) {
      // leave no copy of ours in flight: the last load into this lane's slot
      uint32_t never = 0;
      ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[lane]), (uses - 1) & 1, &never, kTmaWaitLimit);
    }
    return;
  }

  // ---------------- consumers: warp pair p takes tiles n = p, p + 4, ... ----------------
  const int pair = warp >> 1;
  // Thread (rb, cb) owns rows rb * VE .. rb * VE + VE - 1 of the tile and its cb-th
  // 16-byte column.  Row rb * VE + k sits at row rb of the slot's k-th group, stored at
  // 16-byte position cb ^ rb, so the eight lanes of a quarter-warp (same cb, rb = 0..7)
  // read eight distinct bank groups; the same eight lanes then write one whole
  // 128-byte line of the output.
  const int rb = lane & 7;
  const int cb = ((warp & 1) << 2) + (lane >> 3);
  // The slot count is a multiple of the pair count: this pair walks slots pair, pair + pairs, ...
  int s = pair;
  uint32_t use = 0;
  for (int64_t n = pair; n < my_tiles; n += kTmaConsumerWarps / 2, s += kTmaConsumerWarps / 2) {
    if (s >= stages) {
      s -= stages;
      ++use;
    }
    if (!ptx::mbar_wait_bounded(ptx::smem_u32(&ctl->full[s]), use & 1, abort_flag, kTmaWaitLimit)) {
      *abort_flag = 1;
      atomicCAS(status, 0u, 0x70000u | (uint32_t)s);
      break;
    }
    const int64_t ob = ctl->out_base[s];
    const uint4* tile = reinterpret_cast<const uint4*>(tiles + s * TILE_BYTES);
    uint4 r[VE];
#pragma unroll
    for (int k = 0; k < VE; ++k) r[k] = tile[(k * 8 + rb) * 8 + (cb ^ rb)];
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&ctl->empty[s]));
    uint4 w[VE];
    if (EB == 4) {
      const uint32_t* a0 = reinterpret_cast<const uint32_t*>(&r[0]);
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        uint32_t* d = reinterpret_cast<uint32_t*>(&w[e]);
#pragma unroll
        for (int k = 0; k < VE; ++k) d[k] = a0[k * 4 + e];
      }
    } else if (EB == 8) {
      const uint2* a0 = reinterpret_cast<const uint2*>(&r[0]);
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        uint2* d = reinterpret_cast<uint2*>(&w[e]);
#pragma unroll
        for (int k = 0; k < VE; ++k) d[k] = a0[k * 2 + e];
      }
    } else {  // EB == 2: 8 x 8 block of 16-bit elements, two source rows per output word
      const uint32_t* a0 = reinterpret_cast<const uint32_t*>(&r[0]);
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        uint32_t* d = reinterpret_cast<uint32_t*>(&w[e]);
#pragma unroll
        for (int k2 = 0; k2 < VE / 2; ++k2)
          d[k2] = __byte_perm(a0[(2 * k2) * 4 + e / 2], a0[(2 * k2 + 1) * 4 + e / 2], (e & 1) ? 0x7632 : 0x5410);
      }
    }
    uint8_t* obase = out + (ob + (int64_t)rb * VE) * EB;
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int i = cb * VE + e;
      __stcs(reinterpret_cast<uint4*>(obase + (int64_t)i * P.s_out_i * EB), w[e]);
    }
  }
}

// ---- planning --------------------------------------------------------------------

bool is_pow2(int64_t x) { return x > 0 && (x & (x - 1)) == 0; }
int ilog2(int64_t x) { int l = 0; while (((int64_t)1 << l) < x) ++l; return l; }
bool aligned(const void* p, int a) { return ((uintptr_t)p % (uintptr_t)a) == 0; }

int32_t same_domain(const lego_layout_t* a, const lego_layout_t* b) {
  if (a->rank != b->rank) return LEGO_ERR_DOMAIN;
  for (int k = 0; k < a->rank; ++k)
    if (a->dims[k] != b->dims[k]) return LEGO_ERR_DOMAIN;
  return LEGO_OK;
}

void plan_gather(const std::vector<PairDigit>& merged, int64_t size, int eb, const void* in,
                 const void* out, Plan* pl) {
  // run = length of the stretch that is contiguous on both sides
  int64_t run = 1;
  for (const PairDigit& d : merged)
    if (d.sa == 1 && d.sb == 1) run = d.radix;
  int vb = 16;
  while (vb > eb && ((run * eb) % vb != 0 || !aligned(in, vb) || !aligned(out, vb))) vb >>= 1;
  if (vb < eb) vb = eb;
  pl->kind = KIND_GATHER;
  pl->vec_bytes = vb;
  GatherParams& gp = pl->gather;
  std::memset(&gp, 0, sizeof(gp));
  gp.elems_per_vec = vb / eb;
  gp.n_vec = size / gp.elems_per_vec;
  gp.g.n_src = 1;
  gp.g.n_dst = 1;
  gp.g.wide = size > ((int64_t)1 << 31) ? 1 : 0;
  for (const PairDigit& d : merged) {
    if (d.radix == 1) continue;
    const bool top = (d.sb * d.radix == size);
    set_term(&gp.g.t[gp.g.n_terms++], 0, 0, d.sb, top ? 0 : d.radix, d.sa);
  }
  pl->tile_in = run;
  pl->tile_out = run;
}

// Fill the tiled plan for an in-tile pair (I: sa == 1, O: sb == 1) and the outer
// programs already stored in pl->tiled; false if the shape does not qualify.
bool finish_tiled(int64_t ti, int64_t to, int64_t s_out_i, int64_t s_in_o, int eb, const void* in,
                  const void* out, Plan* pl) {
  const int ve = 16 / eb;
  if (!is_pow2(ti) || !is_pow2(to) || ti < ve || to < ve) return false;
  const int64_t vpt = ti * to / ve;
  if (vpt > kCtaVectors) return false;
  if (!aligned(in, 16) || !aligned(out, 16)) return false;
  if ((s_out_i * eb) % 16 || (s_in_o * eb) % 16) return false;
  TiledParams& tp = pl->tiled;
  for (int j = 0; j < tp.p2.n_terms; ++j)
    if ((tp.p2.t[j].b * (uint64_t)eb) % 16) return false;
  int64_t g = kCtaVectors / vpt;
  if (g > kMaxTilesPerCta) g = kMaxTilesPerCta;
  if (g > tp.n_tiles) g = tp.n_tiles;
  tp.tiles_per_cta = (int32_t)g;
  tp.log_ti = ilog2(ti);
  tp.log_to = ilog2(to);
  tp.s_in_o = s_in_o;
  tp.s_out_i = s_out_i;
  pl->kind = KIND_TILED;
  pl->vec_bytes = 16;
  pl->tile_in = ti;
  pl->tile_out = to;
  // The TMA-fed kernel takes tiles of exactly 128 bytes x 8 vectors.
  if ((eb == 2 || eb == 4 || eb == 8) && ti * eb == 128 && to == 8 * ve && s_in_o < ((int64_t)1 << 31) &&
      pl->size / s_in_o < ((int64_t)1 << 31)) {
    pl->kind = KIND_TMA;
    pl->tma.p1 = tp.p1;
    pl->tma.p2 = tp.p2;
    pl->tma.n_tiles = tp.n_tiles;
    pl->tma.tile_begin = 0;
    pl->tma.pitch = s_in_o;
    pl->tma.s_out_i = s_out_i;
  }
  return true;
}

}  // namespace
// Most vectors per tile of the chunk-tiled permute (lego_tune): 3072 = 48 KiB lets three or four
// CTAs share an SM, so that some load while others store.
std::atomic<int> g_chunk_tile_vecs{3072};
// DMA permute (lego_tune): most bytes per tile, 0 = never use it; CTAs per SM.
std::atomic<int> g_dma_tile_bytes{16384};
std::atomic<int> g_dma_ctas_per_sm{2};
std::atomic<int> g_dma_long_runs{1};  // 1: also pairs whose common run is a whole line or more (large problems)
namespace {

// Chunk-tiled plan (see ChunkParams); false when the pair of layouts has no common run of
// whole 16-byte vectors, or nothing continues it on one of the sides.
bool plan_chunk(const std::vector<PairDigit>& merged, int64_t size, int eb, const void* in, const void* out,
                Plan* pl) {
  if (eb > 16 || !aligned(in, 16) || !aligned(out, 16) || size >= ((int64_t)1 << 40)) return false;
  const int64_t ev = 16 / eb;  // elements per vector
  int c = -1;
  for (size_t j = 0; j < merged.size(); ++j)
    if (merged[j].sa == 1 && merged[j].sb == 1) c = (int)j;
  if (c < 0 || (merged[c].radix * eb) % 16) return false;
  const int64_t rv = merged[c].radix * eb / 16;
  if (rv < 1 || rv >= 8) return false;  // runs of a whole 128-byte line: the plain vector copy is already coalesced
  struct D { int64_t radix, sa, sb; bool in_tile; };
  std::vector<D> ds;
  for (size_t j = 0; j < merged.size(); ++j) {
    if ((int)j == c || merged[j].radix == 1) continue;
    if (merged[j].sa % ev || merged[j].sb % ev) return false;
    ds.push_back({merged[j].radix, merged[j].sa / ev, merged[j].sb / ev, false});
  }
  // the digits continuing the run on either side, up to two per side and about a KiB per piece
  // (the two sides take turns, so that a digit both could use goes to the side that is shorter)
  std::vector<int> chain_in, chain_out;
  int64_t len_i = rv, len_o = rv;
  bool open_i = true, open_o = true;
  while (open_i || open_o) {
    const bool turn_in = open_i && (!open_o || len_i <= len_o);
    std::vector<int>& ch = turn_in ? chain_in : chain_out;
    int64_t& len = turn_in ? len_i : len_o;
    bool& open = turn_in ? open_i : open_o;
    int f = -1;
    if (ch.size() < 2 && len * 16 < 1024)
      for (size_t j = 0; j < ds.size(); ++j)
        if (!ds[j].in_tile && (turn_in ? ds[j].sa : ds[j].sb) == len) f = (int)j;
    if (f < 0) { open = false; continue; }
    ds[f].in_tile = true;
    ch.push_back(f);
    len *= ds[f].radix;
  }
  if (chain_in.empty() || chain_out.empty()) return false;
  // fit the tile into shared memory: cut the slowest digit of the longer side
  auto tile_vecs = [&]() {
    int64_t v = rv;
    for (const D& d : ds)
      if (d.in_tile) v *= d.radix;
    return v;
  };
  // (Smaller tiles for small inputs, to fill the last wave, were slower: an eighth of the 384^3
  // bricks in 768-vector tiles 23.0 us against 19.8 us in 3072-vector tiles.)
  const int64_t max_vecs = g_chunk_tile_vecs.load();
  for (int guard = 0; tile_vecs() > max_vecs && guard < 16; ++guard) {
    int64_t len_in = rv, len_out = rv;
    for (int j : chain_in) len_in *= ds[j].radix;
    for (int j : chain_out) len_out *= ds[j].radix;
    std::vector<int>& ch = len_in >= len_out ? chain_in : chain_out;
    D& d = ds[ch.back()];
    const int64_t over = (tile_vecs() + max_vecs - 1) / max_vecs;
    int64_t part = 0;
    for (int64_t p = d.radix / over; p >= 2; --p)
      if (d.radix % p == 0) { part = p; break; }
    if (part < 2) {
      if (ch.size() == 1) return false;
      d.in_tile = false;
      ch.pop_back();
      continue;
    }
    ds.push_back({d.radix / part, d.sa * part, d.sb * part, false});  // the rest of the digit stays outside
    ds[ch.back()].radix = part;
  }
  if (tile_vecs() > max_vecs) return false;
  int64_t span_in = rv, span_out = rv;  // vectors from a tile's first to its last, on either side
  for (const D& d : ds)
    if (d.in_tile) {
      span_in += (d.radix - 1) * d.sa;
      span_out += (d.radix - 1) * d.sb;
    }
  if (span_in >= ((int64_t)1 << 31) || span_out >= ((int64_t)1 << 31)) return false;

  ChunkParams& cp = pl->chunk;
  std::memset(&cp, 0, sizeof(cp));
  std::vector<int> inner;
  for (size_t j = 0; j < ds.size(); ++j)
    if (ds[j].in_tile) inner.push_back((int)j);
  if ((int)inner.size() > kChunkMaxInner) return false;
  std::vector<int> by_in = inner, by_out = inner;
  std::sort(by_in.begin(), by_in.end(), [&](int a, int b) { return ds[a].sa < ds[b].sa; });
  std::sort(by_out.begin(), by_out.end(), [&](int a, int b) { return ds[a].sb < ds[b].sb; });
  std::vector<int64_t> w_smem(ds.size(), 0), w_out(ds.size(), 0);
  int64_t acc = 1;
  for (int j : by_in) { w_smem[j] = acc; acc *= ds[j].radix; }
  cp.tile_runs = (int32_t)acc;
  acc = 1;
  for (int j : by_out) { w_out[j] = acc; acc *= ds[j].radix; }
  auto fill = [&](ChunkDigit* dst, const std::vector<int>& order) {
    for (size_t k = 0; k < order.size(); ++k) {
      const D& d = ds[order[k]];
      dst[k].radix = (uint32_t)d.radix;
      dst[k].w_smem = (uint32_t)w_smem[order[k]];
      dst[k].w_out = (uint32_t)w_out[order[k]];
      dst[k].fd = make_fastdiv((uint64_t)d.radix);
      dst[k].s_in = (uint32_t)d.sa;
      dst[k].s_out = (uint32_t)d.sb;
    }
  };
  fill(cp.by_in, by_in);
  fill(cp.by_out, by_out);
  cp.n_inner = (int32_t)inner.size();
  cp.rv = (int32_t)rv;
  // The XOR on the low three position bits must be one value per aligned group of eight
  // vectors in shared memory: the input-chain digits (which vary inside such a group) must
  // not reach the low bits of rv * output-order index, and the input pieces must be whole groups.
  int64_t piece_in = rv;
  bool swz = (rv == 1 || rv == 2 || rv == 4 || rv == 8);
  for (int j : chain_in) {
    piece_in *= ds[j].radix;
    if ((w_out[j] * rv) % 8) swz = false;
  }
  if (piece_in % 8) swz = false;
  cp.swizzle = swz ? 1 : 0;

  // outer digits: everything not in the tile
  const int32_t wide = size > ((int64_t)1 << 31) ? 1 : 0;
  cp.p1.n_src = 1;
  cp.p2.n_dst = 2;
  cp.p1.wide = cp.p2.wide = wide;
  int64_t before = 1;
  int n_outer = 0;
  std::vector<int> outer;
  for (size_t j = 0; j < ds.size(); ++j)
    if (!ds[j].in_tile) outer.push_back((int)j);
  if ((int)outer.size() > LEGO_MAX_RANK || 2 * (int)outer.size() > LEGO_MAX_TERMS) return false;
  // neighbouring tile ids walk the digit that is contiguous on the output side first
  std::sort(outer.begin(), outer.end(), [&](int a, int b) { return ds[a].sb < ds[b].sb; });
  for (int j : outer) {
    const bool last = (j == outer.back());
    set_term(&cp.p1.t[cp.p1.n_terms++], 0, n_outer, before, last ? 0 : ds[j].radix, 1);
    set_term(&cp.p2.t[cp.p2.n_terms++], n_outer, 0, 1, 0, ds[j].sa);
    set_term(&cp.p2.t[cp.p2.n_terms++], n_outer, 1, 1, 0, ds[j].sb);
    before *= ds[j].radix;
    ++n_outer;
  }
  cp.p1.n_dst = cp.p2.n_src = n_outer;
  cp.n_tiles = before;
  if (cp.n_tiles >= ((int64_t)1 << 31)) return false;
  pl->kind = KIND_CHUNK;
  pl->vec_bytes = 16;
  pl->tile_in = piece_in * ev;
  int64_t piece_out = rv;
  for (int j : chain_out) piece_out *= ds[j].radix;
  pl->tile_out = piece_out * ev;
  return true;
}

// DMA plan (see DmaParams); false when the pair has no common run of whole 16-byte vectors,
// when nothing continues it on one of the sides, or when one of the sides needs a tensor map
// of more than five dimensions.
bool plan_dma(const std::vector<PairDigit>& merged, int64_t size, int eb, const void* in, const void* out,
              Plan* pl) {
  const int64_t max_tile = g_dma_tile_bytes.load();
  if (max_tile <= 0 || eb > 16 || !aligned(in, 16) || !aligned(out, 16) || size >= ((int64_t)1 << 40)) return false;
  const int64_t unit = eb == 16 ? 2 : 1;  // 16-byte elements are written as two 8-byte ones
  const int64_t ebx = eb == 16 ? 8 : eb;
  struct D { int64_t radix, sa, sb, box; bool in_tile; };
  std::vector<D> ds;
  int c = -1;
  for (const PairDigit& d : merged) {
    if (d.radix == 1) continue;
    if (d.sa == 1 && d.sb == 1) {
      c = (int)ds.size();
      ds.push_back({d.radix * unit, 1, 1, d.radix * unit, true});
    } else {
      ds.push_back({d.radix, d.sa * unit, d.sb * unit, 1, false});
    }
  }
  if (c < 0) return false;
  const int64_t run = ds[c].radix;  // elements of ebx bytes
  if ((run * ebx) % 16) return false;
  // Runs of a whole line or more: the output-order vector copy is coalesced already (5.0 - 5.4 TB/s),
  // the copy engine does a little better (5.9) on problems large enough to fill it; a dimension of a
  // box holds at most 256 elements, so a longer run is cut into a low part (the box rows) and a high
  // part that continues it on both sides.
  const bool long_run = run * ebx >= 128;
  if (long_run) {
    if (!g_dma_long_runs.load() || size * eb < ((int64_t)4 << 20)) return false;
    int64_t lo = 0;
    for (int64_t p = run < 256 ? run : 256; p >= 1; --p)
      if (run % p == 0 && (p * ebx) % 16 == 0) { lo = p; break; }
    if (lo * ebx < 128) return false;
    if (lo < run) {
      ds[c].radix = ds[c].box = lo;
      ds.push_back({run / lo, lo, lo, 1, false});
    }
  }
  const int64_t run_lo = ds[c].radix;
  const int64_t budget = max_tile / ebx;  // elements per tile
  std::vector<int> order{c};              // the tile's digits, fastest in shared memory first
  int64_t tile = run_lo, len_i = run_lo, len_o = run_lo, piece_i = run_lo, piece_o = run_lo;
  // Take the next digit of a side's contiguous chain into the tile, whole or the largest part
  // (a divisor of its radix) that keeps the piece within max_len and the tile within budget.
  // (keep_out_head: leave the digit that continues the run on the output side to that side.)
  auto extend = [&](bool in_side, int64_t max_len, bool keep_out_head) {
    int64_t& len = in_side ? len_i : len_o;
    for (size_t j = 0; j < ds.size(); ++j) {
      if (ds[j].in_tile || (in_side ? ds[j].sa : ds[j].sb) != len) continue;
      if (keep_out_head && ds[j].sb == len_o) return false;
      int64_t e = 0;
      for (int64_t p = ds[j].radix; p >= 2; --p)
        if (ds[j].radix % p == 0 && len * p <= max_len && tile * p <= budget) { e = p; break; }
      if (e < 2) return false;
      ds[j].box = e;
      ds[j].in_tile = true;
      order.push_back((int)j);
      tile *= e;
      (in_side ? piece_i : piece_o) *= e;
      len = e == ds[j].radix ? len * e : -1;  // a digit taken in part ends the chain
      return true;
    }
    return false;
  };
  // Rows of up to 256 bytes for the loads first (the copy engine fetches a box row by row),
  // then whatever continues the run on the output side, then longer load rows if room is left.
  const int64_t row = 256 / ebx;
  int n_in = 0, n_out = 0;
  while (len_i > 0 && len_i < row && extend(true, row, true)) ++n_in;
  while (len_o > 0 && tile < budget && extend(false, budget, false)) ++n_out;
  if (len_i < 0) {
    // the input chain ended with part of a digit: a larger part of it, if room is left
    const int j = [&] { int last = -1; for (int k : order) if (ds[k].box != ds[k].radix) { last = k; break; } return last; }();
    if (j >= 0 && ds[j].sa * ds[j].box == piece_i) {
      for (int64_t p = ds[j].radix; p > ds[j].box; --p)
        if (ds[j].radix % p == 0 && piece_i / ds[j].box * p <= 256 && tile / ds[j].box * p <= budget) {
          tile = tile / ds[j].box * p;
          piece_i = piece_i / ds[j].box * p;
          ds[j].box = p;
          if (p == ds[j].radix) len_i = piece_i;
          break;
        }
    }
  }
  while (len_i > 0 && tile < budget && extend(true, 256, false)) ++n_in;
  if (long_run ? n_in + n_out == 0 : (n_in == 0 || n_out == 0)) return false;
  if (tile * ebx < 2048) return false;  // too little per copy to keep the engine busy

  // One side's tensor map: consecutive tile digits whose strides continue one another share a
  // dimension (the box is their product, at most 256 elements); digits outside the tile join a
  // dimension they continue, or get one of their own with box 1.
  struct Place { int dim; int64_t mul; };
  auto build_side = [&](bool in_side, DmaMapSpec* spec, std::vector<Place>* place) {
    struct Dim { int64_t stride, size, box; bool open; };
    std::vector<Dim> dims;
    place->assign(ds.size(), Place{-1, 0});
    auto stride_of = [&](int j) { return in_side ? ds[j].sa : ds[j].sb; };
    for (int j : order) {
      const int64_t st = stride_of(j);
      if (!dims.empty() && dims.back().open && st == dims.back().stride * dims.back().size &&
          dims.back().box * ds[j].box <= 256) {
        Dim& d = dims.back();
        (*place)[j] = Place{(int)dims.size() - 1, d.size * ds[j].box};
        d.box *= ds[j].box;
        d.size *= ds[j].radix;
        d.open = ds[j].box == ds[j].radix;
      } else {
        dims.push_back({st, ds[j].radix, ds[j].box, ds[j].box == ds[j].radix});
        (*place)[j] = Place{(int)dims.size() - 1, ds[j].box};
      }
    }
    std::vector<int> rest;
    for (size_t j = 0; j < ds.size(); ++j)
      if (!ds[j].in_tile) rest.push_back((int)j);
    std::sort(rest.begin(), rest.end(), [&](int a, int b) { return stride_of(a) < stride_of(b); });
    for (int j : rest) {
      const int64_t st = stride_of(j);
      bool joined = false;
      for (size_t k = 0; k < dims.size() && !joined; ++k)
        if (st == dims[k].stride * dims[k].size) {
          (*place)[j] = Place{(int)k, dims[k].size};
          dims[k].size *= ds[j].radix;
          dims[k].open = false;
          joined = true;
        }
      if (!joined) {
        dims.push_back({st, ds[j].radix, 1, false});
        (*place)[j] = Place{(int)dims.size() - 1, 1};
      }
    }
    if (dims.size() < 2 || dims.size() > 5 || dims[0].stride != 1) return false;
    spec->rank = (int)dims.size();
    for (size_t k = 0; k < dims.size(); ++k) {
      if (dims[k].size >= ((int64_t)1 << 31) || dims[k].box > 256) return false;
      if (k > 0 && ((dims[k].stride * ebx) % 16 || dims[k].stride * ebx >= ((int64_t)1 << 40))) return false;
      spec->size[k] = (uint64_t)dims[k].size;
      spec->stride[k] = (uint64_t)dims[k].stride;
      spec->box[k] = (uint32_t)dims[k].box;
    }
    return true;
  };
  std::vector<Place> pl_in, pl_out;
  if (!build_side(true, &pl->dma_ld, &pl_in) || !build_side(false, &pl->dma_st, &pl_out)) return false;

  DmaParams& dp = pl->dma;
  std::memset(&dp, 0, sizeof(dp));
  // the digits of the tile id: what is left of every digit outside the box; neighbouring ids
  // walk the digit that is contiguous on the output side first
  std::vector<int> outer;
  for (size_t j = 0; j < ds.size(); ++j)
    if (ds[j].radix / ds[j].box > 1) outer.push_back((int)j);
  if ((int)outer.size() > kDmaMaxOuter) return false;
  std::sort(outer.begin(), outer.end(), [&](int a, int b) { return ds[a].sb < ds[b].sb; });
  int64_t n_tiles = 1;
  for (int j : outer) {
    DmaOuter& o = dp.o[dp.n_outer++];
    const int64_t r = ds[j].radix / ds[j].box;
    o.fd = make_fastdiv((uint64_t)r);
    o.radix = (uint32_t)r;
    if (pl_in[j].mul * r >= ((int64_t)1 << 31) || pl_out[j].mul * r >= ((int64_t)1 << 31)) return false;
    o.ld_dim = pl_in[j].dim;
    o.ld_mul = (int32_t)pl_in[j].mul;
    o.st_dim = pl_out[j].dim;
    o.st_mul = (int32_t)pl_out[j].mul;
    n_tiles *= r;
    if (n_tiles >= ((int64_t)1 << 31)) return false;
  }
  dp.n_tiles = n_tiles;
  dp.ld_rank = pl->dma_ld.rank;
  dp.st_rank = pl->dma_st.rank;
  dp.tile_bytes = (uint32_t)(tile * ebx);
  dp.slot_bytes = (dp.tile_bytes + 127u) & ~127u;
  pl->dma_elem_bytes = (int)ebx;
  pl->kind = KIND_DMA;
  pl->vec_bytes = 16;
  pl->tile_in = piece_i / unit;   // contiguous elements per piece read / written
  pl->tile_out = piece_o / unit;
  return true;
}

int32_t make_plan(int eb, const lego_layout_t* src, const lego_layout_t* dst,
                  const lego_layout_t* order, const void* in, const void* out, Plan* pl, bool allow_dma = true,
                  int64_t slab_count = -1, int64_t* n_slabs = nullptr, int64_t* slab_elems = nullptr) {
  if (!src || !dst) return LEGO_ERR_NULL;
  if (eb != 1 && eb != 2 && eb != 4 && eb != 8 && eb != 16) return LEGO_ERR_SIZE;
  int64_t size = 0, osize = 0;
  int32_t st = check_layout(src, &size);
  if (st != LEGO_OK) return st;
  st = check_layout(dst, nullptr);
  if (st != LEGO_OK) return st;
  st = same_domain(src, dst);
  if (st != LEGO_OK) return st;
  if (order) {
    st = check_layout(order, &osize);
    if (st != LEGO_OK) return st;
    if (order->rank > src->rank) return LEGO_ERR_DOMAIN;
    for (int k = 0; k < order->rank; ++k)
      if (order->dims[k] != src->dims[k]) return LEGO_ERR_DOMAIN;
  }
  pl->elem_bytes = eb;
  pl->size = size;
  pl->tile_in = pl->tile_out = 1;
  pl->by_order = false;

  std::vector<Digit> ds, dd, dor;
  const int32_t fs = fold_layout(src, &ds);
  const int32_t fd = fold_layout(dst, &dd);
  std::vector<PairDigit> pairs;
  if (fs != LEGO_OK || fd != LEGO_OK || !refine_pair(ds, dd, &pairs)) {
    if ((fs != LEGO_OK && fs != LEGO_ERR_UNSUPPORTED)) return fs;
    if ((fd != LEGO_OK && fd != LEGO_ERR_UNSUPPORTED)) return fd;
    if (slab_count >= 0 || n_slabs) return LEGO_ERR_UNSUPPORTED;  // slabs are read off the folded digits
    pl->kind = KIND_STAGED;
    pl->vec_bytes = eb;
    st = build_staged(src, &pl->staged_src);
    if (st != LEGO_OK) return st;
    return build_staged(dst, &pl->staged_dst);
  }
  const int32_t wide = size > ((int64_t)1 << 31) ? 1 : 0;

  // (i) tiles named by tile_order: a tile is every index sharing the leading coordinates.
  if (order && slab_count < 0 && !n_slabs && fold_layout(order, &dor) == LEGO_OK) {
    int64_t tile_elems = 1;
    for (int k = order->rank; k < src->rank; ++k) tile_elems *= src->dims[k];
    std::vector<PairDigit> inner;
    for (const PairDigit& d : pairs)
      if (d.pos < tile_elems) inner.push_back(d);
    merge_pairs(&inner);
    if (inner.size() == 2 && inner[0].sa == 1 && inner[1].sb == 1) {
      TiledParams& tp = pl->tiled;
      std::memset(&tp, 0, sizeof(tp));
      program_inv(dor, order->rank, osize, &tp.p1);
      tp.p2.n_src = order->rank;
      tp.p2.n_dst = 2;
      tp.p2.wide = wide;
      tp.p1.wide = wide;
      for (const Digit& d : ds)
        if (d.src < order->rank) set_term(&tp.p2.t[tp.p2.n_terms++], d.src, 0, d.div, d.mod, d.stride);
      for (const Digit& d : dd)
        if (d.src < order->rank) set_term(&tp.p2.t[tp.p2.n_terms++], d.src, 1, d.div, d.mod, d.stride);
      tp.n_tiles = osize;
      if (finish_tiled(inner[0].radix, inner[1].radix, inner[0].sb, inner[1].sa, eb, in, out, pl)) {
        pl->by_order = true;
        return LEGO_OK;
      }
    }
  }

  // (ii) tiles chosen here from the merged digit permutation.
  std::vector<PairDigit> merged = pairs;
  merge_pairs(&merged);
  if (slab_count >= 0 || n_slabs) {
    // The digit that is slowest in BOTH buffers cuts the re-layout into independent slabs, each
    // contiguous on either side; `slab_count` of them are the same permutation with that digit's
    // radix reduced (the buffers then hold those slabs only).
    int top = -1;
    for (size_t j = 0; j < merged.size(); ++j)
      if (merged[j].radix > 1 && merged[j].sa * merged[j].radix == size && merged[j].sb * merged[j].radix == size)
        top = (int)j;
    if (top < 0) return LEGO_ERR_UNSUPPORTED;
    if (n_slabs) *n_slabs = merged[top].radix;
    if (slab_elems) *slab_elems = size / merged[top].radix;
    if (slab_count >= 0) {
      if (slab_count > merged[top].radix) return LEGO_ERR_SIZE;
      size = size / merged[top].radix * slab_count;
      merged[top].radix = slab_count;
      pl->size = size;
      if (slab_count == 0) return LEGO_OK;
    }
  }
  int ii = -1, oo = -1;
  for (size_t j = 0; j < merged.size(); ++j) {
    if (merged[j].sa == 1) ii = (int)j;
    if (merged[j].sb == 1) oo = (int)j;
  }
  if (ii >= 0 && oo >= 0 && ii != oo && eb <= 16) {
    const int ve = 16 / eb;
    int64_t t = ve;
    while ((t * 2) * (t * 2) / ve <= kCtaVectors) t *= 2;
    int64_t ti = t, to = t;
    const int64_t tma_ti = 128 / eb, tma_to = 8 * ve;
    if ((eb == 2 || eb == 4 || eb == 8) && merged[ii].radix % tma_ti == 0 && merged[oo].radix % tma_to == 0) {
      ti = tma_ti;  // the shape the TMA-fed kernel moves
      to = tma_to;
    } else {
      while (ti > 1 && merged[ii].radix % ti) ti >>= 1;
      while (to > 1 && merged[oo].radix % to) to >>= 1;
      // grow the narrower side while the tile still fits
      while (ti * 2 * to / ve <= kCtaVectors && merged[ii].radix % (ti * 2) == 0 && ti < 4 * t) ti *= 2;
      while (ti * to * 2 / ve <= kCtaVectors && merged[oo].radix % (to * 2) == 0 && to < 4 * t) to *= 2;
    }
    // outer digits, input-contiguous tile column fastest
    struct Outer { int64_t radix, sa, sb; };
    std::vector<Outer> outer;
    if (merged[ii].radix / ti > 1) outer.push_back({merged[ii].radix / ti, ti, merged[ii].sb * ti});
    if (merged[oo].radix / to > 1) outer.push_back({merged[oo].radix / to, merged[oo].sa * to, to});
    for (size_t j = 0; j < merged.size(); ++j)
      if ((int)j != ii && (int)j != oo && merged[j].radix > 1)
        outer.push_back({merged[j].radix, merged[j].sa, merged[j].sb});
    if ((int)outer.size() <= LEGO_MAX_RANK && 2 * (int)outer.size() <= LEGO_MAX_TERMS) {
      TiledParams& tp = pl->tiled;
      std::memset(&tp, 0, sizeof(tp));
      tp.p1.n_src = 1;
      tp.p1.n_dst = (int32_t)outer.size();
      tp.p2.n_src = (int32_t)outer.size();
      tp.p2.n_dst = 2;
      tp.p1.wide = tp.p2.wide = wide;
      int64_t before = 1;
      for (size_t c = 0; c < outer.size(); ++c) {
        const bool last = (c + 1 == outer.size());
        set_term(&tp.p1.t[tp.p1.n_terms++], 0, (int)c, before, last ? 0 : outer[c].radix, 1);
        set_term(&tp.p2.t[tp.p2.n_terms++], (int)c, 0, 1, 0, outer[c].sa);
        set_term(&tp.p2.t[tp.p2.n_terms++], (int)c, 1, 1, 0, outer[c].sb);
        before *= outer[c].radix;
      }
      tp.n_tiles = before;
      if (finish_tiled(ti, to, merged[ii].sb, merged[oo].sa, eb, in, out, pl)) return LEGO_OK;
    }
  }
  if (allow_dma && plan_dma(merged, size, eb, in, out, pl)) return LEGO_OK;
  if (plan_chunk(merged, size, eb, in, out, pl)) return LEGO_OK;
  plan_gather(merged, size, eb, in, out, pl);
  return LEGO_OK;
}

template <int EB>
int32_t launch(const Plan& pl, const void* in, void* out, DeviceCtx* ctx, cudaStream_t s) {
  const uint8_t* pin = (const uint8_t*)in;
  uint8_t* pout = (uint8_t*)out;
  if (pl.kind == KIND_TILED) {
    const TiledParams& tp = pl.tiled;
    const int64_t ctas = (tp.n_tiles + tp.tiles_per_cta - 1) / tp.tiles_per_cta;
    if (ctas > 0x7fffffff) return LEGO_ERR_SIZE;
    if (tp.p1.wide)
      tiled_transpose_kernel<EB, true><<<(unsigned)ctas, kThreads, 0, s>>>(tp, pin, pout);
    else
      tiled_transpose_kernel<EB, false><<<(unsigned)ctas, kThreads, 0, s>>>(tp, pin, pout);
  } else if (pl.kind == KIND_STAGED) {
    int64_t blocks = (pl.size + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)ctx->sm_count * 16;
    if (blocks > cap) blocks = cap;
    staged_permute_kernel<EB><<<(unsigned)blocks, kThreads, 0, s>>>(pl.staged_src, pl.staged_dst, pin, pout,
                                                                   pl.size);
  }
  return cuda_status(cudaGetLastError());
}

template <int EB>
int32_t launch_tma(const Plan& pl, const void* in, void* out, DeviceCtx* ctx, cudaStream_t s) {
  constexpr int TILE_BYTES = 8 * (16 / EB) * 128;
  int32_t err = LEGO_OK;
  EncodeFn enc = encode_fn(&err);
  if (!enc) return err;
  TmaParams tp = pl.tma;
  if (tp.n_tiles >= ((int64_t)1 << 31)) return LEGO_ERR_SIZE;
  // Measured on B200 (fp32 4096^2, back-to-back launches): two CTAs per SM with eight ring
  // slots each (5.74 TB/s); 1 x 16 or 1 x 32 slots 5.45, 3 x 4 slots 5.40, 3 x 8 slots 5.2,
  // 2 x 4 slots 4.8, 2 x 16 slots 5.0; 4, 8 or 16 consumer warps make no difference.  About 64 KiB
  // of tiles in flight per SM is enough, and leaving half of the SM's shared memory and
  // thread slots free lets the next grid of the stream become resident and plan its first
  // tiles while this one drains (programmatic dependent launch).  The tile order (row-,
  // column-major, 2 x 2 .. 16 x 16 blocks) moves the result by less than 3 %.  A slot must
  // always be drained by the same consumer pair (a waiter two uses ahead of an mbarrier
  // cannot tell its phase from the one two back), so the slot count is a multiple of the
  // number of pairs.
  const int ctas_per_sm = 2;
  const int stages = 8;
  static_assert(kTmaStages % (kTmaConsumerWarps / 2) == 0, "slots per consumer pair");
  tp.stages = stages;
  const size_t SMEM = (size_t)stages * TILE_BYTES + sizeof(TmaCtl) + 1024;
  CUtensorMap tmap;
  const CUtensorMapDataType dt = EB == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                               : EB == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT64;
  err = make_tmap_group_major(enc, &tmap, dt, in, (uint64_t)tp.pitch, (uint64_t)(pl.size / tp.pitch),
                              (uint64_t)tp.pitch * EB, 16 / EB, 128 / EB, 8);
  tp.one_load = err == LEGO_OK ? 1 : 0;
  if (err != LEGO_OK)
    err = make_tmap_row_groups(enc, &tmap, dt, in, (uint64_t)tp.pitch, (uint64_t)(pl.size / tp.pitch),
                               (uint64_t)tp.pitch * EB, 16 / EB, 128 / EB, 8);
  if (err != LEGO_OK) return err;
  static PerDeviceFlag configured[2];  // one per instantiation (SMEM is a constant of EB)
  const int wide = tp.p1.wide ? 1 : 0;
  if (!configured[wide].test(ctx->device)) {
    if (wide) LEGO_CUDA_TRY(cudaFuncSetAttribute(tma_transpose_kernel<EB, true>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    else LEGO_CUDA_TRY(cudaFuncSetAttribute(tma_transpose_kernel<EB, false>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    configured[wide].set(ctx->device);
  }
  int64_t grid = (int64_t)ctx->sm_count * ctas_per_sm;
  if (grid > tp.n_tiles) grid = tp.n_tiles;
  if (grid < 1) grid = 1;
  cudaError_t e;
  if (wide)
    e = launch_overlapped(tma_transpose_kernel<EB, true>, dim3((unsigned)grid), dim3(kTmaThreads), SMEM, s, tmap, tp,
                          (uint8_t*)out, ctx->status_word);
  else
    e = launch_overlapped(tma_transpose_kernel<EB, false>, dim3((unsigned)grid), dim3(kTmaThreads), SMEM, s, tmap, tp,
                          (uint8_t*)out, ctx->status_word);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return cuda_status(e);
}

int32_t launch_chunk(const Plan& pl, const void* in, void* out, DeviceCtx* ctx, cudaStream_t s) {
  const ChunkParams& cp = pl.chunk;
  const size_t vecs = ((size_t)cp.tile_runs * cp.rv + 7) & ~(size_t)7;
  const size_t smem = vecs * 16;
  static PerDeviceFlag configured[2];
  const int wide = cp.p1.wide ? 1 : 0;
  if (!configured[wide].test(ctx->device)) {
    if (wide) LEGO_CUDA_TRY(cudaFuncSetAttribute(chunk_permute_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 kChunkMaxVecs * 16));
    else LEGO_CUDA_TRY(cudaFuncSetAttribute(chunk_permute_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            kChunkMaxVecs * 16));
    configured[wide].set(ctx->device);
  }
  if (wide)
    chunk_permute_kernel<true><<<(unsigned)cp.n_tiles, kThreads, smem, s>>>(cp, (const uint4*)in, (uint4*)out);
  else
    chunk_permute_kernel<false><<<(unsigned)cp.n_tiles, kThreads, smem, s>>>(cp, (const uint4*)in, (uint4*)out);
  return cuda_status(cudaGetLastError());
}

// The tensor map of one side of a DMA plan.
int32_t encode_dma_map(EncodeFn enc, CUtensorMap* map, const DmaMapSpec& sp, int ebx, const void* base) {
  const CUtensorMapDataType dt = ebx == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                               : ebx == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                               : ebx == 4 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT64;
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5], estr[5];
  for (int k = 0; k < sp.rank; ++k) {
    dims[k] = sp.size[k];
    box[k] = sp.box[k];
    estr[k] = 1;
    if (k > 0) strides[k - 1] = sp.stride[k] * (uint64_t)ebx;
  }
  const CUresult r = enc(map, dt, (cuuint32_t)sp.rank, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? LEGO_OK : LEGO_ERR_UNSUPPORTED;
}

// LEGO_ERR_UNSUPPORTED (nothing launched) when the driver refuses one of the tensor maps: the
// caller then plans again without this kernel.
int32_t launch_dma(const Plan& pl, const void* in, void* out, DeviceCtx* ctx, cudaStream_t s) {
  int32_t err = LEGO_OK;
  EncodeFn enc = encode_fn(&err);
  if (!enc) return err;
  CUtensorMap ld_map, st_map;
  err = encode_dma_map(enc, &ld_map, pl.dma_ld, pl.dma_elem_bytes, in);
  if (err != LEGO_OK) return err;
  err = encode_dma_map(enc, &st_map, pl.dma_st, pl.dma_elem_bytes, out);
  if (err != LEGO_OK) return err;
  DmaParams dp = pl.dma;
  // Shared memory of an SM split among the CTAs that share it; every CTA keeps
  // kDmaStoresInFlight slots for stores that are reading and the rest for loads in flight.
  int ctas_per_sm = g_dma_ctas_per_sm.load();
  const int64_t usable = (int64_t)ctx->smem_optin - 2048;
  int64_t stages = 0;
  for (; ctas_per_sm >= 1; --ctas_per_sm) {
    stages = (usable / ctas_per_sm - (int64_t)sizeof(DmaCtl) - 1152) / dp.slot_bytes;
    if (stages >= kDmaStoresInFlight + 2) break;
  }
  if (ctas_per_sm < 1) return LEGO_ERR_UNSUPPORTED;
  if (stages > kDmaMaxStages) stages = kDmaMaxStages;
  dp.stages = (int32_t)stages;
  const size_t smem = (size_t)stages * dp.slot_bytes + sizeof(DmaCtl) + 128;
  static PerDeviceFlag configured;
  if (!configured.test(ctx->device)) {
    LEGO_CUDA_TRY(cudaFuncSetAttribute(dma_permute_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       ctx->smem_optin));
    configured.set(ctx->device);
  }
  int64_t grid = (int64_t)ctx->sm_count * ctas_per_sm;
  if (grid > dp.n_tiles) grid = dp.n_tiles;
  const cudaError_t e = launch_overlapped(dma_permute_kernel, dim3((unsigned)grid), dim3(kDmaThreads), smem, s, ld_map,
                                          st_map, dp, ctx->status_word);
  if (e != cudaSuccess) (void)cudaGetLastError();
  return cuda_status(e);
}

template <int VB>
int32_t launch_gather(const Plan& pl, const void* in, void* out, DeviceCtx* ctx, cudaStream_t s) {
  const GatherParams& gp = pl.gather;
  int64_t blocks = (gp.n_vec + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)ctx->sm_count * 32;
  if (blocks > cap) blocks = cap;
  if (gp.g.wide)
    gather_kernel<VB, true><<<(unsigned)blocks, kThreads, 0, s>>>(gp, (const uint8_t*)in, (uint8_t*)out);
  else
    gather_kernel<VB, false><<<(unsigned)blocks, kThreads, 0, s>>>(gp, (const uint8_t*)in, (uint8_t*)out);
  return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace lego

using namespace lego;

extern "C" {

int32_t lego_permute_plan(int32_t elem_bytes, const lego_layout_t* src, const lego_layout_t* dst,
                          const lego_layout_t* tile_order, int32_t* kernel_kind, int64_t* tile_in,
                          int64_t* tile_out) {
  Plan* pl = new Plan();
  // Planning for inspection assumes 16-byte aligned buffers, as torch allocations are.
  const int32_t st = make_plan(elem_bytes, src, dst, tile_order, nullptr, nullptr, pl);
  if (st == LEGO_OK) {
    if (kernel_kind) *kernel_kind = pl->kind;
    if (tile_in) *tile_in = pl->tile_in;
    if (tile_out) *tile_out = pl->tile_out;
  }
  delete pl;
  return st;
}

int32_t lego_permute_dma_plan(int32_t elem_bytes, const lego_layout_t* src, const lego_layout_t* dst,
                              int64_t slab_count, lego_dma_plan_t* plan) {
  if (!plan) return LEGO_ERR_NULL;
  Plan* pl = new Plan();
  int32_t st = make_plan(elem_bytes, src, dst, nullptr, nullptr, nullptr, pl, true, slab_count < 0 ? -1 : slab_count);
  if (st == LEGO_OK && pl->kind != KIND_DMA) st = LEGO_ERR_UNSUPPORTED;
  if (st == LEGO_OK) {
    std::memset(plan, 0, sizeof(*plan));
    plan->elem_bytes = pl->dma_elem_bytes;
    plan->n_outer = pl->dma.n_outer;
    plan->n_tiles = pl->dma.n_tiles;
    plan->tile_bytes = pl->dma.tile_bytes;
    const DmaMapSpec* specs[2] = {&pl->dma_ld, &pl->dma_st};
    lego_dma_side_t* sides[2] = {&plan->load, &plan->store};
    for (int k = 0; k < 2; ++k) {
      sides[k]->rank = specs[k]->rank;
      for (int d = 0; d < specs[k]->rank; ++d) {
        sides[k]->size[d] = (int64_t)specs[k]->size[d];
        sides[k]->stride[d] = d == 0 ? 1 : (int64_t)specs[k]->stride[d];
        sides[k]->box[d] = specs[k]->box[d];
      }
    }
    for (int j = 0; j < pl->dma.n_outer; ++j) {
      const DmaOuter& o = pl->dma.o[j];
      plan->outer[j].radix = o.radix;
      plan->outer[j].ld_dim = o.ld_dim;
      plan->outer[j].ld_mul = o.ld_mul;
      plan->outer[j].st_dim = o.st_dim;
      plan->outer[j].st_mul = o.st_mul;
    }
  }
  delete pl;
  return st;
}

// tile_count < 0: every tile.  Otherwise only the tiles tile_begin .. tile_begin +
// tile_count - 1 of tile_order are moved, which needs a plan whose tiles are tile_order's.
static int32_t run_permute(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                           const lego_layout_t* dst, const lego_layout_t* tile_order, int64_t tile_begin,
                           int64_t tile_count, void* stream, int64_t slab_count = -1) {
  if (!in || !out) return LEGO_ERR_NULL;
  if (in == out) return LEGO_ERR_UNSUPPORTED;  // in-place reorganisation is not defined
  if (!aligned(in, elem_bytes > 0 ? elem_bytes : 1) || !aligned(out, elem_bytes > 0 ? elem_bytes : 1))
    return LEGO_ERR_ALIGN;
  Plan* pl = new Plan();
  int32_t st = make_plan(elem_bytes, src, dst, tile_order, in, out, pl, true, slab_count);
  if (st == LEGO_OK && tile_count >= 0) {
    if (!tile_order) st = LEGO_ERR_NULL;
    else if (!pl->by_order) st = LEGO_ERR_UNSUPPORTED;  // this pair of layouts is not moved tile_order-tile by tile
    else if (tile_begin < 0 || tile_begin + tile_count > pl->tiled.n_tiles) st = LEGO_ERR_SIZE;
    else {
      pl->tiled.tile_begin = pl->tma.tile_begin = tile_begin;
      pl->tiled.n_tiles = pl->tma.n_tiles = tile_count;
      if (pl->tiled.tiles_per_cta > tile_count) pl->tiled.tiles_per_cta = (int32_t)(tile_count > 0 ? tile_count : 1);
      if (tile_count == 0) pl->size = 0;
    }
  }
  if (st == LEGO_OK && pl->size > 0) {
    int32_t err = LEGO_OK;
    DeviceCtx* ctx = device_ctx(&err);
    cudaStream_t s = (cudaStream_t)stream;
    if (!ctx) {
      st = err;
    } else if (pl->kind == KIND_GATHER) {
      switch (pl->vec_bytes) {
        case 1: st = launch_gather<1>(*pl, in, out, ctx, s); break;
        case 2: st = launch_gather<2>(*pl, in, out, ctx, s); break;
        case 4: st = launch_gather<4>(*pl, in, out, ctx, s); break;
        case 8: st = launch_gather<8>(*pl, in, out, ctx, s); break;
        default: st = launch_gather<16>(*pl, in, out, ctx, s); break;
      }
    } else if (pl->kind == KIND_DMA) {
      st = launch_dma(*pl, in, out, ctx, s);
      if (st == LEGO_ERR_UNSUPPORTED) {  // a tensor map the driver does not take: the kernels without one
        st = make_plan(elem_bytes, src, dst, tile_order, in, out, pl, false, slab_count);
        if (st == LEGO_OK && pl->kind == KIND_CHUNK) st = launch_chunk(*pl, in, out, ctx, s);
        else if (st == LEGO_OK) st = LEGO_ERR_UNSUPPORTED;
      }
    } else if (pl->kind == KIND_CHUNK) {
      st = launch_chunk(*pl, in, out, ctx, s);
    } else if (pl->kind == KIND_TMA) {
      switch (elem_bytes) {
        case 2: st = launch_tma<2>(*pl, in, out, ctx, s); break;
        case 4: st = launch_tma<4>(*pl, in, out, ctx, s); break;
        default: st = launch_tma<8>(*pl, in, out, ctx, s); break;
      }
    } else {
      switch (elem_bytes) {
        case 1: st = launch<1>(*pl, in, out, ctx, s); break;
        case 2: st = launch<2>(*pl, in, out, ctx, s); break;
        case 4: st = launch<4>(*pl, in, out, ctx, s); break;
        case 8: st = launch<8>(*pl, in, out, ctx, s); break;
        default: st = launch<16>(*pl, in, out, ctx, s); break;
      }
    }
  }
  delete pl;
  return st;
}

int32_t lego_permute(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                     const lego_layout_t* dst, const lego_layout_t* tile_order, void* stream) {
  return run_permute(in, out, elem_bytes, src, dst, tile_order, 0, -1, stream);
}

int32_t lego_permute_slab_info(int32_t elem_bytes, const lego_layout_t* src, const lego_layout_t* dst,
                               int64_t* n_slabs, int64_t* slab_elems) {
  if (!n_slabs || !slab_elems) return LEGO_ERR_NULL;
  Plan* pl = new Plan();
  const int32_t st = make_plan(elem_bytes, src, dst, nullptr, nullptr, nullptr, pl, true, -1, n_slabs, slab_elems);
  delete pl;
  return st;
}

int32_t lego_permute_slabs(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                           const lego_layout_t* dst, int64_t slab_count, void* stream) {
  if (slab_count < 0) return LEGO_ERR_SIZE;
  return run_permute(in, out, elem_bytes, src, dst, nullptr, 0, -1, stream, slab_count);
}

int32_t lego_permute_tiles(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                           const lego_layout_t* dst, const lego_layout_t* tile_order, int64_t tile_begin,
                           int64_t tile_count, void* stream) {
  if (tile_count < 0) return LEGO_ERR_SIZE;
  return run_permute(in, out, elem_bytes, src, dst, tile_order, tile_begin, tile_count, stream);
}

}  // extern "C"
