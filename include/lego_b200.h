/*
 * lego_b200 -- C ABI of the B200 (sm_100a) back end for LEGO layouts.
 *
 * The reference library (tavakkoliamirmohammad/LEGO) has no native interface:
 * a layout is turned into index-expression text and pasted into Triton / MLIR /
 * CUDA templates.  This header is what a binding for that path would call
 * instead.  Every entry point is extern "C", takes plain pointers and sizes,
 * returns an int32 status (0 = OK, < 0 = argument rejected on the host before
 * any launch, > 0 = CUDA runtime error code + LEGO_ERR_CUDA_BASE or a device
 * status), never throws and never aborts.
 *
 * Buffers named "dev" are device pointers owned by the caller.  `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream); all work is
 * enqueued on it and the call returns without synchronising unless said
 * otherwise.  The library keeps one small lazily created workspace per device
 * (tensor maps, a status word), released by lego_shutdown().
 */
#ifndef LEGO_B200_H_
#define LEGO_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LEGO_MAX_RANK    12   /* logical coordinates of a layout / dims of one block   */
#define LEGO_MAX_BLOCKS   4   /* permutation blocks in one OrderBy                      */
#define LEGO_MAX_STAGES   8   /* OrderBy stages in one GroupBy                          */
#define LEGO_MAX_TERMS   32   /* digits of a folded layout                              */
#define LEGO_MAX_GROUPS 256   /* problems in one grouped GEMM call                      */
#define LEGO_MAX_LUT (1 << 24) /* entries of one table-driven (LUT) permutation block   */

/* status codes */
enum {
  LEGO_OK                = 0,
  LEGO_ERR_NULL          = -1,   /* a required pointer is NULL                          */
  LEGO_ERR_RANK          = -2,   /* rank / count outside the limits above or mismatched */
  LEGO_ERR_PERM          = -3,   /* perm[] is not a permutation                         */
  LEGO_ERR_DIM           = -4,   /* a dimension is < 1                                  */
  LEGO_ERR_NOT_BIJECTIVE = -5,   /* a stage's size differs from the logical size        */
  LEGO_ERR_SIZE          = -6,   /* sizes inconsistent with the operation               */
  LEGO_ERR_ALIGN         = -7,   /* pointer or leading dimension not aligned as needed  */
  LEGO_ERR_UNSUPPORTED   = -8,   /* valid request this build has no kernel for          */
  LEGO_ERR_DOMAIN        = -9,   /* layouts of one call disagree on the logical domain  */
  LEGO_ERR_OVERFLOW      = -10,  /* index space does not fit in 63 bits                 */
  LEGO_ERR_CUDA_BASE     = 1000, /* status = LEGO_ERR_CUDA_BASE + cudaError_t           */
  LEGO_ERR_DEVICE_TIMEOUT = 2001 /* a bounded wait inside a kernel ran out              */
};

/* block kinds */
enum {
  LEGO_BLOCK_REGP     = 0,  /* regular permutation: flatten(sigma(idx), sigma(dims))    */
  LEGO_BLOCK_ANTIDIAG = 1,  /* GenP: anti-diagonal enumeration of a square, dims = (n,n)*/
  LEGO_BLOCK_REVERSE  = 2,  /* GenP: (n1-1-i)*n2 + (n2-1-j), dims = (n1,n2)             */
  LEGO_BLOCK_LUT      = 3   /* GenP with arbitrary callables, tabulated over its domain */
};

/* One permutation block: RegP / Row / Col of lego/lego.py:197-240, one of the
 * GenP bodies of lego/lego.py:490-535, or any GenP (lego/lego.py:150-178) given
 * by its tables.  sigma(v)[i] = v[perm[i]].
 * LEGO_BLOCK_LUT: the binding evaluates the block's f_apply once over the whole
 * domain (at most LEGO_MAX_LUT entries) and passes two device tables of
 * prod(dims) int64 each, owned by the caller and alive while the layout is used:
 * lut_apply[row-major id of idx over dims] = f_apply(idx), a permutation of
 * 0 .. prod(dims)-1, and lut_inv its inverse (row-major id of f_inv(flat)).
 * The host services cannot read device memory: the binding vouches that the
 * tables are permutations.  Other kinds leave both pointers NULL.               */
typedef struct lego_block {
  int32_t rank;
  int32_t kind;
  int64_t dims[LEGO_MAX_RANK];
  int32_t perm[LEGO_MAX_RANK];
  const int64_t* lut_apply;
  const int64_t* lut_inv;
} lego_block_t;

/* One OrderBy (lego/lego.py:243-362): blocks concatenated big-endian.          */
typedef struct lego_stage {
  int32_t n_blocks;
  int32_t reserved;
  lego_block_t blocks[LEGO_MAX_BLOCKS];
} lego_stage_t;

/* One GroupBy (lego/lego.py:365-404): logical dims and its `objects`, in the
 * order the reference stores them (apply walks them last to first).            */
typedef struct lego_layout {
  int32_t rank;
  int32_t n_stages;
  int64_t dims[LEGO_MAX_RANK];
  lego_stage_t stages[LEGO_MAX_STAGES];
} lego_layout_t;

/* Folded form: flat = sum_j ((idx[src_j] / div_j) % mod_j) * stride_j, and
 * idx[k] = sum_{j: src_j = k} ((flat / stride_j) % mod_j) * div_j.             */
typedef struct lego_term {
  int32_t src;
  int32_t reserved;
  int64_t div;
  int64_t mod;
  int64_t stride;
} lego_term_t;

typedef struct lego_folded {
  int32_t foldable;   /* 1: terms[] is exact; 0: only the staged form applies   */
  int32_t n_terms;
  int64_t size;       /* product of the logical dims                            */
  lego_term_t terms[LEGO_MAX_TERMS];
} lego_folded_t;

/* ---- host-side layout services (no GPU needed) ---------------------------- */

/* Validate ranks, permutations, dimensions and that every stage covers exactly
 * the logical index space (the condition under which GroupBy.apply of
 * lego/lego.py:388-404 is a bijection).                                        */
int32_t lego_layout_check(const lego_layout_t* layout);

/* Constant-fold a layout into digit strides.  Replaces the reference's
 * simplify_ops fix-point (lego/z3_simplifier.py:367-386) for concrete dims.    */
int32_t lego_layout_fold(const lego_layout_t* layout, lego_folded_t* out);

/* Plan of a permute call, for inspection: which kernel lego_permute would pick
 * (0 staged interpreter, 1 output-order gather, 2 shared-memory tiled transpose,
 * 3 TMA-fed tiled transpose, 4 chunk-tiled permute for layouts that share a
 * contiguous run, e.g. a volume into bricks, 5 the same pairs (and large problems
 * with longer common runs) moved by the copy engine alone: one tiled TMA load and one tiled TMA store per box of digits; if
 * the driver refuses a tensor map at call time, kernel 4 runs instead) and the
 * contiguous extents it reads and writes, in elements.                         */
int32_t lego_permute_plan(int32_t elem_bytes, const lego_layout_t* src, const lego_layout_t* dst,
                          const lego_layout_t* tile_order, int32_t* kernel_kind, int64_t* tile_in,
                          int64_t* tile_out);

/* The DMA plan of a pair of layouts (kernel 5 of lego_permute_plan), for inspection and
 * for checking the planner on a host without a GPU: the two tensor maps as the encoder
 * receives them (dimension 0 innermost; strides and sizes in elements of elem_bytes,
 * which is 8 for 16-byte data) and the digits of the tile id with the tensor-map
 * coordinate each one moves on either side.  Tile t = sum_j d_j * prod_{i<j} radix_i is
 * the box at load coordinates  c[outer[j].ld_dim] += d_j * outer[j].ld_mul  and store
 * coordinates  c[outer[j].st_dim] += d_j * outer[j].st_mul;  both boxes hold the same
 * bytes in the same order.  slab_count < 0: the whole re-layout; otherwise the plan of that
 * many slabs (lego_permute_slabs).  LEGO_ERR_UNSUPPORTED when the pair is not moved this way.
 * No counterpart in the reference.                                              */
typedef struct lego_dma_side {
  int32_t rank;
  int32_t reserved;
  int64_t size[5];
  int64_t stride[5];
  int64_t box[5];
} lego_dma_side_t;

typedef struct lego_dma_outer {
  int64_t radix;
  int32_t ld_dim, ld_mul, st_dim, st_mul;
  int32_t reserved;
} lego_dma_outer_t;

typedef struct lego_dma_plan {
  int32_t elem_bytes;
  int32_t n_outer;
  int64_t n_tiles;
  int64_t tile_bytes;
  lego_dma_side_t load, store;
  lego_dma_outer_t outer[8];
} lego_dma_plan_t;

int32_t lego_permute_dma_plan(int32_t elem_bytes, const lego_layout_t* src, const lego_layout_t* dst,
                              int64_t slab_count, lego_dma_plan_t* plan);

/* ---- index-map evaluator -------------------------------------------------- */

/* flat[i] = layout.apply(idx[i*rank .. i*rank+rank-1]); GroupBy.apply,
 * lego/lego.py:388-404.  idx, flat: dev int64.                                 */
int32_t lego_eval_apply(const lego_layout_t* layout, const int64_t* idx, int64_t* flat, int64_t n,
                        void* stream);

/* idx[i*rank ..] = layout.inv(flat[i]); GroupBy.inv, lego/lego.py:406-433.     */
int32_t lego_eval_inv(const lego_layout_t* layout, const int64_t* flat, int64_t* idx, int64_t n,
                      void* stream);

/* flat_out[i] = layout.apply(unflatten(begin + i, dims)) for i in [0, n): the
 * loop the reference generates with generate_loop over prod(layout.dims())
 * (lego/lego_mlir.py:85-108).                                                  */
int32_t lego_eval_range(const lego_layout_t* layout, int64_t begin, int64_t n, int64_t* flat_out,
                        void* stream);

/* ---- layout reorganisation ------------------------------------------------ */

/* out_flat[dst(idx)] = in_flat[src(idx)] for every idx of the common logical
 * domain; elem_bytes in {1,2,4,8,16}.  tile_order (nullable) is a layout whose
 * logical dims equal the leading dims of src/dst: tile_order.inv(cta) names the
 * tile a CTA moves, as the block-id maps of benchmarks/mlir/transpose_smem.py:
 * 52-55 do.  Replaces the generated programs mlir_generated/transpose/
 * transpose_{naive,smem}_N.mlir.                                               */
int32_t lego_permute(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                     const lego_layout_t* dst, const lego_layout_t* tile_order, void* stream);

/* The same for a contiguous range of tiles: only the tiles tile_order.inv(t), t in
 * [tile_begin, tile_begin + tile_count), are moved; the rest of `out` is left as it is.
 * This is how one GPU of several moves its slab of a reorganisation (the block ids of
 * benchmarks/mlir/transpose_smem.py:52-55 restricted to a sub-grid): with a column-major
 * tile order over the source's tile grid a range of ids is a slab of output rows.
 * tile_order is required, and the two layouts must be a pair the library moves tile by
 * tile (lego_permute_plan kinds 2 and 3 with a tile order); otherwise
 * LEGO_ERR_UNSUPPORTED.  A range outside the order's ids is LEGO_ERR_SIZE.        */
int32_t lego_permute_tiles(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                           const lego_layout_t* dst, const lego_layout_t* tile_order,
                           int64_t tile_begin, int64_t tile_count, void* stream);

/* Slabs.  When the slowest-varying digit of the flat index is the same logical digit in
 * both layouts (the outermost brick coordinate of benchmarks/cuda/bricks_f3d.py:10-13, the
 * batch index of a batched transpose), the re-layout falls apart into *n_slabs independent
 * pieces of *slab_elems elements, each contiguous in the input and in the output.
 * lego_permute_slab_info reports them (host only; LEGO_ERR_UNSUPPORTED when the pair does
 * not split).  lego_permute_slabs moves slab_count consecutive slabs: `in` and `out` hold
 * those slabs only (slab_count * slab_elems elements each), so a caller can stage a large
 * host buffer through the device piece by piece, or give every GPU its own range.  The
 * reference has no counterpart: its CUDA programs move the whole volume in one kernel. */
int32_t lego_permute_slab_info(int32_t elem_bytes, const lego_layout_t* src, const lego_layout_t* dst,
                               int64_t* n_slabs, int64_t* slab_elems);
int32_t lego_permute_slabs(const void* in, void* out, int32_t elem_bytes, const lego_layout_t* src,
                           const lego_layout_t* dst, int64_t slab_count, void* stream);

/* ---- row-wise kernels ----------------------------------------------------- */

/* y = softmax(x) along the last axis of a contiguous rows x cols matrix, fp32
 * arithmetic; replaces softmax_kernel, triton_generated/softmax/softmax.py:33-58
 * and its host softmax(), :97-160.  row_map (nullable) is a layout over `rows`
 * logical ids whose apply() gives the row a work item processes (the reference
 * strides rows over persistent programs).                                      */
int32_t lego_softmax_f16(const void* x, void* y, int64_t rows, int64_t cols,
                         const lego_layout_t* row_map, void* stream);
int32_t lego_softmax_f32(const void* x, void* y, int64_t rows, int64_t cols,
                         const lego_layout_t* row_map, void* stream);

/* LayerNorm forward: y = (x - mean) * rstd * gamma + beta, biased variance,
 * fp32 statistics written to mean/rstd (dev float[rows]); replaces
 * _lego_layer_norm_fwd_fused, triton_generated/layernorm/layernorm.py:58-101
 * and LEGOLayerNorm.forward, :279-307.  x, gamma, beta, y: dev fp16.           */
int32_t lego_layernorm_fwd_f16(const void* x, const void* gamma, const void* beta, void* y,
                               float* mean, float* rstd, int64_t rows, int64_t cols, float eps,
                               const lego_layout_t* row_map, void* stream);

/* LayerNorm backward: dx per row, dgamma/dbeta by a deterministic two-stage
 * column reduction; replaces _lego_layer_norm_bwd_dx_fused and
 * _lego_layer_norm_bwd_dwdb, layernorm.py:163-267.  partial: dev float
 * [2 * lego_layernorm_bwd_partial_rows(rows, cols) * cols] scratch supplied by
 * the caller.                                                                  */
int64_t lego_layernorm_bwd_partial_rows(int64_t rows, int64_t cols);
int32_t lego_layernorm_bwd_f16(const void* dy, const void* x, const void* gamma, const float* mean,
                               const float* rstd, void* dx, void* dgamma, void* dbeta,
                               float* partial, int64_t rows, int64_t cols, void* stream);

/* ---- GEMM ----------------------------------------------------------------- */

enum { LEGO_ACT_NONE = 0, LEGO_ACT_LEAKY_RELU = 1 };

/* C[M,N] = act(op(A) . op(B)), fp16 in, fp32 accumulate on tcgen05/TMEM, fp16
 * out; replaces matmul_kernel / matmul(), triton_generated/matmul/
 * matmul_NTA_NTB.py:97-145 (and the _TA/_TB variants).  trans_a = 0: A is
 * row-major [M,K]; 1: A is stored as row-major [K,M].  trans_b = 0: B is
 * row-major [K,N]; 1: stored as row-major [N,K].  tile_order (nullable) is a
 * layout with logical dims (M/128, N/256) whose inv(pid) gives (pid_m, pid_n),
 * the grouped swizzle of benchmarks/triton/matmul_sympy.py:57-65; NULL = row-
 * major tile order.  Any M; N % 8 == 0, K % 8 == 0 (M % 8 == 0 with trans_a):
 * rows are 16-byte multiples; tile edges are masked (the reference kernel has no
 * masks and needs M % 128 == N % 256 == K % 64 == 0).                           */
int32_t lego_gemm_f16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                      int32_t trans_a, int32_t trans_b, int32_t activation,
                      const lego_layout_t* tile_order, void* stream);

/* The same GEMM with 8-bit floating-point operands (e5m2: 1 sign, 5 exponent, 2
 * mantissa bits; torch.float8_e5m2), fp32 accumulate (tcgen05 kind::f8f6f4), fp16
 * C; replaces matmul() called on fp8 tensors, benchmarks/triton/
 * matmul_sympy.py:346-364 (TORCH_HAS_FP8 branch).  Arguments as lego_gemm_f16;
 * operand rows are 16-byte multiples: K % 16 == 0, N % 16 == 0 unless trans_b,
 * M % 16 == 0 with trans_a; N % 8 == 0 always (C is fp16).                      */
int32_t lego_gemm_e5m2(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                       int32_t trans_a, int32_t trans_b, int32_t activation,
                       const lego_layout_t* tile_order, void* stream);

/* The same two GEMMs with a caller-owned scratch buffer that lets the library split the
 * partial last wave of tiles along K (a stream-K tail; opt-in through lego_tune): when
 * the tile count is not a multiple of what the GPU holds at once -- 8192 x 8192 x 8192 is
 * 13.8 waves, a 1024-row slab of it 1.7 -- every pair of SMs gets the same number of k-steps, partial fp32
 * accumulators travel through the buffer and the tile's owner adds them in a fixed order
 * (same bits on every run).  No counterpart in the reference, whose matmul() launches
 * one program per tile and leaves the tail to the hardware scheduler
 * (triton_generated/matmul/matmul_NTA_NTB.py:136-145).
 *
 * workspace: device memory, 16-byte aligned, lego_gemm_workspace_bytes() bytes for the
 * current device (NULL or a smaller buffer: the call runs like lego_gemm_f16).  Its first
 * 8 KiB are flags: zero them once after allocating; every call that completes leaves
 * them zero.  After a LEGO_ERR_DEVICE_TIMEOUT zero them again.  Calls that may overlap
 * on the GPU need a buffer each.                                                 */
int64_t lego_gemm_workspace_bytes(void);
int32_t lego_gemm_f16_ws(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                         int32_t trans_a, int32_t trans_b, int32_t activation,
                         const lego_layout_t* tile_order, void* workspace, int64_t workspace_bytes,
                         void* stream);
int32_t lego_gemm_e5m2_ws(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                          int32_t trans_a, int32_t trans_b, int32_t activation,
                          const lego_layout_t* tile_order, void* workspace, int64_t workspace_bytes,
                          void* stream);

/* Process-wide tuning knobs of the GEMMs (the reference exposes the same kind of choice
 * through its @triton.autotune lists, matmul_NTA_NTB.py:17-52).
 *   LEGO_TUNE_GEMM_BLOCKS   0 = library's choice, 1 = 256 x 256 output per SM pair,
 *                           2 = 512 x 256 per SM pair when the tile order allows it
 *   LEGO_TUNE_GEMM_STREAMK  0 = never split along K (default), 1 = when a workspace is given and
 *                           the last wave of tiles would leave SMs idle, 2 = whenever a
 *                           workspace is given and the tile count is not a multiple of the
 *                           resident SM pairs
 *   LEGO_TUNE_GEMM_LAG      0..4 k-steps by which the first accumulator block of a 512 x 256
 *                           tile leads the second at the start of a tile (the second block of the
 *                           previous tile is still being read out of tensor memory meanwhile)
 *   LEGO_TUNE_LNBWD_SPLIT   LayerNorm backward: rows wider than this many columns are taken by
 *                           one group of 512 threads, narrower ones by several groups
 *   LEGO_TUNE_PERMUTE_TILE_VECS  most 16-byte vectors per tile of the chunk-tiled permute (64 .. 6144)
 *   LEGO_TUNE_PERMUTE_DMA_TILE   most bytes per box of the DMA permute (2048 .. 49152); 0 = the
 *                           chunk-tiled kernel takes those pairs of layouts instead
 *   LEGO_TUNE_PERMUTE_DMA_CTAS   CTAs per SM of the DMA permute (1 .. 4)
 *   LEGO_TUNE_PERMUTE_DMA_LONG   1 (default) = the DMA permute also takes pairs of layouts whose common
 *                           run is a whole 128-byte line or more (problems of 4 MiB and more), 0 = the
 *                           output-order vector copy keeps them
 *   LEGO_TUNE_PDL_LAST_WAVE      index-map kernels: 1 (default) = a grid that fills at most half of
 *                           the machine lets the next grid of the stream become resident beside
 *                           it, 0 = rule by grid depth alone
 *   LEGO_TUNE_LNBWD_LANES        LayerNorm backward, grouped kernel: 0 = one producer thread, 1
 *                           (default) = a producer lane per group where a ring slot holds one
 *                           row, 2 = the same and never a block of rows per slot; + 8 = every
 *                           group writes its own partial row of column sums (no fold in the CTA)
 *   LEGO_TUNE_LNBWD_MIN_ROWS     LayerNorm backward: fewest rows for which the ring-fed kernels are
 *                           used (below, one CTA per row with the row in registers)
 *   LEGO_TUNE_LNBWD_FOLD_WARP    LayerNorm backward, rows of up to 4 Ki columns: most consumer groups
 *                           for which an extra warp per group adds up the rows' sums (0 .. 3; 0:
 *                           every consumer thread folds its group's sums itself) */
enum { LEGO_TUNE_GEMM_BLOCKS = 1, LEGO_TUNE_GEMM_STREAMK = 2, LEGO_TUNE_GEMM_LAG = 3, LEGO_TUNE_LNBWD_SPLIT = 4,
       LEGO_TUNE_PERMUTE_TILE_VECS = 5, LEGO_TUNE_PERMUTE_DMA_TILE = 6, LEGO_TUNE_PERMUTE_DMA_CTAS = 7,
       LEGO_TUNE_PDL_LAST_WAVE = 8, LEGO_TUNE_LNBWD_LANES = 9, LEGO_TUNE_PERMUTE_DMA_LONG = 10,
       LEGO_TUNE_LNBWD_MIN_ROWS = 11, LEGO_TUNE_LNBWD_FOLD_WARP = 12 };
int32_t lego_tune(int32_t knob, int32_t value);

/* G independent problems C_g = A_g . B_g (row-major, contiguous), walked by
 * persistent CTAs through the concatenated tile lists; replaces
 * lego_grouped_matmul_kernel / lego_group_gemm_fn, triton_generated/
 * grouped_gemm/grouped_gemm.py:39-162.  A, B, C: host arrays of G device
 * pointers; mnk: host int64 [G,3].  tile_orders (nullable): host array of G
 * layout pointers, entry g with logical dims (M_g/128, N_g/256).  The call uploads
 * its problem table from host memory that does not outlive it, so it cannot be
 * part of a stream capture: on a capturing stream it returns
 * LEGO_ERR_UNSUPPORTED and enqueues nothing.                                    */
int32_t lego_grouped_gemm_f16(const void* const* A, const void* const* B, void* const* C,
                              const int64_t* mnk, int32_t G,
                              const lego_layout_t* const* tile_orders, void* stream);

/* Grouped GEMM for callers that must not allocate.  No counterpart in the
 * reference: its lego_group_gemm_fn allocates freely through torch.
 *
 * Who needs it: code that runs where a device allocation is impossible or
 * unwelcome -- inside a serving loop whose memory is entirely owned by a
 * framework's caching allocator (a cudaMalloc there can fail or stall every
 * stream of the device while the driver maps memory), or in a process that has
 * handed all free memory to other libraries.  lego_grouped_gemm_f16 creates a
 * per-device workspace with cudaMalloc on its first use; this variant calls no
 * cudaMalloc / cudaFree and no allocating library routine at all.  Its scratch
 * (the problem table the persistent CTAs read, and a status word) is a
 * file-scope __device__ array of LEGO_STATIC_SCRATCH_BYTES that every GPU
 * loading the library holds until the process exits; the host-side records are
 * built on the stack.
 *
 * Same arguments and results as lego_grouped_gemm_f16, plus dev_status: a
 * device uint32 owned and zeroed by the caller that receives the code of a
 * bounded wait that ran out, or NULL to use a word inside the array, which
 * lego_device_status reads and clears (without allocating anything either).
 * G > LEGO_STATIC_MAX_GROUPS is rejected with LEGO_ERR_SIZE.
 *
 * The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and the SM count.  Like
 * lego_grouped_gemm_f16, no call of this entry point may be part of a stream
 * capture (the problem table is uploaded from the caller's stack): on a capturing
 * stream it returns LEGO_ERR_UNSUPPORTED and enqueues nothing.  Every call on a
 * device shares the one array and overwrites what the previous call left there,
 * so two calls whose kernels may overlap on the GPU (different streams) race:
 * order them.                                                                  */
#define LEGO_STATIC_MAX_GROUPS     64
#define LEGO_STATIC_SCRATCH_BYTES  (256 + LEGO_STATIC_MAX_GROUPS * 640)
int32_t lego_grouped_gemm_f16_static(const void* const* A, const void* const* B, void* const* C,
                                     const int64_t* mnk, int32_t G,
                                     const lego_layout_t* const* tile_orders, uint32_t* dev_status,
                                     void* stream);

/* ---- housekeeping --------------------------------------------------------- */

/* Strided copy of `height` rows of `width_bytes` between any two of host (pinned for a
 * copy that overlaps) and device memory, enqueued on `stream` (cudaMemcpy2DAsync,
 * direction inferred).  It lets a binding stage a column slab of a host matrix without
 * packing it first, which is how the host-buffer transpose overlaps copy-in, kernel and
 * copy-out.  No counterpart in the reference (its harnesses keep everything on the
 * device, lego/lego_mlir.py:114-165).                                               */
int32_t lego_copy_2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch,
                     int64_t width_bytes, int64_t height, void* stream);


/* Synchronise `stream` and return (then clear) the current device's status word:
 * LEGO_OK or LEGO_ERR_DEVICE_TIMEOUT; *detail (nullable) receives the raw word.
 * Covers the workspace's word and the one inside the static array; allocates nothing. */
int32_t lego_device_status(void* stream, uint32_t* detail);

/* Runs the give-up path of the kernels' bounded waits for real, without a fault: one
 * CTA waits on a barrier nothing will ever complete, gives up after limit_cycles SM
 * cycles (1 .. 2e9), records code 0x7e570000 in the status word like a production
 * kernel does, and returns.  lego_device_status then reports
 * LEGO_ERR_DEVICE_TIMEOUT once; the device stays usable.  No counterpart in the
 * reference (its kernels have no waits to bound).                              */
int32_t lego_selftest_bounded_wait(int64_t limit_cycles, void* stream);

const char* lego_status_string(int32_t status);

/* Free every per-device workspace.  Safe to call more than once.               */
int32_t lego_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* LEGO_B200_H_ */
