/*
 * aiehlc_b200 -- C ABI of the B200 kernel-call path.
 *
 * These entry points are what a host program written against aiehlc's kernel-call
 * surface binds to when the AIE tile kernels are replaced by sm_100a kernels.  Each one
 * cites the reference construct it stands in for (paths relative to the aiehlc tree).
 *
 * Layout contract (the reference's CPU golden loop, example/perf/aieml_perf.cc:199-231):
 *   A[M][K] row-major, B stored [N][K] ("column-major B": the K-vector of every output
 *   column is contiguous), C[M][N] row-major, integer accumulation in 32 bits:
 *       C[i][j] = sum_k A[i][k] * B[j][k]
 *
 * Conventions
 *   - every function returns AIEHLC_OK (0) or a negative error code; no exceptions cross
 *     the boundary; aiehlc_last_error() gives the message of the calling thread's last failure;
 *   - `_dev` functions take device pointers, enqueue on `stream` (a cudaStream_t passed as
 *     void*; NULL is CUDA's default stream) and return without synchronising;
 *   - `_host` functions take host pointers, stage through context-owned device buffers on the
 *     context's own stream (H2D copy, kernel, D2H copy) and return after the result is in the
 *     host buffer;
 *   - there is no CPU fallback: without a usable CUDA device aiehlc_create() fails.
 *   - one context per host thread / stream: calls on one context must not overlap.
 */
#ifndef AIEHLC_B200_H
#define AIEHLC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AIEHLC_OK 0
#define AIEHLC_ERR_INVALID (-1)     /* bad argument (null pointer, negative size, shift > 31 ...) */
#define AIEHLC_ERR_CUDA (-2)        /* a CUDA runtime / driver call failed */
#define AIEHLC_ERR_UNSUPPORTED (-3) /* shape outside what the kernel family covers */
#define AIEHLC_ERR_DEVICE (-4)      /* a kernel reported a non-zero status word (bounded wait ran out) */
#define AIEHLC_ERR_NOMEM (-5)

typedef struct aiehlc_ctx aiehlc_ctx;

/* Device bring-up.  Stands in for the XAie_CfgInitialize / XAie_PartitionInitialize sequence
 * of every example's main() (example/perf/aieml_perf.cc:265-313): selects CUDA device `device`,
 * creates the context's stream and its status word. */
int aiehlc_create(int device, aiehlc_ctx** out);
/* XAie_PartitionTeardown (aieml_perf.cc:321): frees every buffer the context owns. */
int aiehlc_destroy(aiehlc_ctx* ctx);
const char* aiehlc_last_error(void);
int aiehlc_sm_count(const aiehlc_ctx* ctx);
/* Waits for `stream`, then reads and clears the device status word.
 * Non-zero *status means a kernel gave up on a bounded wait; results of that launch are invalid.
 * Plays the part of the XAie_CoreWaitForDone poll (aieml_perf.cc:174-184). */
int aiehlc_sync(aiehlc_ctx* ctx, void* stream, int* status);

/* ---- the reference's own kernel: int32 x int32 -> int32 (wrap-around) ----------------------
 * `perf` (example/perf/aieml_perf.cc:61-83) and `mm` (example/matrixmultiply/aieml_mm.cc:41-93),
 * generalised from 16x16x16 to M,N,K.  `in` is the packed window the examples fill: A (M*K
 * words) followed by B (N*K words); `out` is C (M*N words).  Arithmetic is uint32 wrap-around
 * exactly as the kernel's `ret += vec1[..] * vec2[..]` (aieml_perf.cc:74-82). */
int aiehlc_mm_i32_dev(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K,
                      void* stream);
int aiehlc_mm_i32_host(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K);

/* ---- int8 x int8 -> int32 tile GEMM (tcgen05 kind::i8, int32 accumulators in TMEM) ---------
 * The golden loop of aieml_perf.cc:199-231 with int8 operands sign-extended to 32 bits; the
 * tile shape / K-loop-then-flush structure follows the compiler's matmul tiling
 * (src/mlir/mlirfront/tilinglinalg/tilinglinalg.cpp:101-129, tiling.py:299-333).
 * accumulate != 0: C += A.B^T, i.e. stage s>0 of a multi-launch cascade over K slices (the
 * chained-kernel pattern of example/multi/multi_tile.cpp:105-145, seq_full_col.cpp:132-153). */
int aiehlc_gemm_i8_i32_dev(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int32_t* C, int M,
                           int N, int K, int accumulate, void* stream);
/* The same product ADDED into a row-sharded C: rows [g * rows_per_shard, (g + 1) * rows_per_shard) of
 * C are the dense int32 matrix shards[g] ([rows][N]; the last used shard holds
 * M - g * rows_per_shard rows).  A shard may be memory of ANOTHER GPU that this device can address
 * (peer access enabled, or a mapping of the owner's allocation): the epilogue adds its results with
 * system-scope reductions, so every GPU of a split-K group can run this call on its K slice at the same time
 * and the owner of a shard ends with the sum -- the GEMM and the reduce-scatter of the cascade
 * (the K-slice stages of example/multi/multi_tile.cpp:105-145 spread over GPUs) in one kernel, with
 * no partial-sum matrix.  The caller zeroes the shards before the first contribution and orders
 * "all zeroed" -> calls -> "all done" -> reads across the GPUs (e.g. with two barriers).
 * rows_per_shard must be a multiple of 128, num_shards <= AIEHLC_MAX_SHARDS.
 * first_shard: when M fills every shard, consecutive tiles belong to consecutive shards (first_shard,
 * first_shard + 1, ...), so the tiles in flight at any moment spread over all owners and GPUs that
 * pass different values (own rank + 1) lean on different owners; it never changes the result. */
#define AIEHLC_MAX_SHARDS 16
int aiehlc_gemm_i8_i32_scatter_dev(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int32_t* const* shards,
                                   int num_shards, int rows_per_shard, int first_shard, int M, int N, int K,
                                   void* stream);
int aiehlc_gemm_i8_i32_host(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int32_t* C, int M,
                            int N, int K);

/* ---- int8 GEMM with the fused shift-round-saturate output stage ---------------------------
 * C(int8)[i][j] = srs( sum_k A[i][k]*B[j][k] + (acc_in ? acc_in[i][j] : 0), s_j )
 *   s_j = shift_vec ? shift_vec[j] : shift,   0 <= s <= 31
 *   srs(x, s): q = x >> s (arithmetic); r = x & (2^s - 1); q += (r > 2^(s-1)) || (r == 2^(s-1) && q odd);
 *              result = clamp(q, -128, 127)            -- round half to even, saturate; s = 0: clamp only
 * `splitk` (>= 1, must divide K): the K range is walked as `splitk` consecutive equal slices that are
 * accumulated in slice order inside TMEM and flushed once -- the cascade formulation executed
 * within one launch.  Integer addition is associative, so the result equals the unsplit one.
 * The reference has no srs stage of its own; this definition is the contract (no counterpart file). */
int aiehlc_gemm_i8_srs_dev(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int8_t* C, int M, int N,
                           int K, int shift, const uint8_t* shift_vec, const int32_t* acc_in,
                           int splitk, void* stream);
int aiehlc_gemm_i8_srs_host(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int8_t* C, int M,
                            int N, int K, int shift, const uint8_t* shift_vec, int splitk);

/* Flush of a cascade kept in an int32 buffer: out(int8) = srs(in, shift) element-wise over a
 * rows x cols row-major matrix (shift_vec indexes columns).  The last hop of the chain in
 * example/multi/seq_full_col.cpp:156-159 (tile -> external memory). */
int aiehlc_srs_i32_i8_dev(aiehlc_ctx* ctx, const int32_t* in, int8_t* out, long long rows,
                          long long cols, int shift, const uint8_t* shift_vec, void* stream);

/* ---- bf16 x bf16 -> bf16 GEMM (tcgen05 kind::f16, fp32 accumulators in TMEM) ---------------
 * Same loop nest and layout as above; operands and result are raw bf16 bit patterns.
 * No counterpart kernel in the reference (its kernels are integer). */
int aiehlc_gemm_bf16_dev(aiehlc_ctx* ctx, const uint16_t* A, const uint16_t* B, uint16_t* C, int M,
                         int N, int K, void* stream);
int aiehlc_gemm_bf16_host(aiehlc_ctx* ctx, const uint16_t* A, const uint16_t* B, uint16_t* C, int M,
                          int N, int K);

/* ---- int8 conv2d as an implicit GEMM, per-output-channel srs ------------------------------
 * x: NHWC int8 [n][h][w][cin]; w: HWIO int8 [kh][kw][cin][cout]; y: NHWC int8 [n][h][w][cout]
 * stride 1, zero padding `pad` on every side, output spatial size = input spatial size
 * (requires kh = kw = 2*pad + 1).  y = srs( sum_{kh,kw,ci} x[n][oh+kh-pad][ow+kw-pad][ci] * w[kh][kw][ci][co], shift_vec[co] ).
 * No counterpart kernel in the reference. */
int aiehlc_conv2d_i8_srs_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n,
                             int h, int wd, int cin, int cout, int kh, int kw, int pad,
                             const uint8_t* shift_vec, void* stream);
int aiehlc_conv2d_i8_srs_host(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n,
                              int h, int wd, int cin, int cout, int kh, int kw, int pad,
                              const uint8_t* shift_vec);

/* Weights that do not change between calls (inference) can be re-laid once: pack_weights writes
 * w[kh][kw][cin][cout] as [kh*kw][cout][cin] (kh*kw*cin*cout bytes, 16-byte aligned) and the _packed
 * entry point runs the convolution on that copy with a single kernel launch.  Tensor-core shapes only
 * (cin 32, 64 or a multiple of 128; cout a multiple of 16). */
int aiehlc_conv2d_pack_weights_dev(aiehlc_ctx* ctx, const int8_t* w, int8_t* packed, int kh, int kw, int cin,
                                   int cout, void* stream);
int aiehlc_conv2d_i8_srs_packed_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* packed, int8_t* y, int n,
                                    int h, int wd, int cin, int cout, int kh, int kw, int pad,
                                    const uint8_t* shift_vec, void* stream);

/* ---- tiling plan --------------------------------------------------------------------------
 * What the GEMM entry points will do for a problem, without running it: tile shape, tile grid,
 * waves over the persistent CTAs (or CTA pairs), pipeline depth, and how operands are shared.
 * Counterpart of the compiler's matmul tiling and broadcast analysis
 * (src/mlir/mlirfront/tilinglinalg/tilinglinalg.cpp:38-146, tilingpass.cpp:98-150), which prints the
 * tile grid and which operand must be broadcast along which grid dimension. */
typedef struct {
  int tile_m, tile_n, tile_k_bytes;  /* output tile of one CTA (or CTA pair); K bytes per pipeline stage */
  int cta_pair;                      /* 1: two CTAs (tcgen05 cta_group::2) per tile */
  int grid_m, grid_n;                /* tile grid */
  long long tiles;
  int slots;                         /* tiles in flight: persistent CTAs or CTA pairs */
  int waves;                         /* ceil(tiles / slots) */
  double wave_efficiency;            /* tiles / (waves * slots) */
  int group_m;                       /* tile row-blocks walked before the next tile column */
  int stages, smem_bytes, tmem_columns, k_blocks;
  int a_shared_by;                   /* tiles reading the same rows of A (A is shared along the N grid dimension) */
  int b_shared_by;                   /* tiles reading the same rows of B (B is shared along the M grid dimension) */
  long long wave_footprint_bytes;    /* operand bytes the tiles of one wave touch (L2 working set) */
  double cost_units;                 /* the quantity the choice minimises: waves x tile_n / efficiency factor */
  int split_k_tiles;                 /* int8 CTA-pair launches whose last wave is at most half full: that many tail tiles run as
                                        two K halves on different pairs (the upper halves first, the lower halves last, their
                                        int32 partial sums meeting in the output stage of the lower half); 0 = none */
  int split_k_at;                    /* the K block (of 128 bytes) where those tiles are cut */
  int narrow_tail_tiles;             /* tiles of a thin last wave that are cut into two column ranges, else 0 */
} aiehlc_gemm_plan;
/* kind: 0 = int8, 1 = bf16.  ctx may be NULL: the plan is then made for a 148-SM B200 with default knobs. */
int aiehlc_plan_gemm(aiehlc_ctx* ctx, int kind, int M, int N, int K, aiehlc_gemm_plan* plan);
/* The order in which that plan's tiles are visited (the traversal the compiler's tiling pass fixes when it
 * walks the tile grid, tilinglinalg.cpp:101-129), computed by the function the kernels themselves call:
 * tile t covers row block row_block[t] (of plan.tile_m rows) and column block col_block[t]; with *slots
 * persistent CTAs (or CTA pairs) slot s runs tiles s, s + slots, ...  num_shards > 0 gives the order of
 * aiehlc_gemm_i8_i32_scatter_dev (consecutive tiles on consecutive shards, slot count coprime with
 * the shard count); 0 the plain order.  Returns the number of tiles (<= capacity) or a negative error.
 * Needs no GPU (ctx may be NULL). */
int aiehlc_plan_tile_order(aiehlc_ctx* ctx, int kind, int M, int N, int K, int num_shards, int rows_per_shard,
                           int first_shard, int* row_block, int* col_block, int capacity, int* slots);

/* What the convolution entry points will do for a problem, without running it (needs no GPU; ctx may be
 * NULL: planned for a 148-SM B200 with default knobs).  The reference's compiler decides tile shapes and
 * data movement per kernel at compile time (tilinglinalg.cpp:38-146); this is that decision for conv2d. */
typedef struct {
  int form;                  /* 1 = patch form (one input patch + all taps' weights per CTA and cin chunk),
                                0 = per-tap form, 2 = CUDA-core kernel (shape outside the tensor-core tiling) */
  int tile_rows, tile_width; /* output pixels of one CTA: image rows x columns */
  int patch_rows, patch_width; /* input rows x pixels one activation box brings (patch form: + kh-1, + kw-1) */
  int m_rows_used;           /* of the 128 MMA rows (patch form computes and drops kw-1 columns per image row) */
  int cout_tile, cin_chunk;  /* N of the MMA; K bytes per box */
  int ctas, tma_boxes_per_cta, mmas_per_cta, stages, smem_bytes;
  int launches;              /* kernels per aiehlc_conv2d_i8_srs_dev call: 1, or 2 when the HWIO weights are re-laid first
                                (16-byte aligned weights assumed) */
  int persistent;            /* 1 = many tiles per SM: `ctas` persistent CTAs keep the weights in shared memory and walk
                                the tiles (stages = input patches in flight); tma_boxes_per_cta and mmas_per_cta then
                                count a CTA's whole walk */
} aiehlc_conv_plan;
int aiehlc_plan_conv2d(aiehlc_ctx* ctx, int n, int h, int wd, int cin, int cout, int kh, int kw, int pad,
                       aiehlc_conv_plan* plan);

/* ---- the same convolution for callers that must not allocate -----------------------------
 * (No counterpart in the reference: aiehlc has neither a convolution nor a device allocator.)
 * Meant for callers that cannot reach the device allocator when they call: a frozen memory pool, a
 * latency-critical loop that must not take the driver's allocation lock, a host that has handed
 * the whole device to someone else.  Same arguments and bit-identical results as
 * aiehlc_conv2d_i8_srs_dev, but the re-laid weights live in a fixed array inside the library
 * (AIEHLC_CONV_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until the process
 * ends) instead of a workspace that grows with cudaMalloc.  Form, tiling and kernels are those of the
 * regular entry point (aiehlc_plan_conv2d describes both); shapes whose HWIO weights feed the tensor
 * cores as they are do not touch the array at all.
 *   - kh*kw*cin*cout above AIEHLC_CONV_STATIC_SCRATCH_BYTES is refused with AIEHLC_ERR_UNSUPPORTED.
 *   - The FIRST call on a device is not allocation-free: it resolves the array's device address
 *     (cudaGetSymbolAddress) and, with CUDA's lazy module loading, makes the driver load the kernels
 *     and the array itself, which allocates device memory.  Make one warm-up call per device while
 *     allocation is still allowed -- before the pool is frozen and before any stream capture.  Every
 *     later call performs no cudaMalloc / cudaFree and calls no allocating routine.
 *   - All calls on a GPU share the one array and it keeps what the last call left there; each call
 *     rewrites every byte it later reads, so results never depend on earlier calls -- but two calls
 *     that overlap on the GPU (different streams, or different contexts on one device) race on it.
 *     Serialise them. */
#define AIEHLC_CONV_STATIC_SCRATCH_BYTES (1u << 20)
int aiehlc_conv2d_i8_srs_static_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n,
                                    int h, int wd, int cin, int cout, int kh, int kw, int pad,
                                    const uint8_t* shift_vec, void* stream);

/* Number of kernel launches this context has enqueued since creation. */
long long aiehlc_launch_count(const aiehlc_ctx* ctx);
/* Number of times this context has moved one of its device workspaces (staging buffers of the _host
 * entry points, re-pitched operands, re-laid convolution weights, ...) to a larger allocation.  A CUDA
 * graph recorded over calls on this context holds the old addresses: it must be recorded again once
 * this number has changed (XAie_GraphLaunch checks exactly that). */
long long aiehlc_workspace_generation(const aiehlc_ctx* ctx);

/* Tuning knobs and measurement aids are declared in aiehlc_b200_tuning.h; nothing a caller of the entry
 * points above needs. */

#ifdef __cplusplus
}
#endif
#endif /* AIEHLC_B200_H */
