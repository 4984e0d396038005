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
  int split_tail_tiles;              /* tiles of a thin last wave that are cut along K (int8 pair kernel), else 0 */
  int split_tail_parts;              /* K ranges per such tile (1 = none) */
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
 * ends) instead of a workspace that grows with cudaMalloc.  The call performs no cudaMalloc /
 * cudaFree and calls no allocating routine.
 *   - kh*kw*cin*cout above AIEHLC_CONV_STATIC_SCRATCH_BYTES is refused with AIEHLC_ERR_UNSUPPORTED.
 *   - The first call on a device resolves the array's device address (cudaGetSymbolAddress); make
 *     that first call before starting any stream capture.
 *   - All calls on a GPU share the one array and it keeps what the last call left there; each call
 *     rewrites every byte it later reads, so results never depend on earlier calls -- but two calls
 *     that overlap on the GPU (different streams, or different contexts on one device) race on it.
 *     Serialise them. */
#define AIEHLC_CONV_STATIC_SCRATCH_BYTES (1u << 20)
int aiehlc_conv2d_i8_srs_static_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n,
                                    int h, int wd, int cin, int cout, int kh, int kw, int pad,
                                    const uint8_t* shift_vec, void* stream);

/* Tuning knob for experiments: force the N extent of the GEMM tile (64, 128 or 256; 0 = choose). */
int aiehlc_set_tile_n(aiehlc_ctx* ctx, int tile_n);
/* Tuning knob: 1 = run the GEMM tiles on CTA pairs (tcgen05 cta_group::2, 256-row tiles, each CTA
 * fetching half of the B tile) wherever M > 128, 0 = one CTA per 128-row tile, -1 = choose per
 * shape (the default). */
int aiehlc_set_cta_pair(aiehlc_ctx* ctx, int mode);
/* Tuning knob for the CTA-pair kernel: 128-byte K blocks fetched by one TMA tile load (and held by one
 * pipeline stage).  2 needs K * element size to be a multiple of 128 bytes; 0 (default) = 2 where that
 * holds, else 1. */
int aiehlc_set_k_per_load(aiehlc_ctx* ctx, int k_blocks);
/* Tuning knob: 1 (default) = the int32 and bf16 GEMM epilogues stage 32 rows x 128 bytes of results in
 * shared memory and write them with a TMA tile store (whole 128-byte lines, clipped at the edges of C;
 * `accumulate` uses the add-reduction form); 2 = the int8 srs epilogue does so too (measured slower than
 * its per-thread 32-byte stores); 0 = every thread stores its own row directly.  Tile stores need C
 * 16-byte aligned with a 16-byte row pitch; otherwise the direct path is taken whatever the setting. */
int aiehlc_set_tma_store(aiehlc_ctx* ctx, int on);
/* Tuning knob for the CTA-pair kernel: groups of four epilogue warps per CTA.  2 = the two warps of a
 * TMEM lane quarter each drain half of a tile's columns (one staging buffer per warp; more accumulator
 * reads, proxy fences and tile stores in flight: where the output stage sets the pace, K <= 1024 bytes,
 * results leave 10-18 % faster); 1 = four warps with two staging buffers each (1-2 % faster where K is
 * deep); 0 (default) = 2 up to 8 K blocks of 128 bytes for int8 operands and 4 for bf16 (and never for a
 * row-sharded output, which the wire bounds), else 1. */
int aiehlc_set_epilogue_groups(aiehlc_ctx* ctx, int groups);
/* Tuning knob for a thin last wave (at most half of the CTA pairs busy) of a CTA-pair launch:
 *   1 = (int8 only) its tiles are cut along K into up to 4 ranges run by otherwise idle pairs; the ranges
 *       exchange int32 partial sums through a context workspace and each runs the output stage on its
 *       share of the columns (integer sums: bit-identical results);
 *   2 = (default) its 256-column tiles are cut into two 128-column ranges run by different pairs (narrower
 *       MMAs, nothing to exchange; every output element is still one accumulation over K in the same
 *       order); measured 48.3 us against 49.7 us on the 4096^3 benchmark;
 *   0 = every tile computed whole. */
int aiehlc_set_split_tail(aiehlc_ctx* ctx, int on);
/* Tuning knob for the *_host GEMM entry points: number of row blocks of A / C that upload, kernel and
 * download are pipelined over (0 = default 4; blocks are whole 256-row tiles). */
int aiehlc_set_host_blocks(aiehlc_ctx* ctx, int blocks);
/* Tuning knob for the convolution kernel: 1 (default) = a CTA fetches its tile's whole input patch
 * (rows + kh - 1 image rows of width + kw - 1 pixels, zero-filled outside the image) with ONE TMA box and
 * every tap's weights with another, and the kh * kw taps are kh * kw views into that one patch; 0 = one
 * activation box and one weight box per tap.  Filters whose taps do not fit in shared memory take the
 * second form whatever the setting. */
int aiehlc_set_conv_halo(aiehlc_ctx* ctx, int on);
/* Tuning knob for aiehlc_mm_i32_*: 1 (default) = products of at least 2^24 multiply-adds (K >= 64) run on the
 * int8 tensor cores: the int32 operands are cut into unsigned bytes, four int8 GEMMs (one per power of
 * 256, operands of K, 2K, 3K and 4K bytes; K in ranges of 8192 so that no partial sum can reach 2^31) add
 * their shifted results, which is the reference kernel's uint32 wrap-around arithmetic bit for bit;
 * 0 = always the CUDA-core kernel; 2 = always the tensor cores, whatever the size (for tests: the reference's
 * 16 x 16 x 16 fixture through this form). */
int aiehlc_set_mm_i32_tensor(aiehlc_ctx* ctx, int on);
/* Tuning knob for aiehlc_conv2d_i8_srs_dev / _host: 1 (default) = where the patch form applies and the
 * output-channel tile is 32, 64 or 128 wide, the HWIO weights are fetched as they are (rows of output
 * channels: the tensor core's N-major operand layout) and the convolution is one launch; 0 = weights
 * are always re-laid to [tap][cout][cin] by a pre-pass launch first. */
int aiehlc_set_conv_hwio_direct(aiehlc_ctx* ctx, int on);
/* Tuning knob for the convolution's patch form: 1 = the kw taps of a filter row are ONE MMA with
 * N = kw * (output-channel tile) and the epilogue adds the taps' column blocks of neighbouring rows (filters up
 * to 4 wide, kw * tile <= 256); 0 (default) = one MMA per tap and 32-byte K step.  Same bits either way;
 * measured slower on the 56 x 56 x 64 benchmark (5.7 us against 4.9 us: the wider MMAs wait for the same
 * weight boxes and the epilogue has three accumulator blocks to add). */
int aiehlc_set_conv_wide_n(aiehlc_ctx* ctx, int on);
/* Tuning knob for aiehlc_gemm_i8_i32_scatter_dev: 1 (default) = results leave as add-reducing TMA tile
 * stores (32 rows x 128 bytes per store; needs N a multiple of 4 and 16-byte aligned shards, else the
 * other form is used), 0 = as per-row reduction instructions issued by the epilogue warps.  Measured
 * between two B200 (65536 x 8192 x 4096 per GPU, half of the tiles remote): 2.04 ms against 2.10 ms,
 * all shards local 1.63 ms against 2.08 ms. */
int aiehlc_set_shard_tile_stores(aiehlc_ctx* ctx, int on);
/* Tuning knob: number of tile row-blocks the persistent scheduler walks before it moves to the next
 * tile column (the L2 footprint of one wave is group_m row-blocks of A plus slots/group_m column-blocks
 * of B).  0 = default: 8 for CTA-pair tiles, 16 for single-CTA tiles (about square wave footprints). */
int aiehlc_set_group_m(aiehlc_ctx* ctx, int group_m);
/* Tuning knob: 1 (default) = the tensor-core kernels are launched with programmatic stream
 * serialization, so their set-up (barriers, TMEM allocation) overlaps the tail of the kernel before
 * them in the stream; they still wait for that kernel to complete before touching global memory.
 * 0 = plain stream-ordered launches. */
int aiehlc_set_pdl(aiehlc_ctx* ctx, int on);
/* Measurement aid for the GEMM kernels (results are then meaningless): 1 = skip the TMA loads and
 * run the MMAs on whatever shared memory holds (tensor-pipe ceiling), 2 = skip the MMAs and only
 * stream the operands (operand-feed ceiling), 4 = int32 results are staged in shared memory but their
 * tile stores are not issued, 5 = the output stage is skipped after the accumulator reads, 0 = normal.
 * Test aid: 3 = the producer warp neither loads nor signals.  Every other warp's wait then runs out
 * (about one second), the kernel records which wait gave up in the status word, frees its TMEM and
 * returns; aiehlc_sync reports AIEHLC_ERR_DEVICE with the code (102 = the MMA issuer waited for
 * operands) and clears it, and the context stays usable.  This is how the bounded-wait exit is tested
 * without faulting or hanging the GPU. */
int aiehlc_set_debug(aiehlc_ctx* ctx, int mode);
/* Measurement aid: while `device_buffer` is non-NULL, the first CTA of every GEMM launch writes
 * clock64() stamps for each of its tiles into it, 8 int64 slots per tile: [0] MMA loop start,
 * [1] MMA loop issued, [2] epilogue starts waiting, [3] accumulator ready, [4] epilogue done;
 * tile 0 also holds [5] kernel entry, [6] kernel exit (clock64) and [7] / word 15 the global
 * nanosecond timer at entry / exit.  The buffer must hold 8 * max(2, tiles per CTA) words.  NULL switches the stamps off. */
int aiehlc_set_trace(aiehlc_ctx* ctx, long long* device_buffer);
/* Measurement aid: while `device_buffer` is non-NULL, every CTA of a CTA-pair GEMM launch writes the
 * global nanosecond timer at its entry and exit into words [2 * CTA] and [2 * CTA + 1] (the buffer
 * must hold 2 * 148 words): shows which pairs finish last.  NULL switches it off. */
int aiehlc_set_cta_times(aiehlc_ctx* ctx, long long* device_buffer);
/* Number of kernel launches this context has enqueued since creation. */
long long aiehlc_launch_count(const aiehlc_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* AIEHLC_B200_H */
