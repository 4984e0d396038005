// Host side of the tcgen05 tile GEMM: tensor-map construction, tile-shape choice, launch.
#include <cstdio>
#include <cstdlib>

#include "context.h"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_pair.cuh"

namespace aiehlc {

namespace {

int encode_kmajor_map(aiehlc_ctx* ctx, CUtensorMap* map, int kind, const void* base, long long rows,
                      long long k, long long ld_elems, int box_rows) {
  const int esize = kind == KIND_I8 ? 1 : 2;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld_elems) * esize};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockKBytes / esize),
                             static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = ctx->encode(
      map, kind == KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
      const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[160];
    snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled failed (CUresult %d) rows=%lld k=%lld ld=%lld",
             static_cast<int>(r), rows, k, ld_elems);
    return fail(AIEHLC_ERR_CUDA, msg);
  }
  return AIEHLC_OK;
}

// Tile choice: fewest "tile-time units" over whole waves of persistent CTAs (or CTA pairs).
// A narrow tile fetches more operand bytes per MMA and the kernels are bound by the shared-memory
// feed, hence the efficiency factors (measured on int8 4096^3: N = 256 / 128 / 64 tiles take
// 56.8 / 82.0 / 143.9 us).  A CTA pair does the work of two single-CTA tiles with two thirds of
// the operand traffic per SM (measured on int8 8192^3: 373 us against 391 us).
}  // namespace

// The same K-major operand as a 3-D tensor {128 bytes, rows, K / 128 bytes}: a box then spans
// `k_blocks` consecutive 128-byte K blocks of `box_rows` rows.  Needs K * element size to be a
// multiple of 128 bytes (a partial last block would otherwise spill into the next row).
int encode_kmajor_map_3d(aiehlc_ctx* ctx, CUtensorMap* map, int kind, const void* base, long long rows, long long k,
                         long long ld_elems, int box_rows, int k_blocks) {
  const int esize = kind == KIND_I8 ? 1 : 2;
  const cuuint64_t inner = kBlockKBytes / esize;
  const cuuint64_t dims[3] = {inner, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(k * esize / kBlockKBytes)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld_elems) * esize, kBlockKBytes};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(inner), static_cast<cuuint32_t>(box_rows),
                             static_cast<cuuint32_t>(k_blocks)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = ctx->encode(
      map, kind == KIND_I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
      const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[160];
    snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled (3-D) failed (CUresult %d) rows=%lld k=%lld ld=%lld",
             static_cast<int>(r), rows, k, ld_elems);
    return fail(AIEHLC_ERR_CUDA, msg);
  }
  return AIEHLC_OK;
}

// C as a tiled tensor for the epilogue's tile stores: box of 32 rows x one staged row (128 bytes,
// or the tile width where that is less), swizzle mode matching the staged row width.
int encode_c_map(aiehlc_ctx* ctx, CUtensorMap* map, int epi, int bn, void* base, long long rows, long long cols,
                 long long ld) {
  const int esize = epi == EPI_I8_SRS ? 1 : (epi == EPI_BF16 ? 2 : 4);
  const int group_bytes = bn * esize < 128 ? bn * esize : 128;
  const CUtensorMapDataType dt = epi == EPI_I8_SRS ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : epi == EPI_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_INT32;
  const CUtensorMapSwizzle sw = group_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : group_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * esize};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(group_bytes / esize), 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = ctx->encode(map, dt, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                 CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(AIEHLC_ERR_CUDA, "cuTensorMapEncodeTiled failed for the output tensor");
  return AIEHLC_OK;
}

// Tail balancing of a CTA-pair launch along K (int8).  With `slots` pairs, tiles = full * slots + rem tiles
// take full + 1 waves of which the last keeps only rem pairs busy.  When rem <= slots / 2 the rem tail tiles
// are cut into two K halves that run side by side in the first round, on 2 rem pairs, while the other pairs
// start on whole tiles; after that every pair has `full` whole tiles left, so no pair has more than
// full + 1/2 tile times of work.  The upper half leaves its partial sums in a workspace; the lower half
// owns the output stage and adds them while its pair is already multiplying its next tile.  Needs one full
// wave (so that there is a next tile) and a K of at least 16 blocks (halves of >= 8).  Returns the number
// of tail tiles cut (0: none) and the K block where they are cut.
//   mode 1: wherever that applies;  else: never.
int split_k_tail(int tiles, int slots, int k_blocks, int mode, int* cut_at) {
  if (cut_at) *cut_at = 0;
  if (mode != 1 || slots <= 0 || k_blocks < 16) return 0;
  const int full = tiles / slots, rem = tiles % slots;
  if (full < 1 || rem == 0 || rem * 2 > slots) return 0;
  if (cut_at) *cut_at = (k_blocks / 2 + 1) & ~1;  // an even number of K blocks in the lower half
  return rem;
}

// Whether the CTA-pair kernel fetches two 128-byte K blocks with one tile load: K must be a whole
// number of blocks (the 3-D tensor map has no partial last block) and there must be enough of them.
static bool wide_k_loads(const aiehlc_ctx* ctx, int esize, int K) {
  const long long kbytes = static_cast<long long>(K) * esize;
  return ctx->k_per_load != 1 && kbytes % kBlockKBytes == 0 && kbytes >= 4 * kBlockKBytes;
}

// The other cure for a thin last wave: its tiles are cut into two column ranges (half as wide MMAs, no
// exchange between the ranges).  Only for 256-column pair tiles, whose halves are still full-rate MMAs.
void narrow_tail(int tiles, int slots, int tile_n, int enabled, int* first, int* parts) {
  *first = tiles;
  *parts = 1;
  if ((enabled != 2 && enabled != 3) || slots <= 0 || tile_n != 256) return;
  const int rem = tiles % slots;
  if (rem == 0 || rem * 2 > slots) return;
  *first = tiles - rem;
  *parts = 2;
}

// The planner: B200 counterpart of the compiler's matmul tiling (tilinglinalg::creatematmul,
// src/mlir/mlirfront/tilinglinalg/tilinglinalg.cpp:38-146: grid of tiles + per-tile block) and of
// its data-pattern analysis (tilingpass.cpp:98-150: which operand is broadcast along which grid
// dimension).  launch_gemm() executes exactly the plan this function returns.
int plan_gemm(const aiehlc_ctx* ctx, int kind, int M, int N, int K, aiehlc_gemm_plan* out) {
  const int cand[3] = {256, 128, 64};
  const double eff[3] = {1.0, 0.60, 0.35};
  const int sms = ctx->usable_sms();
  const int esize = kind == KIND_I8 ? 1 : 2;
  aiehlc_gemm_plan best{};
  double best_cost = -1;
  for (int pr = 0; pr < 2; ++pr) {
    if (pr == 1 && ctx->pair_mode == 0) continue;                  // pairs switched off
    // pairs forced where they apply (more than one row-block, and not the 64-wide tile they lack)
    if (pr == 0 && ctx->pair_mode == 1 && M > kBlockM && ctx->force_tile_n != 64) continue;
    for (int i = 0; i < 3; ++i) {
      const int bn = cand[i];
      if (ctx->force_tile_n && bn != ctx->force_tile_n) continue;
      if (pr == 1 && (bn == 64 || sms < 2)) continue;
      const int tm = pr ? kPairM : kBlockM;
      aiehlc_gemm_plan pl{};
      pl.tile_m = tm;
      pl.tile_n = bn;
      pl.tile_k_bytes = kBlockKBytes;
      pl.cta_pair = pr;
      pl.grid_m = (M + tm - 1) / tm;
      pl.grid_n = (N + bn - 1) / bn;
      pl.tiles = static_cast<long long>(pl.grid_m) * pl.grid_n;
      pl.slots = pr ? sms / 2 : sms;
      pl.waves = static_cast<int>((pl.tiles + pl.slots - 1) / pl.slots);
      pl.wave_efficiency = static_cast<double>(pl.tiles) / (static_cast<double>(pl.waves) * pl.slots);
      // rows of the last row-block that fall outside M are computed all the same
      double waves = pl.waves;
      {
        const int kb = static_cast<int>((static_cast<long long>(K) * esize + kBlockKBytes - 1) / kBlockKBytes);
        const int mode = pr ? ctx->split_tail : 0;
        int first = 0, parts = 1;
        if (kind == KIND_I8 && split_k_tail(static_cast<int>(pl.tiles), pl.slots, kb, mode, nullptr) > 0) {
          // the tail tiles run as K halves: half a wave (plus the meeting of the partial sums)
          waves = pl.waves - 0.5 + 0.04;
        } else {
          // a thin last wave of 256-column pair tiles runs as 128-column ranges: measured 0.87 of a whole tile's time
          narrow_tail(static_cast<int>(pl.tiles), pl.slots, bn, mode, &first, &parts);
          if (parts > 1) waves -= 0.13;
        }
      }
      // Pairs halve the B traffic per SM, which pays once tiles follow one another; a single wave of 256-column
      // tiles runs 5-14 % faster on single CTAs (measured: 2048^3 10.7 against 11.5 us, 1536 x 3072 x 4096 15.6
      // against 17.3), two waves run alike, 4096^3 (3.5 waves) 46.6 against 52.7 us for the pairs.
      const double pair_factor = !pr ? 1.0 : (pl.waves == 1 && bn == 256 ? 1.06 : 0.97);
      pl.cost_units = waves * bn / eff[i] * pair_factor;
      if (best_cost < 0 || pl.cost_units < best_cost) { best_cost = pl.cost_units; best = pl; }
    }
  }
  if (best_cost < 0) return fail(AIEHLC_ERR_INVALID, "plan_gemm: no tile shape satisfies the forced settings");
  const int k_per = best.cta_pair && wide_k_loads(ctx, esize, K) ? 2 : 1;
  best.tile_k_bytes = kBlockKBytes * k_per;
  const int stage_bytes = (best.cta_pair ? kBlockM * kBlockKBytes + best.tile_n / 2 * kBlockKBytes
                                         : kBlockM * kBlockKBytes + best.tile_n * kBlockKBytes) * k_per;
  int stages = (227 * 1024 - 2048 - kStoreStagingBytes) / stage_bytes;
  if (stages > 8) stages = 8;
  best.stages = stages;
  best.smem_bytes = stages * stage_bytes + kStoreStagingBytes + 512 + 1024;
  best.tmem_columns = 2 * best.tile_n < 32 ? 32 : 2 * best.tile_n;
  best.k_blocks = static_cast<int>((static_cast<long long>(K) * esize + kBlockKBytes - 1) / kBlockKBytes);
  int g = ctx->group_m > 0 ? ctx->group_m : (best.cta_pair ? 8 : 16);
  if (g > best.grid_m) g = best.grid_m;
  best.group_m = g;
  // every tile of a grid row reads the same rows of A, every tile of a grid column the same rows of B
  best.a_shared_by = best.grid_n;
  best.b_shared_by = best.grid_m;
  const long long wave_cols = (best.slots + g - 1) / g;
  best.wave_footprint_bytes = (static_cast<long long>(g) * best.tile_m +
                               (wave_cols < best.grid_n ? wave_cols : best.grid_n) * best.tile_n) *
                              static_cast<long long>(K) * esize;
  int first = 0, parts = 1;
  const int mode = best.cta_pair ? ctx->split_tail : 0;
  best.split_k_tiles = kind == KIND_I8 ? split_k_tail(static_cast<int>(best.tiles), best.slots, best.k_blocks, mode, &best.split_k_at) : 0;
  best.narrow_tail_tiles = 0;
  if (best.split_k_tiles == 0) {
    narrow_tail(static_cast<int>(best.tiles), best.slots, best.tile_n, mode, &first, &parts);
    best.narrow_tail_tiles = parts > 1 ? static_cast<int>(best.tiles) - first : 0;
  }
  *out = best;
  return AIEHLC_OK;
}

namespace {

// Shard-interleaved visiting order: possible when every shard is full and holds a whole number of
// row-block groups (otherwise the rows are visited in order, which is still correct).
void set_shard_rotation(GemmParams& p, const GemmCall& c, int tile_m) {
  p.rot_shards = 0;
  if (c.num_shards < 2 || c.rows_per_shard % tile_m != 0) return;
  const int bps = c.rows_per_shard / tile_m;
  if (static_cast<long long>(c.num_shards) * c.rows_per_shard != c.M || p.group_m <= 0 || bps % p.group_m != 0) return;
  p.rot_shards = c.num_shards;
  p.rot_first = ((c.first_shard % c.num_shards) + c.num_shards) % c.num_shards;
  p.rot_blocks_per_shard = bps;
}

// With `slots` persistent CTAs (or pairs) a slot runs tiles slot, slot + slots, ...; its tiles cycle
// through all shards only if slots and the number of shards have no common factor.  Otherwise some
// slots would send everything to one remote owner while others only add locally.
int coprime_slots(int slots, int shards) {
  auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
  while (slots > 1 && gcd(slots, shards) != 1) --slots;
  return slots;
}

template <int kKind, int kBN, int kEpi>
int launch_one(aiehlc_ctx* ctx, const GemmCall& c, cudaStream_t st) {
  using S = GemmSmem<kBN>;
  CUtensorMap ma, mb;
  int rc = encode_kmajor_map(ctx, &ma, kKind, c.A, c.M, c.K, c.lda, kBlockM);
  if (rc) return rc;
  rc = encode_kmajor_map(ctx, &mb, kKind, c.B, c.N, c.K, c.ldb, kBN > 128 ? 128 : kBN);
  if (rc) return rc;

  const int esize = kKind == KIND_I8 ? 1 : 2;
  const int cesize = kEpi == EPI_I8_SRS ? 1 : (kEpi == EPI_BF16 ? 2 : 4);
  GemmParams p{};
  p.M = c.M; p.N = c.N; p.K = c.K;
  p.C = c.C; p.ldc = c.ldc;
  p.acc_in = c.acc_in; p.ld_acc = c.ld_acc;
  p.shift_vec = c.shift_vec; p.shift = c.shift;
  // 32-bit rounding needs |acc| + 2^shift < 2^31; |acc| <= K * 2^14 unless partial sums are added
  p.srs_wide = (c.acc_in != nullptr || c.K > 32768 || c.shift > 29) ? 1 : 0;
  p.num_m_blocks = (c.M + kBlockM - 1) / kBlockM;
  p.num_n_blocks = (c.N + kBN - 1) / kBN;
  p.num_k_blocks = static_cast<int>((static_cast<long long>(c.K) * esize + kBlockKBytes - 1) / kBlockKBytes);
  p.group_m = c.group_m;
  p.unsigned_ab = c.unsigned_ab; p.out_shift = c.out_shift;
  p.early_operands = (ctx->operands_ready && ctx->pdl && !c.operands_from_kernel) ? 1 : 0;
  // 32 consecutive outputs per thread are written with 16-byte stores when every row start is aligned.
  bool vec = (reinterpret_cast<uintptr_t>(c.C) % 16 == 0) && ((c.ldc * cesize) % 16 == 0);
  p.vec_ok = vec ? 1 : 0;
  // int8 results are 32 contiguous bytes per thread and chunk (whole sectors) and that epilogue is
  // bound by its integer arithmetic: per-thread stores are faster there unless tile stores are forced (2)
  p.tma_store = (vec && (ctx->tma_store == 2 || (ctx->tma_store == 1 && kEpi != EPI_I8_SRS))) ? 1 : 0;
  CUtensorMap mc = ma;  // unused unless tma_store
  if (c.num_shards > 0) {
    p.vec_ok = 1; p.tma_store = 1;  // the whole warp takes part in every chunk (the shards were checked by the caller)
    for (int g = 0; g < c.num_shards; ++g) p.shard[g] = c.shards[g];
    p.rows_per_shard = c.rows_per_shard; p.num_shards = c.num_shards;
    p.shard_maps = c.shard_maps;
    set_shard_rotation(p, c, kBlockM);
  } else if (p.tma_store && (rc = encode_c_map(ctx, &mc, kEpi, kBN, c.C, c.M, c.N, c.ldc))) return rc;
  p.status = ctx->d_status;
  p.debug = ctx->debug_mode;
  p.trace = ctx->trace;
  p.cta_times = ctx->cta_times;

  auto kern = gemm_tn_kernel<kKind, kBN, kEpi>;
  KernelSetup& ks = ctx->kernel_setup[reinterpret_cast<const void*>(kern)];
  if (int rc2 = ensure_dynamic_smem(ctx->device, reinterpret_cast<const void*>(kern), S::kTotal, &ks.smem_attr)) return rc2;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  int grid = tiles < ctx->usable_sms() ? tiles : ctx->usable_sms();
  if (p.rot_shards > 0) grid = coprime_slots(grid, p.rot_shards);
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  AIEHLC_CUDA(cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, p));
  ctx->launches++;
  return AIEHLC_OK;
}


// CTA-pair kernel: a 1-D grid of 2-CTA clusters, one cluster per 256 x kBN tile in flight.
template <int kKind, int kBN, int kEpi, int kKPer, int kEpiGroups>
int launch_pair(aiehlc_ctx* ctx, const GemmCall& c, cudaStream_t st) {
  using S = PairSmem<kBN, kKPer>;
  CUtensorMap ma, mb, mb_narrow;
  int rc;
  if (kKPer == 1) {
    rc = encode_kmajor_map(ctx, &ma, kKind, c.A, c.M, c.K, c.lda, kBlockM);
    if (rc) return rc;
    rc = encode_kmajor_map(ctx, &mb, kKind, c.B, c.N, c.K, c.ldb, kBN / 2);
    if (rc) return rc;
  } else {
    rc = encode_kmajor_map_3d(ctx, &ma, kKind, c.A, c.M, c.K, c.lda, kBlockM, kKPer);
    if (rc) return rc;
    rc = encode_kmajor_map_3d(ctx, &mb, kKind, c.B, c.N, c.K, c.ldb, kBN / 2, kKPer);
    if (rc) return rc;
  }
  mb_narrow = mb;  // replaced below when tail tiles are cut into column ranges

  const int esize = kKind == KIND_I8 ? 1 : 2;
  const int cesize = kEpi == EPI_I8_SRS ? 1 : (kEpi == EPI_BF16 ? 2 : 4);
  GemmParams p{};
  p.M = c.M; p.N = c.N; p.K = c.K;
  p.C = c.C; p.ldc = c.ldc;
  p.acc_in = c.acc_in; p.ld_acc = c.ld_acc;
  p.shift_vec = c.shift_vec; p.shift = c.shift;
  // 32-bit rounding needs |acc| + 2^shift < 2^31; |acc| <= K * 2^14 unless partial sums are added
  p.srs_wide = (c.acc_in != nullptr || c.K > 32768 || c.shift > 29) ? 1 : 0;
  p.num_m_blocks = (c.M + kPairM - 1) / kPairM;
  p.num_n_blocks = (c.N + kBN - 1) / kBN;
  p.num_k_blocks = static_cast<int>((static_cast<long long>(c.K) * esize + kBlockKBytes - 1) / kBlockKBytes);
  p.group_m = c.group_m;
  p.unsigned_ab = c.unsigned_ab; p.out_shift = c.out_shift;
  p.early_operands = (ctx->operands_ready && ctx->pdl && !c.operands_from_kernel) ? 1 : 0;
  p.vec_ok = ((reinterpret_cast<uintptr_t>(c.C) % 16 == 0) && ((c.ldc * cesize) % 16 == 0)) ? 1 : 0;
  p.tma_store = (p.vec_ok && (ctx->tma_store == 2 || (ctx->tma_store == 1 && kEpi != EPI_I8_SRS))) ? 1 : 0;
  CUtensorMap mc = ma;  // unused unless tma_store
  if (c.num_shards > 0) {
    p.vec_ok = 1; p.tma_store = 1;  // the whole warp takes part in every chunk (the shards were checked by the caller)
    for (int g = 0; g < c.num_shards; ++g) p.shard[g] = c.shards[g];
    p.rows_per_shard = c.rows_per_shard; p.num_shards = c.num_shards;
    p.shard_maps = c.shard_maps;
    set_shard_rotation(p, c, kPairM);
  } else if (p.tma_store && (rc = encode_c_map(ctx, &mc, kEpi, kBN, c.C, c.M, c.N, c.ldc))) return rc;
  p.status = ctx->d_status;
  p.debug = ctx->debug_mode;
  p.trace = ctx->trace;
  p.cta_times = ctx->cta_times;
#ifdef AIEHLC_MEASURE
  if (const char* e = getenv("AIEHLC_TRACE_CTA")) p.trace_cta = atoi(e);
#endif

  auto kern = gemm_tn_pair_kernel<kKind, kBN, kEpi, kKPer, kEpiGroups>;
  KernelSetup& ks = ctx->kernel_setup[reinterpret_cast<const void*>(kern)];
  if (int rc2 = ensure_dynamic_smem(ctx->device, reinterpret_cast<const void*>(kern), S::kTotal, &ks.smem_attr)) return rc2;
  const int tiles = p.num_m_blocks * p.num_n_blocks;
  int max_pairs = ctx->sm_count / 2;
  const int pair_limit = ctx->usable_sms() / 2 > 0 ? ctx->usable_sms() / 2 : 1;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(pair_threads(kEpiGroups));
  cfg.dynamicSmemBytes = S::kTotal;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 2 : 1;
  if (ks.max_clusters == 0) {
    // every cluster of the persistent grid must be resident at once
    cfg.gridDim = dim3(2 * max_pairs);
    int active = 0;
    const int na = cfg.numAttrs;
    cfg.numAttrs = 1;  // the cluster shape is what matters for occupancy
    if (cudaOccupancyMaxActiveClusters(&active, kern, &cfg) == cudaSuccess && active > 0)
      ks.max_clusters = active < max_pairs ? active : max_pairs;
    else {
      cudaGetLastError();
      ks.max_clusters = max_pairs;
    }
    cfg.numAttrs = na;
  }
  max_pairs = ks.max_clusters < pair_limit ? ks.max_clusters : pair_limit;
  int pairs = tiles < max_pairs ? tiles : max_pairs;
  // Tail tiles as K halves (int32 accumulation only: sums of partial sums are exact, fp32 would change
  // rounding; the lower half runs the plain output stage: not into a sharded output)
  p.sk_tiles = 0;
  p.sk_cut = 0;
  if (kKind == KIND_I8 && c.num_shards == 0 && tiles >= max_pairs) {
    p.sk_tiles = split_k_tail(tiles, max_pairs, p.num_k_blocks, ctx->split_tail, &p.sk_cut);
    if (p.sk_tiles > 0) {
      // one slot and one counter per tail tile and CTA rank
      const size_t cta_ints = static_cast<size_t>(kBN / 32) * kSkChunkInts;
      const size_t scratch_bytes = static_cast<size_t>(p.sk_tiles) * 2 * cta_ints * sizeof(int32_t);
      const size_t flag_bytes = static_cast<size_t>(p.sk_tiles) * 2 * sizeof(int);
      if (ctx->sk_scratch.reserve(scratch_bytes)) return AIEHLC_ERR_NOMEM;
      if (flag_bytes > ctx->sk_flags.bytes) {
        if (ctx->sk_flags.reserve(flag_bytes)) return AIEHLC_ERR_NOMEM;
        AIEHLC_CUDA(cudaMemset(ctx->sk_flags.ptr, 0, ctx->sk_flags.bytes));  // counters start at zero
      }
      p.sk_scratch = static_cast<int32_t*>(ctx->sk_scratch.ptr);
      p.sk_flags = static_cast<int*>(ctx->sk_flags.ptr);
      pairs = max_pairs;  // at least one full wave: every pair has work
    }
  }
  p.nt_first_tile = tiles;
  p.nt_parts = 1;
  if (p.sk_tiles == 0) {
    narrow_tail(tiles, tiles < max_pairs ? max_pairs : pairs, kBN, ctx->split_tail, &p.nt_first_tile, &p.nt_parts);
    if (p.nt_parts > 1) {
      rc = kKPer == 1 ? encode_kmajor_map(ctx, &mb_narrow, kKind, c.B, c.N, c.K, c.ldb, kBN / 2 / p.nt_parts)
                      : encode_kmajor_map_3d(ctx, &mb_narrow, kKind, c.B, c.N, c.K, c.ldb, kBN / 2 / p.nt_parts, kKPer);
      if (rc) return rc;
      const int units = p.nt_first_tile + (tiles - p.nt_first_tile) * p.nt_parts;
      pairs = units < max_pairs ? units : max_pairs;
    }
  }
  if (p.rot_shards > 0) pairs = coprime_slots(pairs, p.rot_shards);
  cfg.gridDim = dim3(2 * pairs);
  AIEHLC_CUDA(cudaLaunchKernelEx(&cfg, kern, ma, mb, mb_narrow, mc, p));
  ctx->launches++;
  return AIEHLC_OK;
}

template <int kKind, int kEpi>
int dispatch_bn(aiehlc_ctx* ctx, const GemmCall& c, int bn, bool pair, cudaStream_t st) {
  if (pair) {
    // two K blocks per tile load when K is a whole number of 128-byte blocks (and there are enough of them)
    const bool wide = wide_k_loads(ctx, kKind == KIND_I8 ? 1 : 2, c.K);
    // Two groups of epilogue warps pay where the output stage, not the MMAs, sets a tile's pace: measured
    // 10-18 % faster up to 8 K blocks for int8 (int32 or srs results) and up to 4 for bf16 (half the result
    // bytes per tile), equal to 5 % slower from twice that depth on.  A row-sharded output is bound by the
    // wire to the other GPUs, not by the output stage: one group, as measured.
    const long long k_bytes = static_cast<long long>(c.K) * (kKind == KIND_I8 ? 1 : 2);
    const long long two_groups_up_to = (kKind == KIND_I8 ? 8 : 4) * kBlockKBytes;
    const int groups = ctx->epi_groups ? ctx->epi_groups : (k_bytes <= two_groups_up_to && c.num_shards == 0 ? 2 : 1);
    if (groups == 1) {
      if (bn == 256) return wide ? launch_pair<kKind, 256, kEpi, 2, 1>(ctx, c, st) : launch_pair<kKind, 256, kEpi, 1, 1>(ctx, c, st);
      return wide ? launch_pair<kKind, 128, kEpi, 2, 1>(ctx, c, st) : launch_pair<kKind, 128, kEpi, 1, 1>(ctx, c, st);
    }
    if (bn == 256) return wide ? launch_pair<kKind, 256, kEpi, 2, 2>(ctx, c, st) : launch_pair<kKind, 256, kEpi, 1, 2>(ctx, c, st);
    return wide ? launch_pair<kKind, 128, kEpi, 2, 2>(ctx, c, st) : launch_pair<kKind, 128, kEpi, 1, 2>(ctx, c, st);
  }
  switch (bn) {
    case 256: return launch_one<kKind, 256, kEpi>(ctx, c, st);
    case 128: return launch_one<kKind, 128, kEpi>(ctx, c, st);
    default: return launch_one<kKind, 64, kEpi>(ctx, c, st);
  }
}

}  // namespace

// The order in which a launch visits its tiles, computed by the very function the kernels call:
// tile t is (row_block[t], col_block[t]); with `slots` persistent CTAs (or pairs) slot s runs tiles
// s, s + slots, ...  Returns the number of tiles, or a negative error.
int tile_order(const aiehlc_ctx* ctx, int kind, int M, int N, int K, int num_shards, int rows_per_shard, int first_shard,
               int* row_block, int* col_block, int capacity, int* slots_out) {
  aiehlc_gemm_plan plan{};
  if (int rc = plan_gemm(ctx, kind, M, N, K, &plan)) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.num_m_blocks = plan.grid_m; p.num_n_blocks = plan.grid_n; p.group_m = plan.group_m;
  int slots = static_cast<int>(plan.tiles < plan.slots ? plan.tiles : plan.slots);
  if (num_shards > 0) {
    GemmCall c{};
    c.M = M; c.num_shards = num_shards; c.rows_per_shard = rows_per_shard; c.first_shard = first_shard;
    set_shard_rotation(p, c, plan.tile_m);
    if (p.rot_shards > 0) slots = coprime_slots(slots, p.rot_shards);
  }
  if (slots_out) *slots_out = slots;
  if (plan.tiles > capacity) return fail(AIEHLC_ERR_INVALID, "tile_order: the output arrays are too short");
  for (int t = 0; t < static_cast<int>(plan.tiles); ++t) tile_coords(t, p, row_block[t], col_block[t]);
  return static_cast<int>(plan.tiles);
}

int launch_gemm(aiehlc_ctx* ctx, const GemmCall& call, cudaStream_t st) {
  GemmCall c = call;
  if (c.M <= 0 || c.N <= 0 || c.K <= 0) return fail(AIEHLC_ERR_INVALID, "gemm: M, N, K must be positive");
  const int esize = c.kind == KIND_I8 ? 1 : 2;

  // TMA wants 16-byte aligned bases and row pitches.  Operands that do not comply are first
  // copied to a pitched workspace (the K tail beyond the true extent is never read: the
  // tensor map keeps K as its inner extent and the hardware zero-fills past it).
  auto needs_pack = [&](const void* ptr, long long ld) {
    return reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || (ld * esize) % 16 != 0;
  };
  if (needs_pack(c.A, c.lda)) {
    const long long ld = (static_cast<long long>(c.K) * esize + 15) / 16 * 16 / esize;
    if (ctx->pack_a.reserve(static_cast<size_t>(c.M) * ld * esize)) return AIEHLC_ERR_NOMEM;
    int rc = launch_repack(ctx, c.A, ctx->pack_a.ptr, c.M, c.K, c.lda, ld, esize, st);
    if (rc) return rc;
    c.A = ctx->pack_a.ptr; c.lda = ld;
    c.operands_from_kernel = 1;
  }
  if (needs_pack(c.B, c.ldb)) {
    const long long ld = (static_cast<long long>(c.K) * esize + 15) / 16 * 16 / esize;
    if (ctx->pack_b.reserve(static_cast<size_t>(c.N) * ld * esize)) return AIEHLC_ERR_NOMEM;
    int rc = launch_repack(ctx, c.B, ctx->pack_b.ptr, c.N, c.K, c.ldb, ld, esize, st);
    if (rc) return rc;
    c.B = ctx->pack_b.ptr; c.ldb = ld;
    c.operands_from_kernel = 1;
  }

  aiehlc_gemm_plan plan{};
  if (int rc = plan_gemm(ctx, c.kind, c.M, c.N, c.K, &plan)) return rc;
  c.group_m = plan.group_m;
  const int bn = plan.tile_n;
  const bool pair = plan.cta_pair != 0;
  if (c.kind == KIND_I8) {
    switch (c.epi) {
      case EPI_I32: return dispatch_bn<KIND_I8, EPI_I32>(ctx, c, bn, pair, st);
      case EPI_I32_ACC: return dispatch_bn<KIND_I8, EPI_I32_ACC>(ctx, c, bn, pair, st);
      case EPI_I8_SRS: return dispatch_bn<KIND_I8, EPI_I8_SRS>(ctx, c, bn, pair, st);
      default: return fail(AIEHLC_ERR_INVALID, "gemm: bad output stage for int8");
    }
  }
  if (c.epi != EPI_BF16) return fail(AIEHLC_ERR_INVALID, "gemm: bad output stage for bf16");
  return dispatch_bn<KIND_BF16, EPI_BF16>(ctx, c, bn, pair, st);
}

}  // namespace aiehlc
