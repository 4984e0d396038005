// CTA-pair variant of the tile GEMM (tcgen05 cta_group::2): two CTAs on neighbouring SMs share
// one 256 x kBN output tile.
//
// Why: the single-CTA kernel is bound by the L2 -> shared-memory feed (a 128 x 256 int8 tile needs
// 96 operand bytes per clock per SM at full MMA rate).  In a pair each CTA fetches its own 128 rows
// of A and only HALF of the B tile (kBN/2 rows); the tensor cores of both SMs read both B halves
// across the pair.  The feed drops to 64 bytes per clock per SM with no byte fetched twice.
//
//   both CTAs : warp 0 fetches this CTA's A rows and its B half; the byte counts of BOTH CTAs are
//               credited to the leader's "full" barrier
//   leader    : warp 1 issues tcgen05.mma.cta_group::2 (M = 256); each CTA's TMEM receives its
//               128 rows of the accumulator; completion is signalled to both CTAs' barriers
//   both CTAs : warps 2-5 (and 6-9 where the kernel is built with two epilogue groups) drain their
//               128 accumulator rows through the fused output stage and tell the leader when the
//               accumulator buffer is free
//
// The reference's formulation is unchanged: C = A . B^T with A[M][K], B[N][K], all K slices
// accumulated in TMEM before one flush (example/perf/aieml_perf.cc:199-231; tiling.py:299-333).
#pragma once
#include "gemm_tcgen05.cuh"

namespace aiehlc {

constexpr int kPairM = 256;

// kKPer = K blocks (of 128 bytes) fetched by ONE tile load and held by one pipeline stage.  The TMA
// unit of an SM completes a tile load ("box") roughly every 280-340 cycles whatever its size up to
// at least 16 KB (measured: stages of two boxes arrive 580-680 cycles apart for 5.5 KB, 24 KB and
// 32 KB alike, three boxes 750), so with one K block per box the 512 MMA cycles of a 256 x 256
// K block are not quite covered.  With kKPer = 2 the operands are viewed as 3-D tensors
// {128 bytes, rows, K / 128 bytes} and a box {128 B, rows, 2} brings two K blocks at once.
template <int kBN, int kKPer>
struct PairSmem {
  static constexpr int kABlock = kBlockM * kBlockKBytes;           // one K block of this CTA's 128 rows of A
  static constexpr int kBBlock = (kBN / 2) * kBlockKBytes;         // one K block of this CTA's half of B
  static constexpr int kABytes = kABlock * kKPer;
  static constexpr int kBBytes = kBBlock * kKPer;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBudget = 227 * 1024 - 2048 - kStoreStagingBytes;
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kBarBytes = 512;
  static constexpr int kTotal = kStages * kStageBytes + kStoreStagingBytes + kBarBytes + 1024;
};

// One unit of work of a CTA pair: a whole tile, one K half of a tail tile, or one column range of a tail tile.
struct WorkUnit {
  int tile, kb0, kb1;   // K blocks [kb0, kb1) of the tile
  int n_part, n_parts;  // column range n_part of n_parts (1 = all kBN columns)
};

// Unit number `u` of the launch (pair p runs units p, p + pairs, p + 2 pairs, ...).
//
// Tail balancing along K (p.sk_tiles > 0): with T = full * pairs + rem tiles, full >= 1 and rem <= pairs / 2,
// the last rem tiles are cut at K block p.sk_cut into two halves, and the units are ordered
//     [upper K halves of the rem tail tiles] [pairs whole tiles] [their lower K halves] [the other whole tiles]
// Dealt round-robin over the pairs: pairs 0 .. rem-1 start with an upper half, pairs rem .. 2 rem - 1 take the
// lower half of the same tile as their SECOND unit, after a whole tile -- by then the upper half's partial sums
// have long been deposited, so the output stage of the lower half never waits for them (with both halves in the
// first round it waited 11 k cycles and held its accumulator for 24 k, which stalled the pair's third unit).
// Every pair has at most full + 1/2 tile times of work instead of full + 1.
__device__ __forceinline__ bool work_unit(int u, const GemmParams& p, int num_tiles, int num_pairs, WorkUnit& w) {
  if (p.sk_tiles > 0) {
    const int n = p.sk_tiles, first = num_tiles - n;  // the tail tiles are the last n tiles
    if (u < n) {
      w = WorkUnit{first + u, p.sk_cut, p.num_k_blocks, 0, 1};
      return true;
    }
    if (u >= num_pairs + n && u < num_pairs + 2 * n) {
      w = WorkUnit{first + (u - num_pairs - n), 0, p.sk_cut, 0, 1};
      return true;
    }
    u -= u < num_pairs + n ? n : 2 * n;
    if (u >= first) return false;
    w = WorkUnit{u, 0, p.num_k_blocks, 0, 1};
    return true;
  }
  if (p.nt_parts > 1 && u >= p.nt_first_tile) {
    const int v = u - p.nt_first_tile;
    w = WorkUnit{p.nt_first_tile + v / p.nt_parts, 0, p.num_k_blocks, v % p.nt_parts, p.nt_parts};
    return w.tile < num_tiles;
  }
  if (u >= num_tiles) return false;
  w = WorkUnit{u, 0, p.num_k_blocks, 0, 1};
  return true;
}

constexpr int kSkChunkInts = kBlockM * 32;  // one 32-column chunk of a CTA's 128 accumulator rows

// The two K halves of a tail tile meet in the output stage.  The upper half deposits its 128 x kBN int32
// partial sums per CTA in the tile's slot of the workspace and raises the slot's counter; the lower half
// waits for the counter (bounded), streams the slot through its warps' staging buffers with bulk copies
// (two 4 KB pieces in flight per warp), adds it to its own accumulator chunk by chunk and runs the
// output stage.  Integer sums: the result is the whole-tile result bit for bit.
// Layout of a deposited chunk: [warp quadrant][j = 0..7][lane][4 words], so that every store
// instruction of a warp moves 512 contiguous bytes and a warp's share of a chunk is 4 contiguous KB
// (the layout never leaves this file).
__device__ __forceinline__ void deposit_chunk(const uint32_t (&r)[32], int32_t* chunk, int quad, int lane) {
  int4* dst = reinterpret_cast<int4*>(chunk + quad * 1024) + lane;
#pragma unroll
  for (int j = 0; j < 8; ++j) dst[j * 32] = make_int4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
}
// Adds this lane's words of a chunk that a bulk copy has placed in shared memory (same layout).
__device__ __forceinline__ void add_chunk_from_smem(uint32_t (&r)[32], const uint8_t* chunk, int lane) {
  const int4* src = reinterpret_cast<const int4*>(chunk) + lane;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int4 v = src[j * 32];
    r[4 * j] += v.x; r[4 * j + 1] += v.y; r[4 * j + 2] += v.z; r[4 * j + 3] += v.w;
  }
}

// Warps of a CTA of the pair kernel: producer, MMA issuer and two groups of four epilogue warps.  A
// warp reads the 32 TMEM lanes its number modulo 4 selects, so the two warps of a lane quarter share
// a tile's rows and each takes half of its columns: twice as many accumulator reads, proxy fences and
// tile stores are in flight as with one group.
// With one group (kEpiGroups = 1) every warp drains whole rows of the tile and has two staging buffers.
constexpr int pair_threads(int epi_groups) { return 64 + epi_groups * 128; }

template <int kKind, int kBN, int kEpi, int kKPer, int kEpiGroups>
__global__ void __launch_bounds__(pair_threads(kEpiGroups), 1)
gemm_tn_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_b_narrow, const __grid_constant__ CUtensorMap tmap_c,
                    const GemmParams p) {
  using S = PairSmem<kBN, kKPer>;
  constexpr int kStages = S::kStages;
  static_assert(kStages >= 2, "pipeline needs at least two stages");
  constexpr int kBHalf = kBN / 2;
  constexpr uint32_t kTmemCols = 2 * kBN;
  constexpr int kElemBytes = kKind == KIND_I8 ? 1 : 2;
  constexpr int kBlockKElems = kBlockKBytes / kElemBytes;
  static_assert(kBN == 128 || kBN == 256, "pair tile N");
  static_assert(kEpiGroups == 1 || kEpiGroups == 2, "epilogue warp groups");
  static_assert(kEpiGroups * 4 * kStoreBufBytes <= kStoreStagingBytes, "at least one staging buffer per epilogue warp");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* store_staging = smem + kStages * S::kStageBytes;  // 1024-byte aligned: stages are multiples of 1 KB
  uint8_t* bar_mem = store_staging + kStoreStagingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);   // used in the leader CTA
  uint64_t* empty_bar = full_bar + kStages;                    // one set per CTA
  uint64_t* tmem_full_bar = empty_bar + kStages;               // one set per CTA
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;                // used in the leader CTA
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* sk_warps_done = reinterpret_cast<int*>(tmem_base_slot + 2);
  uint64_t* dep_bar = reinterpret_cast<uint64_t*>(tmem_base_slot + 4);  // two per epilogue warp quadrant (tail K halves)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = static_cast<int>(cluster_id_x());
  const int num_pairs = static_cast<int>(cluster_count_x());
  const long long entry_clock = clock64();
  const unsigned long long entry_ns = globaltimer_ns();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 8 * kEpiGroups);  // every epilogue warp of the two CTAs
    }
    for (int q = 0; q < 8; ++q) mbar_init(smem_u32(&dep_bar[q]), 1);
    *abort_flag = 0;
    *sk_warps_done = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.nt_parts > 1) tma_prefetch_desc(&tmap_b_narrow);
  }
  if (warp == 1) {
    tmem_alloc<2>(smem_u32(tmem_base_slot), kTmemCols);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  cluster_sync_all();  // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_launch_dependents();
  // from here on global memory may be read and written (operands declared ready: warps 0 and 1 go ahead)
  if (!(p.early_operands && warp < 2)) pdl_wait();
  if (kMeasure && p.trace && blockIdx.x == p.trace_cta && threadIdx.x == 0) {
    p.trace[5] = entry_clock;
    p.trace[7] = static_cast<long long>(entry_ns);
  }

  const int num_tiles = p.num_m_blocks * p.num_n_blocks;  // num_m_blocks counts 256-row blocks

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkUnit w;
      for (int u = pair_id; ok && work_unit(u, p, num_tiles, num_pairs, w); u += num_pairs) {
        int mb, nb;
        tile_coords(w.tile, p, mb, nb);
        for (int kb = w.kb0; kb < w.kb1; kb += kKPer) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY);
          if (!ok) break;
          const uint32_t fb_local = smem_u32(&full_bar[stage]);
          if ((kMeasure && p.debug == 1) || p.debug == 3) {
            if (kMeasure && p.debug == 1 && leader) mbar_arrive(fb_local);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
            continue;
          }
          // a column range of a tail tile brings kBHalf / n_parts rows of B per CTA (its own tensor map: smaller box)
          const int b_rows = kBHalf / w.n_parts;
          if (leader) mbar_expect_tx(fb_local, 2 * (S::kABytes + S::kBBytes / w.n_parts));  // both CTAs' bytes
          const uint32_t fb = mapa_u32(fb_local, 0);  // the same barrier in the leader CTA
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          const int row_a = mb * kPairM + static_cast<int>(rank) * kBlockM;
          const int row_b = nb * kBN + w.n_part * 2 * b_rows + static_cast<int>(rank) * b_rows;
          const CUtensorMap* tb = w.n_parts == 1 ? &tmap_b : &tmap_b_narrow;
          if constexpr (kKPer == 1) {
            tma_load_2d_pair(smem_u32(sa), &tmap_a, fb, kb * kBlockKElems, row_a);
            tma_load_2d_pair(smem_u32(sb), tb, fb, kb * kBlockKElems, row_b);
          } else {
            // K blocks kb .. kb + kKPer - 1 in one box each; blocks past the end of K read as zero
            tma_load_3d_pair(smem_u32(sa), &tmap_a, fb, 0, row_a, kb);
            tma_load_3d_pair(smem_u32(sb), tb, fb, 0, row_b, kb);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      WorkUnit w;
      for (int u = pair_id; ok && work_unit(u, p, num_tiles, num_pairs, w); u += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status,
                       ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        if (kMeasure && p.trace && blockIdx.x == p.trace_cta) p.trace[it * 8 + 0] = clock64();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        const uint32_t idesc = make_idesc<kKind>(kPairM, kBN / w.n_parts) &
                               ~(p.unsigned_ab ? ((1u << 7) | (1u << 10)) : 0u);  // bits 7, 10: signed A, B
        const uint32_t b_block = S::kBBlock / w.n_parts;  // the K blocks of a box lie back to back
        for (int kb = w.kb0; kb < w.kb1; kb += kKPer) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, ST_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          if (!(kMeasure && p.debug == 2)) {
#pragma unroll
            for (int kk = 0; kk < kKPer; ++kk) {
              if (kb + kk >= w.kb1) break;  // K blocks of this stage beyond the range: loaded, not multiplied
              const uint64_t adesc = make_kmajor_desc(sa + kk * S::kABlock, 1024, 2);
              const uint64_t bdesc = make_kmajor_desc(sb + kk * b_block, 1024, 2);
#pragma unroll
              for (int k = 0; k < kBlockKBytes / kUmmaKBytes; ++k)
                umma_ss<kKind, 2>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc,
                                  (kb + kk > w.kb0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit_pair_mask(smem_u32(&empty_bar[stage]), 3);  // frees the stage in both CTAs
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair_mask(smem_u32(&tmem_full_bar[acc]), 3);
        if (kMeasure && p.trace && blockIdx.x == p.trace_cta) p.trace[it * 8 + 1] = clock64();
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int quad = warp & 3;
    const int group = (warp - 2) >> 2;
    // one staging buffer per warp with two groups (the tile stores of the other group overlap the refill)
    uint8_t* stage0 = store_staging + (kEpiGroups == 1 ? quad * 2 : warp - 2) * kStoreBufBytes;
    StoreCtx sc{&tmap_c, {stage0, kEpiGroups == 1 ? stage0 + kStoreBufBytes : stage0}, 0, 0, lane, 0, nullptr, 0};
    int it = 0;
    bool ok = true;
    WorkUnit w;
    for (int u = pair_id; ok && work_unit(u, p, num_tiles, num_pairs, w); u += num_pairs, ++it) {
      int mb, nb;
      tile_coords(w.tile, p, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const bool tracer = kMeasure && p.trace && blockIdx.x == p.trace_cta && warp == 2 && lane == 0;
      if (tracer) p.trace[it * 8 + 2] = clock64();
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      if (tracer) p.trace[it * 8 + 3] = clock64();
      const int lane_row = quad * 32 + lane;
      const int row = mb * kPairM + static_cast<int>(rank) * kBlockM + lane_row;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBN;
      sc.warp_row0 = row - lane;
      select_shard(p, mb * kPairM + static_cast<int>(rank) * kBlockM, sc);
      if (w.kb0 == 0 && w.kb1 == p.num_k_blocks) {
        const int ncols = kBN / w.n_parts;
        const int n0 = nb * kBN + w.n_part * ncols;
        // each group takes half of the columns where a half is whole 64-column drain steps and whole store groups
        constexpr int kGran = StoreGroup<kEpi, kBN>::kCols > 64 ? StoreGroup<kEpi, kBN>::kCols : 64;
        const int share = ncols / kEpiGroups;
        if (share % kGran == 0)
          drain_accumulator<kBN, kEpi>(p, taddr + group * share, row, row_ok, n0 + group * share, sc, share);
        else if (group == 0)
          drain_accumulator<kBN, kEpi>(p, taddr, row, row_ok, n0, sc, ncols);
      } else if (group == 0) {
        // one K half of a tail tile; workspace slots and counters are per tail tile and CTA rank
        constexpr int kChunks = kBN / 32;
        constexpr long long kCtaInts = static_cast<long long>(kChunks) * kSkChunkInts;
        const int slot_id = (w.tile - (num_tiles - p.sk_tiles)) * 2 + static_cast<int>(rank);
        int32_t* slot = p.sk_scratch + slot_id * kCtaInts;
        if (w.kb0 > 0) {
          // upper half: hand the partial sums over and go on
#pragma unroll 1
          for (int c = 0; c < kChunks; c += 2) {
            uint32_t ra[32], rb[32];
            tmem_ld_32x32b_x32(taddr + c * 32, ra);
            tmem_ld_32x32b_x32(taddr + c * 32 + 32, rb);
            tmem_ld_wait();
            deposit_chunk(ra, slot + c * kSkChunkInts, quad, lane);
            deposit_chunk(rb, slot + (c + 1) * kSkChunkInts, quad, lane);
          }
          fence_proxy_async_global();  // the other side reads the slot with bulk copies
          __syncwarp();
          if (lane == 0) red_release_gpu_add(p.sk_flags + slot_id, 1);  // one arrival per epilogue warp
        } else {
          // lower half: owns the tile's output stage.  The slot arrives through this warp's two staging
          // buffers (with two epilogue groups: its own and that of the idle warp of the other group).
          // kLand pieces in flight: both staging buffers of the warp (with two epilogue groups a warp has one)
          constexpr int kLand = kEpiGroups == 1 ? 2 : 1;
          uint8_t* land[2] = {stage0, stage0 + kStoreBufBytes};
          const uint32_t bar[2] = {smem_u32(&dep_bar[quad * 2]), smem_u32(&dep_bar[quad * 2 + 1])};
          const int32_t* src = slot + quad * 1024;
          if (lane == 0) {
            tma_store_wait_read<0>();   // tile stores of an earlier unit have read the staging buffers
            const long long t0 = clock64();
            while (ok && ld_acquire_gpu(p.sk_flags + slot_id) < 4) {   // the upper half's four epilogue warps
              if (*abort_flag) ok = false;
              else if (clock64() - t0 > kWaitLimitCycles) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, ST_TIMEOUT_PEER);
                ok = false;
              }
            }
            if (ok) {
              fence_proxy_async_global();
              fence_proxy_async_smem();
#pragma unroll
              for (int b = 0; b < kLand; ++b) {
                mbar_expect_tx(bar[b], 4096);
                bulk_load_g2s(smem_u32(land[b]), src + b * kSkChunkInts, 4096, bar[b]);
              }
            }
          }
          ok = __all_sync(0xFFFFFFFFu, ok);
          if (tracer) p.trace[it * 8 + 6] = clock64();
#pragma unroll 1
          for (int c = 0; ok && c < kChunks; ++c) {
            const int b = c % kLand;
            __syncwarp();
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c * 32, r);
            ok = mbar_wait(bar[b], (c / kLand) & 1, abort_flag, p.status, ST_TIMEOUT_PEER);
            ok = __all_sync(0xFFFFFFFFu, ok);
            tmem_ld_wait();
            if (!ok) break;
            add_chunk_from_smem(r, land[b], lane);
            __syncwarp();   // every lane has read the buffer before it is refilled
            if (lane == 0 && c + kLand < kChunks) {
              fence_proxy_async_smem();
              mbar_expect_tx(bar[b], 4096);
              bulk_load_g2s(smem_u32(land[b]), src + (c + kLand) * kSkChunkInts, 4096, bar[b]);
            }
            // the staging buffers are taken: per-thread stores
            const int col0 = nb * kBN + c * 32;
            if (row_ok && col0 < p.N) store_chunk<kEpi, kBN, true>(p, r, row, col0, row_ok, sc);
          }
          if (ok) {
            // The last of the four warps to finish puts the counter back to zero for the next launch (by
            // then every warp is past its wait).  No blocking barrier among the four: a warp that gave up
            // on its wait must not be able to strand the others.
            __syncwarp();
            if (lane == 0 && atomicAdd(sk_warps_done, 1) == 3) {
              *sk_warps_done = 0;
              p.sk_flags[slot_id] = 0;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (tracer) p.trace[it * 8 + 4] = clock64();
      if (lane == 0) mbar_arrive_remote(smem_u32(&tmem_empty_bar[acc]), 0);
    }
    if (lane == 0) tma_store_wait_all();  // tile stores in flight still read this CTA's shared memory
  }

  // Neither CTA may retire (or free TMEM) while its partner can still read its shared memory,
  // write its TMEM or signal its barriers.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, kTmemCols);
  }
  if (kMeasure && p.trace && blockIdx.x == p.trace_cta && threadIdx.x == 0) {
    p.trace[6] = clock64();
    p.trace[15] = static_cast<long long>(globaltimer_ns());
  }
  if (kMeasure && p.cta_times && threadIdx.x == 0) {
    p.cta_times[2 * blockIdx.x] = static_cast<long long>(entry_ns);
    p.cta_times[2 * blockIdx.x + 1] = static_cast<long long>(globaltimer_ns());
  }
}

}  // namespace aiehlc
