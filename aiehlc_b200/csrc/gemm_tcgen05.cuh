// Persistent, warp-specialised tile GEMM for sm_100a:  C[M][N] = A[M][K] . B[N][K]^T
//
// This is the B200 counterpart of the reference's per-tile matmul kernels
// (example/perf/aieml_perf.cc:61-83 `perf`, example/matrixmultiply/aieml_mm.cc:41-93 `mm`):
// A row-major, B stored [N][K] ("column-major B"), C row-major, exactly the
// layout of the reference's CPU golden loop (aieml_perf.cc:199-231).  Both
// operands are K-major, which is the native operand layout of tcgen05.mma.
//
//   warp 0   TMA producer   : cp.async.bulk.tensor tiles of A and B into a kStages-deep smem ring
//   warp 1   MMA issuer     : tcgen05.mma (kind::i8 -> s32, kind::f16 -> f32) into TMEM; owns TMEM
//   warps 2-5 epilogue      : tcgen05.ld the accumulator, fused output stage, global stores
//
// The accumulator is double-buffered in TMEM so the epilogue of tile i overlaps
// the K loop of tile i+1.  The whole K range (all split-K slices of the
// reference's "cascade" formulation) is accumulated in TMEM before one flush.
//
// Output stages (kEpi):
//   EPI_I32      C(int32)  = acc
//   EPI_I32_ACC  C(int32) += acc                       (stage s>0 of a multi-launch cascade)
//   EPI_I8_SRS   C(int8)   = srs(acc [+ acc_in], shift[col])   shift-round(half-even)-saturate
//   EPI_BF16     C(bf16)   = rn(acc)                    (kind::f16, fp32 accumulate)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "sm100_ptx.cuh"

namespace aiehlc {

enum : int { KIND_I8 = 0, KIND_BF16 = 1 };
enum : int { EPI_I32 = 0, EPI_I32_ACC = 1, EPI_I8_SRS = 2, EPI_BF16 = 3 };

constexpr int kBlockM = 128;        // rows of C per tile = TMEM lanes
constexpr int kBlockKBytes = 128;   // one 128B swizzle span of K per stage
constexpr int kUmmaKBytes = 32;     // K bytes consumed by one tcgen05.mma (32 x i8, 16 x bf16)
constexpr int kGemmThreads = 192;
// Results leave the epilogue through shared memory: 2 buffers of 32 rows x 128 B for each of the 4 warps.
constexpr int kStoreBufBytes = 4096;
constexpr int kStoreStagingBytes = 4 * 2 * kStoreBufBytes;

constexpr int kMaxShards = 16;

// Clock stamps and the debug modes that skip part of a kernel exist only in libraries built with
// -DAIEHLC_MEASURE; in the regular build kMeasure is a constant false and those branches are gone.
#ifdef AIEHLC_MEASURE
constexpr bool kMeasure = true;
#else
constexpr bool kMeasure = false;
#endif

struct GemmParams {
  int M, N, K;
  void* C;                 // int32 / int8 / bf16, row-major, leading dimension ldc (elements)
  long long ldc;
  const int32_t* acc_in;   // EPI_I8_SRS: optional int32 partial sums [M][ld_acc] added before srs
  long long ld_acc;
  const uint8_t* shift_vec;  // EPI_I8_SRS: optional per-output-column shift
  int shift;                 // EPI_I8_SRS: shift used when shift_vec == nullptr
  int srs_wide;              // EPI_I8_SRS: |acc| may approach 2^31: round in 64-bit arithmetic
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int group_m;             // rasterisation: tiles walk group_m row-blocks before the next column
  int vec_ok;              // C (and acc_in) rows are 16-byte aligned: vector stores allowed
  int tma_store;           // results leave through shared memory and TMA tile stores (needs vec_ok)
  int* status;             // device status word (0 = ok)
  // Tail balancing of the pair kernel along K (int8 only): the last sk_tiles tiles are cut at K block sk_cut
  // into two halves that run on different CTA pairs at different times; the upper half deposits its int32
  // partial sums in the workspace, the lower half adds them in its output stage (gemm_tcgen05_pair.cuh).
  // 0: every tile whole.
  int sk_tiles, sk_cut;
  int32_t* sk_scratch;     // [tail tile][CTA rank][32-column chunk] partial sums of the upper K half
  int* sk_flags;           // [tail tile][CTA rank] epilogue warps that have deposited; zero between launches
  // Row-sharded output (EPI_I32_ACC only): rows [g * rows_per_shard, (g + 1) * rows_per_shard) of C are
  // the dense int32 matrix shard[g] (pitch N), which may lie in the memory of another GPU; results are
  // ADDED there with system-scope reductions, one 128-byte row segment per warp instruction (measured
  // between two B200: 697 GB/s from 18 SMs on, where add-reducing tile stores of 128-byte rows need 74
  // SMs pushing at once and held the tile loads of the main loop back).  rows_per_shard is a multiple
  // of 128, so the 128 rows of a CTA never straddle two shards.  num_shards == 0: C is one matrix.
  int32_t* shard[kMaxShards];
  int rows_per_shard, num_shards;
  // The same shards as tensors (device array of num_shards maps, box 32 x 32 words), or null.  When
  // given, results leave as add-reducing TMA tile stores instead of per-row reduction instructions.
  const CUtensorMap* shard_maps;
  // Visiting order for a sharded output: consecutive tiles belong to consecutive shards, starting with
  // shard rot_first, so that the tiles in flight at any moment spread over all owners (every link busy
  // throughout, local and remote adds mixed) and GPUs that run the same product with different
  // rot_first lean on different owners.  rot_shards == 0: rows in order.
  int rot_shards, rot_first, rot_blocks_per_shard;
  // The other form of tail balancing: tiles >= nt_first_tile are cut into nt_parts column ranges
  // (narrower MMAs, no exchange between the ranges).  nt_parts == 1: off.  Never together with sk_tiles > 0.
  int nt_first_tile, nt_parts;
  // int32 products on the int8 tensor cores (see launch_mm_i32_tensor): operands are unsigned bytes and
  // the int32 result is shifted left (wrapping) before it is stored or added.
  int unsigned_ab, out_shift;
  // The caller has declared that A and B are not written by the kernel launched before this one in the
  // stream.  The warps that touch nothing but the operands and on-chip state (the TMA producer and the MMA
  // issuer) then do not wait for that kernel to drain: the first tiles are multiplied while it finishes.
  // The epilogue warps, which read and write everything else, always wait.
  int early_operands;
  long long* cta_times;    // kMeasure (pair kernel): global nanosecond timer at entry / exit of every CTA, or null
  long long* trace;        // kMeasure: per-tile clock64 stamps of CTA trace_cta (8 slots per tile), or null
  int trace_cta;           // kMeasure: which CTA writes the stamps (environment variable AIEHLC_TRACE_CTA, default 0)
  int debug;               // test aid: 3 = the producer neither loads nor signals, so every consumer wait
                           // runs out and the kernel leaves through its bounded-wait exit;
                           // kMeasure: 1 = no TMA loads (MMA ceiling), 2 = no MMAs (feed ceiling),
                           // 4 = int32 results staged but their tile stores not issued, 5 = no output stage
};

// Shift-round-saturate, pure integer: round half to even on the dropped bits, saturate to int8.
__host__ __device__ __forceinline__ int srs_i8(int acc, int s) {
  int q = acc;
  if (s > 0) {
    q = acc >> s;  // arithmetic shift: floor
    const unsigned mask = (s >= 32) ? 0xFFFFFFFFu : ((1u << s) - 1u);
    const unsigned r = static_cast<unsigned>(acc) & mask;
    const unsigned h = 1u << (s - 1);
    if (r > h || (r == h && (q & 1))) q += 1;
  }
  return q > 127 ? 127 : (q < -128 ? -128 : q);
}


// The same rounding without branches, for the epilogue's inner loop:
//   q = (acc + (2^(s-1) - 1) + bit_s(acc)) >> s        (s >= 1;  q = acc for s = 0)
// bit_s(acc) is the parity of floor(acc / 2^s), so an exact half rounds to the even neighbour.
// `hm1` = 2^(s-1) - 1 (0 for s = 0), `bmask` = 1 (0 for s = 0).  The 32-bit form needs
// |acc| + 2^s < 2^31, which the host checks from K (|acc| <= K * 2^14); otherwise kWide.
template <bool kWide>
__device__ __forceinline__ int srs_round(int acc, int s, int hm1, int bmask) {
  if constexpr (kWide) {
    const long long t = static_cast<long long>(acc) + hm1 + ((acc >> s) & bmask);
    return static_cast<int>(t >> s);
  } else {
    return (acc + hm1 + ((acc >> s) & bmask)) >> s;
  }
}
// Saturate four 32-bit values to int8 and pack them, e0 in the low byte.
__device__ __forceinline__ uint32_t pack_sat_s8x4(int e0, int e1, int e2, int e3) {
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(e3), "r"(e2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(e1), "r"(e0), "r"(hi));
  return out;
}

template <int kBN>
struct GemmSmem {
  static constexpr int kABytes = kBlockM * kBlockKBytes;
  static constexpr int kBBytes = kBN * kBlockKBytes;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBudget = 227 * 1024 - 2048 - kStoreStagingBytes;  // barriers, alignment, store staging
  static constexpr int kStagesRaw = kBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kBarBytes = 512;
  static constexpr int kTotal = kStages * kStageBytes + kStoreStagingBytes + kBarBytes + 1024;
};

__host__ __device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& mb, int& nb) {
  if (p.rot_shards > 0) {
    // consecutive tiles (the ones in flight together) belong to consecutive shards; inside a shard the
    // usual walk over groups of group_m row-blocks
    const int shard = (t + p.rot_first) % p.rot_shards;
    const int j = t / p.rot_shards;
    const int per_group = p.group_m * p.num_n_blocks;
    const int g = j / per_group;
    const int r = j - g * per_group;
    mb = shard * p.rot_blocks_per_shard + g * p.group_m + r % p.group_m;
    nb = r / p.group_m;
    return;
  }
  const int per_group = p.group_m * p.num_n_blocks;
  const int g = t / per_group;
  const int first_m = g * p.group_m;
  const int rows = p.group_m < p.num_m_blocks - first_m ? p.group_m : p.num_m_blocks - first_m;
  const int r = t - g * per_group;
  mb = first_m + r % rows;
  nb = r / rows;
}

// Where an epilogue warp puts its results when they leave through TMA tile stores.
struct StoreCtx {
  const void* tmap;     // C as a tiled tensor, box = 32 columns x 32 rows
  uint8_t* buf[2];      // this warp's two staging buffers (1024-byte aligned)
  int which;            // buffer the current group of chunks goes to
  int chunk_in_group;   // 32-column chunks already staged in that buffer
  int lane;
  int warp_row0;        // first row of C this warp's 32 TMEM lanes map to
  int32_t* shard_row0;  // sharded output: where that row starts in the owning shard
  int rows_left;        // sharded output: M - warp_row0
};

// Row-sharded output: points the warp's reductions at the shard that owns the CTA's 128 rows.
__device__ __forceinline__ void select_shard(const GemmParams& p, int cta_row0, StoreCtx& sc) {
  if (p.num_shards == 0) return;
  int owner = cta_row0 / p.rows_per_shard;
  if (owner >= p.num_shards) owner = p.num_shards - 1;  // rows past M: masked by rows_left
  sc.rows_left = p.M - sc.warp_row0;                    // rows of this warp's 32 that exist
  sc.shard_row0 = p.shard[owner] + static_cast<long long>(sc.warp_row0 - owner * p.rows_per_shard) * p.N;
  if (p.shard_maps != nullptr) {
    sc.tmap = p.shard_maps + owner;                     // rows past the shard's extent are clipped by the hardware
    sc.warp_row0 -= owner * p.rows_per_shard;
  }
}

// Adds one 32-column chunk of this warp's 32 rows into the shard.  Every thread holds one row; the
// chunk is turned through the warp's staging buffer so that each reduction instruction covers the 32
// consecutive words of ONE row (a single 128-byte request on the way to the owner).
__device__ __forceinline__ void shard_add_chunk(const GemmParams& p, StoreCtx& sc, const uint32_t* words, int col0) {
  uint8_t* buf = sc.buf[0];
  const int swz = sc.lane & 7;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<uint4*>(buf + sc.lane * 128 + ((j ^ swz) << 4)) =
        make_uint4(words[4 * j], words[4 * j + 1], words[4 * j + 2], words[4 * j + 3]);
  __syncwarp();
  const bool col_ok = col0 + sc.lane < p.N;
  int32_t* dst = sc.shard_row0 + col0 + sc.lane;
  const int rows = sc.rows_left < 32 ? sc.rows_left : 32;
#pragma unroll 4
  for (int r = 0; r < rows; ++r) {
    const int v = *reinterpret_cast<const int*>(buf + r * 128 + ((((sc.lane >> 2) ^ (r & 7)) << 4) | ((sc.lane & 3) << 2)));
    if (col_ok) asm volatile("red.relaxed.sys.global.add.s32 [%0], %1;" ::"l"(dst + static_cast<long long>(r) * p.N), "r"(v) : "memory");
  }
  __syncwarp();  // the buffer is rewritten by the next chunk
}

// Stages one 32-column chunk of this warp's 32 rows; once a group of chunks fills a row of
// kGroupBytes (128 B, or the whole tile width if that is less) one tile store (or add-reduction)
// writes the group.  Each thread writes its own row in 16-byte pieces whose position is
// XOR-swizzled with the row number exactly as the tensor map's swizzle mode expects, which also
// spreads the rows over the shared-memory banks.  The hardware clips rows >= M and columns >= N.
template <int kGroupBytes, int kPieceBytes, bool kReduceAdd>
__device__ __forceinline__ void tma_emit(StoreCtx& sc, const uint32_t* words, int col0, bool issue = true) {
  constexpr int kPerGroup = kGroupBytes / kPieceBytes;
  constexpr int kPieces = kPieceBytes / 16;
  const int k = sc.chunk_in_group;
  uint8_t* buf = sc.buf[sc.which];
  if (k == 0) {
    // the store issued from this buffer (two groups ago, or the last one where the warp has one buffer) has read it
    if (sc.lane == 0) {
      if (sc.buf[0] == sc.buf[1]) tma_store_wait_read<0>();
      else tma_store_wait_read<1>();
    }
    __syncwarp();
  }
  const int swz = kGroupBytes == 128 ? (sc.lane & 7) : kGroupBytes == 64 ? ((sc.lane >> 1) & 3) : ((sc.lane >> 2) & 1);
#pragma unroll
  for (int j = 0; j < kPieces; ++j)
    *reinterpret_cast<uint4*>(buf + sc.lane * kGroupBytes + (((k * kPieces + j) ^ swz) << 4)) =
        make_uint4(words[4 * j], words[4 * j + 1], words[4 * j + 2], words[4 * j + 3]);
  if (k == kPerGroup - 1) {
    fence_proxy_async_smem();
    __syncwarp();
    if (sc.lane == 0 && issue) {
      const int group_col0 = col0 - k * 32;
      if constexpr (kReduceAdd) tma_reduce_add_2d(sc.tmap, smem_u32(buf), group_col0, sc.warp_row0);
      else tma_store_2d(sc.tmap, smem_u32(buf), group_col0, sc.warp_row0);
      tma_store_commit();
    }
    sc.which ^= 1;
    sc.chunk_in_group = 0;
  } else {
    sc.chunk_in_group = k + 1;
  }
}

// Bytes of one staged row: 128, or the tile width in bytes where that is less.
template <int kEpi, int kBN>
struct StoreGroup {
  static constexpr int kElem = kEpi == EPI_I8_SRS ? 1 : (kEpi == EPI_BF16 ? 2 : 4);
  static constexpr int kBytes = kBN * kElem < 128 ? kBN * kElem : 128;
  static constexpr int kCols = kBytes / kElem;
};

// Output stage for 32 consecutive accumulator columns of one row.  Direct stores: the caller has
// checked row < M and col0 < N.  TMA stores (p.tma_store): called by the whole warp for EVERY chunk
// of the tile in column order; rows >= M and columns >= N are staged like the others and clipped
// by the hardware.
template <int kEpi, int kBN, bool kForceDirect = false>
__device__ __forceinline__ void store_chunk(const GemmParams& p, uint32_t (&r)[32], int row, int col0, bool row_ok,
                                            StoreCtx& sc) {
  const int ncols = min(32, p.N - col0);
  if (kMeasure && p.debug == 5) return;
  if constexpr (kEpi == EPI_I32 || kEpi == EPI_I32_ACC) {
    if (p.out_shift) {
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] <<= p.out_shift;
    }
    if (kEpi == EPI_I32_ACC && p.num_shards > 0 && p.shard_maps == nullptr) {
      shard_add_chunk(p, sc, r, col0);
      return;
    }
    if (!kForceDirect && p.tma_store) {
      tma_emit<128, 128, kEpi == EPI_I32_ACC>(sc, r, col0, !(kMeasure && p.debug == 4));
      return;
    }
    int32_t* dst = static_cast<int32_t*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (p.vec_ok && ncols == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        int4 v = make_int4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        if constexpr (kEpi == EPI_I32_ACC) {
          const int4 o = *reinterpret_cast<const int4*>(dst + j);
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *reinterpret_cast<int4*>(dst + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) {
          if constexpr (kEpi == EPI_I32_ACC) dst[j] += static_cast<int32_t>(r[j]);
          else dst[j] = static_cast<int32_t>(r[j]);
        }
    }
  } else if constexpr (kEpi == EPI_I8_SRS) {
    int8_t* dst = static_cast<int8_t*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (p.acc_in != nullptr && row_ok) {
      const int32_t* ai = p.acc_in + static_cast<long long>(row) * p.ld_acc + col0;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) r[j] += static_cast<uint32_t>(ai[j]);
    }
    uint32_t packed[8];
    if (p.shift_vec == nullptr) {
      const int sh = p.shift;
      const int hm1 = sh > 0 ? (1 << (sh - 1)) - 1 : 0;
      const int bmask = sh > 0 ? 1 : 0;
      if (p.srs_wide) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          packed[j >> 2] = pack_sat_s8x4(srs_round<true>(r[j], sh, hm1, bmask), srs_round<true>(r[j + 1], sh, hm1, bmask),
                                         srs_round<true>(r[j + 2], sh, hm1, bmask), srs_round<true>(r[j + 3], sh, hm1, bmask));
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          packed[j >> 2] = pack_sat_s8x4(srs_round<false>(r[j], sh, hm1, bmask), srs_round<false>(r[j + 1], sh, hm1, bmask),
                                         srs_round<false>(r[j + 2], sh, hm1, bmask), srs_round<false>(r[j + 3], sh, hm1, bmask));
      }
    } else {
      // per-column shifts: the 32 shift bytes of this chunk are the same for every row; a whole chunk's
      // bytes come with two 16-byte loads where the vector is aligned (col0 is a multiple of 32)
      uint32_t sw[8];
      if (ncols == 32 && (reinterpret_cast<uintptr_t>(p.shift_vec) & 15) == 0) {
        const uint4 s0 = *reinterpret_cast<const uint4*>(p.shift_vec + col0);
        const uint4 s1 = *reinterpret_cast<const uint4*>(p.shift_vec + col0 + 16);
        sw[0] = s0.x; sw[1] = s0.y; sw[2] = s0.z; sw[3] = s0.w;
        sw[4] = s1.x; sw[5] = s1.y; sw[6] = s1.z; sw[7] = s1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) sw[j] = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ncols) sw[j >> 2] |= static_cast<uint32_t>(p.shift_vec[col0 + j]) << (8 * (j & 3));
      }
      int q[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int sh = static_cast<int>((sw[j >> 2] >> (8 * (j & 3))) & 0xFFu);
        const int hm1 = max(static_cast<int>((1u << sh) >> 1) - 1, 0);
        q[j] = srs_round<true>(r[j], sh, hm1, min(sh, 1));
      }
#pragma unroll
      for (int j = 0; j < 32; j += 4) packed[j >> 2] = pack_sat_s8x4(q[j], q[j + 1], q[j + 2], q[j + 3]);
    }
    if (!kForceDirect && p.tma_store) {
      tma_emit<StoreGroup<kEpi, kBN>::kBytes, 32, false>(sc, packed, col0);
      return;
    }
    if (p.vec_ok && ncols == 32) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<uint4*>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) dst[j] = static_cast<int8_t>((packed[j >> 2] >> (8 * (j & 3))) & 0xFFu);
    }
  } else {  // EPI_BF16
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    uint32_t packed[16];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
      packed[j >> 1] = *reinterpret_cast<const uint32_t*>(&h);
    }
    if (!kForceDirect && p.tma_store) {
      tma_emit<128, 64, false>(sc, packed, col0);
      return;
    }
    if (p.vec_ok && ncols == 32) {
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<uint4*>(dst + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) {
          const uint16_t bits = static_cast<uint16_t>(packed[j >> 1] >> (16 * (j & 1)));
          reinterpret_cast<uint16_t*>(dst)[j] = bits;
        }
    }
  }
}

// Drains kBN accumulator columns of this warp's 32 TMEM lanes through the output stage, 64 columns
// per step: two TMEM loads are issued back to back, then waited for once.
template <int kBN, int kEpi>
__device__ __forceinline__ void drain_accumulator(const GemmParams& p, uint32_t taddr, int row, bool row_ok,
                                                  int n0, StoreCtx& sc, int ncols = kBN) {
  static_assert(kBN % 64 == 0, "accumulator is drained 64 columns at a time");
#pragma unroll 1
  for (int c = 0; c < ncols; c += 64) {
    __syncwarp();  // lanes that skipped stores rejoin before the warp-wide TMEM loads
    uint32_t ra[32], rb[32];
    tmem_ld_32x32b_x32(taddr + c, ra);
    tmem_ld_32x32b_x32(taddr + c + 32, rb);
    tmem_ld_wait();
    if (p.tma_store || (row_ok && n0 + c < p.N)) store_chunk<kEpi, kBN>(p, ra, row, n0 + c, row_ok, sc);
    if (p.tma_store || (row_ok && n0 + c + 32 < p.N)) store_chunk<kEpi, kBN>(p, rb, row, n0 + c + 32, row_ok, sc);
  }
}

template <int kKind, int kBN, int kEpi>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using S = GemmSmem<kBN>;
  constexpr int kStages = S::kStages;
  constexpr int kBBoxRows = kBN > 128 ? 128 : kBN;     // B arrives in boxes of at most 128 rows
  constexpr int kBBoxes = kBN / kBBoxRows;
  constexpr uint32_t kTmemCols = (2 * kBN) < 32 ? 32 : 2 * kBN;  // two accumulators
  constexpr int kElemBytes = kKind == KIND_I8 ? 1 : 2;
  constexpr int kBlockKElems = kBlockKBytes / kElemBytes;
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "TMEM columns");
  static_assert(kBN % 16 == 0 && kBN >= 16 && kBN <= 256, "UMMA N");

  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte aligned bases.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* store_staging = smem + kStages * S::kStageBytes;  // 1024-byte aligned: stages are multiples of 1 KB
  uint8_t* bar_mem = store_staging + kStoreStagingBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full_bar = empty_bar + kStages;
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long entry_clock = clock64();
  const unsigned long long entry_ns = globaltimer_ns();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_base_slot), kTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_launch_dependents();
  // from here on global memory may be read and written (operands declared ready: warps 0 and 1 go ahead)
  if (!(p.early_operands && warp < 2)) pdl_wait();
  if (kMeasure && p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    p.trace[5] = entry_clock;
    p.trace[7] = static_cast<long long>(entry_ns);
  }

  const int num_tiles = p.num_m_blocks * p.num_n_blocks;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mb, nb;
        tile_coords(t, p, mb, nb);
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status,
                         ST_TIMEOUT_EMPTY);
          if (!ok) break;
          const uint32_t fb = smem_u32(&full_bar[stage]);
          if ((kMeasure && p.debug == 1) || p.debug == 3) {
            if (kMeasure && p.debug == 1) mbar_arrive(fb);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
            continue;
          }
          mbar_expect_tx(fb, S::kStageBytes);
          uint8_t* sa = smem + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kABytes;
          tma_load_2d(smem_u32(sa), &tmap_a, fb, kb * kBlockKElems, mb * kBlockM);
#pragma unroll
          for (int b = 0; b < kBBoxes; ++b)
            tma_load_2d(smem_u32(sb + b * kBBoxRows * kBlockKBytes), &tmap_b, fb,
                        kb * kBlockKElems, nb * kBN + b * kBBoxRows);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // Aborting: give copies already in flight time to land before the CTA retires.
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // bits 7 and 10: A and B are signed bytes (cleared: unsigned)
      const uint32_t idesc = make_idesc<kKind>(kBlockM, kBN) & ~(p.unsigned_ab ? ((1u << 7) | (1u << 10)) : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1, abort_flag, p.status,
                       ST_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        if (kMeasure && p.trace && blockIdx.x == 0) p.trace[it * 8 + 0] = clock64();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, ST_TIMEOUT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::kStageBytes);
          const uint32_t sb = sa + S::kABytes;
          const uint64_t adesc = make_kmajor_desc(sa, 1024, 2);
          const uint64_t bdesc = make_kmajor_desc(sb, 1024, 2);
          if (!(kMeasure && p.debug == 2)) {
#pragma unroll
            for (int k = 0; k < kBlockKBytes / kUmmaKBytes; ++k) {
              // K-step inside the swizzle span: advance the start-address field by 32 B (>>4 = 2).
              umma_ss<kKind, 1>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc,
                                (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(&empty_bar[stage]));  // frees the stage when these MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(smem_u32(&tmem_full_bar[acc]));
        if (kMeasure && p.trace && blockIdx.x == 0) p.trace[it * 8 + 1] = clock64();
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    StoreCtx sc{&tmap_c, {store_staging + (quad * 2) * kStoreBufBytes, store_staging + (quad * 2 + 1) * kStoreBufBytes},
                0, 0, lane, 0, nullptr, 0};
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mb, nb;
      tile_coords(t, p, mb, nb);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      const bool tracer = kMeasure && p.trace && blockIdx.x == 0 && warp == 2 && lane == 0;
      if (tracer) p.trace[it * 8 + 2] = clock64();
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase, abort_flag, p.status,
                     ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      if (tracer) p.trace[it * 8 + 3] = clock64();
      const int row = mb * kBlockM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBN;
      sc.warp_row0 = row - lane;
      select_shard(p, mb * kBlockM, sc);
      drain_accumulator<kBN, kEpi>(p, taddr, row, row_ok, nb * kBN, sc);
      // Accumulator drained: hand it back to the MMA issuer.
      tc_fence_before();
      __syncwarp();
      if (tracer) p.trace[it * 8 + 4] = clock64();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
    }
    if (lane == 0) tma_store_wait_all();  // tile stores in flight still read this CTA's shared memory
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, kTmemCols);
  }
  if (kMeasure && p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    p.trace[6] = clock64();
    p.trace[15] = static_cast<long long>(globaltimer_ns());
  }
}

}  // namespace aiehlc
