// int8 conv2d (NHWC x HWIO, stride 1, "same" zero padding) as an implicit GEMM on tcgen05,
// with the per-output-channel shift-round-saturate stage fused into the epilogue.
//
//   GEMM view:  M = n*h*w output pixels, N = cout, K = kh*kw*cin in (kh, kw, ci) order.
//   A tile   :  for one filter tap (kh,kw) the 128 x cin operand is simply the input image
//               shifted by the tap offset, so one 4-D TMA box {cin, Wt, R, 1} fetches it and the
//               hardware's out-of-bounds zero fill *is* the padding -- no im2col buffer exists.
//   B tile   :  the weights re-laid once per call as [tap][cout][cin] (K-major) by a small
//               pre-pass, then fetched by 2-D TMA boxes.
//
// One CTA computes one output tile of R image rows x Wt columns (R*Wt <= 128 = TMEM lanes) for
// up to 256 output channels.  The reference has no convolution; the kernel follows the tiling
// vocabulary of its matmul path (K loop, accumulate, flush once: tiling.py:299-333).
#include <cstdio>
#include <mutex>
#include <string>

#include "context.h"
#include "gemm_tcgen05.cuh"

namespace aiehlc {

constexpr int kConvMaxStages = 12;
constexpr int kConvThreads = 192;
constexpr int kConvPersistentThreads = 320;   // producer, MMA issuer, two groups of four epilogue warps

struct ConvParams {
  int n, h, w, cin, cout, kh, kw, pad;
  int wt, rows_per_tile;           // output tile: rows_per_tile image rows x wt columns
  int tiles_w, tiles_h;            // tiles per image
  int chunk;                       // K bytes per stage (cin chunk): 32, 64 or 128
  int chunks_per_tap;              // cin / chunk
  int cout_tile;                   // N of the MMA (multiple of 16, <= 256)
  int stages, stage_bytes, a_bytes;
  uint32_t tx_bytes;               // bytes one stage's two TMA boxes deliver
  // Halo form (halo != 0): ONE activation box per cin chunk brings the whole input patch of the tile,
  // (rows_per_tile + kh - 1) image rows of row_w = wt + kw - 1 pixels, and ONE weight box brings that
  // chunk of every tap.  The GEMM's M index runs over the patch rows (m = r * row_w + c, the kw - 1
  // extra columns per row are computed and dropped), so the A operand of tap (fh, fw) is the same
  // patch read from (fh * row_w + fw) rows further on: nine descriptors into one tile instead of
  // nine tiles.  Two boxes per CTA and chunk instead of 2 * kh * kw.
  int halo;
  int row_w;                       // pixels per M row group: wt + kw - 1 (halo) or wt
  uint32_t w_block_bytes;          // halo: one tap's cout_tile x chunk block inside the weight box
  // Patch form on weights as the caller holds them (HWIO: [tap][cin][cout], output channels contiguous):
  // the weight box is {cout_tile, cin chunk, taps}, i.e. rows of cout_tile bytes, one per input channel,
  // which is the tensor core's N-major ("MN-major") operand layout with a swizzle span of cout_tile bytes
  // (32, 64 or 128).  No re-layout pass, no second launch.
  int w_n_major;
  uint32_t b_swizzle_code, b_sbo_bytes, b_kstep;  // B descriptor: swizzle, 8-row group pitch, start step (>>4) per MMA
  // Patch form with one cin chunk: the weights arrive as one box per FILTER ROW, each on its own barrier,
  // so the first row's taps are multiplied while the other rows are still on their way (the TMA unit
  // needs about 4 cycles per box row; the weight rows are most of a CTA's load time).
  int w_split;
  uint32_t w_row_bytes;            // bytes of one filter row's box: kw taps
  // Patch form, wide N: the kw taps of a filter row become ONE MMA with N = kw * cout_tile (the taps' weight
  // blocks lie side by side in shared memory), so a CTA issues kh * cin / 32 instructions instead of
  // kh * kw * cin / 32 (an option kept from the time each small MMA cost the issuing thread ~200 cycles; with
  // the unrolled issue loops it is no faster, and its output stage is heavier).  Tap fw's product of patch
  // row m belongs to output row m - fw: the epilogue adds column block fw of row m + fw to block 0 of row m
  // (neighbouring lanes by shuffle, the first rows of the next warp through shared memory).
  int wide_n;
  uint32_t b_lbo_bytes;            // N-major weights: distance between the taps' column blocks
  uint32_t swizzle_code, sbo_bytes;
  uint32_t tmem_cols;
  // Persistent form (many tiles per SM: batches): a CTA keeps its channel tile's weights -- every tap -- in
  // shared memory for its whole life and walks spatial tiles blockIdx.x, blockIdx.x + gridDim.x, ...; input
  // patches arrive through a ring of `stages` buffers and the accumulator is double-buffered, so the loads,
  // the MMAs and the output stage of consecutive tiles overlap.  Patch form with one cin chunk only.
  int persistent;
  int spatial_tiles;               // n * tiles_h * tiles_w
  uint32_t w_region_bytes;         // shared memory reserved for the weights (multiple of 1 KB)
  uint32_t acc_stride;             // TMEM columns between accumulators
  int mma_group;                   // tiles whose MMAs are issued interleaved (1, 2 or 4): 2 * mma_group accumulators in TMEM
  int srs_wide;                    // |acc| + 2^shift may reach 2^31: round in 64-bit arithmetic
  // tile index -> (image, tile row, tile column) without dividing: floor(2^32 / d) + 1 for d = tiles_w and
  // tiles_h, exact while index * d < 2^32; 0 where that cannot be promised (the kernels divide then)
  uint32_t magic_w, magic_h;
  int8_t* y;
  const uint8_t* shift_vec;
  int* status;
  long long* trace;   // kMeasure: clock64 stamps of CTA 0, or null
};

// n / d for 0 <= n, d >= 1 with the host's multiplier (ConvParams::magic_w): a division by a run-time number costs
// the thread that does it several hundred cycles, and in a 4 us kernel the first tile load waits for it.
__device__ __forceinline__ int fast_div(int n, int d, uint32_t magic) {
  if (d == 1) return n;
  return magic != 0u ? static_cast<int>(__umulhi(static_cast<uint32_t>(n), magic)) : n / d;
}

// How an epilogue warp rounds: decided once per CTA from the channel tile's shifts.
struct SrsPlan {
  int mode;                 // 0: one shift for every channel, 32-bit; 1: per channel, 32-bit; 2: per channel, 64-bit
  int sh, half, mask;       // mode 0: the shift, 2^(shift-1) - 1 and 1 (0 and 0 for shift 0), kept in registers
};
// 32-bit rounding needs |acc| + 2^shift < 2^31: `acc_wide` says whether |acc| <= taps * cin * 2^14 can pass 2^30,
// the shifts are read here.
__device__ __forceinline__ SrsPlan srs_plan(const uint8_t* shift_smem, int cout_tile, bool acc_wide) {
  int max_shift = 0, min_shift = 255;
  for (int c = 0; c < cout_tile; ++c) {
    const int sh = static_cast<int>(shift_smem[c]);
    max_shift = max(max_shift, sh);
    min_shift = min(min_shift, sh);
  }
  SrsPlan pl;
  const bool wide = acc_wide || max_shift > 29;
  pl.mode = wide ? 2 : (min_shift == max_shift ? 0 : 1);
  pl.sh = max_shift;
  pl.half = max_shift > 0 ? static_cast<int>((1u << (max_shift - 1)) - 1u) : 0;
  pl.mask = min(max_shift, 1);
  return pl;
}
// 32 accumulator columns of one output pixel -> srs -> int8 -> global memory.  `shifts` and `halves` point at the
// chunk's first channel (halves[c] = 2^(shift-1) - 1, 0 for shift 0).
__device__ __forceinline__ void conv_store_chunk(const uint32_t (&v)[32], const SrsPlan& pl, const uint8_t* shifts,
                                                 const int* halves, int8_t* dst, int ncols, bool vec) {
  int q[32];
  if (pl.mode == 0) {
#pragma unroll
    for (int j = 0; j < 32; ++j) q[j] = srs_round<false>(static_cast<int>(v[j]), pl.sh, pl.half, pl.mask);
  } else if (pl.mode == 1) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int sh = static_cast<int>(shifts[j]);
      q[j] = srs_round<false>(static_cast<int>(v[j]), sh, halves[j], min(sh, 1));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int sh = static_cast<int>(shifts[j]);
      q[j] = srs_round<true>(static_cast<int>(v[j]), sh, halves[j], min(sh, 1));
    }
  }
  uint32_t packed[8];
#pragma unroll
  for (int j = 0; j < 32; j += 4) packed[j >> 2] = pack_sat_s8x4(q[j], q[j + 1], q[j + 2], q[j + 3]);
  if (vec && ncols == 32) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) dst[j] = static_cast<int8_t>((packed[j >> 2] >> (8 * (j & 3))) & 0xFFu);
  }
}

// The MMAs of one tile in the patch form: for every tap and K step one MMA, the operand descriptors given as
// their 32-bit halves (only the address field moves, and never past its 14 bits: every operand lies below
// 256 KB).  KH, KW, KS > 0 fix the filter and the K steps per tap at compile time, so the loops unroll and the
// offsets are a few multiples of row_step: the one issuing thread, which spends ~10 cycles on every dependent
// instruction of its own, is left with an add and the MMA per product (measured on the 3 x 3 x 64 layer:
// ~75 cycles per MMA instead of ~220 with 64-bit descriptor sums inside counted loops).
// `w_row_bar` != nullptr: the weights of filter row fh arrive on their own barrier, waited for here.
template <int KH, int KW, int KS>
__device__ __forceinline__ bool conv_issue_tile(uint32_t d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t idesc, uint32_t accum, int kh, int kw, int ksteps,
                                                uint32_t row_step, uint32_t px_step, uint32_t w_step, uint32_t b_kstep,
                                                uint64_t* w_row_bar, volatile int* abort_flag, int* status) {
  const int nh = KH > 0 ? KH : kh, nw = KW > 0 ? KW : kw, nk = KS > 0 ? KS : ksteps;
#pragma unroll
  for (int fh = 0; fh < nh; ++fh) {
    if (w_row_bar != nullptr) {
      if (!mbar_wait(smem_u32(&w_row_bar[fh]), 0, abort_flag, status, ST_TIMEOUT_FULL)) return false;
      tc_fence_after();
    }
#pragma unroll
    for (int fw = 0; fw < nw; ++fw) {
#pragma unroll
      for (int k = 0; k < nk; ++k) {
        umma_ss_i8_halves(d, a_lo + fh * row_step + fw * px_step + 2 * k, a_hi,
                          b_lo + (fh * nw + fw) * w_step + k * b_kstep, b_hi, idesc, accum);
        accum = 1u;
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(kConvThreads, 1)
conv2d_i8_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* bar_mem = smem + p.stages * p.stage_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);
  uint64_t* empty_bar = full_bar + kConvMaxStages;
  uint64_t* tmem_full_bar = empty_bar + kConvMaxStages;
  uint64_t* w_row_bar = tmem_full_bar + 1;           // one per filter row (w_split)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(w_row_bar + kConvMaxStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  uint8_t* shift_smem = reinterpret_cast<uint8_t*>(tmem_base_slot + 2);  // this CTA's cout_tile shift bytes (<= 256)
  // wide N: rows 0 .. kw-2 of every warp's column blocks 1 .. kw-1, for the warp before it (behind the barriers' 1 KB)
  uint32_t* xchg = reinterpret_cast<uint32_t*>(bar_mem + 1024);
  int* half_smem = reinterpret_cast<int*>(bar_mem + 1024 + 8192);   // 2^(shift-1) - 1 per channel (0 for shift 0)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long entry_clock = clock64();
  const bool tracing = kMeasure && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(tmem_full_bar), 1);
    for (int r = 0; r < kConvMaxStages; ++r) mbar_init(smem_u32(&w_row_bar[r]), 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_base_slot), p.tmem_cols);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_launch_dependents();
  pdl_wait();  // the weight pre-pass before this kernel has completed; global memory may be touched
  if (tracing && threadIdx.x == 0) {
    p.trace[0] = entry_clock;
    p.trace[1] = clock64();
  }
  // the epilogue warps fetch the per-channel shifts once; they are needed only after the main loop
  SrsPlan plan{};
  if (warp >= 2) {
    const int i = threadIdx.x - 64;
    for (int c = i; c < 256; c += 128) {
      const int col = blockIdx.y * p.cout_tile + c;
      const int sh = (c < p.cout_tile && col < p.cout) ? p.shift_vec[col] : 0;
      shift_smem[c] = static_cast<uint8_t>(sh);
      half_smem[c] = sh > 0 ? static_cast<int>((1u << (sh - 1)) - 1u) : 0;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
    plan = srs_plan(shift_smem, p.cout_tile, p.srs_wide != 0);   // while the loads and the MMAs run
  }

  // tile -> (image, first output row, first output column, first output channel)
  const int t_row = fast_div(blockIdx.x, p.tiles_w, p.magic_w);
  const int tw = static_cast<int>(blockIdx.x) - t_row * p.tiles_w;
  const int img = fast_div(t_row, p.tiles_h, p.magic_h);
  const int th = t_row - img * p.tiles_h;
  const int oh0 = th * p.rows_per_tile;
  const int ow0 = tw * p.wt;
  const int co0 = blockIdx.y * p.cout_tile;
  const int taps = p.kh * p.kw;
  const int num_kb = p.halo ? p.chunks_per_tap : taps * p.chunks_per_tap;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY);
        if (!ok) break;
        const uint32_t fb = smem_u32(&full_bar[stage]);
        uint8_t* sa = smem + stage * p.stage_bytes;
        uint8_t* sb = sa + p.a_bytes;
        if (p.halo && p.w_split) {
          // one chunk, one stage: the patch on the stage's barrier, each filter row's weights on its own
          mbar_expect_tx(fb, p.tx_bytes - p.kh * p.w_row_bytes);
          tma_load_4d(smem_u32(sa), &tmap_x, fb, 0, ow0 - p.pad, oh0 - p.pad, img);
          for (int fh = 0; fh < p.kh; ++fh) {
            const uint32_t wb = smem_u32(&w_row_bar[fh]);
            mbar_expect_tx(wb, p.w_row_bytes);
            const uint32_t dst = smem_u32(sb + fh * p.w_row_bytes);
            if (p.w_n_major) tma_load_3d(dst, &tmap_w, wb, co0, 0, fh * p.kw);
            else tma_load_3d(dst, &tmap_w, wb, 0, co0, fh * p.kw);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
          continue;
        }
        mbar_expect_tx(fb, p.tx_bytes);
        if (p.halo) {
          // the whole patch (zero-filled outside the image: that is the padding) and every tap's weights
          tma_load_4d(smem_u32(sa), &tmap_x, fb, kb * p.chunk, ow0 - p.pad, oh0 - p.pad, img);
          if (p.w_n_major) tma_load_3d(smem_u32(sb), &tmap_w, fb, co0, kb * p.chunk, 0);   // {cout, cin, tap}
          else tma_load_3d(smem_u32(sb), &tmap_w, fb, kb * p.chunk, co0, 0);                 // {cin, cout, tap}
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
          continue;
        }
        const int tap = kb / p.chunks_per_tap;
        const int c0 = (kb - tap * p.chunks_per_tap) * p.chunk;
        const int fh = tap / p.kw, fw = tap - fh * p.kw;
        // Innermost coordinate (channel) is a multiple of the chunk size, hence 16-byte aligned;
        // the spatial coordinates may be negative or past the edge: those elements read as zero.
        tma_load_4d(smem_u32(sa), &tmap_x, fb, c0, ow0 + fw - p.pad, oh0 + fh - p.pad, img);
        tma_load_2d(smem_u32(sb), &tmap_w, fb, c0, tap * p.cout + co0);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // bit 16: B is N-major (rows of output channels, one per input channel) instead of K-major
      const uint32_t idesc = make_idesc<KIND_I8>(kBlockM, p.wide_n ? p.kw * p.cout_tile : p.cout_tile) |
                             (p.w_n_major ? (1u << 16) : 0u);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, ST_TIMEOUT_FULL);
        if (!ok) break;
        tc_fence_after();
        if (tracing && kb == 0) p.trace[2] = clock64();
        if (tracing && kb < 12) p.trace[8 + kb] = clock64();
        const uint32_t sa = smem_u32(smem + stage * p.stage_bytes);
        const uint32_t sb = sa + p.a_bytes;
        if (p.halo) {
          // Tap (fh, fw) reads the patch from (fh * row_w + fw) rows further on.  The descriptor's start
          // address simply moves by that many rows: TMA laid the swizzle pattern down as a function of
          // the absolute shared-memory address and the tensor core applies it to the addresses it
          // computes, so a start that is not on an 8-row pattern boundary needs nothing else (the
          // descriptor's base-offset field stays 0; setting it to the start's phase gives wrong data).
          // One thread issues everything; see conv_issue_tile for what that costs and why the common filters
          // are unrolled.  (Also measured: consecutive taps into different accumulators, and M = 64 instead of
          // 128: no faster.)
          const uint64_t a0 = make_kmajor_desc(sa, p.sbo_bytes, p.swizzle_code);
          uint64_t bd = make_kmajor_desc(sb, p.b_sbo_bytes, p.b_swizzle_code);
          const uint32_t px_step = static_cast<uint32_t>(p.chunk) >> 4;
          const uint32_t row_step = px_step * p.row_w, w_step = p.w_block_bytes >> 4;
          const int ksteps = p.chunk / kUmmaKBytes;
          uint32_t accum = kb != 0 ? 1u : 0u;
          if (!p.wide_n) {
            const uint32_t a_lo = static_cast<uint32_t>(a0), a_hi = static_cast<uint32_t>(a0 >> 32);
            const uint32_t b_lo = static_cast<uint32_t>(bd), b_hi = static_cast<uint32_t>(bd >> 32);
            const uint32_t bk = static_cast<uint32_t>(p.b_kstep);
            uint64_t* rows = p.w_split ? w_row_bar : nullptr;
            if (p.kh == 3 && p.kw == 3 && ksteps == 2)
              ok = conv_issue_tile<3, 3, 2>(tmem_base, a_lo, a_hi, b_lo, b_hi, idesc, accum, 3, 3, 2, row_step, px_step,
                                            w_step, bk, rows, abort_flag, p.status);
            else if (p.kh == 3 && p.kw == 3 && ksteps == 1)
              ok = conv_issue_tile<3, 3, 1>(tmem_base, a_lo, a_hi, b_lo, b_hi, idesc, accum, 3, 3, 1, row_step, px_step,
                                            w_step, bk, rows, abort_flag, p.status);
            else if (p.kh == 3 && p.kw == 3 && ksteps == 4)
              ok = conv_issue_tile<3, 3, 4>(tmem_base, a_lo, a_hi, b_lo, b_hi, idesc, accum, 3, 3, 4, row_step, px_step,
                                            w_step, bk, rows, abort_flag, p.status);
            else
              ok = conv_issue_tile<0, 0, 0>(tmem_base, a_lo, a_hi, b_lo, b_hi, idesc, accum, p.kh, p.kw, ksteps, row_step,
                                            px_step, w_step, bk, rows, abort_flag, p.status);
          } else {
            // all kw taps of a filter row at once: B = their kw column blocks (K-major weights: kw * cout_tile
            // consecutive rows; N-major weights: blocks b_lbo_bytes apart, which the descriptor's
            // leading-dimension field states)
            for (int fh = 0; fh < p.kh; ++fh) {
              if (p.w_split) {
                ok = mbar_wait(smem_u32(&w_row_bar[fh]), 0, abort_flag, p.status, ST_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
              }
              const uint64_t ad = a0 + fh * row_step;
              uint64_t bw = bd;
              if (p.w_n_major) bw = (bw & ~(0x3FFFull << 16)) | (static_cast<uint64_t>(p.b_lbo_bytes >> 4) << 16);
#pragma unroll 4
              for (int k = 0; k < ksteps; ++k) {
                umma_ss<KIND_I8, 1>(tmem_base, ad + 2 * k, bw + k * p.b_kstep, idesc, accum);
                accum = 1u;
              }
              bd += w_step * p.kw;
            }
          }
        } else {
          const uint64_t adesc = make_kmajor_desc(sa, p.sbo_bytes, p.swizzle_code);
          const uint64_t bdesc = make_kmajor_desc(sb, p.sbo_bytes, p.swizzle_code);
          for (int k = 0; k < p.chunk / kUmmaKBytes; ++k)
            umma_ss<KIND_I8, 1>(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        if (!ok) break;
        umma_commit(smem_u32(&empty_bar[stage]));
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (ok) umma_commit(smem_u32(tmem_full_bar));
      if (tracing) p.trace[3] = clock64();
    }
  } else {
    const int quad = warp & 3;
    bool ok = mbar_wait(smem_u32(tmem_full_bar), 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    ok = __all_sync(0xFFFFFFFFu, ok);
    if (ok) {
      tc_fence_after();
      if (tracing && warp == 2 && lane == 0) p.trace[4] = clock64();
      const int m = quad * 32 + lane;
      const int mr = m / p.row_w, mc = m - mr * p.row_w;   // image row and column inside the tile
      const int oh = oh0 + mr, ow = ow0 + mc;
      const bool pix_ok = mr < p.rows_per_tile && mc < p.wt && oh < p.h && ow < p.w;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      int8_t* yrow = p.y + ((static_cast<long long>(img) * p.h + oh) * p.w + ow) * p.cout;
      const bool vec = (reinterpret_cast<uintptr_t>(p.y) % 16 == 0) && (p.cout % 16 == 0);
      if (!p.wide_n) {
        // 64 columns per round, both loads in flight at once
        for (int c = 0; c < p.cout_tile; c += 64) {
          __syncwarp();
          uint32_t v[2][32];
          const bool second = c + 32 < p.cout_tile;
          tmem_ld_32x32b_x32(taddr + c, v[0]);
          if (second) tmem_ld_32x32b_x32(taddr + c + 32, v[1]);
          tmem_ld_wait();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int cc = c + hh * 32, col0 = co0 + cc;
            if ((hh == 1 && !second) || !pix_ok || col0 >= p.cout) continue;
            conv_store_chunk(v[hh], plan, shift_smem + cc, half_smem + cc, yrow + col0,
                             min(32, min(p.cout_tile - cc, p.cout - col0)), vec);
          }
        }
      } else {
        for (int c = 0; c < p.cout_tile; c += 32) {
          __syncwarp();
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          // out[m] = sum_fw D_fw[m + fw]: column block fw of the row fw lanes further on
          for (int fw = 1; fw < p.kw; ++fw) {
            uint32_t t[32];
            tmem_ld_32x32b_x32(taddr + fw * p.cout_tile + c, t);
            tmem_ld_wait();
            // the first fw rows of this warp are what the last fw lanes of the warp before need
            if (lane < fw && quad > 0) {
              uint32_t* dst = xchg + ((quad * 4 + fw) * 4 + lane) * 32;
#pragma unroll
              for (int j = 0; j < 32; ++j) dst[j] = t[j];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const bool from_next = lane + fw >= 32;
            const uint32_t* src = xchg + (((quad + 1) * 4 + fw) * 4 + (lane + fw - 32)) * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const uint32_t v = __shfl_down_sync(0xFFFFFFFFu, t[j], fw);
              r[j] += (from_next && quad < 3) ? src[j] : (from_next ? 0u : v);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");   // before the next round overwrites the exchange rows
          }
          const int col0 = co0 + c;
          if (!pix_ok || col0 >= p.cout) continue;
          conv_store_chunk(r, plan, shift_smem + c, half_smem + c, yrow + col0,
                           min(32, min(p.cout_tile - c, p.cout - col0)), vec);
        }
      }
    }
  }

  if (tracing && warp == 2 && lane == 0) p.trace[5] = clock64();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, p.tmem_cols);
  }
  if (tracing && threadIdx.x == 0) p.trace[6] = clock64();
}

// The MMAs of one group of up to four tiles (persistent form), tile j into accumulator d[j]: for every tap and
// K step one MMA per tile.  KH, KW, KS > 0 fix the filter and the K steps per tap at compile time: the loops
// unroll, the operand offsets become a few multiples of row_step, and the one issuing thread (which spends
// ~10 cycles per dependent instruction) is left with an add and the MMA per product.
template <int KH, int KW, int KS>
__device__ __forceinline__ void conv_issue_group(const uint32_t (&d)[4], const uint32_t (&a_lo)[4], uint32_t a_hi,
                                                 uint32_t b_lo, uint32_t b_hi, int nt, uint32_t idesc, int kh, int kw,
                                                 int ksteps, uint32_t row_step, uint32_t px_step, uint32_t w_step,
                                                 uint32_t b_kstep) {
  const int nh = KH > 0 ? KH : kh, nw = KW > 0 ? KW : kw, nk = KS > 0 ? KS : ksteps;
  uint32_t accum = 0u;
#pragma unroll
  for (int fh = 0; fh < nh; ++fh) {
#pragma unroll
    for (int fw = 0; fw < nw; ++fw) {
#pragma unroll
      for (int k = 0; k < nk; ++k) {
        // tap (fh, fw) reads the patch (fh * row_w + fw) rows further on; K step k the next 32 bytes of every row
        const uint32_t ao = fh * row_step + fw * px_step + 2 * k;
        const uint32_t bo = (fh * nw + fw) * w_step + k * b_kstep;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < nt) umma_ss_i8_halves(d[j], a_lo[j] + ao, a_hi, b_lo + bo, b_hi, idesc, accum);
        accum = 1u;
      }
    }
  }
}

// The persistent form of the kernel above (ConvParams::persistent): same tiles, same operand views, same
// arithmetic; what changes is that a CTA outlives its tile.
//   warp 0   : the channel tile's weights once, then one input patch per tile into the ring
//   warp 1   : per tile kh * kw * chunk / 32 MMAs (every tap a view into the patch); the MMAs of up to four
//              consecutive tiles are issued interleaved, each tile into its own accumulator (2 x 4 in TMEM)
//   warps 2-9: two groups of four; group e takes this CTA's tiles e, e + 2, ...: the output stage (per-channel
//              srs) of the accumulator the MMAs have left.
// The loops carry their tile coordinates, ring positions and phases along instead of dividing: a division by a
// run-time number costs a single thread several hundred cycles, and the issuing thread has ~80 per MMA to spare.
__global__ void __launch_bounds__(kConvPersistentThreads, 1)
conv2d_i8_persistent_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                            const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* w_smem = smem;                                   // [tap][cout_tile x chunk] (or the N-major box)
  uint8_t* patches = smem + p.w_region_bytes;               // `stages` patches of a_bytes each
  uint8_t* bar_mem = patches + p.stages * p.a_bytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(bar_mem);
  uint64_t* empty_bar = full_bar + kConvMaxStages;
  uint64_t* group_full_bar = empty_bar + kConvMaxStages;    // two: the MMAs of tile group g (g & 1) have completed
  uint64_t* tmem_empty_bar = group_full_bar + 2;            // one per accumulator (up to eight)
  uint64_t* w_bar = tmem_empty_bar + 8;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(w_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  uint8_t* shift_smem = reinterpret_cast<uint8_t*>(tmem_base_slot + 2);  // this CTA's cout_tile shift bytes (<= 256)
  int* half_smem = reinterpret_cast<int*>(bar_mem + 1024);               // 2^(shift-1) - 1 per channel (0 for shift 0)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool tracing = kMeasure && p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;   // 4 stamps per tile of CTA 0

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 4);       // the four epilogue warps, once they have seen the tile's MMAs complete
    }
    for (int a = 0; a < 8; ++a) mbar_init(smem_u32(&tmem_empty_bar[a]), 4);  // one arrival per epilogue warp
    for (int g = 0; g < 2; ++g) mbar_init(smem_u32(&group_full_bar[g]), 1);
    mbar_init(smem_u32(w_bar), 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_base_slot), p.tmem_cols);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_launch_dependents();
  pdl_wait();  // a weight pre-pass before this kernel has completed; global memory may be touched
  const int co0 = blockIdx.y * p.cout_tile;
  const int taps = p.kh * p.kw;
  if (warp >= 2) {
    const int c = threadIdx.x - 64;   // 256 epilogue threads, one channel of the tile each
    const int col = co0 + c;
    const int sh = (c < p.cout_tile && col < p.cout) ? p.shift_vec[col] : 0;
    shift_smem[c] = static_cast<uint8_t>(sh);
    half_smem[c] = sh > 0 ? static_cast<int>((1u << (sh - 1)) - 1u) : 0;
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the epilogue warps only
  }
  // a step of `step` tiles through (image, tile row, tile column), as carries instead of divisions
  struct TileWalk {
    int tw, th, img, dw, dh, dn;
    __device__ void init(int t, int step, const ConvParams& p) {
      int r = fast_div(t, p.tiles_w, p.magic_w);
      tw = t - r * p.tiles_w; img = fast_div(r, p.tiles_h, p.magic_h); th = r - img * p.tiles_h;
      r = fast_div(step, p.tiles_w, p.magic_w);
      dw = step - r * p.tiles_w; dn = fast_div(r, p.tiles_h, p.magic_h); dh = r - dn * p.tiles_h;
    }
    __device__ void next(int tiles_w, int tiles_h) {
      tw += dw; th += dh; img += dn;
      if (tw >= tiles_w) { tw -= tiles_w; ++th; }
      if (th >= tiles_h) { th -= tiles_h; ++img; }
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t wb = smem_u32(w_bar);
      mbar_expect_tx(wb, static_cast<uint32_t>(taps) * p.w_block_bytes);
      if (p.w_n_major) tma_load_3d(smem_u32(w_smem), &tmap_w, wb, co0, 0, 0);   // {cout, cin, tap}
      else tma_load_3d(smem_u32(w_smem), &tmap_w, wb, 0, co0, 0);                 // {cin, cout, tap}
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileWalk at;
      at.init(blockIdx.x, gridDim.x, p);
      for (int t = blockIdx.x; ok && t < p.spatial_tiles; t += gridDim.x, at.next(p.tiles_w, p.tiles_h)) {
        ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY);
        if (!ok) break;
        const uint32_t fb = smem_u32(&full_bar[stage]);
        mbar_expect_tx(fb, p.tx_bytes);
        // the whole patch; what lies outside the image reads as zero: that is the padding
        tma_load_4d(smem_u32(patches + stage * p.a_bytes), &tmap_x, fb, 0, at.tw * p.wt - p.pad,
                    at.th * p.rows_per_tile - p.pad, at.img);
        if (++stage == p.stages) { stage = 0; phase ^= 1; }
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc<KIND_I8>(kBlockM, p.cout_tile) | (p.w_n_major ? (1u << 16) : 0u);
      bool ok = mbar_wait(smem_u32(w_bar), 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      const uint64_t b0 = make_kmajor_desc(smem_u32(w_smem), p.b_sbo_bytes, p.b_swizzle_code);
      const uint64_t a_first = make_kmajor_desc(smem_u32(patches), p.sbo_bytes, p.swizzle_code);
      const uint32_t b_lo = static_cast<uint32_t>(b0), b_hi = static_cast<uint32_t>(b0 >> 32);
      const uint32_t a_hi = static_cast<uint32_t>(a_first >> 32), a_lo0 = static_cast<uint32_t>(a_first);
      // every operand lies below 256 KB, so an offset never carries out of the descriptor's 14-bit address field
      const uint32_t px_step = static_cast<uint32_t>(p.chunk) >> 4;
      const uint32_t row_step = px_step * p.row_w, w_step = p.w_block_bytes >> 4, a_step = p.a_bytes >> 4;
      const uint32_t b_kstep = static_cast<uint32_t>(p.b_kstep);
      const int ksteps = p.chunk / kUmmaKBytes;
      // The MMAs of a GROUP of up to four consecutive tiles are issued interleaved, each tile into its own
      // accumulator, with one commit and one round of barrier polls per group: what bounds this warp is the
      // latency of its own instructions (a poll that succeeds at once still costs ~250 cycles, a commit ~450),
      // so everything that can be shared by four tiles is.
      const int G = p.mma_group, accs = 2 * G;   // accumulators in TMEM: the tile with sequence number s uses s % accs
      int seq = 0, group = 0;                    // tiles and groups this CTA has started
      int tiles_left = (p.spatial_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
      int st = 0;                                // ring position of tile seq, and the parity of its round
      uint32_t st_phase = 0;
      for (; ok && tiles_left > 0; ++group) {
        const int nt = tiles_left < G ? tiles_left : G;
        uint32_t d[4], a_lo[4], bar_acc[4], bar_patch[4], par_acc[4], par_patch[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int s_ = seq + j, acc = s_ & (accs - 1);   // G is 1, 2 or 4
          d[j] = tmem_base + acc * p.acc_stride;
          a_lo[j] = a_lo0 + st * a_step;
          bar_acc[j] = smem_u32(&tmem_empty_bar[acc]);
          par_acc[j] = (s_ & accs) ? 0u : 1u;
          bar_patch[j] = smem_u32(&full_bar[st]);
          par_patch[j] = st_phase;
          if (j < nt && ++st == p.stages) { st = 0; st_phase ^= 1; }
        }
        // accumulators free, patches landed: all polls first (their latencies overlap), the bounded waits for
        // whatever was not ready yet
        bool ready = true;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < nt) {
            const bool r0 = mbar_try_wait(bar_acc[j], par_acc[j]);
            const bool r1 = mbar_try_wait(bar_patch[j], par_patch[j]);
            ready = ready && r0 && r1;
          }
        if (!ready) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (j < nt && ok) {
              ok = mbar_wait(bar_acc[j], par_acc[j], abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY);
              if (ok) ok = mbar_wait(bar_patch[j], par_patch[j], abort_flag, p.status, ST_TIMEOUT_FULL);
            }
        }
        if (!ok) break;
        tc_fence_after();
        if (tracing && seq < 60) p.trace[seq * 4 + 0] = clock64();
        if (p.kh == 3 && p.kw == 3 && ksteps == 2)
          conv_issue_group<3, 3, 2>(d, a_lo, a_hi, b_lo, b_hi, nt, idesc, 3, 3, 2, row_step, px_step, w_step, b_kstep);
        else if (p.kh == 3 && p.kw == 3 && ksteps == 1)
          conv_issue_group<3, 3, 1>(d, a_lo, a_hi, b_lo, b_hi, nt, idesc, 3, 3, 1, row_step, px_step, w_step, b_kstep);
        else if (p.kh == 3 && p.kw == 3 && ksteps == 4)
          conv_issue_group<3, 3, 4>(d, a_lo, a_hi, b_lo, b_hi, nt, idesc, 3, 3, 4, row_step, px_step, w_step, b_kstep);
        else
          conv_issue_group<0, 0, 0>(d, a_lo, a_hi, b_lo, b_hi, nt, idesc, p.kh, p.kw, ksteps, row_step, px_step, w_step,
                                    b_kstep);
        umma_commit(smem_u32(&group_full_bar[group & 1]));   // every tile of the group: accumulator ready, patch read
        if (tracing && seq < 60) p.trace[seq * 4 + 1] = clock64();
        seq += nt;
        tiles_left -= nt;
      }
    }
  } else {
    const int quad = warp & 3;              // the TMEM lanes this warp may read
    const int egroup = (warp - 2) >> 2;     // which of the two epilogue groups
    const int m = quad * 32 + lane;
    const int mr = m / p.row_w, mc = m - mr * p.row_w;   // image row and column inside the tile
    const bool vec = (reinterpret_cast<uintptr_t>(p.y) % 16 == 0) && (p.cout % 16 == 0);
    const SrsPlan plan = srs_plan(shift_smem, p.cout_tile, p.srs_wide != 0);
    const int G = p.mma_group, accs = 2 * G, g_log2 = G == 4 ? 2 : (G == 2 ? 1 : 0);
    const int step = 2 * static_cast<int>(gridDim.x);
    TileWalk at;
    at.init(static_cast<int>(blockIdx.x) + egroup * static_cast<int>(gridDim.x), step, p);
    int stage = egroup % p.stages;          // ring position of tile `it`
    bool ok = true;
    for (int it = egroup, t = static_cast<int>(blockIdx.x) + egroup * static_cast<int>(gridDim.x); t < p.spatial_tiles;
         it += 2, t += step, at.next(p.tiles_w, p.tiles_h)) {
      const int acc = it & (accs - 1), group = it >> g_log2;
      ok = mbar_wait(smem_u32(&group_full_bar[group & 1]), (group >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));   // the tile's MMAs have read its patch
      stage += 2;
      if (stage >= p.stages) stage -= p.stages;
      if (tracing && warp == 2 && lane == 0 && it < 60) p.trace[it * 4 + 2] = clock64();
      const int oh = at.th * p.rows_per_tile + mr, ow = at.tw * p.wt + mc;
      const bool pix_ok = mr < p.rows_per_tile && mc < p.wt && oh < p.h && ow < p.w;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * p.acc_stride;
      int8_t* yrow = p.y + ((static_cast<long long>(at.img) * p.h + oh) * p.w + ow) * p.cout;
      // 64 columns per round: both loads in flight at once; after the last round's loads the accumulator goes
      // back to the MMA issuer before the arithmetic starts
      for (int c = 0; c < p.cout_tile; c += 64) {
        __syncwarp();
        uint32_t v[2][32];
        const bool second = c + 32 < p.cout_tile;
        tmem_ld_32x32b_x32(taddr + c, v[0]);
        if (second) tmem_ld_32x32b_x32(taddr + c + 32, v[1]);
        tmem_ld_wait();
        if (c + 64 >= p.cout_tile) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
        }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int cc = c + hh * 32, col0 = co0 + cc;
          if ((hh == 1 && !second) || !pix_ok || col0 >= p.cout) continue;
          conv_store_chunk(v[hh], plan, shift_smem + cc, half_smem + cc, yrow + col0,
                           min(32, min(p.cout_tile - cc, p.cout - col0)), vec);
        }
      }
      if (tracing && warp == 2 && lane == 0 && it < 60) p.trace[it * 4 + 3] = clock64();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, p.tmem_cols);
  }
}

// HWIO [tap][cin][cout] -> [tap][cout][cin]: makes the weights K-major like every other operand.
__global__ void conv_weight_prepack_kernel(const int8_t* __restrict__ w, int8_t* __restrict__ wp,
                                           int taps, int cin, int cout) {
  const long long n = static_cast<long long>(taps) * cin * cout;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int ci = static_cast<int>(i % cin);
    const long long r = i / cin;
    const int co = static_cast<int>(r % cout);
    const int tap = static_cast<int>(r / cout);
    wp[i] = w[(static_cast<long long>(tap) * cin + ci) * cout + co];
  }
}

// Direct form for shapes the tensor-core tiling does not cover (cin not a multiple of 32, ...).
__global__ void conv2d_i8_direct_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                                        int8_t* __restrict__ y, int n, int h, int wd, int cin, int cout,
                                        int kh, int kw, int pad, const uint8_t* __restrict__ shift_vec) {
  const long long total = static_cast<long long>(n) * h * wd * cout;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int co = static_cast<int>(i % cout);
    long long r = i / cout;
    const int ow = static_cast<int>(r % wd); r /= wd;
    const int oh = static_cast<int>(r % h);
    const int img = static_cast<int>(r / h);
    int acc = 0;
    for (int fh = 0; fh < kh; ++fh) {
      const int ih = oh + fh - pad;
      if (ih < 0 || ih >= h) continue;
      for (int fw = 0; fw < kw; ++fw) {
        const int iw = ow + fw - pad;
        if (iw < 0 || iw >= wd) continue;
        const int8_t* xp = x + ((static_cast<long long>(img) * h + ih) * wd + iw) * cin;
        const int8_t* wp = w + (static_cast<long long>(fh * kw + fw) * cin) * cout + co;
        for (int ci = 0; ci < cin; ++ci) acc += static_cast<int>(xp[ci]) * static_cast<int>(wp[static_cast<long long>(ci) * cout]);
      }
    }
    y[i] = static_cast<int8_t>(srs_i8(acc, shift_vec[co]));
  }
}

// Shapes the tensor-core tiling covers (the others take the direct CUDA-core kernel).
bool conv_tensor_path(const int8_t* x, int cin, int cout) {
  return (cin % 32 == 0) && (cin == 32 || cin == 64 || cin % 128 == 0) && (cout % 16 == 0) &&
         (reinterpret_cast<uintptr_t>(x) % 16 == 0);
}

int launch_conv_pack_weights(aiehlc_ctx* ctx, const int8_t* w, int8_t* packed, int taps, int cin, int cout,
                             cudaStream_t st) {
  const long long wbytes = static_cast<long long>(taps) * cin * cout;
  long long g = (wbytes + 255) / 256;
  if (g > ctx->sm_count * 8LL) g = ctx->sm_count * 8LL;
  conv_weight_prepack_kernel<<<static_cast<int>(g), 256, 0, st>>>(w, packed, taps, cin, cout);
  AIEHLC_CUDA(cudaGetLastError());
  ctx->launches++;
  return AIEHLC_OK;
}

int launch_conv2d_packed(aiehlc_ctx* ctx, const int8_t* x, const int8_t* packed, int8_t* y, int n, int h, int wd,
                         int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st);
int launch_conv_tensor(aiehlc_ctx* ctx, const int8_t* x, const int8_t* weights, bool hwio, int8_t* y, int n, int h,
                       int wd, int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st);
bool conv_hwio_direct(const aiehlc_ctx* ctx, const int8_t* w, int n, int h, int wd, int cin, int cout, int kh, int kw,
                      int pad);
struct ConvParams;
void conv_persistent_setup(const aiehlc_ctx* ctx, ConvParams& p, int n_tiles);

int launch_conv2d(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n, int h, int wd,
                  int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st,
                  int8_t* weight_scratch) {
  const bool tensor_ok = conv_tensor_path(x, cin, cout);
  if (!tensor_ok) {
    const long long total = static_cast<long long>(n) * h * wd * cout;
    long long g = (total + 255) / 256;
    if (g > ctx->sm_count * 16LL) g = ctx->sm_count * 16LL;
    conv2d_i8_direct_kernel<<<static_cast<int>(g), 256, 0, st>>>(x, w, y, n, h, wd, cin, cout, kh, kw,
                                                                 pad, shift_vec);
    AIEHLC_CUDA(cudaGetLastError());
    ctx->launches++;
    return AIEHLC_OK;
  }

  // weights consumed as they are (one launch) where the patch form and the channel tile allow it
  if (conv_hwio_direct(ctx, w, n, h, wd, cin, cout, kh, kw, pad))
    return launch_conv_tensor(ctx, x, w, true, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec, st);
  const int taps = kh * kw;
  const size_t wbytes = static_cast<size_t>(taps) * cin * cout;
  int8_t* packed = weight_scratch;
  if (packed == nullptr) {
    if (ctx->pack_b.reserve(wbytes)) return AIEHLC_ERR_NOMEM;
    packed = static_cast<int8_t*>(ctx->pack_b.ptr);
  }
  // every byte the convolution kernel reads ([0, wbytes)) is rewritten here: nothing an earlier call
  // left in the scratch can reach this one
  if (int rc = launch_conv_pack_weights(ctx, w, packed, taps, cin, cout, st)) return rc;
  return launch_conv2d_packed(ctx, x, packed, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec, st);
}

// Tiling of the tensor-core kernel for the problem already written into p (n .. pad): fills the tile,
// pipeline and form fields; *n_tiles = output-channel tiles (grid y).  The patch form is taken when the
// context allows it and the tile's patch plus every tap's weights fit in shared memory.
void configure_conv(const aiehlc_ctx* ctx, ConvParams& p, int* n_tiles_out) {
  const int n = p.n, h = p.h, wd = p.w, cin = p.cin, cout = p.cout, kh = p.kh, kw = p.kw;
  const int taps = kh * kw;
  const int budget = 200 * 1024;
  int n_tiles = 1;
  // Tiling for one of the two forms; false if the patch form does not fit in shared memory.
  auto configure = [&](bool halo) -> bool {
    p.halo = halo ? 1 : 0;
    if (halo) {
      // the M rows of a tile run over patch rows of wt + kw - 1 pixels (see ConvParams::halo)
      p.wt = wd + kw - 1 <= kBlockM ? wd : kBlockM - (kw - 1);
      p.rows_per_tile = kBlockM / (p.wt + kw - 1);
    } else {
      p.wt = wd <= kBlockM ? wd : kBlockM;
      p.rows_per_tile = wd <= kBlockM ? kBlockM / wd : 1;
    }
    if (p.rows_per_tile > h) p.rows_per_tile = h;
    p.tiles_w = (wd + p.wt - 1) / p.wt;
    p.chunk = cin >= 128 ? 128 : cin;
    p.chunks_per_tap = cin / p.chunk;
    p.cout_tile = cout <= 256 ? cout : 256;
    if (cout > 256 && cout % 256 != 0) {
      // keep every channel tile a legal MMA N: use the largest multiple of 16 that divides cout
      int ct = 256;
      while (ct > 16 && cout % ct != 0) ct -= 16;
      p.cout_tile = ct;
    }
    // A small problem is bound by the latency of a CTA's TMA boxes, not by the tensor pipe: while fewer
    // than half of the SMs would have a tile, give each CTA fewer image rows, then fewer output
    // channels (halves that still divide cout and stay multiples of 16).
    auto ctas = [&]() {
      return static_cast<long long>(n) * ((h + p.rows_per_tile - 1) / p.rows_per_tile) * p.tiles_w *
             ((cout + p.cout_tile - 1) / p.cout_tile);
    };
    while (ctas() * 2 < ctx->sm_count && p.rows_per_tile > 1) p.rows_per_tile = (p.rows_per_tile + 1) / 2;
    while (ctas() * 2 < ctx->sm_count && p.cout_tile % 32 == 0 && p.cout_tile >= 64) p.cout_tile /= 2;
    // the halo form holds every tap's weights of a channel tile at once: narrow the tile until they fit
    if (halo)
      while (taps * p.cout_tile * p.chunk > 96 * 1024 && p.cout_tile % 32 == 0 && cout % (p.cout_tile / 2) == 0)
        p.cout_tile /= 2;
    p.tiles_h = (h + p.rows_per_tile - 1) / p.rows_per_tile;
    n_tiles = (cout + p.cout_tile - 1) / p.cout_tile;
    p.swizzle_code = p.chunk == 128 ? 2u : (p.chunk == 64 ? 4u : 6u);
    p.sbo_bytes = 8u * p.chunk;
    p.row_w = p.wt;
    int num_kb = taps * p.chunks_per_tap;
    int b_bytes = (p.cout_tile * p.chunk + 1023) / 1024 * 1024;
    p.a_bytes = kBlockM * p.chunk;                       // 128 rows reserved, R*Wt of them written
    p.tx_bytes = static_cast<uint32_t>(p.chunk) * (p.wt * p.rows_per_tile + p.cout_tile);
    if (halo) {
      const int row_w = p.wt + kw - 1;
      const int patch_rows = (p.rows_per_tile + kh - 1) * row_w;
      // the last tap's descriptor starts (kh-1)*row_w + kw-1 rows in and the MMA reads 128 rows from there
      const int reach = (kh - 1) * row_w + (kw - 1) + kBlockM;
      const int a_rows = patch_rows > reach ? patch_rows : reach;
      const int a_bytes = (a_rows * p.chunk + 1023) / 1024 * 1024;
      const int w_bytes = (taps * p.cout_tile * p.chunk + 1023) / 1024 * 1024;
      if (a_bytes + w_bytes > budget || p.rows_per_tile + kh - 1 > 256 || row_w > 256 || taps > 256) return false;
      p.row_w = row_w;
      p.a_bytes = a_bytes;
      b_bytes = w_bytes;
      p.w_block_bytes = static_cast<uint32_t>(p.cout_tile) * p.chunk;
      p.tx_bytes = static_cast<uint32_t>(p.chunk) * (patch_rows + taps * p.cout_tile);
      num_kb = p.chunks_per_tap;
    }
    p.stage_bytes = p.a_bytes + b_bytes;
    int stages = budget / p.stage_bytes;
    if (stages > kConvMaxStages) stages = kConvMaxStages;
    if (stages > num_kb) stages = num_kb;
    p.stages = stages;
    return true;
  };
  if (!(ctx->conv_halo && taps > 1 && kw <= kBlockM / 2 && configure(true))) configure(false);
  *n_tiles_out = n_tiles;
}

// Whether a configured convolution runs in the persistent form, and its shared-memory / TMEM layout.
// Taken when every SM would otherwise see two or more CTAs of the one-tile kernel (batches, large images):
// then the weights are fetched once per CTA instead of once per tile and consecutive tiles overlap.
void conv_persistent_setup(const aiehlc_ctx* ctx, ConvParams& p, int n_tiles) {
  p.persistent = 0;
  p.spatial_tiles = p.n * p.tiles_h * p.tiles_w;
  // the largest number divided is below 2 * spatial_tiles (a tile index, or the persistent form's step)
  auto magic = [&](int d) -> uint32_t {
    if (d <= 1 || 2LL * p.spatial_tiles * d >= (1LL << 32)) return 0u;
    return static_cast<uint32_t>((1ULL << 32) / static_cast<uint32_t>(d)) + 1u;
  };
  p.magic_w = magic(p.tiles_w);
  p.magic_h = magic(p.tiles_h);
  // |acc| <= taps * cin * 2^14: below 2^30 the kernels may round in 32 bits where the shifts allow it too
  p.srs_wide = static_cast<long long>(p.kh) * p.kw * p.cin > 65535 ? 1 : 0;
  if (!ctx->conv_persistent || !p.halo || p.chunks_per_tap != 1 || p.wide_n) return;
  if (static_cast<long long>(p.spatial_tiles) * n_tiles < 2LL * ctx->sm_count) return;
  const int taps = p.kh * p.kw;
  const uint32_t w_bytes = (static_cast<uint32_t>(taps) * p.w_block_bytes + 1023u) / 1024u * 1024u;
  const int budget = 200 * 1024;
  int stages = (budget - static_cast<int>(w_bytes)) / p.a_bytes;
  if (stages < 2) return;                       // no room to overlap loads with MMAs: keep the one-tile form
  if (stages > 8) stages = 8;
  p.persistent = 1;
  p.w_split = 0;                                // the weights arrive once, as one box
  p.w_region_bytes = w_bytes;
  p.stages = stages;
  p.tx_bytes = static_cast<uint32_t>(p.chunk) * p.row_w * (p.rows_per_tile + p.kh - 1);   // one patch
  p.acc_stride = static_cast<uint32_t>(p.cout_tile + 31) / 32u * 32u;
  // the MMAs of up to four tiles interleaved, as far as 2 G accumulators fit in TMEM and 2 G patches in the ring
  int g = ctx->conv_mma_group > 0 ? ctx->conv_mma_group : 4;
  while (g > 1 && (2 * g * p.acc_stride > 512 || stages < 2 * g)) g /= 2;
  p.mma_group = g;
  uint32_t cols = 32;
  while (cols < 2 * p.mma_group * p.acc_stride) cols <<= 1;
  p.tmem_cols = cols;
}

// What launch_conv2d_packed will do, for the exported planner.
int plan_conv2d(const aiehlc_ctx* ctx, int n, int h, int wd, int cin, int cout, int kh, int kw, int pad,
                aiehlc_conv_plan* out) {
  aiehlc_conv_plan pl{};
  if ((cin % 32 != 0) || !(cin == 32 || cin == 64 || cin % 128 == 0) || cout % 16 != 0) {
    pl.form = 2;  // CUDA-core kernel: one thread per output element
    const long long total = static_cast<long long>(n) * h * wd * cout;
    long long g = (total + 255) / 256;
    if (g > ctx->sm_count * 16LL) g = ctx->sm_count * 16LL;
    pl.ctas = static_cast<int>(g);
    pl.launches = 1;
    *out = pl;
    return AIEHLC_OK;
  }
  ConvParams p{};
  p.n = n; p.h = h; p.w = wd; p.cin = cin; p.cout = cout; p.kh = kh; p.kw = kw; p.pad = pad;
  int n_tiles = 1;
  configure_conv(ctx, p, &n_tiles);
  pl.form = p.halo ? 1 : 0;
  pl.tile_rows = p.rows_per_tile;
  pl.tile_width = p.wt;
  pl.patch_rows = p.halo ? p.rows_per_tile + kh - 1 : p.rows_per_tile;
  pl.patch_width = p.row_w;
  pl.cout_tile = p.cout_tile;
  pl.cin_chunk = p.chunk;
  pl.ctas = n * p.tiles_h * p.tiles_w * n_tiles;
  const int taps = kh * kw;
  pl.tma_boxes_per_cta = p.halo ? 2 * p.chunks_per_tap : 2 * taps * p.chunks_per_tap;
  pl.mmas_per_cta = taps * p.chunks_per_tap * (p.chunk / kUmmaKBytes);
  pl.stages = p.stages;
  pl.smem_bytes = p.stages * p.stage_bytes + 1024 + 8192 + 1024 + 1024;
  pl.m_rows_used = p.rows_per_tile * p.row_w;
  pl.launches = (ctx->conv_hwio_direct && p.halo && (p.cout_tile == 32 || p.cout_tile == 64 || p.cout_tile == 128) &&
                 cout % p.cout_tile == 0) ? 1 : 2;
  p.w_block_bytes = static_cast<uint32_t>(p.cout_tile) * p.chunk;
  p.wide_n = (p.halo && ctx->conv_wide_n && kw > 1 && kw <= 4 && kw * p.cout_tile <= 256) ? 1 : 0;
  conv_persistent_setup(ctx, p, n_tiles);
  pl.persistent = p.persistent;
  if (p.persistent) {
    const int per_channel_tile = ctx->sm_count / n_tiles > 0 ? ctx->sm_count / n_tiles : 1;
    pl.ctas = (p.spatial_tiles < per_channel_tile ? p.spatial_tiles : per_channel_tile) * n_tiles;
    pl.stages = p.stages;
    pl.smem_bytes = static_cast<int>(p.w_region_bytes) + p.stages * p.a_bytes + 2048;
    pl.tma_boxes_per_cta = 1 + (p.spatial_tiles * n_tiles + pl.ctas - 1) / pl.ctas;   // the weights, then a patch per tile
    pl.mmas_per_cta *= (p.spatial_tiles * n_tiles + pl.ctas - 1) / pl.ctas;
  }
  *out = pl;
  return AIEHLC_OK;
}

// The implicit-GEMM kernel on weights that are already [tap][cout][cin].
int launch_conv2d_packed(aiehlc_ctx* ctx, const int8_t* x, const int8_t* packed, int8_t* y, int n, int h, int wd,
                         int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st) {
  return launch_conv_tensor(ctx, x, packed, false, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec, st);
}

// Whether HWIO weights can feed the tensor cores directly: patch form, and a channel tile whose bytes are
// a swizzle span (the N-major operand's row).
bool conv_hwio_direct(const aiehlc_ctx* ctx, const int8_t* w, int n, int h, int wd, int cin, int cout, int kh, int kw,
                      int pad) {
  if (!ctx->conv_hwio_direct || reinterpret_cast<uintptr_t>(w) % 16 != 0) return false;
  ConvParams p{};
  p.n = n; p.h = h; p.w = wd; p.cin = cin; p.cout = cout; p.kh = kh; p.kw = kw; p.pad = pad;
  int n_tiles = 1;
  configure_conv(ctx, p, &n_tiles);
  return p.halo && (p.cout_tile == 32 || p.cout_tile == 64 || p.cout_tile == 128) && cout % p.cout_tile == 0;
}

// `weights`: [tap][cout][cin] (hwio == false) or the caller's HWIO array (hwio == true, only where
// conv_hwio_direct() said yes).
int launch_conv_tensor(aiehlc_ctx* ctx, const int8_t* x, const int8_t* packed, bool hwio, int8_t* y, int n, int h,
                       int wd, int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st) {
  const int taps = kh * kw;
  ConvParams p{};
  p.n = n; p.h = h; p.w = wd; p.cin = cin; p.cout = cout; p.kh = kh; p.kw = kw; p.pad = pad;
  int n_tiles = 1;
  configure_conv(ctx, p, &n_tiles);
  p.w_split = (p.halo && p.chunks_per_tap == 1 && kh <= kConvMaxStages && kh > 1 && ctx->conv_split_weights) ? 1 : 0;
  p.w_row_bytes = static_cast<uint32_t>(kw) * p.w_block_bytes;
  p.wide_n = (p.halo && ctx->conv_wide_n && kw > 1 && kw <= 4 && kw * p.cout_tile <= 256) ? 1 : 0;
  p.b_lbo_bytes = p.w_block_bytes;
  p.w_n_major = hwio ? 1 : 0;
  p.b_swizzle_code = p.swizzle_code;
  p.b_sbo_bytes = p.sbo_bytes;
  p.b_kstep = kUmmaKBytes >> 4;
  if (hwio) {
    p.b_swizzle_code = p.cout_tile == 128 ? 2u : (p.cout_tile == 64 ? 4u : 6u);
    p.b_sbo_bytes = 8u * p.cout_tile;                         // 8 input channels (rows of cout_tile bytes)
    p.b_kstep = static_cast<uint32_t>(kUmmaKBytes * p.cout_tile) >> 4;  // 32 input channels further on
  }
  uint32_t cols = 32;
  const uint32_t acc_cols = p.wide_n ? static_cast<uint32_t>((kw - 1) * p.cout_tile + (p.cout_tile + 31) / 32 * 32)
                                     : static_cast<uint32_t>(p.cout_tile);
  while (cols < acc_cols) cols <<= 1;
  p.tmem_cols = cols;
  // many tiles per SM: the persistent form (weights resident, patches and accumulators double-buffered)
  conv_persistent_setup(ctx, p, n_tiles);
  p.y = y; p.shift_vec = shift_vec; p.status = ctx->d_status;
  p.trace = ctx->trace;

  // x as a 4-D tensor {cin, w, h, n}; box {chunk, wt, rows_per_tile, 1}
  CUtensorMap mx, mw;
  {
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(wd),
                                static_cast<cuuint64_t>(h), static_cast<cuuint64_t>(n)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(cin) * wd,
                                   static_cast<cuuint64_t>(cin) * wd * h};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(p.chunk), static_cast<cuuint32_t>(p.row_w),
                               static_cast<cuuint32_t>(p.halo ? p.rows_per_tile + kh - 1 : p.rows_per_tile), 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapSwizzle sw = p.chunk == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : p.chunk == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_32B;
    CUresult r = ctx->encode(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<int8_t*>(x), dims, strides,
                             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AIEHLC_ERR_CUDA, "cuTensorMapEncodeTiled failed for conv input");
    const cuuint64_t wdims[2] = {static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(taps) * cout};
    const cuuint64_t wstrides[1] = {static_cast<cuuint64_t>(cin)};
    const cuuint32_t wbox[2] = {static_cast<cuuint32_t>(p.chunk), static_cast<cuuint32_t>(p.cout_tile)};
    if (hwio) {
      // the caller's HWIO weights as {cout, cin, taps}: one box holds cout_tile channels x a cin chunk x every tap,
      // laid down as rows of cout_tile bytes (swizzle span = cout_tile)
      const CUtensorMapSwizzle wsw = p.cout_tile == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                     : p.cout_tile == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
      const cuuint64_t w3dims[3] = {static_cast<cuuint64_t>(cout), static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(taps)};
      const cuuint64_t w3strides[2] = {static_cast<cuuint64_t>(cout), static_cast<cuuint64_t>(cin) * cout};
      const cuuint32_t w3box[3] = {static_cast<cuuint32_t>(p.cout_tile), static_cast<cuuint32_t>(p.chunk),
                                   static_cast<cuuint32_t>(p.w_split ? kw : taps)};
      r = ctx->encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(packed), w3dims, w3strides, w3box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, wsw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else if (p.halo) {
      // the packed weights as {cin, cout, taps}: one box holds a cin chunk of every tap for this channel tile
      const cuuint64_t w3dims[3] = {static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(cout), static_cast<cuuint64_t>(taps)};
      const cuuint64_t w3strides[2] = {static_cast<cuuint64_t>(cin), static_cast<cuuint64_t>(cin) * cout};
      const cuuint32_t w3box[3] = {static_cast<cuuint32_t>(p.chunk), static_cast<cuuint32_t>(p.cout_tile),
                                   static_cast<cuuint32_t>(p.w_split ? kw : taps)};
      r = ctx->encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(packed), w3dims, w3strides, w3box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
      r = ctx->encode(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(packed), wdims, wstrides, wbox, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(AIEHLC_ERR_CUDA, "cuTensorMapEncodeTiled failed for conv weights");
  }

  const int smem_bytes = p.persistent ? static_cast<int>(p.w_region_bytes) + p.stages * p.a_bytes + 2048 + 1024
                                      : p.stages * p.stage_bytes + 1024 + 8192 + 1024 + 1024;
  auto kern = p.persistent ? conv2d_i8_persistent_kernel : conv2d_i8_kernel;
  KernelSetup& ks = ctx->kernel_setup[reinterpret_cast<const void*>(kern)];
  if (int rc = ensure_dynamic_smem(ctx->device, reinterpret_cast<const void*>(kern), smem_bytes, &ks.smem_attr))
    return rc;
  dim3 grid(n * p.tiles_h * p.tiles_w, n_tiles);
  if (p.persistent) {
    const int per_channel_tile = ctx->sm_count / n_tiles > 0 ? ctx->sm_count / n_tiles : 1;
    grid.x = p.spatial_tiles < per_channel_tile ? p.spatial_tiles : per_channel_tile;
  }
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = grid;
  cfg.blockDim = dim3(p.persistent ? kConvPersistentThreads : kConvThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  AIEHLC_CUDA(cudaLaunchKernelEx(&cfg, kern, mx, mw, p));
  ctx->launches++;
  return AIEHLC_OK;
}

}  // namespace aiehlc

// =====================================================================================
// Allocation-free variant of the convolution.
//
// Some callers may not allocate device memory at the moment they call: code running while a
// memory pool is frozen, inside a real-time loop that forbids the driver's allocator lock, or
// under a host framework that owns every byte of the device and hands none out.  The regular
// entry point keeps the re-laid weights ([tap][cout][cin]) in a context workspace that grows with
// cudaMalloc; this one keeps them in a fixed array that is part of the library image instead.
// Every GPU that loads the library carries the array until the process exits.
namespace aiehlc {

constexpr size_t kConvStaticScratchBytes = AIEHLC_CONV_STATIC_SCRATCH_BYTES;

// In host code this name is only a handle for the symbol, not a device address: the address the
// kernels need comes from cudaGetSymbolAddress (below).
static __device__ __align__(256) int8_t g_conv_static_weights[kConvStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
int8_t* g_static_weights_ptr[kMaxDevices] = {};
std::mutex g_static_weights_mu;

// Once per device, with that device current: resolve the array's device address.
int static_weights_address(int device, int8_t** out) {
  if (device < 0 || device >= kMaxDevices) return fail(AIEHLC_ERR_UNSUPPORTED, "device index too large");
  std::lock_guard<std::mutex> lk(g_static_weights_mu);
  if (!g_static_weights_ptr[device]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_conv_static_weights);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_conv_static_weights)");
    if (p == nullptr || reinterpret_cast<uintptr_t>(p) % 256 != 0)
      return fail(AIEHLC_ERR_CUDA, "static conv scratch resolved to a null or misaligned address");
    g_static_weights_ptr[device] = static_cast<int8_t*>(p);
  }
  *out = g_static_weights_ptr[device];
  return AIEHLC_OK;
}
}  // namespace

// The regular launcher -- same forms, same tiling (configure_conv), same kernels -- with the re-laid
// weights, where the shape needs them, in the static array instead of the context's workspace.
int launch_conv2d_static(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n, int h, int wd,
                         int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st) {
  const size_t wbytes = static_cast<size_t>(kh) * kw * cin * cout;
  if (wbytes > kConvStaticScratchBytes)
    return fail(AIEHLC_ERR_UNSUPPORTED,
                "conv2d (static scratch): kh*kw*cin*cout = " + std::to_string(wbytes) + " bytes of weights exceed the " +
                    std::to_string(kConvStaticScratchBytes) + "-byte static scratch; use aiehlc_conv2d_i8_srs_dev");
  int8_t* packed = nullptr;
  if (int rc = static_weights_address(ctx->device, &packed)) return rc;
  return launch_conv2d(ctx, x, w, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec, st, packed);
}

}  // namespace aiehlc

extern "C" int aiehlc_conv2d_i8_srs_static_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n,
                                               int h, int wd, int cin, int cout, int kh, int kw, int pad,
                                               const uint8_t* shift_vec, void* stream) {
  using namespace aiehlc;
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  AIEHLC_CUDA(cudaSetDevice(ctx->device));
  if (n < 0 || h < 0 || wd < 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || pad < 0)
    return fail(AIEHLC_ERR_INVALID, "conv2d (static scratch): bad size");
  if (kh != 2 * pad + 1 || kw != 2 * pad + 1)
    return fail(AIEHLC_ERR_UNSUPPORTED, "conv2d (static scratch): only stride 1 with kh = kw = 2*pad+1");
  if (n == 0 || h == 0 || wd == 0) return AIEHLC_OK;
  if (!x || !w || !y || !shift_vec) return fail(AIEHLC_ERR_INVALID, "conv2d (static scratch): null pointer");
  return launch_conv2d_static(ctx, x, w, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec,
                              static_cast<cudaStream_t>(stream));
}
