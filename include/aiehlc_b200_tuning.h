/*
 * aiehlc_b200 -- tuning knobs and measurement aids of the B200 kernel-call path.
 *
 * Nothing here is part of the drop-in boundary (aiehlc_b200.h): every knob has a default that the
 * library chooses per problem, and the entry points behave the same whatever the settings -- same
 * results, bit for bit; only the schedule changes.  The knobs exist for experiments and for the tests
 * that prove the alternative schedules equal.  No counterpart in the reference.
 *
 * The measurement aids at the end (clock stamps, the debug modes that skip part of a kernel) are
 * compiled into the kernels only when the library is built with -DAIEHLC_MEASURE
 * (AIEHLC_MEASURE=1 python -m aiehlc_b200.build gives libaiehlc_b200_measure.so); in the regular build
 * those calls return AIEHLC_ERR_UNSUPPORTED and the kernels carry no such branches.
 */
#ifndef AIEHLC_B200_TUNING_H
#define AIEHLC_B200_TUNING_H

#include "aiehlc_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

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
 * `accumulate` uses the add-reduction form); 2 = the int8 srs epilogue does so too (slower than
 * its per-thread 32-byte stores); 0 = every thread stores its own row directly.  Tile stores need C
 * 16-byte aligned with a 16-byte row pitch; otherwise the direct path is taken whatever the setting. */
int aiehlc_set_tma_store(aiehlc_ctx* ctx, int on);
/* Tuning knob for the CTA-pair kernel: groups of four epilogue warps per CTA.  2 = the two warps of a
 * TMEM lane quarter each drain half of a tile's columns (one staging buffer per warp; more accumulator
 * reads, proxy fences and tile stores in flight: pays where the output stage sets the pace, K <= 1024 bytes);
 * 1 = four warps with two staging buffers each (better where K is deep); 0 (default) = 2 up to 8 K blocks of 128
 * bytes for int8 operands and 4 for bf16 (and never for a
 * row-sharded output, which the wire bounds), else 1. */
int aiehlc_set_epilogue_groups(aiehlc_ctx* ctx, int groups);
/* Tuning knob for a CTA-pair launch whose last wave is at most half full:
 *   1 = (int8, at least one full wave, K >= 2048 bytes) the tail tiles run as two K halves on different
 *       pairs: the upper halves first, the lower halves last, so that every pair has at most half a tile
 *       more than the full waves; the upper half leaves its int32 partial sums in a context workspace and
 *       the lower half adds them in its output stage (integer sums: bit-identical results);
 *   2 = the 256-column tail tiles are cut into two 128-column ranges run by different pairs (narrower
 *       MMAs, nothing to exchange; every output element is still one accumulation over K in the same
 *       order);
 *   3 = (default) whichever of the two measured faster: 2 (the halves' meeting through L2 costs the
 *       feed-bound main loops more than the halves save);
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
/* Tuning knob for the convolution kernel: 1 (default) = where every SM would see two or more tiles (batches,
 * large images; patch form, cin 32, 64 or 128) a CTA keeps its channel tile's weights in shared memory for its
 * whole life and walks the tiles, input patches arriving through a ring of buffers and the accumulator
 * double-buffered, so loads, MMAs and output stage of consecutive tiles overlap; 0 = always one CTA per tile;
 * 2 / 3 / 4 = as 1, with the MMAs of one tile at a time / of two / of four tiles issued interleaved before one
 * commit (1 chooses four where eight accumulators fit in TMEM and the ring holds eight patches, else two, else
 * one). */
int aiehlc_set_conv_persistent(aiehlc_ctx* ctx, int on);
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
 * slower on small images (the wider MMAs wait for the same weight boxes and the epilogue has kw
 * accumulator blocks to add). */
int aiehlc_set_conv_wide_n(aiehlc_ctx* ctx, int on);
/* Tuning knob for aiehlc_gemm_i8_i32_scatter_dev: 1 (default) = results leave as add-reducing TMA tile
 * stores (32 rows x 128 bytes per store; needs N a multiple of 4 and 16-byte aligned shards, else the
 * other form is used), 0 = as per-row reduction instructions issued by the epilogue warps. */
int aiehlc_set_shard_tile_stores(aiehlc_ctx* ctx, int on);
/* Tuning knob: number of tile row-blocks the persistent scheduler walks before it moves to the next
 * tile column (the L2 footprint of one wave is group_m row-blocks of A plus slots/group_m column-blocks
 * of B).  0 = default: 8 for CTA-pair tiles, 16 for single-CTA tiles (about square wave footprints). */
int aiehlc_set_group_m(aiehlc_ctx* ctx, int group_m);
/* Number of SMs the persistent tensor-core GEMM kernels may occupy (one CTA each; CTA pairs take two):
 * the planner sizes waves and picks tile shapes for that many, and the launch uses no more.  0 (default)
 * = all SMs of the device.  This is what the Col x Row tile grid of the kernel-call form
 * k<Col,Row,...>(in, out) turns into (aiehlc_kernels.h), and it lets several contexts share one GPU
 * side by side the way partitions share the AIE array. */
int aiehlc_set_cta_limit(aiehlc_ctx* ctx, int sms);
/* A promise by the caller, 0 (default) = none: with 1 the caller declares that, for every GEMM call on this
 * context from now on, the operands A and B are NOT written by the kernel that precedes the call in its
 * stream (they come from copies, or from kernels further back).  The GEMM kernels then let their loader
 * and multiplier warps start on the first tiles while that preceding kernel is still draining, and only
 * the output stage -- which reads acc_in and writes C -- waits for it to complete.  Back-to-back GEMMs on
 * independent or long-resident operands overlap by up to a tile this way.  The library switches the early
 * start off by itself where it has just launched a kernel that writes an operand (re-pitched operands,
 * the byte planes of the int32 product).  Breaking the promise gives undefined results, never a fault.
 * Only with programmatic launches (aiehlc_set_pdl 1). */
int aiehlc_set_operands_ready(aiehlc_ctx* ctx, int on);
/* Tuning knob: 1 (default) = the tensor-core kernels are launched with programmatic stream
 * serialization, so their set-up (barriers, TMEM allocation) overlaps the tail of the kernel before
 * them in the stream; they still wait for that kernel to complete before touching global memory.
 * 0 = plain stream-ordered launches. */
int aiehlc_set_pdl(aiehlc_ctx* ctx, int on);
/* Test aid, in every build: 3 = the producer warp neither loads nor signals.  Every other warp's wait then runs out
 * (about one second), the kernel records which wait gave up in the status word, frees its TMEM and
 * returns; aiehlc_sync reports AIEHLC_ERR_DEVICE with the code (102 = the MMA issuer waited for
 * operands) and clears it, and the context stays usable.  This is how the bounded-wait exit is tested
 * without faulting or hanging the GPU.  0 = normal.
 * Measurement aids, AIEHLC_MEASURE builds only (results are then meaningless): 1 = skip the TMA loads and
 * run the MMAs on whatever shared memory holds (tensor-pipe ceiling), 2 = skip the MMAs and only
 * stream the operands (operand-feed ceiling), 4 = int32 results are staged in shared memory but their
 * tile stores are not issued, 5 = the output stage is skipped after the accumulator reads. */
int aiehlc_set_debug(aiehlc_ctx* ctx, int mode);
/* Measurement aid (AIEHLC_MEASURE builds only): while `device_buffer` is non-NULL, the first CTA of every GEMM
 * launch writes
 * clock64() stamps for each of its tiles into it, 8 int64 slots per tile: [0] MMA loop start,
 * [1] MMA loop issued, [2] epilogue starts waiting, [3] accumulator ready, [4] epilogue done;
 * tile 0 also holds [5] kernel entry, [6] kernel exit (clock64) and [7] / word 15 the global
 * nanosecond timer at entry / exit.  The buffer must hold 8 * max(2, tiles per CTA) words.  NULL switches the
 * stamps off. */
int aiehlc_set_trace(aiehlc_ctx* ctx, long long* device_buffer);
/* Measurement aid (AIEHLC_MEASURE builds only): while `device_buffer` is non-NULL, every CTA of a CTA-pair GEMM
 * launch writes the
 * global nanosecond timer at its entry and exit into words [2 * CTA] and [2 * CTA + 1] (the buffer
 * must hold 2 * 148 words): shows which pairs finish last.  NULL switches it off. */
int aiehlc_set_cta_times(aiehlc_ctx* ctx, long long* device_buffer);
#ifdef __cplusplus
}
#endif
#endif /* AIEHLC_B200_TUNING_H */
