// int8 GEMM with srs through the XAie_* run-time surface, as a 4-stage cascade over K.
//
// Same shape as aiehlc's chained examples (example/multi/multi_tile.cpp:65-168,
// seq_full_col.cpp:95-159): one kernel per tile of a column, external memory -> first tile,
// tile -> tile moves between stages, last tile -> external memory, one XAie_Run per stage.
// Stage s multiplies K slice s and adds the int32 partial sums handed down by stage s-1; the last
// stage applies shift-round-saturate.  The in-file check is the reference's golden loop
// (example/perf/aieml_perf.cc:199-231) on int8 operands.
//
//   usage: cascade_gemm [M N K shift]      (K must be a multiple of 4)
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "aiehlc_kernels.h"
#include "xaiengine.h"
#include "xil_cache.h"
#include "xtime_l.h"

#define HW_GEN XAIE_DEV_GEN_AIEML
#define XAIE_BASE_ADDR 0x20000000000
#define XAIE_COL_SHIFT 25
#define XAIE_ROW_SHIFT 20
#define XAIE_NUM_ROWS 11
#define XAIE_NUM_COLS 38
#define XAIE_SHIM_ROW 0
#define XAIE_RES_TILE_ROW_START 1
#define XAIE_RES_TILE_NUM_ROWS 2
#define XAIE_AIE_TILE_ROW_START 3
#define XAIE_AIE_TILE_NUM_ROWS 8

#define CORE_IP_MEM 0x1000   // operand window
#define CORE_ACC_MEM 0x3000  // int32 partial sums from the previous stage
#define CORE_OP_MEM 0x6000   // result window
#define STAGES 4
#define COL 4
#define ROW0 3

static int srs(int acc, int s) {
  long long q = acc;
  if (s > 0) {
    q = (long long)acc >> s;
    long long r = (long long)acc & ((1LL << s) - 1), h = 1LL << (s - 1);
    if (r > h || (r == h && (q & 1))) q += 1;
  }
  return q > 127 ? 127 : (q < -128 ? -128 : (int)q);
}

int main(int argc, char** argv) {
  int M = 512, N = 384, K = 1024, shift = 8;
  if (argc == 5) { M = atoi(argv[1]); N = atoi(argv[2]); K = atoi(argv[3]); shift = atoi(argv[4]); }
  if (K % STAGES) { printf("K must be a multiple of %d\n", STAGES); return 2; }
  const int ks = K / STAGES;

  XAie_SetupConfig(ConfigPtr, HW_GEN, XAIE_BASE_ADDR, XAIE_COL_SHIFT, XAIE_ROW_SHIFT, XAIE_NUM_COLS, XAIE_NUM_ROWS,
                   XAIE_SHIM_ROW, XAIE_RES_TILE_ROW_START, XAIE_RES_TILE_NUM_ROWS, XAIE_AIE_TILE_ROW_START,
                   XAIE_AIE_TILE_NUM_ROWS);
  XAie_InstDeclare(DevInst, &ConfigPtr);
  if (XAie_CfgInitialize(&DevInst, &ConfigPtr) != XAIE_OK) {
    printf("Driver initialization failed: %s\n", XAie_LastError());
    return 1;
  }
  XAie_PartitionInitialize(&DevInst, NULL);

  // one kernel per stage: int32 partial sums for stages 0..2, srs flush in the last one
  XAie_GemmArgs args = {M, N, ks, shift, 0, 1, 0, 0};
  for (int s = 0; s < STAGES; ++s) {
    XAie_LocType loc = XAie_TileLoc(COL, ROW0 + s);
    XAie_CoreReset(&DevInst, loc);
    XAie_CoreUnreset(&DevInst, loc);
    const bool last = s == STAGES - 1;
    if (XAie_LoadElfMem(&DevInst, loc, (unsigned char*)(last ? (void*)aiehlc_k_gemm_i8_srs : (void*)aiehlc_k_gemm_i8_i32)) != XAIE_OK) {
      printf("load failed: %s\n", XAie_LastError());
      return 1;
    }
  }
  XAie_RoutingInstance* ri = XAie_InitRoutingHandler(&DevInst);
  const XAie_LocType shim = XAie_TileLoc(2, 0);
  for (int s = 0; s < STAGES; ++s) XAie_Route(ri, NULL, shim, XAie_TileLoc(COL, ROW0 + s));
  for (int s = 0; s + 1 < STAGES; ++s) XAie_Route(ri, NULL, XAie_TileLoc(COL, ROW0 + s), XAie_TileLoc(COL, ROW0 + s + 1));
  XAie_Route(ri, NULL, XAie_TileLoc(COL, ROW0 + STAGES - 1), shim);

  // operands: A[M][K] row-major, B[N][K]; every stage gets its K slice as a packed window A_s | B_s
  std::vector<signed char> A((size_t)M * K), B((size_t)N * K);
  unsigned long long z = 2;
  for (auto& v : A) { z = z * 6364136223846793005ULL + 1442695040888963407ULL; v = (signed char)(z >> 56); }
  for (auto& v : B) { z = z * 6364136223846793005ULL + 1442695040888963407ULL; v = (signed char)(z >> 56); }
  const u64 off_b = aiehlc_window_offset_b(&args, 1);
  const u64 win_bytes = off_b + (u64)N * ks;
  XAie_MemInst* in[STAGES];
  for (int s = 0; s < STAGES; ++s) {
    in[s] = XAie_MemAllocate(&DevInst, win_bytes, XAIE_MEM_CACHEABLE);
    signed char* p = (signed char*)XAie_MemGetVAddr(in[s]);
    for (int i = 0; i < M; ++i) memcpy(p + (size_t)i * ks, &A[(size_t)i * K + (size_t)s * ks], ks);
    for (int j = 0; j < N; ++j) memcpy(p + off_b + (size_t)j * ks, &B[(size_t)j * K + (size_t)s * ks], ks);
    XAie_MemSyncForDev(in[s]);
  }
  XAie_MemInst* out = XAie_MemAllocate(&DevInst, (u64)M * N, XAIE_MEM_CACHEABLE);
  signed char* out_ptr = (signed char*)XAie_MemGetVAddr(out);
  memset(out_ptr, 0x55, (size_t)M * N);

  XTime t0, t1;
  XTime_GetTime(&t0);
  for (int s = 0; s < STAGES; ++s) {
    XAie_LocType loc = XAie_TileLoc(COL, ROW0 + s);
    XAie_GemmArgs a = args;
    a.accumulate = 0;
    a.use_acc = (s == STAGES - 1);
    XAie_KernelSetArgs(&DevInst, loc, &a, sizeof a);
    XAie_MoveDataExternal2Aie64(ri, shim, in[s], win_bytes, CORE_IP_MEM, loc);
    if (s > 0) {
      // partial sums of the stages so far: this tile's previous-stage output plus what was handed down
      XAie_LocType prev = XAie_TileLoc(COL, ROW0 + s - 1);
      if (s < STAGES - 1) {
        // stages 1..2 accumulate into their own output window: seed it with the incoming partials
        XAie_MoveData(ri, prev, (void*)CORE_OP_MEM, (u32)((u64)M * N * 4), (void*)CORE_OP_MEM, loc);
        a.accumulate = 1;
        XAie_KernelSetArgs(&DevInst, loc, &a, sizeof a);
      } else {
        XAie_MoveData(ri, prev, (void*)CORE_OP_MEM, (u32)((u64)M * N * 4), (void*)CORE_ACC_MEM, loc);
      }
    }
    if (XAie_Run(ri, 1) != XAIE_OK) { printf("run failed: %s\n", XAie_LastError()); return 1; }
    while (XAie_CoreWaitForDone(&DevInst, loc, 0) != XAIE_OK) {
    }
  }
  XAie_MoveDataAie2External64(ri, XAie_TileLoc(COL, ROW0 + STAGES - 1), CORE_OP_MEM, (u64)M * N, out, shim);
  XAie_MemSyncForCPU(out);
  XTime_GetTime(&t1);
  printf("cascade of %d stages took %.2f us.\n", STAGES, 1.0 * (t1 - t0) / (COUNTS_PER_SECOND / 1000000));

  // CPU golden: result[i][j] += A[i][k] * B[j][k], then srs
  int mismatches = 0;
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      int acc = 0;
      for (int k = 0; k < K; ++k) acc += (int)A[(size_t)i * K + k] * (int)B[(size_t)j * K + k];
      const int want = srs(acc, shift);
      if (want != out_ptr[(size_t)i * N + j]) {
        if (mismatches < 8) printf("Mismatch at (%d,%d): CPU=%d, device=%d\n", i, j, want, out_ptr[(size_t)i * N + j]);
        mismatches++;
      }
    }
  if (mismatches == 0) printf("CPU result matches device output.\n");
  else printf("There were %d mismatches.\n", mismatches);
  printf("kernel launches: %llu\n", (unsigned long long)XAie_LaunchCount(&DevInst));
  XAie_PartitionTeardown(&DevInst);
  return mismatches == 0 ? 0 : 1;
}
