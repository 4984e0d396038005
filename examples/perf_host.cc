// The host flow of aiehlc's example/perf/aieml_perf.cc (test_routing, lines 105-254) against the
// B200 run-time: reset, load, route, allocate, move in, run, poll, move out, golden compare.  The
// AIE kernel body is replaced by one declaration that binds `perf` to the library's int32 matmul.
#include <stdint.h>
#include <stdio.h>

#include "aiehlc_kernels.h"
#include "xaiengine.h"
#include "xil_cache.h"

#define CORE_IP_MEM 0x1000
#define CORE_OP_MEM 0x6000
#define MAT_SIZE 256
#define N 16

AIEHLC_KERNEL_MM_I32(perf, N, N, N, CORE_IP_MEM, CORE_OP_MEM);

int main() {
  Xil_DCacheDisable();
  XAie_SetupConfig(ConfigPtr, XAIE_DEV_GEN_AIEML, 0x20000000000, 25, 20, 38, 11, 0, 1, 2, 3, 8);
  XAie_InstDeclare(DevInst, &ConfigPtr);
  if (XAie_SetupPartitionConfig(&DevInst, 0x20000000000 + (2ull << 25), 2, 34) != XAIE_OK) return 1;
  if (XAie_CfgInitialize(&DevInst, &ConfigPtr) != XAIE_OK) {
    printf("Driver initialization failed: %s\n", XAie_LastError());
    return 1;
  }
  XAie_SetIOBackend(&DevInst, XAIE_IO_BACKEND_BAREMETAL);
  if (XAie_PartitionInitialize(&DevInst, NULL) != XAIE_OK) return 1;

  const XAie_LocType tile = XAie_TileLoc(4, 4), shim = XAie_TileLoc(33, 0);
  XAie_CoreReset(&DevInst, tile);
  XAie_CoreUnreset(&DevInst, tile);
  if (XAie_LoadElfMem(&DevInst, tile, (unsigned char*)perf) != XAIE_OK) {
    printf("load failed: %s\n", XAie_LastError());
    return 1;
  }
  XAie_RoutingInstance* ri = XAie_InitRoutingHandler(&DevInst);
  XAie_Route(ri, NULL, shim, tile);
  XAie_Route(ri, NULL, tile, shim);

  const u32 mlen = MAT_SIZE * 2;
  XAie_MemInst* in = XAie_MemAllocate(&DevInst, mlen * sizeof(u32), XAIE_MEM_CACHEABLE);
  XAie_MemInst* out = XAie_MemAllocate(&DevInst, mlen * sizeof(u32), XAIE_MEM_CACHEABLE);
  // the examples keep only the low 32 bits of the address (aieml_perf.cc:133): buffers sit below 4 GiB
  int32_t* vmem = (int32_t*)(uintptr_t)(u32)XAie_MemGetDevAddr(in);
  int32_t* vmem_out = (int32_t*)(uintptr_t)(u32)XAie_MemGetDevAddr(out);
  for (u32 i = 0; i < mlen; i++) { vmem[i] = (int32_t)i + 1; vmem_out[i] = 0; }
  XAie_MemSyncForDev(in);
  XAie_MemSyncForCPU(out);

  XAie_MoveDataExternal2Aie(ri, shim, in, mlen * sizeof(u32), CORE_IP_MEM, tile);
  XAie_RouteDmaWait(ri, shim, tile, 1);
  XAie_Run(ri, 1);
  while (XAie_CoreWaitForDone(&DevInst, tile, 0) != XAIE_OK) {
  }
  XAie_MoveDataAie2External(ri, tile, CORE_OP_MEM, mlen * sizeof(u32), out, shim);

  int mismatches = 0;
  for (int i = 0; i < N; i++)
    for (int j = 0; j < N; j++) {
      int32_t acc = 0;
      for (int k = 0; k < N; k++) acc += vmem[i * N + k] * vmem[MAT_SIZE + j * N + k];
      if (acc != vmem_out[i * N + j]) mismatches++;
    }
  printf("C[0]=%d C[255]=%d\n", vmem_out[0], vmem_out[255]);
  if (mismatches == 0) printf("CPU result matches vmem_out.\n");
  else printf("There were %d mismatches.\n", mismatches);
  XAie_PartitionTeardown(&DevInst);
  return mismatches == 0 ? 0 : 1;
}
