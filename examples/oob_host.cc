// The short "out of the box" host flow of aiehlc (example/other/aieoob.c:75-141): no device instance,
// routing handle or GMIO buffer -- load a kernel by name, name the two shim tiles, push, run, wait,
// pull, compare with the host's own triple loop.  Here `mm` is the library's int32 matmul kernel bound
// at 8 x 8 x 8 on the windows the sketch uses; the data is the sketch's fixture h_a[i] = i.
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "xaie_placeholder.h"

#define DATA_SIZE 128
#define MAT_SIZE 64
#define N 8

AIEHLC_KERNEL_MM_I32(mm, N, N, N, /*in*/ 0x1000, /*out*/ 0x6000);

int main() {
  const size_t bytes = DATA_SIZE * sizeof(uint32_t);
  uint32_t* h_a = (uint32_t*)malloc(bytes);
  uint32_t* h_c = (uint32_t*)malloc(bytes);
  for (int i = 0; i < DATA_SIZE; i++) { h_a[i] = i; h_c[i] = 0xdeadbeef; }

  XAie_Kernel_Inst* kinst = XAie_LoadKernel("mm", 12, 3);
  if (!kinst) { printf("XAie_LoadKernel failed: %s\n", XAie_LastError()); return 1; }
  AieRC rc = XAie_RoutingHostToAie(kinst, XAie_TileLoc(2, 0));
  if (rc == XAIE_OK) rc = XAie_RoutingAieToHost(kinst, XAie_TileLoc(35, 0));
  if (rc == XAIE_OK) rc = XAie_MoveDataToAie(kinst, 1, h_a, bytes);
  if (rc == XAIE_OK) rc = XAie_RunCore(kinst);
  if (rc == XAIE_OK) rc = XAie_WaitOutData(kinst);
  if (rc == XAIE_OK) rc = XAie_MoveAieToData(kinst, 1, h_c, bytes);   // 512 bytes asked, 256 produced
  if (rc != XAIE_OK) { printf("flow failed (%d): %s\n", (int)rc, XAie_LastError()); return 1; }

  int mismatches = 0;
  for (int i = 0; i < N; i++)
    for (int j = 0; j < N; j++) {
      int32_t acc = 0;
      for (int k = 0; k < N; k++) acc += (int32_t)h_a[i * N + k] * (int32_t)h_a[MAT_SIZE + j * N + k];
      if (acc != (int32_t)h_c[i * N + j]) {
        printf("Mismatch at index %d: CPU=%d, vmem_out=%d\n", i * N + j, acc, (int32_t)h_c[i * N + j]);
        mismatches++;
      }
    }
  for (int i = MAT_SIZE; i < DATA_SIZE; i++)
    if (h_c[i] != 0) mismatches++;                                     // beyond the result: zero
  printf("C[0]=%d C[63]=%d\n", (int32_t)h_c[0], (int32_t)h_c[63]);
  if (mismatches == 0) printf("CPU result matches vmem_out.\n");
  else printf("Total mismatches = %d\n", mismatches);

  // a second kernel instance under the library's own name for the kernel, with its size given as arguments
  XAie_Kernel_Inst* k2 = XAie_LoadKernel("mm_i32", 13, 3);
  if (!k2) { printf("second XAie_LoadKernel failed: %s\n", XAie_LastError()); return 1; }
  XAie_MmArgs a4 = {4, 4, 4};
  uint32_t in4[32], out4[16];
  for (int i = 0; i < 32; i++) in4[i] = i + 1;
  rc = XAie_KernelInstSetArgs(k2, &a4, sizeof a4);
  if (rc == XAIE_OK) rc = XAie_RoutingHostToAie(k2, XAie_TileLoc(3, 0));
  if (rc == XAIE_OK) rc = XAie_RoutingAieToHost(k2, XAie_TileLoc(3, 0));
  if (rc == XAIE_OK) rc = XAie_MoveDataToAie(k2, 1, in4, sizeof in4);
  if (rc == XAIE_OK) rc = XAie_RunCore(k2);
  if (rc == XAIE_OK) rc = XAie_WaitOutData(k2);
  if (rc == XAIE_OK) rc = XAie_MoveAieToData(k2, 1, out4, sizeof out4);
  if (rc != XAIE_OK) { printf("second flow failed (%d): %s\n", (int)rc, XAie_LastError()); return 1; }
  int bad4 = 0;
  for (int i = 0; i < 4; i++)
    for (int j = 0; j < 4; j++) {
      int32_t acc = 0;
      for (int k = 0; k < 4; k++) acc += (int32_t)in4[i * 4 + k] * (int32_t)in4[16 + j * 4 + k];
      if (acc != (int32_t)out4[i * 4 + j]) bad4++;
    }
  printf("4x4: %d mismatches\n", bad4);
  // misuse is reported, not ignored
  const int e1 = XAie_LoadKernel("no_such_kernel", 12, 3) == NULL;
  const int e2 = XAie_MoveDataToAie(kinst, 2, h_a, bytes) != XAIE_OK;
  const int e3 = XAie_RoutingHostToAie(kinst, XAie_TileLoc(2, 3)) != XAIE_OK;   // not a shim tile
  printf("errors reported: %d %d %d\n", e1, e2, e3);
  XAie_UnloadKernel(k2);
  XAie_UnloadKernel(kinst);
  free(h_a);
  free(h_c);
  return (mismatches == 0 && bad4 == 0 && e1 && e2 && e3) ? 0 : 1;
}
