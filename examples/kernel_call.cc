// The kernel-call form of aiehlc (example/nokernelload/aie_nokernelload.cc:100-131): no explicit
// load, route or move -- allocate GMIO buffers, fill them, call k<Col,Row,colstart,rowstart,M,N,K>(in, out).
// First the reference's own 16x16x16 int32 fixture through `perf`, then an int8 GEMM with srs.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "aiehlc_kernels.h"
#include "xaiengine.h"

AIEHLC_KERNEL_CALL_MM_I32(perf)
AIEHLC_KERNEL_CALL_GEMM_I8_SRS(gemm_srs8, /*shift*/ 8, /*split-K*/ 4)

#define MAT_SIZE 256
#define N 16

static int srs(int acc, int s) {
  long long q = (long long)acc >> s, r = (long long)acc & ((1LL << s) - 1), h = 1LL << (s - 1);
  if (r > h || (r == h && (q & 1))) q += 1;
  return q > 127 ? 127 : (q < -128 ? -128 : (int)q);
}

int main() {
  XAie_SetupConfig(ConfigPtr, XAIE_DEV_GEN_AIEML, 0x20000000000, 25, 20, 38, 11, 0, 1, 2, 3, 8);
  XAie_InstDeclare(DevInst, &ConfigPtr);
  if (XAie_CfgInitialize(&DevInst, &ConfigPtr) != XAIE_OK) {
    printf("Driver initialization failed: %s\n", XAie_LastError());
    return 1;
  }
  int bad = 0;

  // ---- the reference's flow: u32 mlen = MAT_SIZE*2 words in, MAT_SIZE words out
  const u32 mlen = MAT_SIZE * 2;
  XAie_MemInst* in = XAie_MemAllocate(&DevInst, mlen * sizeof(u32), XAIE_MEM_CACHEABLE);
  XAie_MemInst* out = XAie_MemAllocate(&DevInst, mlen * sizeof(u32), XAIE_MEM_CACHEABLE);
  u64 phy = (u32)XAie_MemGetDevAddr(in), phy_out = (u32)XAie_MemGetDevAddr(out);
  for (u32 i = 0; i < mlen; i++) { ((int32_t*)phy)[i] = i + 1; ((int32_t*)phy_out)[i] = 0; }
  XAie_MemSyncForDev(in);
  perf<1, 1, 4, 4, N, N, N>(phy, phy_out);   // run the kernel in 1 tile
  if (XAie_KernelCallStatus() != XAIE_OK) { printf("perf call failed: %s\n", XAie_LastError()); return 1; }
  for (int i = 0; i < N; i++)
    for (int j = 0; j < N; j++) {
      int32_t acc = 0;
      for (int k = 0; k < N; k++) acc += ((int32_t*)phy)[i * N + k] * ((int32_t*)phy)[MAT_SIZE + j * N + k];
      if (acc != ((int32_t*)phy_out)[i * N + j]) bad++;
    }
  printf("perf: C[0]=%d C[255]=%d, %d mismatches\n", ((int32_t*)phy_out)[0], ((int32_t*)phy_out)[255], bad);

  // ---- int8 GEMM 256 x 192 x 512 with srs shift 8, cascade split-K 4
  constexpr int M = 256, NN = 192, K = 512;
  XAie_GemmArgs shape = {M, NN, K, 8, 0, 4, 0, 0};
  const u64 off_b = aiehlc_window_offset_b(&shape, 1);
  XAie_MemInst* gin = XAie_MemAllocate(&DevInst, off_b + (u64)NN * K, XAIE_MEM_CACHEABLE);
  XAie_MemInst* gout = XAie_MemAllocate(&DevInst, (u64)M * NN, XAIE_MEM_CACHEABLE);
  signed char* a = (signed char*)XAie_MemGetVAddr(gin);
  signed char* b = a + off_b;
  signed char* c = (signed char*)XAie_MemGetVAddr(gout);
  unsigned long long z = 7;
  for (int i = 0; i < M * K; i++) { z = z * 6364136223846793005ULL + 1442695040888963407ULL; a[i] = (signed char)(z >> 56); }
  for (int i = 0; i < NN * K; i++) { z = z * 6364136223846793005ULL + 1442695040888963407ULL; b[i] = (signed char)(z >> 56); }
  gemm_srs8<8, 16, 4, 4, M, NN, K>(XAie_MemGetDevAddr(gin), XAie_MemGetDevAddr(gout));
  if (XAie_KernelCallStatus() != XAIE_OK) { printf("gemm call failed: %s\n", XAie_LastError()); return 1; }
  int gbad = 0;
  for (int i = 0; i < M; i++)
    for (int j = 0; j < NN; j++) {
      int acc = 0;
      for (int k = 0; k < K; k++) acc += (int)a[i * K + k] * (int)b[j * K + k];
      if (srs(acc, 8) != c[i * NN + j]) gbad++;
    }
  printf("gemm_srs8: %d mismatches\n", gbad);

  // ---- the reference's own int32 kernel far beyond its 16 x 16 tile: perf<.., 384, 256, 512> with full-range
  // words; a product of this size runs as unsigned int8 limb GEMMs on the tensor cores, wrap-around intact
  constexpr int BM = 384, BN = 256, BK = 512;
  XAie_MemInst* bin = XAie_MemAllocate(&DevInst, (u64)(BM + BN) * BK * sizeof(u32), XAIE_MEM_CACHEABLE);
  XAie_MemInst* bout = XAie_MemAllocate(&DevInst, (u64)BM * BN * sizeof(u32), XAIE_MEM_CACHEABLE);
  u32* win = (u32*)XAie_MemGetVAddr(bin);
  u32* res = (u32*)XAie_MemGetVAddr(bout);
  for (int i = 0; i < (BM + BN) * BK; i++) { z = z * 6364136223846793005ULL + 1442695040888963407ULL; win[i] = (u32)(z >> 32); }
  perf<8, 16, 4, 4, BM, BN, BK>(XAie_MemGetDevAddr(bin), XAie_MemGetDevAddr(bout));
  if (XAie_KernelCallStatus() != XAIE_OK) { printf("big perf call failed: %s\n", XAie_LastError()); return 1; }
  int bbad = 0;
  for (int i = 0; i < BM; i += 7)                 // every 7th row, all columns
    for (int j = 0; j < BN; j++) {
      u32 acc = 0;
      for (int k = 0; k < BK; k++) acc += win[i * BK + k] * win[BM * BK + j * BK + k];
      if (acc != res[i * BN + j]) bbad++;
    }
  printf("perf 384x256x512: %d mismatches\n", bbad);
  if (bad == 0 && gbad == 0 && bbad == 0) printf("CPU result matches device output.\n");
  XAie_PartitionTeardown(&DevInst);
  return (bad || gbad || bbad) ? 1 : 0;
}
