// Binding file for aiehlc's example/multi/multi_kernel.cc (compiled unmodified): two kernels loaded
// one after the other on the same tile (multi_kernel.cc:46-54).
#include "bind_cuda.cuh"

void k1(int*, int*);   // defined by the example
void k2(void*, int*);

__global__ void k1_cuda(const int*, int* out) {
  for (int i = 0; i < 20; ++i) out[i] = 100 + i;
}
__global__ void k2_cuda(const int*, int* out) {
  for (int i = 0; i < 20; ++i) out[i] = 200 + i;
}
AIEHLC_BIND_CUDA(k1, k1_cuda, 0x1000, 0x5000, 80)
AIEHLC_BIND_CUDA(k2, k2_cuda, 0x1000, 0x5000, 80)
