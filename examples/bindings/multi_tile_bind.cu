// Binding file for aiehlc's example/multi/multi_tile.cpp and seq_full_col.cpp (compiled unmodified):
// CUDA bodies for the two chain kernels (multi_tile.cpp:39-47) registered under the examples' own
// k1 / k2 symbols, windows at the compiler's default addresses (in 0x1000, out 0x5000).
#include "bind_cuda.cuh"

void k1(int*, int*);  // defined by the example
void k2(int*, int*);

__global__ void k1_cuda(const int* in, int* out) {
  for (int i = 0; i < 20; ++i) out[i] = *in + 1;
}
__global__ void k2_cuda(const int* in, int* out) {
  for (int i = 0; i < 20; ++i) out[i] = *in + 10;
}
AIEHLC_BIND_CUDA(k1, k1_cuda, 0x1000, 0x5000, 80)
AIEHLC_BIND_CUDA(k2, k2_cuda, 0x1000, 0x5000, 80)
