// Binding file for aiehlc's tutorial/example.cpp (compiled unmodified): loop_kernel writes 100 + i
// (tutorial/example.cpp:26-31).
#include "bind_cuda.cuh"

void loop_kernel(int*, int*);  // defined by the example

__global__ void loop_kernel_cuda(const int*, int* out) {
  for (int i = 0; i < 20; ++i) out[i] = 100 + i;
}
AIEHLC_BIND_CUDA(loop_kernel, loop_kernel_cuda, 0x1000, 0x5000, 80)
