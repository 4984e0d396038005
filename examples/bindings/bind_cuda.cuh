// Helper for the binding files in this directory: registers a CUDA kernel under the address of a
// host symbol that an (unmodified) aiehlc example passes to XAie_LoadElfMem.
#pragma once
#include <cuda_runtime.h>

#include "aiehlc_kernels.h"

#define AIEHLC_BIND_CUDA(host_symbol, cuda_kernel, in_addr_, out_addr_, out_bytes_)                  \
  static int aiehlc_launch_##host_symbol(const XAie_KernelLaunchInfo* info) {                        \
    cuda_kernel<<<1, 1, 0, (cudaStream_t)info->stream>>>((const int*)info->in, (int*)info->out);     \
    return (int)cudaGetLastError();                                                                  \
  }                                                                                                  \
  static void __attribute__((constructor)) aiehlc_bind_##host_symbol(void) {                         \
    XAie_KernelDesc d = {#host_symbol, aiehlc_launch_##host_symbol, 0, (out_bytes_), (in_addr_),     \
                         (out_addr_), 0, 0, 0, 0};                                                   \
    XAie_KernelRegister((const void*)host_symbol, &d);                                               \
  }
