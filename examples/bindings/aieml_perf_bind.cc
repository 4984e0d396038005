// Binding file for aiehlc's example/perf/aieml_perf.cc, compiled UNMODIFIED next to it.
// The example's `perf` function (an AIE kernel body that addresses tile memory at fixed
// addresses, aieml_perf.cc:61-83) is never executed here: its address is the key under which
// the library's int32 matmul kernel is registered, with the window addresses of the example's
// annotations (0x1000 in, 0x6000 out) and its 16x16x16 tile.
#include "aiehlc_kernels.h"

void perf(input_window_int32*, output_window_int32*);  // defined by the example

static void __attribute__((constructor)) bind_perf(void) {
  static const XAie_MmArgs args = {16, 16, 16};
  XAie_KernelBind((const void*)perf, "perf", (const void*)aiehlc_k_mm_i32, &args, sizeof args, 0x1000, 0x6000, 0);
}
