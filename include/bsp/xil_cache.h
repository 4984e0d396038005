/* Stand-in for the BSP cache-control header.  The examples switch the ARM caches off before
 * talking to the array (example/perf/aieml_perf.cc:258-259); pinned host memory is coherent with
 * the GPU's copy engines, so these are no-ops. */
#ifndef XIL_CACHE_H
#define XIL_CACHE_H
static inline void Xil_DCacheDisable(void) {}
static inline void Xil_ICacheDisable(void) {}
static inline void Xil_DCacheEnable(void) {}
static inline void Xil_ICacheEnable(void) {}
static inline void Xil_DCacheFlush(void) {}
static inline void Xil_DCacheInvalidate(void) {}
#endif
