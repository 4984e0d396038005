/* Stand-in for the BSP global-timer header: XTime_GetTime / COUNTS_PER_SECOND as used around the
 * move-run-move window of example/matrixmultiply/aieml_mm.cc:112,148,189-190. */
#ifndef XTIME_L_H
#define XTIME_L_H
#include <stdint.h>
#include <time.h>
typedef uint64_t XTime;
#define COUNTS_PER_SECOND 1000000000ULL
static inline void XTime_GetTime(XTime* t) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  *t = (XTime)ts.tv_sec * COUNTS_PER_SECOND + (XTime)ts.tv_nsec;
}
#endif
