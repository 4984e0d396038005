/* Stand-in for the newer BSP timer header (used when AIE_GEN > 2): same interface as xtime_l.h. */
#ifndef XILTIMER_H
#define XILTIMER_H
#include "xtime_l.h"
#endif
