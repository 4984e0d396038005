/* Stand-in for the BSP sleep header (example/multi/vek385_verification.cpp). */
#ifndef AIEHLC_BSP_SLEEP_H
#define AIEHLC_BSP_SLEEP_H
#include <unistd.h>
#endif
