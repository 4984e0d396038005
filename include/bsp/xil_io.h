/* Stand-in for the BSP register-access header; the examples include it but call nothing in it. */
#ifndef XIL_IO_H
#define XIL_IO_H
#include <stdint.h>
#endif
