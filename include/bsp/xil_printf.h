/* Stand-in for the Xilinx standalone BSP header of the same name (thirdparty/arch in the aiehlc
 * tree): aiehlc host programs include it for printing; on a hosted system stdio does the job. */
#ifndef XIL_PRINTF_H
#define XIL_PRINTF_H
#include <stdio.h>
#define xil_printf printf
#endif
