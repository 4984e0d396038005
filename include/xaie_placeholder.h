/* The short host API the reference sketches in example/other/aieoob.c:88-95 (and, in a second
 * spelling, example/other/aie-driver-host-kernel.c:27-36): load a kernel by name on a tile, declare
 * the two shim routes, push the input, run, wait, pull the output -- no device instance, routing
 * handle or GMIO buffer in sight.  The reference includes a header of this name and never ships it;
 * the signatures below are the ones its call sites in aieoob.c imply.
 *
 * On B200 the calls sit on the XAie_* run-time of xaiengine.h: the first XAie_LoadKernel brings up
 * an implicit device instance with the array geometry of aieoob.c:8-19 (38 columns x 11 rows, shim
 * row 0, tiles from row 3) unless the program has initialised one itself, in which case that one
 * is used.  Kernel names are the ones given to the registry (XAie_KernelBind / the AIEHLC_KERNEL_*
 * macros of aiehlc_kernels.h; the library's own kernels answer to "mm_i32", "gemm_i8_i32",
 * "gemm_i8_srs", "gemm_bf16", "conv2d_i8_srs" and "srs_i32_i8"). */
#ifndef XAIE_PLACEHOLDER_H
#define XAIE_PLACEHOLDER_H

#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>

#include "xaiengine.h"
#include "aiehlc_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct XAie_Kernel_Inst XAie_Kernel_Inst;

/* aieoob.c:88  XAie_LoadKernel("mm", 12, 3).  NULL on failure (XAie_LastError() says why). */
XAie_Kernel_Inst* XAie_LoadKernel(const char* KernelName, int Col, int Row);
/* aieoob.c:89-90: the shim tiles data enters and leaves through (recorded and validated as routes). */
AieRC XAie_RoutingHostToAie(XAie_Kernel_Inst* Kinst, XAie_LocType ShimLoc);
AieRC XAie_RoutingAieToHost(XAie_Kernel_Inst* Kinst, XAie_LocType ShimLoc);
/* aieoob.c:92: `Bytes` of host memory become the contents of the kernel's input window; Port counts
 * from 1 and only port 1 (the packed A | B window of the matmul kernels) exists. */
AieRC XAie_MoveDataToAie(XAie_Kernel_Inst* Kinst, int Port, const void* Src, size_t Bytes);
/* aieoob.c:93-94: start the kernel; wait until it has finished (bounded: XAIE_CORE_STATUS_TIMEOUT after
 * ten seconds, XAIE_ERR_DEVICE if the kernel reported a failure). */
AieRC XAie_RunCore(XAie_Kernel_Inst* Kinst);
AieRC XAie_WaitOutData(XAie_Kernel_Inst* Kinst);
/* aieoob.c:95: the output window into host memory; bytes beyond what the kernel wrote read as zero
 * (the sketch asks for 512 bytes of a 256-byte result). */
AieRC XAie_MoveAieToData(XAie_Kernel_Inst* Kinst, int Port, void* Dst, size_t Bytes);
/* Argument block for kernels that need one (sizes other than the bound default). */
AieRC XAie_KernelInstSetArgs(XAie_Kernel_Inst* Kinst, const void* Args, u32 Bytes);
/* Unloads nothing on the GPU; frees the handle. */
void XAie_UnloadKernel(XAie_Kernel_Inst* Kinst);

#ifdef __cplusplus
}
#endif
#endif /* XAIE_PLACEHOLDER_H */
