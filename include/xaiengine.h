/*
 * xaiengine.h -- the subset of the AI-Engine run-time API that aiehlc host programs call,
 * implemented for B200 by libaiehlc_b200.so.
 *
 * aiehlc's examples drive the device through AMD's aie-rt driver (XAie_* functions).  That
 * driver is not part of the aiehlc tree, so the signatures below are taken from the call sites
 * in the examples (cited per function, paths relative to the aiehlc tree).  A host program
 * written for aiehlc keeps its `main()` / `test_*()` code; only the kernel definition changes
 * (see aiehlc_kernels.h: a kernel is bound to a CUDA implementation instead of an AIE ELF).
 *
 * Mapping to CUDA
 *   device instance / partition  -> one CUDA device + one stream
 *   tile (col,row)               -> a logical kernel slot with its own device-side data memory
 *   GMIO buffer (XAie_MemInst)   -> pinned host memory the host reads/writes directly
 *   XAie_MoveData*               -> cudaMemcpyAsync on the stream (H2D, D2D, D2H)
 *   XAie_Run                     -> kernel launch(es) on the stream
 *   XAie_CoreWaitForDone         -> event query
 * All functions return XAIE_OK on success.  Nothing here falls back to the CPU.
 */
#ifndef XAIENGINE_H
#define XAIENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint8_t u8;
typedef uint16_t u16;
typedef uint32_t u32;
typedef uint64_t u64;
typedef int8_t s8;
typedef int32_t s32;

typedef enum {
  XAIE_OK = 0,
  XAIE_ERR = 1,
  XAIE_INVALID_DEVICE,
  XAIE_INVALID_ARGS,
  XAIE_INVALID_TILE,
  XAIE_INVALID_ELF,          /* XAie_LoadElfMem: the pointer is not a registered kernel */
  XAIE_CORE_STATUS_TIMEOUT,  /* XAie_CoreWaitForDone: still running */
  XAIE_INVALID_ADDRESS,      /* tile address outside any region the tile owns */
  XAIE_ERR_OUTOFMEM,
  XAIE_ERR_DEVICE            /* CUDA error or kernel status word non-zero */
} AieRC;

/* device generations: preprocessor constants, the examples test them in #if (aieml_perf.cc:160) */
#define XAIE_DEV_GEN_AIE 1U
#define XAIE_DEV_GEN_AIEML 2U
#define XAIE_DEV_GEN_AIE2IPU 3U
#define XAIE_DEV_GEN_AIE2P 4U
#define XAIE_DEV_GEN_AIE2PS 5U

typedef enum {
  XAIE_IO_BACKEND_METAL,
  XAIE_IO_BACKEND_SIM,
  XAIE_IO_BACKEND_CDO,
  XAIE_IO_BACKEND_BAREMETAL,
  XAIE_IO_BACKEND_DEBUG,
  XAIE_IO_BACKEND_LINUX,
  XAIE_IO_BACKEND_CUDA
} XAie_BackendType;

typedef enum { XAIE_MEM_CACHEABLE, XAIE_MEM_NONCACHEABLE } XAie_MemCacheProp;

typedef struct { u8 Row; u8 Col; } XAie_LocType;

typedef struct { XAie_BackendType Type; } XAie_Backend;

/* Array geometry as the examples describe it (aieml_perf.cc:265-269). */
typedef struct {
  u8 AieGen;
  u64 BaseAddr;
  u8 ColShift, RowShift;
  u8 NumRows, NumCols;
  u8 ShimRowNum, MemTileRowStart, MemTileNumRows, AieTileRowStart, AieTileNumRows;
} XAie_Config;

typedef struct XAie_DevInst {
  XAie_Config Cfg;
  u8 IsReady;
  u8 StartCol, PartNumCols;          /* XAie_SetupPartitionConfig */
  u64 PartBaseAddr;
  const XAie_Backend* Backend;       /* examples read DevInst.Backend->Type (aieml_perf.cc:298) */
  XAie_Backend BackendStorage;
  void* Priv;                        /* run-time state: CUDA device, stream, tiles */
  int CudaDevicePlus1;               /* XAie_SetCudaDevice: GPU index + 1; 0 = not chosen by the program */
} XAie_DevInst;

typedef struct XAie_MemInst XAie_MemInst;
typedef struct XAie_RoutingInstance XAie_RoutingInstance;

/* XAie_SetupConfig(ConfigPtr, HW_GEN, base, colshift, rowshift, ncols, nrows, shimrow,
 *                  memrow0, nmemrows, aierow0, naierows)            -- aieml_perf.cc:265-269 */
#define XAie_SetupConfig(Name, Gen, Base, ColShift_, RowShift_, NumCols_, NumRows_, ShimRow_, \
                         MemRow0_, NumMemRows_, AieRow0_, NumAieRows_)                        \
  XAie_Config Name = {(u8)(Gen), (u64)(Base), (u8)(ColShift_), (u8)(RowShift_), (u8)(NumRows_), \
                      (u8)(NumCols_), (u8)(ShimRow_), (u8)(MemRow0_), (u8)(NumMemRows_),       \
                      (u8)(AieRow0_), (u8)(NumAieRows_)}

/* XAie_InstDeclare(DevInst, &ConfigPtr)                                   -- aieml_perf.cc:273 */
#define XAie_InstDeclare(Inst, ConfigPtr) \
  XAie_DevInst Inst = {*(ConfigPtr), 0, 0, 0, 0, &(Inst).BackendStorage, {XAIE_IO_BACKEND_CUDA}, NULL, 0}

static inline XAie_LocType XAie_TileLoc(u8 Col, u8 Row) {
  XAie_LocType l;
  l.Row = Row;
  l.Col = Col;
  return l;
}

/* ---- bring-up / teardown (aieml_perf.cc:281-321) ------------------------------------------
 * One device instance drives one GPU.  Which one, in order of precedence:
 *   1. XAie_SetCudaDevice(&DevInst, gpu), called before XAie_CfgInitialize (an addition; no counterpart);
 *   2. the environment variable AIEHLC_DEVICE (one GPU for the whole process);
 *   3. the partition: XAie_SetupPartitionConfig(&DevInst, base, startcol, ncols) (aieml_perf.cc:281) places the
 *      instance on a range of array columns; the array's NumCols columns are dealt evenly over the visible
 *      GPUs and the instance runs on GPU  startcol * gpus / NumCols  (one GPU: always GPU 0);
 *   4. GPU 0.
 * Instances are independent: a host thread per instance (per GPU) needs no locking, and the calls that
 * name no instance (the kernel-call form, xaie_placeholder.h) resolve it from the GMIO buffer they are
 * given or from the instance the calling thread initialised last. */
AieRC XAie_SetCudaDevice(XAie_DevInst* DevInst, int Device);
int XAie_GetCudaDevice(XAie_DevInst* DevInst);   /* the GPU an initialised instance runs on, else -1 */
AieRC XAie_SetupPartitionConfig(XAie_DevInst* DevInst, u64 PartBaseAddr, u8 PartStartCol, u8 PartNumCols);
AieRC XAie_CfgInitialize(XAie_DevInst* DevInst, XAie_Config* ConfigPtr);
AieRC XAie_SetIOBackend(XAie_DevInst* DevInst, XAie_BackendType Backend);
AieRC XAie_UpdateNpiAddr(XAie_DevInst* DevInst, u64 NpiAddr);
AieRC XAie_PartitionInitialize(XAie_DevInst* DevInst, void* Opts);
AieRC XAie_PartitionTeardown(XAie_DevInst* DevInst);
AieRC XAie_PmRequestTiles(XAie_DevInst* DevInst, XAie_LocType* Loc, u32 NumTiles);
AieRC XAie_Finish(XAie_DevInst* DevInst);

/* ---- core control (aieml_perf.cc:112-113; vek385_verification.cpp:78,129,161; seq_full_col.cpp:72)
 * Reset clears the tile's "done" state; Status is non-zero for rows that hold compute tiles. */
AieRC XAie_CoreReset(XAie_DevInst* DevInst, XAie_LocType Loc);
AieRC XAie_CoreUnreset(XAie_DevInst* DevInst, XAie_LocType Loc);
AieRC XAie_CoreEnable(XAie_DevInst* DevInst, XAie_LocType Loc);
AieRC XAie_CoreDisable(XAie_DevInst* DevInst, XAie_LocType Loc);
AieRC XAie_CoreGetStatus(XAie_DevInst* DevInst, XAie_LocType Loc, u32* CoreStatus);
AieRC XAie_CoreReadDoneBit(XAie_DevInst* DevInst, XAie_LocType Loc, u8* DoneBit);
/* XAIE_OK once every launch of the tile has completed, XAIE_CORE_STATUS_TIMEOUT while it is
 * running (TimeOut in microseconds; 0 = poll once) -- polled in a loop at aieml_perf.cc:174-184. */
AieRC XAie_CoreWaitForDone(XAie_DevInst* DevInst, XAie_LocType Loc, u32 TimeOut);

/* ---- kernel load: the examples pass the kernel FUNCTION cast to unsigned char*
 * (aieml_perf.cc:114; aiehlc rewrites it to the embedded ELF, src/llvm/aiehlc.cc:301-322).
 * Here the pointer is looked up in the kernel registry (aiehlc_kernels.h). */
AieRC XAie_LoadElfMem(XAie_DevInst* DevInst, XAie_LocType Loc, const unsigned char* KernelFn);

/* ---- GMIO buffers (aieml_perf.cc:132-149; multi_kernel.cc:72-75) ----------------------------
 * Pinned host memory.  Small buffers are placed below 4 GiB so that the examples' habit of
 * truncating XAie_MemGetDevAddr() to u32 and using it as a CPU pointer keeps working. */
XAie_MemInst* XAie_MemAllocate(XAie_DevInst* DevInst, u64 Size, XAie_MemCacheProp Cache);
AieRC XAie_MemFree(XAie_MemInst* MemInst);
void* XAie_MemGetVAddr(XAie_MemInst* MemInst);
u64 XAie_MemGetDevAddr(XAie_MemInst* MemInst);
AieRC XAie_MemSyncForDev(XAie_MemInst* MemInst);
AieRC XAie_MemSyncForCPU(XAie_MemInst* MemInst);   /* waits for the stream: pending D2H copies land */

/* ---- routing (aieml_perf.cc:117-122): records the edges of the dataflow graph; moves between
 * two locations are accepted only along a recorded edge. */
XAie_RoutingInstance* XAie_InitRoutingHandler(XAie_DevInst* DevInst);
AieRC XAie_Route(XAie_RoutingInstance* RoutingInstance, void* Constraints, XAie_LocType Source,
                 XAie_LocType Destination);
AieRC XAie_RouteDmaWait(XAie_RoutingInstance* RoutingInstance, XAie_LocType Source,
                        XAie_LocType Destination, u8 Blocking);
AieRC XAie_RoutingInstanceFree(XAie_RoutingInstance* RoutingInstance);

/* ---- data movement ---------------------------------------------------------------------------
 * External2Aie (aieml_perf.cc:156): H2D copy of `Bytes` from the GMIO buffer into the tile's data
 *   memory at TileAddr; arms the tile for the next XAie_Run.
 * Aie2External (aieml_perf.cc:188): D2H copy, returns when the data is in the GMIO buffer.
 * MoveData (aieml_mm.cc:149-151,184-186; multi_tile.cpp:125-127): the generic form.  A location
 *   in the shim row means "external memory" and its pointer is a host address; any other
 *   location is a tile and its pointer is a tile data-memory address. */
AieRC XAie_MoveDataExternal2Aie(XAie_RoutingInstance* RoutingInstance, XAie_LocType ShimLoc,
                                XAie_MemInst* Src, u32 Bytes, u32 TileAddr, XAie_LocType DstLoc);
AieRC XAie_MoveDataAie2External(XAie_RoutingInstance* RoutingInstance, XAie_LocType SrcLoc,
                                u32 TileAddr, u32 Bytes, XAie_MemInst* Dst, XAie_LocType ShimLoc);
AieRC XAie_MoveData(XAie_RoutingInstance* RoutingInstance, XAie_LocType SrcLoc, void* Src, u32 Bytes,
                    void* Dst, XAie_LocType DstLoc);
/* 64-bit sizes for operands beyond 4 GiB (additive; no counterpart call site). */
AieRC XAie_MoveDataExternal2Aie64(XAie_RoutingInstance* RoutingInstance, XAie_LocType ShimLoc,
                                  XAie_MemInst* Src, u64 Bytes, u64 TileAddr, XAie_LocType DstLoc);
AieRC XAie_MoveDataAie2External64(XAie_RoutingInstance* RoutingInstance, XAie_LocType SrcLoc,
                                  u64 TileAddr, u64 Bytes, XAie_MemInst* Dst, XAie_LocType ShimLoc);

/* XAie_Run (aieml_perf.cc:167): launches, `Count` times, every loaded tile that received input
 * since its last run (all loaded tiles if none did). */
AieRC XAie_Run(XAie_RoutingInstance* RoutingInstance, u32 Count);

/* Debug peek/poke of tile data memory (aieml_perf.cc:88-89; vek385_verification.cpp:86,122). */
AieRC XAie_DataMemBlockRead(XAie_DevInst* DevInst, XAie_LocType Loc, u64 Addr, void* Dst, u32 Size);
AieRC XAie_DataMemBlockWrite(XAie_DevInst* DevInst, XAie_LocType Loc, u64 Addr, const void* Src, u32 Size);

/* ---- recorded chains (no counterpart in aie-rt) ----------------------------------------------
 * The examples drive a kernel chain with a host round trip per stage (run, poll, move tile->tile,
 * run, ...: example/multi/multi_tile.cpp:105-145).  Between BeginCapture and EndCapture the same
 * calls (XAie_MoveData*, XAie_Run; XAie_CoreWaitForDone returns XAIE_OK at once) are recorded into a
 * CUDA graph instead of being executed.  XAie_GraphLaunch replays the whole chain with one launch and
 * returns immediately; XAie_GraphWait polls for its completion like XAie_CoreWaitForDone (TimeOut in
 * microseconds, 0 = poll once).  GMIO buffers are read and written when the graph runs, so new input
 * is: fill the buffer, launch, wait, read the output buffer.  Run the sequence once normally before
 * recording it (tile windows must already exist with their size: a window that would have to be created
 * or to grow during recording is refused).  A graph holds device addresses: once a tile window or one of
 * the context's workspaces has moved to a larger allocation, XAie_GraphLaunch refuses the graph
 * (XAIE_ERR, "graph is stale") before any work is issued; record it again. */
typedef struct XAie_Graph XAie_Graph;
AieRC XAie_GraphBeginCapture(XAie_DevInst* DevInst);
AieRC XAie_GraphEndCapture(XAie_DevInst* DevInst, XAie_Graph** Graph);
AieRC XAie_GraphLaunch(XAie_Graph* Graph);
AieRC XAie_GraphWait(XAie_Graph* Graph, u32 TimeOut);
AieRC XAie_GraphDestroy(XAie_Graph* Graph);

/* ---- additions for parameterised kernels (no counterpart in aie-rt) ------------------------- */
/* Per-tile kernel arguments (a struct from aiehlc_kernels.h); copied. */
AieRC XAie_KernelSetArgs(XAie_DevInst* DevInst, XAie_LocType Loc, const void* Args, u32 Bytes);
/* Last error text of the calling thread. */
const char* XAie_LastError(void);
/* Number of kernel launches issued through this device instance. */
u64 XAie_LaunchCount(XAie_DevInst* DevInst);
/* Test hook: the next `Count` completion polls report a non-zero device status (failure-path
 * tests run without faulting a GPU). */
AieRC XAie_DebugInjectStatus(XAie_DevInst* DevInst, u32 Status, u32 Count);

#ifdef __cplusplus
}
#endif
#endif /* XAIENGINE_H */
