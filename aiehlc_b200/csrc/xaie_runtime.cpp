// The XAie_* run-time surface of include/xaiengine.h on top of CUDA.
//
// aiehlc host programs (example/perf/aieml_perf.cc:105-254, example/multi/multi_tile.cpp:65-168)
// talk to the device through AMD's aie-rt driver, which is not part of the aiehlc tree; its
// behaviour at the call sites of the examples is what this file reproduces:
//   tile data memory  -> per-tile device regions keyed by tile address
//   shim DMA          -> cudaMemcpyAsync on the instance's stream
//   core run / done   -> kernel launch + event
#include <cuda_runtime.h>
#include <sys/mman.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/aiehlc_b200.h"
#include "../../include/aiehlc_b200_tuning.h"
#include "../../include/aiehlc_kernels.h"
#include "../../include/xaie_placeholder.h"
#include "../../include/xaiengine.h"

namespace {

thread_local std::string g_err;
AieRC fail(AieRC rc, const std::string& msg) {
  g_err = msg;
  return rc;
}
AieRC cuda_fail(cudaError_t e, const char* what) {
  g_err = std::string(what) + ": " + cudaGetErrorString(e);
  return XAIE_ERR_DEVICE;
}
#define XCUDA(call)                                         \
  do {                                                      \
    cudaError_t e__ = (call);                               \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call);   \
  } while (0)

// ------------------------------------------------------------------------------ kernel registry
struct KernelEntry {
  std::string name;
  XAie_KernelLaunchFn launch = nullptr;
  XAie_KernelOutBytesFn out_bytes = nullptr;
  u64 out_bytes_default = 0;
  u32 in_addr = 0x1000, out_addr = 0x6000, acc_addr = 0;
  std::vector<uint8_t> default_args;
  void* user = nullptr;
};

struct Registry {
  std::mutex mu;
  std::map<const void*, KernelEntry> map;
};
Registry& registry() {
  static Registry* r = new Registry();  // never destroyed: constructors of user code may run late
  return *r;
}
void seed_library_kernels();

bool lookup_kernel(const void* key, KernelEntry* out) {
  seed_library_kernels();
  Registry& r = registry();
  std::lock_guard<std::mutex> lk(r.mu);
  auto it = r.map.find(key);
  if (it == r.map.end()) return false;
  *out = it->second;
  return true;
}

// ------------------------------------------------------------------------------ run-time state
struct Region {
  u64 addr = 0;
  size_t cap = 0;
  void* dptr = nullptr;
};

struct Tile {
  bool loaded = false;
  KernelEntry kernel;
  std::vector<uint8_t> args;
  std::vector<Region> regions;
  cudaEvent_t done = nullptr;
  bool launched = false;
  bool armed = false;
  u64 in_bytes = 0;
  u64 out_bytes = 0;     // bytes the kernel's last launch produced in its output window
  bool enabled = true;
};

struct Runtime;
}  // namespace

struct XAie_MemInst {
  Runtime* rt = nullptr;
  void* host = nullptr;
  size_t bytes = 0;
  size_t map_bytes = 0;
  bool mmapped = false;     // low-4GiB mmap + cudaHostRegister, else cudaMallocHost
};

struct XAie_RoutingInstance {
  Runtime* rt = nullptr;
  std::vector<std::pair<u16, u16>> edges;
};

struct XAie_Graph {
  Runtime* rt = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaEvent_t done = nullptr;
  bool launched = false;
  // what the recorded device addresses depended on: see Runtime::generation
  u64 rt_generation = 0;
  long long ctx_generation = 0;
};

namespace {

inline u16 loc_key(XAie_LocType l) { return static_cast<u16>((l.Col << 8) | l.Row); }

struct Runtime {
  XAie_DevInst* dev = nullptr;
  int device = 0;
  aiehlc_ctx* ctx = nullptr;
  cudaStream_t stream = nullptr;
  std::map<u16, Tile> tiles;
  std::vector<XAie_MemInst*> mems;
  std::mutex mems_mu;       // the list is also read by kernel calls of other threads looking for a buffer's owner
  std::vector<XAie_RoutingInstance*> routes;
  u64 launches = 0;
  u32 inject_status = 0, inject_count = 0;
  bool capturing = false;   // between XAie_GraphBeginCapture and XAie_GraphEndCapture
  // Counts the times a tile window moved to a larger allocation.  A recorded graph holds raw device
  // addresses of windows (and of the context's workspaces, which have their own counter); replaying it
  // after either moved would touch freed memory, so XAie_GraphLaunch compares both counters first.
  u64 generation = 0;

  bool is_shim(XAie_LocType l) const { return l.Row == dev->Cfg.ShimRowNum; }
  bool valid_loc(XAie_LocType l) const {
    return l.Row < dev->Cfg.NumRows && l.Col < dev->Cfg.NumCols;
  }
  bool is_core_row(XAie_LocType l) const {
    return l.Row >= dev->Cfg.AieTileRowStart && l.Row < dev->Cfg.AieTileRowStart + dev->Cfg.AieTileNumRows;
  }
  Tile& tile(XAie_LocType l) { return tiles[loc_key(l)]; }

  // Tile data memory is a set of WINDOWS, each starting at an address the kernel declares (input,
  // accumulator, output) or at the first address something was moved to.  An address belongs to
  // the window with the greatest start at or below it, whatever the sizes: on the AIE a window is a
  // few KiB, here a GEMM operand window may hold hundreds of MiB, and it must not swallow the
  // addresses of the windows declared above it.
  u64 window_start(const Tile& t, u64 addr) const {
    bool found = false;
    u64 best = 0;
    auto consider = [&](u64 s) {
      if (s <= addr && (!found || s > best)) { best = s; found = true; }
    };
    if (t.loaded) {
      consider(t.kernel.in_addr);
      consider(t.kernel.out_addr);
      if (t.kernel.acc_addr) consider(t.kernel.acc_addr);
    }
    for (const auto& r : t.regions) consider(r.addr);
    return found ? best : addr;
  }
  Region* find_window(Tile& t, u64 start) {
    for (auto& r : t.regions)
      if (r.addr == start) return &r;
    return nullptr;
  }
  // Existing bytes at [addr, addr+bytes): the window must exist and cover the start address.
  Region* find_region(Tile& t, u64 addr, size_t bytes) {
    Region* r = find_window(t, window_start(t, addr));
    if (!r || addr + (bytes ? 1 : 0) > r->addr + r->cap) return nullptr;
    return r;
  }
  // Window that holds [addr, addr+bytes): reuse, grow (contents kept) or create.
  AieRC ensure_region(Tile& t, u64 addr, size_t bytes, void** dptr) {
    if (bytes == 0) bytes = 1;
    const u64 start = window_start(t, addr);
    const size_t need = static_cast<size_t>(addr - start) + bytes;
    if (Region* r = find_window(t, start)) {
      if (need > r->cap) {
        if (capturing) return fail(XAIE_ERR, "a tile window would have to grow while a graph is being recorded; run the sequence once before recording it");
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, need);
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(tile window)");
        XCUDA(cudaMemcpyAsync(p, r->dptr, r->cap, cudaMemcpyDeviceToDevice, stream));
        // like tile data memory, bytes nothing has written read as zero
        XCUDA(cudaMemsetAsync(static_cast<uint8_t*>(p) + r->cap, 0, need - r->cap, stream));
        XCUDA(cudaStreamSynchronize(stream));
        cudaFree(r->dptr);
        r->dptr = p;
        r->cap = need;
        ++generation;
      }
      *dptr = static_cast<uint8_t*>(r->dptr) + (addr - start);
      return XAIE_OK;
    }
    Region r;
    r.addr = start;
    r.cap = need;
    cudaError_t e = cudaMalloc(&r.dptr, need);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(tile window)");
    if (capturing) {
      cudaFree(r.dptr);
      return fail(XAIE_ERR, "a tile window would have to be created while a graph is being recorded; run the sequence once before recording it");
    }
    XCUDA(cudaMemsetAsync(r.dptr, 0, need, stream));  // unwritten bytes read as zero
    t.regions.push_back(r);
    *dptr = static_cast<uint8_t*>(r.dptr) + (addr - start);
    return XAIE_OK;
  }
};

// Kernel-call expressions carry no instance argument.  They run on the instance that owns the GMIO
// buffer their input address lies in; the short host API, which names no instance either, uses the one
// the CALLING THREAD initialised last.  Nothing here is shared between host threads except the list
// below (under its mutex), so one device instance per thread needs no further locking.
thread_local Runtime* g_current_rt = nullptr;
std::mutex g_runtimes_mu;
std::vector<Runtime*> g_runtimes;

Runtime* rt_of(XAie_DevInst* d) { return d ? static_cast<Runtime*>(d->Priv) : nullptr; }

AieRC need_rt(XAie_DevInst* d, Runtime** out) {
  if (!d) return fail(XAIE_INVALID_ARGS, "null device instance");
  Runtime* rt = rt_of(d);
  if (!rt || !d->IsReady) return fail(XAIE_INVALID_DEVICE, "device instance not initialised (XAie_CfgInitialize)");
  cudaError_t e = cudaSetDevice(rt->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  *out = rt;
  return XAIE_OK;
}

bool edge_ok(XAie_RoutingInstance* ri, XAie_LocType s, XAie_LocType d) {
  if (ri->edges.empty()) return true;  // nothing routed: moves are unchecked
  for (auto& e : ri->edges)
    if (e.first == loc_key(s) && e.second == loc_key(d)) return true;
  return false;
}

AieRC h2t(Runtime* rt, XAie_LocType dst, u64 tile_addr, const void* src, size_t bytes) {
  if (!rt->valid_loc(dst) || rt->is_shim(dst)) return fail(XAIE_INVALID_TILE, "destination is not a tile");
  Tile& t = rt->tile(dst);
  void* p = nullptr;
  AieRC rc = rt->ensure_region(t, tile_addr, bytes, &p);
  if (rc != XAIE_OK) return rc;
  if (bytes) XCUDA(cudaMemcpyAsync(p, src, bytes, cudaMemcpyHostToDevice, rt->stream));
  t.armed = true;
  if (!t.loaded || tile_addr == t.kernel.in_addr) t.in_bytes = bytes;
  return XAIE_OK;
}

// Tile -> host.  Like real tile data memory, bytes of the range that no window covers read as
// zero (the examples read a whole 2 KiB window back although the kernel wrote 1 KiB of it,
// example/perf/aieml_perf.cc:188); the range must at least start inside a window.
AieRC t2h(Runtime* rt, XAie_LocType src, u64 tile_addr, void* dst, size_t bytes) {
  if (!rt->valid_loc(src) || rt->is_shim(src)) return fail(XAIE_INVALID_TILE, "source is not a tile");
  Tile& t = rt->tile(src);
  Region* r = rt->find_region(t, tile_addr, bytes);
  if (!r) return fail(XAIE_INVALID_ADDRESS, "tile address was never written or produced");
  const size_t avail = static_cast<size_t>(r->addr + r->cap - tile_addr);
  const size_t n = bytes < avail ? bytes : avail;
  if (n)
    XCUDA(cudaMemcpyAsync(dst, static_cast<uint8_t*>(r->dptr) + (tile_addr - r->addr), n,
                          cudaMemcpyDeviceToHost, rt->stream));
  if (!rt->capturing) XCUDA(cudaStreamSynchronize(rt->stream));  // a recorded copy lands when the graph runs
  if (bytes > n) memset(static_cast<uint8_t*>(dst) + n, 0, bytes - n);
  return XAIE_OK;
}

AieRC t2t(Runtime* rt, XAie_LocType src, u64 saddr, XAie_LocType dst, u64 daddr, size_t bytes) {
  Tile& ts = rt->tile(src);
  Region* r = rt->find_region(ts, saddr, bytes);
  if (!r || saddr + bytes > r->addr + r->cap)
    return fail(XAIE_INVALID_ADDRESS, "source tile address range was never written or produced");
  const void* sp = static_cast<uint8_t*>(r->dptr) + (saddr - r->addr);
  Tile& td = rt->tile(dst);
  void* dp = nullptr;
  AieRC rc = rt->ensure_region(td, daddr, bytes, &dp);
  if (rc != XAIE_OK) return rc;
  if (bytes) XCUDA(cudaMemcpyAsync(dp, sp, bytes, cudaMemcpyDeviceToDevice, rt->stream));
  td.armed = true;
  if (!td.loaded || daddr == td.kernel.in_addr) td.in_bytes = bytes;
  return XAIE_OK;
}

AieRC launch_tile(Runtime* rt, Tile& t, u32 count) {
  XAie_KernelLaunchInfo info{};
  const void* args = t.args.empty() ? t.kernel.default_args.data() : t.args.data();
  const u32 args_bytes = static_cast<u32>(t.args.empty() ? t.kernel.default_args.size() : t.args.size());
  if (Region* r = rt->find_region(t, t.kernel.in_addr, 1)) {
    info.in = static_cast<uint8_t*>(r->dptr) + (t.kernel.in_addr - r->addr);
    info.in_bytes = r->cap - (t.kernel.in_addr - r->addr);
  }
  u64 ob = t.kernel.out_bytes ? t.kernel.out_bytes(args, args_bytes, t.in_bytes, t.kernel.user)
                              : t.kernel.out_bytes_default;
  if (ob == 0) ob = 16;
  void* op = nullptr;
  AieRC rc = rt->ensure_region(t, t.kernel.out_addr, ob, &op);
  if (rc != XAIE_OK) return rc;
  info.out = op;
  info.out_bytes = ob;
  t.out_bytes = ob;
  if (t.kernel.acc_addr) {
    if (Region* r = rt->find_region(t, t.kernel.acc_addr, 1)) {
      info.acc = static_cast<uint8_t*>(r->dptr) + (t.kernel.acc_addr - r->addr);
      info.acc_bytes = r->cap - (t.kernel.acc_addr - r->addr);
    }
  }
  info.args = args;
  info.args_bytes = args_bytes;
  info.stream = rt->stream;
  info.ctx = rt->ctx;
  info.user = t.kernel.user;
  for (u32 i = 0; i < count; ++i) {
    const int r = t.kernel.launch(&info);
    if (r != 0) {
      if (g_err.empty()) g_err = "kernel '" + t.kernel.name + "' launch failed (code " + std::to_string(r) + ")";
      return XAIE_ERR_DEVICE;
    }
    rt->launches++;
  }
  if (!rt->capturing) {
    if (!t.done) XCUDA(cudaEventCreateWithFlags(&t.done, cudaEventDisableTiming));
    XCUDA(cudaEventRecord(t.done, rt->stream));
  }
  t.launched = true;
  t.armed = false;
  return XAIE_OK;
}

void free_runtime(Runtime* rt) {
  if (!rt) return;
  cudaSetDevice(rt->device);
  if (rt->stream) cudaStreamSynchronize(rt->stream);
  for (auto& kv : rt->tiles) {
    for (auto& r : kv.second.regions) cudaFree(r.dptr);
    if (kv.second.done) cudaEventDestroy(kv.second.done);
  }
  for (XAie_MemInst* m : rt->mems) {
    if (m->mmapped) {
      cudaHostUnregister(m->host);
      munmap(m->host, m->map_bytes);
    } else if (m->host) {
      cudaFreeHost(m->host);
    }
    delete m;
  }
  for (XAie_RoutingInstance* ri : rt->routes) delete ri;
  if (rt->stream) cudaStreamDestroy(rt->stream);
  if (rt->ctx) aiehlc_destroy(rt->ctx);
  delete rt;
}

}  // namespace

// =================================================================================== C surface
extern "C" {

const char* XAie_LastError(void) { return g_err.c_str(); }

AieRC XAie_SetupPartitionConfig(XAie_DevInst* DevInst, u64 PartBaseAddr, u8 PartStartCol, u8 PartNumCols) {
  if (!DevInst) return fail(XAIE_INVALID_ARGS, "null device instance");
  if (PartNumCols == 0) return fail(XAIE_INVALID_ARGS, "partition without columns");
  DevInst->PartBaseAddr = PartBaseAddr;
  DevInst->StartCol = PartStartCol;
  DevInst->PartNumCols = PartNumCols;
  return XAIE_OK;
}

AieRC XAie_CfgInitialize(XAie_DevInst* DevInst, XAie_Config* ConfigPtr) {
  if (!DevInst || !ConfigPtr) return fail(XAIE_INVALID_ARGS, "null argument");
  if (ConfigPtr->NumRows == 0 || ConfigPtr->NumCols == 0) return fail(XAIE_INVALID_ARGS, "empty array geometry");
  if (DevInst->IsReady && DevInst->Priv) return XAIE_OK;
  DevInst->Cfg = *ConfigPtr;
  DevInst->Backend = &DevInst->BackendStorage;
  DevInst->BackendStorage.Type = XAIE_IO_BACKEND_CUDA;
  // Which GPU: XAie_SetCudaDevice if it was called; else the environment variable AIEHLC_DEVICE; else,
  // when a partition was configured, the array's columns are dealt evenly over the visible GPUs and
  // the partition runs on the GPU that owns its start column; else GPU 0.
  int device = 0;
  if (DevInst->CudaDevicePlus1 > 0) {
    device = DevInst->CudaDevicePlus1 - 1;
  } else if (const char* e = getenv("AIEHLC_DEVICE")) {
    device = atoi(e);
  } else if (DevInst->PartNumCols > 0) {
    int gpus = 0;
    if (cudaGetDeviceCount(&gpus) != cudaSuccess) { cudaGetLastError(); gpus = 0; }
    if (gpus > 1) device = static_cast<int>(DevInst->StartCol) * gpus / ConfigPtr->NumCols;
    if (device >= gpus && gpus > 0) device = gpus - 1;
  }
  aiehlc_ctx* ctx = nullptr;
  if (aiehlc_create(device, &ctx) != AIEHLC_OK) return fail(XAIE_INVALID_DEVICE, aiehlc_last_error());
  Runtime* rt = new Runtime();
  rt->dev = DevInst;
  rt->device = device;
  rt->ctx = ctx;
  cudaError_t e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    aiehlc_destroy(ctx);
    delete rt;
    return cuda_fail(e, "cudaStreamCreate");
  }
  DevInst->Priv = rt;
  DevInst->IsReady = 1;
  g_current_rt = rt;
  {
    std::lock_guard<std::mutex> lk(g_runtimes_mu);
    g_runtimes.push_back(rt);
  }
  return XAIE_OK;
}

AieRC XAie_SetCudaDevice(XAie_DevInst* DevInst, int Device) {
  if (!DevInst) return fail(XAIE_INVALID_ARGS, "null device instance");
  if (DevInst->IsReady && DevInst->Priv) return fail(XAIE_ERR, "XAie_SetCudaDevice: call it before XAie_CfgInitialize");
  if (Device < 0) return fail(XAIE_INVALID_ARGS, "XAie_SetCudaDevice: negative device");
  DevInst->CudaDevicePlus1 = Device + 1;
  return XAIE_OK;
}

int XAie_GetCudaDevice(XAie_DevInst* DevInst) {
  Runtime* rt = rt_of(DevInst);
  return rt ? rt->device : -1;
}

AieRC XAie_SetIOBackend(XAie_DevInst* DevInst, XAie_BackendType Backend) {
  if (!DevInst) return fail(XAIE_INVALID_ARGS, "null device instance");
  // Recorded so that programs branching on Backend->Type take the path they asked for; the
  // transport is CUDA whatever the value.
  DevInst->BackendStorage.Type = Backend;
  DevInst->Backend = &DevInst->BackendStorage;
  return XAIE_OK;
}

AieRC XAie_UpdateNpiAddr(XAie_DevInst* DevInst, u64) {
  return DevInst ? XAIE_OK : fail(XAIE_INVALID_ARGS, "null device instance");
}
AieRC XAie_PartitionInitialize(XAie_DevInst* DevInst, void*) {
  Runtime* rt;
  return need_rt(DevInst, &rt);
}
AieRC XAie_PmRequestTiles(XAie_DevInst* DevInst, XAie_LocType*, u32) {
  return DevInst ? XAIE_OK : fail(XAIE_INVALID_ARGS, "null device instance");
}
AieRC XAie_PartitionTeardown(XAie_DevInst* DevInst) {
  if (!DevInst) return fail(XAIE_INVALID_ARGS, "null device instance");
  if (g_current_rt == rt_of(DevInst)) g_current_rt = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_runtimes_mu);
    for (size_t i = 0; i < g_runtimes.size(); ++i)
      if (g_runtimes[i] == rt_of(DevInst)) {
        g_runtimes.erase(g_runtimes.begin() + i);
        break;
      }
  }
  free_runtime(rt_of(DevInst));
  DevInst->Priv = nullptr;
  DevInst->IsReady = 0;
  return XAIE_OK;
}
AieRC XAie_Finish(XAie_DevInst* DevInst) { return XAie_PartitionTeardown(DevInst); }

AieRC XAie_CoreReset(XAie_DevInst* DevInst, XAie_LocType Loc) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!rt->valid_loc(Loc)) return fail(XAIE_INVALID_TILE, "tile outside the array");
  Tile& t = rt->tile(Loc);
  t.launched = false;
  t.armed = false;
  return XAIE_OK;
}
AieRC XAie_CoreUnreset(XAie_DevInst* DevInst, XAie_LocType Loc) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  return rt->valid_loc(Loc) ? XAIE_OK : fail(XAIE_INVALID_TILE, "tile outside the array");
}
AieRC XAie_CoreEnable(XAie_DevInst* DevInst, XAie_LocType Loc) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!rt->valid_loc(Loc)) return fail(XAIE_INVALID_TILE, "tile outside the array");
  rt->tile(Loc).enabled = true;
  return XAIE_OK;
}
AieRC XAie_CoreDisable(XAie_DevInst* DevInst, XAie_LocType Loc) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!rt->valid_loc(Loc)) return fail(XAIE_INVALID_TILE, "tile outside the array");
  rt->tile(Loc).enabled = false;
  return XAIE_OK;
}
AieRC XAie_CoreGetStatus(XAie_DevInst* DevInst, XAie_LocType Loc, u32* CoreStatus) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!CoreStatus) return fail(XAIE_INVALID_ARGS, "null status pointer");
  // Non-zero ("enabled") exactly for the rows that hold compute tiles (seq_full_col.cpp:68-80).
  *CoreStatus = (rt->valid_loc(Loc) && rt->is_core_row(Loc)) ? 1u : 0u;
  return XAIE_OK;
}

static AieRC poll_done(Runtime* rt, Tile& t) {
  if (rt->inject_count > 0) {
    rt->inject_count--;
    return fail(XAIE_ERR_DEVICE, "injected device status " + std::to_string(rt->inject_status));
  }
  if (!t.loaded) return fail(XAIE_INVALID_TILE, "no kernel loaded on this tile");
  if (!t.launched) return fail(XAIE_CORE_STATUS_TIMEOUT, "tile has not been run");
  if (rt->capturing) return XAIE_OK;  // recording: ordering is the graph's, completion is XAie_GraphWait's
  cudaError_t e = cudaEventQuery(t.done);
  if (e == cudaErrorNotReady) return XAIE_CORE_STATUS_TIMEOUT;
  if (e != cudaSuccess) return cuda_fail(e, "cudaEventQuery");
  int status = 0;
  if (aiehlc_sync(rt->ctx, rt->stream, &status) != AIEHLC_OK && status == 0)
    return fail(XAIE_ERR_DEVICE, aiehlc_last_error());
  if (status != 0) {
    // Reported once (aiehlc_sync cleared the word): the next poll says "done", so the examples'
    // `while (XAie_CoreWaitForDone(...) != XAIE_OK)` loops end instead of spinning on a dead launch.
    fprintf(stderr, "aiehlc: kernel '%s' reported device status %d\n", t.kernel.name.c_str(), status);
    return fail(XAIE_ERR_DEVICE, "kernel status word = " + std::to_string(status));
  }
  return XAIE_OK;
}

AieRC XAie_CoreWaitForDone(XAie_DevInst* DevInst, XAie_LocType Loc, u32 TimeOut) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!rt->valid_loc(Loc)) return fail(XAIE_INVALID_TILE, "tile outside the array");
  Tile& t = rt->tile(Loc);
  rc = poll_done(rt, t);
  if (rc != XAIE_CORE_STATUS_TIMEOUT || TimeOut == 0 || !t.launched) return rc;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::microseconds(TimeOut);
  while (std::chrono::steady_clock::now() < deadline) {
    rc = poll_done(rt, t);
    if (rc != XAIE_CORE_STATUS_TIMEOUT) return rc;
    std::this_thread::yield();
  }
  return XAIE_CORE_STATUS_TIMEOUT;
}

AieRC XAie_CoreReadDoneBit(XAie_DevInst* DevInst, XAie_LocType Loc, u8* DoneBit) {
  if (!DoneBit) return fail(XAIE_INVALID_ARGS, "null pointer");
  const AieRC rc = XAie_CoreWaitForDone(DevInst, Loc, 0);
  *DoneBit = rc == XAIE_OK ? 1 : 0;
  return (rc == XAIE_OK || rc == XAIE_CORE_STATUS_TIMEOUT) ? XAIE_OK : rc;
}

AieRC XAie_LoadElfMem(XAie_DevInst* DevInst, XAie_LocType Loc, const unsigned char* KernelFn) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!rt->valid_loc(Loc) || rt->is_shim(Loc)) return fail(XAIE_INVALID_TILE, "kernels load on tiles, not on the shim row");
  if (!KernelFn) return fail(XAIE_INVALID_ELF, "null kernel");
  KernelEntry k;
  if (!lookup_kernel(KernelFn, &k))
    return fail(XAIE_INVALID_ELF, "XAie_LoadElfMem: pointer is not a registered kernel (declare it with an "
                                  "AIEHLC_KERNEL_* macro or XAie_KernelRegister)");
  Tile& t = rt->tile(Loc);
  t.kernel = k;
  t.loaded = true;
  t.launched = false;
  t.args.clear();
  return XAIE_OK;
}

AieRC XAie_KernelSetArgs(XAie_DevInst* DevInst, XAie_LocType Loc, const void* Args, u32 Bytes) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!rt->valid_loc(Loc)) return fail(XAIE_INVALID_TILE, "tile outside the array");
  Tile& t = rt->tile(Loc);
  if (!t.loaded) return fail(XAIE_INVALID_TILE, "no kernel loaded on this tile");
  if (!Args && Bytes) return fail(XAIE_INVALID_ARGS, "null arguments");
  t.args.assign(static_cast<const uint8_t*>(Args), static_cast<const uint8_t*>(Args) + Bytes);
  return XAIE_OK;
}

// ---------------------------------------------------------------------------------- GMIO buffers
XAie_MemInst* XAie_MemAllocate(XAie_DevInst* DevInst, u64 Size, XAie_MemCacheProp) {
  Runtime* rt;
  if (need_rt(DevInst, &rt) != XAIE_OK) return nullptr;
  if (Size == 0) {
    fail(XAIE_INVALID_ARGS, "XAie_MemAllocate: zero size");
    return nullptr;
  }
  XAie_MemInst* m = new XAie_MemInst();
  m->rt = rt;
  m->bytes = Size;
#if defined(MAP_32BIT)
  if (Size <= (64u << 20)) {
    const size_t page = 4096;
    const size_t mb = (Size + page - 1) / page * page;
    void* p = mmap(nullptr, mb, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_32BIT, -1, 0);
    if (p != MAP_FAILED) {
      if (cudaHostRegister(p, mb, cudaHostRegisterPortable) == cudaSuccess) {
        m->host = p;
        m->map_bytes = mb;
        m->mmapped = true;
      } else {
        cudaGetLastError();
        munmap(p, mb);
      }
    }
  }
#endif
  if (!m->host) {
    cudaError_t e = cudaMallocHost(&m->host, Size);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaMallocHost");
      delete m;
      return nullptr;
    }
  }
  {
    std::lock_guard<std::mutex> lk(rt->mems_mu);
    rt->mems.push_back(m);
  }
  return m;
}

AieRC XAie_MemFree(XAie_MemInst* m) {
  if (!m) return fail(XAIE_INVALID_ARGS, "null buffer");
  Runtime* rt = m->rt;
  cudaStreamSynchronize(rt->stream);
  {
    std::lock_guard<std::mutex> lk(rt->mems_mu);
    for (size_t i = 0; i < rt->mems.size(); ++i)
      if (rt->mems[i] == m) {
        rt->mems.erase(rt->mems.begin() + i);
        break;
      }
  }
  if (m->mmapped) {
    cudaHostUnregister(m->host);
    munmap(m->host, m->map_bytes);
  } else {
    cudaFreeHost(m->host);
  }
  delete m;
  return XAIE_OK;
}

void* XAie_MemGetVAddr(XAie_MemInst* m) { return m ? m->host : nullptr; }
u64 XAie_MemGetDevAddr(XAie_MemInst* m) { return m ? reinterpret_cast<u64>(m->host) : 0; }
AieRC XAie_MemSyncForDev(XAie_MemInst* m) {
  // Pinned memory is coherent with the copy engines: nothing to flush.
  return m ? XAIE_OK : fail(XAIE_INVALID_ARGS, "null buffer");
}
AieRC XAie_MemSyncForCPU(XAie_MemInst* m) {
  if (!m) return fail(XAIE_INVALID_ARGS, "null buffer");
  XCUDA(cudaSetDevice(m->rt->device));
  if (!m->rt->capturing) XCUDA(cudaStreamSynchronize(m->rt->stream));
  return XAIE_OK;
}

// ---------------------------------------------------------------------------------- routing
XAie_RoutingInstance* XAie_InitRoutingHandler(XAie_DevInst* DevInst) {
  Runtime* rt;
  if (need_rt(DevInst, &rt) != XAIE_OK) return nullptr;
  XAie_RoutingInstance* ri = new XAie_RoutingInstance();
  ri->rt = rt;
  rt->routes.push_back(ri);
  return ri;
}

AieRC XAie_Route(XAie_RoutingInstance* ri, void*, XAie_LocType s, XAie_LocType d) {
  if (!ri) return fail(XAIE_INVALID_ARGS, "null routing instance");
  if (!ri->rt->valid_loc(s) || !ri->rt->valid_loc(d)) return fail(XAIE_INVALID_TILE, "route endpoint outside the array");
  if (loc_key(s) == loc_key(d)) return fail(XAIE_INVALID_ARGS, "route from a location to itself");
  ri->edges.emplace_back(loc_key(s), loc_key(d));
  return XAIE_OK;
}

AieRC XAie_RouteDmaWait(XAie_RoutingInstance* ri, XAie_LocType, XAie_LocType, u8) {
  if (!ri) return fail(XAIE_INVALID_ARGS, "null routing instance");
  XCUDA(cudaSetDevice(ri->rt->device));
  if (!ri->rt->capturing) XCUDA(cudaStreamSynchronize(ri->rt->stream));
  return XAIE_OK;
}

AieRC XAie_RoutingInstanceFree(XAie_RoutingInstance* ri) {
  if (!ri) return XAIE_OK;
  Runtime* rt = ri->rt;
  for (size_t i = 0; i < rt->routes.size(); ++i)
    if (rt->routes[i] == ri) {
      rt->routes.erase(rt->routes.begin() + i);
      break;
    }
  delete ri;
  return XAIE_OK;
}

// ---------------------------------------------------------------------------------- data movement
AieRC XAie_MoveDataExternal2Aie64(XAie_RoutingInstance* ri, XAie_LocType shim, XAie_MemInst* src, u64 bytes,
                                  u64 tile_addr, XAie_LocType dst) {
  if (!ri || !src) return fail(XAIE_INVALID_ARGS, "null argument");
  Runtime* rt = ri->rt;
  XCUDA(cudaSetDevice(rt->device));
  if (bytes > src->bytes) return fail(XAIE_INVALID_ARGS, "move larger than the source buffer");
  if (!edge_ok(ri, shim, dst)) return fail(XAIE_ERR, "no route from the shim location to the destination tile");
  return h2t(rt, dst, tile_addr, src->host, bytes);
}
AieRC XAie_MoveDataExternal2Aie(XAie_RoutingInstance* ri, XAie_LocType shim, XAie_MemInst* src, u32 bytes,
                                u32 tile_addr, XAie_LocType dst) {
  return XAie_MoveDataExternal2Aie64(ri, shim, src, bytes, tile_addr, dst);
}

AieRC XAie_MoveDataAie2External64(XAie_RoutingInstance* ri, XAie_LocType src, u64 tile_addr, u64 bytes,
                                  XAie_MemInst* dst, XAie_LocType shim) {
  if (!ri || !dst) return fail(XAIE_INVALID_ARGS, "null argument");
  Runtime* rt = ri->rt;
  XCUDA(cudaSetDevice(rt->device));
  if (bytes > dst->bytes) return fail(XAIE_INVALID_ARGS, "move larger than the destination buffer");
  if (!edge_ok(ri, src, shim)) return fail(XAIE_ERR, "no route from the source tile to the shim location");
  return t2h(rt, src, tile_addr, dst->host, bytes);
}
AieRC XAie_MoveDataAie2External(XAie_RoutingInstance* ri, XAie_LocType src, u32 tile_addr, u32 bytes,
                                XAie_MemInst* dst, XAie_LocType shim) {
  return XAie_MoveDataAie2External64(ri, src, tile_addr, bytes, dst, shim);
}

AieRC XAie_MoveData(XAie_RoutingInstance* ri, XAie_LocType sl, void* src, u32 bytes, void* dst, XAie_LocType dl) {
  if (!ri) return fail(XAIE_INVALID_ARGS, "null routing instance");
  Runtime* rt = ri->rt;
  XCUDA(cudaSetDevice(rt->device));
  if (!rt->valid_loc(sl) || !rt->valid_loc(dl)) return fail(XAIE_INVALID_TILE, "location outside the array");
  if (!edge_ok(ri, sl, dl)) return fail(XAIE_ERR, "no route between the two locations");
  const bool s_ext = rt->is_shim(sl), d_ext = rt->is_shim(dl);
  if (s_ext && d_ext) return fail(XAIE_INVALID_ARGS, "external to external move");
  if (s_ext) {
    if (!src) return fail(XAIE_INVALID_ARGS, "null host source");
    return h2t(rt, dl, reinterpret_cast<u64>(dst), src, bytes);
  }
  if (d_ext) {
    if (!dst) return fail(XAIE_INVALID_ARGS, "null host destination");
    return t2h(rt, sl, reinterpret_cast<u64>(src), dst, bytes);
  }
  return t2t(rt, sl, reinterpret_cast<u64>(src), dl, reinterpret_cast<u64>(dst), bytes);
}

AieRC XAie_Run(XAie_RoutingInstance* ri, u32 Count) {
  if (!ri) return fail(XAIE_INVALID_ARGS, "null routing instance");
  Runtime* rt = ri->rt;
  XCUDA(cudaSetDevice(rt->device));
  if (Count == 0) return XAIE_OK;
  bool any_armed = false, any_loaded = false;
  for (auto& kv : rt->tiles) {
    any_loaded |= kv.second.loaded && kv.second.enabled;
    any_armed |= kv.second.loaded && kv.second.enabled && kv.second.armed;
  }
  if (!any_loaded) return fail(XAIE_ERR, "XAie_Run: no kernel loaded");
  g_err.clear();
  for (auto& kv : rt->tiles) {
    Tile& t = kv.second;
    if (!t.loaded || !t.enabled) continue;
    if (any_armed && !t.armed) continue;
    AieRC rc = launch_tile(rt, t, Count);
    if (rc != XAIE_OK) return rc;
  }
  return XAIE_OK;
}

AieRC XAie_DataMemBlockRead(XAie_DevInst* DevInst, XAie_LocType Loc, u64 Addr, void* Dst, u32 Size) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!Dst) return fail(XAIE_INVALID_ARGS, "null destination");
  return t2h(rt, Loc, Addr, Dst, Size);
}
AieRC XAie_DataMemBlockWrite(XAie_DevInst* DevInst, XAie_LocType Loc, u64 Addr, const void* Src, u32 Size) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!Src) return fail(XAIE_INVALID_ARGS, "null source");
  rc = h2t(rt, Loc, Addr, Src, Size);
  if (rc != XAIE_OK) return rc;
  if (!rt->capturing) XCUDA(cudaStreamSynchronize(rt->stream));  // Src may be pageable and short-lived
  return XAIE_OK;
}

u64 XAie_LaunchCount(XAie_DevInst* DevInst) {
  Runtime* rt = rt_of(DevInst);
  return rt ? rt->launches : 0;
}

AieRC XAie_DebugInjectStatus(XAie_DevInst* DevInst, u32 Status, u32 Count) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  rt->inject_status = Status;
  rt->inject_count = Count;
  return XAIE_OK;
}

// ---------------------------------------------------------------------------------- recorded chains
// The reference drives a chain of kernels with a host round trip per stage (run, poll, move, run,
// ...: example/multi/multi_tile.cpp:105-145, seq_full_col.cpp:132-153).  The same call sequence can
// be recorded once into a CUDA graph and replayed with one launch: intermediates stay on the device,
// the host re-enters only to wait for the whole chain.
AieRC XAie_GraphBeginCapture(XAie_DevInst* DevInst) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (rt->capturing) return fail(XAIE_ERR, "a graph is already being recorded on this device instance");
  XCUDA(cudaStreamSynchronize(rt->stream));
  aiehlc_set_pdl(rt->ctx, 0);  // plain kernel nodes inside the graph
  cudaError_t e = cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeRelaxed);
  if (e != cudaSuccess) {
    aiehlc_set_pdl(rt->ctx, 1);
    return cuda_fail(e, "cudaStreamBeginCapture");
  }
  rt->capturing = true;
  return XAIE_OK;
}

AieRC XAie_GraphEndCapture(XAie_DevInst* DevInst, XAie_Graph** Out) {
  Runtime* rt;
  AieRC rc = need_rt(DevInst, &rt);
  if (rc != XAIE_OK) return rc;
  if (!Out) return fail(XAIE_INVALID_ARGS, "null graph pointer");
  *Out = nullptr;
  if (!rt->capturing) return fail(XAIE_ERR, "no graph is being recorded");
  rt->capturing = false;
  aiehlc_set_pdl(rt->ctx, 1);
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(rt->stream, &g);
  if (e != cudaSuccess || !g) return cuda_fail(e, "cudaStreamEndCapture");
  XAie_Graph* gr = new XAie_Graph();
  gr->rt = rt;
  gr->graph = g;
  gr->rt_generation = rt->generation;
  gr->ctx_generation = aiehlc_workspace_generation(rt->ctx);
  e = cudaGraphInstantiate(&gr->exec, g, 0);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&gr->done, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaGraphInstantiate");
    if (gr->exec) cudaGraphExecDestroy(gr->exec);
    cudaGraphDestroy(g);
    delete gr;
    return XAIE_ERR_DEVICE;
  }
  *Out = gr;
  return XAIE_OK;
}

AieRC XAie_GraphLaunch(XAie_Graph* Graph) {
  if (!Graph) return fail(XAIE_INVALID_ARGS, "null graph");
  Runtime* rt = Graph->rt;
  XCUDA(cudaSetDevice(rt->device));
  if (rt->capturing) return fail(XAIE_ERR, "cannot launch a graph while another one is being recorded");
  if (Graph->rt_generation != rt->generation || Graph->ctx_generation != aiehlc_workspace_generation(rt->ctx))
    return fail(XAIE_ERR, "graph is stale: a tile window or a workspace it recorded has since moved to a larger "
                          "allocation; record it again");
  XCUDA(cudaGraphLaunch(Graph->exec, rt->stream));
  XCUDA(cudaEventRecord(Graph->done, rt->stream));
  Graph->launched = true;
  return XAIE_OK;
}

AieRC XAie_GraphWait(XAie_Graph* Graph, u32 TimeOut) {
  if (!Graph) return fail(XAIE_INVALID_ARGS, "null graph");
  if (!Graph->launched) return fail(XAIE_CORE_STATUS_TIMEOUT, "graph has not been launched");
  Runtime* rt = Graph->rt;
  XCUDA(cudaSetDevice(rt->device));
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::microseconds(TimeOut);
  for (;;) {
    cudaError_t e = cudaEventQuery(Graph->done);
    if (e == cudaSuccess) break;
    if (e != cudaErrorNotReady) return cuda_fail(e, "cudaEventQuery");
    if (TimeOut == 0 || std::chrono::steady_clock::now() >= deadline) return XAIE_CORE_STATUS_TIMEOUT;
    std::this_thread::yield();
  }
  int status = 0;
  if (aiehlc_sync(rt->ctx, rt->stream, &status) != AIEHLC_OK)
    return fail(XAIE_ERR_DEVICE, status ? "kernel status word = " + std::to_string(status) : std::string(aiehlc_last_error()));
  return XAIE_OK;
}

AieRC XAie_GraphDestroy(XAie_Graph* Graph) {
  if (!Graph) return XAIE_OK;
  cudaSetDevice(Graph->rt->device);
  cudaStreamSynchronize(Graph->rt->stream);
  if (Graph->exec) cudaGraphExecDestroy(Graph->exec);
  if (Graph->graph) cudaGraphDestroy(Graph->graph);
  if (Graph->done) cudaEventDestroy(Graph->done);
  delete Graph;
  return XAIE_OK;
}

// ---------------------------------------------------------------------------------- kernel-call form
// k<Col,Row,colstart,rowstart,M,N,K>(in, out) -- example/nokernelload/aie_nokernelload.cc:130; the
// compiler declares the template (src/llvm/aiehlc.cc:583-588) but lowers it to nothing.  Here the
// call is the whole load / move-in / run / wait / move-out sequence on tile (colstart,rowstart):
// `in` and `out` are addresses inside GMIO buffers (what XAie_MemGetDevAddr returns).
static XAie_MemInst* find_mem(Runtime* rt, u64 addr, u64* offset) {
  std::lock_guard<std::mutex> lk(rt->mems_mu);
  for (XAie_MemInst* m : rt->mems) {
    const u64 base = reinterpret_cast<u64>(m->host);
    if (addr >= base && addr < base + m->bytes) {
      *offset = addr - base;
      return m;
    }
  }
  return nullptr;
}

AieRC XAie_KernelCall(const void* kernel_key, const void* args, u32 args_bytes, int Col, int Row, int colstart,
                      int rowstart, u64 in_addr, u64 out_addr) {
  // the instance that owns the input buffer; the calling thread's own instance is tried first
  Runtime* rt = nullptr;
  {
    u64 off0 = 0;
    if (g_current_rt && find_mem(g_current_rt, in_addr, &off0)) rt = g_current_rt;
    if (!rt) {
      std::lock_guard<std::mutex> lk(g_runtimes_mu);
      for (Runtime* r : g_runtimes)
        if (find_mem(r, in_addr, &off0)) { rt = r; break; }
    }
  }
  if (!rt) {
    if (!g_current_rt) return fail(XAIE_INVALID_DEVICE, "kernel call before XAie_CfgInitialize");
    return fail(XAIE_INVALID_ADDRESS, "kernel call: input address is not inside a GMIO buffer");
  }
  XCUDA(cudaSetDevice(rt->device));
  if (Col < 1 || Row < 1) return fail(XAIE_INVALID_ARGS, "kernel call: Col and Row must be at least 1");
  const XAie_LocType loc = XAie_TileLoc(static_cast<u8>(colstart), static_cast<u8>(rowstart));
  if (colstart < 0 || rowstart < 0 || !rt->valid_loc(loc) || rt->is_shim(loc))
    return fail(XAIE_INVALID_TILE, "kernel call: (colstart,rowstart) is not a tile of the array");
  AieRC rc = XAie_LoadElfMem(rt->dev, loc, static_cast<const unsigned char*>(kernel_key));
  if (rc != XAIE_OK) return rc;
  if (args && args_bytes) {
    rc = XAie_KernelSetArgs(rt->dev, loc, args, args_bytes);
    if (rc != XAIE_OK) return rc;
  }
  Tile& t = rt->tile(loc);
  u64 off = 0;
  XAie_MemInst* min = find_mem(rt, in_addr, &off);
  if (!min) return fail(XAIE_INVALID_ADDRESS, "kernel call: input address is not inside a GMIO buffer");
  rc = h2t(rt, loc, t.kernel.in_addr, static_cast<const uint8_t*>(min->host) + off, min->bytes - off);
  if (rc != XAIE_OK) return rc;
  XAie_MemInst* mout = find_mem(rt, out_addr, &off);
  if (!mout) return fail(XAIE_INVALID_ADDRESS, "kernel call: output address is not inside a GMIO buffer");
  g_err.clear();
  // Col x Row tiles of the array become Col x Row SMs: the persistent GEMM kernels plan their tile
  // shape and waves for that many and occupy no more (a grid larger than the GPU means all of it)
  const long long grid_sms = static_cast<long long>(Col) * Row;
  aiehlc_set_cta_limit(rt->ctx, grid_sms > 0x7FFFFFFF ? 0 : static_cast<int>(grid_sms));
  rc = launch_tile(rt, t, 1);
  aiehlc_set_cta_limit(rt->ctx, 0);
  if (rc != XAIE_OK) return rc;
  Region* r = rt->find_region(t, t.kernel.out_addr, 1);
  if (!r) return fail(XAIE_INVALID_ADDRESS, "kernel call: kernel produced no output window");
  u64 n = t.out_bytes;   // what this launch produced, not the window's capacity
  if (n > mout->bytes - off) n = mout->bytes - off;
  rc = t2h(rt, loc, t.kernel.out_addr, static_cast<uint8_t*>(mout->host) + off, n);  // waits for the stream
  if (rc != XAIE_OK) return rc;
  int status = 0;
  if (aiehlc_sync(rt->ctx, rt->stream, &status) != AIEHLC_OK) return fail(XAIE_ERR_DEVICE, aiehlc_last_error());
  return XAIE_OK;
}

// ---------------------------------------------------------------- the short host API (xaie_placeholder.h)
}  // extern "C"

struct XAie_Kernel_Inst {
  Runtime* rt = nullptr;
  XAie_LocType loc{};
  XAie_RoutingInstance* ri = nullptr;
  XAie_LocType shim_in{}, shim_out{};
  bool has_in = false, has_out = false;
};

namespace {
// The device instance behind XAie_LoadKernel when the program has not initialised one itself:
// the array of example/other/aieoob.c:8-19.
thread_local XAie_DevInst g_implicit_dev;
bool lookup_kernel_by_name(const char* name, const void** key) {
  seed_library_kernels();
  Registry& r = registry();
  std::lock_guard<std::mutex> lk(r.mu);
  for (auto& kv : r.map)
    if (kv.second.name == name) {
      *key = kv.first;
      return true;
    }
  return false;
}
}  // namespace

extern "C" {

XAie_Kernel_Inst* XAie_LoadKernel(const char* name, int col, int row) {
  if (!name) {
    fail(XAIE_INVALID_ARGS, "XAie_LoadKernel: null kernel name");
    return nullptr;
  }
  const void* key = nullptr;
  if (!lookup_kernel_by_name(name, &key)) {
    fail(XAIE_INVALID_ELF, std::string("XAie_LoadKernel: no kernel registered under the name '") + name + "'");
    return nullptr;
  }
  if (!g_current_rt) {
    XAie_Config cfg = {2, 0x20000000000ull, 25, 20, 11, 38, 0, 1, 2, 3, 8};
    if (XAie_CfgInitialize(&g_implicit_dev, &cfg) != XAIE_OK) return nullptr;
  }
  Runtime* rt = g_current_rt;
  if (col < 0 || row < 0 || col > 255 || row > 255) {
    fail(XAIE_INVALID_TILE, "XAie_LoadKernel: tile outside the array");
    return nullptr;
  }
  const XAie_LocType loc = XAie_TileLoc(static_cast<u8>(col), static_cast<u8>(row));
  if (XAie_LoadElfMem(rt->dev, loc, static_cast<const unsigned char*>(key)) != XAIE_OK) return nullptr;
  XAie_Kernel_Inst* k = new XAie_Kernel_Inst();
  k->rt = rt;
  k->loc = loc;
  k->ri = XAie_InitRoutingHandler(rt->dev);
  if (!k->ri) {
    delete k;
    return nullptr;
  }
  return k;
}

AieRC XAie_RoutingHostToAie(XAie_Kernel_Inst* k, XAie_LocType shim) {
  if (!k) return fail(XAIE_INVALID_ARGS, "null kernel instance");
  if (!k->rt->valid_loc(shim) || !k->rt->is_shim(shim)) return fail(XAIE_INVALID_TILE, "host data enters through a shim tile");
  const AieRC rc = XAie_Route(k->ri, nullptr, shim, k->loc);
  if (rc == XAIE_OK) { k->shim_in = shim; k->has_in = true; }
  return rc;
}

AieRC XAie_RoutingAieToHost(XAie_Kernel_Inst* k, XAie_LocType shim) {
  if (!k) return fail(XAIE_INVALID_ARGS, "null kernel instance");
  if (!k->rt->valid_loc(shim) || !k->rt->is_shim(shim)) return fail(XAIE_INVALID_TILE, "results leave through a shim tile");
  const AieRC rc = XAie_Route(k->ri, nullptr, k->loc, shim);
  if (rc == XAIE_OK) { k->shim_out = shim; k->has_out = true; }
  return rc;
}

AieRC XAie_MoveDataToAie(XAie_Kernel_Inst* k, int port, const void* src, size_t bytes) {
  if (!k || (!src && bytes)) return fail(XAIE_INVALID_ARGS, "XAie_MoveDataToAie: null argument");
  if (port != 1) return fail(XAIE_INVALID_ARGS, "XAie_MoveDataToAie: the kernels have one input port (1)");
  if (!k->has_in) return fail(XAIE_ERR, "XAie_MoveDataToAie: no host-to-tile route declared (XAie_RoutingHostToAie)");
  XCUDA(cudaSetDevice(k->rt->device));
  return h2t(k->rt, k->loc, k->rt->tile(k->loc).kernel.in_addr, src, bytes);
}

AieRC XAie_RunCore(XAie_Kernel_Inst* k) {
  if (!k) return fail(XAIE_INVALID_ARGS, "null kernel instance");
  XCUDA(cudaSetDevice(k->rt->device));
  g_err.clear();
  return launch_tile(k->rt, k->rt->tile(k->loc), 1);
}

AieRC XAie_WaitOutData(XAie_Kernel_Inst* k) {
  if (!k) return fail(XAIE_INVALID_ARGS, "null kernel instance");
  return XAie_CoreWaitForDone(k->rt->dev, k->loc, 10u * 1000u * 1000u);
}

AieRC XAie_MoveAieToData(XAie_Kernel_Inst* k, int port, void* dst, size_t bytes) {
  if (!k || (!dst && bytes)) return fail(XAIE_INVALID_ARGS, "XAie_MoveAieToData: null argument");
  if (port != 1) return fail(XAIE_INVALID_ARGS, "XAie_MoveAieToData: the kernels have one output port (1)");
  if (!k->has_out) return fail(XAIE_ERR, "XAie_MoveAieToData: no tile-to-host route declared (XAie_RoutingAieToHost)");
  XCUDA(cudaSetDevice(k->rt->device));
  return t2h(k->rt, k->loc, k->rt->tile(k->loc).kernel.out_addr, dst, bytes);
}

AieRC XAie_KernelInstSetArgs(XAie_Kernel_Inst* k, const void* args, u32 bytes) {
  if (!k) return fail(XAIE_INVALID_ARGS, "null kernel instance");
  return XAie_KernelSetArgs(k->rt->dev, k->loc, args, bytes);
}

void XAie_UnloadKernel(XAie_Kernel_Inst* k) {
  if (!k) return;
  XAie_RoutingInstanceFree(k->ri);
  delete k;
}

// ---------------------------------------------------------------------------------- registry API
AieRC XAie_KernelRegister(const void* key, const XAie_KernelDesc* d) {
  if (!key || !d || !d->launch) return fail(XAIE_INVALID_ARGS, "XAie_KernelRegister: null key or launch function");
  KernelEntry k;
  k.name = d->name ? d->name : "kernel";
  k.launch = d->launch;
  k.out_bytes = d->out_bytes;
  k.out_bytes_default = d->out_bytes_default;
  k.in_addr = d->in_addr;
  k.out_addr = d->out_addr;
  k.acc_addr = d->acc_addr;
  if (d->default_args && d->default_args_bytes)
    k.default_args.assign(static_cast<const uint8_t*>(d->default_args),
                          static_cast<const uint8_t*>(d->default_args) + d->default_args_bytes);
  k.user = d->user;
  Registry& r = registry();
  std::lock_guard<std::mutex> lk(r.mu);
  r.map[key] = k;
  return XAIE_OK;
}

AieRC XAie_KernelBind(const void* key, const char* name, const void* library_kernel, const void* args,
                      u32 args_bytes, u32 in_addr, u32 out_addr, u32 acc_addr) {
  KernelEntry base;
  if (!key || !lookup_kernel(library_kernel, &base))
    return fail(XAIE_INVALID_ARGS, "XAie_KernelBind: unknown library kernel");
  base.name = name ? name : base.name;
  if (args && args_bytes)
    base.default_args.assign(static_cast<const uint8_t*>(args), static_cast<const uint8_t*>(args) + args_bytes);
  base.in_addr = in_addr;
  base.out_addr = out_addr;
  base.acc_addr = acc_addr;
  Registry& r = registry();
  std::lock_guard<std::mutex> lk(r.mu);
  r.map[key] = base;
  return XAIE_OK;
}

// ---------------------------------------------------------------------------------- library kernels
static u64 align16(u64 v) { return (v + 15) & ~static_cast<u64>(15); }

u64 aiehlc_window_offset_b(const XAie_GemmArgs* a, u32 eb) { return align16(static_cast<u64>(a->M) * a->K * eb); }
u64 aiehlc_window_offset_shift(const XAie_GemmArgs* a, u32 eb) {
  return align16(aiehlc_window_offset_b(a, eb) + static_cast<u64>(a->N) * a->K * eb);
}
u64 aiehlc_conv_offset_w(const XAie_ConvArgs* a) { return align16(static_cast<u64>(a->n) * a->h * a->w * a->cin); }
u64 aiehlc_conv_offset_shift(const XAie_ConvArgs* a) {
  return align16(aiehlc_conv_offset_w(a) + static_cast<u64>(a->kh) * a->kw * a->cin * a->cout);
}

// Host-side symbols whose addresses name the kernels; they are never called.
void aiehlc_k_mm_i32(input_window_int32*, output_window_int32*) {}
void aiehlc_k_gemm_i8_i32(const s8*, s32*) {}
void aiehlc_k_gemm_i8_srs(const s8*, s8*) {}
void aiehlc_k_gemm_bf16(const u16*, u16*) {}
void aiehlc_k_conv2d_i8_srs(const s8*, s8*) {}
void aiehlc_k_srs_i32_i8(const s32*, s8*) {}

}  // extern "C"

namespace {

template <typename T>
const T* args_as(const XAie_KernelLaunchInfo* i) {
  if (i->args_bytes < sizeof(T) || !i->args) {
    g_err = "kernel arguments missing or too short (XAie_KernelSetArgs)";
    return nullptr;
  }
  return static_cast<const T*>(i->args);
}
int need_in(const XAie_KernelLaunchInfo* i, u64 bytes) {
  if (!i->in || i->in_bytes < bytes) {
    g_err = "input window holds " + std::to_string(i->in_bytes) + " bytes, kernel needs " + std::to_string(bytes);
    return 1;
  }
  return 0;
}
int from_capi(int rc) {
  if (rc != AIEHLC_OK) g_err = aiehlc_last_error();
  return rc;
}

int k_mm_i32(const XAie_KernelLaunchInfo* i) {
  auto* a = args_as<XAie_MmArgs>(i);
  if (!a) return 1;
  if (need_in(i, (static_cast<u64>(a->M) + a->N) * a->K * 4)) return 1;
  return from_capi(aiehlc_mm_i32_dev(static_cast<aiehlc_ctx*>(i->ctx), static_cast<const int32_t*>(i->in),
                                     static_cast<int32_t*>(i->out), a->M, a->N, a->K, i->stream));
}
u64 ob_mm_i32(const void* args, u32 n, u64, void*) {
  if (n < sizeof(XAie_MmArgs)) return 0;
  auto* a = static_cast<const XAie_MmArgs*>(args);
  return static_cast<u64>(a->M) * a->N * 4;
}

int k_gemm_i8_i32(const XAie_KernelLaunchInfo* i) {
  auto* a = args_as<XAie_GemmArgs>(i);
  if (!a) return 1;
  const u64 ob = aiehlc_window_offset_b(a, 1);
  if (need_in(i, ob + static_cast<u64>(a->N) * a->K)) return 1;
  const int8_t* base = static_cast<const int8_t*>(i->in);
  return from_capi(aiehlc_gemm_i8_i32_dev(static_cast<aiehlc_ctx*>(i->ctx), base, base + ob,
                                          static_cast<int32_t*>(i->out), a->M, a->N, a->K, a->accumulate, i->stream));
}
u64 ob_gemm_i32(const void* args, u32 n, u64, void*) {
  if (n < sizeof(XAie_GemmArgs)) return 0;
  auto* a = static_cast<const XAie_GemmArgs*>(args);
  return static_cast<u64>(a->M) * a->N * 4;
}

int k_gemm_i8_srs(const XAie_KernelLaunchInfo* i) {
  auto* a = args_as<XAie_GemmArgs>(i);
  if (!a) return 1;
  const u64 ob = aiehlc_window_offset_b(a, 1), os = aiehlc_window_offset_shift(a, 1);
  if (need_in(i, a->has_shift_vec ? os + a->N : ob + static_cast<u64>(a->N) * a->K)) return 1;
  const int8_t* base = static_cast<const int8_t*>(i->in);
  const int32_t* acc = nullptr;
  if (a->use_acc) {
    if (!i->acc || i->acc_bytes < static_cast<u64>(a->M) * a->N * 4) {
      g_err = "gemm_i8_srs: accumulator window missing or too small";
      return 1;
    }
    acc = static_cast<const int32_t*>(i->acc);
  }
  return from_capi(aiehlc_gemm_i8_srs_dev(
      static_cast<aiehlc_ctx*>(i->ctx), base, base + ob, static_cast<int8_t*>(i->out), a->M, a->N, a->K, a->shift,
      a->has_shift_vec ? reinterpret_cast<const uint8_t*>(base + os) : nullptr, acc, a->splitk < 1 ? 1 : a->splitk,
      i->stream));
}
u64 ob_gemm_i8(const void* args, u32 n, u64, void*) {
  if (n < sizeof(XAie_GemmArgs)) return 0;
  auto* a = static_cast<const XAie_GemmArgs*>(args);
  return static_cast<u64>(a->M) * a->N;
}

int k_gemm_bf16(const XAie_KernelLaunchInfo* i) {
  auto* a = args_as<XAie_GemmArgs>(i);
  if (!a) return 1;
  const u64 ob = aiehlc_window_offset_b(a, 2);
  if (need_in(i, ob + static_cast<u64>(a->N) * a->K * 2)) return 1;
  const uint8_t* base = static_cast<const uint8_t*>(i->in);
  return from_capi(aiehlc_gemm_bf16_dev(static_cast<aiehlc_ctx*>(i->ctx), reinterpret_cast<const uint16_t*>(base),
                                        reinterpret_cast<const uint16_t*>(base + ob), static_cast<uint16_t*>(i->out),
                                        a->M, a->N, a->K, i->stream));
}
u64 ob_gemm_bf16(const void* args, u32 n, u64, void*) {
  if (n < sizeof(XAie_GemmArgs)) return 0;
  auto* a = static_cast<const XAie_GemmArgs*>(args);
  return static_cast<u64>(a->M) * a->N * 2;
}

int k_conv(const XAie_KernelLaunchInfo* i) {
  auto* a = args_as<XAie_ConvArgs>(i);
  if (!a) return 1;
  const u64 ow = aiehlc_conv_offset_w(a), os = aiehlc_conv_offset_shift(a);
  if (need_in(i, os + a->cout)) return 1;
  const int8_t* base = static_cast<const int8_t*>(i->in);
  return from_capi(aiehlc_conv2d_i8_srs_dev(static_cast<aiehlc_ctx*>(i->ctx), base, base + ow,
                                            static_cast<int8_t*>(i->out), a->n, a->h, a->w, a->cin, a->cout, a->kh,
                                            a->kw, a->pad, reinterpret_cast<const uint8_t*>(base + os), i->stream));
}
u64 ob_conv(const void* args, u32 n, u64, void*) {
  if (n < sizeof(XAie_ConvArgs)) return 0;
  auto* a = static_cast<const XAie_ConvArgs*>(args);
  return static_cast<u64>(a->n) * a->h * a->w * a->cout;
}

int k_srs(const XAie_KernelLaunchInfo* i) {
  auto* a = args_as<XAie_SrsArgs>(i);
  if (!a) return 1;
  const u64 nb = align16(static_cast<u64>(a->rows) * a->cols * 4);
  if (need_in(i, a->has_shift_vec ? nb + a->cols : static_cast<u64>(a->rows) * a->cols * 4)) return 1;
  const uint8_t* base = static_cast<const uint8_t*>(i->in);
  return from_capi(aiehlc_srs_i32_i8_dev(static_cast<aiehlc_ctx*>(i->ctx), reinterpret_cast<const int32_t*>(base),
                                         static_cast<int8_t*>(i->out), a->rows, a->cols, a->shift,
                                         a->has_shift_vec ? base + nb : nullptr, i->stream));
}
u64 ob_srs(const void* args, u32 n, u64, void*) {
  if (n < sizeof(XAie_SrsArgs)) return 0;
  auto* a = static_cast<const XAie_SrsArgs*>(args);
  return static_cast<u64>(a->rows) * a->cols;
}

void seed_library_kernels() {
  static std::once_flag once;
  std::call_once(once, [] {
    static const XAie_MmArgs mm16 = {16, 16, 16};  // the reference's fixed tile (aieml_perf.cc:55-56)
    struct Row {
      const void* key; const char* name; XAie_KernelLaunchFn fn; XAie_KernelOutBytesFn ob;
      const void* da; u32 dab; u32 acc;
    };
    const Row rows[] = {
        {reinterpret_cast<const void*>(aiehlc_k_mm_i32), "mm_i32", k_mm_i32, ob_mm_i32, &mm16, sizeof mm16, 0},
        {reinterpret_cast<const void*>(aiehlc_k_gemm_i8_i32), "gemm_i8_i32", k_gemm_i8_i32, ob_gemm_i32, nullptr, 0, 0},
        {reinterpret_cast<const void*>(aiehlc_k_gemm_i8_srs), "gemm_i8_srs", k_gemm_i8_srs, ob_gemm_i8, nullptr, 0, 0x3000},
        {reinterpret_cast<const void*>(aiehlc_k_gemm_bf16), "gemm_bf16", k_gemm_bf16, ob_gemm_bf16, nullptr, 0, 0},
        {reinterpret_cast<const void*>(aiehlc_k_conv2d_i8_srs), "conv2d_i8_srs", k_conv, ob_conv, nullptr, 0, 0},
        {reinterpret_cast<const void*>(aiehlc_k_srs_i32_i8), "srs_i32_i8", k_srs, ob_srs, nullptr, 0, 0},
    };
    for (const Row& r : rows) {
      XAie_KernelDesc d{};
      d.name = r.name;
      d.launch = r.fn;
      d.out_bytes = r.ob;
      d.in_addr = 0x1000;
      d.out_addr = 0x6000;
      d.acc_addr = r.acc;
      d.default_args = r.da;
      d.default_args_bytes = r.dab;
      XAie_KernelRegister(r.key, &d);
    }
  });
}

}  // namespace
