// CPU stand-in for the aie-rt driver, used ONLY to run the aiehlc reference's own example
// programs (their AIE kernels and their in-file golden checks) on the host, so that the oracle can
// be pinned against what the reference itself computes.  TEST INFRASTRUCTURE: never linked into
// libaiehlc_b200.so and never used by the product.
//
// The reference's kernels are plain C that addresses tile data memory at fixed addresses
// (0x70000 + window address: example/perf/aieml_perf.cc:70-71; the compiler places windows at
// 0x70000 + address, src/mlir/mlirfront/mlirpass/aiehybrid.cc:83-88).  The emulator maps 64 KiB at
// 0x70000, copies a tile's data memory in, calls the kernel function the example passed to
// XAie_LoadElfMem, and copies the memory back.  Window arguments default to 0x1000 (input) and
// 0x5000 (output), the compiler's defaults (src/mlir/mlirfront/AieFrontEnd.cc:307,351-367).
//
// Set AIEHLC_REF_DUMP=<file> to append every tile -> external transfer to <file> (raw bytes).
#include <sys/mman.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <vector>

#include "xaiengine.h"

namespace {
constexpr uintptr_t kWindowBase = 0x70000;
constexpr size_t kTileMem = 0x10000;
typedef void (*KernelFn)(void*, void*);

struct Tile {
  std::vector<uint8_t> mem = std::vector<uint8_t>(kTileMem, 0);
  KernelFn fn = nullptr;
  bool armed = false, done = false;
};
struct State {
  XAie_DevInst* dev = nullptr;
  std::map<int, Tile> tiles;
  void* window = nullptr;
};
State g;

int key(XAie_LocType l) { return (l.Col << 8) | l.Row; }
bool shim(XAie_LocType l) { return l.Row == g.dev->Cfg.ShimRowNum; }

void dump(const void* p, size_t n) {
  const char* path = getenv("AIEHLC_REF_DUMP");
  if (!path) return;
  FILE* f = fopen(path, "ab");
  if (!f) return;
  fwrite(p, 1, n, f);
  fclose(f);
}
bool in_tile(u64 addr, u64 bytes) { return addr + bytes <= kTileMem; }
}  // namespace

struct XAie_MemInst { void* host; size_t bytes; };
struct XAie_RoutingInstance { int unused; };

extern "C" {
const char* XAie_LastError(void) { return ""; }
AieRC XAie_SetupPartitionConfig(XAie_DevInst* d, u64 b, u8 s, u8 n) { d->PartBaseAddr = b; d->StartCol = s; d->PartNumCols = n; return XAIE_OK; }
AieRC XAie_CfgInitialize(XAie_DevInst* d, XAie_Config* c) {
  d->Cfg = *c;
  d->IsReady = 1;
  d->Backend = &d->BackendStorage;
  g.dev = d;
  if (!g.window) {
    void* p = mmap(reinterpret_cast<void*>(kWindowBase), kTileMem, PROT_READ | PROT_WRITE,
                   MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED_NOREPLACE, -1, 0);
    if (p != reinterpret_cast<void*>(kWindowBase)) {
      fprintf(stderr, "emulator: cannot map the tile window at 0x70000\n");
      return XAIE_ERR;
    }
    g.window = p;
  }
  return XAIE_OK;
}
AieRC XAie_SetIOBackend(XAie_DevInst* d, XAie_BackendType t) { d->BackendStorage.Type = t; return XAIE_OK; }
AieRC XAie_UpdateNpiAddr(XAie_DevInst*, u64) { return XAIE_OK; }
AieRC XAie_PartitionInitialize(XAie_DevInst*, void*) { return XAIE_OK; }
AieRC XAie_PartitionTeardown(XAie_DevInst*) { return XAIE_OK; }
AieRC XAie_PmRequestTiles(XAie_DevInst*, XAie_LocType*, u32) { return XAIE_OK; }
AieRC XAie_CoreReset(XAie_DevInst*, XAie_LocType l) { g.tiles[key(l)].done = false; return XAIE_OK; }
AieRC XAie_CoreUnreset(XAie_DevInst*, XAie_LocType) { return XAIE_OK; }
AieRC XAie_CoreEnable(XAie_DevInst*, XAie_LocType) { return XAIE_OK; }
AieRC XAie_CoreDisable(XAie_DevInst*, XAie_LocType) { return XAIE_OK; }
AieRC XAie_CoreGetStatus(XAie_DevInst* d, XAie_LocType l, u32* s) {
  *s = (l.Row >= d->Cfg.AieTileRowStart && l.Row < d->Cfg.AieTileRowStart + d->Cfg.AieTileNumRows) ? 1 : 0;
  return XAIE_OK;
}
AieRC XAie_CoreWaitForDone(XAie_DevInst*, XAie_LocType l, u32) {
  return g.tiles[key(l)].done ? XAIE_OK : XAIE_CORE_STATUS_TIMEOUT;
}
AieRC XAie_CoreReadDoneBit(XAie_DevInst*, XAie_LocType l, u8* b) { *b = g.tiles[key(l)].done; return XAIE_OK; }
AieRC XAie_LoadElfMem(XAie_DevInst*, XAie_LocType l, const unsigned char* fn) {
  Tile& t = g.tiles[key(l)];
  t.fn = reinterpret_cast<KernelFn>(const_cast<unsigned char*>(fn));
  t.done = false;
  return XAIE_OK;
}
XAie_MemInst* XAie_MemAllocate(XAie_DevInst*, u64 size, XAie_MemCacheProp) {
  const size_t mb = (size + 4095) / 4096 * 4096;
  void* p = mmap(nullptr, mb, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_32BIT, -1, 0);
  if (p == MAP_FAILED) return nullptr;
  return new XAie_MemInst{p, static_cast<size_t>(size)};
}
void* XAie_MemGetVAddr(XAie_MemInst* m) { return m->host; }
u64 XAie_MemGetDevAddr(XAie_MemInst* m) { return reinterpret_cast<u64>(m->host); }
AieRC XAie_MemSyncForDev(XAie_MemInst*) { return XAIE_OK; }
AieRC XAie_MemSyncForCPU(XAie_MemInst*) { return XAIE_OK; }
XAie_RoutingInstance* XAie_InitRoutingHandler(XAie_DevInst*) { return new XAie_RoutingInstance{0}; }
AieRC XAie_Route(XAie_RoutingInstance*, void*, XAie_LocType, XAie_LocType) { return XAIE_OK; }
AieRC XAie_RouteDmaWait(XAie_RoutingInstance*, XAie_LocType, XAie_LocType, u8) { return XAIE_OK; }

static AieRC to_tile(XAie_LocType l, u64 addr, const void* src, u64 bytes) {
  if (!in_tile(addr, bytes)) return XAIE_INVALID_ADDRESS;
  Tile& t = g.tiles[key(l)];
  memcpy(t.mem.data() + addr, src, bytes);
  t.armed = true;
  return XAIE_OK;
}
static AieRC from_tile(XAie_LocType l, u64 addr, void* dst, u64 bytes) {
  if (!in_tile(addr, bytes)) return XAIE_INVALID_ADDRESS;
  memcpy(dst, g.tiles[key(l)].mem.data() + addr, bytes);
  dump(dst, bytes);
  return XAIE_OK;
}
AieRC XAie_MoveDataExternal2Aie(XAie_RoutingInstance*, XAie_LocType, XAie_MemInst* src, u32 bytes, u32 addr, XAie_LocType dst) {
  return to_tile(dst, addr, src->host, bytes);
}
AieRC XAie_MoveDataAie2External(XAie_RoutingInstance*, XAie_LocType src, u32 addr, u32 bytes, XAie_MemInst* dst, XAie_LocType) {
  return from_tile(src, addr, dst->host, bytes);
}
AieRC XAie_MoveData(XAie_RoutingInstance*, XAie_LocType sl, void* src, u32 bytes, void* dst, XAie_LocType dl) {
  if (shim(sl)) return to_tile(dl, reinterpret_cast<u64>(dst), src, bytes);
  if (shim(dl)) return from_tile(sl, reinterpret_cast<u64>(src), dst, bytes);
  const u64 sa = reinterpret_cast<u64>(src), da = reinterpret_cast<u64>(dst);
  if (!in_tile(sa, bytes) || !in_tile(da, bytes)) return XAIE_INVALID_ADDRESS;
  std::vector<uint8_t> tmp(g.tiles[key(sl)].mem.begin() + sa, g.tiles[key(sl)].mem.begin() + sa + bytes);
  Tile& t = g.tiles[key(dl)];
  memcpy(t.mem.data() + da, tmp.data(), bytes);
  t.armed = true;
  return XAIE_OK;
}
AieRC XAie_Run(XAie_RoutingInstance*, u32 count) {
  bool any_armed = false;
  for (auto& kv : g.tiles) any_armed |= kv.second.fn && kv.second.armed;
  for (auto& kv : g.tiles) {
    Tile& t = kv.second;
    if (!t.fn || (any_armed && !t.armed)) continue;
    for (u32 i = 0; i < count; ++i) {
      memcpy(g.window, t.mem.data(), kTileMem);
      t.fn(reinterpret_cast<void*>(kWindowBase + 0x1000), reinterpret_cast<void*>(kWindowBase + 0x5000));
      memcpy(t.mem.data(), g.window, kTileMem);
    }
    t.armed = false;
    t.done = true;
  }
  return XAIE_OK;
}
AieRC XAie_DataMemBlockRead(XAie_DevInst*, XAie_LocType l, u64 addr, void* dst, u32 size) {
  if (!in_tile(addr, size)) return XAIE_INVALID_ADDRESS;
  memcpy(dst, g.tiles[key(l)].mem.data() + addr, size);
  return XAIE_OK;
}
AieRC XAie_DataMemBlockWrite(XAie_DevInst*, XAie_LocType l, u64 addr, const void* src, u32 size) {
  if (!in_tile(addr, size)) return XAIE_INVALID_ADDRESS;
  memcpy(g.tiles[key(l)].mem.data() + addr, src, size);
  return XAIE_OK;
}
}  // extern "C"
