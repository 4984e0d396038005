// Per-device context behind the C ABI: stream, status word, grow-only device workspaces.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/aiehlc_b200.h"

namespace aiehlc {

void set_error(const std::string& msg);
int fail(int rc, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

#define AIEHLC_CUDA(call)                                         \
  do {                                                            \
    cudaError_t e__ = (call);                                     \
    if (e__ != cudaSuccess) return ::aiehlc::cuda_fail(e__, #call); \
  } while (0)

// A device buffer that only ever grows (cudaMalloc on demand, freed with the context).
struct DevBuf {
  void* ptr = nullptr;
  size_t bytes = 0;
  unsigned long long* generation = nullptr;  // bumped whenever the buffer moves (see aiehlc_ctx::workspace_generation)
  int reserve(size_t need);
  void release();
};

// Raises the dynamic shared-memory limit of kernel `func` on `device` to at least `bytes`.  The limit
// belongs to the device and the function, not to a context, and a launch that needs more than the
// current value fails: it is therefore kept in one process-wide table and only ever raised.
// `cached` is the caller's own copy of the value (fast path: no lock once it is large enough).
int ensure_dynamic_smem(int device, const void* func, int bytes, int* cached);

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace aiehlc

namespace aiehlc {
// What has been established once per kernel function on this context's device.
struct KernelSetup {
  int smem_attr = 0;     // dynamic shared memory limit already raised to this many bytes
  int max_clusters = 0;  // co-resident clusters of the persistent pair kernel (0 = not queried)
};
}  // namespace aiehlc

struct aiehlc_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t stream = nullptr;   // uploads and kernels of the *_host entry points
  cudaStream_t stream2 = nullptr;  // their downloads, overlapped with the next block's upload
  cudaStream_t stream_up = nullptr;  // their uploads, back to back whatever the kernels do
  std::vector<cudaEvent_t> block_ev;  // per row block of a host GEMM: "rows uploaded", "kernel done"
  int block_events(int block, cudaEvent_t* up, cudaEvent_t* done) {
    while (block_ev.size() < 2 * static_cast<size_t>(block + 1)) {
      cudaEvent_t ev = nullptr;
      if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return AIEHLC_ERR_CUDA;
      block_ev.push_back(ev);
    }
    *up = block_ev[2 * block];
    *done = block_ev[2 * block + 1];
    return AIEHLC_OK;
  }
  cudaEvent_t block_done = nullptr;
  int* d_status = nullptr;      // device status word
  int* h_status = nullptr;      // pinned mirror
  aiehlc::EncodeTiledFn encode = nullptr;
  int force_tile_n = 0;
  int pair_mode = -1;           // -1: choose per shape, 0: single-CTA tiles only, 1: CTA pairs wherever M > 128
  int k_per_load = 0;           // 0: choose, 1: one 128-byte K block per tile load, 2: two where K allows
  int epi_groups = 0;           // groups of four epilogue warps in the CTA-pair kernel (1 or 2; 0 = by K)
  int tma_store = 1;            // epilogue results leave through shared memory + TMA tile stores when C allows
  int split_tail = 3;           // last wave at most half full: 1 = its tiles run as two K halves (int8), 2 = as two column
                                // ranges, 3 = the faster of the two as measured (column ranges), 0 = whole tiles
  int group_m = 0;              // row-blocks per rasterisation group (0 = default for the kernel family)
  int host_blocks = 0;           // row blocks the *_host GEMM entry points pipeline over (0 = default)
  int conv_wide_n = 0;          // patch form: the kw taps of a filter row in one MMA (N = kw * cout_tile)
  int conv_split_weights = 1;   // patch form: one weight box per filter row, each on its own barrier
  int conv_hwio_direct = 1;     // conv consumes HWIO weights as an N-major operand where it can (no re-layout launch)
  int conv_halo = 1;            // conv kernel fetches a tile's whole input patch and all taps' weights in two boxes
  int conv_mma_group = 0;       // persistent conv: 0 choose, 1 = one tile's MMAs at a time, 2 = two tiles interleaved
  int conv_persistent = 1;      // many tiles per SM: CTAs keep the weights and walk the tiles (patches, accumulators double-buffered)
  int cta_limit = 0;            // persistent GEMM kernels occupy at most this many SMs (0 = all of them)
  int usable_sms() const { return cta_limit > 0 && cta_limit < sm_count ? cta_limit : sm_count; }
  int operands_ready = 0;       // caller's promise: GEMM operands are never written by the kernel just before in the stream
  int pdl = 1;                  // launch the tensor-core kernels with programmatic stream serialization
  int debug_mode = 0;           // see GemmParams::debug
  long long* cta_times = nullptr;  // see GemmParams::cta_times (device pointer owned by the caller)
  long long* trace = nullptr;   // see GemmParams::trace (device pointer owned by the caller)
  long long launches = 0;
  // counts re-allocations of the context's device workspaces: a recorded CUDA graph that holds pointers
  // into them is stale once this has moved on
  unsigned long long workspace_generation = 0;
  std::unordered_map<const void*, aiehlc::KernelSetup> kernel_setup;
  // staging for *_host entry points and for operands that TMA cannot address directly
  aiehlc::DevBuf buf_a, buf_b, buf_c, buf_aux, pack_a, pack_b;
  aiehlc::DevBuf limb_a, limb_b;        // byte planes of int32 operands (mm_i32 on the tensor cores)
  int mm_i32_tensor = 1;                // large int32 products run as int8 limb GEMMs on the tensor cores
  aiehlc::DevBuf sk_scratch, sk_flags;  // partial sums and deposit counters of tail tiles cut along K
  int shard_tile_stores = 1;            // sharded output leaves as add-reducing TMA tile stores (else row reductions)
  aiehlc::DevBuf shard_maps;            // tensor maps of a row-sharded output, as the kernels read them
  std::vector<unsigned long long> shard_key;  // what those maps were made from
};

namespace aiehlc {

// `_dev` entry points run on exactly the stream they are given (NULL is CUDA's default stream).
inline cudaStream_t pick_stream(aiehlc_ctx* /*ctx*/, void* stream) {
  return static_cast<cudaStream_t>(stream);
}

// tcgen05 tile GEMM launcher (gemm_launch.cu).  kind: KIND_I8 / KIND_BF16; epi: EPI_*.
struct GemmCall {
  int kind, epi;
  const void* A; const void* B; void* C;
  int M, N, K;
  long long lda, ldb, ldc;      // elements
  const int32_t* acc_in; long long ld_acc;
  const uint8_t* shift_vec; int shift;
  int group_m;                  // filled in from the plan
  int unsigned_ab = 0, out_shift = 0;   // see GemmParams
  int operands_from_kernel = 0;         // A or B was produced by a kernel this library launched just before (never early)
  // row-sharded add-reduction output (see GemmParams::shard); C is unused when num_shards > 0
  int32_t* const* shards = nullptr;
  const CUtensorMap* shard_maps = nullptr;   // optional: the shards as tensors for add-reducing tile stores
  int rows_per_shard = 0, num_shards = 0, first_shard = 0;
};
int launch_gemm(aiehlc_ctx* ctx, const GemmCall& c, cudaStream_t st);
int encode_c_map(aiehlc_ctx* ctx, CUtensorMap* map, int epi, int bn, void* base, long long rows, long long cols,
                 long long ld);
int plan_gemm(const aiehlc_ctx* ctx, int kind, int M, int N, int K, aiehlc_gemm_plan* out);
int tile_order(const aiehlc_ctx* ctx, int kind, int M, int N, int K, int num_shards, int rows_per_shard, int first_shard,
               int* row_block, int* col_block, int capacity, int* slots_out);
// Tail tiles of a CTA-pair launch that run as two K halves (0: none) and where they are cut; see gemm_launch.cu.
int split_k_tail(int tiles, int slots, int k_blocks, int mode, int* cut_at);
void narrow_tail(int tiles, int slots, int tile_n, int enabled, int* first, int* parts);

// SIMT helpers (simt_kernels.cu)
int launch_mm_i32(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K, cudaStream_t st);
int launch_mm_i32_tensor(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K, cudaStream_t st);
bool mm_i32_tensor_ok(const aiehlc_ctx* ctx, int M, int N, int K);
int launch_srs(aiehlc_ctx* ctx, const int32_t* in, int8_t* out, long long rows, long long cols, int shift,
               const uint8_t* shift_vec, cudaStream_t st);
int launch_fill_i32(aiehlc_ctx* ctx, int32_t* out, long long n, int value, cudaStream_t st);
// Copy a rows x cols matrix of `esize`-byte elements from leading dimension ld_src to ld_dst.
int launch_repack(aiehlc_ctx* ctx, const void* src, void* dst, long long rows, long long cols,
                  long long ld_src, long long ld_dst, int esize, cudaStream_t st);

// implicit-GEMM conv (conv_tcgen05.cu)
// `weight_scratch`: where re-laid weights ([tap][cout][cin], kh*kw*cin*cout bytes) are kept when the
// shape needs them; null = the context's growing workspace.
int launch_conv2d(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n, int h, int wd,
                  int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st,
                  int8_t* weight_scratch = nullptr);

bool conv_tensor_path(const int8_t* x, int cin, int cout);
int plan_conv2d(const aiehlc_ctx* ctx, int n, int h, int wd, int cin, int cout, int kh, int kw, int pad,
                aiehlc_conv_plan* out);
int launch_conv_pack_weights(aiehlc_ctx* ctx, const int8_t* w, int8_t* packed, int taps, int cin, int cout,
                             cudaStream_t st);
int launch_conv2d_packed(aiehlc_ctx* ctx, const int8_t* x, const int8_t* packed, int8_t* y, int n, int h, int wd,
                         int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec, cudaStream_t st);

}  // namespace aiehlc
