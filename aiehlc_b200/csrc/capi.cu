// extern "C" entry points declared in include/aiehlc_b200.h.
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/aiehlc_b200_tuning.h"
#include "context.h"
#include "gemm_tcgen05.cuh"

namespace aiehlc {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int rc, const std::string& msg) {
  g_last_error = msg;
  return rc;
}
int cuda_fail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return AIEHLC_ERR_CUDA;
}

int DevBuf::reserve(size_t need) {
  if (need <= bytes) return 0;
  if (ptr) {
    cudaFree(ptr);
    if (generation) ++*generation;  // whoever recorded the old address must not use it again
  }
  ptr = nullptr;
  bytes = 0;
  const size_t want = (need + (1u << 20) - 1) & ~static_cast<size_t>((1u << 20) - 1);
  cudaError_t e = cudaMalloc(&ptr, want);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaMalloc(workspace)");
    ptr = nullptr;
    return AIEHLC_ERR_NOMEM;
  }
  bytes = want;
  return 0;
}
void DevBuf::release() {
  if (ptr) cudaFree(ptr);
  ptr = nullptr;
  bytes = 0;
}

int ensure_dynamic_smem(int device, const void* func, int bytes, int* cached) {
  if (cached && *cached >= bytes) return AIEHLC_OK;
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> limit;  // (device, kernel) -> bytes already granted
  std::lock_guard<std::mutex> lk(mu);
  int& have = limit[{device, func}];
  if (have < bytes) {
    AIEHLC_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    have = bytes;
  }
  if (cached) *cached = have;
  return AIEHLC_OK;
}

static int check_ctx(aiehlc_ctx* ctx) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
  return AIEHLC_OK;
}

static int check_shift(int shift, const uint8_t* /*shift_vec*/) {
  if (shift < 0 || shift > 31) return fail(AIEHLC_ERR_INVALID, "srs shift must be in [0, 31]");
  return AIEHLC_OK;
}

}  // namespace aiehlc

using namespace aiehlc;

extern "C" {

const char* aiehlc_last_error(void) { return g_last_error.c_str(); }

int aiehlc_create(int device, aiehlc_ctx** out) {
  if (!out) return fail(AIEHLC_ERR_INVALID, "aiehlc_create: null out pointer");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0)
    return fail(AIEHLC_ERR_CUDA, std::string("aiehlc_create: no CUDA device (") +
                                     (e != cudaSuccess ? cudaGetErrorString(e) : "count = 0") +
                                     "); this library has no CPU path");
  if (device < 0 || device >= count) return fail(AIEHLC_ERR_INVALID, "aiehlc_create: device out of range");
  AIEHLC_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  AIEHLC_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(AIEHLC_ERR_UNSUPPORTED, "aiehlc_create: kernels are built for sm_100a only (found sm_" +
                                            std::to_string(prop.major) + std::to_string(prop.minor) + ")");
  aiehlc_ctx* ctx = new aiehlc_ctx();
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  for (DevBuf* b : {&ctx->buf_a, &ctx->buf_b, &ctx->buf_c, &ctx->buf_aux, &ctx->pack_a, &ctx->pack_b, &ctx->limb_a,
                    &ctx->limb_b, &ctx->sk_scratch, &ctx->sk_flags, &ctx->shard_maps})
    b->generation = &ctx->workspace_generation;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    delete ctx;
    return fail(AIEHLC_ERR_CUDA, "aiehlc_create: cuTensorMapEncodeTiled not available from the driver");
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream2, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream_up, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ctx->block_done, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaMalloc(&ctx->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&ctx->h_status, sizeof(int));
  if (e != cudaSuccess) {
    cuda_fail(e, "aiehlc_create");
    aiehlc_destroy(ctx);
    return AIEHLC_ERR_CUDA;
  }
  *ctx->h_status = 0;
  *out = ctx;
  return AIEHLC_OK;
}

int aiehlc_destroy(aiehlc_ctx* ctx) {
  if (!ctx) return AIEHLC_OK;
  cudaSetDevice(ctx->device);
  if (ctx->stream) {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
  }
  if (ctx->stream2) {
    cudaStreamSynchronize(ctx->stream2);
    cudaStreamDestroy(ctx->stream2);
  }
  if (ctx->stream_up) {
    cudaStreamSynchronize(ctx->stream_up);
    cudaStreamDestroy(ctx->stream_up);
  }
  if (ctx->block_done) cudaEventDestroy(ctx->block_done);
  for (cudaEvent_t ev : ctx->block_ev) cudaEventDestroy(ev);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  ctx->buf_a.release(); ctx->buf_b.release(); ctx->buf_c.release(); ctx->buf_aux.release();
  ctx->pack_a.release(); ctx->pack_b.release();
  ctx->limb_a.release(); ctx->limb_b.release();
  ctx->sk_scratch.release(); ctx->sk_flags.release(); ctx->shard_maps.release();
  delete ctx;
  return AIEHLC_OK;
}

int aiehlc_sm_count(const aiehlc_ctx* ctx) { return ctx ? ctx->sm_count : 0; }
long long aiehlc_launch_count(const aiehlc_ctx* ctx) { return ctx ? ctx->launches : 0; }
long long aiehlc_workspace_generation(const aiehlc_ctx* ctx) {
  return ctx ? static_cast<long long>(ctx->workspace_generation) : 0;
}

int aiehlc_set_tile_n(aiehlc_ctx* ctx, int tile_n) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 256)
    return fail(AIEHLC_ERR_INVALID, "tile_n must be 0, 64, 128 or 256");
  ctx->force_tile_n = tile_n;
  return AIEHLC_OK;
}

int aiehlc_set_cta_pair(aiehlc_ctx* ctx, int mode) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (mode < -1 || mode > 1) return fail(AIEHLC_ERR_INVALID, "pair mode must be -1, 0 or 1");
  ctx->pair_mode = mode;
  return AIEHLC_OK;
}

int aiehlc_plan_gemm(aiehlc_ctx* ctx, int kind, int M, int N, int K, aiehlc_gemm_plan* plan) {
  if (!plan) return fail(AIEHLC_ERR_INVALID, "plan_gemm: null plan");
  if (kind != KIND_I8 && kind != KIND_BF16) return fail(AIEHLC_ERR_INVALID, "plan_gemm: kind must be 0 (int8) or 1 (bf16)");
  if (M <= 0 || N <= 0 || K <= 0) return fail(AIEHLC_ERR_INVALID, "plan_gemm: M, N, K must be positive");
  if (!ctx) {
    // no device needed to plan: a B200 with default settings
    aiehlc_ctx defaults;
    defaults.sm_count = 148;
    return plan_gemm(&defaults, kind, M, N, K, plan);
  }
  return plan_gemm(ctx, kind, M, N, K, plan);
}

int aiehlc_plan_tile_order(aiehlc_ctx* ctx, int kind, int M, int N, int K, int num_shards, int rows_per_shard,
                           int first_shard, int* row_block, int* col_block, int capacity, int* slots) {
  if (kind != KIND_I8 && kind != KIND_BF16) return fail(AIEHLC_ERR_INVALID, "plan_tile_order: kind must be 0 (int8) or 1 (bf16)");
  if (M <= 0 || N <= 0 || K <= 0 || !row_block || !col_block || capacity < 0)
    return fail(AIEHLC_ERR_INVALID, "plan_tile_order: bad argument");
  if (num_shards < 0 || num_shards > AIEHLC_MAX_SHARDS || (num_shards > 0 && (rows_per_shard <= 0 || rows_per_shard % 128 != 0)))
    return fail(AIEHLC_ERR_INVALID, "plan_tile_order: bad sharding");
  if (!ctx) {
    aiehlc_ctx defaults;
    defaults.sm_count = 148;
    return tile_order(&defaults, kind, M, N, K, num_shards, rows_per_shard, first_shard, row_block, col_block, capacity, slots);
  }
  return tile_order(ctx, kind, M, N, K, num_shards, rows_per_shard, first_shard, row_block, col_block, capacity, slots);
}

int aiehlc_set_k_per_load(aiehlc_ctx* ctx, int k_blocks) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (k_blocks < 0 || k_blocks > 2) return fail(AIEHLC_ERR_INVALID, "k_per_load must be 0, 1 or 2");
  ctx->k_per_load = k_blocks;
  return AIEHLC_OK;
}

int aiehlc_set_tma_store(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (on < 0 || on > 2) return fail(AIEHLC_ERR_INVALID, "tma_store must be 0, 1 or 2");
  ctx->tma_store = on;
  return AIEHLC_OK;
}

int aiehlc_set_epilogue_groups(aiehlc_ctx* ctx, int groups) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (groups < 0 || groups > 2) return fail(AIEHLC_ERR_INVALID, "epilogue groups must be 0, 1 or 2");
  ctx->epi_groups = groups;
  return AIEHLC_OK;
}

int aiehlc_set_split_tail(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (on < 0 || on > 3) return fail(AIEHLC_ERR_INVALID, "split_tail: 0 (off), 1 (K halves), 2 (column ranges) or 3 (choose)");
  ctx->split_tail = on;
  return AIEHLC_OK;
}

int aiehlc_set_host_blocks(aiehlc_ctx* ctx, int blocks) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (blocks < 0 || blocks > 64) return fail(AIEHLC_ERR_INVALID, "host_blocks: 0 (default) .. 64");
  ctx->host_blocks = blocks;
  return AIEHLC_OK;
}

int aiehlc_set_mm_i32_tensor(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (on < 0 || on > 2) return fail(AIEHLC_ERR_INVALID, "mm_i32_tensor: 0 (never), 1 (large products) or 2 (always)");
  ctx->mm_i32_tensor = on;
  return AIEHLC_OK;
}

int aiehlc_set_conv_wide_n(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  ctx->conv_wide_n = on ? 1 : 0;
  return AIEHLC_OK;
}

int aiehlc_set_conv_hwio_direct(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  ctx->conv_hwio_direct = on ? 1 : 0;
  return AIEHLC_OK;
}

int aiehlc_set_conv_persistent(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (on < 0 || on > 4) return fail(AIEHLC_ERR_INVALID, "conv_persistent: 0 (off), 1 (on), 2 / 3 / 4 (on, one / two / four tiles per MMA group)");
  ctx->conv_persistent = on ? 1 : 0;
  ctx->conv_mma_group = on >= 2 ? (on == 4 ? 4 : on - 1) : 0;
  return AIEHLC_OK;
}

int aiehlc_set_conv_halo(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  ctx->conv_halo = on ? 1 : 0;
  return AIEHLC_OK;
}

int aiehlc_set_shard_tile_stores(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  ctx->shard_tile_stores = on ? 1 : 0;
  return AIEHLC_OK;
}

int aiehlc_set_group_m(aiehlc_ctx* ctx, int group_m) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (group_m < 0) return fail(AIEHLC_ERR_INVALID, "group_m must be >= 0");
  ctx->group_m = group_m;
  return AIEHLC_OK;
}

int aiehlc_set_cta_limit(aiehlc_ctx* ctx, int sms) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (sms < 0) return fail(AIEHLC_ERR_INVALID, "cta_limit must be >= 0");
  ctx->cta_limit = sms;
  return AIEHLC_OK;
}

int aiehlc_set_operands_ready(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  ctx->operands_ready = on ? 1 : 0;
  return AIEHLC_OK;
}

int aiehlc_set_pdl(aiehlc_ctx* ctx, int on) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  ctx->pdl = on ? 1 : 0;
  return AIEHLC_OK;
}

static int need_measure_build(const char* what) {
  if (kMeasure) return AIEHLC_OK;
  return fail(AIEHLC_ERR_UNSUPPORTED, std::string(what) + ": this library was built without AIEHLC_MEASURE");
}

int aiehlc_set_cta_times(aiehlc_ctx* ctx, long long* device_buffer) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (device_buffer) if (int rc = need_measure_build("aiehlc_set_cta_times")) return rc;
  ctx->cta_times = device_buffer;
  return AIEHLC_OK;
}

int aiehlc_set_trace(aiehlc_ctx* ctx, long long* device_buffer) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (device_buffer) if (int rc = need_measure_build("aiehlc_set_trace")) return rc;
  ctx->trace = device_buffer;
  return AIEHLC_OK;
}

int aiehlc_set_debug(aiehlc_ctx* ctx, int mode) {
  if (!ctx) return fail(AIEHLC_ERR_INVALID, "null context");
  if (mode < 0 || mode > 5) return fail(AIEHLC_ERR_INVALID, "debug mode must be 0..5");
  if (mode != 0 && mode != 3) if (int rc = need_measure_build("aiehlc_set_debug (modes 1, 2, 4, 5)")) return rc;
  ctx->debug_mode = mode;
  return AIEHLC_OK;
}

int aiehlc_sync(aiehlc_ctx* ctx, void* stream, int* status) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  cudaStream_t st = pick_stream(ctx, stream);
  AIEHLC_CUDA(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, st));
  AIEHLC_CUDA(cudaMemsetAsync(ctx->d_status, 0, sizeof(int), st));
  AIEHLC_CUDA(cudaStreamSynchronize(st));
  const int s = *ctx->h_status;
  if (status) *status = s;
  if (s != 0 && ctx->sk_flags.ptr) {
    // a launch gave up half-way: its tail-tile deposit counters may be left non-zero
    cudaMemsetAsync(ctx->sk_flags.ptr, 0, ctx->sk_flags.bytes, st);
    cudaStreamSynchronize(st);
  }
  if (s != 0) return fail(AIEHLC_ERR_DEVICE, "kernel status word = " + std::to_string(s) + " (a bounded wait ran out)");
  return AIEHLC_OK;
}

// ------------------------------------------------------------------ device-pointer entry points
int aiehlc_mm_i32_dev(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K, void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "mm_i32: negative size");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!in || !out) return fail(AIEHLC_ERR_INVALID, "mm_i32: null pointer");
  if (mm_i32_tensor_ok(ctx, M, N, K)) return launch_mm_i32_tensor(ctx, in, out, M, N, K, pick_stream(ctx, stream));
  return launch_mm_i32(ctx, in, out, M, N, K, pick_stream(ctx, stream));
}

int aiehlc_gemm_i8_i32_dev(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K,
                           int accumulate, void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32: negative size");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!C) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32: null C");
  cudaStream_t st = pick_stream(ctx, stream);
  if (K == 0) {
    if (accumulate) return AIEHLC_OK;
    return launch_fill_i32(ctx, C, static_cast<long long>(M) * N, 0, st);
  }
  if (!A || !B) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32: null operand");
  GemmCall c{};
  c.kind = KIND_I8; c.epi = accumulate ? EPI_I32_ACC : EPI_I32;
  c.A = A; c.B = B; c.C = C; c.M = M; c.N = N; c.K = K; c.lda = K; c.ldb = K; c.ldc = N;
  return launch_gemm(ctx, c, st);
}

int aiehlc_gemm_i8_i32_scatter_dev(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int32_t* const* shards,
                                   int num_shards, int rows_per_shard, int first_shard, int M, int N, int K,
                                   void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32_scatter: negative size");
  if (num_shards < 1 || num_shards > AIEHLC_MAX_SHARDS || !shards)
    return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32_scatter: 1 .. AIEHLC_MAX_SHARDS shards");
  if (rows_per_shard <= 0 || rows_per_shard % 128 != 0)
    return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32_scatter: rows_per_shard must be a positive multiple of 128");
  if (static_cast<long long>(num_shards) * rows_per_shard < M)
    return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32_scatter: the shards do not cover M rows");
  if (M == 0 || N == 0 || K == 0) return AIEHLC_OK;  // nothing to add
  if (!A || !B) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32_scatter: null operand");
  static_assert(AIEHLC_MAX_SHARDS == kMaxShards, "header and kernel agree on the shard limit");
  const int used = (M + rows_per_shard - 1) / rows_per_shard;
  for (int g = 0; g < used; ++g)
    if (!shards[g] || reinterpret_cast<uintptr_t>(shards[g]) % 4 != 0)
      return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32_scatter: shard pointers must be non-null and 4-byte aligned");
  cudaStream_t st = pick_stream(ctx, stream);

  GemmCall c{};
  c.kind = KIND_I8; c.epi = EPI_I32_ACC;
  c.A = A; c.B = B; c.C = nullptr; c.M = M; c.N = N; c.K = K; c.lda = K; c.ldb = K; c.ldc = N;
  if (ctx->shard_tile_stores && N % 4 == 0) {
    bool aligned = true;
    for (int g = 0; g < used; ++g) aligned = aligned && reinterpret_cast<uintptr_t>(shards[g]) % 16 == 0;
    if (aligned) {
      // the shards' tensor maps live in a context buffer; they are rebuilt only when the call differs
      std::vector<unsigned long long> key = {static_cast<unsigned long long>(M), static_cast<unsigned long long>(N),
                                             static_cast<unsigned long long>(rows_per_shard),
                                             static_cast<unsigned long long>(num_shards)};
      for (int g = 0; g < used; ++g) key.push_back(reinterpret_cast<unsigned long long>(shards[g]));
      if (key != ctx->shard_key) {
        CUtensorMap maps[AIEHLC_MAX_SHARDS];
        for (int g = 0; g < num_shards; ++g) {
          const int src = g < used ? g : 0;  // shards past M are never addressed
          const long long rows = src == used - 1 ? M - static_cast<long long>(src) * rows_per_shard : rows_per_shard;
          if ((rc = encode_c_map(ctx, &maps[g], EPI_I32_ACC, 256, shards[src], rows, N, N))) return rc;
        }
        if (ctx->shard_maps.reserve(sizeof maps)) return AIEHLC_ERR_NOMEM;
        // Rare (once per set of shards): wait for the copy, so that later calls may reuse the maps from
        // any stream, and for earlier launches on `st` that may still be reading the previous maps.
        AIEHLC_CUDA(cudaStreamSynchronize(st));
        AIEHLC_CUDA(cudaMemcpyAsync(ctx->shard_maps.ptr, maps, sizeof(CUtensorMap) * num_shards, cudaMemcpyHostToDevice, st));
        AIEHLC_CUDA(cudaStreamSynchronize(st));
        ctx->shard_key = key;
      }
    }
  }
  int32_t* ptrs[AIEHLC_MAX_SHARDS];
  for (int g = 0; g < num_shards; ++g) ptrs[g] = shards[g < used ? g : 0];  // shards past M are never addressed
  c.shards = ptrs;
  if (ctx->shard_tile_stores && N % 4 == 0 && !ctx->shard_key.empty()) {
    bool aligned = true;
    for (int g = 0; g < used; ++g) aligned = aligned && reinterpret_cast<uintptr_t>(shards[g]) % 16 == 0;
    if (aligned) c.shard_maps = static_cast<const CUtensorMap*>(ctx->shard_maps.ptr);
  }
  c.rows_per_shard = rows_per_shard; c.num_shards = num_shards; c.first_shard = first_shard;
  return launch_gemm(ctx, c, st);
}

int aiehlc_srs_i32_i8_dev(aiehlc_ctx* ctx, const int32_t* in, int8_t* out, long long rows, long long cols,
                          int shift, const uint8_t* shift_vec, void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (rows < 0 || cols < 0) return fail(AIEHLC_ERR_INVALID, "srs: negative size");
  if ((rc = check_shift(shift, shift_vec))) return rc;
  if (rows == 0 || cols == 0) return AIEHLC_OK;
  if (!in || !out) return fail(AIEHLC_ERR_INVALID, "srs: null pointer");
  return launch_srs(ctx, in, out, rows, cols, shift, shift_vec, pick_stream(ctx, stream));
}

int aiehlc_gemm_i8_srs_dev(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                           int shift, const uint8_t* shift_vec, const int32_t* acc_in, int splitk,
                           void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: negative size");
  if ((rc = check_shift(shift, shift_vec))) return rc;
  if (splitk < 1 || (K > 0 && K % splitk != 0))
    return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: splitk must be >= 1 and divide K");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!C) return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: null C");
  cudaStream_t st = pick_stream(ctx, stream);
  if (K == 0) {
    // empty contraction: the result is srs(acc_in) or srs(0) = 0
    if (acc_in) return launch_srs(ctx, acc_in, C, M, N, shift, shift_vec, st);
    AIEHLC_CUDA(cudaMemsetAsync(C, 0, static_cast<size_t>(M) * N, st));
    return AIEHLC_OK;
  }
  if (!A || !B) return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: null operand");
  // The K loop of one launch visits the splitk slices in order and keeps the running sum in
  // TMEM, so the slice count does not change the schedule: it only has to divide K.
  GemmCall c{};
  c.kind = KIND_I8; c.epi = EPI_I8_SRS;
  c.A = A; c.B = B; c.C = C; c.M = M; c.N = N; c.K = K; c.lda = K; c.ldb = K; c.ldc = N;
  c.acc_in = acc_in; c.ld_acc = N; c.shift_vec = shift_vec; c.shift = shift;
  return launch_gemm(ctx, c, st);
}

int aiehlc_gemm_bf16_dev(aiehlc_ctx* ctx, const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N,
                         int K, void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_bf16: negative size");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!C) return fail(AIEHLC_ERR_INVALID, "gemm_bf16: null C");
  cudaStream_t st = pick_stream(ctx, stream);
  if (K == 0) {
    AIEHLC_CUDA(cudaMemsetAsync(C, 0, static_cast<size_t>(M) * N * 2, st));
    return AIEHLC_OK;
  }
  if (!A || !B) return fail(AIEHLC_ERR_INVALID, "gemm_bf16: null operand");
  GemmCall c{};
  c.kind = KIND_BF16; c.epi = EPI_BF16;
  c.A = A; c.B = B; c.C = C; c.M = M; c.N = N; c.K = K; c.lda = K; c.ldb = K; c.ldc = N;
  return launch_gemm(ctx, c, st);
}

int aiehlc_conv2d_i8_srs_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n, int h, int wd,
                             int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec,
                             void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (n < 0 || h < 0 || wd < 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || pad < 0)
    return fail(AIEHLC_ERR_INVALID, "conv2d: bad size");
  if (kh != 2 * pad + 1 || kw != 2 * pad + 1)
    return fail(AIEHLC_ERR_UNSUPPORTED, "conv2d: only stride 1 with kh = kw = 2*pad+1 (same-size output)");
  if (n == 0 || h == 0 || wd == 0) return AIEHLC_OK;
  if (!x || !w || !y || !shift_vec) return fail(AIEHLC_ERR_INVALID, "conv2d: null pointer");
  return launch_conv2d(ctx, x, w, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec, pick_stream(ctx, stream));
}

int aiehlc_plan_conv2d(aiehlc_ctx* ctx, int n, int h, int wd, int cin, int cout, int kh, int kw, int pad,
                       aiehlc_conv_plan* plan) {
  if (!plan) return fail(AIEHLC_ERR_INVALID, "plan_conv2d: null plan");
  if (n <= 0 || h <= 0 || wd <= 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || pad < 0)
    return fail(AIEHLC_ERR_INVALID, "plan_conv2d: bad size");
  if (kh != 2 * pad + 1 || kw != 2 * pad + 1)
    return fail(AIEHLC_ERR_UNSUPPORTED, "conv2d: only stride 1 with kh = kw = 2*pad+1 (same-size output)");
  if (!ctx) {
    aiehlc_ctx defaults;  // no device needed to plan: a 148-SM B200 with default settings
    defaults.sm_count = 148;
    return plan_conv2d(&defaults, n, h, wd, cin, cout, kh, kw, pad, plan);
  }
  return plan_conv2d(ctx, n, h, wd, cin, cout, kh, kw, pad, plan);
}

int aiehlc_conv2d_pack_weights_dev(aiehlc_ctx* ctx, const int8_t* w, int8_t* packed, int kh, int kw, int cin,
                                   int cout, void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (kh <= 0 || kw <= 0 || cin <= 0 || cout <= 0) return fail(AIEHLC_ERR_INVALID, "conv2d pack: bad size");
  if (!w || !packed) return fail(AIEHLC_ERR_INVALID, "conv2d pack: null pointer");
  if (reinterpret_cast<uintptr_t>(packed) % 16 != 0) return fail(AIEHLC_ERR_INVALID, "conv2d pack: destination must be 16-byte aligned");
  return launch_conv_pack_weights(ctx, w, packed, kh * kw, cin, cout, pick_stream(ctx, stream));
}

int aiehlc_conv2d_i8_srs_packed_dev(aiehlc_ctx* ctx, const int8_t* x, const int8_t* packed, int8_t* y, int n, int h,
                                    int wd, int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec,
                                    void* stream) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (n < 0 || h < 0 || wd < 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || pad < 0)
    return fail(AIEHLC_ERR_INVALID, "conv2d: bad size");
  if (kh != 2 * pad + 1 || kw != 2 * pad + 1)
    return fail(AIEHLC_ERR_UNSUPPORTED, "conv2d: only stride 1 with kh = kw = 2*pad+1 (same-size output)");
  if (n == 0 || h == 0 || wd == 0) return AIEHLC_OK;
  if (!x || !packed || !y || !shift_vec) return fail(AIEHLC_ERR_INVALID, "conv2d: null pointer");
  if (!conv_tensor_path(x, cin, cout) || reinterpret_cast<uintptr_t>(packed) % 16 != 0)
    return fail(AIEHLC_ERR_UNSUPPORTED, "conv2d (packed weights): needs cin in {32, 64, k*128}, cout a multiple of 16 and "
                                        "16-byte aligned x and weights; use aiehlc_conv2d_i8_srs_dev for other shapes");
  return launch_conv2d_packed(ctx, x, packed, y, n, h, wd, cin, cout, kh, kw, pad, shift_vec, pick_stream(ctx, stream));
}

// ------------------------------------------------------------------ host-pointer entry points
// H2D copy of the operands, the same kernels, D2H copy of the result, one synchronisation.
static int finish_host(aiehlc_ctx* ctx) {
  int status = 0;
  return aiehlc_sync(ctx, ctx->stream, &status);
}

int aiehlc_mm_i32_host(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "mm_i32: negative size");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!in || !out) return fail(AIEHLC_ERR_INVALID, "mm_i32: null pointer");
  const size_t in_bytes = (static_cast<size_t>(M) + N) * K * 4, out_bytes = static_cast<size_t>(M) * N * 4;
  if (ctx->buf_a.reserve(in_bytes ? in_bytes : 4) || ctx->buf_c.reserve(out_bytes)) return AIEHLC_ERR_NOMEM;
  AIEHLC_CUDA(cudaMemcpyAsync(ctx->buf_a.ptr, in, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
  rc = aiehlc_mm_i32_dev(ctx, static_cast<const int32_t*>(ctx->buf_a.ptr), static_cast<int32_t*>(ctx->buf_c.ptr),
                         M, N, K, ctx->stream);
  if (rc) return rc;
  AIEHLC_CUDA(cudaMemcpyAsync(out, ctx->buf_c.ptr, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return finish_host(ctx);
}

static int stage_ab(aiehlc_ctx* ctx, const void* A, const void* B, size_t a_bytes, size_t b_bytes,
                    size_t c_bytes) {
  if (ctx->buf_a.reserve(a_bytes ? a_bytes : 16) || ctx->buf_b.reserve(b_bytes ? b_bytes : 16) ||
      ctx->buf_c.reserve(c_bytes ? c_bytes : 16))
    return AIEHLC_ERR_NOMEM;
  if (a_bytes) AIEHLC_CUDA(cudaMemcpyAsync(ctx->buf_a.ptr, A, a_bytes, cudaMemcpyHostToDevice, ctx->stream));
  if (b_bytes) AIEHLC_CUDA(cudaMemcpyAsync(ctx->buf_b.ptr, B, b_bytes, cudaMemcpyHostToDevice, ctx->stream));
  return AIEHLC_OK;
}

}  // extern "C"

// Host-buffer GEMM as a pipeline over blocks of A rows and of B rows (= C columns) on three streams:
//   stream_up : A_0, B_0, B_1, A_1, B_2, A_2, ... -> device, back to back
//   stream    : after each upload, ONE kernel for the part of C that has just become computable: the new
//               row block against every B block present, or every A block present against the new B block
//   stream2   : that rectangle of C -> host as soon as its kernel is done
// so the first kernel starts after one block of each operand (not after all of B), the link never waits
// for a kernel in either direction, and what is left after the last upload is one block's kernel and
// download.  With pinned host buffers the copies are truly asynchronous; with pageable ones the runtime
// stages them and the result is the same, only slower.
//   launch_rect(A rows, B rows, C corner, rows, cols, first column): C[rows][cols] (pitch N) = A . B^T
template <typename LaunchRect>
static int host_gemm_pipelined(aiehlc_ctx* ctx, const void* A, const void* B, void* C, int M, int N, int K, int in_esize,
                               int out_esize, LaunchRect launch_rect) {
  const size_t a_bytes = static_cast<size_t>(M) * K * in_esize, b_bytes = static_cast<size_t>(N) * K * in_esize;
  const size_t c_bytes = static_cast<size_t>(M) * N * out_esize;
  if (ctx->buf_a.reserve(a_bytes ? a_bytes : 16) || ctx->buf_b.reserve(b_bytes ? b_bytes : 16) ||
      ctx->buf_c.reserve(c_bytes ? c_bytes : 16))
    return AIEHLC_ERR_NOMEM;
  // whatever the caller queued on the context's stream before (shift bytes, ...) precedes the uploads
  AIEHLC_CUDA(cudaEventRecord(ctx->block_done, ctx->stream));
  AIEHLC_CUDA(cudaStreamWaitEvent(ctx->stream_up, ctx->block_done, 0));
  // blocks of whole 256-row tiles; small problems (and empty contractions) go in one piece
  const int blocks = ctx->host_blocks > 0 ? ctx->host_blocks : 4;
  int a_rows = ((M + blocks - 1) / blocks + 255) / 256 * 256;
  int b_rows = ((N + blocks - 1) / blocks + 255) / 256 * 256;
  if (K == 0 || static_cast<size_t>(a_rows) * K * in_esize < (1u << 20)) a_rows = M;
  if (K == 0 || static_cast<size_t>(b_rows) * K * in_esize < (1u << 20)) b_rows = N;
  // block boundaries.  What follows the LAST upload cannot overlap any copy in the other direction's shadow: the
  // kernel on the block just uploaded and the download of its rows of C.  That last upload is a block of A (see
  // the order below), so A's last block gives up all but one row of tiles to a block of its own before it.
  std::vector<int> a_cut{0}, b_cut{0};
  for (int r = a_rows; r < M; r += a_rows) a_cut.push_back(r);
  for (int r = b_rows; r < N; r += b_rows) b_cut.push_back(r);
  if (a_cut.size() > 1 && M - a_cut.back() >= 512) a_cut.push_back((M - 1) / 256 * 256);
  a_cut.push_back(M);
  b_cut.push_back(N);
  const int na = static_cast<int>(a_cut.size()) - 1, nb = static_cast<int>(b_cut.size()) - 1;
  uint8_t* da = static_cast<uint8_t*>(ctx->buf_a.ptr);
  uint8_t* db = static_cast<uint8_t*>(ctx->buf_b.ptr);
  uint8_t* dc = static_cast<uint8_t*>(ctx->buf_c.ptr);
  int ev = 0;
  // the rectangle rows [r0, r1) x columns [c0, c1) of C: kernel once the upload just queued has landed, then download
  auto rect = [&](int r0, int r1, int c0, int c1) -> int {
    cudaEvent_t up = nullptr, done = nullptr;
    if (int rc = ctx->block_events(ev++, &up, &done)) return rc;
    AIEHLC_CUDA(cudaEventRecord(up, ctx->stream_up));
    AIEHLC_CUDA(cudaStreamWaitEvent(ctx->stream, up, 0));
    uint8_t* corner = dc + (static_cast<size_t>(r0) * N + c0) * out_esize;
    if (int rc = launch_rect(da + static_cast<size_t>(r0) * K * in_esize, db + static_cast<size_t>(c0) * K * in_esize, corner,
                             r1 - r0, c1 - c0, c0))
      return rc;
    AIEHLC_CUDA(cudaEventRecord(done, ctx->stream));
    AIEHLC_CUDA(cudaStreamWaitEvent(ctx->stream2, done, 0));
    uint8_t* host = static_cast<uint8_t*>(C) + (static_cast<size_t>(r0) * N + c0) * out_esize;
    if (c0 == 0 && c1 == N)
      AIEHLC_CUDA(cudaMemcpyAsync(host, corner, static_cast<size_t>(r1 - r0) * N * out_esize, cudaMemcpyDeviceToHost, ctx->stream2));
    else
      AIEHLC_CUDA(cudaMemcpy2DAsync(host, static_cast<size_t>(N) * out_esize, corner, static_cast<size_t>(N) * out_esize,
                                    static_cast<size_t>(c1 - c0) * out_esize, r1 - r0, cudaMemcpyDeviceToHost, ctx->stream2));
    return AIEHLC_OK;
  };
  auto upload = [&](uint8_t* dev, const void* host, int row0, int rows) -> int {
    if (K > 0 && rows > 0)
      AIEHLC_CUDA(cudaMemcpyAsync(dev + static_cast<size_t>(row0) * K * in_esize,
                                  static_cast<const uint8_t*>(host) + static_cast<size_t>(row0) * K * in_esize,
                                  static_cast<size_t>(rows) * K * in_esize, cudaMemcpyHostToDevice, ctx->stream_up));
    return AIEHLC_OK;
  };
  int ia = 0, ib = 0;  // blocks of A and of B on the device so far
  if (int rc = upload(da, A, 0, a_cut[1])) return rc;
  if (int rc = upload(db, B, 0, b_cut[1])) return rc;
  ia = ib = 1;
  if (int rc = rect(0, a_cut[1], 0, b_cut[1])) return rc;
  while (ia < na || ib < nb) {
    // the operand that is further behind goes next; on a tie B, so that the last piece of C is whole rows
    const bool take_b = ib < nb && (ia >= na || static_cast<long long>(b_cut[ib]) * M <= static_cast<long long>(a_cut[ia]) * N);
    if (take_b) {
      if (int rc = upload(db, B, b_cut[ib], b_cut[ib + 1] - b_cut[ib])) return rc;
      if (int rc = rect(0, a_cut[ia], b_cut[ib], b_cut[ib + 1])) return rc;
      ++ib;
    } else {
      if (int rc = upload(da, A, a_cut[ia], a_cut[ia + 1] - a_cut[ia])) return rc;
      if (int rc = rect(a_cut[ia], a_cut[ia + 1], 0, b_cut[ib])) return rc;
      ++ia;
    }
  }
  AIEHLC_CUDA(cudaStreamSynchronize(ctx->stream2));
  return finish_host(ctx);
}

// One rectangle of a host GEMM: the tile GEMM on device operands with C's pitch given (the public _dev entry
// points fix it at N).
static int gemm_rect(aiehlc_ctx* ctx, int kind, int epi, const void* A, const void* B, void* C, int M, int N, int K,
                     long long ldc, int shift, const uint8_t* shift_vec) {
  GemmCall c{};
  c.kind = kind; c.epi = epi;
  c.A = A; c.B = B; c.C = C; c.M = M; c.N = N; c.K = K; c.lda = K; c.ldb = K; c.ldc = ldc;
  c.shift = shift; c.shift_vec = shift_vec;
  return launch_gemm(ctx, c, ctx->stream);
}

extern "C" {

int aiehlc_gemm_i8_i32_host(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32: negative size");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(AIEHLC_ERR_INVALID, "gemm_i8_i32: null pointer");
  return host_gemm_pipelined(ctx, A, B, C, M, N, K, 1, 4, [&](uint8_t* da, uint8_t* db, uint8_t* dc, int rows, int cols, int) {
    if (K == 0) return aiehlc_gemm_i8_i32_dev(ctx, nullptr, nullptr, reinterpret_cast<int32_t*>(dc), rows, cols, 0, 0, ctx->stream);
    return gemm_rect(ctx, KIND_I8, EPI_I32, da, db, dc, rows, cols, K, N, 0, nullptr);
  });
}

int aiehlc_gemm_i8_srs_host(aiehlc_ctx* ctx, const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                            int shift, const uint8_t* shift_vec, int splitk) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: negative size");
  if ((rc = check_shift(shift, shift_vec))) return rc;
  if (splitk < 1 || (K > 0 && K % splitk != 0))
    return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: splitk must be >= 1 and divide K");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(AIEHLC_ERR_INVALID, "gemm_i8_srs: null pointer");
  const uint8_t* dsv = nullptr;
  if (shift_vec) {
    for (int j = 0; j < N; ++j)
      if (shift_vec[j] > 31) return fail(AIEHLC_ERR_INVALID, "srs shift must be in [0, 31]");
    if (ctx->buf_aux.reserve(N)) return AIEHLC_ERR_NOMEM;
    AIEHLC_CUDA(cudaMemcpyAsync(ctx->buf_aux.ptr, shift_vec, N, cudaMemcpyHostToDevice, ctx->stream));
    dsv = static_cast<const uint8_t*>(ctx->buf_aux.ptr);
  }
  return host_gemm_pipelined(ctx, A, B, C, M, N, K, 1, 1, [&](uint8_t* da, uint8_t* db, uint8_t* dc, int rows, int cols, int c0) {
    if (K == 0)   // whole C in one piece: srs(0) = 0
      return aiehlc_gemm_i8_srs_dev(ctx, nullptr, nullptr, reinterpret_cast<int8_t*>(dc), rows, cols, 0, shift, dsv, nullptr, 1,
                                    ctx->stream);
    return gemm_rect(ctx, KIND_I8, EPI_I8_SRS, da, db, dc, rows, cols, K, N, shift, dsv ? dsv + c0 : nullptr);
  });
}

int aiehlc_gemm_bf16_host(aiehlc_ctx* ctx, const uint16_t* A, const uint16_t* B, uint16_t* C, int M, int N,
                          int K) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (M < 0 || N < 0 || K < 0) return fail(AIEHLC_ERR_INVALID, "gemm_bf16: negative size");
  if (M == 0 || N == 0) return AIEHLC_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(AIEHLC_ERR_INVALID, "gemm_bf16: null pointer");
  return host_gemm_pipelined(ctx, A, B, C, M, N, K, 2, 2, [&](uint8_t* da, uint8_t* db, uint8_t* dc, int rows, int cols, int) {
    if (K == 0) return aiehlc_gemm_bf16_dev(ctx, nullptr, nullptr, reinterpret_cast<uint16_t*>(dc), rows, cols, 0, ctx->stream);
    return gemm_rect(ctx, KIND_BF16, EPI_BF16, da, db, dc, rows, cols, K, N, 0, nullptr);
  });
}

int aiehlc_conv2d_i8_srs_host(aiehlc_ctx* ctx, const int8_t* x, const int8_t* w, int8_t* y, int n, int h, int wd,
                              int cin, int cout, int kh, int kw, int pad, const uint8_t* shift_vec) {
  int rc = check_ctx(ctx);
  if (rc) return rc;
  if (n < 0 || h < 0 || wd < 0 || cin <= 0 || cout <= 0 || kh <= 0 || kw <= 0 || pad < 0)
    return fail(AIEHLC_ERR_INVALID, "conv2d: bad size");
  if (n == 0 || h == 0 || wd == 0) return AIEHLC_OK;
  if (!x || !w || !y || !shift_vec) return fail(AIEHLC_ERR_INVALID, "conv2d: null pointer");
  for (int j = 0; j < cout; ++j)
    if (shift_vec[j] > 31) return fail(AIEHLC_ERR_INVALID, "srs shift must be in [0, 31]");
  const size_t xb = static_cast<size_t>(n) * h * wd * cin, wb = static_cast<size_t>(kh) * kw * cin * cout,
               yb = static_cast<size_t>(n) * h * wd * cout;
  if ((rc = stage_ab(ctx, x, w, xb, wb, yb))) return rc;
  if (ctx->buf_aux.reserve(cout)) return AIEHLC_ERR_NOMEM;
  AIEHLC_CUDA(cudaMemcpyAsync(ctx->buf_aux.ptr, shift_vec, cout, cudaMemcpyHostToDevice, ctx->stream));
  rc = aiehlc_conv2d_i8_srs_dev(ctx, static_cast<const int8_t*>(ctx->buf_a.ptr),
                                static_cast<const int8_t*>(ctx->buf_b.ptr), static_cast<int8_t*>(ctx->buf_c.ptr),
                                n, h, wd, cin, cout, kh, kw, pad, static_cast<const uint8_t*>(ctx->buf_aux.ptr),
                                ctx->stream);
  if (rc) return rc;
  AIEHLC_CUDA(cudaMemcpyAsync(y, ctx->buf_c.ptr, yb, cudaMemcpyDeviceToHost, ctx->stream));
  return finish_host(ctx);
}

}  // extern "C"
