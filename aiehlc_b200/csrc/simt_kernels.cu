// CUDA-core kernels around the tensor-core path: the reference's own int32 matmul (which has
// no tensor-core data type), the element-wise srs flush, and small data-movement helpers.
#include "context.h"
#include "gemm_tcgen05.cuh"  // srs_i8

namespace aiehlc {

// out[i*N+j] = sum_k A[i*K+k] * B[j*K+k] in uint32 wrap-around arithmetic, accumulator zeroed
// per output -- the loop of example/perf/aieml_perf.cc:74-82 (kernel) and :199-231 (golden).
// `in` = A (M*K words) followed by B (N*K words), as the examples pack their input window.
// Register-tiled: a CTA of 256 threads owns a 64 x 64 tile of C and walks K in steps of 16; every thread
// keeps a 4 x 4 block of outputs, so one pair of 16-byte shared-memory reads feeds 16 multiply-adds.
constexpr int kMmTile = 64;
constexpr int kMmK = 16;
__global__ void __launch_bounds__(256) mm_i32_kernel(const uint32_t* __restrict__ in,
                                                     uint32_t* __restrict__ out, int M, int N, int K) {
  // [k][row]: the 4 rows (or columns) a thread needs are contiguous; +4 words keeps the 16-byte alignment
  // and spreads the transposing stores over the banks
  __shared__ __align__(16) uint32_t sa[kMmK][kMmTile + 4];
  __shared__ __align__(16) uint32_t sb[kMmK][kMmTile + 4];
  const uint32_t* A = in;
  const uint32_t* B = in + static_cast<size_t>(M) * K;
  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;          // 16 x 16 threads, 4 x 4 outputs each
  const int lrow = t >> 2, lk = (t & 3) * 4;   // loader: tile row 0..63, k offset 0/4/8/12
  const int row0 = blockIdx.y * kMmTile, col0 = blockIdx.x * kMmTile;
  const bool vec = (K % 4 == 0) && (reinterpret_cast<uintptr_t>(in) % 16 == 0) &&
                   ((static_cast<size_t>(M) * K) % 4 == 0);
  uint32_t acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += kMmK) {
    uint32_t av[4] = {0, 0, 0, 0}, bv[4] = {0, 0, 0, 0};
    const int k = k0 + lk;
    if (row0 + lrow < M) {
      const uint32_t* src = A + static_cast<size_t>(row0 + lrow) * K + k;
      if (vec && k + 3 < K) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        av[0] = v.x; av[1] = v.y; av[2] = v.z; av[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (k + i < K) av[i] = src[i];
      }
    }
    if (col0 + lrow < N) {
      const uint32_t* src = B + static_cast<size_t>(col0 + lrow) * K + k;
      if (vec && k + 3 < K) {
        const uint4 v = *reinterpret_cast<const uint4*>(src);
        bv[0] = v.x; bv[1] = v.y; bv[2] = v.z; bv[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (k + i < K) bv[i] = src[i];
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sa[lk + i][lrow] = av[i];
      sb[lk + i][lrow] = bv[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMmK; ++kk) {
      const uint4 a = *reinterpret_cast<const uint4*>(&sa[kk][ty * 4]);
      const uint4 b = *reinterpret_cast<const uint4*>(&sb[kk][tx * 4]);
      const uint32_t ar[4] = {a.x, a.y, a.z, a.w}, br[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] += ar[r] * br[c];   // uint32: wraps like the reference's loop
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int row = row0 + ty * 4 + r;
    if (row >= M) continue;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int col = col0 + tx * 4 + c;
      if (col < N) out[static_cast<size_t>(row) * N + col] = acc[r][c];
    }
  }
}

__global__ void srs_flush_kernel(const int32_t* __restrict__ in, int8_t* __restrict__ out,
                                 long long rows, long long cols, int shift,
                                 const uint8_t* __restrict__ shift_vec) {
  const long long n = rows * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int s = shift_vec ? static_cast<int>(shift_vec[i % cols]) : shift;
    out[i] = static_cast<int8_t>(srs_i8(in[i], s));
  }
}

__global__ void fill_i32_kernel(int32_t* out, long long n, int value) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = value;
}

template <typename T>
__global__ void repack_kernel(const T* __restrict__ src, T* __restrict__ dst, long long rows,
                              long long cols, long long ld_src, long long ld_dst) {
  const long long n = rows * cols;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    dst[r * ld_dst + c] = src[r * ld_src + c];
  }
}

static int grid_for(aiehlc_ctx* ctx, long long n, int block) {
  long long g = (n + block - 1) / block;
  const long long cap = static_cast<long long>(ctx->sm_count) * 8;
  if (g > cap) g = cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

int launch_mm_i32(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K,
                  cudaStream_t st) {
  dim3 grid((N + kMmTile - 1) / kMmTile, (M + kMmTile - 1) / kMmTile);
  mm_i32_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t*>(in),
                                      reinterpret_cast<uint32_t*>(out), M, N, K);
  AIEHLC_CUDA(cudaGetLastError());
  ctx->launches++;
  return AIEHLC_OK;
}

int launch_srs(aiehlc_ctx* ctx, const int32_t* in, int8_t* out, long long rows, long long cols,
               int shift, const uint8_t* shift_vec, cudaStream_t st) {
  srs_flush_kernel<<<grid_for(ctx, rows * cols, 256), 256, 0, st>>>(in, out, rows, cols, shift,
                                                                    shift_vec);
  AIEHLC_CUDA(cudaGetLastError());
  ctx->launches++;
  return AIEHLC_OK;
}

int launch_fill_i32(aiehlc_ctx* ctx, int32_t* out, long long n, int value, cudaStream_t st) {
  fill_i32_kernel<<<grid_for(ctx, n, 256), 256, 0, st>>>(out, n, value);
  AIEHLC_CUDA(cudaGetLastError());
  ctx->launches++;
  return AIEHLC_OK;
}

int launch_repack(aiehlc_ctx* ctx, const void* src, void* dst, long long rows, long long cols,
                  long long ld_src, long long ld_dst, int esize, cudaStream_t st) {
  const int g = grid_for(ctx, rows * cols, 256);
  if (esize == 1)
    repack_kernel<uint8_t><<<g, 256, 0, st>>>(static_cast<const uint8_t*>(src),
                                             static_cast<uint8_t*>(dst), rows, cols, ld_src, ld_dst);
  else
    repack_kernel<uint16_t><<<g, 256, 0, st>>>(static_cast<const uint16_t*>(src),
                                              static_cast<uint16_t*>(dst), rows, cols, ld_src, ld_dst);
  AIEHLC_CUDA(cudaGetLastError());
  ctx->launches++;
  return AIEHLC_OK;
}

}  // namespace aiehlc
