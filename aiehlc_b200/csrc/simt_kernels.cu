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

// Copies a matrix whose base or row pitch is not 16-byte aligned into a pitched workspace, 16 output
// bytes per thread.  The source bytes of a vector start at any address: they are fetched as five aligned
// 32-bit words and shifted into place; vectors at the very ends of the source (where an aligned word
// would reach outside it) and the ragged end of a row go byte by byte.  Bytes of the workspace past the
// row's true extent are zeroed.
__global__ void repack_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long rows,
                              long long row_bytes, long long ld_src_bytes, long long ld_dst_bytes) {
  const long long vecs_per_row = ld_dst_bytes / 16;
  const uint8_t* const src_end = src + (rows - 1) * ld_src_bytes + row_bytes;
  for (long long row = blockIdx.y; row < rows; row += gridDim.y) {
    const uint8_t* srow = src + row * ld_src_bytes;
    uint4* drow = reinterpret_cast<uint4*>(dst + row * ld_dst_bytes);
    for (long long v = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; v < vecs_per_row;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      const long long b = v * 16;
      const uint8_t* s = srow + b;
      const long long left = row_bytes - b;
      const uintptr_t addr = reinterpret_cast<uintptr_t>(s);
      const unsigned a = static_cast<unsigned>(addr & 3);
      const uint8_t* w0 = s - a;
      uint4 out;
      if (left >= 16 && w0 >= src && w0 + 20 <= src_end) {
        const uint32_t* w = reinterpret_cast<const uint32_t*>(w0);
        const uint32_t x0 = w[0], x1 = w[1], x2 = w[2], x3 = w[3];
        const uint32_t x4 = a ? w[4] : 0u;
        const unsigned sh = a * 8;
        out.x = __funnelshift_r(x0, x1, sh);
        out.y = __funnelshift_r(x1, x2, sh);
        out.z = __funnelshift_r(x2, x3, sh);
        out.w = __funnelshift_r(x3, x4, sh);
      } else {
        uint32_t o[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (j < left) o[j >> 2] |= static_cast<uint32_t>(s[j]) << (8 * (j & 3));
        out = make_uint4(o[0], o[1], o[2], o[3]);
      }
      drow[v] = out;
    }
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

// ---- int32 x int32 -> int32 (mod 2^32) on the int8 tensor cores ---------------------------------
// a = sum_t a_t 2^(8t) with unsigned bytes a_t, likewise b, so
//   a * b mod 2^32 = sum_{s=0..3} 2^(8s) * sum_{t=0..s} a_t * b_(s-t)        (terms with t + u > 3 vanish).
// For every s the inner sums over t AND over k are one int8 GEMM with K' = (s+1) * K: the operand of group
// s is, side by side, limbs 0..s of A (for B: limbs s..0).  A group's sums stay below 2^31 while
// (s+1) * K * 255^2 < 2^31, i.e. K <= 8256, so nothing depends on how the accumulator overflows; longer K
// goes in ranges of 8192 columns.  Four launches per range: group 0 stores (adds, after the first range),
// groups 1..3 add their result shifted left by 8 s (wrapping), which is exactly the reference kernel's
// uint32 arithmetic (example/perf/aieml_perf.cc:74-82).
// src: rows x K int32 (row pitch ld words).  dst: [rows][4 * Kp] bytes, block t of a row holding limb t of
// its K words (reversed: limb 3 - t).  Kp = K rounded up to 16; the padding columns are written as zero.
// Group s of A is then the first (s+1) blocks of every row, group s of B the last (s+1) blocks: the same
// buffer serves all four GEMMs through the row pitch.
__global__ void limb_split_kernel(const uint32_t* __restrict__ src, uint8_t* __restrict__ dst, long long rows, int K,
                                  long long ld, int Kp, int reversed) {
  const long long total = rows * (Kp / 4);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / (Kp / 4);
    const int k = static_cast<int>(i - row * (Kp / 4)) * 4;
    uint32_t v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = (k + e < K) ? src[row * ld + k + e] : 0u;
#pragma unroll
    for (int limb = 0; limb < 4; ++limb) {
      const uint32_t word = ((v[0] >> (8 * limb)) & 0xFFu) | (((v[1] >> (8 * limb)) & 0xFFu) << 8) |
                            (((v[2] >> (8 * limb)) & 0xFFu) << 16) | (((v[3] >> (8 * limb)) & 0xFFu) << 24);
      const int block = reversed ? 3 - limb : limb;
      *reinterpret_cast<uint32_t*>(dst + row * (4LL * Kp) + static_cast<long long>(block) * Kp + k) = word;
    }
  }
}

bool mm_i32_tensor_ok(const aiehlc_ctx* ctx, int M, int N, int K) {
  if (ctx->mm_i32_tensor == 2) return K > 0;   // forced: any size (the 16 x 16 x 16 fixture included)
  return ctx->mm_i32_tensor && K >= 64 && M >= 128 && N >= 64 && static_cast<long long>(M) * N * K >= (1LL << 24);
}

int launch_mm_i32_tensor(aiehlc_ctx* ctx, const int32_t* in, int32_t* out, int M, int N, int K, cudaStream_t st) {
  // K ranges of at most 8192 columns (a multiple of 16 below the 8256 limit), one after the other: the first
  // range's group 0 stores, everything else adds
  const int kc_max = 8192;
  const int kp_max = ((K < kc_max ? K : kc_max) + 15) / 16 * 16;
  if (ctx->limb_a.reserve(static_cast<size_t>(M) * kp_max * 4) || ctx->limb_b.reserve(static_cast<size_t>(N) * kp_max * 4))
    return AIEHLC_ERR_NOMEM;
  const uint32_t* A = reinterpret_cast<const uint32_t*>(in);
  const uint32_t* B = A + static_cast<size_t>(M) * K;
  uint8_t* la = static_cast<uint8_t*>(ctx->limb_a.ptr);
  uint8_t* lb = static_cast<uint8_t*>(ctx->limb_b.ptr);
  for (int k0 = 0; k0 < K; k0 += kc_max) {
    const int kc = K - k0 < kc_max ? K - k0 : kc_max;
    const int Kp = (kc + 15) / 16 * 16;
    limb_split_kernel<<<grid_for(ctx, static_cast<long long>(M) * (Kp / 4), 256), 256, 0, st>>>(A + k0, la, M, kc, K, Kp, 0);
    AIEHLC_CUDA(cudaGetLastError());
    limb_split_kernel<<<grid_for(ctx, static_cast<long long>(N) * (Kp / 4), 256), 256, 0, st>>>(B + k0, lb, N, kc, K, Kp, 1);
    AIEHLC_CUDA(cudaGetLastError());
    ctx->launches += 2;
    for (int s = 0; s < 4; ++s) {
      GemmCall c{};
      c.kind = 0;                                  // int8 operands
      c.epi = (s == 0 && k0 == 0) ? 0 : 1;         // store once, then add
      c.A = la;                                          // limbs 0..s: the first s+1 blocks of a row
      c.B = lb + static_cast<size_t>(3 - s) * Kp;        // limbs s..0: the last s+1 blocks of a row
      c.C = out;
      c.M = M; c.N = N; c.K = (s + 1) * Kp;
      c.lda = 4LL * Kp; c.ldb = 4LL * Kp; c.ldc = N;
      c.unsigned_ab = 1;
      c.operands_from_kernel = 1;                  // the byte planes were written by the kernels just before
      c.out_shift = 8 * s;
      if (int rc = launch_gemm(ctx, c, st)) return rc;
    }
  }
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
  // ld_dst * esize is a multiple of 16 and dst 16-byte aligned (a workspace of this library)
  const long long vecs = ld_dst * esize / 16;
  const unsigned gx = static_cast<unsigned>(vecs > 256 * 4 ? 4 : (vecs + 255) / 256);
  const long long cap = static_cast<long long>(ctx->sm_count) * 16 / gx;
  const unsigned gy = static_cast<unsigned>(rows < cap ? rows : cap);
  repack_kernel<<<dim3(gx ? gx : 1, gy ? gy : 1), 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst),
                                                           rows, cols * esize, ld_src * esize, ld_dst * esize);
  AIEHLC_CUDA(cudaGetLastError());
  ctx->launches++;
  return AIEHLC_OK;
}

}  // namespace aiehlc
