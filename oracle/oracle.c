/*
 * CPU oracle for the aiehlc matmul hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's kernels and of its in-file
 * CPU golden check.  It exists to check the CUDA path; nothing in the product (the aiehlc_b200
 * package, libaiehlc_b200.so) calls, links or imports it.  Only tests/, __graft_entry__.smoke()
 * and the cpu_baseline / reference legs of bench.py may use it.
 *
 * Parity status
 *   pinned   : oracle_mm_i32 -- against the known answers of the reference's own fixtures
 *              (example/perf/aieml_perf.cc:141-144, example/matrixmultiply/aieml_mm.cc:137-140,
 *              example/other/aieoob.c:83-86) and against the output of the reference's own
 *              `perf` kernel + golden loop compiled from its source (oracle/_ref, see ref_build.sh).
 *   pinned by construction: oracle_gemm_i8_i32 is the same loop nest with int8 operands
 *              sign-extended to 32 bits; tests check it against oracle_mm_i32 on widened inputs.
 *   UNPINNED : srs, split-K order, conv2d, bf16 -- the reference contains none of them
 *              ("parity unpinned").  Their definitions below are the written contract.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* The reference kernel and golden, generalised from N=16 to (M,N,K).
 *   kernel : example/perf/aieml_perf.cc:72-82   ret = 0; ret += vec1[i*N+k] * vec2[j*N+k]  (uint32_t)
 *   golden : example/perf/aieml_perf.cc:199-231 A_mat[i][j] = in[i*N+j]; B_mat[i][j] = in[MAT_SIZE+i*N+j];
 *            result zero-initialised (:201); result[i][j] += A_mat[i][k] * B_mat[j][k]; row-major flatten
 *   same loop in example/matrixmultiply/aieml_mm.cc:198-230 and example/other/aieoob.c:101-133.
 * `in` = A (M*K words) followed by B (N*K words) -- the packed window the examples fill.
 * uint32 wrap-around makes the int32 golden and the uint32 kernel one function. */
void oracle_mm_i32(const int32_t* in, int32_t* out, int M, int N, int K) {
  const uint32_t* A = (const uint32_t*)in;
  const uint32_t* B = (const uint32_t*)in + (size_t)M * K;
  for (int i = 0; i < M; i++)
    for (int j = 0; j < N; j++) {
      uint32_t ret = 0;
      for (int k = 0; k < K; k++) ret += A[(size_t)i * K + k] * B[(size_t)j * K + k];
      ((uint32_t*)out)[(size_t)i * N + j] = ret;
    }
}

/* Same contraction, int8 operands widened to int32, int32 accumulate
 * (aieml_perf.cc:199-231 with A[M][K] row-major, B stored [N][K]). */
void oracle_gemm_i8_i32(const int8_t* A, const int8_t* B, int32_t* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; i++) {
    const int8_t* a = A + (size_t)i * K;
    for (int j = 0; j < N; j++) {
      const int8_t* b = B + (size_t)j * K;
      int32_t acc = 0;
      for (int k = 0; k < K; k++) acc += (int32_t)a[k] * (int32_t)b[k];
      C[(size_t)i * N + j] = acc;
    }
  }
}

/* Shift-round-saturate (no counterpart in the reference; definition fixed by the project's
 * benchmark configuration: "shift = s, round half to even, saturating to int8"):
 *   q = acc >> s (arithmetic, floor); r = acc & (2^s - 1); h = 2^(s-1)
 *   q += 1 if r > h, or r == h and q is odd;  result = clamp(q, -128, 127);  s = 0: clamp only. */
int8_t oracle_srs_i8(int32_t acc, int s) {
  int64_t q = acc;
  if (s > 0) {
    const int64_t a = acc;
    q = a >> s;
    const int64_t r = a & (((int64_t)1 << s) - 1);
    const int64_t h = (int64_t)1 << (s - 1);
    if (r > h || (r == h && (q & 1))) q += 1;
  }
  if (q > 127) q = 127;
  if (q < -128) q = -128;
  return (int8_t)q;
}

void oracle_srs_i32_i8(const int32_t* in, int8_t* out, long long rows, long long cols, int shift,
                       const uint8_t* shift_vec) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < rows; i++)
    for (long long j = 0; j < cols; j++)
      out[i * cols + j] = oracle_srs_i8(in[i * cols + j], shift_vec ? (int)shift_vec[j] : shift);
}

/* int8 GEMM + srs.  splitk > 1: partial int32 sums over equal contiguous K slices, added in slice
 * order, srs once after the last slice (the cascade formulation; chain pattern of
 * example/multi/multi_tile.cpp:105-145).  acc_in (optional) is added before srs. */
void oracle_gemm_i8_srs(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K, int shift,
                        const uint8_t* shift_vec, const int32_t* acc_in, int splitk) {
  if (splitk < 1) splitk = 1;
  const int ks = K / splitk;
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; i++) {
    const int8_t* a = A + (size_t)i * K;
    for (int j = 0; j < N; j++) {
      const int8_t* b = B + (size_t)j * K;
      uint32_t total = acc_in ? (uint32_t)acc_in[(size_t)i * N + j] : 0u;
      for (int s = 0; s < splitk; s++) {
        int32_t part = 0;
        const int k1 = (s == splitk - 1) ? K : (s + 1) * ks;
        for (int k = s * ks; k < k1; k++) part += (int32_t)a[k] * (int32_t)b[k];
        total += (uint32_t)part;
      }
      C[(size_t)i * N + j] = oracle_srs_i8((int32_t)total, shift_vec ? (int)shift_vec[j] : shift);
    }
  }
}

/* conv2d, direct 7-loop nest (no counterpart in the reference):
 *   y[n][oh][ow][co] = srs( sum_{kh,kw,ci} x[n][oh+kh-pad][ow+kw-pad][ci] * w[kh][kw][ci][co], shift_vec[co] )
 * x NHWC, w HWIO, stride 1, out-of-range x = 0, output spatial size = input spatial size. */
void oracle_conv2d_i8_srs(const int8_t* x, const int8_t* w, int8_t* y, int n, int h, int wd, int cin,
                          int cout, int kh, int kw, int pad, const uint8_t* shift_vec) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int in_ = 0; in_ < n; in_++)
    for (int oh = 0; oh < h; oh++)
      for (int ow = 0; ow < wd; ow++)
        for (int co = 0; co < cout; co++) {
          int32_t acc = 0;
          for (int fh = 0; fh < kh; fh++) {
            const int ih = oh + fh - pad;
            if (ih < 0 || ih >= h) continue;
            for (int fw = 0; fw < kw; fw++) {
              const int iw = ow + fw - pad;
              if (iw < 0 || iw >= wd) continue;
              const int8_t* xp = x + (((size_t)in_ * h + ih) * wd + iw) * cin;
              const int8_t* wp = w + ((size_t)(fh * kw + fw) * cin) * cout + co;
              for (int ci = 0; ci < cin; ci++) acc += (int32_t)xp[ci] * (int32_t)wp[(size_t)ci * cout];
            }
          }
          y[(((size_t)in_ * h + oh) * wd + ow) * cout + co] = oracle_srs_i8(acc, shift_vec[co]);
        }
}

static float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);  /* quiet NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* bf16 GEMM reference values (no counterpart in the reference): products of the bf16 inputs
 * accumulated in fp32 in k order; C32 receives the fp32 sums, Cbf (optional) their bf16 rounding. */
void oracle_gemm_bf16(const uint16_t* A, const uint16_t* B, float* C32, uint16_t* Cbf, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; i++) {
    const uint16_t* a = A + (size_t)i * K;
    for (int j = 0; j < N; j++) {
      const uint16_t* b = B + (size_t)j * K;
      float acc = 0.f;
      for (int k = 0; k < K; k++) acc += bf16_to_f32(a[k]) * bf16_to_f32(b[k]);
      if (C32) C32[(size_t)i * N + j] = acc;
      if (Cbf) Cbf[(size_t)i * N + j] = f32_to_bf16_rne(acc);
    }
  }
}
