/*
 * aiehlc_kernels.h -- how a kernel named in XAie_LoadElfMem() is bound to a CUDA implementation.
 *
 * In aiehlc a kernel is a `__global__` function in the host file; the compiler cuts it out,
 * builds an AIE ELF and rewrites XAie_LoadElfMem(dev, loc, (unsigned char*)kernel) to load that
 * ELF (src/llvm/aiehlc.cc:301-322).  On B200 the same call looks the function pointer up in a
 * registry.  The host file replaces the kernel *definition* by one declaration macro; the rest
 * of the host code (load, route, move, run, wait) is unchanged:
 *
 *     // was: __global__ void perf(input_window_int32* in, output_window_int32* out) { ...16x16 loop... }
 *     AIEHLC_KERNEL_MM_I32(perf, 16, 16, 16, 0x1000, 0x6000);
 *     ...
 *     XAie_LoadElfMem(DevInst, XAie_TileLoc(4,4), (unsigned char*)perf);   // unchanged
 *
 * Tile data-memory addresses keep their role: `in_addr` / `out_addr` are the addresses the host
 * passes to XAie_MoveData* (the reference's annotate("mem_address:...") / CORE_IP_MEM, CORE_OP_MEM,
 * example/perf/aieml_perf.cc:53-54,61-62).
 */
#ifndef AIEHLC_KERNELS_H
#define AIEHLC_KERNELS_H

#include "xaiengine.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque window types of the reference's kernel signatures (aieml_perf.cc:61-62). */
typedef struct input_window_int32 input_window_int32;
typedef struct output_window_int32 output_window_int32;

/* What a launch callback receives.  Pointers are device pointers into the tile's data memory. */
typedef struct {
  void* in;   u64 in_bytes;    /* region at the kernel's input address (NULL if nothing was moved in) */
  void* out;  u64 out_bytes;   /* region at the kernel's output address (allocated before launch) */
  void* acc;  u64 acc_bytes;   /* region at the kernel's accumulator address (cascade input), or NULL */
  const void* args; u32 args_bytes;
  void* stream;                /* cudaStream_t */
  void* ctx;                   /* aiehlc_ctx* of the device instance (see aiehlc_b200.h) */
  void* user;
} XAie_KernelLaunchInfo;

typedef int (*XAie_KernelLaunchFn)(const XAie_KernelLaunchInfo* info);           /* 0 = ok */
typedef u64 (*XAie_KernelOutBytesFn)(const void* args, u32 args_bytes, u64 in_bytes, void* user);

typedef struct {
  const char* name;
  XAie_KernelLaunchFn launch;
  XAie_KernelOutBytesFn out_bytes;   /* NULL: out_bytes_default */
  u64 out_bytes_default;
  u32 in_addr, out_addr, acc_addr;   /* acc_addr 0 = kernel has no accumulator input */
  const void* default_args; u32 default_args_bytes;
  void* user;
} XAie_KernelDesc;

/* Registers `key` (any unique address, normally a function) as a loadable kernel.  Re-registering
 * a key replaces its description.  Thread-safe. */
AieRC XAie_KernelRegister(const void* key, const XAie_KernelDesc* desc);

/* ---- argument blocks of the library kernels ------------------------------------------------ */
typedef struct { s32 M, N, K; } XAie_MmArgs;

/* Input window of the GEMM kernels: A[M][K] then B[N][K] (B starts at the next multiple of 16
 * bytes), then, if has_shift_vec, N shift bytes (again 16-byte aligned).  Output window: C[M][N].
 * Accumulator window (gemm_i8_srs only, optional): int32 partial sums [M][N] added before srs. */
typedef struct {
  s32 M, N, K;
  s32 shift;          /* srs shift when has_shift_vec == 0 */
  s32 has_shift_vec;
  s32 splitk;         /* slices accumulated inside one launch (>= 1, divides K) */
  s32 accumulate;     /* gemm_i8_i32: C += A.B^T (C is the tile's output window, kept across runs) */
  s32 use_acc;        /* gemm_i8_srs: add the accumulator window before srs */
} XAie_GemmArgs;

/* Input window of the conv kernel: x NHWC, then w HWIO, then cout shift bytes, each part starting
 * at a multiple of 16 bytes.  Output window: y NHWC. */
typedef struct { s32 n, h, w, cin, cout, kh, kw, pad; } XAie_ConvArgs;

/* srs flush of an int32 window: input int32 [rows][cols] (+ cols shift bytes if has_shift_vec). */
typedef struct { s32 rows, cols, shift, has_shift_vec; } XAie_SrsArgs;

/* ---- library kernels: pass these to XAie_LoadElfMem, set sizes with XAie_KernelSetArgs ------
 * Default window addresses: in 0x1000, out 0x6000, accumulator 0x3000. */
void aiehlc_k_mm_i32(input_window_int32* in, output_window_int32* out);   /* the reference's perf / mm */
void aiehlc_k_gemm_i8_i32(const s8* in, s32* out);
void aiehlc_k_gemm_i8_srs(const s8* in, s8* out);
void aiehlc_k_gemm_bf16(const u16* in, u16* out);
void aiehlc_k_conv2d_i8_srs(const s8* in, s8* out);
void aiehlc_k_srs_i32_i8(const s32* in, s8* out);

u64 aiehlc_window_offset_b(const XAie_GemmArgs* a, u32 elem_bytes);      /* byte offset of B in the input window */
u64 aiehlc_window_offset_shift(const XAie_GemmArgs* a, u32 elem_bytes);  /* byte offset of the shift vector */
u64 aiehlc_conv_offset_w(const XAie_ConvArgs* a);
u64 aiehlc_conv_offset_shift(const XAie_ConvArgs* a);

/* Binds a local symbol to one of the library kernels with fixed arguments and window addresses. */
AieRC XAie_KernelBind(const void* key, const char* name, const void* library_kernel, const void* args,
                      u32 args_bytes, u32 in_addr, u32 out_addr, u32 acc_addr);

/* The kernel-call form k<Col,Row,colstart,rowstart,M,N,K>(in, out) of
 * example/nokernelload/aie_nokernelload.cc:130 as one blocking call: loads `kernel_key` on tile
 * (colstart,rowstart), sets its arguments, moves the GMIO data at host address `in` to the kernel's
 * input window, runs it, and moves what the kernel produced back to host address `out` (both addresses
 * must lie inside buffers from XAie_MemAllocate; the call runs on the device instance that owns the
 * input buffer, so host threads with an instance each can call side by side).
 * Col x Row is the tile grid the caller asks for.  On the AIE array it is the number of tiles the kernel
 * is spread over; here it is the number of SMs: the persistent tensor-core GEMM kernels pick their tile
 * shape and waves for Col x Row SMs (aiehlc_plan_gemm with that limit) and launch no more CTAs than
 * that -- 8 x 16 = 128 of a B200's 148, 1 x 1 = a single CTA.  Kernels without a persistent grid (the
 * int32 CUDA-core kernel, conv, srs) size their grid from the problem.
 * Allocation: the tile's windows are created by the first call and reused; a later call whose operands
 * and result fit in them allocates nothing. */
AieRC XAie_KernelCall(const void* kernel_key, const void* args, u32 args_bytes, int Col, int Row, int colstart,
                      int rowstart, u64 in, u64 out);

#ifdef __cplusplus
}  /* extern "C" */
#endif

#ifdef __cplusplus
/* C++ declaration of a kernel in the call form.  aiehlc injects
 *     template <int Col, int Row, int colstart, int rowstart, int M, int N, int K, typename... Args>
 *     inline void NAME(Args&&... args) { return; }
 * in front of the user's source (src/llvm/aiehlc.cc:583-588); these macros declare the same template
 * with a body that runs the kernel, so `NAME<1,1,4,4,16,16,16>(phy, phy_out);` compiles unchanged.
 * AieRC of the last call: XAie_KernelCallStatus(). */
inline AieRC& XAie_KernelCallStatus() {
  static thread_local AieRC rc = XAIE_OK;
  return rc;
}
#define AIEHLC_KERNEL_CALL_MM_I32(NAME)                                                               \
  template <int Col, int Row, int colstart, int rowstart, int M, int N, int K, typename... Args>      \
  inline void NAME(Args&&... args) {                                                                  \
    static_assert(sizeof...(Args) == 2, "kernel call takes (in, out)");                               \
    const u64 io[2] = {(u64)(args)...};                                                               \
    const XAie_MmArgs a = {M, N, K};                                                                  \
    XAie_KernelCallStatus() = XAie_KernelCall((const void*)aiehlc_k_mm_i32, &a, sizeof a, Col, Row,   \
                                              colstart, rowstart, io[0], io[1]);                      \
  }
/* int8 GEMM + srs (shift, split-K fixed at declaration), input window A | B, output window C int8 */
#define AIEHLC_KERNEL_CALL_GEMM_I8_SRS(NAME, SHIFT, SPLITK)                                           \
  template <int Col, int Row, int colstart, int rowstart, int M, int N, int K, typename... Args>      \
  inline void NAME(Args&&... args) {                                                                  \
    static_assert(sizeof...(Args) == 2, "kernel call takes (in, out)");                               \
    const u64 io[2] = {(u64)(args)...};                                                               \
    const XAie_GemmArgs a = {M, N, K, (SHIFT), 0, (SPLITK), 0, 0};                                    \
    XAie_KernelCallStatus() = XAie_KernelCall((const void*)aiehlc_k_gemm_i8_srs, &a, sizeof a, Col,   \
                                              Row, colstart, rowstart, io[0], io[1]);                 \
  }
#define AIEHLC_KERNEL_CALL_GEMM_I8_I32(NAME)                                                          \
  template <int Col, int Row, int colstart, int rowstart, int M, int N, int K, typename... Args>      \
  inline void NAME(Args&&... args) {                                                                  \
    static_assert(sizeof...(Args) == 2, "kernel call takes (in, out)");                               \
    const u64 io[2] = {(u64)(args)...};                                                               \
    const XAie_GemmArgs a = {M, N, K, 0, 0, 1, 0, 0};                                                 \
    XAie_KernelCallStatus() = XAie_KernelCall((const void*)aiehlc_k_gemm_i8_i32, &a, sizeof a, Col,   \
                                              Row, colstart, rowstart, io[0], io[1]);                 \
  }
#endif

/* Declaration macros: define a symbol with the reference kernel's name and register it before
 * main() runs.  The symbol is never called on the host; its address is the registry key. */
#if defined(__GNUC__)
#define AIEHLC_CTOR_(name) static void __attribute__((constructor)) aiehlc_ctor_##name(void)
#else
#error "aiehlc_kernels.h needs constructor functions (gcc / clang / nvcc host compiler)"
#endif

#define AIEHLC_KERNEL_MM_I32(name, M_, N_, K_, in_addr_, out_addr_)                              \
  void name(input_window_int32* in_unused, output_window_int32* out_unused) {                    \
    (void)in_unused; (void)out_unused;                                                           \
  }                                                                                              \
  AIEHLC_CTOR_(name) {                                                                           \
    static const XAie_MmArgs a = {(M_), (N_), (K_)};                                             \
    XAie_KernelBind((const void*)name, #name, (const void*)aiehlc_k_mm_i32, &a, sizeof a,        \
                    (in_addr_), (out_addr_), 0);                                                 \
  }

#define AIEHLC_KERNEL_GEMM(name, library_kernel, M_, N_, K_, shift_, splitk_, in_addr_, out_addr_) \
  void name(void* in_unused, void* out_unused) { (void)in_unused; (void)out_unused; }             \
  AIEHLC_CTOR_(name) {                                                                            \
    static const XAie_GemmArgs a = {(M_), (N_), (K_), (shift_), 0, (splitk_), 0, 0};              \
    XAie_KernelBind((const void*)name, #name, (const void*)library_kernel, &a, sizeof a,          \
                    (in_addr_), (out_addr_), 0);                                                  \
  }

/* A kernel written by the user in CUDA: `launch_expr` is a statement that launches it on
 * `stream` with the device pointers `in` and `out` (int*), e.g.
 *     __global__ void k1_cuda(int* in, int* out) { for (int i = 0; i < 20; ++i) out[i] = *in + 1; }
 *     AIEHLC_KERNEL_CUDA(k1, 0x1000, 0x5000, 80, k1_cuda<<<1, 1, 0, stream>>>(in, out));
 * The launch runs in the user's translation unit, so it uses the user's CUDA runtime. */
#define AIEHLC_KERNEL_CUDA(name, in_addr_, out_addr_, out_bytes_, launch_expr)                    \
  void name(int* in_unused, int* out_unused) { (void)in_unused; (void)out_unused; }               \
  static int aiehlc_launch_##name(const XAie_KernelLaunchInfo* info) {                            \
    int* in = (int*)info->in;                                                                     \
    int* out = (int*)info->out;                                                                   \
    cudaStream_t stream = (cudaStream_t)info->stream;                                             \
    (void)in; (void)out; (void)stream;                                                            \
    launch_expr;                                                                                  \
    return (int)cudaGetLastError();                                                               \
  }                                                                                               \
  AIEHLC_CTOR_(name) {                                                                            \
    XAie_KernelDesc d = {#name, aiehlc_launch_##name, 0, (out_bytes_), (in_addr_), (out_addr_), 0, \
                         0, 0, 0};                                                                \
    XAie_KernelRegister((const void*)name, &d);                                                   \
  }

#endif /* AIEHLC_KERNELS_H */
