"""Python face of the kernel-call path: one `Context` per GPU, methods named after the C ABI.

Device methods take and return CUDA torch tensors (torch is used for device memory and streams
only; every computation is a call into libaiehlc_b200.so on torch's current stream).  Host
methods take and return numpy arrays and go through the `_host` entry points, which copy
host -> device, run the kernel and copy back.

Layout contract (the reference's golden loop, example/perf/aieml_perf.cc:199-231):
A[M][K] row-major, B stored [N][K], C[M][N] row-major.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _capi


def _np_ptr(a: np.ndarray | None) -> C.c_void_p:
    return C.c_void_p(None) if a is None else C.c_void_p(a.ctypes.data)


def plan_gemm(M: int, N: int, K: int, kind: str = "int8", ctx: "Context | None" = None) -> dict:
    """The tiling the GEMM entry points use for this problem (aiehlc_plan_gemm); needs no GPU when
    ctx is None (planned for a 148-SM B200 with default knobs)."""
    plan = _capi.GemmPlan()
    h = ctx._h if ctx is not None else C.c_void_p(None)
    _capi.check(_capi.load().aiehlc_plan_gemm(h, {"int8": 0, "bf16": 1}[kind], int(M), int(N), int(K), C.byref(plan)))
    return plan.as_dict()


def plan_conv2d(n: int, h: int, w: int, cin: int, cout: int, kh: int = 3, kw: int = 3, pad: int = 1,
                ctx: "Context | None" = None) -> dict:
    """The form and tiling the convolution entry points use for this problem (aiehlc_plan_conv2d); needs no GPU
    when ctx is None."""
    plan = _capi.ConvPlan()
    hdl = ctx._h if ctx is not None else C.c_void_p(None)
    _capi.check(_capi.load().aiehlc_plan_conv2d(hdl, int(n), int(h), int(w), int(cin), int(cout), int(kh), int(kw),
                                                int(pad), C.byref(plan)))
    return plan.as_dict()


def plan_tile_order(M: int, N: int, K: int, kind: str = "int8", num_shards: int = 0, rows_per_shard: int = 0,
                    first_shard: int = 0, ctx: "Context | None" = None):
    """(row_block, col_block) of every tile in the order a launch visits them, and the number of persistent
    CTAs (or pairs) that share them round-robin (aiehlc_plan_tile_order); needs no GPU when ctx is None."""
    import numpy as np
    plan = plan_gemm(M, N, K, kind, ctx)
    n = int(plan["tiles"])
    rb = np.empty(n, dtype=np.int32)
    cb = np.empty(n, dtype=np.int32)
    slots = C.c_int(0)
    h = ctx._h if ctx is not None else C.c_void_p(None)
    got = _capi.load().aiehlc_plan_tile_order(h, {"int8": 0, "bf16": 1}[kind], int(M), int(N), int(K), int(num_shards),
                                              int(rows_per_shard), int(first_shard), rb.ctypes.data, cb.ctypes.data, n,
                                              C.byref(slots))
    if got < 0:
        _capi.check(got)
    return rb[:got], cb[:got], int(slots.value)


class Context:
    """Owns an `aiehlc_ctx` (device bring-up; stands in for the XAie_CfgInitialize /
    XAie_PartitionInitialize sequence of example/perf/aieml_perf.cc:265-313)."""

    def __init__(self, device: int = 0):
        self._lib = _capi.load()
        h = C.c_void_p()
        _capi.check(self._lib.aiehlc_create(int(device), C.byref(h)))
        self._h = h
        self.device = int(device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.aiehlc_destroy(self._h)
            self._h = None

    def __del__(self):  # noqa: D105
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass

    # ------------------------------------------------------------------ misc
    @property
    def sm_count(self) -> int:
        return self._lib.aiehlc_sm_count(self._h)

    @property
    def launch_count(self) -> int:
        return int(self._lib.aiehlc_launch_count(self._h))

    def set_tile_n(self, tile_n: int) -> None:
        _capi.check(self._lib.aiehlc_set_tile_n(self._h, int(tile_n)))

    def set_cta_pair(self, mode: int) -> None:
        _capi.check(self._lib.aiehlc_set_cta_pair(self._h, int(mode)))

    def set_host_blocks(self, blocks: int) -> None:
        _capi.check(self._lib.aiehlc_set_host_blocks(self._h, int(blocks)))

    def set_conv_hwio_direct(self, on: bool) -> None:
        _capi.check(self._lib.aiehlc_set_conv_hwio_direct(self._h, 1 if on else 0))

    def set_mm_i32_tensor(self, mode) -> None:
        """0/False: CUDA cores only, 1/True: tensor cores for large products (default), 2: tensor cores always."""
        _capi.check(self._lib.aiehlc_set_mm_i32_tensor(self._h, int(mode)))

    def set_conv_wide_n(self, on: bool) -> None:
        _capi.check(self._lib.aiehlc_set_conv_wide_n(self._h, 1 if on else 0))

    def set_conv_persistent(self, on) -> None:
        """0/False: one CTA per tile; 1/True: persistent form where it applies; 2 / 3: the same with the MMAs of one tile
        at a time / of two tiles interleaved."""
        _capi.check(self._lib.aiehlc_set_conv_persistent(self._h, int(on)))

    def set_conv_halo(self, on: bool) -> None:
        _capi.check(self._lib.aiehlc_set_conv_halo(self._h, 1 if on else 0))

    def set_shard_tile_stores(self, on: bool) -> None:
        _capi.check(self._lib.aiehlc_set_shard_tile_stores(self._h, 1 if on else 0))

    def set_k_per_load(self, k_blocks: int) -> None:
        _capi.check(self._lib.aiehlc_set_k_per_load(self._h, int(k_blocks)))

    def set_tma_store(self, mode: int) -> None:
        """0: per-thread stores, 1: tile stores for int32/bf16 results (default), 2: for int8 results too."""
        _capi.check(self._lib.aiehlc_set_tma_store(self._h, int(mode)))

    def set_epilogue_groups(self, groups: int) -> None:
        """CTA-pair kernel: 1 or 2 groups of four epilogue warps; 0 (default) chooses by K."""
        _capi.check(self._lib.aiehlc_set_epilogue_groups(self._h, int(groups)))

    def set_split_tail(self, mode) -> None:
        """Last wave at most half full: 0/False = tiles whole, 1/True = K halves, 2 = column ranges, 3 = choose (default)."""
        _capi.check(self._lib.aiehlc_set_split_tail(self._h, int(mode)))

    def set_group_m(self, group_m: int) -> None:
        _capi.check(self._lib.aiehlc_set_group_m(self._h, int(group_m)))

    def set_cta_limit(self, sms: int) -> None:
        """SMs the persistent GEMM kernels may occupy (0 = all)."""
        _capi.check(self._lib.aiehlc_set_cta_limit(self._h, int(sms)))

    def set_operands_ready(self, on: bool) -> None:
        """Promise that GEMM operands are never written by the kernel just before the call in its stream: loader and
        multiplier warps then start while that kernel drains (aiehlc_set_operands_ready)."""
        _capi.check(self._lib.aiehlc_set_operands_ready(self._h, 1 if on else 0))

    def set_pdl(self, on: bool) -> None:
        _capi.check(self._lib.aiehlc_set_pdl(self._h, 1 if on else 0))

    def set_debug(self, mode: int) -> None:
        _capi.check(self._lib.aiehlc_set_debug(self._h, int(mode)))

    def set_trace(self, buf) -> None:
        """buf: int64 CUDA tensor (8 words per tile of one CTA) or None."""
        import torch
        ptr = C.c_void_p(None) if buf is None else self._dev(buf, torch.int64, "trace")
        _capi.check(self._lib.aiehlc_set_trace(self._h, ptr))

    def set_cta_times(self, buf) -> None:
        """buf: int64 CUDA tensor of 2 * 148 words (entry / exit nanoseconds of every CTA of a pair launch) or None."""
        import torch
        ptr = C.c_void_p(None) if buf is None else self._dev(buf, torch.int64, "cta_times")
        _capi.check(self._lib.aiehlc_set_cta_times(self._h, ptr))

    def sync(self, on_torch_stream: bool = True) -> int:
        """Waits for the stream and returns the device status word (raises if it is non-zero)."""
        st = C.c_int32(0)
        stream = self._stream() if on_torch_stream else C.c_void_p(None)
        _capi.check(self._lib.aiehlc_sync(self._h, stream, C.byref(st)))
        return st.value

    def _stream(self) -> C.c_void_p:
        import torch
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _dev(self, t, dtype, name):
        import torch
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.device.index != self.device:
            raise TypeError(f"{name}: expected a CUDA tensor on device {self.device}")
        if t.dtype != dtype:
            raise TypeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
        if not t.is_contiguous():
            raise ValueError(f"{name}: tensor must be contiguous")
        return C.c_void_p(t.data_ptr())

    # ------------------------------------------------ pre-bound calls for launch-rate-bound loops
    def bound_gemm_i8_srs(self, A, B, out, shift: int = 0, splitk: int = 1):
        """Returns a zero-argument callable that issues aiehlc_gemm_i8_srs_dev on torch's current stream
        with every argument converted once (the per-call Python work drops to one foreign call)."""
        import torch
        (M, K), N = A.shape, B.shape[0]
        args = (self._h, self._dev(A, torch.int8, "A"), self._dev(B, torch.int8, "B"), self._dev(out, torch.int8, "C"),
                M, N, K, int(shift), C.c_void_p(None), C.c_void_p(None), int(splitk), self._stream())
        fn, check = self._lib.aiehlc_gemm_i8_srs_dev, _capi.check
        return lambda: check(fn(*args))

    def bound_gemm_i8_i32(self, A, B, out, accumulate: bool = False):
        import torch
        (M, K), N = A.shape, B.shape[0]
        args = (self._h, self._dev(A, torch.int8, "A"), self._dev(B, torch.int8, "B"), self._dev(out, torch.int32, "C"),
                M, N, K, 1 if accumulate else 0, self._stream())
        fn, check = self._lib.aiehlc_gemm_i8_i32_dev, _capi.check
        return lambda: check(fn(*args))

    def bound_gemm_bf16(self, A, B, out):
        import torch
        (M, K), N = A.shape, B.shape[0]
        args = (self._h, self._dev(A, torch.bfloat16, "A"), self._dev(B, torch.bfloat16, "B"),
                self._dev(out, torch.bfloat16, "C"), M, N, K, self._stream())
        fn, check = self._lib.aiehlc_gemm_bf16_dev, _capi.check
        return lambda: check(fn(*args))

    def bound_conv2d_i8_srs(self, x, w, shift_vec, out, pad: int = 1):
        import torch
        n, h, wd, cin = x.shape
        kh, kw, _, cout = w.shape
        args = (self._h, self._dev(x, torch.int8, "x"), self._dev(w, torch.int8, "w"), self._dev(out, torch.int8, "y"),
                n, h, wd, cin, cout, kh, kw, int(pad), self._dev(shift_vec, torch.uint8, "shift_vec"), self._stream())
        fn, check = self._lib.aiehlc_conv2d_i8_srs_dev, _capi.check
        return lambda: check(fn(*args))

    # --------------------------------------------------------- device tensors
    def mm_i32(self, packed, M: int, N: int, K: int, out=None):
        """The reference's `perf` / `mm` kernel: packed = A (M*K int32) then B (N*K int32)."""
        import torch
        if packed.numel() < (M + N) * K:
            raise ValueError("mm_i32: input window shorter than (M+N)*K words")
        if out is None:
            out = torch.empty((M, N), dtype=torch.int32, device=packed.device)
        _capi.check(self._lib.aiehlc_mm_i32_dev(self._h, self._dev(packed, torch.int32, "in"),
                                                self._dev(out, torch.int32, "out"), M, N, K, self._stream()))
        return out

    def gemm_i8_i32(self, A, B, out=None, accumulate: bool = False):
        import torch
        M, K = A.shape
        N, K2 = B.shape
        if K != K2:
            raise ValueError("gemm_i8_i32: A is [M][K], B is [N][K]; K differs")
        if out is None:
            if accumulate:
                raise ValueError("gemm_i8_i32: accumulate needs an existing output")
            out = torch.empty((M, N), dtype=torch.int32, device=A.device)
        _capi.check(self._lib.aiehlc_gemm_i8_i32_dev(
            self._h, self._dev(A, torch.int8, "A"), self._dev(B, torch.int8, "B"),
            self._dev(out, torch.int32, "C"), M, N, K, 1 if accumulate else 0, self._stream()))
        return out

    def bound_gemm_i8_i32_scatter(self, A, B, shard_ptrs, rows_per_shard: int, N: int, first_shard: int = 0):
        """C += A . B^T with rows [g * rows_per_shard, ...) of C at device address shard_ptrs[g] (dense int32
        [rows][N]; may be another GPU's memory).  Returns a callable that issues the launch."""
        import ctypes
        import torch
        M, K = A.shape
        if B.shape != (N, K):
            raise ValueError("gemm_i8_i32_scatter: B must be [N][K]")
        arr = (ctypes.c_void_p * len(shard_ptrs))(*[int(p) for p in shard_ptrs])
        args = (self._h, self._dev(A, torch.int8, "A"), self._dev(B, torch.int8, "B"), arr, len(shard_ptrs),
                int(rows_per_shard), int(first_shard), M, N, K, self._stream())
        fn, check = self._lib.aiehlc_gemm_i8_i32_scatter_dev, _capi.check
        return lambda: check(fn(*args))

    def gemm_i8_i32_scatter(self, A, B, shards, rows_per_shard: int, first_shard: int = 0):
        """Adds A . B^T into the row shards (a list of int32 tensors [rows][N] on this or a peer GPU)."""
        N = shards[0].shape[1]
        for s in shards:
            if s.dtype != __import__("torch").int32 or not s.is_contiguous() or s.shape[1] != N:
                raise ValueError("gemm_i8_i32_scatter: shards must be contiguous int32 [rows][N]")
        self.bound_gemm_i8_i32_scatter(A, B, [s.data_ptr() for s in shards], rows_per_shard, N, first_shard)()
        return shards

    def gemm_i8_srs(self, A, B, shift: int = 0, shift_vec=None, acc_in=None, splitk: int = 1, out=None):
        import torch
        M, K = A.shape
        N, K2 = B.shape
        if K != K2:
            raise ValueError("gemm_i8_srs: A is [M][K], B is [N][K]; K differs")
        if out is None:
            out = torch.empty((M, N), dtype=torch.int8, device=A.device)
        sv = C.c_void_p(None) if shift_vec is None else self._dev(shift_vec, torch.uint8, "shift_vec")
        ai = C.c_void_p(None) if acc_in is None else self._dev(acc_in, torch.int32, "acc_in")
        _capi.check(self._lib.aiehlc_gemm_i8_srs_dev(
            self._h, self._dev(A, torch.int8, "A"), self._dev(B, torch.int8, "B"),
            self._dev(out, torch.int8, "C"), M, N, K, int(shift), sv, ai, int(splitk), self._stream()))
        return out

    def gemm_i8_srs_cascade(self, A, B, stages: int, shift: int = 0, shift_vec=None, out=None):
        """Multi-launch cascade over `stages` equal K slices: stage s adds its partial sums into an
        int32 buffer that stays on the device (the tile -> tile hop of
        example/multi/multi_tile.cpp:125-127), the last stage adds its own slice and flushes
        through srs.  Bit-identical to the single-launch form."""
        import torch
        M, K = A.shape
        N = B.shape[0]
        if stages < 1 or K % stages:
            raise ValueError("cascade: stages must divide K")
        if stages == 1:
            return self.gemm_i8_srs(A, B, shift, shift_vec, out=out)
        ks = K // stages
        partial = torch.empty((M, N), dtype=torch.int32, device=A.device)
        for s in range(stages - 1):
            a_s = A[:, s * ks:(s + 1) * ks].contiguous()
            b_s = B[:, s * ks:(s + 1) * ks].contiguous()
            self.gemm_i8_i32(a_s, b_s, out=partial, accumulate=s > 0)
        s = stages - 1
        return self.gemm_i8_srs(A[:, s * ks:].contiguous(), B[:, s * ks:].contiguous(), shift, shift_vec,
                                acc_in=partial, out=out)

    def srs_i32_i8(self, acc, shift: int = 0, shift_vec=None, out=None):
        import torch
        rows, cols = acc.shape
        if out is None:
            out = torch.empty((rows, cols), dtype=torch.int8, device=acc.device)
        sv = C.c_void_p(None) if shift_vec is None else self._dev(shift_vec, torch.uint8, "shift_vec")
        _capi.check(self._lib.aiehlc_srs_i32_i8_dev(self._h, self._dev(acc, torch.int32, "in"),
                                                    self._dev(out, torch.int8, "out"), rows, cols, int(shift),
                                                    sv, self._stream()))
        return out

    def gemm_bf16(self, A, B, out=None):
        import torch
        M, K = A.shape
        N, K2 = B.shape
        if K != K2:
            raise ValueError("gemm_bf16: A is [M][K], B is [N][K]; K differs")
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
        _capi.check(self._lib.aiehlc_gemm_bf16_dev(
            self._h, self._dev(A, torch.bfloat16, "A"), self._dev(B, torch.bfloat16, "B"),
            self._dev(out, torch.bfloat16, "C"), M, N, K, self._stream()))
        return out

    def conv2d_i8_srs(self, x, w, shift_vec, pad: int = 1, out=None):
        """x NHWC int8, w HWIO int8, shift_vec uint8[cout]; stride 1, same-size output."""
        import torch
        n, h, wd, cin = x.shape
        kh, kw, cin2, cout = w.shape
        if cin != cin2:
            raise ValueError("conv2d: channel mismatch between x (NHWC) and w (HWIO)")
        if out is None:
            out = torch.empty((n, h, wd, cout), dtype=torch.int8, device=x.device)
        _capi.check(self._lib.aiehlc_conv2d_i8_srs_dev(
            self._h, self._dev(x, torch.int8, "x"), self._dev(w, torch.int8, "w"),
            self._dev(out, torch.int8, "y"), n, h, wd, cin, cout, kh, kw, int(pad),
            self._dev(shift_vec, torch.uint8, "shift_vec"), self._stream()))
        return out

    def conv2d_pack_weights(self, w):
        """HWIO int8 weights -> the [tap][cout][cin] copy the packed entry point reads."""
        import torch
        kh, kw, cin, cout = w.shape
        packed = torch.empty((kh * kw, cout, cin), dtype=torch.int8, device=w.device)
        _capi.check(self._lib.aiehlc_conv2d_pack_weights_dev(self._h, self._dev(w, torch.int8, "w"),
                                                             self._dev(packed, torch.int8, "packed"), kh, kw, cin, cout,
                                                             self._stream()))
        return packed

    def conv2d_i8_srs_packed(self, x, packed, kernel_hw, shift_vec, pad: int = 1, out=None):
        import torch
        n, h, wd, cin = x.shape
        kh, kw = kernel_hw
        cout = packed.shape[1]
        if out is None:
            out = torch.empty((n, h, wd, cout), dtype=torch.int8, device=x.device)
        _capi.check(self._lib.aiehlc_conv2d_i8_srs_packed_dev(
            self._h, self._dev(x, torch.int8, "x"), self._dev(packed, torch.int8, "packed"),
            self._dev(out, torch.int8, "y"), n, h, wd, cin, cout, kh, kw, int(pad),
            self._dev(shift_vec, torch.uint8, "shift_vec"), self._stream()))
        return out

    # ------------------------------------------------------------ host arrays
    @staticmethod
    def _host(a, dtype, name):
        a = np.ascontiguousarray(a)
        if a.dtype != dtype:
            raise TypeError(f"{name}: expected dtype {dtype}, got {a.dtype}")
        return a

    def mm_i32_host(self, packed, M: int, N: int, K: int):
        packed = self._host(packed, np.int32, "in")
        if packed.size < (M + N) * K:
            raise ValueError("mm_i32: input window shorter than (M+N)*K words")
        out = np.empty((M, N), dtype=np.int32)
        _capi.check(self._lib.aiehlc_mm_i32_host(self._h, _np_ptr(packed), _np_ptr(out), M, N, K))
        return out

    def gemm_i8_i32_host(self, A, B):
        A = self._host(A, np.int8, "A")
        B = self._host(B, np.int8, "B")
        (M, K), (N, K2) = A.shape, B.shape
        if K != K2:
            raise ValueError("gemm_i8_i32: K differs")
        out = np.empty((M, N), dtype=np.int32)
        _capi.check(self._lib.aiehlc_gemm_i8_i32_host(self._h, _np_ptr(A), _np_ptr(B), _np_ptr(out), M, N, K))
        return out

    def gemm_i8_srs_host(self, A, B, shift: int = 0, shift_vec=None, splitk: int = 1, out=None):
        A = self._host(A, np.int8, "A")
        B = self._host(B, np.int8, "B")
        (M, K), (N, K2) = A.shape, B.shape
        if K != K2:
            raise ValueError("gemm_i8_srs: K differs")
        sv = None if shift_vec is None else self._host(shift_vec, np.uint8, "shift_vec")
        if out is None:
            out = np.empty((M, N), dtype=np.int8)
        _capi.check(self._lib.aiehlc_gemm_i8_srs_host(self._h, _np_ptr(A), _np_ptr(B), _np_ptr(out), M, N, K,
                                                      int(shift), _np_ptr(sv), int(splitk)))
        return out

    def gemm_bf16_host(self, A_bits, B_bits):
        """Operands and result are raw bf16 bit patterns (uint16)."""
        A = self._host(A_bits, np.uint16, "A")
        B = self._host(B_bits, np.uint16, "B")
        (M, K), (N, K2) = A.shape, B.shape
        if K != K2:
            raise ValueError("gemm_bf16: K differs")
        out = np.empty((M, N), dtype=np.uint16)
        _capi.check(self._lib.aiehlc_gemm_bf16_host(self._h, _np_ptr(A), _np_ptr(B), _np_ptr(out), M, N, K))
        return out

    def conv2d_i8_srs_host(self, x, w, shift_vec, pad: int = 1):
        x = self._host(x, np.int8, "x")
        w = self._host(w, np.int8, "w")
        sv = self._host(shift_vec, np.uint8, "shift_vec")
        n, h, wd, cin = x.shape
        kh, kw, cin2, cout = w.shape
        if cin != cin2:
            raise ValueError("conv2d: channel mismatch")
        y = np.empty((n, h, wd, cout), dtype=np.int8)
        _capi.check(self._lib.aiehlc_conv2d_i8_srs_host(self._h, _np_ptr(x), _np_ptr(w), _np_ptr(y), n, h, wd, cin,
                                                        cout, kh, kw, int(pad), _np_ptr(sv)))
        return y
