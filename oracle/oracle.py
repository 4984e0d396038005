"""numpy/ctypes face of oracle.c (built by oracle/Makefile into oracle/_build/liboracle.so).

TEST INFRASTRUCTURE: the checker for the CUDA path and the timed CPU baseline.  The product
(aiehlc_b200) never imports this module.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_lib = None


def _cpu_tag() -> str:
    """Hash of this CPU's feature flags: the library is compiled with -march=native."""
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                return hashlib.sha1(line.encode()).hexdigest()[:10]
    except OSError:
        pass
    return "generic"


LIB = HERE / "_build" / f"liboracle-{_cpu_tag()}.so"


def build(force: bool = False) -> Path:
    src = HERE / "oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        cmd = ["make", "-C", str(HERE), "-s", f"OUT=_build/{LIB.name}"] + (["-B"] if force else [])
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"oracle build failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB))
        vp, ci, ll = C.c_void_p, C.c_int, C.c_longlong
        L.oracle_max_threads.restype = ci
        L.oracle_set_threads.argtypes = [ci]
        L.oracle_mm_i32.argtypes = [vp, vp, ci, ci, ci]
        L.oracle_gemm_i8_i32.argtypes = [vp, vp, vp, ci, ci, ci]
        L.oracle_srs_i8.argtypes = [C.c_int32, ci]
        L.oracle_srs_i8.restype = C.c_int8
        L.oracle_srs_i32_i8.argtypes = [vp, vp, ll, ll, ci, vp]
        L.oracle_gemm_i8_srs.argtypes = [vp, vp, vp, ci, ci, ci, ci, vp, vp, ci]
        L.oracle_conv2d_i8_srs.argtypes = [vp, vp, vp] + [ci] * 8 + [vp]
        L.oracle_gemm_bf16.argtypes = [vp, vp, vp, vp, ci, ci, ci]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


def _c(a, dt):
    a = np.ascontiguousarray(a)
    assert a.dtype == dt, (a.dtype, dt)
    return a


def max_threads() -> int:
    return lib().oracle_max_threads()


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def mm_i32(packed, M, N, K):
    packed = _c(packed, np.int32)
    assert packed.size >= (M + N) * K
    out = np.empty((M, N), np.int32)
    lib().oracle_mm_i32(_p(packed), _p(out), M, N, K)
    return out


def gemm_i8_i32(A, B):
    A, B = _c(A, np.int8), _c(B, np.int8)
    (M, K), (N, K2) = A.shape, B.shape
    assert K == K2
    out = np.empty((M, N), np.int32)
    lib().oracle_gemm_i8_i32(_p(A), _p(B), _p(out), M, N, K)
    return out


def srs_i8(acc: int, s: int) -> int:
    return int(lib().oracle_srs_i8(int(acc), int(s)))


def srs_i32_i8(acc, shift=0, shift_vec=None):
    acc = _c(acc, np.int32)
    rows, cols = acc.shape
    sv = None if shift_vec is None else _c(shift_vec, np.uint8)
    out = np.empty((rows, cols), np.int8)
    lib().oracle_srs_i32_i8(_p(acc), _p(out), rows, cols, int(shift), _p(sv))
    return out


def gemm_i8_srs(A, B, shift=0, shift_vec=None, acc_in=None, splitk=1):
    A, B = _c(A, np.int8), _c(B, np.int8)
    (M, K), (N, K2) = A.shape, B.shape
    assert K == K2
    sv = None if shift_vec is None else _c(shift_vec, np.uint8)
    ai = None if acc_in is None else _c(acc_in, np.int32)
    out = np.empty((M, N), np.int8)
    lib().oracle_gemm_i8_srs(_p(A), _p(B), _p(out), M, N, K, int(shift), _p(sv), _p(ai), int(splitk))
    return out


def conv2d_i8_srs(x, w, shift_vec, pad=1):
    x, w, sv = _c(x, np.int8), _c(w, np.int8), _c(shift_vec, np.uint8)
    n, h, wd, cin = x.shape
    kh, kw, cin2, cout = w.shape
    assert cin == cin2 and sv.size == cout
    y = np.empty((n, h, wd, cout), np.int8)
    lib().oracle_conv2d_i8_srs(_p(x), _p(w), _p(y), n, h, wd, cin, cout, kh, kw, int(pad), _p(sv))
    return y


def gemm_bf16(A_bits, B_bits, want_bf16=False):
    """bf16 bit patterns in; fp32-accumulated sums out (and their bf16 rounding if asked)."""
    A, B = _c(A_bits, np.uint16), _c(B_bits, np.uint16)
    (M, K), (N, K2) = A.shape, B.shape
    assert K == K2
    c32 = np.empty((M, N), np.float32)
    cb = np.empty((M, N), np.uint16) if want_bf16 else None
    lib().oracle_gemm_bf16(_p(A), _p(B), _p(c32), _p(cb), M, N, K)
    return (c32, cb) if want_bf16 else c32
