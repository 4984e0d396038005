"""The XAie_* run-time surface on the GPU: the reference's own host programs (compiled unmodified
against libaiehlc_b200.so), this repository's C++ examples, and failure paths driven through
ctypes.  No test here faults, traps or hangs the GPU: failures are made on the host."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

from aiehlc_b200 import _capi, build, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "oracle" / "_ref"


# ------------------------------------------------------------------ compiled programs
@pytest.mark.parametrize("name,expect,count", [
    ("aieml_perf_b200", "CPU result matches vmem_out.", 1),
    ("multi_tile_b200", "Sucess: CPU result matches AIE.", 1),
    ("seq_full_col_b200", "Sucess: CPU result matches AIE.", 1),
    ("multi_kernel_b200", "Sucess: CPU result matches AIE.", 2),
    ("tutorial_example_b200", "Sucess: CPU result matches AIE.", 1),
])
def test_unmodified_reference_host_program_on_b200(name, expect, count):
    """aiehlc's example sources, compiled as they are plus a binding file (examples/bindings/), pass
    their own in-file checks when the run-time underneath is this library."""
    exe = REF / name
    if not exe.exists():
        pytest.skip("oracle/_ref was not built (needs the aiehlc source tree at build time)")
    res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert res.stdout.count(expect) == count, res.stdout[-2000:] + res.stderr[-2000:]
    assert "Mismatch" not in res.stdout and "mismatches." not in res.stdout


def test_cpp_examples():
    exes = {p.name: p for p in build.build_examples()}
    c8 = O.mm_i32(np.arange(0, 128, dtype=np.int32), 8, 8, 8)          # aieoob.c:83-86 through the oracle
    res = subprocess.run([str(exes["perf_host"])], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "CPU result matches vmem_out." in res.stdout, res.stdout + res.stderr
    assert "C[0]=36312 C[255]=2006232" in res.stdout
    for argv in ([], ["300", "200", "400", "6"], ["128", "64", "64", "0"]):
        res = subprocess.run([str(exes["cascade_gemm"]), *argv], capture_output=True, text=True, timeout=300)
        assert res.returncode == 0 and "CPU result matches device output." in res.stdout, res.stdout + res.stderr
        assert "kernel launches: 4" in res.stdout
    # the kernel-call form k<Col,Row,colstart,rowstart,M,N,K>(in, out) of aie_nokernelload.cc:130
    res = subprocess.run([str(exes["kernel_call"])], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "CPU result matches device output." in res.stdout, res.stdout + res.stderr
    assert "perf: C[0]=36312 C[255]=2006232, 0 mismatches" in res.stdout
    assert "perf 384x256x512: 0 mismatches" in res.stdout          # the same kernel on the tensor cores
    # the short host API of example/other/aieoob.c:88-95 on its own 8x8 fixture (h_a[i] = i)
    res = subprocess.run([str(exes["oob_host"])], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0 and "CPU result matches vmem_out." in res.stdout, res.stdout + res.stderr
    assert "C[0]=%d C[63]=%d" % (int(c8[0, 0]), int(c8[7, 7])) in res.stdout
    assert "4x4: 0 mismatches" in res.stdout and "errors reported: 1 1 1" in res.stdout


# ------------------------------------------------------------------ the same surface through ctypes
class Loc(C.Structure):
    _fields_ = [("Row", C.c_uint8), ("Col", C.c_uint8)]


class Backend(C.Structure):
    _fields_ = [("Type", C.c_int)]


class Config(C.Structure):
    _fields_ = [("AieGen", C.c_uint8), ("BaseAddr", C.c_uint64), ("ColShift", C.c_uint8), ("RowShift", C.c_uint8),
                ("NumRows", C.c_uint8), ("NumCols", C.c_uint8), ("ShimRowNum", C.c_uint8),
                ("MemTileRowStart", C.c_uint8), ("MemTileNumRows", C.c_uint8), ("AieTileRowStart", C.c_uint8),
                ("AieTileNumRows", C.c_uint8)]


class DevInst(C.Structure):
    _fields_ = [("Cfg", Config), ("IsReady", C.c_uint8), ("StartCol", C.c_uint8), ("PartNumCols", C.c_uint8),
                ("PartBaseAddr", C.c_uint64), ("Backend", C.POINTER(Backend)), ("BackendStorage", Backend),
                ("Priv", C.c_void_p)]


class GemmArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("M", "N", "K", "shift", "has_shift_vec", "splitk", "accumulate", "use_acc")]


class MmArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("M", "N", "K")]


XAIE_OK, XAIE_INVALID_ELF, XAIE_CORE_STATUS_TIMEOUT = 0, 5, 6


@pytest.fixture()
def xaie():
    lib = _capi.load()
    vp, u32, u64 = C.c_void_p, C.c_uint32, C.c_uint64
    sig = {
        "XAie_CfgInitialize": (C.c_int, [C.POINTER(DevInst), C.POINTER(Config)]),
        "XAie_PartitionTeardown": (C.c_int, [C.POINTER(DevInst)]),
        "XAie_LoadElfMem": (C.c_int, [C.POINTER(DevInst), Loc, vp]),
        "XAie_KernelSetArgs": (C.c_int, [C.POINTER(DevInst), Loc, vp, u32]),
        "XAie_MemAllocate": (vp, [C.POINTER(DevInst), u64, C.c_int]),
        "XAie_MemGetVAddr": (vp, [vp]),
        "XAie_MemGetDevAddr": (u64, [vp]),
        "XAie_InitRoutingHandler": (vp, [C.POINTER(DevInst)]),
        "XAie_Route": (C.c_int, [vp, vp, Loc, Loc]),
        "XAie_MoveDataExternal2Aie": (C.c_int, [vp, Loc, vp, u32, u32, Loc]),
        "XAie_MoveDataAie2External": (C.c_int, [vp, Loc, u32, u32, vp, Loc]),
        "XAie_Run": (C.c_int, [vp, u32]),
        "XAie_CoreWaitForDone": (C.c_int, [C.POINTER(DevInst), Loc, u32]),
        "XAie_CoreGetStatus": (C.c_int, [C.POINTER(DevInst), Loc, C.POINTER(u32)]),
        "XAie_DataMemBlockRead": (C.c_int, [C.POINTER(DevInst), Loc, u64, vp, u32]),
        "XAie_DataMemBlockWrite": (C.c_int, [C.POINTER(DevInst), Loc, u64, vp, u32]),
        "XAie_DebugInjectStatus": (C.c_int, [C.POINTER(DevInst), u32, u32]),
        "XAie_LastError": (C.c_char_p, []),
        "XAie_LaunchCount": (u64, [C.POINTER(DevInst)]),
        "aiehlc_window_offset_b": (u64, [vp, u32]),
        "XAie_MoveData": (C.c_int, [vp, Loc, vp, u32, vp, Loc]),
        "XAie_GraphBeginCapture": (C.c_int, [C.POINTER(DevInst)]),
        "XAie_GraphEndCapture": (C.c_int, [C.POINTER(DevInst), C.POINTER(vp)]),
        "XAie_GraphLaunch": (C.c_int, [vp]),
        "XAie_GraphWait": (C.c_int, [vp, u32]),
        "XAie_GraphDestroy": (C.c_int, [vp]),
    }
    for n, (r, a) in sig.items():
        getattr(lib, n).restype = r
        getattr(lib, n).argtypes = a
    dev = DevInst()
    cfg = Config(2, 0x20000000000, 25, 20, 11, 38, 0, 1, 2, 3, 8)
    assert lib.XAie_CfgInitialize(C.byref(dev), C.byref(cfg)) == XAIE_OK, lib.XAie_LastError()
    yield lib, dev
    assert lib.XAie_PartitionTeardown(C.byref(dev)) == XAIE_OK


def _kernel(lib, name):
    return C.cast(getattr(lib, name), C.c_void_p)


def _host_array(lib, mem, nbytes, dtype):
    addr = lib.XAie_MemGetVAddr(mem)
    return np.ctypeslib.as_array((C.c_uint8 * nbytes).from_address(addr)).view(dtype)


def test_gmio_buffers_sit_below_4gib(xaie):
    lib, dev = xaie
    mem = lib.XAie_MemAllocate(C.byref(dev), 4096, 0)
    assert mem and lib.XAie_MemGetDevAddr(mem) == lib.XAie_MemGetVAddr(mem) < 2**32
    assert lib.XAie_MemAllocate(C.byref(dev), 0, 0) is None


def test_int8_gemm_srs_through_the_runtime_matches_oracle(xaie):
    lib, dev = xaie
    M, N, K = 200, 136, 320
    A = synth.int8_uniform(2, (M, K))
    B = synth.int8_uniform(1002, (N, K))
    tile, shim = Loc(4, 4), Loc(0, 2)
    assert lib.XAie_LoadElfMem(C.byref(dev), tile, _kernel(lib, "aiehlc_k_gemm_i8_srs")) == XAIE_OK
    args = GemmArgs(M, N, K, 7, 0, 4, 0, 0)
    assert lib.XAie_KernelSetArgs(C.byref(dev), tile, C.byref(args), C.sizeof(args)) == XAIE_OK
    ri = lib.XAie_InitRoutingHandler(C.byref(dev))
    assert lib.XAie_Route(ri, None, shim, tile) == XAIE_OK and lib.XAie_Route(ri, None, tile, shim) == XAIE_OK
    off_b = lib.aiehlc_window_offset_b(C.byref(args), 1)
    win = off_b + N * K
    mem_in = lib.XAie_MemAllocate(C.byref(dev), win, 0)
    mem_out = lib.XAie_MemAllocate(C.byref(dev), M * N, 0)
    buf = _host_array(lib, mem_in, win, np.int8)
    buf[:M * K] = A.ravel()
    buf[off_b:off_b + N * K] = B.ravel()
    assert lib.XAie_CoreWaitForDone(C.byref(dev), tile, 0) == XAIE_CORE_STATUS_TIMEOUT      # wait before run
    assert lib.XAie_MoveDataExternal2Aie(ri, shim, mem_in, win, 0x1000, tile) == XAIE_OK
    assert lib.XAie_Run(ri, 1) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_CoreWaitForDone(C.byref(dev), tile, 5_000_000) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_MoveDataAie2External(ri, tile, 0x6000, M * N, mem_out, shim) == XAIE_OK
    got = _host_array(lib, mem_out, M * N, np.int8).reshape(M, N)
    assert np.array_equal(got, O.gemm_i8_srs(A, B, shift=7, splitk=4))
    assert lib.XAie_LaunchCount(C.byref(dev)) == 1
    # debug peek of the result window agrees with the DMA path
    peek = np.empty(64, np.int8)
    assert lib.XAie_DataMemBlockRead(C.byref(dev), tile, 0x6000, peek.ctypes.data, 64) == XAIE_OK
    assert np.array_equal(peek, got.ravel()[:64])


class ConvArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n", "h", "w", "cin", "cout", "kh", "kw", "pad")]


class SrsArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("rows", "cols", "shift", "has_shift_vec")]


def _run_tile(lib, dev, ri, tile, shim, mem_in, in_bytes, out_bytes):
    assert lib.XAie_MoveDataExternal2Aie(ri, shim, mem_in, in_bytes, 0x1000, tile) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_Run(ri, 1) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_CoreWaitForDone(C.byref(dev), tile, 5_000_000) == XAIE_OK, lib.XAie_LastError()
    mem_out = lib.XAie_MemAllocate(C.byref(dev), out_bytes, 0)
    assert lib.XAie_MoveDataAie2External(ri, tile, 0x6000, out_bytes, mem_out, shim) == XAIE_OK, lib.XAie_LastError()
    return mem_out


def test_conv_bf16_and_gemm_to_srs_chain_through_the_runtime(xaie):
    """The other library kernels behind XAie_LoadElfMem: the convolution (input window = x | w | shift bytes),
    the bf16 GEMM, and an int8 GEMM whose int32 result moves tile to tile into the srs kernel (the two-stage
    chain of example/multi/multi_tile.cpp:105-145 with real kernels)."""
    lib, dev = xaie
    lib.aiehlc_conv_offset_w.restype = C.c_uint64
    lib.aiehlc_conv_offset_w.argtypes = [C.c_void_p]
    lib.aiehlc_conv_offset_shift.restype = C.c_uint64
    lib.aiehlc_conv_offset_shift.argtypes = [C.c_void_p]
    ri = lib.XAie_InitRoutingHandler(C.byref(dev))
    shim = Loc(0, 2)
    # ---- convolution 1 x 14 x 14 x 64 -> 64, 3 x 3, per-channel shifts
    t_conv = Loc(3, 5)
    x = synth.int8_uniform(4, (1, 14, 14, 64))
    w = synth.int8_uniform(1004, (3, 3, 64, 64))
    sv = (np.arange(64) % 9).astype(np.uint8)
    ca = ConvArgs(1, 14, 14, 64, 64, 3, 3, 1)
    assert lib.XAie_LoadElfMem(C.byref(dev), t_conv, _kernel(lib, "aiehlc_k_conv2d_i8_srs")) == XAIE_OK
    assert lib.XAie_KernelSetArgs(C.byref(dev), t_conv, C.byref(ca), C.sizeof(ca)) == XAIE_OK
    assert lib.XAie_Route(ri, None, shim, t_conv) == XAIE_OK and lib.XAie_Route(ri, None, t_conv, shim) == XAIE_OK
    ow, osv = lib.aiehlc_conv_offset_w(C.byref(ca)), lib.aiehlc_conv_offset_shift(C.byref(ca))
    win = osv + 64
    mem = lib.XAie_MemAllocate(C.byref(dev), win, 0)
    buf = _host_array(lib, mem, win, np.uint8)
    buf[:x.size] = x.view(np.uint8).ravel()
    buf[ow:ow + w.size] = w.view(np.uint8).ravel()
    buf[osv:osv + 64] = sv
    out = _run_tile(lib, dev, ri, t_conv, shim, mem, win, x.size)
    got = _host_array(lib, out, x.size, np.int8).reshape(1, 14, 14, 64)
    assert np.array_equal(got, O.conv2d_i8_srs(x, w, sv, pad=1))
    # ---- bf16 GEMM 96 x 80 x 64
    t_bf = Loc(3, 6)
    M, N, K = 96, 80, 64
    Ab, Bb = synth.normal_bf16_bits(3, (M, K)), synth.normal_bf16_bits(1003, (N, K))
    ga = GemmArgs(M, N, K, 0, 0, 1, 0, 0)
    assert lib.XAie_LoadElfMem(C.byref(dev), t_bf, _kernel(lib, "aiehlc_k_gemm_bf16")) == XAIE_OK
    assert lib.XAie_KernelSetArgs(C.byref(dev), t_bf, C.byref(ga), C.sizeof(ga)) == XAIE_OK
    assert lib.XAie_Route(ri, None, shim, t_bf) == XAIE_OK and lib.XAie_Route(ri, None, t_bf, shim) == XAIE_OK
    off_b = lib.aiehlc_window_offset_b(C.byref(ga), 2)
    win = off_b + N * K * 2
    mem = lib.XAie_MemAllocate(C.byref(dev), win, 0)
    buf = _host_array(lib, mem, win, np.uint8)
    buf[:M * K * 2] = Ab.view(np.uint8).ravel()
    buf[off_b:off_b + N * K * 2] = Bb.view(np.uint8).ravel()
    out = _run_tile(lib, dev, ri, t_bf, shim, mem, win, M * N * 2)
    got = synth.bf16_bits_to_f32(_host_array(lib, out, M * N * 2, np.uint16).reshape(M, N)).astype(np.float64)
    ref = O.gemm_bf16(Ab, Bb).astype(np.float64)
    assert float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0))) <= 1e-2          # the bf16 tolerance
    # ---- int8 GEMM -> int32 on one tile, result moved tile to tile into the srs kernel on the next
    t_mm, t_srs = Loc(4, 5), Loc(5, 5)
    M, N, K = 130, 72, 256
    A, B = synth.int8_uniform(7, (M, K)), synth.int8_uniform(1007, (N, K))
    g2 = GemmArgs(M, N, K, 0, 0, 1, 0, 0)
    sa = SrsArgs(M, N, 9, 0)
    assert lib.XAie_LoadElfMem(C.byref(dev), t_mm, _kernel(lib, "aiehlc_k_gemm_i8_i32")) == XAIE_OK
    assert lib.XAie_KernelSetArgs(C.byref(dev), t_mm, C.byref(g2), C.sizeof(g2)) == XAIE_OK
    assert lib.XAie_LoadElfMem(C.byref(dev), t_srs, _kernel(lib, "aiehlc_k_srs_i32_i8")) == XAIE_OK
    assert lib.XAie_KernelSetArgs(C.byref(dev), t_srs, C.byref(sa), C.sizeof(sa)) == XAIE_OK
    for a, b in ((shim, t_mm), (t_mm, t_srs), (t_srs, shim)):
        assert lib.XAie_Route(ri, None, a, b) == XAIE_OK
    off_b = lib.aiehlc_window_offset_b(C.byref(g2), 1)
    win = off_b + N * K
    mem = lib.XAie_MemAllocate(C.byref(dev), win, 0)
    buf = _host_array(lib, mem, win, np.int8)
    buf[:M * K] = A.ravel()
    buf[off_b:off_b + N * K] = B.ravel()
    assert lib.XAie_MoveDataExternal2Aie(ri, shim, mem, win, 0x1000, t_mm) == XAIE_OK
    assert lib.XAie_Run(ri, 1) == XAIE_OK, lib.XAie_LastError()                 # only the tile that received data runs
    assert lib.XAie_CoreWaitForDone(C.byref(dev), t_mm, 5_000_000) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_MoveData(ri, t_mm, C.c_void_p(0x6000), M * N * 4, C.c_void_p(0x1000), t_srs) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_Run(ri, 1) == XAIE_OK, lib.XAie_LastError()
    assert lib.XAie_CoreWaitForDone(C.byref(dev), t_srs, 5_000_000) == XAIE_OK, lib.XAie_LastError()
    out = lib.XAie_MemAllocate(C.byref(dev), M * N, 0)
    assert lib.XAie_MoveDataAie2External(ri, t_srs, 0x6000, M * N, out, shim) == XAIE_OK
    got = _host_array(lib, out, M * N, np.int8).reshape(M, N)
    assert np.array_equal(got, O.gemm_i8_srs(A, B, shift=9))


def test_failure_paths_return_codes(xaie):
    lib, dev = xaie
    tile, shim, other = Loc(4, 4), Loc(0, 2), Loc(5, 5)
    # unknown kernel symbol
    bogus = C.c_int(0)
    assert lib.XAie_LoadElfMem(C.byref(dev), tile, C.cast(C.byref(bogus), C.c_void_p)) == XAIE_INVALID_ELF
    assert b"not a registered kernel" in lib.XAie_LastError()
    assert lib.XAie_LoadElfMem(C.byref(dev), shim, _kernel(lib, "aiehlc_k_mm_i32")) != XAIE_OK   # shim row
    assert lib.XAie_LoadElfMem(C.byref(dev), Loc(200, 4), _kernel(lib, "aiehlc_k_mm_i32")) != XAIE_OK
    ri = lib.XAie_InitRoutingHandler(C.byref(dev))
    assert lib.XAie_Run(ri, 1) != XAIE_OK                                     # nothing loaded
    assert lib.XAie_LoadElfMem(C.byref(dev), tile, _kernel(lib, "aiehlc_k_mm_i32")) == XAIE_OK
    lib.XAie_Route(ri, None, shim, tile)
    mem = lib.XAie_MemAllocate(C.byref(dev), 2048, 0)
    assert lib.XAie_MoveDataExternal2Aie(ri, shim, mem, 4096, 0x1000, tile) != XAIE_OK     # larger than the buffer
    assert lib.XAie_MoveDataExternal2Aie(ri, shim, mem, 2048, 0x1000, other) != XAIE_OK    # no such route
    assert lib.XAie_MoveDataAie2External(ri, tile, 0x6000, 1024, mem, shim) != XAIE_OK     # no route back
    # input window too short for the kernel's arguments: the launch is refused on the host
    args = MmArgs(64, 64, 64)
    lib.XAie_KernelSetArgs(C.byref(dev), tile, C.byref(args), C.sizeof(args))
    assert lib.XAie_MoveDataExternal2Aie(ri, shim, mem, 2048, 0x1000, tile) == XAIE_OK
    assert lib.XAie_Run(ri, 1) != XAIE_OK and b"input window" in lib.XAie_LastError()
    # an injected device status surfaces once at the completion poll, then the poll reports done
    args = MmArgs(16, 16, 16)
    lib.XAie_KernelSetArgs(C.byref(dev), tile, C.byref(args), C.sizeof(args))
    assert lib.XAie_Run(ri, 1) == XAIE_OK
    lib.XAie_DebugInjectStatus(C.byref(dev), 104, 1)
    assert lib.XAie_CoreWaitForDone(C.byref(dev), tile, 0) not in (XAIE_OK, XAIE_CORE_STATUS_TIMEOUT)
    assert lib.XAie_CoreWaitForDone(C.byref(dev), tile, 5_000_000) == XAIE_OK
    st = C.c_uint32(9)
    assert lib.XAie_CoreGetStatus(C.byref(dev), Loc(4, 4), C.byref(st)) == XAIE_OK and st.value == 1
    assert lib.XAie_CoreGetStatus(C.byref(dev), Loc(1, 4), C.byref(st)) == XAIE_OK and st.value == 0


def test_recorded_chain_replays_with_new_inputs(xaie):
    """A two-stage cascade (K slice 0 -> int32 partials -> tile-to-tile move -> K slice 1 + srs) recorded
    once as a graph and replayed: every replay reads the GMIO buffers afresh and matches the oracle."""
    lib, dev = xaie
    M, N, K = 192, 160, 512
    ks = K // 2
    t0, t1, shim = Loc(3, 4), Loc(4, 4), Loc(0, 2)
    assert lib.XAie_LoadElfMem(C.byref(dev), t0, _kernel(lib, "aiehlc_k_gemm_i8_i32")) == XAIE_OK
    assert lib.XAie_LoadElfMem(C.byref(dev), t1, _kernel(lib, "aiehlc_k_gemm_i8_srs")) == XAIE_OK
    a0 = GemmArgs(M, N, ks, 0, 0, 1, 0, 0)
    a1 = GemmArgs(M, N, ks, 8, 0, 1, 0, 1)            # use_acc: add the partials handed down by stage 0
    lib.XAie_KernelSetArgs(C.byref(dev), t0, C.byref(a0), C.sizeof(a0))
    lib.XAie_KernelSetArgs(C.byref(dev), t1, C.byref(a1), C.sizeof(a1))
    ri = lib.XAie_InitRoutingHandler(C.byref(dev))
    for s_, d_ in ((shim, t0), (shim, t1), (t0, t1), (t1, shim)):
        assert lib.XAie_Route(ri, None, s_, d_) == XAIE_OK
    off_b = lib.aiehlc_window_offset_b(C.byref(a0), 1)
    win = off_b + N * ks
    mems = [lib.XAie_MemAllocate(C.byref(dev), win, 0) for _ in range(2)]
    mem_out = lib.XAie_MemAllocate(C.byref(dev), M * N, 0)
    bufs = [_host_array(lib, m, win, np.int8) for m in mems]
    out = _host_array(lib, mem_out, M * N, np.int8)

    def fill(seed):
        A = synth.int8_uniform(seed, (M, K))
        B = synth.int8_uniform(seed + 1000, (N, K))
        for s_ in range(2):
            bufs[s_][:M * ks] = A[:, s_ * ks:(s_ + 1) * ks].ravel()
            bufs[s_][off_b:off_b + N * ks] = B[:, s_ * ks:(s_ + 1) * ks].ravel()
        return O.gemm_i8_srs(A, B, shift=8, splitk=2)

    def chain():
        assert lib.XAie_MoveDataExternal2Aie(ri, shim, mems[0], win, 0x1000, t0) == XAIE_OK
        assert lib.XAie_Run(ri, 1) == XAIE_OK, lib.XAie_LastError()
        assert lib.XAie_MoveData(ri, t0, C.c_void_p(0x6000), M * N * 4, C.c_void_p(0x3000), t1) == XAIE_OK
        assert lib.XAie_MoveDataExternal2Aie(ri, shim, mems[1], win, 0x1000, t1) == XAIE_OK
        assert lib.XAie_Run(ri, 1) == XAIE_OK, lib.XAie_LastError()
        assert lib.XAie_MoveDataAie2External(ri, t1, 0x6000, M * N, mem_out, shim) == XAIE_OK

    exp = fill(11)
    chain()                                               # plain run: sizes every tile window
    assert lib.XAie_CoreWaitForDone(C.byref(dev), t1, 5_000_000) == XAIE_OK
    assert np.array_equal(out.reshape(M, N), exp)
    launches_before = lib.XAie_LaunchCount(C.byref(dev))

    assert lib.XAie_GraphBeginCapture(C.byref(dev)) == XAIE_OK, lib.XAie_LastError()
    chain()                                               # recorded, not executed
    graph = C.c_void_p()
    assert lib.XAie_GraphEndCapture(C.byref(dev), C.byref(graph)) == XAIE_OK, lib.XAie_LastError()
    for seed in (21, 22, 23):
        exp = fill(seed)
        out[:] = 0x55
        assert lib.XAie_GraphLaunch(graph) == XAIE_OK, lib.XAie_LastError()
        assert lib.XAie_GraphWait(graph, 5_000_000) == XAIE_OK, lib.XAie_LastError()
        assert np.array_equal(out.reshape(M, N), exp)
    assert lib.XAie_LaunchCount(C.byref(dev)) == launches_before + 2     # recording issued the two launches once
    assert lib.XAie_GraphDestroy(graph) == XAIE_OK
