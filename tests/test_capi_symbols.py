"""The C-ABI library builds, loads and exports every symbol its headers declare (no GPU, no compute)."""
import ctypes as C
import re
from pathlib import Path

import pytest

from aiehlc_b200 import _capi

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions(header: Path, prefix: str):
    text = header.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)         # drop comments
    text = re.sub(r"^\s*#.*?(?<!\\)$", "", text, flags=re.M)  # drop preprocessor lines
    names = set(re.findall(r"\b(%s\w+)\s*\(" % prefix, text))
    return sorted(names)


def test_library_loads():
    lib = _capi.load()
    assert _capi.library_path().exists()
    assert lib.aiehlc_last_error() is not None


def test_every_declared_aiehlc_symbol_is_exported():
    """Two symbol sets: the drop-in boundary (entry points, planners, counters) and, apart from it, the
    tuning knobs and measurement aids."""
    lib = _capi.load()
    boundary = _declared_functions(ROOT / "include" / "aiehlc_b200.h", "aiehlc_")
    tuning = _declared_functions(ROOT / "include" / "aiehlc_b200_tuning.h", "aiehlc_")
    assert len(boundary) >= 24 and len(tuning) >= 17
    assert not [n for n in boundary if n.startswith("aiehlc_set_")], "knobs belong in aiehlc_b200_tuning.h"
    assert all(n.startswith("aiehlc_set_") for n in tuning)
    assert not set(boundary) & set(tuning)
    for n in boundary + tuning:
        assert hasattr(lib, n), f"{n} declared in a header but not exported"
    assert set(_capi.SIGNATURES) <= set(boundary) | set(tuning)
    assert set(boundary) <= set(_capi.SIGNATURES), "every boundary entry point has a ctypes signature"


def test_measurement_aids_are_compiled_out_of_the_regular_build():
    """Clock stamps and the kernel-skipping debug modes exist only in AIEHLC_MEASURE builds; the
    bounded-wait test aid (mode 3) is in every build."""
    import os
    if os.environ.get("AIEHLC_MEASURE", "0") not in ("", "0"):
        pytest.skip("this is a measurement build")
    lib = _capi.load()
    assert lib.aiehlc_set_debug(None, 1) == _capi.ERR_INVALID          # null context comes first
    fake = C.c_void_p(0)
    assert lib.aiehlc_set_trace(fake, None) == _capi.ERR_INVALID


def test_every_declared_xaie_symbol_is_exported():
    lib = _capi.load()
    names = _declared_functions(ROOT / "include" / "xaiengine.h", "XAie_")
    macros_and_inlines = {"XAie_SetupConfig", "XAie_InstDeclare", "XAie_TileLoc"}
    names = [n for n in names if n not in macros_and_inlines]
    assert len(names) >= 35
    for n in names:
        assert hasattr(lib, n), f"{n} declared in xaiengine.h but not exported"
    for n in _declared_functions(ROOT / "include" / "aiehlc_kernels.h", "aiehlc_"):
        assert hasattr(lib, n), f"{n} declared in aiehlc_kernels.h but not exported"
    for n in ("XAie_KernelRegister", "XAie_KernelBind", "XAie_KernelCall"):
        assert hasattr(lib, n)
    short_api = _declared_functions(ROOT / "include" / "xaie_placeholder.h", "XAie_")
    assert len(short_api) >= 9
    for n in short_api:
        assert hasattr(lib, n), f"{n} declared in xaie_placeholder.h but not exported"


def test_create_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _capi.load()
    h = C.c_void_p()
    rc = lib.aiehlc_create(0, C.byref(h))
    assert rc == _capi.ERR_CUDA and not h.value
    assert b"no CPU path" in lib.aiehlc_last_error()
    from aiehlc_b200.ops import Context
    with pytest.raises(_capi.AiehlcError):
        Context(0)


def test_null_and_bad_arguments_are_rejected_before_any_cuda_call():
    lib = _capi.load()
    assert lib.aiehlc_create(0, None) == _capi.ERR_INVALID
    assert lib.aiehlc_set_tile_n(None, 64) == _capi.ERR_INVALID
    assert lib.aiehlc_sm_count(None) == 0
    assert lib.aiehlc_destroy(None) == _capi.OK
    # XAie surface: null handles give error codes, not crashes
    lib.XAie_CfgInitialize.restype = C.c_int
    lib.XAie_CfgInitialize.argtypes = [C.c_void_p, C.c_void_p]
    assert lib.XAie_CfgInitialize(None, None) != 0
    lib.XAie_Run.restype = C.c_int
    lib.XAie_Run.argtypes = [C.c_void_p, C.c_uint32]
    assert lib.XAie_Run(None, 1) != 0
    lib.XAie_MemGetVAddr.restype = C.c_void_p
    lib.XAie_MemGetVAddr.argtypes = [C.c_void_p]
    assert lib.XAie_MemGetVAddr(None) is None
    lib.XAie_KernelRegister.restype = C.c_int
    lib.XAie_KernelRegister.argtypes = [C.c_void_p, C.c_void_p]
    assert lib.XAie_KernelRegister(None, None) != 0
