"""ctypes binding of libaiehlc_b200.so -- the C ABI declared in include/aiehlc_b200.h.

Loading fails loudly: if the shared library is missing it is built with nvcc, and if that is
impossible an ImportError is raised.  There is no Python or CPU implementation behind these
calls.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

from . import build as _build

OK = 0
ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE, ERR_NOMEM = -1, -2, -3, -4, -5

_i32p = C.POINTER(C.c_int32)
_vp = C.c_void_p

# name -> (restype, argtypes); every symbol include/aiehlc_b200.h and include/aiehlc_b200_tuning.h declare
SIGNATURES = {
    "aiehlc_create": (C.c_int, [C.c_int, C.POINTER(_vp)]),
    "aiehlc_destroy": (C.c_int, [_vp]),
    "aiehlc_last_error": (C.c_char_p, []),
    "aiehlc_sm_count": (C.c_int, [_vp]),
    "aiehlc_sync": (C.c_int, [_vp, _vp, _i32p]),
    "aiehlc_mm_i32_dev": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "aiehlc_mm_i32_host": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    "aiehlc_gemm_i8_i32_dev": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "aiehlc_gemm_i8_i32_scatter_dev": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                 C.c_int, _vp]),
    "aiehlc_gemm_i8_i32_host": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    "aiehlc_gemm_i8_srs_dev": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp,
                                         C.c_int, _vp]),
    "aiehlc_gemm_i8_srs_host": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp, C.c_int]),
    "aiehlc_srs_i32_i8_dev": (C.c_int, [_vp, _vp, _vp, C.c_longlong, C.c_longlong, C.c_int, _vp, _vp]),
    "aiehlc_gemm_bf16_dev": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp]),
    "aiehlc_gemm_bf16_host": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int]),
    "aiehlc_conv2d_i8_srs_dev": (C.c_int, [_vp, _vp, _vp, _vp] + [C.c_int] * 8 + [_vp, _vp]),
    "aiehlc_conv2d_i8_srs_host": (C.c_int, [_vp, _vp, _vp, _vp] + [C.c_int] * 8 + [_vp]),
    "aiehlc_conv2d_pack_weights_dev": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "aiehlc_conv2d_i8_srs_packed_dev": (C.c_int, [_vp, _vp, _vp, _vp] + [C.c_int] * 8 + [_vp, _vp]),
    "aiehlc_conv2d_i8_srs_static_dev": (C.c_int, [_vp, _vp, _vp, _vp] + [C.c_int] * 8 + [_vp, _vp]),
    "aiehlc_set_tile_n": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_cta_pair": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_debug": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_pdl": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_cta_limit": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_operands_ready": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_group_m": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_split_tail": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_tma_store": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_epilogue_groups": (C.c_int, [_vp, C.c_int]),
    "aiehlc_plan_conv2d": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "aiehlc_plan_tile_order": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp,
                                         C.c_int, _vp]),
    "aiehlc_set_k_per_load": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_shard_tile_stores": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_conv_halo": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_conv_persistent": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_conv_wide_n": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_mm_i32_tensor": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_conv_hwio_direct": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_host_blocks": (C.c_int, [_vp, C.c_int]),
    "aiehlc_set_trace": (C.c_int, [_vp, _vp]),
    "aiehlc_set_cta_times": (C.c_int, [_vp, _vp]),
    "aiehlc_launch_count": (C.c_longlong, [_vp]),
    "aiehlc_workspace_generation": (C.c_longlong, [_vp]),
}



class GemmPlan(C.Structure):
    """aiehlc_gemm_plan of include/aiehlc_b200.h."""
    _fields_ = [("tile_m", C.c_int), ("tile_n", C.c_int), ("tile_k_bytes", C.c_int), ("cta_pair", C.c_int),
                ("grid_m", C.c_int), ("grid_n", C.c_int), ("tiles", C.c_longlong), ("slots", C.c_int),
                ("waves", C.c_int), ("wave_efficiency", C.c_double), ("group_m", C.c_int), ("stages", C.c_int),
                ("smem_bytes", C.c_int), ("tmem_columns", C.c_int), ("k_blocks", C.c_int), ("a_shared_by", C.c_int),
                ("b_shared_by", C.c_int), ("wave_footprint_bytes", C.c_longlong), ("cost_units", C.c_double),
                ("split_k_tiles", C.c_int), ("split_k_at", C.c_int),
                ("narrow_tail_tiles", C.c_int)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


SIGNATURES["aiehlc_plan_gemm"] = (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(GemmPlan)])


class ConvPlan(C.Structure):
    """aiehlc_conv_plan of include/aiehlc_b200.h."""
    _fields_ = [(n, C.c_int) for n in ("form", "tile_rows", "tile_width", "patch_rows", "patch_width", "m_rows_used",
                                       "cout_tile", "cin_chunk", "ctas", "tma_boxes_per_cta", "mmas_per_cta", "stages",
                                       "smem_bytes", "launches", "persistent")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}

_lib = None


def library_path() -> Path:
    return _build.LIB_PATH


def load() -> C.CDLL:
    """Returns the loaded library, building it first if needed."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if not path.exists():
        try:
            _build.build()
        except Exception as exc:  # noqa: BLE001
            raise ImportError(
                f"aiehlc_b200: {path} is missing and could not be built ({exc}); "
                "the CUDA extension is required, there is no fallback") from exc
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class AiehlcError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"aiehlc error {code}: {message}")
        self.code = code


def check(rc: int) -> None:
    if rc != OK:
        msg = load().aiehlc_last_error()
        raise AiehlcError(rc, msg.decode() if msg else "")
