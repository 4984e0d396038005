"""Builds libaiehlc_b200.so (CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m aiehlc_b200.build            # build if sources are newer than the library
    python -m aiehlc_b200.build --force
    AIEHLC_MEASURE=1 python -m aiehlc_b200.build   # libaiehlc_b200_measure.so: kernels with clock stamps and
                                                   # the debug modes that skip part of a kernel (-DAIEHLC_MEASURE)

nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
MEASURE = os.environ.get("AIEHLC_MEASURE", "0") not in ("", "0")
OBJ_DIR = PKG / ("_obj_measure" if MEASURE else "_obj")
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / ("libaiehlc_b200_measure.so" if MEASURE else "libaiehlc_b200.so")

CUDA_SOURCES = ["capi.cu", "gemm_launch.cu", "simt_kernels.cu", "conv_tcgen05.cu"]
CXX_SOURCES = ["xaie_runtime.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build aiehlc_b200")
    return cand


def _sources() -> list[Path]:
    out = [CSRC / s for s in CUDA_SOURCES + CXX_SOURCES if (CSRC / s).exists()]
    return out


def _newest_input() -> float:
    files = list(CSRC.glob("*")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    return max(f.stat().st_mtime for f in files if f.is_file())


def needs_build() -> bool:
    return (not LIB_PATH.exists()) or LIB_PATH.stat().st_mtime < _newest_input()


def _compile(src: Path, verbose: bool) -> Path:
    obj = OBJ_DIR / (src.name + ".o")
    cmd = [nvcc_path(), *NVCC_FLAGS, *(["-DAIEHLC_MEASURE"] if MEASURE else []),
           "-I", str(INCLUDE), "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB_PATH
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), srcs))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc_path(), "-shared", "-o", str(tmp), *map(str, objs),
           "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-lpthread", "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


EXAMPLES_DIR = PKG.parent / "examples"
EXAMPLES_BIN = EXAMPLES_DIR / "_bin"


def build_examples() -> list[Path]:
    """Compiles examples/*.cc (C++ host programs on the XAie_* surface) against the library."""
    build()
    EXAMPLES_BIN.mkdir(exist_ok=True)
    outs = []
    for src in sorted(EXAMPLES_DIR.glob("*.cc")):
        out = EXAMPLES_BIN / src.stem
        if out.exists() and out.stat().st_mtime > max(src.stat().st_mtime, LIB_PATH.stat().st_mtime):
            outs.append(out)
            continue
        cmd = ["g++", "-std=c++17", "-O2", "-I", str(INCLUDE), "-I", str(INCLUDE / "bsp"), str(src),
               "-L", str(LIB_DIR), "-laiehlc_b200", "-Wl,-rpath,$ORIGIN/../../aiehlc_b200/lib", "-o", str(out)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"example {src.name} failed to build:\n{res.stderr}")
        outs.append(out)
    return outs


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    if "--examples" in sys.argv:
        for e in build_examples():
            print(e)
