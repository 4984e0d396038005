#!/bin/bash
# Compiles the aiehlc reference's own example programs, from their sources where they lie in the
# reference tree, against the CPU tile emulator in ref_shim/.  Outputs go to oracle/_ref/ only.
#   usage: ref_build.sh /path/to/aiehlc
# Each program runs the reference's kernel AND its in-file golden check on the host CPU; the
# oracle is pinned against what they compute (tests/golden/make_golden.py).
# Not built for the CPU emulator: example/matrixmultiply/aieml_mm.cc (its kernel needs the Vitis AIE vector
# API and accumulates into an uninitialised array, aieml_mm.cc:51,73; its host part is built for the GPU
# below with the kernel cut out) and
# example/multi/vek385_verification.cpp (its kernel never terminates).
set -u
REF="${1:-${AIEHLC_REFERENCE:-}}"
if [ -z "$REF" ]; then echo "usage: ref_build.sh /path/to/aiehlc   (or set AIEHLC_REFERENCE)"; exit 2; fi
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/_ref"
INC="$HERE/../include"
mkdir -p "$OUT"
CXX="${CXX:-g++}"
FLAGS="-std=c++17 -O1 -w -fpermissive -no-pie -DAIE_GEN=2 -D__global__= -I$INC -I$INC/bsp -include $INC/aiehlc_kernels.h"
ok=0; bad=0
build() {  # build <source relative to the tree> <output name>
  if [ ! -f "$REF/$1" ]; then echo "ref_build: $1 not found under $REF"; bad=$((bad+1)); return; fi
  if $CXX $FLAGS "$REF/$1" "$HERE/ref_shim/xaie_cpu_emul.cc" -o "$OUT/$2" 2> "$OUT/$2.log"; then
    ok=$((ok+1)); rm -f "$OUT/$2.log"
  else
    echo "ref_build: $1 failed to compile (see $OUT/$2.log)"; bad=$((bad+1))
  fi
}
build example/perf/aieml_perf.cc aieml_perf
build example/multi/multi_tile.cpp multi_tile
build example/multi/seq_full_col.cpp seq_full_col
build example/multi/multi_kernel.cc multi_kernel
build tutorial/example.cpp tutorial_example

# The same unmodified sources once more, this time linked against the B200 run-time
# (libaiehlc_b200.so) plus a small binding file that maps the example's kernel symbol to a CUDA
# kernel (examples/bindings/).  These programs need a GPU to run; tests/ runs them on the GPU box.
LIBDIR="$HERE/../aiehlc_b200/lib"
BIND="$HERE/../examples/bindings"
NVCC="${NVCC:-nvcc}"
NVFLAGS="-std=c++17 -O1 -w -gencode arch=compute_100a,code=sm_100a -I$INC -I$INC/bsp -I$BIND"
build_gpu() {  # build_gpu <source in the tree> <binding file> <output name>
  if [ ! -f "$LIBDIR/libaiehlc_b200.so" ]; then echo "ref_build: libaiehlc_b200.so not built, skipping $3"; return; fi
  # the example itself is host code: the same g++ command line as above, object file only
  if $CXX $FLAGS -c "$REF/$1" -o "$OUT/$3.host.o" 2> "$OUT/$3.log" &&
     $NVCC $NVFLAGS -x cu -c "$BIND/$2" -o "$OUT/$3.bind.o" 2>> "$OUT/$3.log" &&
     $NVCC -Xcompiler -no-pie "$OUT/$3.host.o" "$OUT/$3.bind.o" -L"$LIBDIR" -laiehlc_b200 \
           -Xlinker -rpath -Xlinker '$ORIGIN/../../aiehlc_b200/lib' -o "$OUT/$3" 2>> "$OUT/$3.log"; then
    ok=$((ok+1)); rm -f "$OUT/$3.log" "$OUT/$3.host.o" "$OUT/$3.bind.o"
  else
    echo "ref_build: $1 (B200 link) failed to compile (see $OUT/$3.log)"; bad=$((bad+1))
  fi
}
build_gpu example/perf/aieml_perf.cc aieml_perf_bind.cc aieml_perf_b200
build_gpu example/multi/multi_tile.cpp multi_tile_bind.cu multi_tile_b200
build_gpu example/multi/seq_full_col.cpp multi_tile_bind.cu seq_full_col_b200
build_gpu example/multi/multi_kernel.cc multi_kernel_bind.cu multi_kernel_b200
build_gpu tutorial/example.cpp tutorial_example_bind.cu tutorial_example_b200

# And once more with NOTHING written by hand: aiehlc_b200.bindgen cuts the kernels out of the example
# (the host part is then plain C++ whatever the kernel was written in) and writes the binding file from
# the kernel's text.  This also builds example/matrixmultiply/aieml_mm.cc, whose kernel uses the AIE
# vector API: it is recognised as the int32 matmul loop nest and bound to the library kernel.
PY="${PYTHON:-python}"
GEN="$OUT/gen"
mkdir -p "$GEN"
build_gen() {  # build_gen <source in the tree> <output name>
  if [ ! -f "$LIBDIR/libaiehlc_b200.so" ]; then echo "ref_build: libaiehlc_b200.so not built, skipping $2"; return; fi
  if PYTHONPATH="$HERE/.." $PY -m aiehlc_b200.bindgen "$REF/$1" -o "$GEN/$2_bind.cu" --host-out "$GEN/$2_host.cc" 2> "$OUT/$2.log" &&
     $CXX $FLAGS -c "$GEN/$2_host.cc" -o "$OUT/$2.host.o" 2>> "$OUT/$2.log" &&
     $NVCC $NVFLAGS -x cu -c "$GEN/$2_bind.cu" -o "$OUT/$2.bind.o" 2>> "$OUT/$2.log" &&
     $NVCC -Xcompiler -no-pie "$OUT/$2.host.o" "$OUT/$2.bind.o" -L"$LIBDIR" -laiehlc_b200 \
           -Xlinker -rpath -Xlinker '$ORIGIN/../../aiehlc_b200/lib' -o "$OUT/$2" 2>> "$OUT/$2.log"; then
    ok=$((ok+1)); rm -f "$OUT/$2.log" "$OUT/$2.host.o" "$OUT/$2.bind.o"
  else
    echo "ref_build: $1 (generated binding) failed (see $OUT/$2.log)"; bad=$((bad+1))
  fi
}
build_gen example/perf/aieml_perf.cc aieml_perf_gen
build_gen example/matrixmultiply/aieml_mm.cc aieml_mm_gen
build_gen example/multi/multi_tile.cpp multi_tile_gen
build_gen example/multi/seq_full_col.cpp seq_full_col_gen
build_gen example/multi/multi_kernel.cc multi_kernel_gen
build_gen tutorial/example.cpp tutorial_example_gen
rm -rf "$GEN"   # intermediate sources derived from the tree: not kept
echo "ref_build: $ok built, $bad failed -> $OUT"
[ "$bad" -eq 0 ]
