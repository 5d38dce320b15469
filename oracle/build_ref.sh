#!/bin/bash
# Test infrastructure only.  Builds the reference toolkit's own Cpu-device implementation of the
# LSTM training path into oracle/_ref/libcurrennt_ref.so (serial Thrust host backend, the
# reference's CMake default) and oracle/_ref/libcurrennt_ref_omp.so (Thrust OpenMP host backend).
#
# The sources are compiled from the reference checkout (the directory in $REF); nothing
# of them is kept: one mechanical rewrite is needed for CUDA 12.9 (Thrust 2.8 maps thrust::tuple
# onto cuda::std::tuple, which has no .get<N>() member, so `x.get<N>()` becomes
# `thrust::get<N>(x)`), it is applied to a scratch copy under oracle/_ref/build/ that is deleted
# when the libraries are linked.  Boost and the Configuration singleton are replaced by the small
# stand-ins in oracle/ref_build/.  Does nothing (exit 0) if the reference checkout is absent.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
# the reference checkout: $REF, else a directory named "reference" beside this repository
REF="${REF:-$(cd "$HERE/../.." && pwd)/reference}"
SRC="$REF/CURRENNT_codes/currennt_lib/src"
OUT="$HERE/_ref"
if [ ! -d "$SRC" ]; then echo "build_ref: no reference checkout at $REF, skipping"; exit 0; fi
if [ -f "$OUT/libcurrennt_ref.so" ] && [ -f "$OUT/libcurrennt_ref_omp.so" ] && [ -f "$OUT/libcurrennt_ref_b200.so" ] && [ -z "$FORCE" ] \
   && [ "$OUT/libcurrennt_ref_b200.so" -nt "$HERE/../project-currennt-public_b200/adapter/LstmLayerB200.hpp" ] \
   && [ "$OUT/libcurrennt_ref.so" -nt "$HERE/ref_build/ref_harness.cu" ] \
   && [ "$OUT/libcurrennt_ref.so" -nt "$HERE/ref_build/cfgstub.cpp" ]; then
  echo "build_ref: up to date"; exit 0
fi
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
B="$OUT/build"
rm -rf "$B"; mkdir -p "$B/src"
cp -r "$SRC/." "$B/src/"; chmod -R u+w "$B/src"
find "$B/src" \( -name '*.cu' -o -name '*.cuh' -o -name '*.hpp' \) -print0 | \
  xargs -0 sed -i 's/\([A-Za-z_][A-Za-z0-9_]*\)\.get<\([0-9]\)>()/thrust::get<\2>(\1)/g'
CU="layers/Layer.cu layers/TrainableLayer.cu layers/LstmLayer.cu layers/FeedForwardLayer.cu
    layers/InputLayer.cu layers/PostOutputLayer.cu layers/SsePostOutputLayer.cu
    helpers/Matrix.cu helpers/cublas.cu helpers/misFuncs.cu helpers/vecPoolManager.cu helpers/dataProcess.cu"
CPP="helpers/JsonClasses.cpp data_sets/DataSetFraction.cpp"
INC="-I$HERE/ref_build/shim -I$B/src -I/usr/local/cuda/include"
build_variant() {   # $1 = suffix, $2.. = extra flags
  local sfx="$1"; shift
  local O="$B/obj$sfx"; mkdir -p "$O"
  local pids=()
  for f in $CU; do
    "$NVCC" -std=c++14 -O2 -w -Wno-deprecated-gpu-targets -Xcompiler -fPIC "$@" $INC \
       -c "$B/src/$f" -o "$O/$(basename "$f" .cu).o" & pids+=($!)
  done
  "$NVCC" -std=c++14 -O2 -w -Wno-deprecated-gpu-targets -Xcompiler -fPIC "$@" $INC \
       -c "$HERE/ref_build/ref_harness.cu" -o "$O/ref_harness.o" & pids+=($!)
  for f in $CPP; do
    g++ -std=c++14 -O2 -w -fPIC $INC -c "$B/src/$f" -o "$O/$(basename "$f" .cpp).o" & pids+=($!)
  done
  g++ -std=c++14 -O2 -w -fPIC $INC -c "$HERE/ref_build/cfgstub.cpp" -o "$O/cfgstub.o" & pids+=($!)
  for p in "${pids[@]}"; do wait "$p"; done
  "$NVCC" -shared -o "$OUT/libcurrennt_ref$sfx.so" "$O"/*.o -lcublas "${LINK_EXTRA[@]}"
}
LINK_EXTRA=()
build_variant ""
LINK_EXTRA=(-lgomp)
build_variant "_omp" -Xcompiler -fopenmp -DTHRUST_HOST_SYSTEM=THRUST_HOST_SYSTEM_OMP
# The drop-in claim, compiled: the reference's Gpu-device classes (device code for the B200) with the adapter class
# project-currennt-public_b200/adapter/LstmLayerB200.hpp in place of LstmLayer<Gpu>, linked against libb2lstm.so
# (found at run time beside this repository's package through the run path).
PKG="$(cd "$HERE/../project-currennt-public_b200" && pwd)"
if [ -f "$PKG/libb2lstm.so" ]; then
  LINK_EXTRA=(-L"$PKG" -lb2lstm -Xlinker -rpath -Xlinker '$ORIGIN/../../project-currennt-public_b200')
  build_variant "_b200" -gencode arch=compute_100a,code=sm_100a -DREF_WITH_B200_ADAPTER -I"$PKG/adapter" -I"$HERE/../include"
else
  echo "build_ref: libb2lstm.so not built yet, skipping the adapter variant"
fi
rm -rf "$B"
ls -la "$OUT"
