#!/bin/sh
# Builds libcleave_b200.so for sm_100a next to the package (in-tree, not installed).
set -e
HERE=$(cd "$(dirname "$0")" && pwd)
OUT="$HERE/../libcleave_b200.so"
NVCC=${NVCC:-/usr/local/cuda/bin/nvcc}
FLAGS="-gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 -Xcompiler -fPIC --expt-relaxed-constexpr"
mkdir -p "$HERE/build"
pids=""
for f in "$HERE"/*.cu; do
  o="$HERE/build/$(basename "$f" .cu).o"
  if [ ! -f "$o" ] || [ "$f" -nt "$o" ] || [ "$HERE/common.cuh" -nt "$o" ] || [ "$HERE/stream_walk.cuh" -nt "$o" ] || [ "$HERE/../../include/cleave_b200.h" -nt "$o" ]; then
    $NVCC $FLAGS $EXTRA_NVCC_FLAGS -c "$f" -o "$o" &
    pids="$pids $!"
  fi
done
for p in $pids; do wait $p; done
$NVCC -gencode arch=compute_100a,code=sm_100a -shared -o "$OUT" "$HERE"/build/*.o
echo "built $OUT"
