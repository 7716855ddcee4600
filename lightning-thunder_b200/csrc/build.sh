#!/bin/bash
# Builds libnf4_b200.so for sm_100a (the only target) next to the Python package.
set -e
set -o pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
OUT="$HERE/../nf4_b200/libnf4_b200.so"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
FLAGS="-gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 -Xcompiler -fPIC ${NF4_NVCC_EXTRA}"
mkdir -p "$HERE/build"
pids=()
for f in "$HERE"/*.cu; do
  o="$HERE/build/$(basename "${f%.cu}").o"
  if [ ! -f "$o" ] || [ "$f" -nt "$o" ] || [ "$HERE/nf4_common.cuh" -nt "$o" ] || [ "$HERE/../../include/nf4_b200.h" -nt "$o" ] || [ -n "$NF4_FORCE" ]; then
    $NVCC $FLAGS -c "$f" -o "$o" &
    pids+=($!)
  fi
done
for p in "${pids[@]}"; do wait "$p" || { echo "nvcc failed (see messages above)" >&2; exit 1; }; done
$NVCC -shared -o "$OUT" "$HERE"/build/*.o -lcudart
echo "built $OUT"
