#!/usr/bin/env bash
# Builds the reference's own test programs, unmodified and where they lie in the reference checkout, against
# THIS repository's include/librecuda.h and libdriverapi.so, and compiles their fixture kernels for sm_100a
# under the file names the programs open.  The binaries land in oracle/_ref/compat/<program>/ and are run on
# the GPU by tests/test_compat_programs.py.  This is the drop-in check: if a reference caller stops
# compiling or linking, the boundary has drifted.  TEST INFRASTRUCTURE ONLY; nothing is copied from the
# reference and no disassembly step of the reference's fixture script is run.
#   usage: oracle/build_compat.sh [reference-checkout]
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
root="$(dirname "$here")"
ref="${1:-${LIBRECUDA_REFERENCE:-$root/../reference}}"
lib="$root/librecuda_b200/lib"
[ -d "$ref/tests" ] || { echo "no reference checkout at $ref: skipping compat programs"; exit 0; }
[ -f "$lib/libdriverapi.so" ] || { echo "build libdriverapi.so first (python -m librecuda_b200.build)"; exit 1; }
nvcc="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
for dir in "$ref"/tests/*/; do
  name="$(basename "$dir")"
  [ -f "$dir/main.cpp" ] || continue
  out="$here/_ref/compat/$name"
  mkdir -p "$out"
  g++ -std=c++17 -O1 -w -I"$root/include" "$dir/main.cpp" -L"$lib" -ldriverapi \
      -Wl,-rpath,'$ORIGIN/../../../../librecuda_b200/lib' -o "$out/$name"
  for cu in "$dir"/*.cu; do
    [ -f "$cu" ] || continue
    "$nvcc" -cubin -gencode arch=compute_100a,code=sm_100a -O3 -o "$out/$(basename "${cu%.cu}").cubin" "$cu"
  done
  echo "built $out"
done
