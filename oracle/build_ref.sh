#!/usr/bin/env bash
# Builds the oracle's C restatement and, when a reference checkout is available, the reference's own DtoD
# dispatcher + kernels compiled for the host (oracle/_ref/libref_memcopy.so).  Reference sources are
# compiled where they lie; nothing is copied.  TEST INFRASTRUCTURE ONLY.
#   usage: oracle/build_ref.sh [reference-checkout]      (default: $LIBRECUDA_REFERENCE, else the directory `reference` beside this repository)
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ref="${1:-${LIBRECUDA_REFERENCE:-$(dirname "$here")/../reference}}"
mkdir -p "$here/_build"
gcc -O2 -fPIC -shared -pthread -ffp-contract=off -o "$here/_build/liblcb_oracle.so" "$here/lcb_oracle.c"
echo "built $here/_build/liblcb_oracle.so"
if [ -d "$ref/driverapi/src" ]; then
  mkdir -p "$here/_ref"
  d="$ref/driverapi"
  g++ -std=c++17 -O2 -fPIC -shared -w \
      -I"$d/include" -I"$d/internal" -I"$here" \
      "$d/src/memcopy.cpp" "$d/src/librecuda_status.cpp" \
      -x c++ -include "$here/ref_host_cuda_shim.h" "$d/kernels/memcpy/memcpy.cu" \
      -x none "$here/ref_shim.cpp" \
      -o "$here/_ref/libref_memcopy.so"
  echo "built $here/_ref/libref_memcopy.so"
  # the same kernel source as a real sm_100a image, so the reference's kernels can run on the B200 beside
  # this library's (launched with the reference's grid shapes by tests and, for timing, by bench.py)
  nvcc="${CUDA_HOME:-/usr/local/cuda}/bin/nvcc"
  if [ -x "$nvcc" ]; then
    "$nvcc" -cubin -gencode arch=compute_100a,code=sm_100a -O3 -o "$here/_ref/ref_memcpy_sm100a.cubin" "$d/kernels/memcpy/memcpy.cu"
    echo "built $here/_ref/ref_memcpy_sm100a.cubin"
  fi
else
  echo "no reference checkout at $ref: skipping oracle/_ref"
fi
