#!/usr/bin/env bash
# TEST INFRASTRUCTURE. Compiles the reference project's own CPU reference for the MXFP8
# quantiser from the reference checkout into oracle/_ref/ (git-ignored). Needs nvcc only
# because the reference's host code uses CUDA's host-callable conversion intrinsics; no GPU
# is needed to build or to run the result.
#   usage: oracle/build_ref.sh [/path/to/reference/checkout]
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-/root/reference}"
src="$ref/prime_kernels/rmsnorm"
[ -f "$src/test.cu" ] || { echo "reference checkout not found at $ref; keeping any prebuilt oracle/_ref" >&2; exit 0; }
mkdir -p "$here/_ref"
nvcc -O2 -std=c++17 -shared -Xcompiler -fPIC -w \
  -gencode arch=compute_100a,code=sm_100a \
  -I"$src" -I"$src/src/include" \
  -DREF_TEST_CU="\"$src/test.cu\"" \
  -o "$here/_ref/libref_rmsnorm.so" "$here/ref_rmsnorm_wrapper.cu"
echo "built $here/_ref/libref_rmsnorm.so"
