#!/usr/bin/env bash
# TEST INFRASTRUCTURE. Compiles, from the reference checkout where it lies, into oracle/_ref/
# (git-ignored):
#   libref_rmsnorm.so       the reference's own CPU reference() for the MXFP8 quantiser (needs nvcc only
#                           because its host code uses CUDA's host-callable conversion intrinsics; runs
#                           without a GPU)
#   libref_rmsnorm_gpu.so   the reference's own GPU kernels behind a C entry point (GPU parity tests)
#   ref_rmsnorm_bench       the reference's own benchmark executable (same-box timing of its kernels)
#   libref_megakernel135.so, libref_megakernel360.so, libref_megakernel360f.so
#                           the reference's own SmolLM2-135M / 360M decode megakernels (their sm_89-only device check
#                           shimmed, see ref_megakernel_wrapper.cu): second decode oracle and same-box baseline.
#                           360f is the fast 360M line (decode_megakernel_360m_lossless, entry decode360_lossless),
#                           run with a NULL encoded gate-up table, i.e. on the plain bf16 weights
# The reference's cmake project is not run: its sources are handed to nvcc directly.
#   usage: oracle/build_ref.sh [/path/to/reference/checkout]
set -euo pipefail
here="$(cd "$(dirname "$0")" && pwd)"
ref="${1:-/root/reference}"
src="$ref/prime_kernels/rmsnorm"
[ -f "$src/test.cu" ] || { echo "reference checkout not found at $ref; keeping any prebuilt oracle/_ref" >&2; exit 0; }
mkdir -p "$here/_ref"
# fresh OUT IN...: true when OUT exists and is newer than every input
fresh() { local out="$1"; shift; [ -f "$out" ] || return 1; for f in "$@"; do [ "$out" -nt "$f" ] || return 1; done; }
fresh "$here/_ref/libref_rmsnorm.so" "$src/test.cu" "$here/ref_rmsnorm_wrapper.cu" || \
nvcc -O2 -std=c++17 -shared -Xcompiler -fPIC -w \
  -gencode arch=compute_100a,code=sm_100a \
  -I"$src" -I"$src/src/include" \
  -DREF_TEST_CU="\"$src/test.cu\"" \
  -o "$here/_ref/libref_rmsnorm.so" "$here/ref_rmsnorm_wrapper.cu"
echo "built $here/_ref/libref_rmsnorm.so"
kernels=("$src/rmsnorm.cu" "$src"/src/kernels/rmsnorm_0[0-5]_*.cu)
common=(-O3 -std=c++20 -w -gencode arch=compute_100a,code=sm_100a -I"$src" -I"$src/src/include")
headers=("$src/rmsnorm.cuh" "$src"/src/include/*)
fresh "$here/_ref/libref_rmsnorm_gpu.so" "${kernels[@]}" "${headers[@]}" "$here/ref_rmsnorm_gpu_wrapper.cu" || \
nvcc "${common[@]}" -shared -Xcompiler -fPIC -o "$here/_ref/libref_rmsnorm_gpu.so" \
  "${kernels[@]}" "$here/ref_rmsnorm_gpu_wrapper.cu" -lcuda
echo "built $here/_ref/libref_rmsnorm_gpu.so"
fresh "$here/_ref/ref_rmsnorm_bench" "${kernels[@]}" "${headers[@]}" "$src/bench.cu" || \
nvcc "${common[@]}" -o "$here/_ref/ref_rmsnorm_bench" "${kernels[@]}" "$src/bench.cu" -lcuda
echo "built $here/_ref/ref_rmsnorm_bench"
mk="$ref/prime_kernels/decode_megakernel/csrc/megakernel.cu"
if [ -f "$mk" ]; then
  fresh "$here/_ref/libref_megakernel135.so" "$mk" "$here/ref_megakernel_wrapper.cu" || \
  nvcc -O3 -std=c++17 -w -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC -DMK_PREFETCH=1 \
    -DREF_MEGAKERNEL_CU="\"$mk\"" -o "$here/_ref/libref_megakernel135.so" "$here/ref_megakernel_wrapper.cu"
  echo "built $here/_ref/libref_megakernel135.so"
fi
mk360="$ref/prime_kernels/decode_megakernel_360m/csrc/block360.cu"
if [ -f "$mk360" ]; then
  fresh "$here/_ref/libref_megakernel360.so" "$mk360" "$ref/prime_kernels/decode_megakernel_360m/csrc/block360_kernel.inc" \
        "$here/ref_megakernel_wrapper.cu" || \
  nvcc -O3 -std=c++17 -w -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC \
    -DREF_MEGAKERNEL_CU="\"$mk360\"" -o "$here/_ref/libref_megakernel360.so" "$here/ref_megakernel_wrapper.cu"
  echo "built $here/_ref/libref_megakernel360.so"
fi
mk360f="$ref/prime_kernels/decode_megakernel_360m_lossless/csrc/block360.cu"
if [ -f "$mk360f" ]; then
  fresh "$here/_ref/libref_megakernel360f.so" "$mk360f" "$ref/prime_kernels/decode_megakernel_360m_lossless/csrc/block360_kernel.inc" \
        "$ref/prime_kernels/lossless_bf16/csrc/encoded_gu.h" "$here/ref_megakernel_wrapper.cu" || \
  nvcc -O3 -std=c++17 -w -gencode arch=compute_100a,code=sm_100a -shared -Xcompiler -fPIC \
    -DREF_MEGAKERNEL_CU="\"$mk360f\"" -o "$here/_ref/libref_megakernel360f.so" "$here/ref_megakernel_wrapper.cu"
  echo "built $here/_ref/libref_megakernel360f.so"
fi
