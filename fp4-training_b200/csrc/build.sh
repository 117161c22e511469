#!/usr/bin/env bash
# Builds the C-ABI library for sm_100a into ../lib/libfp4t.so (in-tree, git-ignored).
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
out="$here/../lib"
mkdir -p "$out"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -O3 -lineinfo -std=c++17 \
  -Xcompiler -fPIC -Xcompiler -fvisibility=hidden -shared ${FP4T_NVCC_EXTRA:-} \
  -o "$out/libfp4t.so" \
  "$here/fp4t_quantize.cu" "$here/fp4t_gemm.cu" "$here/fp4t_misc.cu" "$here/fp4t_linear.cu" "$here/fp4t_allreduce.cu" "$here/fp4t_norm.cu"
echo "built $out/libfp4t.so"
