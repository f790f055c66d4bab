#!/bin/sh
# Builds libsparsedrop.so for sm_100a next to the Python package (in-tree, not installed).
set -e
here="$(cd "$(dirname "$0")" && pwd)"
out="$here/../lib"
mkdir -p "$out"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -std=c++17 -O3 -lineinfo -gencode arch=compute_100a,code=sm_100a \
    -Xcompiler -fPIC -Xptxas -v --shared \
    -o "$out/libsparsedrop.so" \
    "$here/sd_api.cu" "$here/sd_plan.cu" "$here/sd_gemm.cu" "$here/sd_conv.cu" "$here/sd_norm.cu" "$here/sd_selftest.cu" "$@"
