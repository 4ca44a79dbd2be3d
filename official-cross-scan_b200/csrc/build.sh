#!/usr/bin/env bash
# Builds the cs2d shared library in-tree for sm_100a.
#   official-cross-scan_b200/csrc/build.sh [extra nvcc flags]
# CS2D_OUT=<file> writes the library elsewhere.
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
out="${CS2D_OUT:-$here/../cs2d/libcs2d.so}"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 \
  -Xcompiler -fPIC -shared -cudart static --threads 7 "$@" \
  -o "$out" "$here/cs2d_api.cu" "$here/cs2d_fwd.cu" "$here/cs2d_bwd.cu" "$here/cs2d_fwd_serial.cu" "$here/cs2d_bwd_serial.cu" "$here/cs2d_stream_fwd.cu" "$here/cs2d_stream_bwd.cu" "$here/cs2d_walk_fwd.cu"
echo "built $out"
