#!/bin/sh
# Regenerates ops_golden.json from the reference's own GPU operators (norm, SiLU, embedding: the ones whose kernels
# follow their formulas).  Needs nvcc and a GPU.  Usage:
#     sh tests/golden/make_golden_gpu.sh /path/to/reference [output.json]
set -e
REF=${1:?path of the reference checkout}
HERE=$(cd "$(dirname "$0")" && pwd)
OUT=${2:-$HERE/ops_golden.json}
TMP=$(mktemp -d)
nvcc -std=c++17 -O1 -w -gencode arch=compute_100a,code=sm_100a -I"$REF/include" "$HERE/golden_ops.cu" "$REF/src/tensor.cpp" \
    "$REF/src/allocator.cpp" "$REF/src/ops/norm.cu" "$REF/src/ops/elementwise.cu" "$REF/src/ops/embedding.cu" -o "$TMP/go"
"$TMP/go" > "$OUT"
rm -rf "$TMP"
echo "wrote $OUT"
