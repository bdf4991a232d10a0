#!/bin/sh
# Regenerates the golden files of this folder from the reference's own CPU sources
# (src/ops/sampling.cpp and src/engine/scheduler.cpp compile with plain g++; its model code
# does not run without a GPU: every tensor it touches is a CUDA tensor).  Usage:
#     sh tests/golden/make_golden.sh /path/to/reference
# The committed *.json files are what the tests read; this script is not run by them.
set -e
REF=${1:?path of the reference checkout}
HERE=$(cd "$(dirname "$0")" && pwd)
TMP=$(mktemp -d)
g++ -std=c++20 -O1 -I"$REF/include" "$HERE/golden_sampling.cpp" "$REF/src/ops/sampling.cpp" -o "$TMP/gs"
"$TMP/gs" > "$HERE/sampling_golden.json"
g++ -std=c++20 -O1 -I"$REF/include" "$HERE/golden_scheduler.cpp" "$REF/src/engine/scheduler.cpp" -o "$TMP/gd"
"$TMP/gd" > "$HERE/scheduler_golden.json"
# The CPU oracles of the reference's attention and head tests (static functions of its test programs; the programs
# are compiled whole with the sources they name, nothing of them runs on a GPU).  Needs nvcc, no GPU.
nvcc -std=c++17 -O1 -w -I"$REF/include" -I"$REF" "$HERE/golden_attention.cu" "$REF/src/tensor.cpp" "$REF/src/allocator.cpp" \
    "$REF/src/kv_cache/block_allocator.cpp" "$REF/src/kv_cache/hash_prefix_cache.cpp" \
    "$REF/src/kv_cache/radix_prefix_cache.cpp" "$REF/src/kv_cache/paged_attention.cu" "$REF/src/ops/lm_head.cu" \
    "$REF/src/ops/gemm.cu" -lcublas -o "$TMP/ga"
"$TMP/ga" > "$HERE/attention_golden.json"
rm -rf "$TMP"
echo "wrote sampling_golden.json, scheduler_golden.json and attention_golden.json"
