#!/bin/sh
# Regenerates the golden files of this folder from the reference's own CPU sources
# (src/ops/sampling.cpp and src/engine/scheduler.cpp compile with plain g++; its model code
# does not: every tensor it touches is a CUDA tensor).  Usage:
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
rm -rf "$TMP"
echo "wrote sampling_golden.json and scheduler_golden.json"
