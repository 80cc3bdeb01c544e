#!/bin/sh
# Compiles the reference's header-only CPU callbacks (against ref_shim/ggml.h) and its tensor class
# (src/utils/tensor.hpp), from where they lie in the reference tree, into oracle/_ref/libedref_cpu.so, and its
# tensor-name conversion into oracle/_ref/libedref_names.so.
# Test infrastructure.
# Usage: sh oracle/build_ref.sh [reference root]
# The reference root comes from the argument, else from EDB200_REFERENCE_DIR, else a directory named
# "reference" beside this repository is tried; without one nothing is built.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${EDB200_REFERENCE_DIR:-$(dirname "$(dirname "$HERE")")/reference}}"
SRC="$REF/src/core/backend/ggml"
if [ ! -f "$SRC/ed_ggml_modulation_ext.hpp" ]; then
    echo "build_ref.sh: reference tree not found at $REF (nothing built)" >&2
    exit 0
fi
mkdir -p "$HERE/_ref"
g++ -O2 -std=c++17 -fPIC -shared -ffp-contract=off -I "$HERE/ref_shim" -I "$SRC" -I "$REF/src/core" -I "$REF/src" \
    "$HERE/ref_driver.cpp" "$HERE/ref_tensor_driver.cpp" -o "$HERE/_ref/libedref_cpu.so"
echo "$HERE/_ref/libedref_cpu.so"
# The reference's tensor-name conversion (src/utils/name_conversion.cpp) behind a C door: pins the weight
# loaders' canonicalisation rules.
g++ -O1 -std=c++17 -fPIC -shared -I "$HERE/ref_shim" -I "$REF/src" -I "$REF/include" -I "$REF/src/core" \
    "$REF/src/utils/name_conversion.cpp" "$HERE/ref_names_driver.cpp" -o "$HERE/_ref/libedref_names.so"
echo "$HERE/_ref/libedref_names.so"
