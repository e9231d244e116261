#!/bin/bash
# Builds the UNMODIFIED reference into baseline/_ref/piccl.so from a writable copy of its
# sources (the reference tree itself is read-only).  Deviations from the reference's
# src/Makefile:8-9, all on the command line, none in the sources:
#   * -I$CUDA_HOME/include/nvtx3   (CUDA >= 12.9 ships <nvToolsExt.h> only under nvtx3/)
#   * no -lnvToolsExt              (NVTX3 is header only)
#   * -gencode arch=compute_100,code=sm_100 (the reference passes no arch at all)
# Usage: baseline/build_ref.sh [reference_root]   (default: $PICCL_REFERENCE_ROOT, else the reference checkout mounted beside this repository)
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
REF="${1:-${PICCL_REFERENCE_ROOT:-$HERE/../../reference}}"
CUDA_HOME="${CUDA_HOME:-/usr/local/cuda}"
OUT="$HERE/_ref"
if [ ! -d "$REF/src" ] && [ -d "$OUT/src" ]; then REF="$OUT"; fi
if [ ! -d "$REF/src" ]; then echo "reference sources not found at $REF" >&2; exit 3; fi
mkdir -p "$OUT"
if [ "$REF" != "$OUT" ]; then [ -d "$OUT/src" ] && chmod -R u+w "$OUT/src"; rm -rf "$OUT/src"; cp -r "$REF/src" "$OUT/src"; chmod -R u+w "$OUT/src"; fi
cd "$OUT/src"
"$CUDA_HOME/bin/nvcc" -gencode arch=compute_100,code=sm_100 -Xcompiler "-fPIC -O2 -w" \
  -I"$CUDA_HOME/include" -I"$CUDA_HOME/include/nvtx3" -I/usr/include -Iinclude \
  piccl.c coll/*.c kernels/*.cu -o "$OUT/piccl.so" -shared -ldl -L"$CUDA_HOME/lib64" -lcudart \
  -L/usr/lib/x86_64-linux-gnu -lnccl
echo "built $OUT/piccl.so"
