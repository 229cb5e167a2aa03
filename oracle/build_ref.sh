#!/bin/sh
# TEST INFRASTRUCTURE. Compiles the reference's own card kernels, from where its sources lie, for sm_100a, with the
# reference's own nvcc flags (build.py:555: -O3 -std=c++17 --fatbin) and only the architecture changed. The output
# goes to oracle/_ref/ (git-ignored) and is loaded by the GPU tests as the bit-level oracle and as the same-box
# speed baseline. No reference source is copied.
set -e
REF="${1:-${BTB_REFERENCE:-$(cd "$(dirname "$0")/../.." && pwd)/reference}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
SRC="$REF/native/cuda/btb_kernels.cu"
[ -f "$SRC" ] || { echo "no reference checkout at $REF: keeping what is built" >&2; exit 0; }
mkdir -p "$HERE/_ref"
OUT="$HERE/_ref/btb_kernels.fatbin"
if [ ! -f "$OUT" ] || [ "$SRC" -nt "$OUT" ]; then
    nvcc -O3 -std=c++17 --fatbin -gencode arch=compute_100a,code=sm_100a -o "$OUT" "$SRC"
fi
echo "$OUT"
