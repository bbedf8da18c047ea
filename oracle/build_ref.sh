#!/bin/bash
# TEST INFRASTRUCTURE.  Builds the reference's own kernels (buaa-hipo/cuSpAMM, cuSpAMM.cu) for sm_100a into
# oracle/_ref/libref_<N>.so, one library per matrix size, for the GPU cross-check in tests/.
#
# The reference fixes its sizes at compile time (para.h:6-8), so the sources are copied to a scratch directory,
# the three size constants of para.h are set there, and ref_wrap.cu (launchers only) is compiled next to them.
# Nothing of the reference is written into this repository; oracle/_ref/ holds build outputs only and is
# git-ignored.  Needs the reference sources ($SPAMM_REFERENCE_DIR, or a directory `reference` beside this repository)
# and nvcc; does nothing when they are absent.
set -euo pipefail
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
REF="${SPAMM_REFERENCE_DIR:-$HERE/../../reference}"
OUT="$HERE/_ref"
SIZES="${SPAMM_REF_SIZES:-512 2048 8192}"
if [ ! -f "$REF/cuSpAMM.cu" ]; then echo "reference sources not found at $REF: nothing built"; exit 0; fi
NVCC="$(command -v nvcc || echo /usr/local/cuda/bin/nvcc)"
mkdir -p "$OUT"
for n in $SIZES; do
    tmp="$(mktemp -d /tmp/spamm_ref_XXXXXX)"
    cp "$REF/cuSpAMM.cu" "$REF/tool.cu" "$REF/main.h" "$REF/para.h" "$tmp/"
    chmod u+w "$tmp"/*
    sed -i -E "s/^const int inM=[0-9]+;/const int inM=$n;/; s/^const int inK=[0-9]+;/const int inK=$n;/; s/^const int inN=[0-9]+;/const int inN=$n;/" "$tmp/para.h"
    grep -q "inM=$n;" "$tmp/para.h" || { echo "could not set the size in para.h"; rm -rf "$tmp"; exit 1; }
    cp "$HERE/ref_wrap.cu" "$tmp/"
    (cd "$tmp" && "$NVCC" -O3 -w -gencode arch=compute_100a,code=sm_100a --std=c++11 -Xcompiler -fopenmp,-fPIC,-fpermissive \
        -shared -o "$OUT/libref_$n.so" ref_wrap.cu tool.cu -lcublas)
    rm -rf "$tmp"
    echo "built $OUT/libref_$n.so"
done
