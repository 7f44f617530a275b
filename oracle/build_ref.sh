#!/bin/sh
# Compiles the reference's own motif-scan and pooling kernels, from the sources
# where they lie in the reference tree, into oracle/_ref/libdeepbind_ref.so.
# Nothing is copied: nvcc reads the reference files in place.  The two backward
# sources include smat_cuda/launch_util.h, whose atomicAdd(double*) shim no longer
# compiles; ref_shadow/ supplies a stand-in that comes first on the include path.
#   usage: build_ref.sh <reference root> [nvcc]
set -e
REF="${1:-/root/reference}"
NVCC="${2:-/usr/local/cuda/bin/nvcc}"
HERE="$(cd "$(dirname "$0")" && pwd)"
L="$REF/code/libs"
K="$L/kangaroo/kangaroo_smat"
OUT="$HERE/_ref"
mkdir -p "$OUT"
FLAGS="-std=c++14 -O2 -use_fast_math -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -w
       -I $HERE/ref_shadow -I $L/smat/src -I $K -include $L/smat/src/nvcc_preinclude.h"
for f in corr1ord corr1ord_bprop poolrgn poolrgn_bprop; do
	"$NVCC" $FLAGS -c "$K/$f.cu" -o "$OUT/$f.o"
done
"$NVCC" $FLAGS -c "$HERE/ref_shim.cu" -o "$OUT/ref_shim.o"
"$NVCC" -gencode arch=compute_100a,code=sm_100a -shared -o "$OUT/libdeepbind_ref.so" \
	"$OUT/corr1ord.o" "$OUT/corr1ord_bprop.o" "$OUT/poolrgn.o" "$OUT/poolrgn_bprop.o" "$OUT/ref_shim.o"
rm -f "$OUT"/*.o
echo "$OUT/libdeepbind_ref.so"
