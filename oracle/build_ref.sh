#!/bin/sh
# Compiles the reference's own kernels and launchers for this path, from the
# sources where they lie in the reference tree, into oracle/_ref/libdeepbind_ref.so:
# the motif scan and pooling kernels with their backward passes, input dropout
# (kangaroo_smat), the update, mask, dropout and block-diagonal product launchers
# (deepity_smat), smat's element-wise kernels (smat_cuda/elemwise2.cu, elemwise3.cu: what
# the reference's bias, rectify, logistic and loss nodes run on, with the array descriptor
# of smat/vm/argument.cpp and smat/shape.cpp) and the element-wise launch rule
# (smat_cuda/launch_util.cpp).
# Nothing is copied: nvcc reads the reference files in place.  ref_shadow/ comes
# first on the include path and stands in for two headers: launch_util.h (its
# atomicAdd(double*) shim no longer compiles) and cuda_context.h (the thread
# context of libsmat's virtual machine, which is not built).
#   usage: build_ref.sh <reference root> [nvcc]
set -e
REF="${1:-${DEEPBIND_REFERENCE_ROOT:?usage: build_ref.sh <reference root> [nvcc]}}"
NVCC="${2:-${NVCC:-nvcc}}"
HERE="$(cd "$(dirname "$0")" && pwd)"
L="$REF/code/libs"
K="$L/kangaroo/kangaroo_smat"
D="$L/deepity/deepity_smat"
OUT="$HERE/_ref"
mkdir -p "$OUT"
FLAGS="-std=c++14 -O2 -use_fast_math -gencode arch=compute_100a,code=sm_100a -Xcompiler -fPIC -w
       -I $HERE/ref_shadow -I $L/smat/src -I $K -I $D -include $L/smat/src/nvcc_preinclude.h"
OBJS=""
for f in "$K/corr1ord.cu" "$K/corr1ord_bprop.cu" "$K/poolrgn.cu" "$K/poolrgn_bprop.cu" "$K/dropoutord.cu" \
         "$D/gradstep.cu" "$D/madd_bcast.cu" "$D/maskout.cu" "$D/dropout.cu" "$D/blockwise_dot.cu" \
         "$L/smat/src/smat_cuda/elemwise2.cu" "$L/smat/src/smat_cuda/elemwise3.cu" \
         "$L/smat/src/smat/vm/argument.cpp" "$L/smat/src/smat/shape.cpp" \
         "$L/smat/src/smat_cuda/launch_util.cpp" "$HERE/ref_shim.cu"; do
	o="$OUT/$(basename "$f" | sed 's/\.[a-z]*$//').o"
	"$NVCC" $FLAGS -x cu -c "$f" -o "$o"
	OBJS="$OBJS $o"
done
"$NVCC" -gencode arch=compute_100a,code=sm_100a -shared -o "$OUT/libdeepbind_ref.so" $OBJS -lcublas
rm -f "${OUT:?}"/*.o
echo "$OUT/libdeepbind_ref.so"
