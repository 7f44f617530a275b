// Stand-in for the reference's smat_cuda/launch_util.h, placed first on the
// include path when the reference's *_bprop.cu files are compiled as a checker.
// The original re-defines atomicAdd(double*, double), which has been a CUDA
// built-in since sm_60 and no longer compiles; this file declares only what the
// two backward sources use.  TEST INFRASTRUCTURE: not part of the product.
#ifndef DEEPBIND_REF_SHADOW_LAUNCH_UTIL_H
#define DEEPBIND_REF_SHADOW_LAUNCH_UTIL_H

#include <smat_cuda/config.h>
#include <smat/dtypes.h>
#include <cuda_runtime.h>

SM_NAMESPACE_BEGIN

struct launchcfg {
	launchcfg(const dim3& g, const dim3& b, unsigned s, cudaStream_t st): gdim(g), bdim(b), smem(s), stream(st) { }
	dim3 gdim, bdim;
	unsigned smem;
	cudaStream_t stream;
};

// One-dimensional grid-stride configuration (defined in ref_shim.cu).
launchcfg make_elemwise_launchcfg(usize_t size);

SM_NAMESPACE_END

#endif
