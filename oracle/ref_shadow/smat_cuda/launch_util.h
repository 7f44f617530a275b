// Stand-in for the reference's smat_cuda/launch_util.h, placed first on the
// include path when reference kernel sources are compiled as a checker.  The
// original re-defines atomicAdd(double*, double), which has been a CUDA built-in
// since sm_60 and no longer compiles; this file declares what the compiled
// sources use: the launch record, the element-wise launch rule (defined by the
// reference's own smat_cuda/launch_util.cpp, compiled beside it) and shorthands
// for the CUDA thread coordinates.  TEST INFRASTRUCTURE: not part of the product.
#ifndef DEEPBIND_REF_SHADOW_LAUNCH_UTIL_H
#define DEEPBIND_REF_SHADOW_LAUNCH_UTIL_H

#include <smat_cuda/config.h>
#include <smat/dtypes.h>
#include <cuda_runtime.h>

// Names the reference kernels use for thread and block coordinates.
#define DECL_KERNEL_VARS \
	const unsigned tx = threadIdx.x, ty = threadIdx.y, bx = blockIdx.x, by = blockIdx.y; \
	const unsigned bdx = blockDim.x, bdy = blockDim.y, gdx = gridDim.x, gdy = gridDim.y; \
	(void)tx; (void)ty; (void)bx; (void)by; (void)bdx; (void)bdy; (void)gdx; (void)gdy;

SM_NAMESPACE_BEGIN

struct launchcfg {
	launchcfg(const dim3& g, const dim3& b, unsigned s, cudaStream_t st): gdim(g), bdim(b), smem(s), stream(st) { }
	dim3 gdim, bdim;
	unsigned smem;
	cudaStream_t stream;
};

// One-dimensional grid-stride configuration (smat_cuda/launch_util.cpp:41-71).
launchcfg make_elemwise_launchcfg(usize_t size);

SM_NAMESPACE_END

#endif
