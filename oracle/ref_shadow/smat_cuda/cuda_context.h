// Stand-in for the reference's smat_cuda/cuda_context.h.  The original is the
// thread context of libsmat's virtual machine; the reference sources compiled
// as a checker only ask it for the device properties, the stream, a cuBLAS
// handle, the per-thread cuRAND states and a scratch allocation, so this class
// offers exactly those (defined in ref_shim.cu).  TEST INFRASTRUCTURE: not part
// of the product.
#ifndef DEEPBIND_REF_SHADOW_CUDA_CONTEXT_H
#define DEEPBIND_REF_SHADOW_CUDA_CONTEXT_H

#include <smat_cuda/config.h>
#include <cuda_runtime.h>
#include <curand.h>
#include <curand_kernel.h>
#include <cublas_v2.h>
#include <cstddef>

SM_NAMESPACE_BEGIN

struct heap_alloc {
	void*  addr;
	size_t size;
};

class ref_heap {
public:
	heap_alloc alloc(size_t size);
	void       free(heap_alloc& a);
};

class cuda_context {
public:
	cudaStream_t          stream() const;
	cublasHandle_t        cublas() const;
	curandState*          curand_state() const;
	const cudaDeviceProp& deviceprop() const;
	ref_heap&             heap();
};

cuda_context& thread_cudactx();

SM_NAMESPACE_END

#endif
