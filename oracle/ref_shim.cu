// C entry points around the reference's own CUDA kernels, compiled from the
// reference tree where it lies (see build_ref.sh).  TEST INFRASTRUCTURE: a second
// checker that pins the CPU oracle against the real reference code on a GPU; the
// product never loads it.  This file only declares the reference's launchers
// (signatures as in kangaroo_smat/kangaroo_smat.cpp:43-82) and supplies the three
// libbase symbols they link against.
#include <cuda_runtime.h>
#include <smat/dtypes.h>
#include <smat_cuda/launch_util.h>
#include <base/assert.h>
#include "kangaroo_smat.h"
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
using namespace sm;

void launch_corr1ord(cudaStream_t stream, dtype_t dtype, const void* W, usize_t m, usize_t nfilter,
                     const uint8_t* X, usize_t n, usize_t nchannel, void* Z);
void launch_corr1ord_bprop_W(cudaStream_t stream, dtype_t dtype, void* dW, usize_t m, usize_t nfilter,
                             const uint8_t* X, usize_t n, usize_t nchannel, const void* dZ);
void launch_poolrgn(cudaStream_t stream, dtype_t dtype, const void* featuremaps, usize_t nfeaturemap,
                    const uindex_t* regions, usize_t nregion, bool per_region_step,
                    void* pooledmap, uindex_t* pooledmap_argmax, pooltype_t ptype);
void launch_poolrgn_bprop(cudaStream_t stream, dtype_t dtype, void* unpooledmaps, usize_t nfeaturemap,
                          const uindex_t* regions, usize_t nregion, bool per_region_step,
                          const void* pooledmaps, const uindex_t* pooledmaps_argmax, pooltype_t ptype);

SM_NAMESPACE_BEGIN
void assert_failed_print(const char* fmt, ...)
{
	va_list ap; va_start(ap, fmt); vfprintf(stderr, fmt, ap); va_end(ap); fputc('\n', stderr);
}
void assert_failed(const char* fmt, ...)
{
	char buf[512]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
	throw std::runtime_error(buf);
}
unsigned lcm(unsigned a, unsigned b)
{
	unsigned x = a, y = b;
	while (y) { unsigned t = x % y; x = y; y = t; }
	return a / x * b;
}
launchcfg make_elemwise_launchcfg(usize_t size)
{
	unsigned bdx = 256, gdx = (size + bdx - 1) / bdx;
	if (gdx < 1) gdx = 1;
	if (gdx > 4096) gdx = 4096;
	return launchcfg(dim3(gdx), dim3(bdx), 0, 0);
}
SM_NAMESPACE_END

#define REF_TRY try {
#define REF_CATCH } catch (const std::exception& e) { fprintf(stderr, "ref: %s\n", e.what()); return 1; } \
	return cudaGetLastError() == cudaSuccess ? 0 : 2;

// dtype: 9 = f32, 10 = f64 (smat/dtypes.h).  n = number of rows written = npos - m + 1.
extern "C" __attribute__((visibility("default")))
int ref_corr1ord(int dtype, const void* W, unsigned m, unsigned nf, const uint8_t* X, unsigned n, void* Z)
{ REF_TRY launch_corr1ord(0, (dtype_t)dtype, W, m, nf, X, n, 4, Z); REF_CATCH }

extern "C" __attribute__((visibility("default")))
int ref_corr1ord_bprop_W(int dtype, void* dW, unsigned m, unsigned nf, const uint8_t* X, unsigned n, const void* dZ)
{ REF_TRY launch_corr1ord_bprop_W(0, (dtype_t)dtype, dW, m, nf, X, n, 4, dZ); REF_CATCH }

extern "C" __attribute__((visibility("default")))
int ref_poolrgn(int dtype, const void* U, unsigned nf, const uint32_t* R, unsigned nregion, int rcols,
                void* P, uint32_t* A, int ptype)
{ REF_TRY launch_poolrgn(0, (dtype_t)dtype, U, nf, R, nregion, rcols == 3, P, A, (pooltype_t)ptype); REF_CATCH }

extern "C" __attribute__((visibility("default")))
int ref_poolrgn_bprop(int dtype, void* U, unsigned nf, const uint32_t* R, unsigned nregion, int rcols,
                      const void* P, const uint32_t* A, int ptype)
{ REF_TRY launch_poolrgn_bprop(0, (dtype_t)dtype, U, nf, R, nregion, rcols == 3, P, A, (pooltype_t)ptype); REF_CATCH }
