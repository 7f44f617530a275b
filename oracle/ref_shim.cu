// C entry points around the reference's own CUDA kernels and host loops, compiled
// from the reference tree where it lies (see build_ref.sh).  TEST INFRASTRUCTURE: a
// second checker that pins the CPU oracle against the real reference code on a GPU;
// the product never loads it.  This file only declares the reference's launchers
// (signatures as in kangaroo_smat/kangaroo_smat.cpp:43-82 and
// deepity_smat/deepity_smat.cpp:42-100), supplies the libbase symbols they link
// against, and defines the small context of ref_shadow/smat_cuda/cuda_context.h
// (stream 0, a cuBLAS handle, cuRAND states seeded as smat_cuda/rand.cu:129-135).
#include <cuda_runtime.h>
#include <smat/dtypes.h>
#include <smat_cuda/launch_util.h>
#include <smat_cuda/cuda_context.h>
#include <smat_cuda/cuda_errors.h>
#include <base/assert.h>
#include <smat/vm/argument.h>
#include <smat/vm/instruction_db.h>
#include "kangaroo_smat.h"
#include <cstring>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>
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

void launch_corr1ord_bprop_X(cudaStream_t stream, dtype_t dtype, void* dX, usize_t n, usize_t nchannel,
                             const void* W, usize_t m, usize_t nfilter, const void* dZ);
void launch_dropoutord_fp_tr(cudaStream_t stream, const uint8_t* X, uint8_t* Z, bool* M, usize_t n, float rate);
void launch_gradstep(cudaStream_t stream, dtype_t dtype, isize_t n, void* P, const void* dP, const void* drate,
                     void* mP, const void* mrate);
void launch_gradstep_nesterov1(cudaStream_t stream, dtype_t dtype, isize_t n, void* P, const void* mP, const void* mrate);
void launch_gradstep_nesterov2(cudaStream_t stream, dtype_t dtype, isize_t n, void* P, const void* dP, const void* drate,
                               void* mP, const void* mrate);
void launch_madd_bcast(cudaStream_t stream, dtype_t dtype, const void* A, const void* b, void* dst,
                       usize_t n, usize_t m, usize_t k);
void launch_maskout(cudaStream_t stream, dtype_t dtype, const bool* M, void* A, usize_t n);
void launch_calc_zmask(cudaStream_t stream, dtype_t dtype, const void* Z, bool* M, usize_t n, usize_t m);
void launch_dropout_fp_tr(cudaStream_t stream, dtype_t dtype, const void* X, const void* rate, void* Z, bool* M,
                          usize_t n, usize_t m, usize_t k, bool matchrows);
void launch_dropout_fp_te(cudaStream_t stream, dtype_t dtype, const void* X, const void* rate, void* Z,
                          usize_t n, usize_t m, usize_t k);
void launch_dropout_bp_tr(cudaStream_t stream, dtype_t dtype, const void* dZ, const bool* M, void* dX, usize_t n);
void launch_dropout_bp_te(cudaStream_t stream, dtype_t dtype, const void* dZ, const void* rate, void* dX,
                          usize_t n, usize_t m, usize_t k);
void launch_blockwise_dot(cudaStream_t stream, dtype_t dtype, int nblock, int n, int m, int k, bool broadcast_x,
                          const void* X, const void* W, void* Z);
void launch_blockwise_dot_nt(cudaStream_t stream, dtype_t dtype, int nblock, int n, int m, int k,
                             const void* dZ, const void* W, void* dX);
void launch_blockwise_dot_tn(cudaStream_t stream, dtype_t dtype, int nblock, int n, int m, int k, bool broadcast_x,
                             const void* X, const void* dZ, void* dW);
void launch_blockwise_dot_combined(cudaStream_t stream, dtype_t dtype, int nblock, int Xoffset, bool Xbroadcast,
                                   int n, int m, int k, int p, const void* X, const void* W, void* Z);
void launch_blockwise_dot_nt_combined(cudaStream_t stream, dtype_t dtype, int nblock, int Xoffset,
                                      int n, int m, int k, int p, void* dX, const void* W, const void* dZ);
void launch_blockwise_dot_tn_combined(cudaStream_t stream, dtype_t dtype, int nblock, int Xoffset, bool Xbroadcast,
                                      int n, int m, int k, int p, const void* X, void* dW, const void* dZ);

// cuRAND states: one per possible resident thread of the largest element-wise launch,
// same seed, sequence number = global thread index (smat_cuda/rand.cu:129-135,
// smat_cuda/cuda_context.cpp:236-240).
__global__ void shim_curand_init(curandState* state, int seed, unsigned n)
{
	unsigned id = blockDim.x*blockIdx.x + threadIdx.x;
	if (id < n) curand_init(seed, id, 0, &state[id]);
}

// The uniforms the next launch of `count` elements would draw, element by element,
// without advancing the stored states: thread tid of the launch takes elements
// tid, tid + threads, ... as every reference dropout kernel does.
__global__ void shim_peek_uniforms(const curandState* state, float* U, unsigned count)
{
	unsigned tid = blockDim.x*blockIdx.x + threadIdx.x;
	curandState local = state[tid];
	for (unsigned i = tid; i < count; i += blockDim.x*gridDim.x)
		U[i] = curand_uniform(&local);
}

SM_NAMESPACE_BEGIN
static cudaDeviceProp  g_prop;
static bool            g_have_prop = false;
static cublasHandle_t  g_cublas = 0;
static curandState*    g_states = 0;
static cuda_context    g_ctx;
static ref_heap        g_heap;

cuda_context& thread_cudactx() { return g_ctx; }
cudaStream_t  cuda_context::stream() const { return 0; }
const cudaDeviceProp& cuda_context::deviceprop() const
{
	if (!g_have_prop) {
		int dev = 0; cudaGetDevice(&dev);
		cudaGetDeviceProperties(&g_prop, dev);
		g_have_prop = true;
	}
	return g_prop;
}
cublasHandle_t cuda_context::cublas() const
{
	if (!g_cublas && cublasCreate(&g_cublas) != CUBLAS_STATUS_SUCCESS)
		throw std::runtime_error("cublasCreate failed");
	return g_cublas;
}
static void seed_states(int seed)
{
	const cudaDeviceProp& p = g_ctx.deviceprop();
	unsigned n = 4*8*p.multiProcessorCount*256;           // the largest grid x block of make_elemwise_launchcfg
	if (!g_states && cudaMalloc(&g_states, (size_t)n*sizeof(curandState)) != cudaSuccess)
		throw std::runtime_error("cudaMalloc of the cuRAND states failed");
	shim_curand_init<<<(n + 255)/256, 256>>>(g_states, seed, n);
}
curandState* cuda_context::curand_state() const
{
	if (!g_states) seed_states(0);
	return g_states;
}
ref_heap& cuda_context::heap() { return g_heap; }
heap_alloc ref_heap::alloc(size_t size)
{
	heap_alloc a; a.addr = 0; a.size = size;
	if (cudaMalloc(&a.addr, size) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
	return a;
}
void ref_heap::free(heap_alloc& a)
{
	cudaDeviceSynchronize();                               // the batched product may still read the pointer table
	cudaFree(a.addr); a.addr = 0; a.size = 0;
}
int dtype_size(dtype_t dt)
{
	switch (dt) {
	case b8: case i8: case u8: return 1;
	case i16: case u16: return 2;
	case i32: case u32: case f32: return 4;
	default: return 8;
	}
}
const char* get_cublas_err_str(cublasStatus_t s) { static char buf[32]; snprintf(buf, sizeof buf, "status %d", (int)s); return buf; }
std::string format(const char* fmt, ...)
{
	char buf[1024]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
	return std::string(buf);
}
void assert_failed_print(const char* fmt, ...)
{
	va_list ap; va_start(ap, fmt); vfprintf(stderr, fmt, ap); va_end(ap); fputc('\n', stderr);
}
void assert_failed(const char* fmt, ...)
{
	char buf[512]; va_list ap; va_start(ap, fmt); vsnprintf(buf, sizeof buf, fmt, ap); va_end(ap);
	throw std::runtime_error(buf);
}
const char* dtype2str(dtype_t dt)
{
	static const char* names[] = {"b8", "i8", "u8", "i16", "u16", "i32", "u32", "i64", "u64", "f32", "f64"};
	return (unsigned)dt < 11u ? names[dt] : "?";
}
unsigned lcm(unsigned a, unsigned b)
{
	unsigned x = a, y = b;
	while (y) { unsigned t = x % y; x = y; y = t; }
	return a / x * b;
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

// ---- rows pinned beyond the scan and pooling kernels ----------------------------------
#define REF_API extern "C" __attribute__((visibility("default")))

// corr1ord_bprop.cu:166-220: the reference computes the input gradient on the host.
REF_API int ref_corr1ord_bprop_X(int dtype, void* dX, unsigned n, const void* W, unsigned m, unsigned nf, const void* dZ)
{ REF_TRY launch_corr1ord_bprop_X(0, (dtype_t)dtype, dX, n, 4, W, m, nf, dZ); REF_CATCH }

REF_API int ref_gradstep(int dtype, int n, void* P, const void* dP, const void* drate, void* mP, const void* mrate)
{ REF_TRY launch_gradstep(0, (dtype_t)dtype, n, P, dP, drate, mP, mrate); REF_CATCH }
REF_API int ref_gradstep_nesterov1(int dtype, int n, void* P, const void* mP, const void* mrate)
{ REF_TRY launch_gradstep_nesterov1(0, (dtype_t)dtype, n, P, mP, mrate); REF_CATCH }
REF_API int ref_gradstep_nesterov2(int dtype, int n, void* P, const void* dP, const void* drate, void* mP, const void* mrate)
{ REF_TRY launch_gradstep_nesterov2(0, (dtype_t)dtype, n, P, dP, drate, mP, mrate); REF_CATCH }
REF_API int ref_madd_bcast(int dtype, const void* A, const void* b, void* dst, unsigned n, unsigned m, unsigned k)
{ REF_TRY launch_madd_bcast(0, (dtype_t)dtype, A, b, dst, n, m, k); REF_CATCH }
REF_API int ref_maskout(int dtype, const void* M, void* A, unsigned n)
{ REF_TRY launch_maskout(0, (dtype_t)dtype, (const bool*)M, A, n); REF_CATCH }
REF_API int ref_calc_zmask(int dtype, const void* Z, void* M, unsigned nrow, unsigned ncol)
{ REF_TRY launch_calc_zmask(0, (dtype_t)dtype, Z, (bool*)M, nrow, ncol); REF_CATCH }

// Dropout.  ref_seed() re-seeds the cuRAND states; ref_peek_uniforms() writes the
// numbers the next dropout launch over `count` elements (count = n, or n/2 with
// matched rows) is going to draw, so that a test can hand the same numbers to the
// kernels under test.
REF_API int ref_seed(int seed)
{ REF_TRY sm::seed_states(seed); REF_CATCH }
REF_API int ref_peek_uniforms(float* U, unsigned count)
{
	REF_TRY
	launchcfg cfg = make_elemwise_launchcfg(count);
	shim_peek_uniforms<<<cfg.gdim, cfg.bdim>>>(thread_cudactx().curand_state(), U, count);
	REF_CATCH
}
REF_API int ref_dropout_fp_tr(int dtype, const void* X, const void* rate, void* Z, void* M,
                              unsigned n, unsigned m, unsigned k, int matchrows)
{ REF_TRY launch_dropout_fp_tr(0, (dtype_t)dtype, X, rate, Z, (bool*)M, n, m, k, matchrows != 0); REF_CATCH }
REF_API int ref_dropout_fp_te(int dtype, const void* X, const void* rate, void* Z, unsigned n, unsigned m, unsigned k)
{ REF_TRY launch_dropout_fp_te(0, (dtype_t)dtype, X, rate, Z, n, m, k); REF_CATCH }
REF_API int ref_dropout_bp_tr(int dtype, const void* dZ, const void* M, void* dX, unsigned n)
{ REF_TRY launch_dropout_bp_tr(0, (dtype_t)dtype, dZ, (const bool*)M, dX, n); REF_CATCH }
REF_API int ref_dropout_bp_te(int dtype, const void* dZ, const void* rate, void* dX, unsigned n, unsigned m, unsigned k)
{ REF_TRY launch_dropout_bp_te(0, (dtype_t)dtype, dZ, rate, dX, n, m, k); REF_CATCH }
REF_API int ref_dropoutord_fp_tr(const uint8_t* X, uint8_t* Z, void* M, unsigned n, float rate)
{ REF_TRY launch_dropoutord_fp_tr(0, X, Z, (bool*)M, n, rate); REF_CATCH }

// Block-diagonal dense products (cuBLAS batched GEMM inside the reference code).
REF_API int ref_blockwise_dot(int dtype, int nblock, int n, int m, int k, int bcast, const void* X, const void* W, void* Z)
{ REF_TRY launch_blockwise_dot(0, (dtype_t)dtype, nblock, n, m, k, bcast != 0, X, W, Z); REF_CATCH }
REF_API int ref_blockwise_dot_nt(int dtype, int nblock, int n, int m, int k, const void* dZ, const void* W, void* dX)
{ REF_TRY launch_blockwise_dot_nt(0, (dtype_t)dtype, nblock, n, m, k, dZ, W, dX); REF_CATCH }
REF_API int ref_blockwise_dot_tn(int dtype, int nblock, int n, int m, int k, int bcast, const void* X, const void* dZ, void* dW)
{ REF_TRY launch_blockwise_dot_tn(0, (dtype_t)dtype, nblock, n, m, k, bcast != 0, X, dZ, dW); REF_CATCH }
REF_API int ref_blockwise_dot_combined(int dtype, int nblock, int Xoffset, int bcast, int n, int m, int k, int p,
                                       const void* X, const void* W, void* Z)
{ REF_TRY launch_blockwise_dot_combined(0, (dtype_t)dtype, nblock, Xoffset, bcast != 0, n, m, k, p, X, W, Z); REF_CATCH }
REF_API int ref_blockwise_dot_nt_combined(int dtype, int nblock, int Xoffset, int n, int m, int k, int p,
                                          void* dX, const void* W, const void* dZ)
{ REF_TRY launch_blockwise_dot_nt_combined(0, (dtype_t)dtype, nblock, Xoffset, n, m, k, p, dX, W, dZ); REF_CATCH }
REF_API int ref_blockwise_dot_tn_combined(int dtype, int nblock, int Xoffset, int bcast, int n, int m, int k, int p,
                                          const void* X, void* dW, const void* dZ)
{ REF_TRY launch_blockwise_dot_tn_combined(0, (dtype_t)dtype, nblock, Xoffset, bcast != 0, n, m, k, p, X, dW, dZ); REF_CATCH }

// ---- smat's element-wise kernels: what the reference's bias, rectify, logistic and loss nodes
// run on (deepity/std/elemwise.py:71-82,162-180, softmax.py:50-61, loss.py:125-155).
SM_NAMESPACE_BEGIN
void execute_elemwise2(opcode_t opcode, const argument& a, const argument& b);
void execute_elemwise3(opcode_t opcode, const argument& a, const argument& b, const argument& c);
SM_NAMESPACE_END

// Opcode of a built-in element-wise instruction by name (smat/vm/instruction_db.h:56-125), -1 if unknown.
REF_API int ref_opcode(const char* name)
{
	static const struct { const char* n; int oc; } tab[] = {
		{"add", oc_add}, {"sub", oc_sub}, {"mul", oc_mul}, {"div", oc_div}, {"maxe", oc_maxe}, {"mine", oc_mine},
		{"exp", oc_exp}, {"log", oc_log}, {"sigm", oc_sigm}, {"sign", oc_sign}, {"sqr", oc_sqr}, {"neg", oc_neg}, {"abs", oc_abs},
	};
	for (const auto& t : tab) if (!strcmp(t.n, name)) return t.oc;
	return -1;
}

// b = f(a), arrays [nrow, ncol]
REF_API int ref_elemwise2(int opcode, int dtype, const void* a, void* b, unsigned nrow, unsigned ncol)
{
	REF_TRY
	execute_elemwise2((opcode_t)opcode, darray((size_t)a, (dtype_t)dtype, shape_t(ncol, nrow)), darray((size_t)b, (dtype_t)dtype, shape_t(ncol, nrow)));
	REF_CATCH
}

// c = f(a, b) with smat's broadcasting: a and b are arrays [arow, acol], [brow, bcol] (a row
// vector, a column vector or a 1 x 1 array broadcast against the other), or, with a NULL
// pointer, the f32 constant given beside it; c has the broadcast shape.
REF_API int ref_elemwise3(int opcode, int dtype, const void* a, float aconst, unsigned arow, unsigned acol,
                          const void* b, float bconst, unsigned brow, unsigned bcol, void* c)
{
	REF_TRY
	const unsigned crow = arow > brow ? arow : brow, ccol = acol > bcol ? acol : bcol;
	argument A = a ? darray((size_t)a, (dtype_t)dtype, shape_t(acol, arow)) : carray(aconst);
	argument B = b ? darray((size_t)b, (dtype_t)dtype, shape_t(bcol, brow)) : carray(bconst);
	execute_elemwise3((opcode_t)opcode, A, B, darray((size_t)c, (dtype_t)dtype, shape_t(ccol, crow)));
	REF_CATCH
}
