// Error channel, stream binding and array handles of libdeepbind_b200.so.
// Mirrors the handful of smat core entry points the DeepBind Python layer
// needs around the hot path (code/libs/smat/src/smat/smat.cpp:612-660);
// the generic lazy-VM matrix library behind them is not reproduced.
#include "db_common.cuh"
#include <vector>

namespace db {

state_t& state()
{
	static thread_local state_t s;   // one context per host thread (smat/vm/context.cpp:71)
	return s;
}

std::string format(const char* fmt, ...)
{
	char buf[1024];
	va_list ap;
	va_start(ap, fmt);
	vsnprintf(buf, sizeof(buf), fmt, ap);
	va_end(ap);
	return std::string(buf);
}

void ensure_device()
{
	state_t& s = state();
	if (s.device >= 0)
		return;
	int count = 0;
	cudaError_t e = cudaGetDeviceCount(&count);
	if (e != cudaSuccess || count == 0)
		throw error(format("AssertionError: CUDA error: no usable CUDA device (%s); this library has no CPU path",
		                   e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e)));
	int dev = 0;
	DB_CUDA(cudaGetDevice(&dev));
	cudaDeviceProp prop;
	DB_CUDA(cudaGetDeviceProperties(&prop, dev));
	DB_REQUIRE(prop.major >= 10, "AssertionError: CUDA error: device %d is sm_%d%d; this library is built for sm_100a only",
	           dev, prop.major, prop.minor);
	s.device = dev;
	s.sm_count = prop.multiProcessorCount;
}

// Scratch for two-stage reductions.  A CUDA graph captured from a training or scoring
// step holds the address it was captured with, so a buffer that has been handed out is
// never freed: when a later call needs more, a larger buffer is allocated and the old
// one is retired, alive until the process ends (growth is by half, so the retired ones
// together stay below twice the live one).  Growing inside a stream capture is refused:
// run the step once before capturing it, or reserve with db_reserve_scratch().
void* scratch(size_t bytes)
{
	state_t& s = state();
	if (bytes > s.scratch_bytes) {
		cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
		DB_CUDA(cudaStreamIsCapturing(s.stream, &cap));
		DB_REQUIRE(cap == cudaStreamCaptureStatusNone,
		           "RuntimeError: %zu bytes of scratch needed while the stream is being captured (have %zu); run the step once "
		           "before capturing it, or call db_reserve_scratch first", bytes, s.scratch_bytes);
		size_t want = bytes < (1u << 20) ? (1u << 20) : bytes + bytes / 2;
		void* fresh = nullptr;
		cudaError_t e = cudaMalloc(&fresh, want);
		if (e != cudaSuccess)
			throw error(format("MemoryError: cudaMalloc of %zu bytes of scratch failed: %s", want, cudaGetErrorString(e)));
		if (s.scratch)
			s.retired_scratch.push_back(s.scratch);
		s.scratch = fresh;
		s.scratch_bytes = want;
	}
	return s.scratch;
}

static smat* new_array(const db_shape* shape, int dtype, bool zero)
{
	DB_REQUIRE(shape != nullptr, "ValueError: shape must not be NULL");
	DB_REQUIRE(shape->x >= 0 && shape->y >= 0, "ValueError: negative shape (%d,%d)", shape->y, shape->x);
	size_t bytes = (size_t)shape->x * (size_t)shape->y * dtype_size(dtype);
	smat* A = new smat();
	A->vtype = DB_VT_DARRAY; A->dtype = dtype;
	A->shape = { shape->x, shape->y, 1 };
	A->strides = { 1, shape->x, 0 };
	A->data = nullptr; A->owns_data = 1; A->device = state().device;
	if (bytes) {
		cudaError_t e = cudaMalloc(&A->data, bytes);
		if (e != cudaSuccess) {
			delete A;
			throw error(format("MemoryError: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e)));
		}
		if (zero)
			DB_CUDA(cudaMemsetAsync(A->data, 0, bytes, state().stream));
	}
	return A;
}

}  // namespace db

using namespace db;

DB_EXPORT const char* api_get_last_error(void)
{
	return state().last_error.empty() ? nullptr : state().last_error.c_str();
}

DB_EXPORT void api_clear_last_error(void) { state().last_error.clear(); }

DB_EXPORT void api_sync(void)
{
	DB_API_TRY
	DB_CUDA(cudaStreamSynchronize(state().stream));
	DB_API_CATCH
}

DB_EXPORT void api_set_stream(void* cuda_stream)
{
	DB_API_TRY_NODEV
	state().stream = (cudaStream_t)cuda_stream;
	DB_API_CATCH
}

DB_EXPORT void* api_get_stream(void) { return (void*)state().stream; }

DB_EXPORT int api_device_count(void)
{
	int count = 0;
	if (cudaGetDeviceCount(&count) != cudaSuccess) { cudaGetLastError(); return 0; }
	return count;
}

DB_EXPORT void api_set_device(int device)
{
	DB_API_TRY_NODEV
	// As in the reference, the device is fixed once the context has been used
	// (code/libs/smat/src/smat_cuda/cuda_context.cpp:171-175).
	DB_REQUIRE(state().device < 0 || state().device == device,
	           "RuntimeError: device already bound to %d for this thread", state().device);
	DB_CUDA(cudaSetDevice(device));
	ensure_device();
	DB_API_CATCH
}

DB_EXPORT uint64_t api_launch_count(void) { return state().launches; }

DB_EXPORT void db_reserve_scratch(size_t bytes)
{
	DB_API_TRY
	scratch(bytes);
	DB_API_CATCH
}

DB_EXPORT size_t db_scratch_bytes(void) { return state().scratch_bytes; }

DB_EXPORT void api_set_seed(uint64_t seed)
{
	state().seed = seed;
	state().rng_calls = 0;
}

DB_EXPORT smat* api_empty(const db_shape* shape, int dtype)
{
	DB_API_TRY
	return new_array(shape, dtype, false);
	DB_API_CATCH_RETURN(nullptr)
}

DB_EXPORT smat* api_zeros(const db_shape* shape, int dtype)
{
	DB_API_TRY
	return new_array(shape, dtype, true);
	DB_API_CATCH_RETURN(nullptr)
}

DB_EXPORT smat* api_wrap(void* device_ptr, int rows, int cols, int dtype)
{
	DB_API_TRY
	DB_REQUIRE(rows >= 0 && cols >= 0, "ValueError: negative shape (%d,%d)", rows, cols);
	dtype_size(dtype);
	smat* A = new smat();
	A->vtype = DB_VT_DARRAY; A->dtype = dtype;
	A->shape = { cols, rows, 1 };
	A->strides = { 1, cols, 0 };
	A->data = device_ptr; A->owns_data = 0; A->device = state().device;
	return A;
	DB_API_CATCH_RETURN(nullptr)
}

DB_EXPORT void api_delete(const smat* M)
{
	DB_API_TRY_NODEV
	if (!M) return;
	if (M->owns_data && M->data) {
		// Work queued on the stream may still read the buffer.
		DB_CUDA(cudaStreamSynchronize(state().stream));
		DB_CUDA(cudaFree(M->data));
	}
	delete M;
	DB_API_CATCH
}

DB_EXPORT int32_t api_nrow(const smat* M) { return M ? M->shape.y : 0; }
DB_EXPORT int32_t api_ncol(const smat* M) { return M ? M->shape.x : 0; }
DB_EXPORT size_t  api_size(const smat* M) { return M ? size_of(M) : 0; }
DB_EXPORT int     api_dtype(const smat* M) { return M ? M->dtype : DB_F32; }
DB_EXPORT void*   api_data(const smat* M) { return M ? M->data : nullptr; }

// Host strides are given in bytes, as smat.cpp:659-660 takes them.
DB_EXPORT void api_copy_from(smat* M, const void* host_src, int32_t row_stride_bytes, int32_t col_stride_bytes)
{
	DB_API_TRY
	require_array(M, "M");
	size_t es = dtype_size(M->dtype);
	DB_REQUIRE(col_stride_bytes == (int32_t)es || M->shape.x <= 1, "ValueError: host array must have unit column stride");
	if (size_of(M) == 0) return;
	DB_CUDA(cudaMemcpy2DAsync(M->data, (size_t)M->strides.y * es, host_src, (size_t)row_stride_bytes,
	                          (size_t)M->shape.x * es, (size_t)M->shape.y, cudaMemcpyHostToDevice, state().stream));
	DB_CUDA(cudaStreamSynchronize(state().stream));
	DB_API_CATCH
}

DB_EXPORT void api_copy_to(const smat* M, void* host_dst, int32_t row_stride_bytes, int32_t col_stride_bytes)
{
	DB_API_TRY
	require_array(M, "M");
	size_t es = dtype_size(M->dtype);
	DB_REQUIRE(col_stride_bytes == (int32_t)es || M->shape.x <= 1, "ValueError: host array must have unit column stride");
	if (size_of(M) == 0) return;
	DB_CUDA(cudaMemcpy2DAsync(host_dst, (size_t)row_stride_bytes, M->data, (size_t)M->strides.y * es,
	                          (size_t)M->shape.x * es, (size_t)M->shape.y, cudaMemcpyDeviceToHost, state().stream));
	DB_CUDA(cudaStreamSynchronize(state().stream));
	DB_API_CATCH
}

DB_EXPORT void api_fill_zero(smat* M)
{
	DB_API_TRY
	require_array(M, "M");
	if (size_of(M))
		DB_CUDA(cudaMemsetAsync(M->data, 0, size_of(M) * dtype_size(M->dtype), state().stream));
	DB_API_CATCH
}

// The reference's loader calls register_ext() to enter the extension's
// instructions into smat's VM tables (kangaroo_smat.cpp:420-488).  This library
// dispatches api_* directly, so there is nothing to register.
DB_EXPORT void register_ext(void) {}

// The reference's autotuner times variants of a kernel the Python layer never
// calls (autotune.cu:91-113); kept as a callable no-op.
DB_EXPORT void api_autotune(void) {}
