// Shared host-side plumbing for libdeepbind_b200.so: error channel, stream,
// argument checks and launch sizing.  Exceptions never cross the C boundary:
// every exported function wraps its body in DB_API_TRY / DB_API_CATCH, which
// stores the message for api_get_last_error() the way the reference's
// SM_API_TRY / SM_API_CATCH do (code/libs/smat/src/smat/config.h:95-105).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../include/deepbind_b200.h"

#define DB_EXPORT extern "C" __attribute__((visibility("default")))

namespace db {

struct state_t {
	std::string  last_error;
	cudaStream_t stream = 0;
	int          device = -1;       // -1: not yet bound
	int          sm_count = 0;
	uint64_t     seed = 0x5eedULL;
	uint64_t     rng_calls = 0;     // advances per random-mask call
	void*        scratch = nullptr; // grow-only device scratch for two-stage reductions
	size_t       scratch_bytes = 0;
	std::vector<void*> retired_scratch; // outgrown scratch buffers, kept: captured graphs may still use them
	uint64_t     launches = 0;      // kernels launched by this library on this thread
};
state_t& state();

std::string format(const char* fmt, ...);

struct error : std::runtime_error {
	explicit error(const std::string& s) : std::runtime_error(s) {}
};

// Binds the calling thread's device on first use and caches its SM count.
void ensure_device();
void* scratch(size_t bytes);   // stream-ordered use only; grows with cudaMalloc, never frees (see db_api.cu)
// FP32 motif scan writing Z [n, nf] (scanpool_f32.cu); n = rows written, X holds n + m - 1 bytes
void launch_corr1ord_f32(const float* W, unsigned m, unsigned nf, const uint8_t* X, unsigned n, float* Z);
// FP32 filter gradient of the scan from dZ [n, nf], accumulated into dW (scanpool_f32.cu)
void launch_corr1ord_bprop_W_f32(float* dW, unsigned m, unsigned nf, const uint8_t* X, unsigned n, const float* dZ);

inline void cuda_check(cudaError_t e, const char* what, const char* file, int line)
{
	if (e != cudaSuccess)
		throw error(format("AssertionError: CUDA error in %s (%s:%d): %s", what, file, line, cudaGetErrorString(e)));
}

}  // namespace db

#define DB_CUDA(call) ::db::cuda_check((call), #call, __FILE__, __LINE__)
#define DB_LAUNCH_CHECK() do { ++::db::state().launches; ::db::cuda_check(cudaGetLastError(), "kernel launch", __FILE__, __LINE__); } while (0)
#define DB_REQUIRE(cond, ...) do { if (!(cond)) throw ::db::error(::db::format(__VA_ARGS__)); } while (0)
#define DB_ASSERT(cond) DB_REQUIRE(cond, "AssertionError: ASSERT FAILED: %s", #cond)

#define DB_API_TRY   try { ::db::ensure_device();
#define DB_API_TRY_NODEV try {
#define DB_API_CATCH } catch (const std::exception& e) { ::db::state().last_error = e.what(); return; }
#define DB_API_CATCH_RETURN(v) } catch (const std::exception& e) { ::db::state().last_error = e.what(); return v; }

namespace db {

inline size_t dtype_size(int dt)
{
	switch (dt) {
	case DB_B8: case DB_I8: case DB_U8: return 1;
	case DB_I16: case DB_U16: return 2;
	case DB_I32: case DB_U32: case DB_F32: return 4;
	case DB_I64: case DB_U64: case DB_F64: return 8;
	}
	throw error(format("TypeError: unknown dtype code %d", dt));
}

inline bool is_float(int dt) { return dt == DB_F32 || dt == DB_F64; }
inline size_t size_of(const smat* A) { return (size_t)A->shape.x * (size_t)A->shape.y; }

// The reference rejects non-contiguous arguments for extension instructions
// (code/libs/smat/src/smat/vm/machine.cpp:207-222).
inline void require_array(const smat* A, const char* name)
{
	DB_REQUIRE(A != nullptr, "ValueError: argument %s must not be NULL", name);
	DB_REQUIRE(A->vtype == DB_VT_DARRAY, "TypeError: argument %s is not a device array", name);
	DB_REQUIRE(A->shape.x == 0 || A->shape.y <= 1 || A->strides.y == A->shape.x,
	           "ValueError: argument %s must be contiguous (row stride %d, %d columns)", name, A->strides.y, A->shape.x);
	DB_REQUIRE(size_of(A) == 0 || A->data != nullptr, "ValueError: argument %s has no device memory", name);
}
inline void require_float(const smat* A, const char* name)
{
	require_array(A, name);
	DB_REQUIRE(is_float(A->dtype), "TypeError: argument %s must be f32 or f64", name);
}
inline void require_dtype(const smat* A, int dt, const char* name, const char* dtname)
{
	require_array(A, name);
	DB_REQUIRE(A->dtype == dt, "TypeError: argument %s must have dtype %s", name, dtname);
}

// Grid for grid-stride elementwise kernels: enough CTAs of 256 threads to fill
// every SM eight deep, never more than the work needs.
inline unsigned elemwise_grid(size_t n, unsigned block = 256)
{
	size_t want = (n + block - 1) / block;
	size_t cap  = (size_t)state().sm_count * 8;
	if (want < 1) want = 1;
	return (unsigned)(want < cap ? want : cap);
}

template <typename T> inline T divup(T a, T b) { return (a + b - 1) / b; }

}  // namespace db
