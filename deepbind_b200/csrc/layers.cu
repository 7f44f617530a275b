// Layer arithmetic that the reference evaluates through generic smat array
// expressions, one launch and one HBM round trip per operator
// (code/libs/deepity/deepity/std/elemwise.py:71-82,162-180, softmax.py:50-77,
// loss.py:52-155).  Plain-pointer f32 entry points; reductions use a fixed
// order so that repeated runs agree bit for bit (the reference's reduce_y is
// also free of atomics, smat_cuda/reduce_y.cuh:52-126).
#include "db_common.cuh"
#include "db_rng.cuh"
#include <mutex>

namespace db {

#define GRID_STRIDE(i, n) for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n); i += (size_t)gridDim.x * blockDim.x)

__global__ void bias_add_kernel(float* Z, const float* X, const float* b, size_t n, unsigned ncol)
{
	GRID_STRIDE(i, n) Z[i] = X[i] + b[i % ncol];
}

__global__ void relu_kernel(float* Z, const float* X, size_t n)
{
	GRID_STRIDE(i, n) Z[i] = fmaxf(0.0f, X[i]);
}

// dZ * sign(Z) with Z the rectified output, so the factor is 0 or 1 (elemwise.py:78).
__global__ void l1_decay_kernel(float* __restrict__ dP, const float* __restrict__ P, const float* __restrict__ decay, size_t n)
{
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
		const float p = P[i];
		const float s = p > 0.f ? 1.f : (p < 0.f ? -1.f : 0.f);
		dP[i] = dP[i] + decay[i] * s;          // the product is exact (s is -1, 0 or 1): one rounding, fused or not
	}
}

__global__ void relu_bprop_kernel(float* dX, const float* dZ, const float* Z, size_t n)
{
	GRID_STRIDE(i, n) { float z = Z[i]; dX[i] = dZ[i] * (z > 0.0f ? 1.0f : (z < 0.0f ? -1.0f : 0.0f)); }
}

__global__ void logistic_kernel(float* Z, const float* X, size_t n)
{
	GRID_STRIDE(i, n) Z[i] = 1.0f / (1.0f + expf(-X[i]));
}

// Column sums, stage 1: a CTA owns 256 rows x 32 columns; 8 row slices are
// summed by 8 thread groups and combined in slice order.
__global__ void __launch_bounds__(256)
colsum_stage1(const float* __restrict__ A, unsigned nrow, unsigned ncol, float* __restrict__ partial)
{
	__shared__ float part[8][32];
	const unsigned c = blockIdx.y * 32 + threadIdx.x % 32, slice = threadIdx.x / 32;
	const unsigned r0 = blockIdx.x * 256, r1 = min(nrow, r0 + 256);
	float s = 0.0f;
	if (c < ncol)
		for (unsigned r = r0 + slice; r < r1; r += 8) s += A[(size_t)r * ncol + c];
	part[slice][threadIdx.x % 32] = s;
	__syncthreads();
	if (slice == 0 && c < ncol) {
		float t = part[0][threadIdx.x];
		for (int k = 1; k < 8; ++k) t += part[k][threadIdx.x];
		partial[(size_t)blockIdx.x * ncol + c] = t;
	}
}

__global__ void colsum_stage2(float* __restrict__ out, const float* __restrict__ partial, unsigned ncol, unsigned nparts)
{
	unsigned c = blockIdx.x * blockDim.x + threadIdx.x;
	if (c >= ncol) return;
	float s = 0.0f;
	for (unsigned p = 0; p < nparts; ++p) s += partial[(size_t)p * ncol + c];
	out[c] = s;
}

// One CTA per output column: masked loss mean and dZ = maskout(Z-Y)/nrow.
__global__ void __launch_bounds__(256)
loss_kernel(int kind, const float* __restrict__ Z, const float* __restrict__ Y, const uint8_t* __restrict__ Ymask,
            const uint8_t* __restrict__ Zmask, unsigned nrow, unsigned ncol, float* __restrict__ loss_out, float* __restrict__ dZ)
{
	__shared__ float red[256];
	const unsigned c = blockIdx.x;
	const float inv = 1.0f / (float)nrow;
	float s = 0.0f;
	for (unsigned r = threadIdx.x; r < nrow; r += blockDim.x) {
		size_t i = (size_t)r * ncol + c;
		float z = Z[i], y = Y[i];
		bool keep = (!Ymask || Ymask[i]) && (!Zmask || Zmask[i]);
		float l;
		if (kind == 0) { float d = z - y; l = d * d; }
		else l = logf(fmaxf(1e-15f, z)) * y + logf(fmaxf(1e-15f, 1.0f - z)) * (1.0f - y);
		if (keep) s += l;
		if (dZ) dZ[i] = keep ? (z - y) * inv : 0.0f;
	}
	red[threadIdx.x] = s;
	__syncthreads();
	for (unsigned w = 128; w > 0; w >>= 1) {
		if (threadIdx.x < w) red[threadIdx.x] += red[threadIdx.x + w];
		__syncthreads();
	}
	if (threadIdx.x == 0 && loss_out)
		loss_out[c] = (kind == 0 ? 0.5f : -1.0f) * (red[0] * inv);
}

}  // namespace db

using namespace db;

DB_EXPORT void db_bias_add(float* Z, const float* X, const float* b, uint32_t nrow, uint32_t ncol)
{
	DB_API_TRY
	size_t n = (size_t)nrow * ncol;
	if (!n) return;
	DB_REQUIRE(Z && X && b, "ValueError: db_bias_add got a NULL pointer");
	bias_add_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(Z, X, b, n, ncol);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_relu(float* Z, const float* X, size_t n)
{
	DB_API_TRY
	if (!n) return;
	DB_REQUIRE(Z && X, "ValueError: db_relu got a NULL pointer");
	relu_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(Z, X, n);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_relu_bprop(float* dX, const float* dZ, const float* Z, size_t n)
{
	DB_API_TRY
	if (!n) return;
	DB_REQUIRE(dX && dZ && Z, "ValueError: db_relu_bprop got a NULL pointer");
	relu_bprop_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(dX, dZ, Z, n);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// L1 weight decay of the reference's trainable layers (corr1ord.py:112-126,
// full.py:102-119): dW += decay * sign(W), with the per-model decay already spread
// over the flat parameter vector (zero on biases), as the rates are.
DB_EXPORT void db_l1_decay(float* dP, const float* P, const float* decay, size_t n)
{
	DB_API_TRY
	if (!n) return;
	DB_REQUIRE(dP && P && decay, "ValueError: db_l1_decay got a NULL pointer");
	l1_decay_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(dP, P, decay, n);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_logistic(float* Z, const float* X, size_t n)
{
	DB_API_TRY
	if (!n) return;
	DB_REQUIRE(Z && X, "ValueError: db_logistic got a NULL pointer");
	logistic_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(Z, X, n);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// Standard normal draws on the device (the reference initialises parameters with
// smat's randn, cuRAND normals: smat_cuda/rand.cu:66-88, then scales them per model
// with madd_bcast: sgd.py:331-340).  Counter-based: element i of call c is the
// Box-Muller transform of two Philox uniforms keyed by (seed, c, i), so a given seed
// gives the same parameters whatever the launch shape.  Streams of different
// generators cannot agree with cuRAND's; what is kept is the distribution.
__global__ void randn_kernel(float* __restrict__ out, size_t n, uint64_t seed, uint64_t call)
{
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
		const float u1 = uniform_01(seed, 2 * call, i), u2 = uniform_01(seed, 2 * call + 1, i);
		out[i] = sqrtf(-2.f * logf(u1)) * cospif(2.f * u2);
	}
}

DB_EXPORT void db_randn(float* out, size_t n)
{
	DB_API_TRY
	if (!n) return;
	DB_REQUIRE(out, "ValueError: db_randn got a NULL pointer");
	randn_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(out, n, state().seed ^ 0x9e3779b97f4a7c15ull, state().rng_calls++);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// Strand choice of kangaroo.predict (predict.py:145-164): rows come in forward /
// reverse-complement pairs; the larger score of each pair is kept, the forward one on ties.
__global__ void strand_max_kernel(float* __restrict__ out, const float* __restrict__ Z, size_t npair, unsigned ncol)
{
	const size_t n = npair * ncol;
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
		const size_t p = i / ncol, c = i - p * ncol;
		const float f = Z[(2 * p) * ncol + c], r = Z[(2 * p + 1) * ncol + c];
		out[i] = f >= r ? f : r;
	}
}

DB_EXPORT void db_strand_max(float* out, const float* Z, uint32_t npair, uint32_t ncol)
{
	DB_API_TRY
	const size_t n = (size_t)npair * ncol;
	if (!n) return;
	DB_REQUIRE(out && Z, "ValueError: db_strand_max got a NULL pointer");
	strand_max_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(out, Z, npair, ncol);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_colsum(float* out, const float* A, uint32_t nrow, uint32_t ncol)
{
	DB_API_TRY
	if (!ncol) return;
	DB_REQUIRE(out && (A || !nrow), "ValueError: db_colsum got a NULL pointer");
	if (!nrow) { DB_CUDA(cudaMemsetAsync(out, 0, (size_t)ncol * 4, state().stream)); return; }
	unsigned parts = divup(nrow, 256u);
	float* partial = (float*)scratch((size_t)parts * ncol * sizeof(float));
	colsum_stage1<<<dim3(parts, divup(ncol, 32u)), 256, 0, state().stream>>>(A, nrow, ncol, partial);
	DB_LAUNCH_CHECK();
	colsum_stage2<<<divup(ncol, 128u), 128, 0, state().stream>>>(out, partial, ncol, parts);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// ---------------------------------------------------------------------------
// Column sums without any allocation.  Some hosts may not create device memory
// when they call us: a process that has handed every byte of the GPU to its own
// pool, a real-time loop that must not take the allocator's locks, or code
// running where cudaMalloc is forbidden altogether.  For them the per-block
// partial sums live in a fixed array that is part of the library image itself.
// Every GPU that loads the library carries these 1 MiB until the process exits.
static constexpr unsigned COLSUM_STATIC_FLOATS = 1u << 18;           // 1 MiB of partial sums
static __device__ __align__(256) float g_colsum_static_scratch[COLSUM_STATIC_FLOATS];

// In host code the array's name is only a handle for the runtime, not an address
// a kernel may use.  The real device address is asked for once per device, with
// that device current, and cached; the cache is filled under a lock because host
// threads bound to different devices may make their first calls at the same time.
// (A cudaDeviceReset in the host process invalidates the cached address.)
static float* colsum_static_scratch_ptr()
{
	static std::mutex lock;
	static float* ptrs[64] = {nullptr};
	int dev = 0;
	DB_CUDA(cudaGetDevice(&dev));
	DB_REQUIRE(dev >= 0 && dev < 64, "RuntimeError: device index %d out of range", dev);
	std::lock_guard<std::mutex> guard(lock);
	if (!ptrs[dev]) {
		void* p = nullptr;
		cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_static_scratch);
		DB_REQUIRE(e == cudaSuccess && p != nullptr, "AssertionError: CUDA error: cudaGetSymbolAddress failed: %s",
		           cudaGetErrorString(e));
		ptrs[dev] = (float*)p;
	}
	return ptrs[dev];
}

DB_EXPORT void db_colsum_static(float* out, const float* A, uint32_t nrow, uint32_t ncol)
{
	DB_API_TRY
	if (!ncol) return;
	DB_REQUIRE(out && (A || !nrow), "ValueError: db_colsum_static got a NULL pointer");
	unsigned parts = divup(nrow, 256u);
	DB_REQUIRE((size_t)parts * ncol <= COLSUM_STATIC_FLOATS,
	           "ValueError: db_colsum_static supports ceil(nrow/256)*ncol <= %u partial sums (got %u x %u); "
	           "use db_colsum for larger inputs", COLSUM_STATIC_FLOATS, parts, ncol);
	float* partial = colsum_static_scratch_ptr();
	if (!nrow) { DB_CUDA(cudaMemsetAsync(out, 0, (size_t)ncol * 4, state().stream)); return; }
	// Stage 1 writes every partial that stage 2 reads, so what an earlier call left
	// in the array does not matter and nothing has to be cleared.
	colsum_stage1<<<dim3(parts, divup(ncol, 32u)), 256, 0, state().stream>>>(A, nrow, ncol, partial);
	DB_LAUNCH_CHECK();
	colsum_stage2<<<divup(ncol, 128u), 128, 0, state().stream>>>(out, partial, ncol, parts);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_loss(int kind, const float* Z, const float* Y, const uint8_t* Ymask, const uint8_t* Zmask,
                       uint32_t nrow, uint32_t ncol, float* loss_out, float* dZ)
{
	DB_API_TRY
	DB_REQUIRE(kind == 0 || kind == 1, "ValueError: loss kind must be 0 (mse) or 1 (nll)");
	if (!nrow || !ncol) return;
	DB_REQUIRE(Z && Y, "ValueError: db_loss got a NULL pointer");
	loss_kernel<<<ncol, 256, 0, state().stream>>>(kind, Z, Y, Ymask, Zmask, nrow, ncol, loss_out, dZ);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// Measurement aid (no counterpart in the reference): a register-only chain of FP32
// adds on every lane of the GPU, eight independent accumulators per thread, 2048
// threads per SM.  Timed by the caller with events on the library's stream, it gives
// the non-FMA FP32 issue rate that the lookup-add kernels are set against.
__global__ void __launch_bounds__(256) fadd_probe_kernel(float* sink, unsigned iters, float d)
{
	float a[8];
	#pragma unroll
	for (int k = 0; k < 8; ++k) a[k] = (float)(threadIdx.x + k);
	for (unsigned i = 0; i < iters; ++i) {
		#pragma unroll
		for (int u = 0; u < 16; ++u)
			#pragma unroll
			for (int k = 0; k < 8; ++k) a[k] = __fadd_rn(a[k], d);
	}
	float s = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
	if (s == -123.456f && sink) sink[0] = s;       // never true for d > 0: keeps the chain alive
}

DB_EXPORT uint64_t db_fadd_probe(float* sink, uint32_t iters)
{
	DB_API_TRY
	const unsigned ncta = (unsigned)state().sm_count * 8;
	fadd_probe_kernel<<<ncta, 256, 0, state().stream>>>(sink, iters, 1.0f);
	DB_LAUNCH_CHECK();
	return (uint64_t)ncta * 256 * 128 * iters;
	DB_API_CATCH_RETURN(0)
}
