// Drop-in deepity_smat entry points: momentum / Nesterov parameter updates with
// per-element rates, per-instance broadcast multiply-add, masks, feature
// dropout and the block-diagonal products that run `ninst` small dense layers
// in one call.
//
// Reference behaviour restated here (code/libs/deepity/deepity_smat/):
//   gradstep.cu:41-72       gradstep, nesterov1, nesterov2
//   madd_bcast.cu:41-47     dst[i] += A[i]*b[(i/k) % m]
//   maskout.cu:41-67        maskout, calc_zmask (strand selection mask)
//   dropout.cu:41-109       dropout forward/backward, train and test
//   blockwise_dot.cu:75-260 block-diagonal GEMMs (cuBLAS batched in the reference)
//   deepity_smat.cpp:102-468 validation and shape derivation
#include "db_common.cuh"
#include "db_rng.cuh"

namespace db {

#define GRID_STRIDE(i, n) for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n); i += (size_t)gridDim.x * blockDim.x)

template <typename T>
__global__ void gradstep_kernel(T* P, const T* dP, const T* drate, T* mP, const T* mrate, size_t n)
{
	GRID_STRIDE(i, n) {
		T delta = mP[i] * mrate[i] - dP[i] * drate[i];
		mP[i] = delta;
		P[i] += delta;
	}
}

template <typename T>
__global__ void gradstep_nesterov1_kernel(T* P, const T* mP, const T* mrate, size_t n)
{
	GRID_STRIDE(i, n) P[i] = P[i] + mrate[i] * mP[i];
}

template <typename T>
__global__ void gradstep_nesterov2_kernel(T* P, const T* dP, const T* drate, T* mP, const T* mrate, size_t n)
{
	GRID_STRIDE(i, n) {
		T delta = dP[i] * drate[i];
		mP[i] = mP[i] * mrate[i] - delta;
		P[i] -= delta;
	}
}

template <typename T>
__global__ void madd_bcast_kernel(const T* A, const T* b, T* dst, size_t n, unsigned m, unsigned k)
{
	GRID_STRIDE(i, n) dst[i] += A[i] * b[(i / k) % m];
}

template <typename T>
__global__ void maskout_kernel(const uint8_t* M, T* A, size_t n)
{
	GRID_STRIDE(i, n) if (!M[i]) A[i] = (T)0;
}

template <typename T>
__global__ void calc_zmask_kernel(const T* Z, uint8_t* M, size_t n, size_t m)
{
	GRID_STRIDE(i, (n * m) / 2) {
		size_t row = (i / m) * 2, col = i % m, index = m * row + col;
		if (Z[index] >= Z[index + m]) M[index] = 1; else M[index + m] = 1;
	}
}

template <typename T>
__global__ void dropout_fp_tr_kernel(const T* X, const T* rate, const float* U, uint64_t seed, uint64_t call,
                                     T* Z, uint8_t* M, size_t n, unsigned m, unsigned k)
{
	GRID_STRIDE(i, n) {
		T p = rate[(i / k) % m];
		float u = U ? U[i] : uniform_01(seed, call, i);
		bool mask = ((T)u >= p);
		M[i] = mask;
		Z[i] = X[i] * (T)mask;
	}
}

template <typename T>
__global__ void dropout_fp_tr_match_kernel(const T* X, const T* rate, const float* U, uint64_t seed, uint64_t call,
                                           T* Z, uint8_t* M, size_t nrow, size_t ncol, unsigned k)
{
	GRID_STRIDE(i, nrow * ncol / 2) {
		size_t row = (i / ncol) * 2, col = i % ncol;
		T p = rate[col / k];
		float u = U ? U[i] : uniform_01(seed, call, i);
		bool mask = ((T)u >= p);
		size_t i0 = row * ncol + col, i1 = i0 + ncol;
		M[i0] = mask; M[i1] = mask;
		Z[i0] = X[i0] * (T)mask; Z[i1] = X[i1] * (T)mask;
	}
}

template <typename T>
__global__ void dropout_scale_kernel(const T* X, const T* rate, T* Z, size_t n, unsigned m, unsigned k)
{
	GRID_STRIDE(i, n) { T scale = 1 - rate[(i / k) % m]; Z[i] = X[i] * scale; }
}

template <typename T>
__global__ void dropout_bp_tr_kernel(const T* dZ, const uint8_t* M, T* dX, size_t n)
{
	GRID_STRIDE(i, n) dX[i] = dZ[i] * (T)(M[i] != 0);
}

// ------------------------------------------------------- block-diagonal dots
// The matrices are tiny (k, m <= a few dozen; n = minibatch), far below what a
// tensor-core tile wants, so each block's weights are staged in shared memory
// and every thread produces outputs with a fixed k-ascending fused
// multiply-add chain: deterministic, one launch for all `nblock` models.
//
//   NN  Z[:,b]  (n x m) = beta*Z + X[:,b] (n x k) . W[b] (k x m)      grid (row tiles, nblock)
//   NT  dX[:,b] (n x k) = dZ[:,b] (n x m) . W[b]^T                    grid (row tiles, nblock)
//   TN  dW[b]   (k x m) = X[:,b]^T . dZ[:,b]   (sum over n rows)      grid (nblock)
// W has p rows per block; the k rows used start at row xoff of the block.
// ldx = k (X shared by all blocks) or k*nblock.
template <typename T>
__global__ void __launch_bounds__(256)
blockwise_nn_kernel(const T* __restrict__ X, const T* __restrict__ W, T* __restrict__ Z,
                    int n, int m, int k, int p, int xoff, int xbroadcast, int nblock, int beta_one)
{
	extern __shared__ __align__(16) unsigned char smem_raw[];
	T* w = reinterpret_cast<T*>(smem_raw);          // [k][m]
	const int b = blockIdx.y;
	const T* Wb = W + ((size_t)b * p + xoff) * m;
	for (int t = threadIdx.x; t < k * m; t += blockDim.x) w[t] = Wb[t];
	__syncthreads();
	const int ldx = k * (xbroadcast ? 1 : nblock), ldz = m * nblock;
	const T* Xb = X + (xbroadcast ? 0 : (size_t)b * k);
	T* Zb = Z + (size_t)b * m;
	const int rows_per_block = 64;
	const int r0 = blockIdx.x * rows_per_block;
	const int rows = min(rows_per_block, n - r0);
	for (int t = threadIdx.x; t < rows * m; t += blockDim.x) {
		int i = r0 + t / m, c = t % m;
		T s = beta_one ? Zb[(size_t)i * ldz + c] : (T)0;
		const T* x = Xb + (size_t)i * ldx;
		for (int u = 0; u < k; ++u) s = fma(x[u], w[u * m + c], s);
		Zb[(size_t)i * ldz + c] = s;
	}
}

template <typename T>
__global__ void __launch_bounds__(256)
blockwise_nt_kernel(T* __restrict__ dX, const T* __restrict__ W, const T* __restrict__ dZ,
                    int n, int m, int k, int p, int xoff, int nblock)
{
	extern __shared__ __align__(16) unsigned char smem_raw[];
	T* w = reinterpret_cast<T*>(smem_raw);          // [k][m+1] padded against bank conflicts
	const int b = blockIdx.y;
	const T* Wb = W + ((size_t)b * p + xoff) * m;
	for (int t = threadIdx.x; t < k * m; t += blockDim.x) w[(t / m) * (m + 1) + t % m] = Wb[t];
	__syncthreads();
	const int ldx = k * nblock, ldz = m * nblock;
	T* Xb = dX + (size_t)b * k;
	const T* Zb = dZ + (size_t)b * m;
	const int rows_per_block = 64;
	const int r0 = blockIdx.x * rows_per_block;
	const int rows = min(rows_per_block, n - r0);
	for (int t = threadIdx.x; t < rows * k; t += blockDim.x) {
		int i = r0 + t / k, u = t % k;
		const T* z = Zb + (size_t)i * ldz;
		T s = 0;
		for (int c = 0; c < m; ++c) s = fma(z[c], w[u * (m + 1) + c], s);
		Xb[(size_t)i * ldx + u] = s;
	}
}

// One CTA per block b.  The n rows are cut into blockDim/32 interleaved slices,
// each summed by one warp, then the partials are added in slice order.
template <typename T>
__global__ void __launch_bounds__(256)
blockwise_tn_kernel(const T* __restrict__ X, T* __restrict__ dW, const T* __restrict__ dZ,
                    int n, int m, int k, int p, int xoff, int xbroadcast, int nblock)
{
	extern __shared__ __align__(16) unsigned char smem_raw[];
	T* part = reinterpret_cast<T*>(smem_raw);       // [nslice][k*m]
	const int nslice = blockDim.x / 32;
	const int b = blockIdx.x;
	const int ldx = k * (xbroadcast ? 1 : nblock), ldz = m * nblock;
	const T* Xb = X + (xbroadcast ? 0 : (size_t)b * k);
	const T* Zb = dZ + (size_t)b * m;
	T* Wb = dW + ((size_t)b * p + xoff) * m;
	const int km = k * m;
	const int slice = threadIdx.x / 32, lane = threadIdx.x % 32;
	for (int o = lane; o < km; o += 32) {
		int u = o / m, c = o % m;
		T s = 0;
		for (int i = slice; i < n; i += nslice) s = fma(Xb[(size_t)i * ldx + u], Zb[(size_t)i * ldz + c], s);
		part[slice * km + o] = s;
	}
	__syncthreads();
	for (int o = threadIdx.x; o < km; o += blockDim.x) {
		T s = part[o];
		for (int sl = 1; sl < nslice; ++sl) s += part[sl * km + o];
		Wb[o] = s;
	}
}

enum { BW_NN = 0, BW_NT = 1, BW_TN = 2 };

static void launch_blockwise(int mode, int dtype, int nblock, int xoff, bool xbroadcast,
                             int n, int m, int k, int p, const void* X, const void* W, const void* Z, bool beta_one)
{
	if (n == 0 || m == 0 || k == 0 || nblock == 0) return;
	size_t es = dtype_size(dtype);
	cudaStream_t st = state().stream;
	if (mode == BW_NN) {
		size_t smem = (size_t)k * m * es;
		DB_REQUIRE(smem <= 48 * 1024, "ValueError: blockwise_dot block of %d x %d exceeds the shared-memory tile", k, m);
		dim3 grid(divup(n, 64), nblock);
		if (dtype == DB_F32) blockwise_nn_kernel<float><<<grid, 256, smem, st>>>((const float*)X, (const float*)W, (float*)Z, n, m, k, p, xoff, xbroadcast, nblock, beta_one);
		else                 blockwise_nn_kernel<double><<<grid, 256, smem, st>>>((const double*)X, (const double*)W, (double*)Z, n, m, k, p, xoff, xbroadcast, nblock, beta_one);
	} else if (mode == BW_NT) {
		size_t smem = (size_t)k * (m + 1) * es;
		DB_REQUIRE(smem <= 48 * 1024, "ValueError: blockwise_dot_nt block of %d x %d exceeds the shared-memory tile", k, m);
		dim3 grid(divup(n, 64), nblock);
		if (dtype == DB_F32) blockwise_nt_kernel<float><<<grid, 256, smem, st>>>((float*)X, (const float*)W, (const float*)Z, n, m, k, p, xoff, nblock);
		else                 blockwise_nt_kernel<double><<<grid, 256, smem, st>>>((double*)X, (const double*)W, (const double*)Z, n, m, k, p, xoff, nblock);
	} else {
		int nslice = 8;
		while (nslice > 1 && (size_t)nslice * k * m * es > 48 * 1024) nslice /= 2;
		size_t smem = (size_t)nslice * k * m * es;
		DB_REQUIRE(smem <= 48 * 1024, "ValueError: blockwise_dot_tn block of %d x %d exceeds the shared-memory tile", k, m);
		if (dtype == DB_F32) blockwise_tn_kernel<float><<<nblock, 32 * nslice, smem, st>>>((const float*)X, (float*)W, (const float*)Z, n, m, k, p, xoff, xbroadcast, nblock);
		else                 blockwise_tn_kernel<double><<<nblock, 32 * nslice, smem, st>>>((const double*)X, (double*)W, (const double*)Z, n, m, k, p, xoff, xbroadcast, nblock);
	}
	DB_LAUNCH_CHECK();
}

static void require_same_float(const smat* A, const smat* B, const char* a, const char* b)
{
	require_float(A, a); require_float(B, b);
	DB_REQUIRE(A->dtype == B->dtype, "TypeError: %s and %s must have the same dtype", a, b);
}

#define DISPATCH_FLOAT(dt, CALL_F32, CALL_F64) do { if ((dt) == DB_F32) { CALL_F32; } else { CALL_F64; } DB_LAUNCH_CHECK(); } while (0)

}  // namespace db

using namespace db;

DB_EXPORT void api_gradstep(smat* P, const smat* dP, const smat* drate, smat* mP, const smat* mrate)
{
	DB_API_TRY
	require_float(P, "P"); require_same_float(P, dP, "P", "dP"); require_same_float(P, drate, "P", "drate");
	require_same_float(P, mP, "P", "mP"); require_same_float(P, mrate, "P", "mrate");
	int n = P->shape.y;
	DB_ASSERT(dP->shape.y == n); DB_ASSERT(mP->shape.y == n); DB_ASSERT(drate->shape.y == n); DB_ASSERT(mrate->shape.y == n);
	size_t N = size_of(P);
	if (!N) return;
	unsigned g = elemwise_grid(N); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(P->dtype,
		(gradstep_kernel<<<g, 256, 0, st>>>((float*)P->data, (const float*)dP->data, (const float*)drate->data, (float*)mP->data, (const float*)mrate->data, N)),
		(gradstep_kernel<<<g, 256, 0, st>>>((double*)P->data, (const double*)dP->data, (const double*)drate->data, (double*)mP->data, (const double*)mrate->data, N)));
	DB_API_CATCH
}

DB_EXPORT void api_gradstep_nesterov1(smat* P, const smat* mP, const smat* mrate)
{
	DB_API_TRY
	require_float(P, "P"); require_same_float(P, mP, "P", "mP"); require_same_float(P, mrate, "P", "mrate");
	int n = P->shape.y;
	DB_ASSERT(mP->shape.y == n); DB_ASSERT(mrate->shape.y == n);
	size_t N = size_of(P);
	if (!N) return;
	unsigned g = elemwise_grid(N); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(P->dtype,
		(gradstep_nesterov1_kernel<<<g, 256, 0, st>>>((float*)P->data, (const float*)mP->data, (const float*)mrate->data, N)),
		(gradstep_nesterov1_kernel<<<g, 256, 0, st>>>((double*)P->data, (const double*)mP->data, (const double*)mrate->data, N)));
	DB_API_CATCH
}

DB_EXPORT void api_gradstep_nesterov2(smat* P, const smat* dP, const smat* drate, smat* mP, const smat* mrate)
{
	DB_API_TRY
	require_float(P, "P"); require_same_float(P, dP, "P", "dP"); require_same_float(P, drate, "P", "drate");
	require_same_float(P, mP, "P", "mP"); require_same_float(P, mrate, "P", "mrate");
	int n = P->shape.y;
	DB_ASSERT(dP->shape.y == n); DB_ASSERT(mP->shape.y == n); DB_ASSERT(drate->shape.y == n); DB_ASSERT(mrate->shape.y == n);
	size_t N = size_of(P);
	if (!N) return;
	unsigned g = elemwise_grid(N); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(P->dtype,
		(gradstep_nesterov2_kernel<<<g, 256, 0, st>>>((float*)P->data, (const float*)dP->data, (const float*)drate->data, (float*)mP->data, (const float*)mrate->data, N)),
		(gradstep_nesterov2_kernel<<<g, 256, 0, st>>>((double*)P->data, (const double*)dP->data, (const double*)drate->data, (double*)mP->data, (const double*)mrate->data, N)));
	DB_API_CATCH
}

DB_EXPORT void api_madd_bcast(const smat* A, const smat* b, uint32_t k, smat* dst)
{
	DB_API_TRY
	require_float(A, "A"); require_float(b, "b"); require_float(dst, "dst");
	DB_ASSERT(A->dtype == dst->dtype); DB_ASSERT(A->dtype == b->dtype);
	DB_ASSERT(size_of(A) == size_of(dst));
	DB_REQUIRE(size_of(b) > 0 && k > 0, "ValueError: madd_bcast needs a non-empty b and k > 0");
	DB_ASSERT(size_of(A) % size_of(b) == 0);
	size_t N = size_of(A);
	if (!N) return;
	unsigned g = elemwise_grid(N), m = (unsigned)size_of(b); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(A->dtype,
		(madd_bcast_kernel<<<g, 256, 0, st>>>((const float*)A->data, (const float*)b->data, (float*)dst->data, N, m, k)),
		(madd_bcast_kernel<<<g, 256, 0, st>>>((const double*)A->data, (const double*)b->data, (double*)dst->data, N, m, k)));
	DB_API_CATCH
}

DB_EXPORT void api_maskout(const smat* M, smat* A)
{
	DB_API_TRY
	require_dtype(M, DB_B8, "M", "b8"); require_float(A, "A");
	DB_ASSERT(size_of(A) == size_of(M));
	size_t N = size_of(A);
	if (!N) return;
	unsigned g = elemwise_grid(N); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(A->dtype,
		(maskout_kernel<<<g, 256, 0, st>>>((const uint8_t*)M->data, (float*)A->data, N)),
		(maskout_kernel<<<g, 256, 0, st>>>((const uint8_t*)M->data, (double*)A->data, N)));
	DB_API_CATCH
}

DB_EXPORT void api_calc_zmask(const smat* Z, smat* M)
{
	DB_API_TRY
	require_float(Z, "Z"); require_dtype(M, DB_B8, "M", "b8");
	DB_ASSERT(size_of(Z) == size_of(M));
	size_t n = Z->shape.y, m = Z->shape.x;
	if (n * m < 2) return;
	unsigned g = elemwise_grid(n * m / 2); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(Z->dtype,
		(calc_zmask_kernel<<<g, 256, 0, st>>>((const float*)Z->data, (uint8_t*)M->data, n, m)),
		(calc_zmask_kernel<<<g, 256, 0, st>>>((const double*)Z->data, (uint8_t*)M->data, n, m)));
	DB_API_CATCH
}

// Keep-mask of one training step drawn on the device, for steps replayed from a CUDA
// graph: the draw index is a counter in device memory (counters[0]; counters[1] counts
// the CTAs of the running launch), read by every CTA before it arrives and advanced by
// the last one, so every replay draws a fresh mask with no host work.  Same Bernoulli
// rule as dropout_fp_tr_kernel (dropout.cu:41-62): keep where u >= rate[model]; with
// matchrows the two strands of a pair share their mask row.
__global__ void __launch_bounds__(256)
dropout_mask_kernel(uint8_t* M, size_t nrow, size_t ncol, const float* rate, unsigned k, int matchrows,
                    uint64_t seed, uint32_t* counters)
{
	__shared__ unsigned s_step;
	if (threadIdx.x == 0) s_step = *reinterpret_cast<volatile uint32_t*>(counters);
	__syncthreads();
	const uint64_t call = ((uint64_t)1 << 40) + s_step;          // apart from the host-counted draws of api_dropout_fp_tr
	if (matchrows) {
		GRID_STRIDE(i, nrow * ncol / 2) {
			const size_t row = (i / ncol) * 2, col = i % ncol;
			const bool mask = uniform_01(seed, call, i) >= rate[col / k];
			M[row * ncol + col] = mask; M[(row + 1) * ncol + col] = mask;
		}
	} else {
		GRID_STRIDE(i, nrow * ncol) M[i] = uniform_01(seed, call, i) >= rate[(i % ncol) / k];
	}
	__syncthreads();
	if (threadIdx.x == 0) {
		__threadfence();
		if (atomicAdd(counters + 1, 1u) == gridDim.x - 1) {
			counters[1] = 0;
			counters[0] = counters[0] + 1;
			__threadfence();
		}
	}
}

DB_EXPORT void db_dropout_mask(uint8_t* M, uint32_t nrow, uint32_t ncol, const float* rate, uint32_t nmodel,
                               int matchrows, uint32_t* counters)
{
	DB_API_TRY
	DB_REQUIRE(M && rate && counters, "ValueError: db_dropout_mask got a NULL pointer");
	DB_REQUIRE(nmodel > 0 && ncol % nmodel == 0, "ValueError: the mask's %u columns do not divide among %u models", ncol, nmodel);
	DB_REQUIRE(!matchrows || nrow % 2 == 0, "ValueError: matched rows need an even number of rows (got %u)", nrow);
	if (!nrow || !ncol) return;
	const size_t n = (size_t)nrow * ncol / (matchrows ? 2 : 1);
	dropout_mask_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(M, nrow, ncol, rate, ncol / nmodel, matchrows, state().seed, counters);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

static void dropout_fp_tr(const smat* X, const smat* rate, const smat* U, smat* Z, smat* M, int matchrows)
{
	require_float(X, "X"); require_float(rate, "rate"); require_float(Z, "Z"); require_dtype(M, DB_B8, "M", "b8");
	DB_ASSERT(X->dtype == rate->dtype); DB_ASSERT(X->dtype == Z->dtype);
	DB_ASSERT(size_of(X) == size_of(Z)); DB_ASSERT(size_of(X) == size_of(M));
	DB_REQUIRE(size_of(rate) > 0, "ValueError: rate must not be empty");
	DB_ASSERT(size_of(X) % size_of(rate) == 0);
	const float* u = nullptr;
	if (U) { require_dtype(U, DB_F32, "U", "f32"); u = (const float*)U->data; }
	size_t N = size_of(X);
	if (!N) return;
	unsigned m = (unsigned)size_of(rate), k = (unsigned)X->shape.x / m;
	DB_REQUIRE(k > 0, "ValueError: X has fewer columns than rate has entries");
	uint64_t call = state().rng_calls++, seed = state().seed;
	cudaStream_t st = state().stream;
	if (matchrows) {
		size_t ncol = (size_t)m * k, nrow = N / ncol;
		if (U) DB_ASSERT(size_of(U) >= nrow * ncol / 2);
		if (nrow * ncol < 2) return;
		unsigned g = elemwise_grid(nrow * ncol / 2);
		DISPATCH_FLOAT(X->dtype,
			(dropout_fp_tr_match_kernel<<<g, 256, 0, st>>>((const float*)X->data, (const float*)rate->data, u, seed, call, (float*)Z->data, (uint8_t*)M->data, nrow, ncol, k)),
			(dropout_fp_tr_match_kernel<<<g, 256, 0, st>>>((const double*)X->data, (const double*)rate->data, u, seed, call, (double*)Z->data, (uint8_t*)M->data, nrow, ncol, k)));
	} else {
		if (U) DB_ASSERT(size_of(U) >= N);
		unsigned g = elemwise_grid(N);
		DISPATCH_FLOAT(X->dtype,
			(dropout_fp_tr_kernel<<<g, 256, 0, st>>>((const float*)X->data, (const float*)rate->data, u, seed, call, (float*)Z->data, (uint8_t*)M->data, N, m, k)),
			(dropout_fp_tr_kernel<<<g, 256, 0, st>>>((const double*)X->data, (const double*)rate->data, u, seed, call, (double*)Z->data, (uint8_t*)M->data, N, m, k)));
	}
}

DB_EXPORT void api_dropout_fp_tr(const smat* X, const smat* rate, smat* Z, smat* M, int matchrows)
{
	DB_API_TRY
	dropout_fp_tr(X, rate, nullptr, Z, M, matchrows);
	DB_API_CATCH
}

DB_EXPORT void api_dropout_fp_tr_u(const smat* X, const smat* rate, const smat* U, smat* Z, smat* M, int matchrows)
{
	DB_API_TRY
	DB_REQUIRE(U != nullptr, "ValueError: argument U must not be NULL");
	dropout_fp_tr(X, rate, U, Z, M, matchrows);
	DB_API_CATCH
}

static void dropout_scale(const smat* X, const smat* rate, smat* Z)
{
	require_float(X, "X"); require_float(rate, "rate"); require_float(Z, "Z");
	DB_ASSERT(X->dtype == rate->dtype); DB_ASSERT(X->dtype == Z->dtype);
	DB_ASSERT(size_of(X) == size_of(Z));
	DB_REQUIRE(size_of(rate) > 0, "ValueError: rate must not be empty");
	DB_ASSERT(size_of(X) % size_of(rate) == 0);
	size_t N = size_of(X);
	if (!N) return;
	unsigned m = (unsigned)size_of(rate), k = (unsigned)X->shape.x / m;
	DB_REQUIRE(k > 0, "ValueError: X has fewer columns than rate has entries");
	unsigned g = elemwise_grid(N); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(X->dtype,
		(dropout_scale_kernel<<<g, 256, 0, st>>>((const float*)X->data, (const float*)rate->data, (float*)Z->data, N, m, k)),
		(dropout_scale_kernel<<<g, 256, 0, st>>>((const double*)X->data, (const double*)rate->data, (double*)Z->data, N, m, k)));
}

DB_EXPORT void api_dropout_fp_te(const smat* X, const smat* rate, smat* Z)
{
	DB_API_TRY
	dropout_scale(X, rate, Z);
	DB_API_CATCH
}

DB_EXPORT void api_dropout_bp_te(const smat* dZ, const smat* rate, smat* dX)
{
	DB_API_TRY
	dropout_scale(dZ, rate, dX);
	DB_API_CATCH
}

DB_EXPORT void api_dropout_bp_tr(const smat* dZ, const smat* M, smat* dX)
{
	DB_API_TRY
	require_float(dZ, "dZ"); require_dtype(M, DB_B8, "M", "b8"); require_float(dX, "dX");
	DB_ASSERT(dX->dtype == dZ->dtype); DB_ASSERT(size_of(dX) == size_of(M)); DB_ASSERT(size_of(dX) == size_of(dZ));
	size_t N = size_of(dX);
	if (!N) return;
	unsigned g = elemwise_grid(N); cudaStream_t st = state().stream;
	DISPATCH_FLOAT(dZ->dtype,
		(dropout_bp_tr_kernel<<<g, 256, 0, st>>>((const float*)dZ->data, (const uint8_t*)M->data, (float*)dX->data, N)),
		(dropout_bp_tr_kernel<<<g, 256, 0, st>>>((const double*)dZ->data, (const uint8_t*)M->data, (double*)dX->data, N)));
	DB_API_CATCH
}

// Shapes as deepity_smat.cpp:269-468 derives them.
DB_EXPORT void api_blockwise_dot(int nblock, const smat* X, const smat* W, smat* Z)
{
	DB_API_TRY
	require_same_float(X, W, "X", "W"); require_same_float(X, Z, "X", "Z");
	DB_REQUIRE(nblock > 0, "ValueError: nblock must be positive");
	DB_ASSERT(X->shape.y == Z->shape.y);
	DB_ASSERT(Z->shape.x == W->shape.x * nblock);
	DB_ASSERT(W->shape.y % nblock == 0);
	DB_ASSERT(X->shape.x == W->shape.y || X->shape.x * nblock == W->shape.y);
	int n = X->shape.y, k = W->shape.y / nblock, m = W->shape.x;
	bool bc = nblock > 1 && X->shape.x * nblock == W->shape.y;
	launch_blockwise(BW_NN, X->dtype, nblock, 0, bc, n, m, k, k, X->data, W->data, Z->data, false);
	DB_API_CATCH
}

DB_EXPORT void api_blockwise_dot_nt(int nblock, const smat* dZ, const smat* W, smat* dX)
{
	DB_API_TRY
	require_same_float(dZ, W, "dZ", "W"); require_same_float(dZ, dX, "dZ", "dX");
	DB_REQUIRE(nblock > 0, "ValueError: nblock must be positive");
	DB_ASSERT(dX->shape.y == dZ->shape.y);
	DB_ASSERT(dZ->shape.x == W->shape.x * nblock);
	DB_ASSERT(W->shape.y % nblock == 0);
	DB_ASSERT(dX->shape.x == W->shape.y);
	int n = dX->shape.y, k = W->shape.y / nblock, m = W->shape.x;
	launch_blockwise(BW_NT, dZ->dtype, nblock, 0, false, n, m, k, k, dX->data, W->data, dZ->data, false);
	DB_API_CATCH
}

DB_EXPORT void api_blockwise_dot_tn(int nblock, const smat* X, const smat* dZ, smat* dW)
{
	DB_API_TRY
	require_same_float(X, dZ, "X", "dZ"); require_same_float(X, dW, "X", "dW");
	DB_REQUIRE(nblock > 0, "ValueError: nblock must be positive");
	DB_ASSERT(X->shape.y == dZ->shape.y);
	DB_ASSERT(dZ->shape.x == dW->shape.x * nblock);
	DB_ASSERT(dW->shape.y % nblock == 0);
	DB_ASSERT(X->shape.x == dW->shape.y || X->shape.x * nblock == dW->shape.y);
	int n = X->shape.y, k = dW->shape.y / nblock, m = dW->shape.x;
	bool bc = nblock > 1 && X->shape.x * nblock == dW->shape.y;
	launch_blockwise(BW_TN, X->dtype, nblock, 0, bc, n, m, k, k, X->data, dW->data, dZ->data, false);
	DB_API_CATCH
}

DB_EXPORT void api_blockwise_dot_combined(int nblock, int Xoffset, int Xbroadcast, const smat* X, const smat* W, smat* Z)
{
	DB_API_TRY
	require_same_float(X, W, "X", "W"); require_same_float(X, Z, "X", "Z");
	DB_REQUIRE(nblock > 0, "ValueError: nblock must be positive");
	DB_ASSERT(X->shape.y == Z->shape.y);
	DB_ASSERT(Z->shape.x == W->shape.x * nblock);
	DB_ASSERT(W->shape.y % nblock == 0);
	int n = X->shape.y, k = Xbroadcast ? X->shape.x : X->shape.x / nblock, m = W->shape.x, p = W->shape.y / nblock;
	DB_REQUIRE(Xoffset >= 0 && Xoffset + k <= p, "ValueError: input columns [%d,%d) exceed the %d weight rows per block", Xoffset, Xoffset + k, p);
	launch_blockwise(BW_NN, X->dtype, nblock, Xoffset, Xbroadcast != 0, n, m, k, p, X->data, W->data, Z->data, Xoffset != 0);
	DB_API_CATCH
}

DB_EXPORT void api_blockwise_dot_nt_combined(int nblock, int Xoffset, int Xbroadcast, smat* dX, const smat* W, const smat* dZ)
{
	DB_API_TRY
	require_same_float(dX, W, "dX", "W"); require_same_float(dX, dZ, "dX", "dZ");
	DB_REQUIRE(nblock > 0, "ValueError: nblock must be positive");
	DB_ASSERT(!Xbroadcast);
	DB_ASSERT(dX->shape.y == dZ->shape.y);
	DB_ASSERT(dZ->shape.x == W->shape.x * nblock);
	DB_ASSERT(W->shape.y % nblock == 0);
	DB_ASSERT(dX->shape.x % nblock == 0);
	int n = dX->shape.y, k = dX->shape.x / nblock, m = W->shape.x, p = W->shape.y / nblock;
	DB_REQUIRE(Xoffset >= 0 && Xoffset + k <= p, "ValueError: input columns [%d,%d) exceed the %d weight rows per block", Xoffset, Xoffset + k, p);
	launch_blockwise(BW_NT, dX->dtype, nblock, Xoffset, false, n, m, k, p, dX->data, W->data, dZ->data, false);
	DB_API_CATCH
}

DB_EXPORT void api_blockwise_dot_tn_combined(int nblock, int Xoffset, int Xbroadcast, const smat* X, smat* dW, const smat* dZ)
{
	DB_API_TRY
	require_same_float(X, dW, "X", "dW"); require_same_float(X, dZ, "X", "dZ");
	DB_REQUIRE(nblock > 0, "ValueError: nblock must be positive");
	DB_ASSERT(X->shape.y == dZ->shape.y);
	DB_ASSERT(dZ->shape.x == dW->shape.x * nblock);
	DB_ASSERT(dW->shape.y % nblock == 0);
	int n = X->shape.y, k = Xbroadcast ? X->shape.x : X->shape.x / nblock, m = dW->shape.x, p = dW->shape.y / nblock;
	DB_REQUIRE(Xoffset >= 0 && Xoffset + k <= p, "ValueError: input columns [%d,%d) exceed the %d weight rows per block", Xoffset, Xoffset + k, p);
	launch_blockwise(BW_TN, X->dtype, nblock, Xoffset, Xbroadcast != 0, n, m, k, p, X->data, dW->data, dZ->data, false);
	DB_API_CATCH
}
