// Drop-in kangaroo_smat entry points: the unfused motif scan, its two backward
// passes, region pooling forward/backward and ordinal-input dropout.
// These keep the reference's operator granularity (one call per graph node,
// the [npos, nfilter] activation materialised in HBM), so they are bound by
// HBM traffic; the fused path in scanpool_f32.cu removes those round trips.
//
// Reference behaviour restated here (code/libs/kangaroo/kangaroo_smat/):
//   corr1ord.cuh:108-164      scan; taps ascending; N = mean of the 4 channels; 254 = 0
//   corr1ord_bprop.cuh:91-138 filter gradient
//   corr1ord_bprop.cu:191-201 input gradient (a host loop in the reference)
//   poolrgn.cuh:44-160        max (first maximum wins) / sum / avg / all
//   poolrgn_bprop.cuh:45-127  pooling backward
//   dropoutord.cu:41-52       ordinal dropout (254 marks a dropped base)
//   kangaroo_smat.cpp:98-294  argument validation and shape derivation
#include "db_common.cuh"
#include "db_rng.cuh"

namespace db {

// Base code used to index the six-entry lookup table of a tap:
// 0..3 = A,C,G,T/U; 4 = any other byte (mean of the four); 5 = 254 (dropped).
__device__ __forceinline__ unsigned base_code(unsigned x) { return x < 4u ? x : (x == 254u ? 5u : 4u); }

// ------------------------------------------------------------------ corr1ord
// One CTA = one chunk of FC filters x a grid-stride sequence of row tiles.
// Shared memory: lut[m][6][FC] and the tile's base codes.  Each thread owns 4
// filters of one row at a time; consecutive threads own consecutive filter
// quads, so a warp writes whole 128-byte lines of Z.
template <typename T, int TR>
__global__ void __launch_bounds__(256)
corr1ord_kernel(const T* __restrict__ W, unsigned m, unsigned nf, unsigned FC,
                const uint8_t* __restrict__ X, unsigned n, T* __restrict__ Z)
{
	extern __shared__ __align__(16) unsigned char smem_raw[];
	T* lut = reinterpret_cast<T*>(smem_raw);
	uint8_t* xs = reinterpret_cast<uint8_t*>(lut + (size_t)m * 6 * FC);

	const unsigned f0 = blockIdx.y * FC;
	const unsigned fc = min(FC, nf - f0);            // filters of this chunk that exist
	for (unsigned t = threadIdx.x; t < m * FC; t += blockDim.x) {
		unsigned j = t / FC, f = t % FC;
		T w0 = 0, w1 = 0, w2 = 0, w3 = 0;
		if (f < fc) {
			w0 = W[(size_t)(4*j+0)*nf + f0 + f]; w1 = W[(size_t)(4*j+1)*nf + f0 + f];
			w2 = W[(size_t)(4*j+2)*nf + f0 + f]; w3 = W[(size_t)(4*j+3)*nf + f0 + f];
		}
		T z = w0; z += w1; z += w2; z += w3;
		T* e = lut + (size_t)j * 6 * FC + f;
		e[0] = w0; e[FC] = w1; e[2*FC] = w2; e[3*FC] = w3; e[4*FC] = z * (T)0.25; e[5*FC] = (T)0;
	}

	const unsigned QC = FC / 4;                       // filter quads per chunk
	const unsigned q = threadIdx.x % QC, rl = threadIdx.x / QC, RL = blockDim.x / QC;
	for (unsigned tile = blockIdx.x; (size_t)tile * TR < n; tile += gridDim.x) {
		const unsigned r0 = tile * TR;
		const unsigned rows = min((unsigned)TR, n - r0);
		__syncthreads();
		for (unsigned t = threadIdx.x; t < rows + m - 1; t += blockDim.x)
			xs[t] = (uint8_t)base_code(X[r0 + t]);
		__syncthreads();
		for (unsigned r = rl; r < rows; r += RL) {
			T z0 = 0, z1 = 0, z2 = 0, z3 = 0;
			for (unsigned j = 0; j < m; ++j) {
				const T* e = lut + ((size_t)j * 6 + xs[r + j]) * FC + 4 * q;
				z0 += e[0]; z1 += e[1]; z2 += e[2]; z3 += e[3];
			}
			T* out = Z + (size_t)(r0 + r) * nf + f0 + 4 * q;
			const unsigned left = fc > 4 * q ? fc - 4 * q : 0;
			if (left > 0) out[0] = z0;
			if (left > 1) out[1] = z1;
			if (left > 2) out[2] = z2;
			if (left > 3) out[3] = z3;
		}
	}
}

template <typename T>
static void launch_corr1ord(const T* W, unsigned m, unsigned nf, const uint8_t* X, unsigned n, T* Z)
{
	if (n == 0 || nf == 0 || m == 0) return;
	const int TR = 256;
	// Largest power-of-two chunk (<= 64 filters) whose table fits in 96 KB.
	unsigned FC = 64;
	while (FC > 4 && (FC / 2 >= nf || (size_t)m * 6 * FC * sizeof(T) > 96 * 1024)) FC /= 2;
	size_t smem = (size_t)m * 6 * FC * sizeof(T) + TR + m + 16;
	DB_REQUIRE(smem <= 200 * 1024, "ValueError: filter length %u is too long for this kernel", m);
	auto kern = corr1ord_kernel<T, TR>;
	DB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	unsigned tiles = divup(n, (unsigned)TR);
	dim3 grid(min(tiles, (unsigned)state().sm_count * 4), divup(nf, FC));
	kern<<<grid, 256, smem, state().stream>>>(W, m, nf, FC, X, n, Z);
	DB_LAUNCH_CHECK();
}

// -------------------------------------------------------------- bprop to W
// Stage 1: one CTA per (row tile, filter chunk).  A thread owns a (tap, filter)
// pair and walks the tile's rows in order, so each partial sum has a fixed
// order.  Stage 2 adds the per-tile partials, tile ascending, into dW.  No
// float atomics: two runs give identical bits (the reference's atomicAdd does
// not, corr1ord_bprop.cuh:136).
template <typename T, int TR, int FC>
__global__ void __launch_bounds__(256)
corr1ord_bprop_W_stage1(unsigned m, unsigned nf, const uint8_t* __restrict__ X, unsigned n,
                        const T* __restrict__ dZ, T* __restrict__ partial)
{
	extern __shared__ __align__(16) unsigned char smem_raw[];
	T* dz = reinterpret_cast<T*>(smem_raw);                 // [TR][FC]
	uint8_t* xs = reinterpret_cast<uint8_t*>(dz + TR * FC); // [TR + m - 1]
	const unsigned r0 = blockIdx.x * TR, f0 = blockIdx.y * FC;
	const unsigned rows = min((unsigned)TR, n - r0);
	const unsigned fc = min((unsigned)FC, nf - f0);
	for (unsigned t = threadIdx.x; t < rows + m - 1; t += blockDim.x)
		xs[t] = (uint8_t)base_code(X[r0 + t]);
	for (unsigned t = threadIdx.x; t < rows * FC; t += blockDim.x) {
		unsigned r = t / FC, f = t % FC;
		dz[t] = f < fc ? dZ[(size_t)(r0 + r) * nf + f0 + f] : (T)0;
	}
	__syncthreads();
	T* out = partial + (size_t)blockIdx.x * 4 * m * nf;
	for (unsigned p = threadIdx.x; p < m * FC; p += blockDim.x) {
		unsigned j = p / FC, f = p % FC;
		T a0 = 0, a1 = 0, a2 = 0, a3 = 0;
		for (unsigned r = 0; r < rows; ++r) {
			T v = dz[r * FC + f];
			unsigned c = xs[r + j];
			if (c == 0) a0 += v; else if (c == 1) a1 += v; else if (c == 2) a2 += v; else if (c == 3) a3 += v;
			else if (c == 4) { T z = v * (T)0.25; a0 += z; a1 += z; a2 += z; a3 += z; }
		}
		if (f < fc) {
			out[(size_t)(4*j+0)*nf + f0 + f] = a0; out[(size_t)(4*j+1)*nf + f0 + f] = a1;
			out[(size_t)(4*j+2)*nf + f0 + f] = a2; out[(size_t)(4*j+3)*nf + f0 + f] = a3;
		}
	}
}

template <typename T>
__global__ void reduce_partials_add(T* __restrict__ dst, const T* __restrict__ partial, size_t count, unsigned nparts)
{
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
		T s = 0;
		for (unsigned p = 0; p < nparts; ++p) s += partial[(size_t)p * count + i];
		dst[i] += s;
	}
}

template <typename T>
static void launch_corr1ord_bprop_W(T* dW, unsigned m, unsigned nf, const uint8_t* X, unsigned n, const T* dZ)
{
	if (n == 0 || nf == 0 || m == 0) return;
	const int TR = 128, FC = 32;
	unsigned tiles = divup(n, (unsigned)TR);
	size_t count = (size_t)4 * m * nf;
	T* partial = (T*)scratch(count * tiles * sizeof(T));
	size_t smem = (size_t)TR * FC * sizeof(T) + TR + m + 16;
	auto k1 = corr1ord_bprop_W_stage1<T, TR, FC>;
	DB_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	k1<<<dim3(tiles, divup(nf, (unsigned)FC)), 256, smem, state().stream>>>(m, nf, X, n, dZ, partial);
	DB_LAUNCH_CHECK();
	reduce_partials_add<T><<<elemwise_grid(count), 256, 0, state().stream>>>(dW, partial, count, tiles);
	DB_LAUNCH_CHECK();
}

// -------------------------------------------------------------- bprop to X
// dX[i,c] += sum_f sum_k dZ[i-k,f] * W[(4k+c)nf+f], filters outer, taps inner,
// products and sums rounded separately: the order and rounding of the
// reference's host loop (corr1ord_bprop.cu:191-201), computed on the device.
// One warp per row i: lane = (tap group, channel); partial sums would change the
// order, so each (i,c) is one thread and the warp covers 8 rows x 4 channels.
template <typename T>
__global__ void corr1ord_bprop_X_kernel(T* __restrict__ dX, unsigned n, const T* __restrict__ W, unsigned m,
                                        unsigned nf, const T* __restrict__ dZ)
{
	size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (t >= (size_t)n * 4) return;
	unsigned i = (unsigned)(t / 4), c = (unsigned)(t % 4);
	T acc = dX[t];
	unsigned kmax = min(m, i + 1);
	for (unsigned f = 0; f < nf; ++f)
		for (unsigned k = 0; k < kmax; ++k) {
			T prod;
			if (sizeof(T) == 4) {
				prod = __fmul_rn((float)dZ[(size_t)(i-k)*nf + f], (float)W[(size_t)(4*k+c)*nf + f]);
				acc = __fadd_rn((float)acc, (float)prod);
			} else {
				prod = __dmul_rn((double)dZ[(size_t)(i-k)*nf + f], (double)W[(size_t)(4*k+c)*nf + f]);
				acc = __dadd_rn((double)acc, (double)prod);
			}
		}
	dX[t] = acc;
}

// The same sums for float, tiled: a CTA owns BXR consecutive rows; the dZ rows its taps
// reach ([i0 - m + 1, i0 + BXR) x nf) and the filter bank, regrouped as [tap][filter][4
// channels], wait in shared memory, and a thread owns one row and all four channels, so
// that one dZ operand and one 16-byte weight operand feed four multiply-adds.  Order and
// rounding per output are those of the kernel above (filters outer, taps inner, product
// and sum rounded separately): the results are bit-identical.
static constexpr int BXR = 128;

__global__ void __launch_bounds__(BXR)
corr1ord_bprop_X_tiled_kernel(float* __restrict__ dX, unsigned n, const float* __restrict__ W, unsigned m,
                              unsigned nf, const float* __restrict__ dZ)
{
	extern __shared__ __align__(16) float bx_smem[];
	float4* w4 = reinterpret_cast<float4*>(bx_smem);                // [m][nf] float4 (channels 0..3)
	float* dz = bx_smem + (size_t)4 * m * nf;                       // [BXR + m - 1][nf + 1]
	const unsigned i0 = blockIdx.x * BXR, ld = nf + 1;
	for (unsigned e = threadIdx.x; e < m * nf; e += BXR) {
		const unsigned k = e / nf, f = e - k * nf;
		w4[e] = make_float4(W[(size_t)(4 * k) * nf + f], W[(size_t)(4 * k + 1) * nf + f],
		                    W[(size_t)(4 * k + 2) * nf + f], W[(size_t)(4 * k + 3) * nf + f]);
	}
	const unsigned nrow = BXR + m - 1;
	for (unsigned e = threadIdx.x; e < nrow * nf; e += BXR) {
		const unsigned r = e / nf, f = e - r * nf;
		const long long row = (long long)i0 + r - (long long)(m - 1);
		dz[r * ld + f] = (row >= 0 && row < (long long)n) ? dZ[(size_t)row * nf + f] : 0.f;
	}
	__syncthreads();
	const unsigned i = i0 + threadIdx.x;
	if (i >= n) return;
	float4 acc = reinterpret_cast<const float4*>(dX)[i];
	const unsigned kmax = min(m, i + 1);
	const float* zrow = dz + (size_t)(threadIdx.x + m - 1) * ld;   // dZ row i; row i - k lies k rows before it
	for (unsigned f = 0; f < nf; ++f)
		for (unsigned k = 0; k < kmax; ++k) {
			const float z = zrow[(ptrdiff_t)f - (ptrdiff_t)k * (ptrdiff_t)ld];
			const float4 w = w4[k * nf + f];
			acc.x = __fadd_rn(acc.x, __fmul_rn(z, w.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(z, w.y));
			acc.z = __fadd_rn(acc.z, __fmul_rn(z, w.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(z, w.w));
		}
	reinterpret_cast<float4*>(dX)[i] = acc;
}

// ------------------------------------------------------------------ poolrgn
// One thread per (region, map): rows ascending, strict '>' so the first maximal
// row wins, running sum in row order (poolrgn.cuh:60-78,99-114,133-159).
template <typename T>
__global__ void poolrgn_kernel(const T* __restrict__ U, unsigned nf, const uint32_t* __restrict__ R, unsigned nregion,
                               unsigned rcols, T* __restrict__ P, uint32_t* __restrict__ A, int ptype)
{
	size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (t >= (size_t)nregion * nf) return;
	unsigned r = (unsigned)(t / nf), f = (unsigned)(t % nf);
	unsigned first = R[r * rcols], last = R[r * rcols + 1];
	unsigned step = rcols == 3 ? R[r * rcols + 2] : 1u;
	if (step == 0) step = 1;
	T x = U[(size_t)first * nf + f];
	T y = x;
	unsigned xi = first;
	unsigned row = first + step;
	if (step == 1) {
		// eight independent loads in flight per thread, then the reduction in row order
		const T* u = U + (size_t)row * nf + f;
		for (; row + 8 <= last; row += 8, u += (size_t)8 * nf) {
			T v[8];
			#pragma unroll
			for (int k = 0; k < 8; ++k) v[k] = u[(size_t)k * nf];
			#pragma unroll
			for (int k = 0; k < 8; ++k) {
				if (v[k] > x) { x = v[k]; xi = row + k; }
				y += v[k];
			}
		}
	}
	for (; row < last; row += step) {
		T v = U[(size_t)row * nf + f];
		if (v > x) { x = v; xi = row; }
		y += v;
	}
	unsigned cnt = ((last - first) + step - 1) / step;
	switch (ptype) {
	case DB_PT_MAX: P[t] = x; if (A) A[t] = xi * nf + f; break;
	case DB_PT_AVG: P[t] = y / (T)cnt; break;
	case DB_PT_SUM: P[t] = y; break;
	default:        P[2*t] = x; P[2*t+1] = y / (T)cnt; if (A) A[t] = xi * nf + f; break;
	}
}

// float, unit step, NF in {4, 8, 16, 32}: a warp takes 32/NF regions at a time, lane =
// (region, map), so that the ordered reduction keeps all 32 lanes busy.  The rows of a
// region are contiguous in memory: for each of its regions the warp copies the next 16 rows
// into its slice of shared memory with 16-byte cp.async (512 contiguous bytes per
// instruction, L2 only), two buffers deep, so that the copies of the next step are in flight
// while every lane walks the staged rows of its own region and map in order: strict '>'
// (first maximum wins) and the running sum in row order, exactly as the scalar kernel.  The
// reads are what should bound this operator (npos*nf*4 bytes of HBM); what is left above
// them is the issue cost of the ordered reduction (about five instructions per row).
static constexpr int PRW = 8;                    // warps per CTA

__device__ __forceinline__ void pool_cp16(void* dst, const void* src)
{
	unsigned d = (unsigned)__cvta_generic_to_shared(dst);
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(d), "l"(src) : "memory");
}

template <int NF, int PRR, int NBUF>             // maps; rows staged per region and step; buffers
__global__ void __launch_bounds__(32 * PRW)
poolrgn_warp_kernel(const float* __restrict__ U, const uint32_t* __restrict__ R, unsigned nregion,
                    float* __restrict__ P, uint32_t* __restrict__ A, int ptype)
{
	constexpr int NSUB = 32 / NF;                                  // regions per warp
	constexpr int Q = NF / 4;                                      // 16-byte units per row
	constexpr int PRL = PRR * Q / 32 > 0 ? PRR * Q / 32 : 1;       // copies per lane, region and step
	__shared__ __align__(16) float stage[PRW][NBUF][NSUB][PRR * NF];
	const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
	const unsigned sub = lane / NF, f = lane % NF;
	for (unsigned r0 = (blockIdx.x * PRW + warp) * NSUB; r0 < nregion; r0 += gridDim.x * PRW * NSUB) {
		// bounds of the warp's regions (lane s fetches region r0+s), then this lane's own
		uint2 rg = make_uint2(0u, 0u);
		if (lane < NSUB && r0 + lane < nregion) rg = reinterpret_cast<const uint2*>(R)[r0 + lane];
		unsigned fs[NSUB], ls[NSUB], longest = 0;
		#pragma unroll
		for (int s = 0; s < NSUB; ++s) {
			fs[s] = __shfl_sync(0xffffffffu, rg.x, s); ls[s] = __shfl_sync(0xffffffffu, rg.y, s);
			longest = max(longest, ls[s] > fs[s] ? ls[s] - fs[s] : 0u);
		}
		const unsigned first = __shfl_sync(0xffffffffu, rg.x, sub), last = __shfl_sync(0xffffffffu, rg.y, sub);
		const bool live = r0 + sub < nregion;
		auto fetch = [&](unsigned off, unsigned buf) {             // always commits a group, an empty one past the end
			#pragma unroll
			for (int s = 0; s < NSUB; ++s) {
				const unsigned row = fs[s] + off;
				const unsigned units = row < ls[s] ? min((unsigned)PRR, ls[s] - row) * Q : 0u;
				const float4* src = reinterpret_cast<const float4*>(U + (size_t)row * NF);
				#pragma unroll
				for (int j = 0; j < PRL; ++j)
					if (lane + 32 * j < units) pool_cp16(reinterpret_cast<float4*>(stage[warp][buf][s]) + lane + 32 * j, src + lane + 32 * j);
			}
			asm volatile("cp.async.commit_group;" ::: "memory");
		};
		#pragma unroll
		for (int b = 0; b < NBUF - 1; ++b) fetch(1 + b * PRR, b);
		float x = 0.f, y = 0.f;
		unsigned xi = first;
		if (live) { x = U[(size_t)first * NF + f]; y = x; }                     // the first row is read even if the region is empty
		unsigned buf = 0;
		for (unsigned off = 1; off < longest; off += PRR, buf = buf + 1 == NBUF ? 0 : buf + 1) {
			fetch(off + (NBUF - 1) * PRR, buf == 0 ? NBUF - 1 : buf - 1);
			asm volatile("cp.async.wait_group %0;" :: "n"(NBUF - 1) : "memory");
			__syncwarp();
			const unsigned row = first + off;
			const unsigned nrow = (live && row < last) ? min((unsigned)PRR, last - row) : 0u;
			const float* col = stage[warp][buf][sub] + f;
			if (nrow == PRR) {
				#pragma unroll
				for (unsigned k = 0; k < PRR; ++k) {
					const float w = col[k * NF];
					if (w > x) { x = w; xi = row + k; }
					y += w;
				}
			} else {
				for (unsigned k = 0; k < nrow; ++k) {
					const float w = col[k * NF];
					if (w > x) { x = w; xi = row + k; }
					y += w;
				}
			}
			__syncwarp();                                                       // all lanes are done with this buffer before it is refilled
		}
		if (live) {
			const size_t t = (size_t)(r0 + sub) * NF + f;
			const unsigned cnt = last - first;
			switch (ptype) {
			case DB_PT_MAX: P[t] = x; if (A) A[t] = xi * NF + f; break;
			case DB_PT_AVG: P[t] = y / (float)cnt; break;
			case DB_PT_SUM: P[t] = y; break;
			default:        P[2*t] = x; P[2*t+1] = y / (float)cnt; if (A) A[t] = xi * NF + f; break;
			}
		}
	}
}

template <typename T>
__global__ void poolrgn_bprop_kernel(T* __restrict__ U, unsigned nf, const uint32_t* __restrict__ R, unsigned nregion,
                                     unsigned rcols, const T* __restrict__ P, const uint32_t* __restrict__ A, int ptype)
{
	size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (t >= (size_t)nregion * nf) return;
	unsigned r = (unsigned)(t / nf), f = (unsigned)(t % nf);
	if (ptype == DB_PT_MAX) { atomicAdd(&U[A[t]], P[t]); return; }
	unsigned first = R[r * rcols], last = R[r * rcols + 1];
	unsigned step = rcols == 3 ? R[r * rcols + 2] : 1u;
	if (step == 0) step = 1;
	unsigned cnt = ((last - first) + step - 1) / step;
	T d = ptype == DB_PT_ALL ? P[2*t+1] : P[t];
	if (ptype != DB_PT_SUM) d /= (T)cnt;
	for (unsigned row = first; row < last; row += step)
		atomicAdd(&U[(size_t)row * nf + f], d);
	if (ptype == DB_PT_ALL) atomicAdd(&U[A[t]], P[2*t]);
}

// float, unit step, nf in {4, 8, ..., 128}: a warp per region.  A lane owns four
// neighbouring filters and every (128/nf)-th row, so one warp instruction adds a
// contiguous 512-byte run of the unpooled maps with 16-byte vector adds: a quarter of
// the atomic operations of the scalar kernel, each fully coalesced.  With disjoint regions
// (the batch layout) every element receives one add, so the result does not depend on the
// order; the adds resolve in L2 and the pass moves one read and one write of U through HBM.
__global__ void __launch_bounds__(256)
poolrgn_bprop_v4_kernel(float* __restrict__ U, unsigned nf, const uint32_t* __restrict__ R, unsigned nregion,
                        const float* __restrict__ P, const uint32_t* __restrict__ A, int ptype)
{
	const unsigned lane = threadIdx.x & 31, q = nf / 4, f = 4 * (lane % q), rl = lane / q, nrl = 32 / q;
	for (unsigned r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < nregion; r += gridDim.x * (blockDim.x >> 5)) {
		const uint2 rg = reinterpret_cast<const uint2*>(R)[r];
		const size_t t = (size_t)r * nf + f;
		float4 d, x = make_float4(0.f, 0.f, 0.f, 0.f);
		if (ptype == DB_PT_ALL) {
			const float4 p0 = *reinterpret_cast<const float4*>(P + 2 * t), p1 = *reinterpret_cast<const float4*>(P + 2 * t + 4);
			x = make_float4(p0.x, p0.z, p1.x, p1.z); d = make_float4(p0.y, p0.w, p1.y, p1.w);
		} else
			d = *reinterpret_cast<const float4*>(P + t);
		if (ptype != DB_PT_SUM) {
			const float cnt = (float)(rg.y - rg.x);
			d.x /= cnt; d.y /= cnt; d.z /= cnt; d.w /= cnt;
		}
		float4* Uf = reinterpret_cast<float4*>(U + f);
		for (unsigned row = rg.x + rl; row < rg.y; row += nrl)
			atomicAdd(Uf + (size_t)row * q, d);
		if (ptype == DB_PT_ALL && rl == 0) {
			const uint4 a = *reinterpret_cast<const uint4*>(A + t);
			atomicAdd(&U[a.x], x.x); atomicAdd(&U[a.y], x.y); atomicAdd(&U[a.z], x.z); atomicAdd(&U[a.w], x.w);
		}
	}
}

// --------------------------------------------------------------- dropoutord
__global__ void dropoutord_kernel(const uint8_t* __restrict__ X, const float* __restrict__ U, uint64_t seed, uint64_t call,
                                  float rate, uint8_t* __restrict__ Z, uint8_t* __restrict__ M, size_t n)
{
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
		float u = U ? U[i] : uniform_01(seed, call, i);
		uint8_t x = X[i];
		bool mask = (x == 255) || (u >= rate);
		M[i] = mask;
		Z[i] = mask ? x : (uint8_t)254;
	}
}

static unsigned check_corr_options(const corr1ord_options_t* options)
{
	DB_REQUIRE(options != nullptr, "ValueError: options must not be NULL");
	DB_REQUIRE(options->nchannel == 4,
	           "NotImplementedError: The given number of channels does not have a matching pre-compiled kernel.");
	return options->nchannel;
}

static void dropoutord(const smat* X, const smat* U, smat* Z, smat* M, float rate)
{
	require_dtype(X, DB_U8, "X", "u8"); require_dtype(Z, DB_U8, "Z", "u8"); require_dtype(M, DB_B8, "M", "b8");
	DB_ASSERT(X->shape.x == Z->shape.x); DB_ASSERT(X->shape.y == Z->shape.y);
	DB_ASSERT(M->shape.x == X->shape.x); DB_ASSERT(M->shape.y == X->shape.y);
	const float* u = nullptr;
	if (U) { require_dtype(U, DB_F32, "U", "f32"); DB_ASSERT(size_of(U) == size_of(X)); u = (const float*)U->data; }
	size_t n = size_of(X);
	if (!n) return;
	uint64_t call = state().rng_calls++;
	dropoutord_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>((const uint8_t*)X->data, u, state().seed, call, rate,
	                                                              (uint8_t*)Z->data, (uint8_t*)M->data, n);
	DB_LAUNCH_CHECK();
}

}  // namespace db

using namespace db;

DB_EXPORT void api_corr1ord(const smat* W, const smat* X, smat* Z, const corr1ord_options_t* options)
{
	DB_API_TRY
	unsigned nchannel = check_corr_options(options);
	require_float(W, "W"); require_array(X, "X"); require_float(Z, "Z");
	DB_ASSERT(W->shape.y % nchannel == 0);
	DB_ASSERT(W->dtype == Z->dtype);
	DB_ASSERT(X->dtype == DB_U8);
	DB_ASSERT(Z->shape.x == W->shape.x);
	DB_ASSERT((size_t)Z->shape.y == size_of(X));
	unsigned m = W->shape.y / nchannel, nf = W->shape.x;
	if (size_of(X) < m) return;                      // no complete window: nothing is written
	unsigned n = (unsigned)size_of(X) - m + 1;      // rows actually written (kangaroo_smat.cpp:105)
	if (Z->dtype == DB_F32) launch_corr1ord_f32((const float*)W->data, m, nf, (const uint8_t*)X->data, n, (float*)Z->data);
	else                    launch_corr1ord((const double*)W->data, m, nf, (const uint8_t*)X->data, n, (double*)Z->data);
	DB_API_CATCH
}

DB_EXPORT void api_corr1ord_bprop_W(smat* dW, const smat* X, const smat* dZ, const corr1ord_options_t* options)
{
	DB_API_TRY
	unsigned nchannel = check_corr_options(options);
	require_float(dW, "dW"); require_array(X, "X"); require_float(dZ, "dZ");
	DB_ASSERT(dW->shape.y % nchannel == 0);
	DB_ASSERT(dW->dtype == dZ->dtype);
	DB_ASSERT(X->dtype == DB_U8);
	DB_ASSERT(dZ->shape.x == dW->shape.x);
	DB_ASSERT((size_t)dZ->shape.y == size_of(X));
	unsigned m = dW->shape.y / nchannel, nf = dW->shape.x;
	if (size_of(X) < m) return;
	unsigned n = (unsigned)size_of(X) - m + 1;
	if (dZ->dtype == DB_F32) launch_corr1ord_bprop_W_f32((float*)dW->data, m, nf, (const uint8_t*)X->data, n, (const float*)dZ->data);
	else                     launch_corr1ord_bprop_W((double*)dW->data, m, nf, (const uint8_t*)X->data, n, (const double*)dZ->data);
	DB_API_CATCH
}

DB_EXPORT void api_corr1ord_bprop_X(smat* dX, const smat* W, const smat* dZ, const corr1ord_options_t* options)
{
	DB_API_TRY
	unsigned nchannel = check_corr_options(options);
	require_float(dX, "dX"); require_float(W, "W"); require_float(dZ, "dZ");
	DB_ASSERT(W->shape.y % nchannel == 0);
	DB_ASSERT(W->dtype == dZ->dtype);
	DB_ASSERT(dX->dtype == dZ->dtype);
	DB_ASSERT((unsigned)dX->shape.x == nchannel);
	DB_ASSERT(dZ->shape.x == W->shape.x);
	DB_ASSERT(dZ->shape.y == dX->shape.y);
	unsigned m = W->shape.y / nchannel, nf = W->shape.x, n = dX->shape.y;
	if (n == 0 || nf == 0) return;
	unsigned grid = (unsigned)divup((size_t)n * 4, (size_t)128);
	if (dZ->dtype == DB_F32)
	{
		const size_t smem = ((size_t)4 * m * nf + (size_t)(BXR + m - 1) * (nf + 1)) * sizeof(float);
		if (smem <= 200 * 1024 && ((uintptr_t)dX->data & 15) == 0) {
			DB_CUDA(cudaFuncSetAttribute(corr1ord_bprop_X_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, (size_t)48 * 1024)));
			corr1ord_bprop_X_tiled_kernel<<<divup(n, (unsigned)BXR), BXR, smem, state().stream>>>((float*)dX->data, n, (const float*)W->data, m, nf, (const float*)dZ->data);
		} else
			corr1ord_bprop_X_kernel<<<grid, 128, 0, state().stream>>>((float*)dX->data, n, (const float*)W->data, m, nf, (const float*)dZ->data);
	}
	else
		corr1ord_bprop_X_kernel<<<grid, 128, 0, state().stream>>>((double*)dX->data, n, (const double*)W->data, m, nf, (const double*)dZ->data);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// Shape/dtype rules shared by api_poolrgn and api_poolrgn_bprop
// (kangaroo_smat.cpp:232-255,270-294), same messages.
static void check_pool_shapes(const smat* unpooled, const smat* regions, const smat* pooled, const smat* argmax,
                              const poolrgn_options_t* options, bool bprop)
{
	DB_REQUIRE(options != nullptr, "ValueError: options must not be NULL");
	require_float(unpooled, "unpooledmaps"); require_dtype(regions, DB_U32, "regions", "u32"); require_float(pooled, "pooledmaps");
	int nf = unpooled->shape.x, nregion = regions->shape.y, pt = options->ptype;
	DB_REQUIRE(pt >= DB_PT_MAX && pt <= DB_PT_ALL, "ValueError: unknown pooling type %d", pt);
	DB_REQUIRE(unpooled->dtype == pooled->dtype, bprop ? "TypeError: unpooledmaps dtype must match pooledmaps dtype."
	                                                   : "TypeError: featuremaps dtype must match pooledmaps dtype.");
	DB_REQUIRE(regions->shape.x == 2 || regions->shape.x == 3, "ValueError: regions array must have 2 or 3 columns.");
	if (pt == DB_PT_ALL)
		DB_REQUIRE(pooled->shape.x == 2 * nf, "ValueError: pooledmaps for \"all\" pooling must have twice as many columns as there are feature maps.");
	else
		DB_REQUIRE(pooled->shape.x == nf, "ValueError: pooledmaps must have as many columns as there are feature maps.");
	DB_REQUIRE(pooled->shape.y == nregion, "ValueError: pooledmaps must have as many rows as there are regions.");
	bool is_max = pt == DB_PT_MAX || pt == DB_PT_ALL;
	if (bprop && is_max)
		DB_REQUIRE(argmax != nullptr, "ValueError: pooledmaps_argmax must be specified for max pooling.");
	if (bprop && !is_max)
		DB_REQUIRE(argmax == nullptr, "ValueError: pooledmaps_argmax can only be specified for max pooling.");
	if (argmax) {
		DB_REQUIRE(is_max, "ValueError: pooledmaps_argmax can only be used for max/all pooling.");
		require_array(argmax, "pooledmaps_argmax");
		DB_REQUIRE(argmax->shape.x == nf, "ValueError: pooledmaps_argmax must have as many columns as there are feature maps.");
		DB_REQUIRE(argmax->dtype == DB_U32, "TypeError: pooledmaps_argmax dtype must be same type as uindex_t.");
		DB_REQUIRE(argmax->shape.y == nregion, "ValueError: pooledmaps_argmax must have as many rows as there are regions.");
	}
}

DB_EXPORT void api_poolrgn(const smat* unpooledmaps, const smat* regions, smat* pooledmaps, smat* pooledmaps_argmax,
                           const poolrgn_options_t* options)
{
	DB_API_TRY
	check_pool_shapes(unpooledmaps, regions, pooledmaps, pooledmaps_argmax, options, false);
	unsigned nf = unpooledmaps->shape.x, nregion = regions->shape.y;
	size_t n = (size_t)nf * nregion;
	if (!n) return;
	unsigned grid = (unsigned)divup(n, (size_t)128);
	uint32_t* A = pooledmaps_argmax ? (uint32_t*)pooledmaps_argmax->data : nullptr;
	const bool vec = unpooledmaps->dtype == DB_F32 && regions->shape.x == 2 && nf % 4 == 0 && nf <= 32 && 32 % nf == 0 &&
	                 ((uintptr_t)unpooledmaps->data & 15) == 0 && ((uintptr_t)regions->data & 7) == 0;
	if (vec) {
		const unsigned ncta = std::min(divup(nregion, (unsigned)PRW * (32u / nf)), 32u * (unsigned)state().sm_count);
#define DB_POOL_LAUNCH(NF_) poolrgn_warp_kernel<NF_, 16, 2><<<ncta, 32 * PRW, 0, state().stream>>>( \
			(const float*)unpooledmaps->data, (const uint32_t*)regions->data, nregion, (float*)pooledmaps->data, A, options->ptype)
		switch (nf) {
		case 4:  DB_POOL_LAUNCH(4); break;
		case 8:  DB_POOL_LAUNCH(8); break;
		case 16: DB_POOL_LAUNCH(16); break;
		default: DB_POOL_LAUNCH(32); break;
		}
#undef DB_POOL_LAUNCH
	}
	else if (unpooledmaps->dtype == DB_F32)
		poolrgn_kernel<<<grid, 128, 0, state().stream>>>((const float*)unpooledmaps->data, nf, (const uint32_t*)regions->data, nregion,
		                                                 (unsigned)regions->shape.x, (float*)pooledmaps->data, A, options->ptype);
	else
		poolrgn_kernel<<<grid, 128, 0, state().stream>>>((const double*)unpooledmaps->data, nf, (const uint32_t*)regions->data, nregion,
		                                                 (unsigned)regions->shape.x, (double*)pooledmaps->data, A, options->ptype);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void api_poolrgn_bprop(smat* unpooledmaps, const smat* regions, const smat* pooledmaps, const smat* pooledmaps_argmax,
                                 const poolrgn_options_t* options)
{
	DB_API_TRY
	check_pool_shapes(unpooledmaps, regions, pooledmaps, pooledmaps_argmax, options, true);
	unsigned nf = unpooledmaps->shape.x, nregion = regions->shape.y;
	size_t n = (size_t)nf * nregion;
	if (!n) return;
	unsigned grid = (unsigned)divup(n, (size_t)128);
	const uint32_t* A = pooledmaps_argmax ? (const uint32_t*)pooledmaps_argmax->data : nullptr;
	const bool aligned = (((uintptr_t)unpooledmaps->data | (uintptr_t)pooledmaps->data | (uintptr_t)A) & 15) == 0 &&
	                     ((uintptr_t)regions->data & 7) == 0;
	if (unpooledmaps->dtype == DB_F32 && options->ptype != DB_PT_MAX && regions->shape.x == 2 && nf % 4 == 0 && nf <= 128 &&
	    32 % (nf / 4) == 0 && aligned && (options->ptype != DB_PT_ALL || A)) {
		unsigned ncta = std::min(divup(nregion, 8u), 16u * (unsigned)state().sm_count);
		poolrgn_bprop_v4_kernel<<<ncta, 256, 0, state().stream>>>((float*)unpooledmaps->data, nf, (const uint32_t*)regions->data, nregion,
		                                                          (const float*)pooledmaps->data, A, options->ptype);
	} else if (unpooledmaps->dtype == DB_F32)
		poolrgn_bprop_kernel<<<grid, 128, 0, state().stream>>>((float*)unpooledmaps->data, nf, (const uint32_t*)regions->data, nregion,
		                                                       (unsigned)regions->shape.x, (const float*)pooledmaps->data, A, options->ptype);
	else
		poolrgn_bprop_kernel<<<grid, 128, 0, state().stream>>>((double*)unpooledmaps->data, nf, (const uint32_t*)regions->data, nregion,
		                                                       (unsigned)regions->shape.x, (const double*)pooledmaps->data, A, options->ptype);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void api_dropoutord_fp_tr(const smat* X, smat* Z, smat* M, float rate)
{
	DB_API_TRY
	dropoutord(X, nullptr, Z, M, rate);
	DB_API_CATCH
}

DB_EXPORT void api_dropoutord_fp_tr_u(const smat* X, const smat* U, smat* Z, smat* M, float rate)
{
	DB_API_TRY
	DB_REQUIRE(U != nullptr, "ValueError: argument U must not be NULL");
	dropoutord(X, U, Z, M, rate);
	DB_API_CATCH
}
