// Fused motif scan + bias + rectify + region pooling, forward and backward, in
// FP32 lookup-add form.  The per-position activation [npos, nf] that the
// reference writes and re-reads eight times per training step never leaves the
// SM: a CTA scans a tile of rows into shared memory and pools it there.
//
// Arithmetic is that of the reference chain, operator by operator:
//   scan      corr1ord.cuh:108-164   taps ascending from +0; N = ((W0+W1)+W2+W3)/4; 254 adds 0
//   bias      elemwise.py:171        Z + b
//   rectify   elemwise.py:74-78      max(0, .)
//   pooling   poolrgn.cuh:44-160     rows ascending; strict '>' (first maximum wins); running
//                                    sum in row order; mean = sum / integer row count
// so max, argmax, sum and mean agree with the unfused path bit for bit.
//
// Work split.  A CTA owns up to 8 regions (sequences) x FB filters.  In the scan
// phase a thread owns one row x 16 filters: a warp is 32 consecutive rows of the
// same 16 filters, so the 32 lanes read at most six distinct 16-byte entries of
// one 128-byte line of the lookup table (conflict-free, broadcast).  The table
// lut[tap][filter quad][code 0..7][4] holds W, the N mean and a zero row.  The
// scan is bound by the shared-memory return path (one 4-byte operand per add),
// not by FP32 issue; the ALU work around it is free.  In the pool phase a thread
// owns one (region, filter) column and walks the tile's rows in order.
//
// Backward, three kernels behind db_scanpool_bwd / api_corr1ord_bprop_W:
//   scanpool_bwd_kernel           mean and max+mean pooling: dZ rebuilt per tile from the
//                                 pooled deltas, argmax and activity bits, then dense one-hot
//                                 FMAs; the next tile's inputs arrive by cp.async meanwhile
//   scanpool_bwd_max_kernel       max pooling: only the argmax row of each (region, filter)
//   corr1ord_bprop_W_f32_kernel   the unfused operator: dZ streamed from HBM by cp.async
// All of them sum in a fixed order (rows, then CTAs or cluster ranks ascending): no float
// atomics, repeated runs agree bit for bit.
#include "db_common.cuh"
#include "scan_lut.cuh"
#include <cooperative_groups.h>

namespace db {

static constexpr int TR = 128;           // rows per tile
static constexpr int GMAX = TR / 16;     // regions per CTA (one pool thread per (region, filter))

__device__ __forceinline__ void cp_async4(void* dst, const void* src, unsigned src_bytes)
{
	// copies src_bytes (0..4) and zero-fills the rest of the 4 bytes
	asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;"
	             :: "r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes) : "memory");
}

struct fwd_args {
	const float* W; const float* bias; const uint8_t* X; const uint32_t* R;
	float* pooled; uint32_t* argmax; uint16_t* actmask;
	unsigned m, nf, npos, n, nregion, G, FB;
	int relu, ptype;
};

template <int M>
__global__ void __launch_bounds__(512)
scanpool_fwd_kernel(const fwd_args a)
{
	extern __shared__ __align__(16) unsigned char smem[];
	const unsigned m = M > 0 ? (unsigned)M : a.m;
	const unsigned FB = a.FB, NQ = FB / 4;
	float* lut = reinterpret_cast<float*>(smem);                       // m*NQ*32 floats
	float* act = lut + (size_t)m * NQ * 32;                            // FB*(TR+1) floats
	uint8_t* xs = reinterpret_cast<uint8_t*>(act + (size_t)FB * (TR + 1));   // TR + m + 8 bytes (4-aligned)
	__shared__ unsigned rg0[GMAX], rg1[GMAX], rcnt[GMAX];
	__shared__ unsigned s_lo, s_hi, s_sum;
	__shared__ __align__(16) float sbias[64];                          // FB <= 64

	const unsigned f0 = blockIdx.y * FB;
	const unsigned g0 = blockIdx.x * a.G;
	const unsigned ng = min(a.G, a.nregion - g0);
	// one thread per region fetches its bounds; the loads are in flight while the table is built
	unsigned my_r0 = 0, my_r1 = 0;
	if (threadIdx.x < ng) { my_r0 = a.R[2 * (g0 + threadIdx.x)]; my_r1 = a.R[2 * (g0 + threadIdx.x) + 1]; }
	build_lut(lut, a.W, m, a.nf, f0, FB);
	if (threadIdx.x < ng) {
		rcnt[threadIdx.x] = my_r1 - my_r0;                 // integer row count (poolrgn.cuh:112,152)
		rg0[threadIdx.x] = my_r0;
		rg1[threadIdx.x] = my_r1 <= my_r0 ? my_r0 + 1 : my_r1;   // an empty region still reads its first row (poolrgn.cuh:60)
	}
	__syncthreads();
	if (threadIdx.x == 0) {
		unsigned lo = 0xffffffffu, hi = 0, sum = 0;
		for (unsigned g = 0; g < ng; ++g) { lo = min(lo, rg0[g]); hi = max(hi, rg1[g]); sum += rg1[g] - rg0[g]; }
		s_lo = lo; s_hi = hi; s_sum = sum;
	}
	__syncthreads();
	// One span over all regions when they sit close together (the batch layout),
	// else one span per region.
	const bool one_span = (s_hi - s_lo) <= 2 * s_sum;
	const unsigned nspan = one_span ? 1 : ng;

	// scan-phase identity
	const unsigned rl = threadIdx.x % TR, fg = threadIdx.x / TR;
	const unsigned char* lutp = reinterpret_cast<const unsigned char*>(lut) + fg * 512;
	const unsigned stride = NQ * 128;
	// the block's biases wait in shared memory: sixteen registers less across the scan
	for (unsigned t = threadIdx.x; t < FB; t += blockDim.x) sbias[t] = (a.bias && f0 + t < a.nf) ? a.bias[f0 + t] : 0.f;
	// pool-phase identity and state
	const unsigned pg = threadIdx.x / FB, pf = threadIdx.x % FB;
	const bool pool_thread = pg < ng && f0 + pf < a.nf;
	float xmax = 0.f, xsum = 0.f; unsigned xidx = 0; bool started = false;

	// Two barriers per tile: the bases of tile i+1 are staged right after the pool phase of
	// tile i (whose scan, the last reader of xs[], ended at the barrier before that phase).
	auto store_x = [&](unsigned t0) {
		for (unsigned t = threadIdx.x; t < TR + m + 3; t += blockDim.x) {
			const unsigned i = t0 + t;
			xs[t] = (uint8_t)code16_of(i < a.npos ? a.X[i] : 254u);
		}
	};
	unsigned s = 0, t0 = one_span ? s_lo : rg0[0];
	for (;;) {
		const unsigned hi = one_span ? s_hi : rg1[s];
		store_x(t0);
		__syncthreads();
		{
			const unsigned row = t0 + rl;
			if (row < hi) {
				float z[16];
				if (row < a.n) scan_row<M>(lutp, stride, xs, rl, m, z);
				else {
					#pragma unroll
					for (int v = 0; v < 16; ++v) z[v] = 0.f;
				}
				unsigned bits = 0;
				float bv[16];
				#pragma unroll
				for (int v = 0; v < 16; v += 4) {
					const float4 q = *reinterpret_cast<const float4*>(sbias + fg * 16 + v);
					bv[v] = q.x; bv[v + 1] = q.y; bv[v + 2] = q.z; bv[v + 3] = q.w;
				}
				#pragma unroll
				for (int v = 0; v < 16; ++v) {
					float x = z[v];
					if (a.bias) x = x + bv[v];
					if (a.relu) x = x > 0.f ? x : 0.f;
					if (x > 0.f) bits |= 1u << v;
					act[(fg * 16 + v) * (TR + 1) + rl] = x;
				}
				if (a.actmask && f0 + fg * 16 < a.nf)
					a.actmask[(size_t)row * ((a.nf + 15) / 16) + (f0 / 16 + fg)] = (uint16_t)bits;
			}
			__syncthreads();
			if (pool_thread && (one_span || pg == s)) {
				unsigned r0 = max(rg0[pg], t0), r1 = min(rg1[pg], min(hi, t0 + TR));
				const float* col = act + pf * (TR + 1);
				for (unsigned r = r0; r < r1; ++r) {
					float v = col[r - t0];
					if (!started) { xmax = v; xidx = r; xsum = v; started = true; }
					else { if (v > xmax) { xmax = v; xidx = r; } xsum += v; }
				}
			}
		}
		t0 += TR;
		if (t0 >= hi) {
			if (++s >= nspan) break;
			t0 = rg0[s];
		}
	}
	if (pool_thread) {
		const unsigned g = g0 + pg, f = f0 + pf;
		const unsigned cnt = rcnt[pg];
		const size_t o = (size_t)g * a.nf + f;
		switch (a.ptype) {
		case DB_PT_MAX: a.pooled[o] = xmax; if (a.argmax) a.argmax[o] = xidx * a.nf + f; break;
		case DB_PT_AVG: a.pooled[o] = xsum / (float)cnt; break;
		case DB_PT_SUM: a.pooled[o] = xsum; break;
		default:
			reinterpret_cast<float2*>(a.pooled)[o] = make_float2(xmax, xsum / (float)cnt);
			if (a.argmax) a.argmax[o] = xidx * a.nf + f;
			break;
		}
	}
}

// ------------------------------------------------- the scan alone (api_corr1ord)
// The same row scan, writing Z [n, nf] instead of pooling it: what the unfused
// operator needs.  A thread owns one row x 16 filters and stores its 64 bytes of Z
// with four 16-byte stores; a CTA keeps its lookup table and walks the row tiles.
struct corr_args {
	const float* W; const uint8_t* X; float* Z;
	unsigned m, nf, npos, n, FB;
	int vec;                     // Z rows are 16-byte aligned at every 16-filter group
};

template <int M>
__global__ void __launch_bounds__(512)
corr1ord_f32_kernel(const corr_args a)
{
	extern __shared__ __align__(16) unsigned char smem[];
	const unsigned m = M > 0 ? (unsigned)M : a.m;
	const unsigned FB = a.FB, NQ = FB / 4;
	float* lut = reinterpret_cast<float*>(smem);                       // m*NQ*32 floats
	uint8_t* xs = reinterpret_cast<uint8_t*>(lut + (size_t)m * NQ * 32);      // TR + m + 8 bytes (4-aligned)
	const unsigned f0 = blockIdx.y * FB;
	build_lut(lut, a.W, m, a.nf, f0, FB);
	const unsigned rl = threadIdx.x % TR, fg = threadIdx.x / TR;
	const unsigned char* lutp = reinterpret_cast<const unsigned char*>(lut) + fg * 512;
	const unsigned stride = NQ * 128;
	const unsigned fbase = f0 + fg * 16;
	for (unsigned t0 = blockIdx.x * TR; t0 < a.n; t0 += gridDim.x * TR) {
		__syncthreads();
		for (unsigned t = threadIdx.x; t < TR + m + 3; t += blockDim.x) {
			unsigned i = t0 + t;
			xs[t] = (uint8_t)(i < a.npos ? code16_of(a.X[i]) : 80u);
		}
		__syncthreads();
		const unsigned row = t0 + rl;
		if (row < a.n && fbase < a.nf) {
			float z[16];
			scan_row<M>(lutp, stride, xs, rl, m, z);
			float* out = a.Z + (size_t)row * a.nf + fbase;
			if (a.vec && fbase + 16 <= a.nf) {
				#pragma unroll
				for (int v = 0; v < 16; v += 4)
					reinterpret_cast<float4*>(out)[v / 4] = make_float4(z[v], z[v + 1], z[v + 2], z[v + 3]);
			} else {
				#pragma unroll
				for (int v = 0; v < 16; ++v)
					if (fbase + v < a.nf) out[v] = z[v];
			}
		}
	}
}

void launch_corr1ord_f32(const float* W, unsigned m, unsigned nf, const uint8_t* X, unsigned n, float* Z)
{
	if (n == 0 || nf == 0 || m == 0) return;
	corr_args a;
	a.W = W; a.X = X; a.Z = Z; a.m = m; a.nf = nf; a.n = n; a.npos = n + m - 1;
	a.FB = nf <= 16 ? 16 : (nf <= 32 ? 32 : 64);
	while (a.FB > 16 && (size_t)m * a.FB * 32 > 120 * 1024) a.FB /= 2;
	DB_REQUIRE((size_t)m * a.FB * 32 <= 160 * 1024, "ValueError: filter length %u is too long for this kernel", m);
	a.vec = (nf % 4 == 0) && (((uintptr_t)Z & 15) == 0);
	size_t smem = (size_t)m * a.FB * 32 + TR + m + 16;
	unsigned tiles = divup(n, (unsigned)TR);
	dim3 grid(std::min(tiles, (unsigned)state().sm_count * 4), divup(nf, a.FB)), block(TR * a.FB / 16);
	auto launch = [&](auto kern) {
		DB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
		kern<<<grid, block, smem, state().stream>>>(a);
	};
	if (m == 24) launch(corr1ord_f32_kernel<24>);
	else if (m == 16) launch(corr1ord_f32_kernel<16>);
	else launch(corr1ord_f32_kernel<0>);
	DB_LAUNCH_CHECK();
}

// --------------------------------------------------------------- backward
// dZ[i,f] = active(i,f) ? (mean share of region(i) + (i is argmax ? max delta : 0)) : 0
// (poolrgn_bprop.cuh:45-127 then elemwise.py:78), dbias = column sums of dZ
// (elemwise.py:176), dW[(4j+k),f] = sum_i dZ[i,f] * [X[i+j]==k]  (+1/4 to all four
// channels for N; corr1ord_bprop.cuh:121-132).  Regions must be disjoint.
// A CTA owns up to 8 regions x FB filters: per tile of TR rows it rebuilds dZ in
// shared memory, then a thread per (group of four taps, filter) adds the tile's rows
// in order into 16 register accumulators: the row's dZ is read once for the four
// taps, and the channel weights of the four rows the taps look at slide through
// registers (one new 16-byte read per row), so the loop issues 16 FMAs for two
// shared-memory reads.  Per-CTA partials go to scratch and are added, CTA ascending,
// by a second kernel: fixed order, no float atomics.
struct bwd_args {
	const uint8_t* X; const uint32_t* R; const float* dpooled; const uint32_t* argmax; const uint16_t* actmask;
	float* partial;
	unsigned m, nf, npos, n, nregion, G, FB;
	int ptype;
	unsigned xaligned, maligned;     // X / actmask start on a 4-byte boundary: their tiles are fetched by cp.async
};

static constexpr int KMAX = 8;           // region groups one CTA of the backward kernel can be dealt

// Shared-memory views of the backward kernel.
struct bwd_smem {
	float* dz; float* davg; float* dmax; unsigned* amax; float4* oh; int* rowg;
	float* rdp; unsigned* ram; unsigned* rx; unsigned* rm;      // raw copies of the next tile's inputs
};

// Asynchronous copies of what group g0's pooling gradient needs: dpooled and argmax of
// its ng x FB (region, filter) pairs.
__device__ __forceinline__ void bwd_fetch_group(const bwd_args& a, const bwd_smem& sm, unsigned g0, unsigned ng,
                                                unsigned f0, unsigned logfb)
{
	const unsigned FB = 1u << logfb;
	for (unsigned t = threadIdx.x; t < (ng << logfb); t += blockDim.x) {
		const unsigned g = t >> logfb, f = f0 + (t & (FB - 1));
		if (f >= a.nf) continue;
		const size_t o = (size_t)(g0 + g) * a.nf + f;
		if (a.ptype == DB_PT_ALL) { cp_async4(sm.rdp + 2 * t, a.dpooled + 2 * o, 4); cp_async4(sm.rdp + 2 * t + 1, a.dpooled + 2 * o + 1, 4); }
		else cp_async4(sm.rdp + 2 * t, a.dpooled + o, 4);
		if (a.ptype == DB_PT_MAX || a.ptype == DB_PT_ALL) cp_async4(sm.ram + t, a.argmax + o, 4);
	}
}

// Asynchronous copies of a tile's bases (4-byte units from t0 on; X is 4-byte aligned
// on this path and t0 is rounded down) and of its activity words (the one or two
// 4-byte units that hold the CTA's FB bits of each row).
__device__ __forceinline__ void bwd_fetch_tile(const bwd_args& a, const bwd_smem& sm, unsigned t0, unsigned srows,
                                               unsigned f0, unsigned nwords, unsigned units)
{
	if (a.xaligned) {
		const unsigned b0 = t0 & ~3u, nunit = ((t0 & 3u) + TR + a.m + 4 + 3) / 4;
		for (unsigned w = threadIdx.x; w < nunit; w += blockDim.x) {
			const unsigned i = b0 + 4 * w;
			const unsigned left = i < a.npos ? min(4u, a.npos - i) : 0u;
			cp_async4(sm.rx + w, a.X + (left ? i : 0u), left);
		}
	}
	if (a.maligned) {
		const size_t total = (size_t)a.npos * nwords;
		for (unsigned t = threadIdx.x; t < srows * units; t += blockDim.x) {
			const unsigned r = units == 2 ? t >> 1 : t, u = units == 2 ? t & 1u : 0u;
			const size_t wi = ((size_t)(t0 + r) * nwords + (f0 >> 4)) & ~(size_t)1;       // first 16-bit word of the unit pair
			const size_t w = wi + 2 * u;
			const unsigned left = w < total ? (unsigned)min((size_t)2, total - w) * 2u : 0u;
			cp_async4(sm.rm + 2 * r + u, a.actmask + (left ? w : 0), left);
		}
	}
}

__global__ void __maxnreg__(56)
scanpool_bwd_kernel(const bwd_args a)
{
	extern __shared__ __align__(16) unsigned char smem[];
	const unsigned m = a.m, FB = a.FB;
	bwd_smem sm;
	sm.dz = reinterpret_cast<float*>(smem);                                // [TR][FB]
	sm.davg = sm.dz + (size_t)TR * FB;                                     // [GMAX][FB] mean share per row
	sm.dmax = sm.davg + GMAX * FB;                                         // [GMAX][FB]
	sm.amax = reinterpret_cast<unsigned*>(sm.dmax + GMAX * FB);            // [GMAX][FB] argmax row
	// per input row the weight each channel's gradient receives: one-hot, 1/4 each for N, 0 for a dropped base
	sm.oh = reinterpret_cast<float4*>(sm.amax + GMAX * FB);                // [TR + m + 4]
	sm.rowg = reinterpret_cast<int*>(sm.oh + TR + m + 4);                  // [TR] region of a row within the group, or -1
	sm.rdp = reinterpret_cast<float*>(sm.rowg + TR);                       // [GMAX][FB][2]
	sm.ram = reinterpret_cast<unsigned*>(sm.rdp + 2 * GMAX * FB);          // [GMAX][FB]
	sm.rm = sm.ram + GMAX * FB;                                            // [TR][2]
	sm.rx = sm.rm + 2 * TR;                                                // [(TR + m + 4 + 3) / 4 + 1]
	float* dz = sm.dz; float4* oh = sm.oh;
	__shared__ unsigned gb0[KMAX][GMAX], gb1[KMAX][GMAX], glo[KMAX], ghi[KMAX];

	const unsigned f0 = blockIdx.y * FB;
	// accumulator identity: unit u = (tap group jg, filter fl) covers taps 4jg .. 4jg+3.
	// The FB threads after the units sum dbias.
	const unsigned nunit = ((m + 3) / 4) * FB;
	const bool is_unit = threadIdx.x < nunit, is_bias = threadIdx.x >= nunit && threadIdx.x < nunit + FB;
	const unsigned logfb = FB == 16 ? 4 : 5;                            // FB is 16 or 32
	const unsigned j0 = 4 * (threadIdx.x >> logfb), fl = threadIdx.x & (FB - 1);
	float c[4][4];
	#pragma unroll
	for (int t = 0; t < 4; ++t)
		#pragma unroll
		for (int k = 0; k < 4; ++k) c[t][k] = 0.f;
	float bsum = 0.f;
	const unsigned nwords = (a.nf + 15) / 16, units = FB == 32 ? 2u : 1u;
	// staging identity: filter column fl, rows sr0, sr0 + srstep, ...  (the block size is a
	// multiple of FB, so the activity word and bit a thread tests are fixed)
	const unsigned sr0 = threadIdx.x >> logfb, srstep = blockDim.x >> logfb;
	const bool sfok = f0 + fl < a.nf;
	const unsigned swi = (f0 + fl) >> 4, ssh = (f0 + fl) & 15;

	// The CTA is dealt every gridDim.x-th region group (at most KMAX of them) and keeps its
	// accumulators over all of them: one partial result per CTA.  Their bounds come first,
	// in one round trip, so that every later load can be issued a tile ahead.
	const unsigned gstride = gridDim.x * a.G;
	unsigned K = 0;
	for (unsigned g0 = blockIdx.x * a.G; g0 < a.nregion && K < KMAX; g0 += gstride) ++K;
	for (unsigned t = threadIdx.x; t < K * GMAX; t += blockDim.x) {
		const unsigned k = t / GMAX, g = t % GMAX, rgn = blockIdx.x * a.G + k * gstride + g;
		const bool ok = g < a.G && rgn < a.nregion;
		gb0[k][g] = ok ? a.R[2 * rgn] : 0u;
		gb1[k][g] = ok ? a.R[2 * rgn + 1] : 0u;
	}
	__syncthreads();
	if (threadIdx.x < K) {
		unsigned lo = 0xffffffffu, hi = 0;
		for (unsigned g = 0; g < GMAX; ++g)
			if (gb1[threadIdx.x][g] > gb0[threadIdx.x][g]) { lo = min(lo, gb0[threadIdx.x][g]); hi = max(hi, gb1[threadIdx.x][g]); }
		glo[threadIdx.x] = lo; ghi[threadIdx.x] = hi;       // empty group: hi 0 <= lo
	}
	__syncthreads();

	// Turns the raw copies of tile (k, t0) into the tile's operands: channel weights oh,
	// the rows' regions, the group's pooling gradient (first tile of a group), then dZ.
	auto convert = [&](unsigned k, unsigned t0, bool first) {
		const unsigned g0 = blockIdx.x * a.G + k * gstride, ng = min(a.G, a.nregion - g0);
		const unsigned srows = min((unsigned)TR, ghi[k] - t0);
		for (unsigned t = threadIdx.x; t < TR + m + 4; t += blockDim.x) {
			const unsigned i = t0 + t;
			unsigned x = 254u;
			if (i < a.npos) x = a.xaligned ? reinterpret_cast<const uint8_t*>(sm.rx)[(t0 & 3u) + t] : a.X[i];
			const float q = (x >= 4u && x != 254u) ? 0.25f : 0.f;
			oh[t] = make_float4(x == 0u ? 1.f : q, x == 1u ? 1.f : q, x == 2u ? 1.f : q, x == 3u ? 1.f : q);
		}
		for (unsigned r = threadIdx.x; r < srows; r += blockDim.x) {
			const unsigned row = t0 + r;
			int g = -1;
			for (unsigned q = 0; q < ng; ++q) if (row >= gb0[k][q] && row < gb1[k][q]) g = (int)q;
			sm.rowg[r] = g;
		}
		if (first)
			for (unsigned t = threadIdx.x; t < (ng << logfb); t += blockDim.x) {
				const unsigned g = t >> logfb, f = f0 + (t & (FB - 1));
				float va = 0.f, vm = 0.f; unsigned am = 0xffffffffu;
				if (f < a.nf) {
					const float cnt = (float)(gb1[k][g] - gb0[k][g]);
					switch (a.ptype) {
					case DB_PT_MAX: vm = sm.rdp[2 * t]; am = sm.ram[t] / a.nf; break;
					case DB_PT_AVG: va = sm.rdp[2 * t] / cnt; break;
					case DB_PT_SUM: va = sm.rdp[2 * t]; break;
					default:        vm = sm.rdp[2 * t]; va = sm.rdp[2 * t + 1] / cnt; am = sm.ram[t] / a.nf; break;
					}
				}
				sm.davg[t] = va; sm.dmax[t] = vm; sm.amax[t] = am;
			}
		__syncthreads();
		#pragma unroll 2
		for (unsigned r = sr0; r < srows; r += srstep) {
			const unsigned row = t0 + r;
			const int g = sm.rowg[r];
			unsigned bits = 0;
			if (g >= 0 && sfok) {
				const size_t wi = (size_t)row * nwords + swi;
				bits = a.maligned ? reinterpret_cast<const uint16_t*>(sm.rm)[4 * r + (unsigned)(wi - (((size_t)row * nwords + (f0 >> 4)) & ~(size_t)1))]
				                  : (unsigned)a.actmask[wi];
			}
			float v = 0.f;
			if ((bits >> ssh) & 1u) {
				v = sm.davg[g * FB + fl];
				if (sm.amax[g * FB + fl] == row) v = v + sm.dmax[g * FB + fl];
			}
			dz[r * FB + fl] = v;
		}
		__syncthreads();
	};
	auto fetch = [&](unsigned k, unsigned t0, bool first) {
		const unsigned g0 = blockIdx.x * a.G + k * gstride;
		if (first) bwd_fetch_group(a, sm, g0, min(a.G, a.nregion - g0), f0, logfb);
		bwd_fetch_tile(a, sm, t0, min((unsigned)TR, ghi[k] - t0), f0, nwords, units);
		asm volatile("cp.async.commit_group;" ::: "memory");
	};

	unsigned k = 0;
	while (k < K && ghi[k] <= glo[k]) ++k;
	if (k < K) {
		unsigned t0 = glo[k];
		fetch(k, t0, true);
		asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		convert(k, t0, true);
		for (;;) {
			// the tile after this one: its copies fly while this one is accumulated
			unsigned nk = k, nt0 = t0 + TR;
			if (nt0 >= ghi[k]) {
				do ++nk; while (nk < K && ghi[nk] <= glo[nk]);
				nt0 = nk < K ? glo[nk] : 0u;
			}
			if (nk < K) fetch(nk, nt0, nk != k);
			// Rows at or past n have no scan output, hence no filter gradient; rows past the
			// last region of the group carry none either (and are not staged).
			const unsigned srows = min((unsigned)TR, ghi[k] - t0);
			const unsigned row_end = min(a.n, ghi[k]);
			const unsigned rows = min((unsigned)TR, row_end > t0 ? row_end - t0 : 0u);
			if (is_unit) {
				// Branch-free: the channel weights are 0, 1/4 or 1, so each product is exact and
				// the fused multiply-add equals the reference's add of dZ (or dZ/4).
				const float* dzc = dz + fl;
				const float4* ohj = oh + j0;
				float4 w0 = ohj[0], w1 = ohj[1], w2 = ohj[2], w3 = ohj[3];
				unsigned r = 0;
				for (; r + 4 <= rows; r += 4) {       // four rows per pass: the window rotates through its registers
					float v = dzc[(r + 0) * FB];
					bwd_fma4(c[0], v, w0); bwd_fma4(c[1], v, w1); bwd_fma4(c[2], v, w2); bwd_fma4(c[3], v, w3);
					w0 = ohj[r + 4];
					v = dzc[(r + 1) * FB];
					bwd_fma4(c[0], v, w1); bwd_fma4(c[1], v, w2); bwd_fma4(c[2], v, w3); bwd_fma4(c[3], v, w0);
					w1 = ohj[r + 5];
					v = dzc[(r + 2) * FB];
					bwd_fma4(c[0], v, w2); bwd_fma4(c[1], v, w3); bwd_fma4(c[2], v, w0); bwd_fma4(c[3], v, w1);
					w2 = ohj[r + 6];
					v = dzc[(r + 3) * FB];
					bwd_fma4(c[0], v, w3); bwd_fma4(c[1], v, w0); bwd_fma4(c[2], v, w1); bwd_fma4(c[3], v, w2);
					w3 = ohj[r + 7];
				}
				for (; r < rows; ++r) {
					const float v = dzc[r * FB];
					bwd_fma4(c[0], v, ohj[r]); bwd_fma4(c[1], v, ohj[r + 1]); bwd_fma4(c[2], v, ohj[r + 2]); bwd_fma4(c[3], v, ohj[r + 3]);
				}
			} else if (is_bias) {
				float s = bsum;
				for (unsigned r = 0; r < srows; ++r) s += dz[r * FB + fl];
				bsum = s;
			}
			asm volatile("cp.async.wait_group 0;" ::: "memory");
			__syncthreads();
			if (nk >= K) break;
			convert(nk, nt0, nk != k);
			k = nk; t0 = nt0;
		}
	}
	// partial[cta][(4m+1)][nf]; row 4m is dbias
	float* out = a.partial + (size_t)blockIdx.x * (4 * m + 1) * a.nf;
	if (is_unit && f0 + fl < a.nf) {
		#pragma unroll
		for (int t = 0; t < 4; ++t)
			if (j0 + t < m) {
				#pragma unroll
				for (int k2 = 0; k2 < 4; ++k2) out[(size_t)(4 * (j0 + t) + k2) * a.nf + f0 + fl] = c[t][k2];
			}
	}
	if (is_bias && f0 + fl < a.nf) out[(size_t)4 * m * a.nf + f0 + fl] = bsum;
}

// ---- max pooling alone: dZ has one nonzero row per (region, filter), the argmax row, so
// the dense accumulation above would add 0 for every other row.  Here a CTA stages, for a
// chunk of regions and FB filters, that row and its delta (0 when the unit was inactive
// there), and a thread per (four taps, filter) adds delta x channel weights
// of the four bases its taps see at that row; regions ascending, so the sums are the
// dense kernel's with the exact zeros left out.  One chunk: results go straight to dW
// and dbias; several: per-chunk partials, added by the second stage.
static constexpr int RC = 32;            // regions staged per round, at most

struct bwdmax_args {
	const uint8_t* X; const uint32_t* R; const float* dpooled; const uint32_t* argmax; const uint16_t* actmask;
	float* partial; float* dW; float* dbias;
	unsigned m, nf, npos, n, nregion, FB, rper, rc;  // rper: regions per chunk; rc: regions per round
	unsigned mode;                                   // 0: one chunk, results written directly; 1: per-chunk partials for
	                                                 // the second stage; 2: the chunks of a filter block form a cluster
	                                                 // and add their partials through distributed shared memory
};

__global__ void __launch_bounds__(512)
scanpool_bwd_max_kernel(const bwdmax_args a)
{
	extern __shared__ __align__(16) unsigned char smem[];       // [rc][FB][mp] bases under the taps at the argmax rows
	__shared__ float dval[RC * 32], dwv[RC * 32];               // delta for dbias; for dW (0 when the row has no scan output)
	const unsigned m = a.m, mp = (m + 3u) & ~3u, FB = a.FB, logfb = FB == 16 ? 4 : 5;
	const unsigned f0 = blockIdx.y * FB;
	const unsigned nunit = ((m + 3) / 4) * FB;
	const bool is_unit = threadIdx.x < nunit, is_bias = threadIdx.x >= nunit && threadIdx.x < nunit + FB;
	const unsigned j0 = 4 * (threadIdx.x >> logfb), fl = threadIdx.x & (FB - 1);
	const unsigned nwords = (a.nf + 15) / 16;
	float c[4][4];
	#pragma unroll
	for (int t = 0; t < 4; ++t)
		#pragma unroll
		for (int k = 0; k < 4; ++k) c[t][k] = 0.f;
	float bsum = 0.f;
	const unsigned gbeg = blockIdx.x * a.rper, gend = min(a.nregion, gbeg + a.rper);
	for (unsigned g0 = gbeg; g0 < gend; g0 += a.rc) {
		const unsigned ng = min(a.rc, gend - g0);
		__syncthreads();
		for (unsigned t = threadIdx.x; t < (ng << logfb); t += blockDim.x) {
			const unsigned g = g0 + (t >> logfb), f = f0 + (t & (FB - 1));
			float d = 0.f; unsigned row = 0;
			if (f < a.nf) {
				const size_t o = (size_t)g * a.nf + f;
				const float dp = a.dpooled[o];                       // independent of the row: in flight with argmax
				row = a.argmax[o] / a.nf;
				const unsigned bits = a.actmask[(size_t)row * nwords + (f >> 4)];
				if ((bits >> (f & 15)) & 1u) d = dp;                 // an empty region's delta lands on its recorded row too (poolrgn_bprop.cuh:57)
			}
			const bool scanned = row < a.n;                      // rows at or past n have no scan output
			dval[t] = d; dwv[t] = scanned ? d : 0.f;
			if (scanned && d != 0.f) {
				unsigned char* w = smem + (size_t)t * mp;
				for (unsigned j = 0; j < m; ++j) w[j] = a.X[row + j];
			}
		}
		__syncthreads();
		if (is_unit) {
			for (unsigned g = 0; g < ng; ++g) {
				const unsigned t = (g << logfb) + fl;
				const float d = dwv[t];
				if (d == 0.f) continue;
				const unsigned xw = *reinterpret_cast<const unsigned*>(smem + (size_t)t * mp + j0);
				#pragma unroll
				for (int k = 0; k < 4; ++k)
					if (j0 + k < m) {
						const unsigned x = (xw >> (8 * k)) & 0xffu;
						const float q = (x >= 4u && x != 254u) ? 0.25f : 0.f;
						c[k][0] = fmaf(d, x == 0u ? 1.f : q, c[k][0]); c[k][1] = fmaf(d, x == 1u ? 1.f : q, c[k][1]);
						c[k][2] = fmaf(d, x == 2u ? 1.f : q, c[k][2]); c[k][3] = fmaf(d, x == 3u ? 1.f : q, c[k][3]);
					}
			}
		} else if (is_bias) {
			float s = bsum;
			for (unsigned g = 0; g < ng; ++g) s += dval[(g << logfb) + fl];
			bsum = s;
		}
	}
	if (a.mode == 2) {
		namespace cg = cooperative_groups;
		cg::cluster_group cluster = cg::this_cluster();
		__syncthreads();                                     // the staged bases are no longer read
		float* part = reinterpret_cast<float*>(smem);        // [(4m+1)][FB], row 4m = dbias
		if (is_unit) {
			#pragma unroll
			for (int t = 0; t < 4; ++t)
				if (j0 + t < m) {
					#pragma unroll
					for (int k = 0; k < 4; ++k) part[((4 * (j0 + t) + k) << logfb) + fl] = c[t][k];
				}
		}
		if (is_bias) part[((4 * m) << logfb) + fl] = bsum;
		cluster.sync();
		// CTA `rank` finishes a slice of the block's outputs, chunks (= ranks) ascending
		const unsigned C = cluster.num_blocks(), rank = cluster.block_rank();
		const unsigned total = (4 * m + 1) << logfb, S = (total + C - 1) / C;
		for (unsigned j = rank * S + threadIdx.x; j < min(total, (rank + 1) * S); j += blockDim.x) {
			float s = 0.f;
			for (unsigned q = 0; q < C; ++q) s += cluster.map_shared_rank(part, q)[j];
			const unsigned row = j >> logfb, f = f0 + (j & (FB - 1));
			if (f < a.nf) {
				if (row < 4 * m) a.dW[(size_t)row * a.nf + f] = s;
				else if (a.dbias) a.dbias[f] = s;
			}
		}
		cluster.sync();                                      // nobody leaves while its partials are being read
		return;
	}
	// one chunk: the results themselves; else partial[chunk][(4m+1)][nf], row 4m = dbias
	const bool direct = a.mode == 0;
	float* out = direct ? a.dW : a.partial + (size_t)blockIdx.x * (4 * m + 1) * a.nf;
	if (is_unit && f0 + fl < a.nf) {
		#pragma unroll
		for (int t = 0; t < 4; ++t)
			if (j0 + t < m) {
				#pragma unroll
				for (int k = 0; k < 4; ++k) out[(size_t)(4 * (j0 + t) + k) * a.nf + f0 + fl] = c[t][k];
			}
	}
	if (is_bias && f0 + fl < a.nf) {
		if (!direct) out[(size_t)4 * m * a.nf + f0 + fl] = bsum;
		else if (a.dbias) a.dbias[f0 + fl] = bsum;
	}
}

// Second stage: sums the per-CTA partial gradients in a fixed order.  A CTA of eight
// warps owns 32 consecutive outputs (one coalesced row segment per part); warp w
// adds the parts w, w+8, ... with four independent chains, and warp 0 combines the
// eight sums.  The order depends on `nparts` only, so repeated runs agree bit for bit.
__global__ void __launch_bounds__(256)
scanpool_bwd_reduce(float* __restrict__ dW, float* __restrict__ dbias, const float* __restrict__ partial,
                    size_t wcount, unsigned nf, unsigned nparts, int accumulate)
{
	__shared__ float part[8][32];
	const size_t total = wcount + nf;
	const unsigned lane = threadIdx.x & 31, w = threadIdx.x >> 5;
	for (size_t base = (size_t)blockIdx.x * 32; base < total; base += (size_t)gridDim.x * 32) {
		const size_t i = base + lane;
		float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
		if (i < total) {
			const float* P = partial + i;
			unsigned p = w;
			for (; p + 24 < nparts; p += 32) {
				s0 += P[(size_t)p * total]; s1 += P[(size_t)(p + 8) * total];
				s2 += P[(size_t)(p + 16) * total]; s3 += P[(size_t)(p + 24) * total];
			}
			for (; p < nparts; p += 8) s0 += P[(size_t)p * total];
		}
		part[w][lane] = (s0 + s1) + (s2 + s3);
		__syncthreads();
		if (w == 0 && i < total) {
			const float s = ((part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane])) +
			                ((part[4][lane] + part[5][lane]) + (part[6][lane] + part[7][lane]));
			if (i < wcount) dW[i] = accumulate ? dW[i] + s : s; else if (dbias) dbias[i - wcount] = s;
		}
		__syncthreads();
	}
}

// Few partials: a thread per output reads them all at once (independent, coalesced
// loads), four chains over parts p mod 4.  Again the order depends on `nparts` only.
__global__ void __launch_bounds__(256)
scanpool_bwd_reduce_few(float* __restrict__ dW, float* __restrict__ dbias, const float* __restrict__ partial,
                        size_t wcount, unsigned nf, unsigned nparts, int accumulate)
{
	const size_t total = wcount + nf;
	const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
	if (i >= total) return;
	const float* P = partial + i;
	float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
	unsigned p = 0;
	#pragma unroll 4
	for (; p + 4 <= nparts; p += 4) {
		s0 += P[(size_t)p * total]; s1 += P[(size_t)(p + 1) * total];
		s2 += P[(size_t)(p + 2) * total]; s3 += P[(size_t)(p + 3) * total];
	}
	for (; p < nparts; ++p) s0 += P[(size_t)p * total];
	const float s = (s0 + s1) + (s2 + s3);
	if (i < wcount) dW[i] = accumulate ? dW[i] + s : s; else if (dbias) dbias[i - wcount] = s;
}

static void launch_bwd_reduce(float* dW, float* dbias, const float* partial, size_t wcount, unsigned nf, unsigned nparts, int accumulate)
{
	const size_t total = wcount + nf;
	if (nparts <= 64 && total >= 8192)
		scanpool_bwd_reduce_few<<<(unsigned)divup(total, (size_t)256), 256, 0, state().stream>>>(dW, dbias, partial, wcount, nf, nparts, accumulate);
	else
		scanpool_bwd_reduce<<<(unsigned)std::min<size_t>(divup(total, (size_t)32), 65535), 256, 0, state().stream>>>(dW, dbias, partial, wcount, nf, nparts, accumulate);
	DB_LAUNCH_CHECK();
}

// ----------------------------------- the filter gradient alone (api_corr1ord_bprop_W)
// dW[(4j+k), f] += sum_i dZ[i, f] * [X[i+j] == k]  (+1/4 on all four channels for N;
// corr1ord_bprop.cuh:91-138) from a dZ that lives in HBM: the accumulation loop of
// the fused backward kernel, fed by coalesced tiles of dZ.  A CTA keeps its 16
// accumulators per thread over every TR-row tile it is dealt and writes one partial
// result; the second stage adds the partials, CTA ascending, into dW.
struct bpw_args {
	const uint8_t* X; const float* dZ; float* partial;
	unsigned m, nf, n, npos, FB, logfb, vec;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, unsigned src_bytes)
{
	// src_bytes 0: nothing is read and the 16 bytes are zero-filled
	asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
	             :: "r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(src_bytes) : "memory");
}

// Tile t0 of dZ into dzb[TR][FB]: 16-byte asynchronous copies when rows of dZ are
// 16-byte aligned (a.vec), else plain loads.
__device__ __forceinline__ void bpw_stage_dz(const bpw_args& a, unsigned t0, unsigned f0, float* dzb)
{
	const unsigned rows = min((unsigned)TR, a.n - t0);
	if (a.vec) {
		const unsigned lq = a.logfb - 2, q = 1u << lq;
		for (unsigned t = threadIdx.x; t < (unsigned)TR << lq; t += blockDim.x) {
			const unsigned r = t >> lq, e = (t & (q - 1)) * 4;
			const bool ok = r < rows && f0 + e < a.nf;
			cp_async16(dzb + (r << a.logfb) + e, ok ? a.dZ + (size_t)(t0 + r) * a.nf + f0 + e : a.dZ, ok ? 16u : 0u);
		}
	} else {
		for (unsigned t = threadIdx.x; t < (unsigned)TR << a.logfb; t += blockDim.x) {
			const unsigned r = t >> a.logfb, e = t & (a.FB - 1);
			dzb[t] = (r < rows && f0 + e < a.nf) ? a.dZ[(size_t)(t0 + r) * a.nf + f0 + e] : 0.f;
		}
	}
	asm volatile("cp.async.commit_group;" ::: "memory");
}

static constexpr int BPW_XB = 3;          // bases a thread carries for the next tile: (TR + m + 4) <= 3 * 128

__device__ __forceinline__ void bpw_load_x(const bpw_args& a, unsigned t0, unsigned (&xb)[BPW_XB])
{
	#pragma unroll
	for (int k = 0; k < BPW_XB; ++k) {
		const unsigned i = t0 + threadIdx.x + k * blockDim.x;
		xb[k] = (threadIdx.x + k * blockDim.x < TR + a.m + 4 && i < a.npos) ? a.X[i] : 254u;
	}
}

__device__ __forceinline__ void bpw_store_oh(const bpw_args& a, const unsigned (&xb)[BPW_XB], float4* ohb)
{
	#pragma unroll
	for (int k = 0; k < BPW_XB; ++k) {
		const unsigned t = threadIdx.x + k * blockDim.x, x = xb[k];
		if (t < TR + a.m + 4) {
			const float q = (x >= 4u && x != 254u) ? 0.25f : 0.f;
			ohb[t] = make_float4(x == 0u ? 1.f : q, x == 1u ? 1.f : q, x == 2u ? 1.f : q, x == 3u ? 1.f : q);
		}
	}
}

__global__ void __launch_bounds__(512)
corr1ord_bprop_W_f32_kernel(const bpw_args a)
{
	extern __shared__ __align__(16) unsigned char smem[];
	const unsigned m = a.m, FB = a.FB, noh = TR + m + 4;
	float* dz = reinterpret_cast<float*>(smem);                             // [2][TR][FB]
	float4* oh = reinterpret_cast<float4*>(dz + 2 * (size_t)TR * FB);       // [2][TR + m + 4]
	const unsigned f0 = blockIdx.y * FB;
	const unsigned nunit = ((m + 3) / 4) * FB;
	const bool is_unit = threadIdx.x < nunit;
	const unsigned j0 = 4 * (threadIdx.x >> a.logfb), fl = threadIdx.x & (FB - 1);
	float c[4][4];
	#pragma unroll
	for (int t = 0; t < 4; ++t)
		#pragma unroll
		for (int k = 0; k < 4; ++k) c[t][k] = 0.f;
	const unsigned stride = gridDim.x * TR;
	unsigned xb[BPW_XB];
	unsigned t0 = blockIdx.x * TR, buf = 0;
	// Two buffers: while a tile is accumulated, the copies of the CTA's next tile are in
	// flight and its bases wait in registers (turned into channel weights once the
	// accumulation is done, when their loads have long returned).
	if (t0 < a.n) {
		bpw_stage_dz(a, t0, f0, dz);
		bpw_load_x(a, t0, xb);
		bpw_store_oh(a, xb, oh);
	}
	for (; t0 < a.n; t0 += stride, buf ^= 1) {
		const unsigned next = t0 + stride;           // stride < 2^31 and n < 2^32 - stride: checked by the launcher
		const bool more = next < a.n;
		if (more) {
			bpw_stage_dz(a, next, f0, dz + (buf ^ 1) * (size_t)TR * FB);
			bpw_load_x(a, next, xb);
			asm volatile("cp.async.wait_group 1;" ::: "memory");
		} else
			asm volatile("cp.async.wait_group 0;" ::: "memory");
		__syncthreads();
		const unsigned rows = min((unsigned)TR, a.n - t0);
		if (is_unit) {
			const float* dzc = dz + buf * (size_t)TR * FB + fl;
			const float4* ohj = oh + buf * noh + j0;
			float4 w0 = ohj[0], w1 = ohj[1], w2 = ohj[2], w3 = ohj[3];
			unsigned r = 0;
			for (; r + 4 <= rows; r += 4) {
				float v = dzc[(r + 0) * FB];
				bwd_fma4(c[0], v, w0); bwd_fma4(c[1], v, w1); bwd_fma4(c[2], v, w2); bwd_fma4(c[3], v, w3);
				w0 = ohj[r + 4];
				v = dzc[(r + 1) * FB];
				bwd_fma4(c[0], v, w1); bwd_fma4(c[1], v, w2); bwd_fma4(c[2], v, w3); bwd_fma4(c[3], v, w0);
				w1 = ohj[r + 5];
				v = dzc[(r + 2) * FB];
				bwd_fma4(c[0], v, w2); bwd_fma4(c[1], v, w3); bwd_fma4(c[2], v, w0); bwd_fma4(c[3], v, w1);
				w2 = ohj[r + 6];
				v = dzc[(r + 3) * FB];
				bwd_fma4(c[0], v, w3); bwd_fma4(c[1], v, w0); bwd_fma4(c[2], v, w1); bwd_fma4(c[3], v, w2);
				w3 = ohj[r + 7];
			}
			for (; r < rows; ++r) {
				const float v = dzc[r * FB];
				bwd_fma4(c[0], v, ohj[r]); bwd_fma4(c[1], v, ohj[r + 1]); bwd_fma4(c[2], v, ohj[r + 2]); bwd_fma4(c[3], v, ohj[r + 3]);
			}
		}
		if (more) bpw_store_oh(a, xb, oh + (buf ^ 1) * noh);
		__syncthreads();
	}
	float* out = a.partial + (size_t)blockIdx.x * 4 * m * a.nf;
	if (is_unit && f0 + fl < a.nf) {
		#pragma unroll
		for (int t = 0; t < 4; ++t)
			if (j0 + t < m) {
				#pragma unroll
				for (int k = 0; k < 4; ++k) out[(size_t)(4 * (j0 + t) + k) * a.nf + f0 + fl] = c[t][k];
			}
	}
}

void launch_corr1ord_bprop_W_f32(float* dW, unsigned m, unsigned nf, const uint8_t* X, unsigned n, const float* dZ)
{
	if (n == 0 || nf == 0 || m == 0) return;
	bpw_args a;
	a.X = X; a.dZ = dZ; a.m = m; a.nf = nf; a.n = n; a.npos = n + m - 1;
	a.FB = nf <= 16 ? 16 : 32;
	while (a.FB > 16 && ((m + 3) / 4) * a.FB > 512) a.FB /= 2;
	a.logfb = a.FB == 16 ? 4 : 5;
	a.vec = (nf % 4 == 0 && ((uintptr_t)dZ & 15) == 0) ? 1u : 0u;
	unsigned threads = (((m + 3) / 4) * a.FB + 31u) & ~31u;
	DB_REQUIRE(threads <= 512, "ValueError: filter length %u is too long for this kernel", m);
	if (threads < 128) threads = 128;
	DB_REQUIRE((unsigned)TR + m + 4 <= BPW_XB * threads, "ValueError: filter length %u is too long for this kernel", m);
	unsigned nfb = divup(nf, a.FB);
	size_t smem = 2 * ((size_t)TR * a.FB * 4 + (size_t)(TR + m + 4) * 16);
	DB_CUDA(cudaFuncSetAttribute(corr1ord_bprop_W_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	int per_sm = 1;
	DB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, corr1ord_bprop_W_f32_kernel, (int)threads, smem));
	// one resident wave; no more than 16 warps an SM, which keep the FMA pipes busy once the
	// copies overlap the arithmetic, so that the second stage has few partials to add
	per_sm = std::max(1, std::min(per_sm, (int)(512 / threads)));
	unsigned slots = (unsigned)state().sm_count * (unsigned)per_sm;
	unsigned ncta = std::min(divup(n, (unsigned)TR), std::max(1u, slots / nfb));
	DB_REQUIRE((uint64_t)n + (uint64_t)ncta * TR < (1ull << 32), "ValueError: too many rows (%u) for this kernel", n);
	size_t wcount = (size_t)4 * m * nf;
	a.partial = (float*)scratch((size_t)ncta * wcount * sizeof(float));
	corr1ord_bprop_W_f32_kernel<<<dim3(ncta, nfb), threads, smem, state().stream>>>(a);
	DB_LAUNCH_CHECK();
	launch_bwd_reduce(dW, nullptr, a.partial, wcount, 0, ncta, 1);
}

static unsigned pick_fb(unsigned nf, unsigned m, size_t per_filter_bytes, size_t budget)
{
	unsigned FB = nf <= 16 ? 16 : (nf <= 32 ? 32 : 64);
	while (FB > 16 && (size_t)m * FB * per_filter_bytes > budget) FB /= 2;
	return FB;
}

// Resident CTAs per SM of a forward kernel instance, remembered per (kernel, m, FB).
template <typename K>
static unsigned fwd_ctas_per_sm(K kern, unsigned m, unsigned FB, size_t smem)
{
	struct entry { const void* k; unsigned m, FB, per_sm; };
	static entry cache[16];
	static unsigned used = 0;
	for (unsigned i = 0; i < used; ++i)
		if (cache[i].k == (const void*)kern && cache[i].m == m && cache[i].FB == FB) return cache[i].per_sm;
	int per_sm = 1;
	DB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	DB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, (int)(TR * FB / 16), smem));
	per_sm = std::max(per_sm, 1);
	if (used < 16) cache[used++] = entry{(const void*)kern, m, FB, (unsigned)per_sm};
	return (unsigned)per_sm;
}

}  // namespace db

using namespace db;

DB_EXPORT void db_scanpool_fwd(const float* W, uint32_t m, uint32_t nf, const float* bias, int relu,
                               const uint8_t* X, uint32_t npos, const uint32_t* regions, uint32_t nregion,
                               int ptype, float* pooled, uint32_t* argmax, uint16_t* actmask)
{
	DB_API_TRY
	DB_REQUIRE(ptype >= DB_PT_MAX && ptype <= DB_PT_ALL, "ValueError: unknown pooling type %d", ptype);
	DB_REQUIRE(m > 0 && nf > 0, "ValueError: filter bank must not be empty (m=%u, nf=%u)", m, nf);
	DB_REQUIRE(!argmax || ptype == DB_PT_MAX || ptype == DB_PT_ALL, "ValueError: pooledmaps_argmax can only be used for max/all pooling.");
	if (nregion == 0) return;
	DB_REQUIRE(W && X && regions && pooled, "ValueError: db_scanpool_fwd got a NULL pointer");
	fwd_args a;
	a.W = W; a.bias = bias; a.X = X; a.R = regions; a.pooled = pooled; a.argmax = argmax; a.actmask = actmask;
	a.m = m; a.nf = nf; a.npos = npos; a.n = npos >= m ? npos - m + 1 : 0; a.nregion = nregion;
	a.relu = relu; a.ptype = ptype;
	const unsigned fbmax = pick_fb(nf, m, 32, 120 * 1024);
	DB_REQUIRE((size_t)m * fbmax * 32 <= 160 * 1024, "ValueError: filter length %u is too long for the fused kernel", m);
	auto smem_of = [&](unsigned FB) { return (size_t)m * FB * 32 + (size_t)FB * (TR + 1) * 4 + TR + m + 16; };
	auto run = [&](auto kern) {
		// Filters per CTA and regions per CTA: the pair with the least work on the busiest SM,
		// a CTA costing its rows plus a fixed share (table build, first loads).  Small batches
		// then run as one well-filled resident wave instead of one and a bit.
		const double rpr = std::max(1u, npos / nregion);
		double best = 0; a.FB = 0; a.G = 1;
		for (unsigned FB = fbmax; FB >= 16; FB /= 2) {
			const unsigned per_sm = fwd_ctas_per_sm(kern, m, FB, smem_of(FB));
			const size_t nfb = divup(nf, FB);
			for (unsigned G = GMAX; G >= 1; --G) {
				const size_t ncta = (size_t)divup(nregion, G) * nfb;
				const size_t load = divup(ncta, (size_t)state().sm_count);
				const double cost = (double)load * FB * (G * rpr + 100.0) * (load > per_sm ? 1.15 : 1.0);
				if (a.FB == 0 || cost < best) { best = cost; a.FB = FB; a.G = G; }
			}
		}
		const size_t smem = smem_of(a.FB);
		dim3 grid(divup(nregion, a.G), divup(nf, a.FB)), block(TR * a.FB / 16);
		DB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_of(fbmax)));
		kern<<<grid, block, smem, state().stream>>>(a);
	};
	if (m == 24) run(scanpool_fwd_kernel<24>);
	else if (m == 16) run(scanpool_fwd_kernel<16>);
	else run(scanpool_fwd_kernel<0>);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_scanpool_bwd(uint32_t m, uint32_t nf, const uint8_t* X, uint32_t npos,
                               const uint32_t* regions, uint32_t nregion, int ptype,
                               const float* dpooled, const uint32_t* argmax, const uint16_t* actmask,
                               float* dW, float* dbias)
{
	DB_API_TRY
	DB_REQUIRE(ptype >= DB_PT_MAX && ptype <= DB_PT_ALL, "ValueError: unknown pooling type %d", ptype);
	DB_REQUIRE(m > 0 && nf > 0, "ValueError: filter bank must not be empty (m=%u, nf=%u)", m, nf);
	DB_REQUIRE(dW != nullptr, "ValueError: db_scanpool_bwd needs dW");
	size_t wcount = (size_t)4 * m * nf;
	if (nregion == 0) {
		DB_CUDA(cudaMemsetAsync(dW, 0, wcount * 4, state().stream));
		if (dbias) DB_CUDA(cudaMemsetAsync(dbias, 0, (size_t)nf * 4, state().stream));
		return;
	}
	DB_REQUIRE(X && regions && dpooled && actmask, "ValueError: db_scanpool_bwd got a NULL pointer");
	DB_REQUIRE(argmax || (ptype != DB_PT_MAX && ptype != DB_PT_ALL), "ValueError: pooledmaps_argmax must be specified for max pooling.");
	if (ptype == DB_PT_MAX) {
		bwdmax_args x;
		x.X = X; x.R = regions; x.dpooled = dpooled; x.argmax = argmax; x.actmask = actmask; x.dW = dW; x.dbias = dbias;
		x.m = m; x.nf = nf; x.npos = npos; x.n = npos >= m ? npos - m + 1 : 0; x.nregion = nregion;
		x.FB = nf <= 16 ? 16 : 32;
		while (x.FB > 16 && ((m + 3) / 4 + 1) * x.FB > 512) x.FB /= 2;
		const unsigned nfb = divup(nf, x.FB);
		unsigned threads = (((m + 3) / 4 + 1) * x.FB + 31u) & ~31u;
		DB_REQUIRE(threads <= 512, "ValueError: filter length %u is too long for the fused backward kernel", m);
		// Chunks of at least eight regions (about one staged (region, filter) pair per thread, so that
		// the dependent loads argmax -> activity word, bases of all pairs are in flight together),
		// no more than fill the GPU four CTAs deep.
		unsigned nchunk = std::max(1u, std::min(nregion / 8, divup(4u * (unsigned)state().sm_count, nfb)));
		x.rper = divup(nregion, nchunk);
		nchunk = divup(nregion, x.rper);
		x.mode = nchunk == 1 ? 0u : (nchunk <= 8 ? 2u : 1u);
		x.partial = x.mode == 1 ? (float*)scratch((size_t)nchunk * (wcount + nf) * sizeof(float)) : nullptr;
		const unsigned mp = (m + 3u) & ~3u;
		x.rc = std::max(1u, std::min((unsigned)RC, (unsigned)(64 * 1024 / ((size_t)x.FB * mp))));
		const size_t smem = std::max((size_t)x.rc * x.FB * mp, (size_t)(4 * m + 1) * x.FB * sizeof(float));
		DB_CUDA(cudaFuncSetAttribute(scanpool_bwd_max_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, (size_t)48 * 1024)));
		if (x.mode == 2) {
			cudaLaunchConfig_t cfg = {};
			cfg.gridDim = dim3(nchunk, nfb); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem; cfg.stream = state().stream;
			cudaLaunchAttribute attr[1];
			attr[0].id = cudaLaunchAttributeClusterDimension;
			attr[0].val.clusterDim.x = nchunk; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
			cfg.attrs = attr; cfg.numAttrs = 1;
			DB_CUDA(cudaLaunchKernelEx(&cfg, scanpool_bwd_max_kernel, x));
		} else
			scanpool_bwd_max_kernel<<<dim3(nchunk, nfb), threads, smem, state().stream>>>(x);
		DB_LAUNCH_CHECK();
		if (x.mode == 1) launch_bwd_reduce(dW, dbias, x.partial, wcount, nf, nchunk, 0);
		return;
	}
	bwd_args a;
	a.X = X; a.R = regions; a.dpooled = dpooled; a.argmax = argmax; a.actmask = actmask;
	a.m = m; a.nf = nf; a.npos = npos; a.n = npos >= m ? npos - m + 1 : 0; a.nregion = nregion; a.ptype = ptype;
	a.FB = nf <= 16 ? 16 : 32;          // 32 filters per CTA: several CTAs per SM, whose staging and FMA phases overlap
	while (a.FB > 16 && ((m + 3) / 4 + 1) * a.FB > 512) a.FB /= 2;
	unsigned nfb = divup(nf, a.FB);
	unsigned threads = (((m + 3) / 4 + 1) * a.FB + 31u) & ~31u;       // one thread per (four taps, filter) and per bias column
	DB_REQUIRE(threads <= 512, "ValueError: filter length %u is too long for the fused backward kernel", m);
	if (threads < 128) threads = 128;
	// Regions per group: about one tile of rows.  CTAs per filter block: as many as are resident
	// at once, each looping over its share of the groups, so that no second, part-filled wave runs.
	a.G = std::max(1u, std::min((unsigned)GMAX, (unsigned)TR / std::max(1u, npos / nregion)));
	a.xaligned = ((uintptr_t)X & 3) == 0; a.maligned = ((uintptr_t)actmask & 3) == 0;
	size_t smem = (size_t)TR * a.FB * 4 + (size_t)GMAX * a.FB * 12 + (size_t)(TR + m + 4) * 16 + (size_t)TR * 4 +
	              (size_t)GMAX * a.FB * 12 + (size_t)TR * 8 + (size_t)(TR + m + 16) + 16;
	DB_CUDA(cudaFuncSetAttribute(scanpool_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	int per_sm = 1;
	DB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, scanpool_bwd_kernel, (int)threads, smem));
	unsigned slots = (unsigned)state().sm_count * (unsigned)std::max(per_sm, 1);
	// With many groups per slot, one CTA per group balances the waves by itself; then the
	// largest group that still leaves four waves keeps the number of partial results small.
	for (unsigned G = GMAX; G > a.G; G /= 2)
		if ((size_t)divup(nregion, G) * nfb >= (size_t)4 * slots) { a.G = G; break; }
	unsigned ngroup = divup(nregion, a.G);
	unsigned ncta = (size_t)ngroup * nfb >= (size_t)4 * slots ? ngroup : std::min(ngroup, std::max(1u, slots / nfb));
	ncta = std::max(ncta, divup(ngroup, (unsigned)KMAX));            // a CTA holds the bounds of at most KMAX groups
	a.partial = (float*)scratch((size_t)ncta * (wcount + nf) * sizeof(float));
	scanpool_bwd_kernel<<<dim3(ncta, nfb), threads, smem, state().stream>>>(a);
	DB_LAUNCH_CHECK();
	launch_bwd_reduce(dW, dbias, a.partial, wcount, nf, ncta, 0);
	DB_API_CATCH
}
