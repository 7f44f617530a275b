// Many-model motif scan on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// With hundreds of models the scan is a dense contraction
//     Z[f, p] = sum_k  Wt[f, k] * onehot(X)[p, k],     k = 4*tap + channel,  K = 4*m
// (corr1ord.cuh:108-164 written as a matrix product: a base selects one of the
// four channel weights of a tap; any other byte contributes 1/4 of each; 254
// contributes nothing).  The one-hot operand is exact in bf16 (values 0, 1/4, 1);
// the weights are split into 1, 2 or 3 bf16 pieces (8, 16 or 24 significant
// bits) that are accumulated into the same FP32 tensor-memory tile, so every
// product is exact and only the summation order differs from the FP32 path.
//
// Layout of one CTA (256 threads, 1 CTA per SM):
//   M = 128 filters of one filter tile (A operand: prepared bf16 weights, K-major,
//       resident in shared memory for the CTA's lifetime, loaded by one bulk copy);
//   N = up to 128 positions of one sequence (B operand);
//   D = FP32 accumulator in tensor memory, 4 slots of 128 columns.
// The B operand is never expanded: the im2col matrix of a sequence is Toeplitz
// (row p, chunk kc of 8 K-values = bases p+2kc, p+2kc+1), so a flat array E of
// 16-byte chunks, E[q] = one-hot pair of bases (q, q+1), IS the K-major operand
// when the shared-memory descriptor uses an 8-row group stride of 128 bytes and a
// K-chunk stride of 32 bytes: row p, chunk kc lives at E + 16*(p + 2*kc).
// Warp roles: warp 0 issues tcgen05.mma; warps 1-3 encode E for the next block of
// sequences (double buffered); warps 4-7 drain the accumulators: each thread owns
// one filter (one TMEM lane) and reduces its row over the positions in registers
// (bias, rectify, max / mean), then either stores the pooled features or folds
// them through each model's linear head (16 lanes = one model, warp shuffles).
// Per-position activations never leave the SM.
//
// Every wait on an mbarrier is bounded by a clock deadline; on expiry the CTA sets
// a status word, releases its tensor memory and returns.
#include "db_common.cuh"
#include <cuda_bf16.h>

namespace db {

static constexpr int TC_NSLOT = 4;          // accumulator slots of 128 TMEM columns
static constexpr int TC_ECAP = 2304;        // 16-byte chunks per E stage (36 KB)
static constexpr int TC_BLKMAX = 64;        // regions per staged block
static constexpr int TC_SLACK = 160;        // chunks past the last row a tile may touch (N padding + K reach)
static constexpr unsigned long long TC_TIMEOUT = 200000000ull;    // clock cycles (about 0.1 s)

struct tc_args {
	const uint8_t* X; const uint32_t* R; const __nv_bfloat16* Wt; const float* bias;
	const float* headW; const float* headB;
	float* pooled; float* scores; int* status;
	unsigned npos, n, nregion, nf, KC, nsplit, seqs_per_cta, nmodel;
	int ptype, relu;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count)
{
	asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
	asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes)
{
	asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity)
{
	unsigned ok;
	asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
	             : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
	return ok != 0;
}
// Bounded wait: false when the deadline passes or another role has aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag)
{
	if (mbar_try_wait(bar, parity)) return true;
	const unsigned long long t0 = clock64();
	while (true) {
		if (mbar_try_wait(bar, parity)) return true;
		if (*abort_flag) return false;
		if (clock64() - t0 > TC_TIMEOUT) { *abort_flag = 1; return false; }
	}
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar)
{
	asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
	             :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, unsigned ncols)
{
	asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
	asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, unsigned ncols)
{
	asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, unsigned accumulate)
{
	asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
	             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
	             :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
	asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32])
{
	uint32_t* r = reinterpret_cast<uint32_t*>(v);
	asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
	             "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
	             "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
	             : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
	               "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
	               "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
	               "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
	             : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core
// matrices; `lbo` = byte step between the two K-halves of an MMA, `sbo` = byte
// step between 8-row groups.  Bits [46,48) = 1 (descriptor version of sm_100).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, unsigned lbo, unsigned sbo)
{
	return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
	       ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// Instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N given.
__device__ __forceinline__ uint32_t instr_desc(unsigned N)
{
	return (1u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);
}

// One-hot (or 1/4, or zero) pattern of a base as four bf16 in 64 bits, channel c at bits [16c, 16c+16).
__device__ __forceinline__ unsigned long long base_pattern(unsigned x)
{
	if (x < 4u) return 0x3F80ull << (16u * x);        // bf16(1.0)
	if (x == 254u) return 0ull;                        // dropped input
	return 0x3E803E803E803E80ull;                      // bf16(0.25) in every channel
}

__device__ __forceinline__ unsigned region_rows(const uint32_t* R, unsigned g) { unsigned a = R[2*g], b = R[2*g+1]; return b > a ? b - a : 0u; }

__global__ void __launch_bounds__(256, 1)
scanpool_tc_kernel(const tc_args a)
{
	extern __shared__ __align__(128) unsigned char smem[];
	const unsigned KC = a.KC, NK = KC / 2;
	const unsigned a_bytes = a.nsplit * KC * 2048u;
	unsigned char* As = smem;                                    // [nsplit][KC][128][8] bf16
	unsigned char* Es = smem + a_bytes;                          // [2][TC_ECAP] 16-byte chunks
	__shared__ __align__(8) uint64_t bar_a, e_full[2], e_empty[2], t_full[TC_NSLOT], t_empty[TC_NSLOT];
	__shared__ uint32_t tmem_base_s;
	__shared__ unsigned blk_lo[2], blk_hi[2], blk_count[2], blk_ok[2];
	__shared__ unsigned blk_r0[2][TC_BLKMAX], blk_rows[2][TC_BLKMAX];   // region table of each staged block
	__shared__ int abort_s;
	volatile int* abort_flag = &abort_s;

	const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const unsigned tile = blockIdx.x;
	const unsigned g_first = blockIdx.y * a.seqs_per_cta;
	const unsigned g_last = min(a.nregion, g_first + a.seqs_per_cta);

	// A CTA of a launch that has already failed returns at once.  One thread reads
	// the status word so that the whole CTA takes the same decision.
	if (threadIdx.x == 0) abort_s = *reinterpret_cast<volatile int*>(a.status);
	__syncthreads();
	if (abort_s != 0) return;
	__syncthreads();
	if (threadIdx.x == 0) {
		abort_s = 0;
		mbar_init(&bar_a, 1);
		for (int i = 0; i < 2; ++i) { mbar_init(&e_full[i], 3); mbar_init(&e_empty[i], 1); }
		for (int i = 0; i < TC_NSLOT; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], 4); }
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0) tmem_alloc(&tmem_base_s, TC_NSLOT * 128);
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_base_s;

	if (warp == 0) {
		// ------------------------------------------------------------ MMA issuer
		if (lane == 0) {
			mbar_expect_tx(&bar_a, a_bytes);
			bulk_g2s(As, reinterpret_cast<const unsigned char*>(a.Wt) + (size_t)tile * a_bytes, a_bytes, &bar_a);
			bool ok = mbar_wait(&bar_a, 0, abort_flag);
			const uint32_t a_addr = smem_u32(As), e_addr = smem_u32(Es);
			unsigned g = g_first, blk = 0, t = 0;
			while (ok && g < g_last) {
				const unsigned st = blk & 1;
				ok = mbar_wait(&e_full[st], (blk >> 1) & 1, abort_flag);
				if (!ok) break;
				tc_fence_after();
				const unsigned lo = blk_lo[st], cnt = blk_count[st];
				for (unsigned i = 0; ok && i < cnt; ++i, ++g) {
					const unsigned r0 = blk_r0[st][i], P = blk_rows[st][i];
					for (unsigned c0 = 0; c0 < P; c0 += 128, ++t) {
						const unsigned slot = t % TC_NSLOT;
						ok = mbar_wait(&t_empty[slot], ((t / TC_NSLOT) & 1) ^ 1, abort_flag);
						if (!ok) break;
						tc_fence_after();
						const unsigned ncols = min(128u, P - c0), N = (ncols + 15u) & ~15u;
						const uint32_t idesc = instr_desc(N);
						const uint32_t d = tmem_base + slot * 128;
						const uint32_t b0 = e_addr + st * (TC_ECAP * 16) + (r0 - lo + c0) * 16;
						unsigned acc = 0;
						for (unsigned s = 0; s < a.nsplit; ++s)
							for (unsigned kk = 0; kk < NK; ++kk) {
								umma_bf16(d, smem_desc(a_addr + s * KC * 2048 + kk * 4096, 2048, 128),
								          smem_desc(b0 + kk * 64, 32, 128), idesc, acc);
								acc = 1;
							}
						umma_commit(&t_full[slot]);
					}
				}
				umma_commit(&e_empty[st]);      // the stage may be rewritten once these MMAs have read it
				++blk;
			}
		}
	} else if (warp < 4) {
		// ---------------------------------------------------------- E builders
		const unsigned bt = threadIdx.x - 32;     // 0..95
		unsigned g = g_first, blk = 0;
		bool ok = true;
		while (ok && g < g_last) {
			const unsigned st = blk & 1;
			// One thread waits (bounded) and publishes the outcome, so that all 96
			// builder threads take the same path to the named barriers below.
			if (bt == 0) blk_ok[st] = mbar_wait(&e_empty[st], ((blk >> 1) & 1) ^ 1, abort_flag) ? 1u : 0u;
			asm volatile("bar.sync 1, 96;" ::: "memory");
			ok = blk_ok[st] != 0;
			if (!ok) break;
			// The next TC_BLKMAX regions go to shared memory in parallel; one thread then
			// takes the longest run whose rows, plus the reach of the last tile, fit in
			// one stage.  Regions normally abut (the batch layout).
			if (bt < TC_BLKMAX) {
				const unsigned h = g + bt;
				unsigned r0 = 0, r1 = 0;
				if (h < g_last) { r0 = a.R[2 * h]; r1 = max(a.R[2 * h + 1], r0); }
				blk_r0[st][bt] = r0; blk_rows[st][bt] = r1 - r0;
			}
			asm volatile("bar.sync 1, 96;" ::: "memory");
			if (bt == 0) {
				unsigned lo = blk_r0[st][0], hi = lo, cnt = 0;
				const unsigned avail = min((unsigned)TC_BLKMAX, g_last - g);
				for (unsigned i = 0; i < avail; ++i) {
					unsigned r0 = blk_r0[st][i], r1 = r0 + blk_rows[st][i];
					unsigned nlo = min(lo, r0), nhi = max(hi, r1);
					if (nhi - nlo + TC_SLACK > TC_ECAP) break;
					lo = nlo; hi = nhi; ++cnt;
				}
				blk_lo[st] = lo; blk_hi[st] = hi; blk_count[st] = cnt;
			}
			asm volatile("bar.sync 1, 96;" ::: "memory");
			const unsigned lo = blk_lo[st], hi = blk_hi[st], cnt = blk_count[st];
			if (cnt == 0) { if (bt == 0) { *abort_flag = 1; atomicExch(a.status, 2); } ok = false; break; }   // region longer than a stage
			const unsigned nchunk = min((unsigned)TC_ECAP, hi - lo + TC_SLACK);
			uint4* E = reinterpret_cast<uint4*>(Es + (size_t)st * TC_ECAP * 16);
			for (unsigned q = bt; q < nchunk; q += 96) {
				const unsigned i0 = lo + q;
				const unsigned x0 = i0 < a.npos ? a.X[i0] : 254u, x1 = i0 + 1 < a.npos ? a.X[i0 + 1] : 254u;
				const unsigned long long p0 = base_pattern(x0), p1 = base_pattern(x1);
				E[q] = make_uint4((unsigned)p0, (unsigned)(p0 >> 32), (unsigned)p1, (unsigned)(p1 >> 32));
			}
			fence_async_smem();
			__syncwarp();
			if (lane == 0) mbar_arrive(&e_full[st]);
			g += cnt; ++blk;
		}
	} else {
		// ------------------------------------------------------------ epilogue
		const unsigned q4 = warp & 3;                       // TMEM lane quarter of this warp
		const unsigned fl = q4 * 32 + lane;                 // filter within the tile
		const unsigned f = tile * 128 + fl;
		const float b = (a.bias && f < a.nf) ? a.bias[f] : 0.f;
		const float nb = -b;
		const bool want_max = a.ptype == DB_PT_MAX || a.ptype == DB_PT_ALL;
		const bool want_sum = a.ptype != DB_PT_MAX;
		// linear head of the model this filter belongs to (16 filters per model)
		float hw_max = 0.f, hw_sum = 0.f, hb = 0.f;
		const unsigned model = f / 16;
		if (a.scores && f < a.nf) {
			const unsigned npool = a.ptype == DB_PT_ALL ? 32u : 16u;
			const unsigned k = f % 16;
			if (a.ptype == DB_PT_ALL) { hw_max = a.headW[model * npool + 2 * k]; hw_sum = a.headW[model * npool + 2 * k + 1]; }
			else if (a.ptype == DB_PT_MAX) hw_max = a.headW[model * npool + k];
			else hw_sum = a.headW[model * npool + k];
			hb = a.headB ? a.headB[model] : 0.f;
		}
		unsigned t = 0;
		bool ok = true;
		unsigned nr0 = 0, nr1 = 0;                      // bounds of the next region, loaded one region ahead
		if (g_first < g_last) { nr0 = a.R[2 * g_first]; nr1 = a.R[2 * g_first + 1]; }
		for (unsigned g = g_first; ok && g < g_last; ++g) {
			const unsigned r0 = nr0, P = nr1 > nr0 ? nr1 - nr0 : 0u;
			if (g + 1 < g_last) { nr0 = a.R[2 * (g + 1)]; nr1 = a.R[2 * (g + 1) + 1]; }
			float mx = -INFINITY, s0 = 0.f, s1 = 0.f;
			for (unsigned c0 = 0; c0 < P; c0 += 128, ++t) {
				const unsigned slot = t % TC_NSLOT;
				// lane 0 waits (bounded); the warp stays converged for the aligned TMEM loads
				unsigned okv = 0;
				if (lane == 0) okv = mbar_wait(&t_full[slot], (t / TC_NSLOT) & 1, abort_flag) ? 1u : 0u;
				ok = __shfl_sync(0xffffffffu, okv, 0) != 0;
				if (!ok) break;
				mbar_try_wait(&t_full[slot], (t / TC_NSLOT) & 1);     // completed: every lane observes the phase
				tc_fence_after();
				const unsigned ncols = min(128u, P - c0);
				// rows at or past n have no scan output (kangaroo_smat.cpp:105): they read as zero
				const unsigned nvalid = a.n > r0 + c0 ? min(ncols, a.n - (r0 + c0)) : 0u;
				const uint32_t taddr = tmem_base + ((q4 * 32u) << 16) + slot * 128;
				for (unsigned c = 0; c < ncols; c += 32) {
					float v[32];
					tmem_ld32(taddr + c, v);
					tmem_ld_wait();
					const unsigned rem = ncols - c;
					if (rem >= 32 && nvalid >= c + 32) {
						#pragma unroll
						for (int i = 0; i < 32; i += 2) {
							if (want_max) mx = fmaxf(mx, fmaxf(v[i], v[i + 1]));
							if (want_sum) { s0 += a.relu ? fmaxf(v[i], nb) : v[i]; s1 += a.relu ? fmaxf(v[i + 1], nb) : v[i + 1]; }
						}
					} else {
						#pragma unroll
						for (int i = 0; i < 32; ++i) {
							if ((unsigned)i < rem) {
								const float x = (c + i < nvalid) ? v[i] : 0.f;
								if (want_max) mx = fmaxf(mx, x);
								if (want_sum) s0 += a.relu ? fmaxf(x, nb) : x;
							}
						}
					}
				}
				tc_fence_before();
				__syncwarp();
				if (lane == 0) mbar_arrive(&t_empty[slot]);
			}
			if (!ok) break;
			// finish the region: max_p relu(z_p + b) = relu(max_p z_p + b); sum_p relu(z_p + b) = sum_p max(z_p, -b) + P*b
			float pmax = mx + b;
			if (a.relu) pmax = fmaxf(pmax, 0.f);
			float psum = (s0 + s1) + (float)P * b;
			const float pavg = psum / (float)P;
			const float second = a.ptype == DB_PT_SUM ? psum : pavg;
			if (a.pooled && f < a.nf) {
				const size_t o = (size_t)g * a.nf + f;
				if (a.ptype == DB_PT_ALL) reinterpret_cast<float2*>(a.pooled)[o] = make_float2(pmax, pavg);
				else a.pooled[o] = want_max ? pmax : second;
			}
			if (a.scores) {
				float part = hw_max * (want_max ? pmax : 0.f) + hw_sum * (want_sum ? second : 0.f);
				part += __shfl_xor_sync(0xffffffffu, part, 8);
				part += __shfl_xor_sync(0xffffffffu, part, 4);
				part += __shfl_xor_sync(0xffffffffu, part, 2);
				part += __shfl_xor_sync(0xffffffffu, part, 1);
				if ((lane & 15) == 0 && f < a.nf) a.scores[(size_t)g * a.nmodel + model] = part + hb;
			}
		}
	}
	tc_fence_before();
	__syncthreads();
	if (threadIdx.x == 0 && abort_s) atomicCAS(a.status, 0, 1);
	if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, TC_NSLOT * 128); }
}

// Prepared weights: for each 128-filter tile, `nsplit` K-major bf16 operand tiles
// in the shared-memory layout [split][K chunk][filter][8], zero padded.
__global__ void tc_prepare_kernel(const float* __restrict__ W, unsigned m, unsigned nf, unsigned KC, unsigned nsplit,
                                  unsigned ntile, __nv_bfloat16* __restrict__ out)
{
	const size_t total = (size_t)ntile * KC * 128 * 8;
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
		const unsigned e = i % 8, fl = (i / 8) % 128, kc = (i / 1024) % KC, tile = (unsigned)(i / ((size_t)1024 * KC));
		const unsigned k = kc * 8 + e, f = tile * 128 + fl;
		float w = (k < 4 * m && f < nf) ? W[(size_t)k * nf + f] : 0.f;
		for (unsigned s = 0; s < nsplit; ++s) {
			__nv_bfloat16 h = __float2bfloat16_rn(w);
			out[(((size_t)tile * nsplit + s) * KC + kc) * 1024 + fl * 8 + e] = h;
			w -= __bfloat162float(h);
		}
	}
}

}  // namespace db

using namespace db;

static void tc_shape(uint32_t m, uint32_t nf, unsigned& KC, unsigned& ntile)
{
	DB_REQUIRE(m > 0 && nf > 0, "ValueError: filter bank must not be empty (m=%u, nf=%u)", m, nf);
	unsigned mpad = (m + 3u) & ~3u;                   // one MMA consumes 4 taps (K = 16)
	KC = mpad / 2;
	ntile = (nf + 127u) / 128u;
}

DB_EXPORT size_t db_tc_weights_bytes(uint32_t m, uint32_t nf, int nsplit)
{
	DB_API_TRY_NODEV
	DB_REQUIRE(nsplit >= 1 && nsplit <= 3, "ValueError: nsplit must be 1, 2 or 3");
	unsigned KC, ntile;
	tc_shape(m, nf, KC, ntile);
	return (size_t)ntile * nsplit * KC * 2048;
	DB_API_CATCH_RETURN(0)
}

DB_EXPORT void db_tc_prepare(const float* W, uint32_t m, uint32_t nf, int nsplit, void* out)
{
	DB_API_TRY
	DB_REQUIRE(nsplit >= 1 && nsplit <= 3, "ValueError: nsplit must be 1, 2 or 3");
	DB_REQUIRE(W && out, "ValueError: db_tc_prepare got a NULL pointer");
	DB_REQUIRE(((uintptr_t)out & 15) == 0, "ValueError: prepared-weight buffer must be 16-byte aligned");
	unsigned KC, ntile;
	tc_shape(m, nf, KC, ntile);
	size_t total = (size_t)ntile * KC * 1024;
	tc_prepare_kernel<<<elemwise_grid(total), 256, 0, state().stream>>>(W, m, nf, KC, (unsigned)nsplit, ntile, (__nv_bfloat16*)out);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_scanpool_tc(const void* Wt, uint32_t m, uint32_t nf, int nsplit, const float* bias, int relu,
                              const uint8_t* X, uint32_t npos, const uint32_t* regions, uint32_t nregion, int ptype,
                              float* pooled, const float* headW, const float* headB, uint32_t nmodel, float* scores,
                              int* status)
{
	DB_API_TRY
	DB_REQUIRE(ptype >= DB_PT_MAX && ptype <= DB_PT_ALL, "ValueError: unknown pooling type %d", ptype);
	DB_REQUIRE(nsplit >= 1 && nsplit <= 3, "ValueError: nsplit must be 1, 2 or 3");
	DB_REQUIRE(status != nullptr, "ValueError: db_scanpool_tc needs a device status word");
	DB_REQUIRE(pooled || scores, "ValueError: db_scanpool_tc needs an output (pooled or scores)");
	if (scores) {
		DB_REQUIRE(headW != nullptr, "ValueError: scores requested without head weights");
		DB_REQUIRE(nmodel * 16 == nf, "ValueError: the fused linear head needs 16 filters per model (nf=%u, nmodel=%u)", nf, nmodel);
	}
	if (nregion == 0) return;
	DB_REQUIRE(Wt && X && regions, "ValueError: db_scanpool_tc got a NULL pointer");
	DB_REQUIRE(((uintptr_t)Wt & 15) == 0, "ValueError: prepared weights must be 16-byte aligned");
	unsigned KC, ntile;
	tc_shape(m, nf, KC, ntile);
	tc_args a;
	a.X = X; a.R = regions; a.Wt = (const __nv_bfloat16*)Wt; a.bias = bias; a.headW = headW; a.headB = headB;
	a.pooled = pooled; a.scores = scores; a.status = status;
	a.npos = npos; a.n = npos >= m ? npos - m + 1 : 0; a.nregion = nregion; a.nf = nf; a.KC = KC; a.nsplit = nsplit;
	a.nmodel = nmodel; a.ptype = ptype; a.relu = relu;
	// Sequence chunks: enough CTAs for about 8 waves over the SMs, at least 64 sequences each.
	unsigned sms = state().sm_count;
	unsigned want_chunks = max(1u, (8 * sms + ntile - 1) / ntile);
	unsigned spc = max(64u, divup(nregion, want_chunks));
	a.seqs_per_cta = spc;
	dim3 grid(ntile, divup(nregion, spc));
	size_t smem = (size_t)nsplit * KC * 2048 + 2 * (size_t)TC_ECAP * 16 + 128;
	DB_REQUIRE(smem <= 220 * 1024, "ValueError: filter length %u is too long for the tensor-core kernel", m);
	DB_CUDA(cudaFuncSetAttribute(scanpool_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	scanpool_tc_kernel<<<grid, 256, smem, state().stream>>>(a);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
