// Forward motif scan + bias + rectify + region pooling for SCORING, FP32, with k-mer
// lookup tables.
//
// The exact kernel (scanpool_f32.cu) adds one table operand per (row, filter, tap), in
// tap order, so that values and argmax agree bit for bit with the reference chain; its
// ceiling is the shared-memory return path: one 4-byte operand per add.  Scoring needs
// neither argmax nor the tap order, so here one operand covers KT taps: the table holds,
// per group of KT taps and per k-mer of bases under them, the SUM of the KT weights
// (corr1ord.cuh:144-158 regrouped: ((w_j[x_j] + w_j+1[x_j+1]) + ...) instead of one tap
// after the other).  The same shared-memory traffic then does KT times the work.
// Results differ from the exact kernel by the rounding of the regrouped FP32 sums only
// (a few ulp of the largest partial sum; the tests state 1e-6 of the largest activation).
//
// Alphabet of a position: A C G T, N (any other byte: the mean of the four channels, the
// padding byte 255 included) and "dropped" (254: contributes nothing), six codes; a group
// of KT taps has 6^KT k-mers.  KT = 2 (36 k-mers) for filters up to 24 taps, KT = 3 (216)
// where the table still fits (up to 18 taps).  Filters whose length is not a multiple of
// KT are padded with zero taps.
//
// Layout.  A CTA owns 16 filters and a contiguous range of regions; it builds its table
// once and walks the rows of its regions in tiles of 128.  Scan: a thread owns one row x
// four filters and reads, per group, one 16-byte table entry.  The entry of k-mer `idx`
// in group g is a 128-byte line [quad 0..3][row parity 0..1][4 floats]: the eight lanes
// of a quarter warp (two rows x four quads) read eight different 16-byte bank groups of
// (at most two) lines, whatever the k-mers are, so every 128-bit load runs conflict-free.
// Pool: rows ascending per (region, filter), the running maximum and sum of a region that
// continues in the next tile are carried through shared memory.  Regions must ascend
// without overlap (the batch layout); the launch reports status 3 otherwise.
#include "db_common.cuh"

namespace db {

static constexpr int KTR = 128;          // rows per tile
static constexpr int KSLOTS = 32;        // regions pooled per pass (512 threads / 16 filters)

struct kmer_args {
	const float* W; const float* bias; const uint8_t* X; const uint32_t* R;
	float* pooled; int* status;
	unsigned m, nf, npos, n, nregion, rper;      // rper: regions per CTA
	int relu, ptype;
};

__device__ __forceinline__ unsigned code6_of(unsigned x)
{
	return x < 4u ? x : (x == 254u ? 5u : 4u);
}

template <int KT> struct kmer_count { static constexpr unsigned value = KT == 1 ? 6u : (KT == 2 ? 36u : 216u); };


template <int M, int KT>
__global__ void __launch_bounds__(512)
scanpool_kmer_kernel(const kmer_args a)
{
	constexpr unsigned NG = (M + KT - 1) / KT;              // tap groups
	constexpr unsigned NIDX = kmer_count<KT>::value;
	extern __shared__ __align__(128) unsigned char smem[];
	float4* tab = reinterpret_cast<float4*>(smem);                           // [NG][NIDX][8] float4
	float4* act = tab + (size_t)NG * NIDX * 8;                               // [KTR][4] float4: row-major activations of 16 filters
	float* wtap = reinterpret_cast<float*>(act + KTR * 4);                   // [NG*KT taps][6 codes][16 filters]: weight of a base at a tap
	uint8_t* xk = reinterpret_cast<uint8_t*>(wtap + NG * KT * 6 * 16);       // k-mer code of every position of the tile (+ reach)
	__shared__ unsigned s_first, s_count, s_bad;
	// by tile parity: written for the next tile while this tile's carry is read
	__shared__ float carry_max[2][16], carry_sum[2][16];
	__shared__ unsigned carry_on[2];
	__shared__ __align__(16) float sbias[16];

	const unsigned tid = threadIdx.x;
	const unsigned f0 = blockIdx.y * 16;
	const unsigned g_lo = blockIdx.x * a.rper, g_hi = min(a.nregion, g_lo + a.rper);
	if (g_lo >= g_hi) return;

	// ---- weight of each of the six codes at every tap (zero taps pad the filter to NG * KT):
	// the four channels, the N mean ((w0 + w1) + w2 + w3) / 4 (corr1ord.cuh:150-154), 0 for a dropped base
	for (unsigned e = tid; e < NG * KT * 16; e += blockDim.x) {
		const unsigned f = e & 15u, j = e >> 4;
		float w[4] = {0.f, 0.f, 0.f, 0.f};
		if (j < (unsigned)M && f0 + f < a.nf) {
			#pragma unroll
			for (int c = 0; c < 4; ++c) w[c] = a.W[(size_t)(4 * j + c) * a.nf + f0 + f];
		}
		float z = w[0]; z += w[1]; z += w[2]; z += w[3];
		float* o = wtap + (size_t)j * 96 + f;
		o[0] = w[0]; o[16] = w[1]; o[32] = w[2]; o[48] = w[3]; o[64] = z * 0.25f; o[80] = 0.f;
	}
	__syncthreads();
	// ---- table: entry (g, idx) = sum over the group's taps of the weight of the k-mer's base there
	for (unsigned e = tid; e < NG * NIDX * 16; e += blockDim.x) {
		const unsigned f = e & 15u, idx = (e >> 4) % NIDX, g = (e >> 4) / NIDX;
		unsigned rest = idx;
		float s = 0.f;
		#pragma unroll
		for (int t = 0; t < KT; ++t) {
			const float w = wtap[(size_t)(g * KT + t) * 96 + (rest % 6u) * 16 + f];
			s = t == 0 ? w : s + w;
			rest /= 6u;
		}
		float* line = reinterpret_cast<float*>(tab + ((size_t)g * NIDX + idx) * 8);
		const unsigned quad = f >> 2, v = f & 3u;
		line[(quad * 2 + 0) * 4 + v] = s;
		line[(quad * 2 + 1) * 4 + v] = s;
	}
	if (tid < 16) sbias[tid] = (a.bias && f0 + tid < a.nf) ? a.bias[f0 + tid] : 0.f;
	if (tid == 0) { carry_on[0] = carry_on[1] = 0; s_bad = 0; s_first = g_lo; }
	__syncthreads();

	// scan identity: row of the tile, quad of four filters, slot of the table line
	const unsigned rl = tid >> 2, quad = tid & 3u;
	const float4* my_tab = tab + quad * 2 + (rl & 1u);
	// pool identity: region slot of the pass, filter
	const unsigned pk = tid >> 4, pf = tid & 15u;

	const unsigned row_lo = a.R[2 * g_lo];
	unsigned row_hi = row_lo;
	{
		const unsigned r0 = a.R[2 * (g_hi - 1)], r1 = a.R[2 * (g_hi - 1) + 1];
		row_hi = max(row_lo, r1 <= r0 ? r0 + 1 : r1);
	}

	unsigned par = 0;
	for (unsigned t0 = row_lo; t0 < row_hi; t0 += KTR, par ^= 1u) {
		// ---- stage the k-mer codes of positions t0 .. t0 + KTR + M - 1
		for (unsigned t = tid; t < KTR + NG * KT; t += blockDim.x) {
			unsigned idx = 0, mul = 1;
			#pragma unroll
			for (int k = 0; k < KT; ++k) {
				const unsigned i = t0 + t + k;
				idx += mul * code6_of(i < a.npos ? a.X[i] : 254u);
				mul *= 6u;
			}
			xk[t] = (uint8_t)idx;
		}
		__syncthreads();
		// ---- scan: one row x four filters per thread
		{
			const unsigned row = t0 + rl;
			float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
			if (row < a.n && row < row_hi) {
				#pragma unroll
				for (unsigned g = 0; g < NG; ++g) {
					const unsigned idx = xk[rl + g * KT];
					const float4 e = my_tab[((size_t)g * NIDX + idx) * 8];
					if (g == 0) z = e;
					else { z.x += e.x; z.y += e.y; z.z += e.z; z.w += e.w; }
				}
			}
			if (a.bias) {
				const float4 b = *reinterpret_cast<const float4*>(sbias + quad * 4);
				z.x += b.x; z.y += b.y; z.z += b.z; z.w += b.w;
			}
			if (a.relu) { z.x = fmaxf(z.x, 0.f); z.y = fmaxf(z.y, 0.f); z.z = fmaxf(z.z, 0.f); z.w = fmaxf(z.w, 0.f); }
			act[rl * 4 + quad] = z;
		}
		// ---- which regions touch this tile: warp 0 looks 32 regions ahead per step of the
		// ascending table (finished regions form a prefix, so do the ones that start in the tile)
		if (tid < 32) {
			const unsigned tile_end = min(t0 + KTR, row_hi);
			unsigned g = s_first;
			for (;;) {
				const unsigned gi = g + tid;
				bool gone = false;
				if (gi < g_hi) {
					const uint2 r = reinterpret_cast<const uint2*>(a.R)[gi];
					gone = max(r.y, r.x + 1u) <= t0;
				}
				const unsigned mask = __ballot_sync(0xffffffffu, gone);
				const unsigned lead = mask == 0xffffffffu ? 32u : (unsigned)__ffs(~mask) - 1u;
				g += lead;
				if (lead < 32u) break;
			}
			unsigned cnt = 0;
			for (;;) {
				const unsigned gi = g + cnt + tid;
				const bool in = gi < g_hi && a.R[2 * gi] < tile_end;
				const unsigned mask = __ballot_sync(0xffffffffu, in);
				const unsigned lead = mask == 0xffffffffu ? 32u : (unsigned)__ffs(~mask) - 1u;
				cnt += lead;
				if (lead < 32u) break;
			}
			if (tid == 0) { s_first = g; s_count = cnt; carry_on[par] = 0; }
		}
		__syncthreads();
		// ---- pool, KSLOTS regions per pass
		const unsigned first = s_first, count = s_count;
		const unsigned tile_hi = min(t0 + KTR, row_hi);
		for (unsigned base = 0; base < count; base += KSLOTS) {
			const unsigned k = base + pk;
			if (k < count) {
				const unsigned g = first + k;
				const uint2 r = reinterpret_cast<const uint2*>(a.R)[g];
				const unsigned r0 = r.x, r1 = r.y <= r.x ? r.x + 1 : r.y;      // an empty region still reads its first row (poolrgn.cuh:60)
				if (pf == 0 && g > 0) {                      // regions must ascend and not overlap the one before (another CTA's, too)
					const unsigned p0 = a.R[2 * g - 2], p1 = a.R[2 * g - 1];
					if (r0 < p0 || (p1 > p0 && r0 < p1)) s_bad = 1;
				}
				const unsigned lo = max(r0, t0), hi = min(r1, tile_hi);
				float mx = 0.f, sm = 0.f;
				bool started = false;
				if (r0 < t0 && carry_on[par ^ 1u]) { mx = carry_max[par ^ 1u][pf]; sm = carry_sum[par ^ 1u][pf]; started = true; }
				const float* col = reinterpret_cast<const float*>(act) + pf;
				for (unsigned row = lo; row < hi; ++row) {
					const float v = col[(row - t0) * 16];
					if (!started) { mx = v; sm = v; started = true; }
					else { mx = fmaxf(mx, v); sm += v; }
				}
				if (r1 > tile_hi) {                          // continues in the next tile: at most one region does
					carry_max[par][pf] = mx; carry_sum[par][pf] = sm;
					if (pf == 0) carry_on[par] = 1;
				} else if (f0 + pf < a.nf) {
					const size_t o = (size_t)g * a.nf + f0 + pf;
					const float cnt = (float)(r.y - r.x);    // integer row count (poolrgn.cuh:112,152)
					switch (a.ptype) {
					case DB_PT_MAX: a.pooled[o] = mx; break;
					case DB_PT_AVG: a.pooled[o] = sm / cnt; break;
					case DB_PT_SUM: a.pooled[o] = sm; break;
					default: reinterpret_cast<float2*>(a.pooled)[o] = make_float2(mx, sm / cnt); break;
					}
				}
			}
		}
		__syncthreads();            // the tile's activations and codes are rewritten next
	}
	if (tid == 0 && s_bad && a.status) atomicCAS(a.status, 0, 3);
}

}  // namespace db

using namespace db;

template <int M, int KT>
static void launch_kmer(const kmer_args& a0)
{
	kmer_args a = a0;
	constexpr unsigned NG = (M + KT - 1) / KT, NIDX = kmer_count<KT>::value;
	const size_t smem = (size_t)NG * NIDX * 128 + (size_t)KTR * 64 + (size_t)NG * KT * 96 * 4 + KTR + NG * KT + 16;
	auto kern = scanpool_kmer_kernel<M, KT>;
	DB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	int per_sm = 1;
	DB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, 512, smem));
	if (per_sm < 1) per_sm = 1;
	// Persistent CTAs: as many as fit at once (a CTA builds its table once), but no fewer
	// than eight tiles' worth of rows each so that short batches still spread over the SMs.
	const unsigned nfb = divup(a.nf, 16u);
	unsigned ncta = std::max(1u, (unsigned)state().sm_count * (unsigned)per_sm / nfb);
	const unsigned rows_per_region = std::max(1u, a.npos / a.nregion);
	const unsigned min_regions = std::max(1u, 2u * KTR / rows_per_region);
	ncta = std::min(ncta, std::max(1u, a.nregion / min_regions));
	a.rper = divup(a.nregion, ncta);
	dim3 grid(divup(a.nregion, a.rper), nfb);
	kern<<<grid, 512, smem, state().stream>>>(a);
}

// Filter lengths are template parameters (the tap groups unroll): the lengths the DeepBind
// models use, each with the widest k-mer whose table fits beside the activation tile.
DB_EXPORT int db_scanpool_score_supported(uint32_t m)
{
	return m == 24 || m == 16 || m == 12 || m == 8 || m == 20 || m == 32;
}

DB_EXPORT void db_scanpool_score(const float* W, uint32_t m, uint32_t nf, const float* bias, int relu,
                                 const uint8_t* X, uint32_t npos, const uint32_t* regions, uint32_t nregion,
                                 int ptype, float* pooled, int* status)
{
	DB_API_TRY
	DB_REQUIRE(ptype >= DB_PT_MAX && ptype <= DB_PT_ALL, "ValueError: unknown pooling type %d", ptype);
	DB_REQUIRE(db_scanpool_score_supported(m), "ValueError: the k-mer scoring kernel is built for filter lengths 8, 12, 16, 20, 24 and 32 "
	           "(got %u); use db_scanpool_fwd", m);
	DB_REQUIRE(nf > 0, "ValueError: filter bank must not be empty");
	if (nregion == 0) return;
	DB_REQUIRE(W && X && regions && pooled, "ValueError: db_scanpool_score got a NULL pointer");
	DB_REQUIRE(((uintptr_t)regions & 7) == 0, "ValueError: the region table must be 8-byte aligned");
	DB_REQUIRE(ptype != DB_PT_ALL || ((uintptr_t)pooled & 7) == 0, "ValueError: pooled must be 8-byte aligned for max+mean pooling");
	kmer_args a;
	a.W = W; a.bias = bias; a.X = X; a.R = regions; a.pooled = pooled; a.status = status;
	a.m = m; a.nf = nf; a.npos = npos; a.n = npos >= m ? npos - m + 1 : 0; a.nregion = nregion;
	a.relu = relu; a.ptype = ptype; a.rper = nregion;
	switch (m) {
	case 8:  launch_kmer<8, 3>(a); break;        //  3 groups x 216 x 128 B =  83 KB
	case 12: launch_kmer<12, 3>(a); break;       //  4 groups            = 111 KB
	case 16: launch_kmer<16, 3>(a); break;       //  6 groups (18 taps)  = 166 KB
	case 20: launch_kmer<20, 2>(a); break;       // 10 groups x 36 x 128 B = 46 KB
	case 24: launch_kmer<24, 2>(a); break;       // 12 groups            =  55 KB
	default: launch_kmer<32, 2>(a); break;       // 16 groups            =  74 KB
	}
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
