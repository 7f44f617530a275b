// Many-model motif scan on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// With hundreds of models the scan is a dense contraction
//     Z[f, p] = sum_k  Wt[f, k] * onehot(X)[p, k],     k = 4*tap + channel,  K = 4*m
// (corr1ord.cuh:108-164 written as a matrix product: a base selects one of the
// four channel weights of a tap; any other byte contributes 1/4 of each; 254
// contributes nothing).  The one-hot operand is exact in bf16 and f16 (values 0,
// 1/4, 1); the weights are split into 1-3 bf16 pieces (8, 16, 24 significant bits)
// or 1-2 f16 pieces of power-of-two prescaled weights (11, 22 bits) that are
// accumulated into the same FP32 tensor-memory tile, so every product is exact and
// only the summation order differs from the FP32 path.
//
// Layout of one CTA (32 * (3 + 16) threads, 1 CTA per SM):
//   M = 128 filters of one filter tile (A operand: prepared 16-bit weights, K-major,
//       resident in shared memory for the CTA's lifetime, loaded by one bulk copy);
//   N = 256 consecutive rows of the ordinal buffer (B operand), whatever sequences
//       they belong to: the regions of a batch abut, so tiling the flat rows wastes
//       nothing on padding and keeps the MMA at its widest N;
//   D = FP32 accumulator in tensor memory, 2 slots of 256 columns.
// The B operand is never expanded: the im2col matrix is Toeplitz (row p, chunk kc
// of 8 K-values = bases p+2kc, p+2kc+1), so a flat array E of 16-byte chunks,
// E[q] = one-hot pair of bases (q, q+1), IS the K-major operand when the
// shared-memory descriptor uses an 8-row group stride of 128 bytes and a K-chunk
// stride of 32 bytes: row p, chunk kc lives at E + 16*(p + 2*kc).
// Warp roles: warp 0 issues tcgen05.mma; warps 1-2 encode E for the next stage of
// 8 tiles (double buffered); warps 3-18 drain the accumulators: each thread owns one
// filter (one TMEM lane); four warps share a lane quarter and take the regions in
// turn, each walking only its own regions.  A warp fetches the columns of its region
// starting at the region's own first column, in pieces of 32/16/8/4/2/1 columns, so
// the reduction (in registers) needs no per-column tests.  The maximum commutes with
// bias and rectifier, which are applied once per region; the rectified sum costs one
// saturating FMA and half a packed add per column.  When a region ends the warp
// either stores the pooled features or folds them through the model's linear head
// (16 lanes = one model, warp shuffles).  Per-position activations never leave the
// SM.  Regions must ascend without overlap (the batch layout).
//
// Every wait on an mbarrier is bounded by a clock deadline; on expiry the CTA sets
// a status word, releases its tensor memory and returns.
#include "db_common.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstring>

namespace db {

static constexpr int TC_STAGE_TILES = 8;    // tiles of 256 flat rows per E stage
static constexpr int TC_ECHUNKS = TC_STAGE_TILES * 256 + 128;   // 16-byte chunks per stage incl. the K reach of the last row
static constexpr int TC_EPI_SETS = 4;      // epilogue warps per TMEM lane quarter; region g is reduced by set g % TC_EPI_SETS
static constexpr int TC_BUILD_WARPS = 2;   // warps that encode the B operand (one stage ahead; a stage lasts 8 tiles)
static constexpr int TC_EPI_WARP0 = 1 + TC_BUILD_WARPS;             // first epilogue warp
static constexpr int TC_SEND_WARP = TC_EPI_WARP0 + 4 * TC_EPI_SETS;  // forwards finished score rows to the peers of a multi-GPU scan
static constexpr int TC_THREADS = 32 * (TC_SEND_WARP + 1);
static_assert(TC_EPI_SETS == 4, "region-aligned tiles pair the four warps of a lane quarter with the two accumulator slots");
static constexpr unsigned long long TC_TIMEOUT = 200000000ull;    // default deadline of a wait, clock cycles (about 0.1 s)

static constexpr int DB_TC_MAX_PEERS = 8;

struct tc_args {
	const uint8_t* X; const uint32_t* R; const __nv_bfloat16* Wt; const float* bias;
	const float* headW; const float* headB;
	float* pooled; float* scores; int* status;
	unsigned npos, n, nregion, nf, m, KC, nsplit, seqs_per_cta, nmodel;
	int ptype, relu;
	unsigned f16;                   // operand type of both MMA inputs: 0 = bf16, 1 = f16 (weights prescaled by a power of two)
	unsigned rep;                   // at most 32 filters: the filter block is repeated in every lane quarter (see tc_replicated)
	const uint32_t* maxabs;         // bit pattern of max |W|, kept behind the prepared tiles
	float* peers[DB_TC_MAX_PEERS];  // score matrices of the ranks of a multi-GPU scan (peer-mapped), or none
	unsigned npeer, row_off;        // this launch's region g is row row_off + g of each of them
	unsigned long long timeout;     // clock cycles a wait may last before the CTA gives up
	unsigned hold_operands;         // test aid: the operand encoders never announce their stage, so the issuer's wait runs out
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
// (A try_wait with a suspend-time hint instead of the short sleep was measured
// 10 % slower: the waiters wake later than they do from a 40 ns sleep.)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, unsigned long long timeout)
{
	if (mbar_try_wait(bar, parity)) return true;
	const unsigned long long t0 = clock64();
	while (true) {
		if (mbar_try_wait(bar, parity)) return true;
		if (*abort_flag) return false;
		if (clock64() - t0 > timeout) { *abort_flag = 1; return false; }
		__nanosleep(40);        // a spinning warp would take issue slots from the epilogue warp of its scheduler
	}
}
// The same for a counter in shared memory that only grows.
__device__ __forceinline__ bool count_wait(volatile unsigned* cnt, unsigned need, volatile int* abort_flag, unsigned long long timeout)
{
	if (*cnt >= need) return true;
	const unsigned long long t0 = clock64();
	while (true) {
		if (*cnt >= need) return true;
		if (*abort_flag) return false;
		if (clock64() - t0 > timeout) { *abort_flag = 1; return false; }
		__nanosleep(100);
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
// The same with the accumulate flag fixed at compile time (the predicate folds away).
template <bool ACC>
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc)
{
	if (ACC)
		asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\t"
		             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
		             :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
	else
		asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, 0, 0;\n\t"
		             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
		             :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
// All MMAs of one accumulator tile: per piece of the weights NK steps of K = 16.  The A
// tiles of all pieces are contiguous (4096 bytes = 256 descriptor units per MMA), B
// advances 64 bytes (4 units) per MMA and restarts for each piece.  NK > 0 unrolls the
// steps with immediate offsets: the issuing thread is alone in its warp, so every
// instruction it spends between two MMAs is latency the tensor pipe sits idle for.
template <int NK>
__device__ __forceinline__ void umma_tile(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, unsigned nsplit, unsigned nk)
{
	if (NK > 0) {
		umma_f16<false>(d, adesc, bdesc, idesc);
		#pragma unroll
		for (int kk = 1; kk < NK; ++kk) umma_f16<true>(d, adesc + 256u * kk, bdesc + 4u * kk, idesc);
		for (unsigned s = 1; s < nsplit; ++s) {
			adesc += 256u * NK;
			#pragma unroll
			for (int kk = 0; kk < NK; ++kk) umma_f16<true>(d, adesc + 256u * kk, bdesc + 4u * kk, idesc);
		}
	} else {
		unsigned acc = 0;
		for (unsigned s = 0; s < nsplit; ++s)
			for (unsigned kk = 0; kk < nk; ++kk) {
				umma_bf16(d, adesc, bdesc + 4u * kk, idesc, acc);
				acc = 1; adesc += 256u;
			}
	}
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
// Instruction descriptor: D = F32, A = B = BF16 (format 1) or F16 (format 0), both
// K-major, M = 128, N given.
__device__ __forceinline__ uint32_t instr_desc(unsigned N, unsigned f16)
{
	const unsigned fmt = f16 ? 0u : 1u;
	return (1u << 4) | (fmt << 7) | (fmt << 10) | ((N >> 3) << 17) | ((128u >> 4) << 24);
}

// f16 operands: the weights are multiplied by the power of two that brings the
// largest magnitude into [2^13, 2^14) before they are split, so that the second
// piece stays a normal f16 number; the epilogue pools in the scaled domain (bias
// scaled alike) and multiplies the pooled values by the inverse.  Exact: powers of two.
__host__ __device__ __forceinline__ float tc_weight_scale(uint32_t maxabs_bits)
{
	int e = (int)((maxabs_bits >> 23) & 0xffu) - 127;          // floor(log2(max |W|))
	if ((maxabs_bits & 0x7fffffffu) == 0u || e < -60 || e > 60) return 1.f;
	const uint32_t bits = (uint32_t)(13 - e + 127) << 23;
#ifdef __CUDA_ARCH__
	return __uint_as_float(bits);
#else
	float f; memcpy(&f, &bits, 4); return f;
#endif
}

// One-hot (or 1/4, or zero) pattern of a base as four 16-bit floats in 64 bits, channel c at
// bits [16c, 16c+16).  1.0 and 0.25 are 0x3F80 / 0x3E80 in bf16 and 0x3C00 / 0x3400 in f16.
__device__ __forceinline__ unsigned long long base_pattern(unsigned x, unsigned f16)
{
	if (x < 4u) return (f16 ? 0x3C00ull : 0x3F80ull) << (16u * x);
	if (x == 254u) return 0ull;                        // dropped input
	return f16 ? 0x3400340034003400ull : 0x3E803E803E803E80ull;
}


#define COMMA ,
// Narrow TMEM loads for the tail of a region segment (32 lanes x N columns, one
// register per column), written into a sub-range of a 32-register buffer.
#define DB_TMEM_LD_SMALL(NAME, N, REGS_OUT, REGS_FMT)                                              \
__device__ __forceinline__ void NAME(uint32_t taddr, float* v)                                     \
{                                                                                                  \
	uint32_t* r = reinterpret_cast<uint32_t*>(v);                                                  \
	asm volatile("tcgen05.ld.sync.aligned.32x32b.x" #N ".b32 {" REGS_FMT "}, [%" #N "];"            \
	             : REGS_OUT : "r"(taddr) : "memory");                                              \
}
DB_TMEM_LD_SMALL(tmem_ld16, 16,
	"=r"(r[0]) COMMA "=r"(r[1]) COMMA "=r"(r[2]) COMMA "=r"(r[3]) COMMA "=r"(r[4]) COMMA "=r"(r[5]) COMMA "=r"(r[6]) COMMA "=r"(r[7]) COMMA
	"=r"(r[8]) COMMA "=r"(r[9]) COMMA "=r"(r[10]) COMMA "=r"(r[11]) COMMA "=r"(r[12]) COMMA "=r"(r[13]) COMMA "=r"(r[14]) COMMA "=r"(r[15]),
	"%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15")
DB_TMEM_LD_SMALL(tmem_ld8, 8,
	"=r"(r[0]) COMMA "=r"(r[1]) COMMA "=r"(r[2]) COMMA "=r"(r[3]) COMMA "=r"(r[4]) COMMA "=r"(r[5]) COMMA "=r"(r[6]) COMMA "=r"(r[7]),
	"%0, %1, %2, %3, %4, %5, %6, %7")
DB_TMEM_LD_SMALL(tmem_ld4, 4, "=r"(r[0]) COMMA "=r"(r[1]) COMMA "=r"(r[2]) COMMA "=r"(r[3]), "%0, %1, %2, %3")
DB_TMEM_LD_SMALL(tmem_ld2, 2, "=r"(r[0]) COMMA "=r"(r[1]), "%0, %1")
DB_TMEM_LD_SMALL(tmem_ld1, 1, "=r"(r[0]), "%0")

// Requests the next min(n, 32) columns starting at `ta` (no wait): see pool_state::add_piece.
__device__ __forceinline__ void load_piece(uint32_t ta, unsigned n, float (&v)[32])
{
	if (n >= 32) { tmem_ld32(ta, v); return; }
	if (n & 16) { tmem_ld16(ta, v); ta += 16; }
	if (n & 8)  { tmem_ld8(ta, v + 16); ta += 8; }
	if (n & 4)  { tmem_ld4(ta, v + 24); ta += 4; }
	if (n & 2)  { tmem_ld2(ta, v + 28); ta += 2; }
	if (n & 1)  { tmem_ld1(ta, v + 30); }
}

// Running pooling state of one filter over the rows of one region.  Four
// independent chains keep a lone warp issuing; there are no per-column tests:
// the columns of a region are fetched from tensor memory starting at the
// region's own first column, in pieces of 64/32/16/8/4/2/1.
// Blackwell-only arithmetic: a three-input maximum and a packed pair of FP32 adds
// (one issue slot each), which trim the per-column cost of the reduction.
__device__ __forceinline__ float max3(float a, float b, float c)
{
	float d;
	asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
	return d;
}
__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
	unsigned long long r;
	asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
	return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b)
{
	unsigned long long r;
	asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
	return r;
}

__device__ __forceinline__ float fma_sat(float x, float m, float c)
{
	float d;
	asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(x), "f"(m), "f"(c));
	return d;
}
// A power of two strictly above `bound` (> 0, finite); 1 for a zero bound.
__device__ __forceinline__ float pow2_above(float bound)
{
	const uint32_t bits = __float_as_uint(bound);
	int e = (int)((bits >> 23) & 0xffu) - 127;
	if ((bits & 0x7fffffffu) == 0u) return 1.f;
	e = max(-100, min(100, e));
	return __uint_as_float((uint32_t)(e + 1 + 127) << 23);
}

// A score goes to the caller's matrix and, in a multi-GPU scan, straight into every rank's
// gathered matrix over NVLink (plain peer stores; posted writes, nothing is read back): the
// all-gather of the score shards happens inside the scan, column by column, and costs no
// pass of its own.  The ranks synchronise after their launches before anyone reads.
template <bool PEERS>
__device__ __forceinline__ void store_score(const tc_args& a, unsigned g, unsigned model, float v)
{
	const size_t o = (size_t)g * a.nmodel + model;
	if (a.scores) a.scores[o] = v;
	if (PEERS) {
		const size_t po = (size_t)a.row_off * a.nmodel + o;
		for (unsigned p = 0; p < a.npeer; ++p) a.peers[p][po] = v;
	}
}

struct pool_state {
	float mx[4];
	unsigned long long sm2[4];      // four packed pairs of partial sums
	float sm1;                      // scalar partial sum (tails shorter than 8 columns)
	__device__ __forceinline__ void reset()
	{
		#pragma unroll
		for (int j = 0; j < 4; ++j) { mx[j] = -INFINITY; sm2[j] = 0ull; }
		sm1 = 0.f;
	}
	// The maximum takes the raw accumulator x (bias and rectifier commute with it and
	// are applied once per region).  The sum takes the rectified activation as
	// relu_term(x) = sat(x*cm + ca) = relu(z + b) / S: one saturating FMA on the FMA
	// pipe instead of an add and a maximum (the FP32 maximum issues at half rate),
	// with S a power of two above any activation of this filter, so that the upper
	// clamp of .sat never acts and the scaling is exact.
	template <bool WANT_MAX, bool WANT_SUM, bool RELU, int N>
	__device__ __forceinline__ void add(const float* v, float cm, float ca)
	{
		if (N >= 8) {
			#pragma unroll
			for (int i = 0; i < N; i += 8) {
				#pragma unroll
				for (int j = 0; j < 4; ++j) {
					const float x0 = v[i + 2 * j], x1 = v[i + 2 * j + 1];
					if (WANT_MAX) mx[j] = max3(mx[j], x0, x1);
					if (WANT_SUM) sm2[j] = add2(sm2[j], pack2(RELU ? fma_sat(x0, cm, ca) : x0, RELU ? fma_sat(x1, cm, ca) : x1));
				}
			}
		} else {
			#pragma unroll
			for (int i = 0; i < N; ++i) {
				if (WANT_MAX) mx[i & 3] = fmaxf(mx[i & 3], v[i]);
				if (WANT_SUM) sm1 += RELU ? fma_sat(v[i], cm, ca) : v[i];
			}
		}
	}
	// A piece of n <= 32 columns in a 32-register buffer: a full piece fills it; a
	// shorter one keeps its 16/8/4/2/1-column parts at fixed offsets 0/16/24/28/30.
	template <bool WANT_MAX, bool WANT_SUM, bool RELU>
	__device__ __forceinline__ void add_piece(const float (&v)[32], unsigned n, float cm, float ca)
	{
		if (n >= 32) { add<WANT_MAX, WANT_SUM, RELU, 32>(v, cm, ca); return; }
		if (n & 16) add<WANT_MAX, WANT_SUM, RELU, 16>(v, cm, ca);
		if (n & 8)  add<WANT_MAX, WANT_SUM, RELU, 8>(v + 16, cm, ca);
		if (n & 4)  add<WANT_MAX, WANT_SUM, RELU, 4>(v + 24, cm, ca);
		if (n & 2)  add<WANT_MAX, WANT_SUM, RELU, 2>(v + 28, cm, ca);
		if (n & 1)  add<WANT_MAX, WANT_SUM, RELU, 1>(v + 30, cm, ca);
	}
	// `cnt` rows whose scan output is zero
	template <bool WANT_MAX, bool WANT_SUM, bool RELU>
	__device__ __forceinline__ void add_zero_rows(unsigned cnt, float cm, float ca)
	{
		if (WANT_MAX) mx[0] = fmaxf(mx[0], 0.f);
		if (WANT_SUM && RELU) sm1 += (float)cnt * fma_sat(0.f, cm, ca);
	}
	__device__ __forceinline__ float max_all() const { return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])); }
	__device__ __forceinline__ float sum_all() const
	{
		const unsigned long long t = add2(add2(sm2[0], sm2[1]), add2(sm2[2], sm2[3]));
		float lo, hi;
		asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(t));
		return (lo + hi) + sm1;
	}
};

// With at most 32 filters only one of the four TMEM lane quarters would hold results, and a
// lane quarter can only be read by the warps of one SM sub-partition: one scheduler would do
// the whole epilogue.  So the prepared operand repeats the filter block in all four quarters
// (the tile has 128 rows either way), every quarter holds every filter, and the sixteen epilogue
// warps share the regions instead of the filters: four schedulers work on the pooling.
__host__ __device__ inline bool tc_replicated(unsigned nf) { return nf <= 32u; }

template <bool WANT_MAX, bool WANT_SUM, bool RELU>
__device__ __forceinline__ void tc_epilogue(const tc_args& a, uint32_t tmem_base, uint64_t* t_full, uint64_t* t_empty,
                                            volatile int* abort_flag, unsigned tile, unsigned g_first, unsigned g_last,
                                            unsigned row_lo, unsigned row_hi, unsigned warp, unsigned lane)
{
	const unsigned q4 = warp & 3;                       // TMEM lane quarter of this warp
	const unsigned set = (warp - TC_EPI_WARP0) >> 2;    // the warps of a quarter take the regions in turn
	// this thread's filter = its TMEM lane; with a repeated filter block, its lane within the quarter
	const unsigned f = a.rep ? lane : tile * 128 + q4 * 32 + lane;
	// regions this warp reduces: every gstep-th from g_first + gidx on
	const unsigned gstep = a.rep ? 4u * TC_EPI_SETS : (unsigned)TC_EPI_SETS;
	const unsigned gidx = a.rep ? set * 4u + q4 : set;
	const uint32_t maxabs_bits = *a.maxabs;
	const float wscale = a.f16 ? tc_weight_scale(maxabs_bits) : 1.f, inv_wscale = 1.f / wscale;    // powers of two
	const float b0 = (a.bias && f < a.nf) ? a.bias[f] : 0.f;
	const float b = b0 * wscale;                        // bias in the accumulator's (scaled) domain
	// |z + b| <= m * max|W| + |b|: the scale of the saturating rectifier (see pool_state::add)
	const float ssat = pow2_above((float)a.m * __uint_as_float(maxabs_bits) + fabsf(b0));
	const float cm = inv_wscale / ssat, ca = b0 / ssat;
	// linear head of the model this filter belongs to (16 filters per model)
	float hw_max = 0.f, hw_sum = 0.f, hb = 0.f;
	const unsigned model = f / 16;
	if ((a.scores || a.npeer) && f < a.nf) {
		const unsigned npool = a.ptype == DB_PT_ALL ? 32u : 16u, k = f % 16;
		if (a.ptype == DB_PT_ALL) { hw_max = a.headW[model * npool + 2 * k]; hw_sum = a.headW[model * npool + 2 * k + 1]; }
		else if (a.ptype == DB_PT_MAX) hw_max = a.headW[model * npool + k];
		else hw_sum = a.headW[model * npool + k];
		hb = a.headB ? a.headB[model] : 0.f;
	}
	pool_state ps;
	ps.reset();
	// This warp reduces the regions g_first + gidx, + gstep, ... and never looks at the others.
	unsigned g = g_first + gidx;
	unsigned r0 = 0, r1 = 0;                            // bounds of the region being reduced
	unsigned nr0 = 0, nr1 = 0, nprev = 0;               // bounds of this warp's next region and the end of the one before it, loaded ahead
	bool ok = true;
	if (g < g_last) {
		r0 = a.R[2 * g]; r1 = max(a.R[2 * g + 1], r0);
		if (g > g_first && r0 < a.R[2 * g - 1]) {      // regions must ascend without overlap
			if (lane == 0) { *abort_flag = 1; atomicExch(a.status, 3); }
			ok = false;
		}
	}
	auto fetch_next = [&]() {
		const unsigned h = g + gstep;
		if (h < g_last) {
			const uint2 r = reinterpret_cast<const uint2*>(a.R)[h];      // regions are (start, end) pairs: cudaMalloc alignment
			nr0 = r.x; nr1 = r.y; nprev = a.R[2 * h - 1];
		}
	};
	fetch_next();

	// Writes region g's outputs and moves to this warp's next region.
	auto finish_region = [&]() -> bool {
		const unsigned P = r1 - r0;
		float pmax = ps.max_all() + b;                 // max_p relu(z_p + b) = relu(max_p z_p + b)
		pmax = (RELU ? fmaxf(pmax, 0.f) : pmax) * inv_wscale;
		// rectified: the terms were relu(z_p + b) / ssat; otherwise they were the raw accumulators
		const float psum = RELU ? ps.sum_all() * ssat : ps.sum_all() * inv_wscale + (float)P * b0;
		const float second = a.ptype == DB_PT_SUM ? psum : __fdividef(psum, (float)P);
		if (a.pooled && f < a.nf) {
			const size_t o = (size_t)g * a.nf + f;
			if (a.ptype == DB_PT_ALL) reinterpret_cast<float2*>(a.pooled)[o] = make_float2(pmax, second);
			else a.pooled[o] = WANT_MAX ? pmax : second;
		}
		if (a.scores || a.npeer) {
			float part = (WANT_MAX ? hw_max * pmax : 0.f) + (WANT_SUM ? hw_sum * second : 0.f);
			part += __shfl_xor_sync(0xffffffffu, part, 8);
			part += __shfl_xor_sync(0xffffffffu, part, 4);
			part += __shfl_xor_sync(0xffffffffu, part, 2);
			part += __shfl_xor_sync(0xffffffffu, part, 1);
			if ((lane & 15) == 0 && f < a.nf) store_score<true>(a, g, model, part + hb);
		}
		ps.reset();
		g += gstep;
		if (g >= g_last) return true;
		r0 = nr0; r1 = max(nr1, nr0);
		const bool bad = r0 < nprev;                   // regions must ascend without overlap
		fetch_next();
		if (bad) {
			if (lane == 0) { *abort_flag = 1; atomicExch(a.status, 3); }
			return false;
		}
		return true;
	};

	const unsigned ntile = (row_hi - row_lo + 255u) / 256u;
	for (unsigned t = 0; ok && t < ntile; ++t) {       // every tile is consumed, so the issuer never waits on us in vain
		const unsigned slot = t & 1;
		// Usually the tile is ready: every lane tests the barrier once.  Otherwise lane 0
		// waits (bounded) and the warp stays converged for the aligned TMEM loads.
		if (!__all_sync(0xffffffffu, mbar_try_wait(&t_full[slot], (t >> 1) & 1))) {
			unsigned okv = 0;
			if (lane == 0) okv = mbar_wait(&t_full[slot], (t >> 1) & 1, abort_flag, a.timeout) ? 1u : 0u;
			ok = __shfl_sync(0xffffffffu, okv, 0) != 0;
			if (!ok) break;
			mbar_try_wait(&t_full[slot], (t >> 1) & 1);    // completed: every lane observes the phase
		}
		tc_fence_after();
		const unsigned tile_lo = row_lo + t * 256u, tile_hi = min(tile_lo + 256u, row_hi);
		const uint32_t taddr = tmem_base + ((q4 * 32u) << 16) + slot * 256u;
		bool released = false;
		while (ok && g < g_last && r0 < tile_hi) {
			const unsigned pos = max(r0, tile_lo), end = min(r1, tile_hi);
			if (end > pos) {
				// rows at or past n have no scan output (kangaroo_smat.cpp:105): they read as zero
				const unsigned live_end = min(end, max(pos, a.n));
				uint32_t ta = taddr + (pos - tile_lo);
				unsigned left = live_end - pos;
				// 64 columns per TMEM round trip (40-60 clocks, hidden by the other warps of
				// the scheduler), then the remaining 0..63 columns with one more wait.
				float va[32];
				while (left >= 32) {
					tmem_ld32(ta, va);
					tmem_ld_wait();
					ps.add<WANT_MAX, WANT_SUM, RELU, 32>(va, cm, ca);
					ta += 32; left -= 32;
				}
				if (left) {
					load_piece(ta, left, va);
					tmem_ld_wait();
					ps.add_piece<WANT_MAX, WANT_SUM, RELU>(va, left, cm, ca);
				}
				if (live_end < end) ps.add_zero_rows<WANT_MAX, WANT_SUM, RELU>(end - live_end, cm, ca);
			}
			if (r1 > tile_hi) break;                       // the region continues in the next tile
			// The warp's last columns of this tile are in registers once its next region starts
			// beyond the tile: the tile goes back before the region's outputs are worked out.
			if (!released && !(g + gstep < g_last && nr0 < tile_hi)) {
				tc_fence_before();
				__syncwarp();
				if (lane == 0) mbar_arrive(&t_empty[slot]);
				released = true;
			}
			ok = finish_region();
		}
		if (!released) {
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(&t_empty[slot]);
		}
	}
	// regions that end exactly where the data ends (and empty regions after it)
	while (ok && g < g_last) ok = finish_region();
}

// Epilogue for region-aligned tiles (uniform batches): tile t holds the CTA's regions
// t*k .. t*k+k-1, region j of it at column j*S, P columns long.  The four warps of a
// lane quarter split into two pairs: one follows the even tiles (accumulator slot 0),
// the other the odd tiles (slot 1), so every warp sees every phase of the one slot it
// waits on; the two warps of a pair take the regions of a tile alternately.  A region is
// always whole: wait for the tile, reduce the P columns, write the outputs; the tile goes
// back once the warp has read its last region of it.
template <bool WANT_MAX, bool WANT_SUM, bool RELU>
__device__ __forceinline__ void tc_epilogue_uniform(const tc_args& a, uint32_t tmem_base, uint64_t* t_full, uint64_t* t_empty,
                                                    volatile int* abort_flag, unsigned tile, unsigned g_first, unsigned nreg,
                                                    unsigned P, unsigned S, unsigned k, unsigned warp, unsigned lane,
                                                    unsigned* done_cnt)
{
	const unsigned q4 = warp & 3;                       // TMEM lane quarter of this warp
	const unsigned set = (warp - TC_EPI_WARP0) >> 2;
	const unsigned f = tile * 128 + q4 * 32 + lane;     // this thread's filter = its TMEM lane
	const uint32_t maxabs_bits = *a.maxabs;
	const float wscale = a.f16 ? tc_weight_scale(maxabs_bits) : 1.f, inv_wscale = 1.f / wscale;    // powers of two
	const float b0 = (a.bias && f < a.nf) ? a.bias[f] : 0.f;
	const float b = b0 * wscale;
	const float ssat = pow2_above((float)a.m * __uint_as_float(maxabs_bits) + fabsf(b0));
	const float cm = inv_wscale / ssat, ca = b0 / ssat;
	float hw_max = 0.f, hw_sum = 0.f, hb = 0.f;
	const unsigned model = f / 16;
	if ((a.scores || a.npeer) && f < a.nf) {
		const unsigned npool = a.ptype == DB_PT_ALL ? 32u : 16u, kk = f % 16;
		if (a.ptype == DB_PT_ALL) { hw_max = a.headW[model * npool + 2 * kk]; hw_sum = a.headW[model * npool + 2 * kk + 1]; }
		else if (a.ptype == DB_PT_MAX) hw_max = a.headW[model * npool + kk];
		else hw_sum = a.headW[model * npool + kk];
		hb = a.headB ? a.headB[model] : 0.f;
	}
	const float fP = (float)P;
	const unsigned slot = set >> 1, sub = set & 1;      // this warp's accumulator slot and its place in the slot's pair
	const unsigned ntile = (nreg + k - 1) / k;
	const uint32_t slot_base = tmem_base + ((q4 * 32u) << 16) + slot * 256u;
	pool_state ps;
	unsigned par = 0;
	for (unsigned t = slot; t < ntile; t += 2, par ^= 1) {
		if (!__all_sync(0xffffffffu, mbar_try_wait(&t_full[slot], par))) {
			unsigned okv = 0;
			if (lane == 0) okv = mbar_wait(&t_full[slot], par, abort_flag, a.timeout) ? 1u : 0u;
			if (__shfl_sync(0xffffffffu, okv, 0) == 0) return;
			mbar_try_wait(&t_full[slot], par);          // completed: every lane observes the phase
		}
		tc_fence_after();
		const unsigned kt = min(k, nreg - t * k);       // regions in this tile
		for (unsigned j = sub; j < kt; j += 2) {
			uint32_t ta = slot_base + j * S;
			ps.reset();
			unsigned left = P;
			float va[32];
			#pragma unroll 1                            // P is loop-invariant: unrolled copies would only cost registers
			while (left >= 32) {
				tmem_ld32(ta, va);
				tmem_ld_wait();
				ps.add<WANT_MAX, WANT_SUM, RELU, 32>(va, cm, ca);
				ta += 32; left -= 32;
			}
			if (left) {
				load_piece(ta, left, va);
				tmem_ld_wait();
				ps.add_piece<WANT_MAX, WANT_SUM, RELU>(va, left, cm, ca);
			}
			if (j + 2 >= kt) {                          // last region of this warp in the tile: the tile goes back first
				tc_fence_before();
				__syncwarp();
				if (lane == 0) mbar_arrive(&t_empty[slot]);
			}
			const unsigned g = g_first + t * k + j;
			float pmax = ps.max_all() + b;              // max_p relu(z_p + b) = relu(max_p z_p + b)
			pmax = (RELU ? fmaxf(pmax, 0.f) : pmax) * inv_wscale;
			const float psum = RELU ? ps.sum_all() * ssat : ps.sum_all() * inv_wscale + fP * b0;
			const float second = a.ptype == DB_PT_SUM ? psum : __fdividef(psum, fP);
			if (a.pooled && f < a.nf) {
				const size_t o = (size_t)g * a.nf + f;
				if (a.ptype == DB_PT_ALL) reinterpret_cast<float2*>(a.pooled)[o] = make_float2(pmax, second);
				else a.pooled[o] = WANT_MAX ? pmax : second;
			}
			if (a.scores || a.npeer) {
				float part = (WANT_MAX ? hw_max * pmax : 0.f) + (WANT_SUM ? hw_sum * second : 0.f);
				part += __shfl_xor_sync(0xffffffffu, part, 8);
				part += __shfl_xor_sync(0xffffffffu, part, 4);
				part += __shfl_xor_sync(0xffffffffu, part, 2);
				part += __shfl_xor_sync(0xffffffffu, part, 1);
				// a multi-GPU scan writes its own matrix here; the sender warp forwards whole rows of
				// the tile to the peers once all warps of the slot are through with it
				if ((lane & 15) == 0 && f < a.nf) store_score<false>(a, g, model, part + hb);
			}
		}
		if (sub >= kt) {                                // no region of this tile is ours: hand it back untouched
			tc_fence_before();
			__syncwarp();
			if (lane == 0) mbar_arrive(&t_empty[slot]);
		}
		if (a.npeer) {                                  // this warp's scores of the tile are written: tell the sender
			__syncwarp();
			if (lane == 0) { __threadfence_block(); atomicAdd(&done_cnt[slot], 1u); }
		}
	}
}

// Multi-GPU scan, region-aligned tiles: the sender warp waits until the eight epilogue warps
// of a tile's slot have written the tile's scores to this rank's matrix, reads the tile's
// rows back (eight consecutive scores per region and filter tile: one 32-byte sector, still
// in L2) and stores each as one 32-byte run into every peer's matrix: an NVLink write packet
// per (region, tile, peer).  The epilogue warps, which bound the kernel, only bump a
// counter.  The counters only grow, so a sender that falls behind is never overtaken.
__device__ __forceinline__ void tc_send_rows(const tc_args& a, volatile int* abort_flag, unsigned tile, unsigned g_first,
                                             unsigned nreg, unsigned k, unsigned lane, unsigned* done_cnt)
{
	const unsigned ntile = (nreg + k - 1) / k;
	const unsigned col = tile * 8u + (lane & 7u);
	for (unsigned t = 0; t < ntile; ++t) {
		unsigned okv = 0;
		if (lane == 0) okv = count_wait(&done_cnt[t & 1u], 2u * TC_EPI_SETS * (t / 2u + 1u), abort_flag, a.timeout) ? 1u : 0u;
		if (__shfl_sync(0xffffffffu, okv, 0) == 0) return;
		__threadfence_block();
		const unsigned kt = min(k, nreg - t * k);
		for (unsigned j = lane >> 3; j < kt; j += 4) {
			if (col >= a.nmodel) continue;
			const size_t o = (size_t)(g_first + t * k + j) * a.nmodel + col;
			const float v = __ldcg(a.scores + o);
			const size_t po = (size_t)a.row_off * a.nmodel + o;
			for (unsigned p = 0; p < a.npeer; ++p) a.peers[p][po] = v;
		}
	}
}

#undef COMMA

__global__ void __launch_bounds__(TC_THREADS, 1)
scanpool_tc_kernel(const tc_args a)
{
	extern __shared__ __align__(128) unsigned char smem[];
	const unsigned KC = a.KC, NK = KC / 2;
	const unsigned a_bytes = a.nsplit * KC * 2048u;
	unsigned char* As = smem;                                    // [nsplit][KC][128][8] bf16
	unsigned char* Es = smem + a_bytes;                          // [2][TC_ECHUNKS] 16-byte chunks
	__shared__ __align__(8) uint64_t bar_a, bar_fin, e_full[2], e_empty[2], t_full[2], t_empty[2];
	__shared__ uint32_t tmem_base_s;
	__shared__ unsigned rows_s[2], blk_ok[2];
	__shared__ int abort_s;
	__shared__ unsigned done_cnt[2];
	volatile int* abort_flag = &abort_s;

	const unsigned warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
	const unsigned tile = blockIdx.x;
	const unsigned g_first = blockIdx.y * a.seqs_per_cta;
	const unsigned g_last = min(a.nregion, g_first + a.seqs_per_cta);

	// A CTA of a launch that has already failed returns at once.  One thread reads
	// the status word so that the whole CTA takes the same decision.
	if (threadIdx.x < 2) done_cnt[threadIdx.x] = 0u;
	if (threadIdx.x == 0) {
		abort_s = *reinterpret_cast<volatile int*>(a.status);
		if (a.maxabs[1] != 0u) {                                    // a weight was Inf or NaN when the bank was prepared
			atomicCAS(a.status, 0, 4);
			abort_s = 4;
		}
		rows_s[0] = a.R[2 * g_first];
		rows_s[1] = max(a.R[2 * (g_last - 1) + 1], rows_s[0]);
	}
	__syncthreads();
	if (abort_s != 0) return;
	// The CTA scans the flat rows [row_lo, row_hi) of its regions in tiles of 256 columns.
	const unsigned row_lo = rows_s[0], row_hi = rows_s[1];
	// Uniform batches (every region of this CTA P rows long, starting S rows after the one
	// before: what equal-length sequences give) take region-aligned tiles: a tile starts at
	// a region boundary and holds k whole regions, so no region straddles two tiles and
	// the epilogue needs neither region bounds nor carried state.  Anything else (ragged
	// lengths, gaps, rows past the scanned range) takes flat tiles of 256 rows.
	const unsigned nreg = g_last - g_first;
	const unsigned P0 = a.R[2 * g_first + 1] - a.R[2 * g_first];
	const unsigned S0 = nreg > 1 ? a.R[2 * g_first + 2] - a.R[2 * g_first] : P0;
	bool same = !a.rep && P0 >= 1u && P0 <= 256u && S0 >= P0 && S0 <= 256u && row_hi <= a.n;
	for (unsigned i = threadIdx.x; same && i < nreg; i += TC_THREADS) {
		const uint2 r = reinterpret_cast<const uint2*>(a.R)[g_first + i];
		same = r.x == row_lo + i * S0 && r.y - r.x == P0;
	}
	const bool uni = __syncthreads_and(same) != 0;
	const unsigned kreg = uni ? (256u - P0) / S0 + 1u : 0u;         // whole regions per tile
	const unsigned tstep = uni ? kreg * S0 : 256u;                  // rows from one tile's first column to the next's
	const unsigned ntile = uni ? (nreg + kreg - 1u) / kreg : (row_hi - row_lo + 255u) / 256u;
	if (threadIdx.x == 0) {
		mbar_init(&bar_a, 1); mbar_init(&bar_fin, 1);
		for (int i = 0; i < 2; ++i) {
			mbar_init(&e_full[i], TC_BUILD_WARPS); mbar_init(&e_empty[i], 1);
			// a tile is released by every warp that follows its slot: all of them (flat tiles),
			// or the pair of each lane quarter bound to the slot (region-aligned tiles)
			mbar_init(&t_full[i], 1); mbar_init(&t_empty[i], uni ? 2 * TC_EPI_SETS : 4 * TC_EPI_SETS);
		}
		asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
	}
	if (warp == 0) tmem_alloc(&tmem_base_s, 512);
	tc_fence_before();
	__syncthreads();
	tc_fence_after();
	const uint32_t tmem_base = tmem_base_s;

	if (warp == 0) {
		// ------------------------------------------------------------ MMA issuer
		if (lane == 0) {
			mbar_expect_tx(&bar_a, a_bytes);
			bulk_g2s(As, reinterpret_cast<const unsigned char*>(a.Wt) + (size_t)tile * a_bytes, a_bytes, &bar_a);
			bool ok = mbar_wait(&bar_a, 0, abort_flag, a.timeout);
			const uint32_t a_addr = smem_u32(As), e_addr = smem_u32(Es);
			// Shared-memory descriptors (see smem_desc): 8-row group stride 128 B; A's K-chunk
			// stride 2048 B, B's 32 B.  Only the start-address field (16-byte units) changes
			// from MMA to MMA, and it never carries out of its 14 bits inside shared memory.
			const uint64_t desc_hi = (uint64_t)((128u >> 4) | (1u << 14)) << 32;
			const uint64_t adesc = desc_hi | (((a_addr >> 4) & 0x3fffu) | ((2048u >> 4) << 16));
			const uint64_t bstage0 = desc_hi | (((e_addr >> 4) & 0x3fffu) | ((32u >> 4) << 16));
			const uint32_t idesc_full = instr_desc(256u, a.f16);
			// Running state instead of divisions per tile: place in the operand stage, stage
			// buffer and its parity, parity of the accumulator slots, rows still to scan.
			unsigned tt = 0, st = 0, par_e = 0, par_t = 1;
			unsigned rows_left = row_hi - row_lo;
			uint64_t bdesc = bstage0;
			for (unsigned t = 0; ok && t < ntile; ++t) {
				if (tt == 0) {
					ok = mbar_wait(&e_full[st], par_e, abort_flag, a.timeout);
					if (!ok) break;
				}
				const unsigned slot = t & 1;
				ok = mbar_wait(&t_empty[slot], par_t, abort_flag, a.timeout);
				if (!ok) break;
				tc_fence_after();
				const uint32_t idesc = rows_left >= 256u ? idesc_full : instr_desc((rows_left + 15u) & ~15u, a.f16);
				const uint32_t d = tmem_base + slot * 256u;
				if (NK == 6) umma_tile<6>(d, adesc, bdesc, idesc, a.nsplit, NK);
				else if (NK == 4) umma_tile<4>(d, adesc, bdesc, idesc, a.nsplit, NK);
				else umma_tile<0>(d, adesc, bdesc, idesc, a.nsplit, NK);
				umma_commit(&t_full[slot]);
				++tt; bdesc += tstep;                       // the next tile's rows start tstep chunks further on
				rows_left = rows_left > tstep ? rows_left - tstep : 0u;
				par_t ^= slot;                              // both slots have been used once more after an odd tile
				if (tt == TC_STAGE_TILES || t + 1 == ntile) {
					umma_commit(&e_empty[st]);              // the stage may be rewritten once the MMAs that read it have finished
					tt = 0; st ^= 1; par_e ^= (st == 0);
					bdesc = bstage0 + st * (unsigned)TC_ECHUNKS;
				}
			}
			// Leaving early (a wait ran out, or another role gave up): the tensor memory is
			// released below, so every MMA issued so far has to finish first.  The commit
			// arrives on bar_fin when they have; that wait is bounded like any other.
			if (*abort_flag) {
				umma_commit(&bar_fin);
				const unsigned long long t0 = clock64();
				while (!mbar_try_wait(&bar_fin, 0) && clock64() - t0 < a.timeout) __nanosleep(40);
			}
		}
	} else if (warp < TC_EPI_WARP0) {
		// ---------------------------------------------------------- E builders
		const unsigned bt = threadIdx.x - 32;     // 0 .. 32*TC_BUILD_WARPS-1
		const unsigned nstage = (ntile + TC_STAGE_TILES - 1) / TC_STAGE_TILES;
		for (unsigned stage = 0; stage < nstage; ++stage) {
			const unsigned st = stage & 1;
			// One thread waits (bounded) and publishes the outcome, so that all
			// builder threads take the same path to the named barrier.
			if (bt == 0) blk_ok[st] = mbar_wait(&e_empty[st], ((stage >> 1) & 1) ^ 1, abort_flag, a.timeout) ? 1u : 0u;
			asm volatile("bar.sync 1, %0;" :: "n"(32 * TC_BUILD_WARPS) : "memory");
			if (blk_ok[st] == 0) break;
			const unsigned base_row = row_lo + stage * (TC_STAGE_TILES * tstep);
			uint4* E = reinterpret_cast<uint4*>(Es + (size_t)st * TC_ECHUNKS * 16);
			// A thread encodes 16 consecutive chunks from 20 bytes fetched as aligned words;
			// the words of its next 16 chunks are requested before it encodes these.
			constexpr unsigned QSTEP = 32 * TC_BUILD_WARPS * 16;
			auto fetch = [&](unsigned q, uint32_t (&w)[6]) {
				const unsigned i0 = base_row + q;
				const size_t addr = (size_t)a.X + i0;
				const uint32_t* wp = reinterpret_cast<const uint32_t*>(addr & ~(size_t)3);
				#pragma unroll
				for (int k = 0; k < 6; ++k)      // a word is read only if its first byte lies inside the buffer
					w[k] = ((long long)i0 + 4 * k - (long long)(addr & 3) < (long long)a.npos) ? wp[k] : 0xfefefefeu;
			};
			uint32_t w[6], wn[6];
			if (bt * 16 < TC_ECHUNKS) fetch(bt * 16, w);
			for (unsigned q = bt * 16; q < TC_ECHUNKS; q += QSTEP) {
				if (q + QSTEP < TC_ECHUNKS) fetch(q + QSTEP, wn);
				const unsigned i0 = base_row + q;
				const unsigned sh = (unsigned)(((size_t)a.X + i0) & 3) * 8;
				uint32_t win[5];
				#pragma unroll
				for (int k = 0; k < 5; ++k) win[k] = __funnelshift_r(w[k], w[k + 1], sh);
				unsigned long long prev = base_pattern(i0 < a.npos ? (win[0] & 0xffu) : 254u, a.f16);
				#pragma unroll
				for (int c = 0; c < 16; ++c) {
					const unsigned x1 = (i0 + c + 1 < a.npos) ? ((win[(c + 1) >> 2] >> (8 * ((c + 1) & 3))) & 0xffu) : 254u;
					const unsigned long long p1 = base_pattern(x1, a.f16);
					E[q + c] = make_uint4((unsigned)prev, (unsigned)(prev >> 32), (unsigned)p1, (unsigned)(p1 >> 32));
					prev = p1;
				}
				#pragma unroll
				for (int k = 0; k < 6; ++k) w[k] = wn[k];
			}
			fence_async_smem();
			__syncwarp();
			if (lane == 0 && !a.hold_operands) mbar_arrive(&e_full[st]);
		}
	} else if (warp == TC_SEND_WARP) {
		// ------------------------------------------------------------ rows to the peers (multi-GPU scan)
		if (uni && a.npeer) tc_send_rows(a, abort_flag, tile, g_first, nreg, kreg, lane, done_cnt);
	} else {
		// ------------------------------------------------------------ epilogue
		#define TC_EPI(MX, SM, RL) do { \
			if (uni) tc_epilogue_uniform<MX, SM, RL>(a, tmem_base, t_full, t_empty, abort_flag, tile, g_first, nreg, P0, S0, kreg, warp, lane, done_cnt); \
			else tc_epilogue<MX, SM, RL>(a, tmem_base, t_full, t_empty, abort_flag, tile, g_first, g_last, row_lo, row_hi, warp, lane); } while (0)
		const bool wm = a.ptype == DB_PT_MAX || a.ptype == DB_PT_ALL, ws = a.ptype != DB_PT_MAX;
		if (a.relu) { if (wm && ws) TC_EPI(true, true, true); else if (wm) TC_EPI(true, false, true); else TC_EPI(false, true, true); }
		else        { if (wm && ws) TC_EPI(true, true, false); else if (wm) TC_EPI(true, false, false); else TC_EPI(false, true, false); }
		#undef TC_EPI
	}
	tc_fence_before();
	__syncthreads();
	if (threadIdx.x == 0 && abort_s) atomicCAS(a.status, 0, 1);
	if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}


// Prepared weights: for each 128-filter tile, `nsplit` K-major 16-bit operand tiles
// in the shared-memory layout [split][K chunk][filter][8], zero padded; behind the
// tiles, 16 bytes whose first word is the bit pattern of max |W| (the prescale of
// the f16 modes and the bound of the epilogue's saturating rectifier derive from it).
__global__ void tc_maxabs_kernel(const float* __restrict__ W, size_t count, uint32_t* __restrict__ out)
{
	uint32_t mx = 0;
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
		const float w = fabsf(W[i]);
		if (w <= 3.4e38f) mx = max(mx, __float_as_uint(w));        // non-negative floats order like their bit patterns
		else out[1] = 1u;                                           // Inf or NaN: the scan refuses the bank (status 4)
	}
	mx = __reduce_max_sync(0xffffffffu, mx);
	if ((threadIdx.x & 31) == 0 && mx) atomicMax(out, mx);
}

__global__ void tc_prepare_kernel(const float* __restrict__ W, unsigned m, unsigned nf, unsigned KC, unsigned nsplit,
                                  unsigned f16, unsigned ntile, uint16_t* __restrict__ out, const uint32_t* __restrict__ maxabs)
{
	const size_t total = (size_t)ntile * KC * 128 * 8;
	const float scale = f16 ? tc_weight_scale(*maxabs) : 1.f;
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
		const unsigned e = i % 8, fl = (i / 8) % 128, kc = (i / 1024) % KC, tile = (unsigned)(i / ((size_t)1024 * KC));
		const unsigned k = kc * 8 + e, f = tc_replicated(nf) ? (fl & 31u) : tile * 128 + fl;
		float w = ((k < 4 * m && f < nf) ? W[(size_t)k * nf + f] : 0.f) * scale;
		for (unsigned s = 0; s < nsplit; ++s) {
			uint16_t bits;
			if (f16) { const __half h = __float2half_rn(w); bits = __half_as_ushort(h); w -= __half2float(h); }
			else { const __nv_bfloat16 h = __float2bfloat16_rn(w); bits = __bfloat16_as_ushort(h); w -= __bfloat162float(h); }
			out[(((size_t)tile * nsplit + s) * KC + kc) * 1024 + fl * 8 + e] = bits;
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

// precision -> (pieces per weight, f16 operands?)
static void tc_mode(int precision, unsigned& nsplit, unsigned& f16)
{
	DB_REQUIRE(precision >= DB_TC_BF16 && precision <= DB_TC_F16,
	           "ValueError: precision must be 1 (bf16), 2 (bf16x2), 3 (bf16x3), 4 (f16x2) or 5 (f16)");
	f16 = precision >= DB_TC_F16X2;
	nsplit = precision == DB_TC_F16X2 ? 2u : precision == DB_TC_F16 ? 1u : (unsigned)precision;
}

// Test aid, per host thread: the deadline of the kernel's waits in clock cycles (0 = the
// default) and whether the operand encoders withhold their "stage ready" signal, which
// makes the issuer's first wait run out with no MMA in flight.  Nothing faults: the
// kernel reports status 1 and returns.
static thread_local float* g_tc_peers[DB_TC_MAX_PEERS];
static thread_local unsigned g_tc_npeer = 0, g_tc_row_off = 0;
static thread_local unsigned long long g_tc_timeout = 0;
static thread_local unsigned g_tc_hold_operands = 0;

DB_EXPORT void db_scanpool_tc_peers(float* const* peer_scores, uint32_t npeer, uint32_t row_offset)
{
	DB_API_TRY_NODEV
	DB_REQUIRE(npeer <= (uint32_t)DB_TC_MAX_PEERS, "ValueError: at most %d peer score matrices (got %u)", DB_TC_MAX_PEERS, npeer);
	DB_REQUIRE(npeer == 0 || peer_scores != nullptr, "ValueError: db_scanpool_tc_peers got a NULL table");
	for (unsigned p = 0; p < npeer; ++p) {
		DB_REQUIRE(peer_scores[p] != nullptr, "ValueError: peer score matrix %u is NULL", p);
		g_tc_peers[p] = peer_scores[p];
	}
	g_tc_npeer = npeer; g_tc_row_off = row_offset;
	DB_API_CATCH
}

DB_EXPORT void db_scanpool_tc_debug(uint64_t timeout_clocks, int hold_operands)
{
	g_tc_timeout = timeout_clocks;
	g_tc_hold_operands = hold_operands ? 1u : 0u;
}

DB_EXPORT size_t db_tc_weights_bytes(uint32_t m, uint32_t nf, int precision)
{
	DB_API_TRY_NODEV
	unsigned KC, ntile, nsplit, f16;
	tc_mode(precision, nsplit, f16);
	tc_shape(m, nf, KC, ntile);
	return (size_t)ntile * nsplit * KC * 2048 + 16;
	DB_API_CATCH_RETURN(0)
}

DB_EXPORT void db_tc_prepare(const float* W, uint32_t m, uint32_t nf, int precision, void* out)
{
	DB_API_TRY
	unsigned KC, ntile, nsplit, f16;
	tc_mode(precision, nsplit, f16);
	DB_REQUIRE(W && out, "ValueError: db_tc_prepare got a NULL pointer");
	DB_REQUIRE(((uintptr_t)out & 15) == 0, "ValueError: prepared-weight buffer must be 16-byte aligned");
	tc_shape(m, nf, KC, ntile);
	uint32_t* trailer = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(out) + (size_t)ntile * nsplit * KC * 2048);
	DB_CUDA(cudaMemsetAsync(trailer, 0, 16, state().stream));
	size_t count = (size_t)4 * m * nf;
	tc_maxabs_kernel<<<elemwise_grid(count), 256, 0, state().stream>>>(W, count, trailer);
	DB_LAUNCH_CHECK();
	size_t total = (size_t)ntile * KC * 1024;
	tc_prepare_kernel<<<elemwise_grid(total), 256, 0, state().stream>>>(W, m, nf, KC, nsplit, f16, ntile, (uint16_t*)out, trailer);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_scanpool_tc(const void* Wt, uint32_t m, uint32_t nf, int precision, const float* bias, int relu,
                              const uint8_t* X, uint32_t npos, const uint32_t* regions, uint32_t nregion, int ptype,
                              float* pooled, const float* headW, const float* headB, uint32_t nmodel, float* scores,
                              int* status)
{
	DB_API_TRY
	DB_REQUIRE(ptype >= DB_PT_MAX && ptype <= DB_PT_ALL, "ValueError: unknown pooling type %d", ptype);
	unsigned nsplit, f16;
	tc_mode(precision, nsplit, f16);
	DB_REQUIRE(status != nullptr, "ValueError: db_scanpool_tc needs a device status word");
	DB_REQUIRE(pooled || scores, "ValueError: db_scanpool_tc needs an output (pooled or scores)");
	if (scores) {
		DB_REQUIRE(headW != nullptr, "ValueError: scores requested without head weights");
		DB_REQUIRE(nmodel * 16 == nf, "ValueError: the fused linear head needs 16 filters per model (nf=%u, nmodel=%u)", nf, nmodel);
	}
	if (nregion == 0) return;
	DB_REQUIRE(Wt && X && regions, "ValueError: db_scanpool_tc got a NULL pointer");
	DB_REQUIRE(((uintptr_t)Wt & 15) == 0, "ValueError: prepared weights must be 16-byte aligned");
	DB_REQUIRE(((uintptr_t)regions & 7) == 0, "ValueError: the region table must be 8-byte aligned");
	unsigned KC, ntile;
	tc_shape(m, nf, KC, ntile);
	tc_args a;
	a.X = X; a.R = regions; a.Wt = (const __nv_bfloat16*)Wt; a.bias = bias; a.headW = headW; a.headB = headB;
	a.pooled = pooled; a.scores = scores; a.status = status;
	a.npos = npos; a.n = npos >= m ? npos - m + 1 : 0; a.nregion = nregion; a.nf = nf; a.m = m; a.KC = KC; a.nsplit = nsplit;
	a.nmodel = nmodel; a.ptype = ptype; a.relu = relu; a.f16 = f16; a.rep = tc_replicated(nf) ? 1u : 0u;
	a.maxabs = reinterpret_cast<const uint32_t*>(static_cast<const unsigned char*>(Wt) + (size_t)ntile * nsplit * KC * 2048);
	a.npeer = scores ? g_tc_npeer : 0u; a.row_off = g_tc_row_off;
	for (unsigned p = 0; p < a.npeer; ++p) a.peers[p] = g_tc_peers[p];
	a.timeout = g_tc_timeout ? g_tc_timeout : TC_TIMEOUT;
	a.hold_operands = g_tc_hold_operands;
	// Sequence chunks: about 8 waves of CTAs over the SMs (one CTA per SM), with the CTA
	// count a multiple of the SM count so that the last wave is full; at least 64
	// sequences per CTA.
	unsigned sms = state().sm_count;
	unsigned g = ntile, h = sms;
	while (h) { unsigned r = g % h; g = h; h = r; }              // gcd(ntile, sms)
	unsigned step = sms / g;                                     // chunk counts that fill whole waves
	unsigned want_chunks = max(1u, (8 * sms + ntile - 1) / ntile);
	want_chunks = divup(want_chunks, step) * step;
	unsigned spc = max(64u, divup(nregion, want_chunks));
	// a small batch: fewer sequences per CTA rather than idle SMs (one wave, at least 8 sequences each)
	if ((size_t)ntile * divup(nregion, spc) < sms) spc = max(8u, divup(nregion, max(1u, sms / ntile)));
	a.seqs_per_cta = spc;
	dim3 grid(ntile, divup(nregion, spc));
	size_t smem = (size_t)nsplit * KC * 2048 + 2 * (size_t)TC_ECHUNKS * 16 + 128;
	if (smem < 120 * 1024) smem = 120 * 1024;       // one CTA per SM: each CTA takes all 512 TMEM columns
	DB_REQUIRE(smem <= 220 * 1024 && 2 * KC + 16 <= 128, "ValueError: filter length %u is too long for the tensor-core kernel", m);
	DB_CUDA(cudaFuncSetAttribute(scanpool_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	scanpool_tc_kernel<<<grid, TC_THREADS, smem, state().stream>>>(a);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
