/*
 * CPU oracle for the DeepBind hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's CUDA
 * kernels for the motif-scan / pooling / update path so that the CUDA
 * implementation can be checked against it.  It is never linked into, loaded
 * by or called from the product library; only the tests, the smoke check and
 * the benchmark's CPU-baseline legs use it.
 *
 * Parity status: the reference ships no golden vectors for this path, so the
 * oracle is pinned by (a) hand-derived known-answer cases in the tests and
 * (b) the reference's own CUDA kernels and launchers -- every kernel restated in
 * this file -- compiled for the test GPU and run on the same inputs (see
 * build_ref.sh, ref_shim.cu).  Each function cites the reference source it
 * follows (paths relative to the reference tree).
 *
 * Build: gcc -O3 -march=native -fopenmp -ffp-contract=off -fno-fast-math
 * (contraction must stay off: the f32 results are bit-level expectations).
 */
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

enum { ORC_PT_MAX = 0, ORC_PT_AVG = 1, ORC_PT_SUM = 2, ORC_PT_ALL = 3 };

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
	return omp_get_max_threads();
#else
	return 1;
#endif
}

ORC_API void orc_set_num_threads(int n)
{
#ifdef _OPENMP
	if (n > 0) omp_set_num_threads(n);
#else
	(void)n;
#endif
}

/* ------------------------------------------------------------------------
 * Per-tap lookup table with six entries per (tap, filter):
 *   0..3  W[(4j+k)*nf+f]                           (corr1ord.cuh:147-148)
 *   4     ((W0+W1)+W2)+W3 times 1/4, in that order  (corr1ord.cuh:149-154)
 *   5     0, the "dropped input" code 254           (corr1ord.cuh:149)
 * Adding entry 4 equals the reference's `Z += z*0.25f` bit for bit (scaling by
 * a power of two is exact, so a fused multiply-add gives the same value).
 * ---------------------------------------------------------------------- */
#define DEFINE_LUT(NAME, REAL)                                                         \
static REAL* NAME(const REAL* W, uint32_t m, uint32_t nf)                              \
{                                                                                      \
	REAL* T = (REAL*)malloc((size_t)m * 6 * nf * sizeof(REAL));                        \
	for (uint32_t j = 0; j < m; ++j)                                                   \
		for (uint32_t f = 0; f < nf; ++f) {                                            \
			REAL w0 = W[(size_t)(4*j+0)*nf+f], w1 = W[(size_t)(4*j+1)*nf+f];           \
			REAL w2 = W[(size_t)(4*j+2)*nf+f], w3 = W[(size_t)(4*j+3)*nf+f];           \
			REAL z = w0; z += w1; z += w2; z += w3;                                    \
			T[((size_t)j*6+0)*nf+f] = w0; T[((size_t)j*6+1)*nf+f] = w1;                \
			T[((size_t)j*6+2)*nf+f] = w2; T[((size_t)j*6+3)*nf+f] = w3;                \
			T[((size_t)j*6+4)*nf+f] = z * (REAL)0.25;                                  \
			T[((size_t)j*6+5)*nf+f] = (REAL)0;                                         \
		}                                                                              \
	return T;                                                                          \
}
DEFINE_LUT(make_lut_f32, float)
DEFINE_LUT(make_lut_f64, double)

static inline uint32_t code_of(uint8_t x) { return x < 4 ? x : (x == 254 ? 5u : 4u); }

/* One row of the scan: z[f] = sum over taps j ascending of T[j][code(X[i+j])][f],
 * starting from +0 (corr1ord.cuh:117-121,144-158). */
#define DEFINE_SCAN_ROW(NAME, REAL)                                                    \
static inline void NAME(const REAL* T, uint32_t m, uint32_t nf, const uint8_t* x, REAL* z) \
{                                                                                      \
	for (uint32_t f = 0; f < nf; ++f) z[f] = (REAL)0;                                  \
	for (uint32_t j = 0; j < m; ++j) {                                                 \
		const REAL* t = T + ((size_t)j*6 + code_of(x[j]))*nf;                          \
		for (uint32_t f = 0; f < nf; ++f) z[f] += t[f];                                \
	}                                                                                  \
}
DEFINE_SCAN_ROW(scan_row_f32, float)
DEFINE_SCAN_ROW(scan_row_f64, double)

/* api_corr1ord (kangaroo_smat.cpp:98-111, corr1ord.cuh:47-166).
 * W is [4m, nf] row-major, X is npos bytes, Z is [npos, nf].  Only rows
 * i < npos-m+1 are written; the last m-1 rows keep what the caller put there. */
#define DEFINE_CORR1ORD(NAME, REAL, LUT, ROW)                                          \
ORC_API void NAME(const REAL* W, uint32_t m, uint32_t nf,                              \
                  const uint8_t* X, uint32_t npos, REAL* Z)                            \
{                                                                                      \
	if (npos < m || m == 0) return;                                                    \
	uint32_t n = npos - m + 1;                                                         \
	REAL* T = LUT(W, m, nf);                                                           \
	_Pragma("omp parallel for schedule(static)")                                       \
	for (int64_t i = 0; i < (int64_t)n; ++i)                                           \
		ROW(T, m, nf, X + i, Z + (size_t)i*nf);                                        \
	free(T);                                                                           \
}
DEFINE_CORR1ORD(orc_corr1ord_f32, float,  make_lut_f32, scan_row_f32)
DEFINE_CORR1ORD(orc_corr1ord_f64, double, make_lut_f64, scan_row_f64)

/* api_corr1ord_bprop_W (corr1ord_bprop.cuh:48-139).  dW += contributions; the
 * reference sums per-block partials with atomicAdd in no fixed order, so the
 * expectation is the exactly-rounded sum: accumulate in double, add once. */
#define DEFINE_BPROP_W(NAME, REAL)                                                     \
ORC_API void NAME(REAL* dW, uint32_t m, uint32_t nf,                                   \
                  const uint8_t* X, uint32_t npos, const REAL* dZ)                     \
{                                                                                      \
	if (npos < m || m == 0) return;                                                    \
	uint32_t n = npos - m + 1;                                                         \
	double* acc = (double*)calloc((size_t)4*m*nf, sizeof(double));                     \
	for (uint32_t i = 0; i < n; ++i)                                                   \
		for (uint32_t j = 0; j < m; ++j) {                                             \
			uint8_t k = X[i+j];                                                        \
			const REAL* dz = dZ + (size_t)i*nf;                                        \
			if (k < 4) {                                                               \
				double* a = acc + (size_t)(4*j+k)*nf;                                  \
				for (uint32_t f = 0; f < nf; ++f) a[f] += (double)dz[f];               \
			} else if (k != 254) {                                                     \
				for (uint32_t c = 0; c < 4; ++c) {                                     \
					double* a = acc + (size_t)(4*j+c)*nf;                              \
					for (uint32_t f = 0; f < nf; ++f)                                  \
						a[f] += (double)(dz[f] * (REAL)0.25);                          \
				}                                                                      \
			}                                                                          \
		}                                                                              \
	for (size_t t = 0; t < (size_t)4*m*nf; ++t) dW[t] = (REAL)((double)dW[t] + acc[t]); \
	free(acc);                                                                         \
}
DEFINE_BPROP_W(orc_corr1ord_bprop_W_f32, float)
DEFINE_BPROP_W(orc_corr1ord_bprop_W_f64, double)

/* api_corr1ord_bprop_X: the reference computes this on the host
 * (corr1ord_bprop.cu:191-201); same loop nest and accumulation order.
 * dX is [n, 4], dZ is [n, nf]. */
#define DEFINE_BPROP_X(NAME, REAL)                                                     \
ORC_API void NAME(REAL* dX, uint32_t n, const REAL* W, uint32_t m, uint32_t nf,        \
                  const REAL* dZ)                                                      \
{                                                                                      \
	_Pragma("omp parallel for schedule(static)")                                       \
	for (int64_t i = 0; i < (int64_t)n; ++i)                                           \
		for (uint32_t j = 0; j < nf; ++j)                                              \
			for (uint32_t k = 0; k < m; ++k) {                                         \
				if ((uint32_t)i < k) continue;                                         \
				for (uint32_t c = 0; c < 4; ++c)                                       \
					dX[(size_t)i*4+c] += dZ[(size_t)(i-k)*nf+j] * W[(size_t)(4*k+c)*nf+j]; \
			}                                                                          \
}
DEFINE_BPROP_X(orc_corr1ord_bprop_X_f32, float)
DEFINE_BPROP_X(orc_corr1ord_bprop_X_f64, double)

/* Pooling of one (region, map) column, shared by api_poolrgn and the fused
 * restatement.  get(row) yields the unpooled value.  Strict '>' keeps the first
 * maximal row (poolrgn.cuh:64-73); the sum runs over rows ascending
 * (poolrgn.cuh:108-110); the mean divides by the integer count
 * (size+step-1)/step (poolrgn.cuh:112,152). */
#define POOL_COLUMN(REAL, FIRST, LAST, STEP, GET, XMAX, XIDX, XSUM)                    \
	do {                                                                               \
		uint32_t r_ = (FIRST);                                                         \
		REAL v_ = GET(r_);                                                             \
		XMAX = v_; XIDX = r_; XSUM = v_;                                               \
		for (r_ = (FIRST) + (STEP); r_ < (LAST); r_ += (STEP)) {                       \
			v_ = GET(r_);                                                              \
			if (v_ > XMAX) { XMAX = v_; XIDX = r_; }                                   \
			XSUM += v_;                                                                \
		}                                                                              \
	} while (0)

/* api_poolrgn (kangaroo_smat.cpp:219-255, poolrgn.cuh:44-160).
 * unpooled [nrow, nf]; regions u32 [nregion, rcols] with rcols 2 or 3;
 * pooled [nregion, nf] (or [nregion, 2nf] interleaved max,avg for "all");
 * argmax u32 [nregion, nf] or NULL, holding the flat index row*nf+f. */
#define DEFINE_POOLRGN(NAME, REAL)                                                     \
ORC_API void NAME(const REAL* U, uint32_t nf, const uint32_t* R, uint32_t nregion,     \
                  uint32_t rcols, REAL* P, uint32_t* A, int ptype)                     \
{                                                                                      \
	_Pragma("omp parallel for schedule(static)")                                       \
	for (int64_t r = 0; r < (int64_t)nregion; ++r) {                                   \
		uint32_t first = R[r*rcols+0], last = R[r*rcols+1];                            \
		uint32_t step = rcols == 3 && R[r*rcols+2] ? R[r*rcols+2] : 1;                                 \
		uint32_t cnt = ((last-first)+step-1)/step;                                     \
		for (uint32_t f = 0; f < nf; ++f) {                                            \
			REAL xmax, xsum; uint32_t xidx;                                            \
			POOL_COLUMN(REAL, first, last, step, GETU, xmax, xidx, xsum);              \
			size_t o = (size_t)r*nf + f;                                               \
			switch (ptype) {                                                           \
			case ORC_PT_MAX: P[o] = xmax; if (A) A[o] = xidx*nf+f; break;              \
			case ORC_PT_AVG: P[o] = xsum / (REAL)cnt; break;                           \
			case ORC_PT_SUM: P[o] = xsum; break;                                       \
			default:         P[2*o] = xmax; P[2*o+1] = xsum / (REAL)cnt;               \
			                 if (A) A[o] = xidx*nf+f; break;                           \
			}                                                                          \
		}                                                                              \
	}                                                                                  \
}
#define GETU(row) U[(size_t)(row)*nf+f]
DEFINE_POOLRGN(orc_poolrgn_f32, float)
DEFINE_POOLRGN(orc_poolrgn_f64, double)
#undef GETU

/* api_poolrgn_bprop (poolrgn_bprop.cuh:45-127).  Accumulates into U (the
 * caller zeroes it).  For "all" the thread of (region,f) first adds the mean
 * share to every row of the region, then adds the max delta at argmax
 * (poolrgn_bprop.cuh:122-126), so with disjoint regions the order is fixed. */
#define DEFINE_POOLRGN_BPROP(NAME, REAL)                                               \
ORC_API void NAME(REAL* U, uint32_t nf, const uint32_t* R, uint32_t nregion,           \
                  uint32_t rcols, const REAL* P, const uint32_t* A, int ptype)         \
{                                                                                      \
	for (uint32_t r = 0; r < nregion; ++r) {                                           \
		uint32_t first = R[r*rcols+0], last = R[r*rcols+1];                            \
		uint32_t step = rcols == 3 && R[r*rcols+2] ? R[r*rcols+2] : 1;                                 \
		uint32_t cnt = ((last-first)+step-1)/step;                                     \
		for (uint32_t f = 0; f < nf; ++f) {                                            \
			size_t o = (size_t)r*nf + f;                                               \
			if (ptype == ORC_PT_MAX) { U[A[o]] += P[o]; continue; }                    \
			REAL d = ptype == ORC_PT_ALL ? P[2*o+1] : P[o];                            \
			if (ptype != ORC_PT_SUM) d /= (REAL)cnt;                                   \
			for (uint32_t row = first; row < last; row += step)                        \
				U[(size_t)row*nf+f] += d;                                              \
			if (ptype == ORC_PT_ALL) U[A[o]] += P[2*o];                                \
		}                                                                              \
	}                                                                                  \
}
DEFINE_POOLRGN_BPROP(orc_poolrgn_bprop_f32, float)
DEFINE_POOLRGN_BPROP(orc_poolrgn_bprop_f64, double)

/* Fused restatement of the scoring chain
 *   corr1ord (zeroed Z) -> bias -> rectify -> poolrgn
 * (kangaroo/_ext/corr1ord.py:97-102, deepity/std/elemwise.py:171,74-78,
 * kangaroo/_ext/poolrgn.py:59,153) without materialising Z.  Rows at or past
 * npos-m+1 read as the zeros corr1ord.py:101 leaves there.  bias may be NULL;
 * relu==0 skips the rectifier.  Step-3 regions are honoured.  This is the
 * function the CPU baseline times. */
#define DEFINE_SCANPOOL(NAME, REAL, LUT, ROW)                                          \
ORC_API void NAME(const REAL* W, uint32_t m, uint32_t nf, const REAL* bias, int relu,  \
                  const uint8_t* X, uint32_t npos, const uint32_t* R, uint32_t nregion,\
                  uint32_t rcols, REAL* P, uint32_t* A, int ptype)                     \
{                                                                                      \
	uint32_t n = npos >= m ? npos - m + 1 : 0;                                         \
	REAL* T = LUT(W, m, nf);                                                           \
	_Pragma("omp parallel")                                                            \
	{                                                                                  \
		REAL* z    = (REAL*)malloc(sizeof(REAL)*nf);                                   \
		REAL* xmax = (REAL*)malloc(sizeof(REAL)*nf);                                   \
		REAL* xsum = (REAL*)malloc(sizeof(REAL)*nf);                                   \
		uint32_t* xidx = (uint32_t*)malloc(sizeof(uint32_t)*nf);                       \
		_Pragma("omp for schedule(dynamic,16)")                                        \
		for (int64_t r = 0; r < (int64_t)nregion; ++r) {                               \
			uint32_t first = R[r*rcols+0], last = R[r*rcols+1];                        \
			uint32_t step = rcols == 3 && R[r*rcols+2] ? R[r*rcols+2] : 1;                             \
			uint32_t cnt = ((last-first)+step-1)/step;                                 \
			for (uint32_t row = first; row == first || row < last; row += step) {      \
				if (row < n) ROW(T, m, nf, X + row, z);                                \
				else for (uint32_t f = 0; f < nf; ++f) z[f] = (REAL)0;                 \
				for (uint32_t f = 0; f < nf; ++f) {                                    \
					REAL v = z[f];                                                     \
					if (bias) v = v + bias[f];                                         \
					if (relu) v = v > (REAL)0 ? v : (REAL)0;                           \
					if (row == first) { xmax[f] = v; xidx[f] = row; xsum[f] = v; }     \
					else { if (v > xmax[f]) { xmax[f] = v; xidx[f] = row; }            \
					       xsum[f] += v; }                                             \
				}                                                                      \
			}                                                                          \
			for (uint32_t f = 0; f < nf; ++f) {                                        \
				size_t o = (size_t)r*nf + f;                                           \
				switch (ptype) {                                                       \
				case ORC_PT_MAX: P[o] = xmax[f]; if (A) A[o] = xidx[f]*nf+f; break;    \
				case ORC_PT_AVG: P[o] = xsum[f] / (REAL)cnt; break;                    \
				case ORC_PT_SUM: P[o] = xsum[f]; break;                                \
				default:         P[2*o] = xmax[f]; P[2*o+1] = xsum[f] / (REAL)cnt;     \
				                 if (A) A[o] = xidx[f]*nf+f; break;                    \
				}                                                                      \
			}                                                                          \
		}                                                                              \
		free(z); free(xmax); free(xsum); free(xidx);                                   \
	}                                                                                  \
	free(T);                                                                           \
}
DEFINE_SCANPOOL(orc_scanpool_f32, float,  make_lut_f32, scan_row_f32)
DEFINE_SCANPOOL(orc_scanpool_f64, double, make_lut_f64, scan_row_f64)

/* kernel_dropoutord_fp_tr (dropoutord.cu:41-52) with the uniform draws U
 * supplied by the caller (cuRAND streams are not reproducible elsewhere). */
ORC_API void orc_dropoutord_fp_tr(const uint8_t* X, const float* U, float rate,
                                  uint8_t* Z, uint8_t* M, uint32_t n)
{
	for (uint32_t i = 0; i < n; ++i) {
		int mask = (X[i] == 255) || (U[i] >= rate);
		M[i] = (uint8_t)mask;
		Z[i] = mask ? X[i] : 254;
	}
}

/* gradstep.cu:41-72 */
#define DEFINE_GRADSTEP(SUF, REAL)                                                     \
ORC_API void orc_gradstep_##SUF(REAL* P, const REAL* dP, const REAL* drate,            \
                                REAL* mP, const REAL* mrate, uint32_t n)               \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) {                                                 \
		REAL delta = mP[i]*mrate[i] - dP[i]*drate[i];                                  \
		mP[i] = delta; P[i] += delta;                                                  \
	}                                                                                  \
}                                                                                      \
ORC_API void orc_gradstep_nesterov1_##SUF(REAL* P, const REAL* mP, const REAL* mrate,  \
                                          uint32_t n)                                  \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) P[i] = P[i] + mrate[i]*mP[i];                     \
}                                                                                      \
ORC_API void orc_gradstep_nesterov2_##SUF(REAL* P, const REAL* dP, const REAL* drate,  \
                                          REAL* mP, const REAL* mrate, uint32_t n)     \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) {                                                 \
		REAL delta = dP[i]*drate[i];                                                   \
		mP[i] = mP[i]*mrate[i] - delta;                                                \
		P[i] -= delta;                                                                 \
	}                                                                                  \
}                                                                                      \
/* madd_bcast.cu:41-47 */                                                              \
ORC_API void orc_madd_bcast_##SUF(const REAL* A, const REAL* b, REAL* dst,             \
                                  uint32_t n, uint32_t m, uint32_t k)                  \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) dst[i] += A[i]*b[(i/k) % m];                      \
}                                                                                      \
/* maskout.cu:41-50 */                                                                 \
ORC_API void orc_maskout_##SUF(const uint8_t* M, REAL* A, uint32_t n)                  \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) if (!M[i]) A[i] = (REAL)0;                        \
}                                                                                      \
/* maskout.cu:52-67: Z is [n, m]; only 'true' is ever written */                       \
ORC_API void orc_calc_zmask_##SUF(const REAL* Z, uint8_t* M, uint32_t n, uint32_t m)   \
{                                                                                      \
	for (uint32_t i = 0; i < (n*m)/2; ++i) {                                           \
		uint32_t row = (i/m)*2, col = i%m, index = m*row+col;                          \
		if (Z[index] >= Z[index+m]) M[index] = 1; else M[index+m] = 1;                 \
	}                                                                                  \
}                                                                                      \
/* deepity_smat/dropout.cu:41-109, uniform draws supplied */                           \
ORC_API void orc_dropout_fp_tr_##SUF(const REAL* X, const REAL* rate, const float* U,  \
                                     REAL* Z, uint8_t* M, uint32_t n, uint32_t m,      \
                                     uint32_t k)                                       \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) {                                                 \
		REAL p = rate[(i/k) % m];                                                      \
		int mask = ((REAL)U[i] >= p);                                                  \
		M[i] = (uint8_t)mask; Z[i] = X[i]*(REAL)mask;                                  \
	}                                                                                  \
}                                                                                      \
ORC_API void orc_dropout_fp_tr_match_##SUF(const REAL* X, const REAL* rate,            \
                                           const float* U, REAL* Z, uint8_t* M,        \
                                           uint32_t nrow, uint32_t ncol, uint32_t k)   \
{                                                                                      \
	for (uint32_t i = 0; i < nrow*ncol/2; ++i) {                                       \
		uint32_t row = (i/ncol)*2, col = i%ncol;                                       \
		REAL p = rate[col/k];                                                          \
		int mask = ((REAL)U[i] >= p);                                                  \
		uint32_t i0 = row*ncol+col, i1 = i0+ncol;                                      \
		M[i0] = (uint8_t)mask; M[i1] = (uint8_t)mask;                                  \
		Z[i0] = X[i0]*(REAL)mask; Z[i1] = X[i1]*(REAL)mask;                            \
	}                                                                                  \
}                                                                                      \
ORC_API void orc_dropout_fp_te_##SUF(const REAL* X, const REAL* rate, REAL* Z,         \
                                     uint32_t n, uint32_t m, uint32_t k)               \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) { REAL s = 1-rate[(i/k) % m]; Z[i] = X[i]*s; }    \
}                                                                                      \
ORC_API void orc_dropout_bp_tr_##SUF(const REAL* dZ, const uint8_t* M, REAL* dX,       \
                                     uint32_t n)                                       \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) dX[i] = dZ[i]*(REAL)(M[i] != 0);                  \
}                                                                                      \
ORC_API void orc_dropout_bp_te_##SUF(const REAL* dZ, const REAL* rate, REAL* dX,       \
                                     uint32_t n, uint32_t m, uint32_t k)               \
{                                                                                      \
	for (uint32_t i = 0; i < n; ++i) { REAL s = 1-rate[(i/k) % m]; dX[i] = dZ[i]*s; }  \
}
DEFINE_GRADSTEP(f32, float)
DEFINE_GRADSTEP(f64, double)

/* Block-diagonal products (blockwise_dot.cu:75-260).  Row-major; the sums are
 * accumulated in double because cuBLAS's order is unspecified.
 *   mode 0  Z[:,b]  (n x m)  = beta*Z + X[:,b] (n x k) . W[b] (k x m)
 *   mode 1  dX[:,b] (n x k)  = dZ[:,b] (n x m) . W[b]^T
 *   mode 2  dW[b]   (k x m)  = X[:,b]^T . dZ[:,b]
 * W has p rows per block and the k rows used start at row xoff of the block;
 * xbroadcast means X has only k columns shared by every block. */
#define DEFINE_BWDOT(SUF, REAL)                                                        \
ORC_API void orc_blockwise_##SUF(int mode, int nblock, int xoff, int xbroadcast,       \
                                 int n, int m, int k, int p,                           \
                                 REAL* X, REAL* W, REAL* Z, int beta_one)              \
{                                                                                      \
	int ldx = k*(xbroadcast ? 1 : nblock), ldw = m, ldz = m*nblock;                    \
	for (int b = 0; b < nblock; ++b) {                                                 \
		REAL* Xb = X + (xbroadcast ? 0 : b*k);                                         \
		REAL* Wb = W + ((size_t)b*p + xoff)*m;                                         \
		REAL* Zb = Z + b*m;                                                            \
		if (mode == 0) {                                                               \
			for (int i = 0; i < n; ++i) for (int c = 0; c < m; ++c) {                  \
				double s = beta_one ? (double)Zb[(size_t)i*ldz+c] : 0.0;               \
				for (int t = 0; t < k; ++t)                                            \
					s += (double)Xb[(size_t)i*ldx+t]*(double)Wb[(size_t)t*ldw+c];      \
				Zb[(size_t)i*ldz+c] = (REAL)s;                                         \
			}                                                                          \
		} else if (mode == 1) {                                                        \
			for (int i = 0; i < n; ++i) for (int t = 0; t < k; ++t) {                  \
				double s = 0.0;                                                        \
				for (int c = 0; c < m; ++c)                                            \
					s += (double)Zb[(size_t)i*ldz+c]*(double)Wb[(size_t)t*ldw+c];      \
				Xb[(size_t)i*ldx+t] = (REAL)s;                                         \
			}                                                                          \
		} else {                                                                       \
			for (int t = 0; t < k; ++t) for (int c = 0; c < m; ++c) {                  \
				double s = 0.0;                                                        \
				for (int i = 0; i < n; ++i)                                            \
					s += (double)Xb[(size_t)i*ldx+t]*(double)Zb[(size_t)i*ldz+c];      \
				Wb[(size_t)t*ldw+c] = (REAL)s;                                         \
			}                                                                          \
		}                                                                              \
	}                                                                                  \
}
DEFINE_BWDOT(f32, float)
DEFINE_BWDOT(f64, double)
