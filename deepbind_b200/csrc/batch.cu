// Minibatch assembly on the device: sequence text -> ordinal buffer + region table.
//
// The reference builds every minibatch on the host with Python string joins and
// translate tables, once per dataset (code/libs/kangaroo/kangaroo/data.py:309-334,
// util.py:43-74), doubling the rows first when both strands are scored
// (data.py:274-283, util.py:58-65).  The same layout, written by one kernel from the
// raw characters:
//     X = pad | s0 | pad | s1 | ... | pad           pad = `pad` bytes of 255
//     R[r] = (start of row r's leading pad, end of row r's sequence)
// A,C,G,T/U (either case) -> 0,1,2,3; every other character -> 255.  With both
// strands, row 2b is sequence b and row 2b+1 its reverse complement.
// Because the text offsets are already a prefix sum of the lengths, each row's
// position in X has a closed form and every row is written independently: the
// kernel is one pass over the bytes, bound by HBM (1 byte read, 1-2 written).
#include "db_common.cuh"

namespace db {

__device__ __forceinline__ unsigned ordinal_of(unsigned ch)
{
	ch |= 0x20u;                                   // fold case: 'A'..'Z' -> 'a'..'z'
	return ch == 'a' ? 0u : ch == 'c' ? 1u : ch == 'g' ? 2u : (ch == 't' || ch == 'u') ? 3u : 255u;
}

// One warp per output row.
__global__ void __launch_bounds__(256)
build_batch_kernel(const uint8_t* __restrict__ text, const uint32_t* __restrict__ off, unsigned nseq, unsigned pad,
                   int rc, uint8_t* __restrict__ X, uint32_t* __restrict__ R)
{
	const unsigned lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
	const unsigned nrow = nseq * (rc ? 2u : 1u);
	const unsigned base = off[0];
	for (unsigned row = blockIdx.x * wpb + (threadIdx.x >> 5); row < nrow; row += gridDim.x * wpb) {
		const unsigned b = rc ? row >> 1 : row, second = rc ? row & 1u : 0u;
		const unsigned s0 = off[b] - base, len = off[b + 1] - off[b];
		// bytes of X before this row: one pad per earlier row, the text of all earlier rows
		const unsigned start = row * pad + (rc ? 2u * s0 + (second ? len : 0u) : s0);
		if (lane == 0) { R[2 * row] = start; R[2 * row + 1] = start + pad + len; }
		for (unsigned t = lane; t < pad; t += 32) X[start + t] = 255;
		const uint8_t* src = text + off[b];
		uint8_t* dst = X + start + pad;
		for (unsigned t = lane; t < len; t += 32) {
			unsigned o = second ? ordinal_of(src[len - 1 - t]) : ordinal_of(src[t]);
			if (second && o < 4u) o = 3u - o;      // complement of an ordinal; N stays N
			dst[t] = (uint8_t)o;
		}
		if (row == nrow - 1)                        // the trailing pad closes the buffer
			for (unsigned t = lane; t < pad; t += 32) X[start + pad + len + t] = 255;
	}
}

// Scan mode (code/libs/kangaroo/kangaroo/predict.py:270-285): every sequence is padded
// with W-1 'N' on both sides and cut into windows of W characters every `stride`
// positions; each window is then scored as a sequence of its own.  Row r of the
// output batch is window r - winoff[b] of sequence b (winoff: prefix sum of the
// window counts); all rows have the same length, so row r starts at r * (pad + W).
// With both strands, row 2w is window w and row 2w+1 its reverse complement.
// One warp per output row.
__global__ void __launch_bounds__(256)
build_windows_kernel(const uint8_t* __restrict__ text, const uint32_t* __restrict__ off, const uint32_t* __restrict__ winoff,
                     unsigned nseq, unsigned W, unsigned stride, unsigned pad, int rc,
                     uint8_t* __restrict__ X, uint32_t* __restrict__ R)
{
	const unsigned lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
	const unsigned nwin = winoff[nseq], nrow = nwin * (rc ? 2u : 1u), rowlen = pad + W;
	for (unsigned row = blockIdx.x * wpb + (threadIdx.x >> 5); row < nrow; row += gridDim.x * wpb) {
		const unsigned w = rc ? row >> 1 : row, second = rc ? row & 1u : 0u;
		unsigned lo = 0, hi = nseq;                        // the sequence b with winoff[b] <= w < winoff[b+1]
		while (hi - lo > 1) { const unsigned mid = (lo + hi) >> 1; if (winoff[mid] <= w) lo = mid; else hi = mid; }
		const unsigned b = lo, first = (w - winoff[b]) * stride;    // first character of the window in the padded sequence
		const unsigned len = off[b + 1] - off[b];
		const uint8_t* src = text + off[b];
		const unsigned start = row * rowlen;
		if (lane == 0) { R[2 * row] = start; R[2 * row + 1] = start + rowlen; }
		for (unsigned t = lane; t < pad; t += 32) X[start + t] = 255;
		uint8_t* dst = X + start + pad;
		for (unsigned t = lane; t < W; t += 32) {
			const unsigned k = first + (second ? W - 1 - t : t);    // position in  N^(W-1) | sequence | N^(W-1)
			unsigned o = (k >= W - 1 && k - (W - 1) < len) ? ordinal_of(src[k - (W - 1)]) : 255u;
			if (second && o < 4u) o = 3u - o;
			dst[t] = (uint8_t)o;
		}
		if (row == nrow - 1)
			for (unsigned t = lane; t < pad; t += 32) X[start + rowlen + t] = 255;
	}
}

}  // namespace db

using namespace db;

DB_EXPORT void db_build_windows(const uint8_t* text, const uint32_t* offsets, const uint32_t* window_offsets,
                                uint32_t nseq, uint32_t nwindow, uint32_t windowsize, uint32_t stride, uint32_t pad,
                                int reverse_complement, uint8_t* X, uint32_t* R)
{
	DB_API_TRY
	DB_REQUIRE(windowsize > 0 && stride > 0, "ValueError: window size and stride must be positive");
	if (nseq == 0 || nwindow == 0) {
		if (pad && X) DB_CUDA(cudaMemsetAsync(X, 255, pad, state().stream));
		return;
	}
	DB_REQUIRE(offsets && window_offsets && X && R, "ValueError: db_build_windows got a NULL pointer");
	unsigned rows = nwindow * (reverse_complement ? 2u : 1u);
	DB_REQUIRE((unsigned long long)rows * (pad + windowsize) + pad < 0xffffffffull, "ValueError: a minibatch is addressed with 32-bit positions; split it");
	unsigned grid = divup(rows, 8u);
	unsigned cap = (unsigned)state().sm_count * 16;
	build_windows_kernel<<<grid < cap ? grid : cap, 256, 0, state().stream>>>(text, offsets, window_offsets, nseq, windowsize, stride,
	                                                                       pad, reverse_complement, X, R);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

// Bytes of X for `nseq` sequences of `total_len` characters in all.
DB_EXPORT size_t db_batch_bytes(uint32_t nseq, size_t total_len, uint32_t pad, int reverse_complement)
{
	size_t rows = (size_t)nseq * (reverse_complement ? 2 : 1);
	return rows * pad + total_len * (reverse_complement ? 2 : 1) + pad;
}

DB_EXPORT void db_build_batch(const uint8_t* text, const uint32_t* offsets, uint32_t nseq, uint32_t pad,
                              int reverse_complement, uint8_t* X, uint32_t* R)
{
	DB_API_TRY
	if (nseq == 0) {
		if (pad && X) DB_CUDA(cudaMemsetAsync(X, 255, pad, state().stream));
		return;
	}
	DB_REQUIRE(offsets && X && R, "ValueError: db_build_batch got a NULL pointer");   // text may be NULL if every sequence is empty
	unsigned rows = nseq * (reverse_complement ? 2u : 1u);
	unsigned grid = divup(rows, 8u);
	unsigned cap = (unsigned)state().sm_count * 16;
	build_batch_kernel<<<grid < cap ? grid : cap, 256, 0, state().stream>>>(text, offsets, nseq, pad, reverse_complement, X, R);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
