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

// ----------------------------------------------------------- minibatch fetch
// The training loop of the reference uploads every minibatch from the host
// (deepity/data.py, kangaroo/data.py:274-354).  With the dataset resident in HBM as
// `nbatch` equally sized minibatches, one launch copies minibatch order[step % nbatch]
// of up to three arrays (sequences, targets, dropout masks) into the buffers a
// captured training step reads, and advances the step counter on the device -- so a
// CUDA graph can replay "fetch, step" with no host work between steps.
// state[0] = step counter, state[1] = arrivals of the current launch.  Every CTA reads
// the counter before it arrives; the last one to arrive advances it: no CTA waits.
struct fetch_args {
	const uint8_t* src[3]; uint8_t* dst[3]; size_t bytes[3];
	uint32_t* state; const uint32_t* order; uint32_t nbatch;
};

__global__ void __launch_bounds__(256) minibatch_fetch_kernel(const fetch_args a)
{
	__shared__ unsigned s_batch;
	if (threadIdx.x == 0) {
		const unsigned step = *reinterpret_cast<volatile uint32_t*>(a.state) % a.nbatch;
		s_batch = a.order ? a.order[step] : step;
	}
	__syncthreads();
	const unsigned b = s_batch;
	const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (size_t)gridDim.x * blockDim.x;
	#pragma unroll
	for (int k = 0; k < 3; ++k) {
		const size_t n = a.bytes[k];
		if (!n) continue;
		const uint8_t* s = a.src[k] + (size_t)b * n;
		uint8_t* d = a.dst[k];
		if ((((uintptr_t)s | (uintptr_t)d | n) & 15) == 0) {
			for (size_t i = tid; i < n / 16; i += nth) reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
		} else {
			for (size_t i = tid; i < n; i += nth) d[i] = s[i];
		}
	}
	__syncthreads();
	if (threadIdx.x == 0) {
		__threadfence();
		if (atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {       // last CTA of this launch
			a.state[1] = 0;
			a.state[0] = a.state[0] + 1;
			__threadfence();
		}
	}
}

DB_EXPORT void db_minibatch_fetch(uint32_t* counters, const uint32_t* order, uint32_t nbatch,
                                  const void* src0, void* dst0, size_t bytes0,
                                  const void* src1, void* dst1, size_t bytes1,
                                  const void* src2, void* dst2, size_t bytes2)
{
	DB_API_TRY
	DB_REQUIRE(counters && nbatch, "ValueError: db_minibatch_fetch needs its two counters and at least one minibatch");
	fetch_args a;
	a.src[0] = (const uint8_t*)src0; a.dst[0] = (uint8_t*)dst0; a.bytes[0] = src0 && dst0 ? bytes0 : 0;
	a.src[1] = (const uint8_t*)src1; a.dst[1] = (uint8_t*)dst1; a.bytes[1] = src1 && dst1 ? bytes1 : 0;
	a.src[2] = (const uint8_t*)src2; a.dst[2] = (uint8_t*)dst2; a.bytes[2] = src2 && dst2 ? bytes2 : 0;
	a.state = counters; a.order = order; a.nbatch = nbatch;
	const size_t most = std::max(a.bytes[0], std::max(a.bytes[1], a.bytes[2]));
	// eight bytes a thread: an array whose minibatches are not multiples of 16 bytes is copied
	// byte by byte, and those loads should all be in flight at once
	const unsigned ncta = (unsigned)std::min<size_t>(std::max<size_t>(1, divup(most, (size_t)(256 * 8))), 2u * (unsigned)state().sm_count);
	minibatch_fetch_kernel<<<ncta, 256, 0, state().stream>>>(a);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
