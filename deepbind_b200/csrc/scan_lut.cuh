// Device functions shared by the FP32 lookup-add kernels: the lookup table of a filter
// block, the scan of one row against it, and the one-hot accumulation step of the filter
// gradient.  Arithmetic as the reference's scan (corr1ord.cuh:108-164): taps ascending from
// +0, N = ((W0+W1)+W2+W3)/4, a dropped base (254) adds 0.
#pragma once
#include "db_common.cuh"

namespace db {

// Byte offset of a base's entry within a table line: A, C, G, T -> 0, 16, 32, 48; N (and
// every other code) -> 64, the mean of the four; 254 (dropped) -> 80, a zero entry.
__device__ __forceinline__ unsigned code16_of(unsigned x)
{
	return x < 4u ? x * 16u : (x == 254u ? 80u : 64u);
}

// Builds lut[j][q][c][4] for the CTA's filter block.
__device__ __forceinline__ void build_lut(float* lut, const float* __restrict__ W, unsigned m, unsigned nf,
                                           unsigned f0, unsigned FB)
{
	const unsigned NQ = FB / 4;
	for (unsigned t = threadIdx.x; t < m * FB; t += blockDim.x) {
		unsigned j = t / FB, f = t % FB;
		float w0 = 0.f, w1 = 0.f, w2 = 0.f, w3 = 0.f;
		if (f0 + f < nf) {
			w0 = W[(size_t)(4*j+0)*nf + f0 + f]; w1 = W[(size_t)(4*j+1)*nf + f0 + f];
			w2 = W[(size_t)(4*j+2)*nf + f0 + f]; w3 = W[(size_t)(4*j+3)*nf + f0 + f];
		}
		float z = w0; z += w1; z += w2; z += w3;
		float* e = lut + ((size_t)(j * NQ + f / 4) * 8) * 4 + (f & 3);
		e[0] = w0; e[4] = w1; e[8] = w2; e[12] = w3; e[16] = z * 0.25f; e[20] = 0.f; e[24] = 0.f; e[28] = 0.f;
	}
}

// z[16] for the row whose window starts at byte `rl` of the staged codes.
template <int M>
__device__ __forceinline__ void scan_row(const unsigned char* lutp, unsigned stride, const uint8_t* xs,
                                         unsigned rl, unsigned m, float (&z)[16])
{
	#pragma unroll
	for (int v = 0; v < 16; ++v) z[v] = 0.f;
	if constexpr (M > 0) {
		constexpr int NW = (M + 3) / 4;
		const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs) + (rl >> 2);
		const unsigned sh = (rl & 3u) * 8u;
		uint32_t win[NW];
		#pragma unroll
		for (int i = 0; i < NW; ++i) win[i] = __funnelshift_r(xw[i], xw[i + 1], sh);
		#pragma unroll
		for (int j = 0; j < M; ++j) {
			unsigned c16 = (win[j >> 2] >> (8 * (j & 3))) & 0xffu;
			const float4* e = reinterpret_cast<const float4*>(lutp + (size_t)j * stride + c16);
			float4 a = e[0], b = e[8], c = e[16], d = e[24];
			z[0] += a.x; z[1] += a.y; z[2]  += a.z; z[3]  += a.w;
			z[4] += b.x; z[5] += b.y; z[6]  += b.z; z[7]  += b.w;
			z[8] += c.x; z[9] += c.y; z[10] += c.z; z[11] += c.w;
			z[12] += d.x; z[13] += d.y; z[14] += d.z; z[15] += d.w;
		}
	} else {
		for (unsigned j = 0; j < m; ++j) {
			unsigned c16 = xs[rl + j];
			const float4* e = reinterpret_cast<const float4*>(lutp + (size_t)j * stride + c16);
			float4 a = e[0], b = e[8], c = e[16], d = e[24];
			z[0] += a.x; z[1] += a.y; z[2]  += a.z; z[3]  += a.w;
			z[4] += b.x; z[5] += b.y; z[6]  += b.z; z[7]  += b.w;
			z[8] += c.x; z[9] += c.y; z[10] += c.z; z[11] += c.w;
			z[12] += d.x; z[13] += d.y; z[14] += d.z; z[15] += d.w;
		}
	}
}

// The same for eight filters (two of the four quads of a 16-filter group; `lutp` points at the
// first of them): two threads share a row where a lone warp per scheduler would otherwise
// wait out its shared-memory loads.
template <int M>
__device__ __forceinline__ void scan_row_half(const unsigned char* lutp, unsigned stride, const uint8_t* xs,
                                              unsigned rl, unsigned m, float (&z)[8])
{
	#pragma unroll
	for (int v = 0; v < 8; ++v) z[v] = 0.f;
	if constexpr (M > 0) {
		constexpr int NW = (M + 3) / 4;
		const uint32_t* xw = reinterpret_cast<const uint32_t*>(xs) + (rl >> 2);
		const unsigned sh = (rl & 3u) * 8u;
		uint32_t win[NW];
		#pragma unroll
		for (int i = 0; i < NW; ++i) win[i] = __funnelshift_r(xw[i], xw[i + 1], sh);
		#pragma unroll
		for (int j = 0; j < M; ++j) {
			unsigned c16 = (win[j >> 2] >> (8 * (j & 3))) & 0xffu;
			const float4* e = reinterpret_cast<const float4*>(lutp + (size_t)j * stride + c16);
			float4 a = e[0], b = e[8];
			z[0] += a.x; z[1] += a.y; z[2] += a.z; z[3] += a.w;
			z[4] += b.x; z[5] += b.y; z[6] += b.z; z[7] += b.w;
		}
	} else {
		for (unsigned j = 0; j < m; ++j) {
			unsigned c16 = xs[rl + j];
			const float4* e = reinterpret_cast<const float4*>(lutp + (size_t)j * stride + c16);
			float4 a = e[0], b = e[8];
			z[0] += a.x; z[1] += a.y; z[2] += a.z; z[3] += a.w;
			z[4] += b.x; z[5] += b.y; z[6] += b.z; z[7] += b.w;
		}
	}
}

__device__ __forceinline__ void bwd_fma4(float (&c)[4], float v, const float4& w)
{
	c[0] = fmaf(v, w.x, c[0]); c[1] = fmaf(v, w.y, c[1]); c[2] = fmaf(v, w.z, c[2]); c[3] = fmaf(v, w.w, c[3]);
}

}  // namespace db
