// Counter-based random draws for the dropout masks: Philox-4x32 with ten
// rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11),
// written out from the published round function.  The reference keeps a
// cuRAND XORWOW state per thread (smat_cuda/cuda_context.cpp:210-242); streams
// of different generators cannot agree, so parity on masks is defined with the
// draws supplied by the caller (the *_u entry points).  A counter-based
// generator needs no state array and gives the same mask for the same
// (seed, call number, element index) whatever the launch shape.
#pragma once
#include <stdint.h>

namespace db {

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k)
{
	const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
	#pragma unroll
	for (int r = 0; r < 10; ++r) {
		uint32_t hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
		uint32_t hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
		c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
		k.x += W0; k.y += W1;
	}
	return c;
}

// Uniform draw in (0,1], the range curand_uniform documents.
__device__ __forceinline__ float uniform_01(uint64_t seed, uint64_t call, uint64_t index)
{
	uint4 c = make_uint4((uint32_t)index, (uint32_t)(index >> 32), (uint32_t)call, (uint32_t)(call >> 32));
	uint2 k = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
	uint32_t x = philox4x32_10(c, k).x;
	return (float)x * 2.3283064365386963e-10f + 1.1641532182693481e-10f;
}

}  // namespace db
