// The dense head of a DeepBind training step in one kernel.
//
// After pooling, the reference runs per minibatch step, each as its own launch
// with a round trip through HBM: dropout (deepity/std/elemwise.py:128-150),
// full -> bias -> rectify -> full -> bias (full.py:78-89, elemwise.py:171,74-78),
// logistic (softmax.py:50-61), the loss and its gradient (loss.py:52-112), and the
// three block-diagonal products of the backward pass (blockwise_dot_nt/_tn) plus
// the bias sums -- about seventeen launches for a few hundred kilobytes of data.
// Here one CTA per model keeps the minibatch of that model in shared memory and
// does all of it: forward, loss, backward, writing the parameter gradients and
// the gradient of the pooled features.  Every sum runs in a fixed order (rows
// ascending), so repeated runs agree bit for bit.
//
// With few models one CTA per model leaves the GPU to a handful of SMs, each grinding
// through its whole minibatch.  Then a thread-block cluster shares a model: every CTA
// of the cluster takes a slice of the rows, and the sums over rows (parameter
// gradients, loss) are finished through distributed shared memory, CTA rank
// ascending -- still a fixed order.
//
// Layouts follow the reference (full.py:57, loss.py:57-65): pooled [B, npool*I],
// W1 [(npool*I), H] stacked on rows per model, b1 [H*I], W2 [(H*I), 1], b2 [I],
// Y [B, I]; H = 0 means a linear head W1 [(npool*I), 1], b1 [I].
#include "db_common.cuh"
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace db {

struct head_args {
	const float* pooled; const uint8_t* mask; const float* Y;
	const float* W1; const float* b1; const float* W2; const float* b2;
	float* loss; float* dpooled; float* dW1; float* db1; float* dW2; float* db2;
	unsigned B, I, npool, H;
	int kind, pairs;
};

// Sum over the rows i = k, k+8, ... of a column, k = lane % 8, then over the eight
// partial sums with a fixed shuffle tree: eight lanes share one output.
__device__ __forceinline__ float sum8(float s)
{
	s += __shfl_xor_sync(0xffffffffu, s, 4);
	s += __shfl_xor_sync(0xffffffffu, s, 2);
	s += __shfl_xor_sync(0xffffffffu, s, 1);
	return s;
}

__global__ void __launch_bounds__(1024)
head_train_kernel(const head_args a)
{
	extern __shared__ __align__(16) float hs[];
	const unsigned B = a.B, np = a.npool, H = a.H, HC = H ? H : 1u, WS = HC + 1;   // WS: padded row stride of W1
	const unsigned b = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
	float* pd  = hs;                       // [B][np]   pooled features after dropout
	float* h1  = pd + (size_t)B * np;      // [B][HC]   hidden pre-activation, then its gradient
	float* a1  = h1 + (size_t)B * HC;      // [B][HC]   rectified hidden activation
	float* w1  = a1 + (size_t)B * HC;      // [np][WS]
	float* w2  = w1 + (size_t)np * WS;     // [HC]
	float* out = w2 + HC;                  // [B]       output, then dout
	float* zb  = out + B;                  // [B]       output after the logistic (nll) or as is (mse)
	float* red = zb + B;                   // [blockDim.x]

	const size_t ldp = (size_t)np * a.I;
	for (unsigned t = tid; t < B * np; t += nt) {
		const unsigned i = t / np, u = t % np;
		const size_t o = (size_t)i * ldp + (size_t)b * np + u;
		float v = a.pooled[o];
		if (a.mask && !a.mask[o]) v = 0.f;                 // maskout semantics: a dropped feature is exactly 0
		pd[t] = v;
	}
	for (unsigned t = tid; t < np * HC; t += nt) w1[(t / HC) * WS + t % HC] = a.W1[(size_t)b * np * HC + t];
	if (H) for (unsigned t = tid; t < H; t += nt) w2[t] = a.W2[(size_t)b * H + t];
	__syncthreads();

	// hidden (or output) layer: h1 = pd . W1 + b1
	for (unsigned t = tid; t < B * HC; t += nt) {
		const unsigned i = t / HC, c = t % HC;
		float s = 0.f;
		for (unsigned u = 0; u < np; ++u) s = fmaf(pd[i * np + u], w1[u * WS + c], s);
		s = s + a.b1[(size_t)b * HC + c];
		h1[t] = s;
		a1[t] = s > 0.f ? s : 0.f;
	}
	__syncthreads();
	for (unsigned i = tid; i < B; i += nt) {
		float o;
		if (H) {
			float s = 0.f;
			for (unsigned c = 0; c < H; ++c) s = fmaf(a1[i * H + c], w2[c], s);
			o = s + a.b2[b];
		} else o = h1[i];
		out[i] = o;
	}
	__syncthreads();

	// loss and dout = (Z - Y) / B   (loss.py:98-112; the logistic's own derivative is not applied, softmax.py:76-77).
	// With strand pairs (rows 2k, 2k+1 = forward, reverse complement) only the row with the larger
	// output Z of each pair, the forward one on ties, contributes to loss and gradient
	// (loss.py:52-65,113-117, maskout.cu:54-67); B still counts every row.
	const float inv = 1.f / (float)B;
	for (unsigned i = tid; i < B; i += nt) {
		const float o = out[i];
		zb[i] = a.kind == 1 ? 1.f / (1.f + expf(-o)) : o;
	}
	__syncthreads();
	float ls = 0.f;
	for (unsigned i = tid; i < B; i += nt) {
		const float y = a.Y[(size_t)i * a.I + b];
		const float z = zb[i];
		bool keep = true;
		if (a.pairs && (i | 1u) < B) keep = (i & 1u) ? !(zb[i - 1] >= z) : (z >= zb[i + 1]);
		float l;
		if (a.kind == 1) l = logf(fmaxf(1e-15f, z)) * y + logf(fmaxf(1e-15f, 1.f - z)) * (1.f - y);
		else { const float d = z - y; l = d * d; }
		ls += keep ? l : 0.f;
		out[i] = keep ? (z - y) * inv : 0.f;
	}
	red[tid] = ls;
	__syncthreads();
	for (unsigned w = nt / 2; w > 0; w >>= 1) {
		if (tid < w) red[tid] += red[tid + w];
		__syncthreads();
	}
	if (tid == 0 && a.loss) a.loss[b] = (a.kind == 0 ? 0.5f : -1.f) * (red[0] * inv);

	// second layer backward; h1 becomes the gradient of the hidden pre-activation.
	// Column sums over the minibatch: eight lanes per output (nt is a multiple of 32).
	const unsigned k8 = tid & 7;
	if (H) {
		for (unsigned c = tid >> 3; c < ((H + 3u) & ~3u); c += nt >> 3) {     // whole warps stay in the loop for the shuffles
			float s = 0.f;
			if (c < H) for (unsigned i = k8; i < B; i += 8) s = fmaf(a1[i * H + c], out[i], s);
			s = sum8(s);
			if (c < H && k8 == 0) a.dW2[(size_t)b * H + c] = s;
		}
		if (tid >= nt - 32) {                                 // the last warp: bias gradient of the output unit
			float s = 0.f;
			for (unsigned i = tid & 31; i < B; i += 32) s += out[i];
			s += __shfl_xor_sync(0xffffffffu, s, 16);
			s = sum8(s + __shfl_xor_sync(0xffffffffu, s, 8));
			if ((tid & 31) == 0) a.db2[b] = s;
		}
		for (unsigned t = tid; t < B * H; t += nt) {
			const unsigned i = t / H, c = t % H;
			h1[t] = a1[t] > 0.f ? out[i] * w2[c] : 0.f;
		}
	} else {
		for (unsigned i = tid; i < B; i += nt) h1[i] = out[i];
	}
	__syncthreads();

	// first layer backward
	for (unsigned c = tid >> 3; c < ((HC + 3u) & ~3u); c += nt >> 3) {
		float s = 0.f;
		if (c < HC) for (unsigned i = k8; i < B; i += 8) s += h1[i * HC + c];
		s = sum8(s);
		if (c < HC && k8 == 0) a.db1[(size_t)b * HC + c] = s;
	}
	for (unsigned t = tid; t < np * HC; t += nt) {
		const unsigned u = t / HC, c = t % HC;
		float s = 0.f;
		for (unsigned i = 0; i < B; ++i) s = fmaf(pd[i * np + u], h1[i * HC + c], s);
		a.dW1[(size_t)b * np * HC + t] = s;
	}
	for (unsigned t = tid; t < B * np; t += nt) {
		const unsigned i = t / np, u = t % np;
		const size_t o = (size_t)i * ldp + (size_t)b * np + u;
		float s = 0.f;
		for (unsigned c = 0; c < HC; ++c) s = fmaf(h1[i * HC + c], w1[u * WS + c], s);
		if (a.mask && !a.mask[o]) s = 0.f;
		a.dpooled[o] = s;
	}
}

// ---- a cluster of CTAs per model: CTA `rank` owns rows [rank*Bc, rank*Bc + Bc) (Bc even,
// so strand pairs stay together) and the cluster adds the per-CTA sums over rows.
__global__ void __launch_bounds__(512)
head_train_cluster_kernel(const head_args a, const unsigned Bc)
{
	extern __shared__ __align__(16) float hs[];
	cg::cluster_group cluster = cg::this_cluster();
	const unsigned C = cluster.num_blocks(), rank = cluster.block_rank();
	const unsigned B = a.B, np = a.npool, H = a.H, HC = H ? H : 1u, WS = HC + 1;
	const unsigned b = blockIdx.x / C, tid = threadIdx.x, nt = blockDim.x;
	const unsigned r0 = min(B, rank * Bc), nb = min(B, r0 + Bc) - r0;       // this CTA's rows
	// sums over rows, per CTA: dW1 [np][HC] | db1 [HC] | dW2 [H] | db2 (if H) | loss
	const unsigned o_db1 = np * HC, o_dw2 = o_db1 + HC, o_db2 = o_dw2 + H, o_loss = o_db2 + (H ? 1u : 0u), NP = o_loss + 1;
	float* pd   = hs;                       // [Bc][np]
	float* h1   = pd + (size_t)Bc * np;     // [Bc][HC]
	float* a1   = h1 + (size_t)Bc * HC;     // [Bc][HC]
	float* w1   = a1 + (size_t)Bc * HC;     // [np][WS]
	float* w2   = w1 + (size_t)np * WS;     // [HC]
	float* out  = w2 + HC;                  // [Bc]
	float* zb   = out + Bc;                 // [Bc]
	float* red  = zb + Bc;                  // [Bc]
	float* part = red + Bc;                 // [NP]

	const size_t ldp = (size_t)np * a.I;
	for (unsigned t = tid; t < nb * np; t += nt) {
		const unsigned i = t / np, u = t % np;
		const size_t o = (size_t)(r0 + i) * ldp + (size_t)b * np + u;
		float v = a.pooled[o];
		if (a.mask && !a.mask[o]) v = 0.f;
		pd[t] = v;
	}
	for (unsigned t = tid; t < np * HC; t += nt) w1[(t / HC) * WS + t % HC] = a.W1[(size_t)b * np * HC + t];
	if (H) for (unsigned t = tid; t < H; t += nt) w2[t] = a.W2[(size_t)b * H + t];
	__syncthreads();

	for (unsigned t = tid; t < nb * HC; t += nt) {
		const unsigned i = t / HC, c = t % HC;
		float s = 0.f;
		for (unsigned u = 0; u < np; ++u) s = fmaf(pd[i * np + u], w1[u * WS + c], s);
		s = s + a.b1[(size_t)b * HC + c];
		h1[t] = s;
		a1[t] = s > 0.f ? s : 0.f;
	}
	__syncthreads();
	for (unsigned i = tid; i < nb; i += nt) {
		float o;
		if (H) {
			float s = 0.f;
			for (unsigned c = 0; c < H; ++c) s = fmaf(a1[i * H + c], w2[c], s);
			o = s + a.b2[b];
		} else o = h1[i];
		zb[i] = a.kind == 1 ? 1.f / (1.f + expf(-o)) : o;
	}
	__syncthreads();
	const float inv = 1.f / (float)B;
	for (unsigned i = tid; i < nb; i += nt) {
		const unsigned gi = r0 + i;
		const float y = a.Y[(size_t)gi * a.I + b];
		const float z = zb[i];
		bool keep = true;
		if (a.pairs && (gi | 1u) < B) keep = (gi & 1u) ? !(zb[i - 1] >= z) : (z >= zb[i + 1]);
		float l;
		if (a.kind == 1) l = logf(fmaxf(1e-15f, z)) * y + logf(fmaxf(1e-15f, 1.f - z)) * (1.f - y);
		else { const float d = z - y; l = d * d; }
		red[i] = keep ? l : 0.f;
		out[i] = keep ? (z - y) * inv : 0.f;
	}
	__syncthreads();
	if (tid < 32) {                                           // loss of this CTA's rows: lane-strided, then a fixed tree
		float s = 0.f;
		for (unsigned i = tid; i < nb; i += 32) s += red[i];
		s += __shfl_xor_sync(0xffffffffu, s, 16);
		s = sum8(s + __shfl_xor_sync(0xffffffffu, s, 8));
		if (tid == 0) part[o_loss] = s;
	}

	const unsigned k8 = tid & 7;
	if (H) {
		for (unsigned c = tid >> 3; c < ((H + 3u) & ~3u); c += nt >> 3) {
			float s = 0.f;
			if (c < H) for (unsigned i = k8; i < nb; i += 8) s = fmaf(a1[i * H + c], out[i], s);
			s = sum8(s);
			if (c < H && k8 == 0) part[o_dw2 + c] = s;
		}
		if (tid >= nt - 32) {
			float s = 0.f;
			for (unsigned i = tid & 31; i < nb; i += 32) s += out[i];
			s += __shfl_xor_sync(0xffffffffu, s, 16);
			s = sum8(s + __shfl_xor_sync(0xffffffffu, s, 8));
			if ((tid & 31) == 0) part[o_db2] = s;
		}
		for (unsigned t = tid; t < nb * H; t += nt) {
			const unsigned i = t / H, c = t % H;
			h1[t] = a1[t] > 0.f ? out[i] * w2[c] : 0.f;
		}
	} else {
		for (unsigned i = tid; i < nb; i += nt) h1[i] = out[i];
	}
	__syncthreads();

	for (unsigned c = tid >> 3; c < ((HC + 3u) & ~3u); c += nt >> 3) {
		float s = 0.f;
		if (c < HC) for (unsigned i = k8; i < nb; i += 8) s += h1[i * HC + c];
		s = sum8(s);
		if (c < HC && k8 == 0) part[o_db1 + c] = s;
	}
	for (unsigned t = tid; t < np * HC; t += nt) {
		const unsigned u = t / HC, c = t % HC;
		float s = 0.f;
		for (unsigned i = 0; i < nb; ++i) s = fmaf(pd[i * np + u], h1[i * HC + c], s);
		part[t] = s;
	}
	for (unsigned t = tid; t < nb * np; t += nt) {
		const unsigned i = t / np, u = t % np;
		const size_t o = (size_t)(r0 + i) * ldp + (size_t)b * np + u;
		float s = 0.f;
		for (unsigned c = 0; c < HC; ++c) s = fmaf(h1[i * HC + c], w1[u * WS + c], s);
		if (a.mask && !a.mask[o]) s = 0.f;
		a.dpooled[o] = s;
	}

	// The cluster's sums: CTA `rank` finishes a slice of the NP outputs, reading every CTA's
	// partials through distributed shared memory, rank ascending.
	cluster.sync();
	const unsigned S = (NP + C - 1) / C;
	for (unsigned j = rank * S + tid; j < min(NP, (rank + 1) * S); j += nt) {
		float s = 0.f;
		for (unsigned q = 0; q < C; ++q) s += cluster.map_shared_rank(part, q)[j];
		if (j < o_db1) a.dW1[(size_t)b * np * HC + j] = s;
		else if (j < o_dw2) a.db1[(size_t)b * HC + (j - o_db1)] = s;
		else if (j < o_db2) a.dW2[(size_t)b * H + (j - o_dw2)] = s;
		else if (j < o_loss) a.db2[b] = s;
		else if (a.loss) a.loss[b] = (a.kind == 0 ? 0.5f : -1.f) * (s * inv);
	}
	cluster.sync();                                           // nobody leaves while its partials are being read
}

static size_t head_cluster_smem_bytes(unsigned Bc, unsigned np, unsigned H)
{
	unsigned HC = H ? H : 1u;
	return ((size_t)Bc * np + 2 * (size_t)Bc * HC + (size_t)np * (HC + 1) + HC + 3 * (size_t)Bc +
	        (size_t)np * HC + HC + H + 2) * sizeof(float);
}

static size_t head_smem_bytes(unsigned B, unsigned np, unsigned H)
{
	unsigned HC = H ? H : 1u;
	return ((size_t)B * np + 2 * (size_t)B * HC + (size_t)np * (HC + 1) + HC + 2 * (size_t)B + 1024) * sizeof(float);
}

}  // namespace db

using namespace db;

// Largest minibatch the fused head takes for the given widths (0: never fits).
DB_EXPORT uint32_t db_head_max_batch(uint32_t npool, uint32_t hidden)
{
	unsigned B = 0;
	while (head_smem_bytes(B + 64, npool, hidden) <= 200 * 1024 && B < 65536) B += 64;
	return B;
}

DB_EXPORT void db_head_train(uint32_t nmodel, uint32_t npool, uint32_t hidden, int loss_kind, int strand_pairs, uint32_t B,
                             const float* pooled, const uint8_t* dropmask, const float* Y,
                             const float* W1, const float* b1, const float* W2, const float* b2,
                             float* loss, float* dpooled, float* dW1, float* db1, float* dW2, float* db2)
{
	DB_API_TRY
	DB_REQUIRE(loss_kind == 0 || loss_kind == 1, "ValueError: loss kind must be 0 (mse) or 1 (nll)");
	DB_REQUIRE(npool > 0, "ValueError: the head needs at least one pooled feature per model");
	if (!nmodel || !B) return;
	DB_REQUIRE(pooled && Y && W1 && b1 && dpooled && dW1 && db1, "ValueError: db_head_train got a NULL pointer");
	DB_REQUIRE(!hidden || (W2 && b2 && dW2 && db2), "ValueError: a hidden layer needs W2, b2, dW2 and db2");
	size_t smem = head_smem_bytes(B, npool, hidden);
	DB_REQUIRE(smem <= 200 * 1024, "ValueError: minibatch of %u rows x %u features x %u hidden units exceeds the fused head's "
	           "shared-memory tile (at most %u rows)", B, npool, hidden, db_head_max_batch(npool, hidden));
	head_args a;
	a.pooled = pooled; a.mask = dropmask; a.Y = Y; a.W1 = W1; a.b1 = b1; a.W2 = W2; a.b2 = b2;
	a.loss = loss; a.dpooled = dpooled; a.dW1 = dW1; a.db1 = db1; a.dW2 = dW2; a.db2 = db2;
	a.B = B; a.I = nmodel; a.npool = npool; a.H = hidden; a.kind = loss_kind; a.pairs = strand_pairs;
	// Few models: a cluster of CTAs per model, each with a slice of the rows.  Sixteen CTAs (a
	// cluster size the device has to grant) when the minibatch is long enough and the device
	// can place such a cluster; else the portable eight or four.
	unsigned C = nmodel <= 16 ? 8u : (nmodel <= 32 ? 4u : 1u);
	auto cluster_cfg = [&](unsigned c, cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, unsigned& Bc) {
		Bc = (divup(B, c) + 1u) & ~1u;
		cfg = cudaLaunchConfig_t{};
		cfg.gridDim = dim3(nmodel * c); cfg.blockDim = dim3(512);      // 512 threads measured best (128: +4 us, 256: +2, 1024: +2)
		cfg.dynamicSmemBytes = head_cluster_smem_bytes(Bc, npool, hidden); cfg.stream = state().stream;
		attr[0].id = cudaLaunchAttributeClusterDimension;
		attr[0].val.clusterDim.x = c; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
		cfg.attrs = attr; cfg.numAttrs = 1;
	};
	if (C > 1 && B >= 4 * C) {
		cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[1]; unsigned Bc = 0;
		static int wide = -1;                                 // can a cluster of 16 be placed? asked once
		if (nmodel <= 8 && B >= 128 && wide != 0) {
			cluster_cfg(16, cfg, attr, Bc);
			if (wide < 0) {
				int n = 0;
				wide = cudaFuncSetAttribute(head_train_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess &&
				       cudaFuncSetAttribute(head_train_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(cfg.dynamicSmemBytes, (size_t)48 * 1024)) == cudaSuccess &&
				       cudaOccupancyMaxActiveClusters(&n, head_train_cluster_kernel, &cfg) == cudaSuccess && n >= 1;
				(void)cudaGetLastError();
			}
			if (wide > 0) C = 16;
		}
		cluster_cfg(C, cfg, attr, Bc);
		DB_CUDA(cudaFuncSetAttribute(head_train_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(cfg.dynamicSmemBytes, (size_t)48 * 1024)));
		DB_CUDA(cudaLaunchKernelEx(&cfg, head_train_cluster_kernel, a, Bc));
		DB_LAUNCH_CHECK();
		return;
	}
	DB_CUDA(cudaFuncSetAttribute(head_train_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
	// otherwise one large CTA per model hides the latency of the short dependent phases
	head_train_kernel<<<nmodel, nmodel <= 64 ? 1024 : 256, smem, state().stream>>>(a);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
