// A whole minibatch step of a small DeepBind model in two launches.
//
// The reference runs a step of deepity.sgd (sgd.py:121-147) as some thirty launches with
// every intermediate in HBM; the fused kernels of this library bring that to seven (fetch,
// look-ahead, scan+pool, dense head, filter gradient, its second stage, update), and for a
// minibatch of 64-128 short sequences those seven are a chain of latencies: about 30 us of
// which little is work.  Everything between the filter bank and the per-sample gradient is
// independent across samples, though: scan, rectifier, pooling, the dense layers, the loss,
// and their backward pass down to the sample's own contribution to every parameter
// gradient.  So here
//
//   ministep_sample_kernel   one CTA per (sample or strand pair, model): scan + bias +
//                            rectify + pool, dropout, dense head, loss, backward through the
//                            head, the pooling and the rectifier, and the sample's filter /
//                            bias gradient; activations never leave shared memory.  Writes
//                            the sample's partial filter gradient and a small record (masked
//                            pooled features, hidden activations, hidden and output deltas,
//                            loss) to scratch.
//   ministep_update_kernel   one thread per parameter: adds the samples' contributions,
//                            sample ascending (a fixed order, no atomics), adds the L1 decay
//                            term, and applies the Nesterov update of gradstep.cu:57-71
//                            followed at once by the next step's look-ahead.
//
// The minibatch is read in place from a device-resident dataset (slot = order[step % nbatch],
// step counter on the device, advanced by the update kernel), so a CUDA graph of N such
// pairs walks N steps with no host work and no copy.
//
// Parameters live in two flat vectors: P (the parameters as the reference holds them
// between steps) and PL = P + mrate*mP (where the gradient is taken, gradstep.cu:46-50).
// The update writes both; whoever changes P or mP from the host refreshes PL
// (db_ministep_lookahead).  The arithmetic per element is the reference's, expression for
// expression, so a run equals the seven-launch path up to the order of the gradient sums.
//
// Layouts as elsewhere in the library: X ordinal bytes, R [B,2] regions, Y [B,I], dropout
// keep-mask bytes [B, npool*I], Wscan [4m, F*I] model-major columns, W1 [(npool*I), H] stacked
// per model, b1 [H*I], W2 [(H*I), 1], b2 [I]; H = 0: W1 [(npool*I), 1], b1 [I].
#include "db_common.cuh"
#include "scan_lut.cuh"

namespace db {

static constexpr int MS_T = 256;          // threads per sample, at most (128 for short regions)
static constexpr int MS_PP = 16;          // row slices of the pooling pass, at most
static constexpr int US_E = 32;           // parameters per CTA of the update kernel
static constexpr int US_S = 8;            // sample slices of the update kernel (one warp each)

struct ministep_dev {
	db_ministep_args a;
	unsigned spc;          // samples (minibatch rows) per CTA: 1, or the 2 strands of a pair
	unsigned T;            // threads per sample: 128 or 256
	float* partial;        // [I][B][(4m+1)*F]
	float* rec;            // [I][B][RS]
	unsigned np, HC, RS, n;
};

// Offsets (in bytes) of a strand's private shared-memory block.
struct ms_layout { unsigned act, oh, small, amax, pp, accs, xs, total; };
__host__ __device__ inline unsigned ms_units(unsigned m, unsigned F) { return ((m + 3) / 4) * F + F; }
__host__ __device__ inline unsigned ms_rsplit(unsigned m, unsigned F, unsigned T) { const unsigned u = ms_units(m, F); return u >= T ? 1u : T / u; }
__host__ __device__ inline ms_layout ms_strand_layout(unsigned max_rows, unsigned m, unsigned F, unsigned HC, unsigned T)
{
	ms_layout l;
	unsigned o = 0;
	l.act = o;   o += max_rows * (F + 4) * 4;
	l.oh = o;    o += (max_rows + m + 4) * 16;
	l.small = o; o += (6 * F + 3 * ((HC + 3) & ~3u) + 8) * 4;       // pooled[2F] pd[2F] dpd[2F] h1 a1 dh misc[8]
	l.amax = o;  o += F * 4;
	l.pp = o;    o += MS_PP * F * 3 * 4;                             // pooling slices: max, row, sum
	l.accs = o;  o += (ms_rsplit(m, F, T) - 1) * ms_units(m, F) * 16 * 4; // gradient sums of the row splits after the first
	l.xs = o;    o += (max_rows + m + 8 + 3) & ~3u;
	l.total = (o + 15) & ~15u;
	return l;
}
__host__ __device__ inline unsigned ms_common_bytes(unsigned m, unsigned F, unsigned np, unsigned HC)
{
	return (m * (F / 4) * 32 + F + ((HC + 3) & ~3u) + np * (HC + 1)) * 4;      // lut, bias, w2, W1 (rows padded by one)
}

// 80 registers: six CTAs of 128 threads per SM, so that 12 models x 64 samples are one wave.
template <int M>
__global__ void __maxnreg__(80)
ministep_sample_kernel(const ministep_dev d)
{
	extern __shared__ __align__(16) unsigned char smem[];
	const db_ministep_args& a = d.a;
	const unsigned m = M > 0 ? (unsigned)M : a.m, F = a.nfilt, NQ = F / 4, AS = F + 4;
	const unsigned nf = F * a.nmodel, np = d.np, H = a.hidden, HC = d.HC;
	const unsigned b = blockIdx.y;
	const unsigned T = d.T;
	const unsigned strand = threadIdx.x / T, tid = threadIdx.x % T;     // which of the CTA's samples; thread within it
	const unsigned row_id = blockIdx.x * d.spc + strand;                // row of the minibatch

	float* lut = reinterpret_cast<float*>(smem);
	float* sb = lut + (size_t)m * NQ * 32;
	float* w2s = sb + F;
	float* w1s = w2s + ((HC + 3) & ~3u);
	const ms_layout L = ms_strand_layout(a.max_rows, m, F, HC, T);
	unsigned char* mine = smem + ms_common_bytes(m, F, np, HC) + (size_t)strand * L.total;
	float* act = reinterpret_cast<float*>(mine + L.act);
	float4* oh = reinterpret_cast<float4*>(mine + L.oh);
	float* pooled = reinterpret_cast<float*>(mine + L.small);
	float* pd = pooled + 2 * F, *dpd = pd + 2 * F;
	float* h1 = dpd + 2 * F, *a1 = h1 + ((HC + 3) & ~3u), *dh = a1 + ((HC + 3) & ~3u), *misc = dh + ((HC + 3) & ~3u);
	unsigned* amax = reinterpret_cast<unsigned*>(mine + L.amax);
	float* pp = reinterpret_cast<float*>(mine + L.pp);
	float* accs = reinterpret_cast<float*>(mine + L.accs);
	uint8_t* xs = mine + L.xs;
	__shared__ unsigned s_slot;
	__shared__ float s_z[4];

	if (threadIdx.x == 0) {
		const unsigned c = a.counters ? *reinterpret_cast<volatile const uint32_t*>(a.counters) % a.nbatch : 0u;
		s_slot = a.order ? a.order[c] : c;
	}
	// The update kernel may be scheduled now (programmatic dependent launch): it fetches the
	// parameters' state and then waits for this whole grid before it touches anything we read or write.
	asm volatile("griddepcontrol.launch_dependents;");
	// everything that does not depend on the minibatch is fetched while the slot is looked up
	// All of it is requested before any of it is used: one trip to L2 instead of one per array.
	const float* PL = a.PL;
	const float b1v = tid < HC ? PL[a.off_b1 + b * HC + tid] : 0.f;
	const float b2v = H ? PL[a.off_b2 + b] : 0.f;
	uint2 rg0 = make_uint2(0u, 0u);
	if (a.R_stride == 0) rg0 = make_uint2(a.R[2 * row_id], a.R[2 * row_id + 1]);    // one region table for all minibatches
	const unsigned lf = F == 16 ? 4u : 5u;                               // F is 16 or 32
	const unsigned WS = HC + 1;                                          // row stride of W1 in shared memory: no bank conflicts either way
	{
		const float* W = PL + a.off_Wscan + b * F;
		const float* W1g = PL + a.off_W1 + (size_t)b * np * HC;
		const unsigned nlut = m * F, nw1 = np * HC, nt = blockDim.x;
		for (unsigned base = 0; base < max(nlut, nw1); base += 4 * nt) {
			float4 w[4]; float v1[4];
			#pragma unroll
			for (int i = 0; i < 4; ++i) {
				const unsigned t = base + i * nt + threadIdx.x;
				w[i] = make_float4(0.f, 0.f, 0.f, 0.f); v1[i] = 0.f;
				if (t < nlut) {
					const unsigned j = t >> lf, f = t & (F - 1);
					w[i] = make_float4(W[(size_t)(4 * j + 0) * nf + f], W[(size_t)(4 * j + 1) * nf + f],
					                   W[(size_t)(4 * j + 2) * nf + f], W[(size_t)(4 * j + 3) * nf + f]);
				}
				if (t < nw1) v1[i] = W1g[t];
			}
			float bs = 0.f, w2v = 0.f;
			if (base == 0) {
				if (threadIdx.x < F) bs = PL[a.off_bscan + b * F + threadIdx.x];
				if (threadIdx.x < H) w2v = PL[a.off_W2 + b * H + threadIdx.x];
			}
			#pragma unroll
			for (int i = 0; i < 4; ++i) {
				const unsigned t = base + i * nt + threadIdx.x;
				if (t < nlut) {                                              // the table entry of build_lut: four channels, their mean for N, zeros
					const unsigned j = t >> lf, f = t & (F - 1);
					float z = w[i].x; z += w[i].y; z += w[i].z; z += w[i].w;
					float* e = lut + ((size_t)(j * NQ + f / 4) * 8) * 4 + (f & 3);
					e[0] = w[i].x; e[4] = w[i].y; e[8] = w[i].z; e[12] = w[i].w; e[16] = z * 0.25f; e[20] = 0.f; e[24] = 0.f; e[28] = 0.f;
				}
				if (t < nw1) w1s[(t / HC) * WS + t % HC] = v1[i];
			}
			if (base == 0) {
				if (threadIdx.x < F) sb[threadIdx.x] = bs;
				if (threadIdx.x < H) w2s[threadIdx.x] = w2v;
			}
		}
	}
	__syncthreads();
	const size_t slot = s_slot;
	const uint8_t* X = a.X + slot * a.X_stride;
	const uint32_t* R = reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(a.R) + slot * a.R_stride);
	const float* Y = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(a.Y) + slot * a.Y_stride);
	const uint8_t* mask = a.dropmask ? a.dropmask + slot * a.mask_stride : nullptr;
	const size_t mrow = (size_t)row_id * np * a.nmodel + (size_t)b * np;     // this sample's features in [B, np*I]
	// the sample's target and mask bytes travel while the scan runs
	const float yv = Y[(size_t)row_id * a.nmodel + b];
	const bool kept = !(mask && tid < np && !mask[mrow + tid]);

	const unsigned r0 = a.R_stride == 0 ? rg0.x : R[2 * row_id], r1 = a.R_stride == 0 ? rg0.y : R[2 * row_id + 1];
	unsigned rows = r1 > r0 ? r1 - r0 : 0u;
	if (rows == 0 || rows > a.max_rows) {                                // reported, and kept inside the staged window
		if (tid == 0 && a.status) atomicMax(a.status, 2);
		rows = rows == 0 ? 1u : a.max_rows;
	}
	// rows of the region that have a scan output (the last m-1 rows of the buffer have none)
	const unsigned rows_w = d.n > r0 ? min(rows, d.n - r0) : 0u;
	for (unsigned t = tid; t < ((rows + m + 8 + 3) & ~3u); t += T) {
		const unsigned i = r0 + t;
		xs[t] = (uint8_t)code16_of(i < a.npos ? X[i] : 254u);
	}
	__syncthreads();

	// ---- scan + bias + rectify: a thread owns one row x 8 filters per pass; and the channel
	// weights of every input row for the backward pass (one-hot, 1/4 each for N, 0 for a dropped base)
	{
		const unsigned FH = F / 8, TRK = T / FH;                        // half groups of 8 filters; rows per pass
		const unsigned rl = tid % TRK, fh = tid / TRK;
		const unsigned char* lutp = reinterpret_cast<const unsigned char*>(lut) + fh * 256;
		for (unsigned p0 = 0; p0 < rows; p0 += TRK) {
			const unsigned row = p0 + rl;
			if (row >= rows) continue;
			float z[8];
			if (row < rows_w) scan_row_half<M>(lutp, NQ * 128, xs, row, m, z);
			else {
				#pragma unroll
				for (int v = 0; v < 8; ++v) z[v] = 0.f;
			}
			#pragma unroll
			for (int v = 0; v < 8; v += 4) {
				const float4 q = *reinterpret_cast<const float4*>(sb + fh * 8 + v);
				float4 x = make_float4(z[v] + q.x, z[v + 1] + q.y, z[v + 2] + q.z, z[v + 3] + q.w);
				x.x = x.x > 0.f ? x.x : 0.f; x.y = x.y > 0.f ? x.y : 0.f; x.z = x.z > 0.f ? x.z : 0.f; x.w = x.w > 0.f ? x.w : 0.f;
				*reinterpret_cast<float4*>(act + row * AS + fh * 8 + v) = x;
			}
		}
		for (unsigned t = tid; t < rows + m + 4; t += T) {
			const unsigned c = xs[t] >> 4;
			const float q = c == 4u ? 0.25f : 0.f;
			oh[t] = make_float4(c == 0u ? 1.f : q, c == 1u ? 1.f : q, c == 2u ? 1.f : q, c == 3u ? 1.f : q);
		}
	}
	__syncthreads();

	// ---- pooling: MS_PP row slices per filter, rows ascending within a slice, slices ascending
	// after that (strict '>' both times: the first maximum wins, as in poolrgn.cuh:60-78)
	const unsigned PP = min((unsigned)MS_PP, T / F);                     // row slices of the pooling pass
	const unsigned slice = (rows + PP - 1) / PP;
	if (tid < PP * F) {
		const unsigned f = tid & (F - 1), part = tid >> lf;
		const unsigned ra = min(rows, part * slice), rb = min(rows, ra + slice);
		float xmax = 0.f, xsum = 0.f; unsigned xi = 0xffffffffu;
		if (ra < rb) {
			const float* col = act + f;
			xmax = col[ra * AS]; xsum = xmax; xi = ra;
			#pragma unroll 4
			for (unsigned r = ra + 1; r < rb; ++r) {
				const float v = col[r * AS];
				if (v > xmax) { xmax = v; xi = r; }
				xsum += v;
			}
		}
		pp[(part * F + f) * 3] = xmax; pp[(part * F + f) * 3 + 1] = __uint_as_float(xi); pp[(part * F + f) * 3 + 2] = xsum;
	}
	__syncthreads();
	if (tid < F) {
		float xmax = pp[tid * 3], xsum = pp[tid * 3 + 2]; unsigned xi = __float_as_uint(pp[tid * 3 + 1]);
		for (unsigned part = 1; part < PP; ++part) {
			const float* e = pp + (part * F + tid) * 3;
			const unsigned ri = __float_as_uint(e[1]);
			if (ri != 0xffffffffu) {
				if (e[0] > xmax) { xmax = e[0]; xi = ri; }
				xsum += e[2];
			}
		}
		const float cnt = (float)rows;
		amax[tid] = xi;
		switch (a.ptype) {
		case DB_PT_MAX: pooled[tid] = xmax; break;
		case DB_PT_AVG: pooled[tid] = xsum / cnt; break;
		case DB_PT_SUM: pooled[tid] = xsum; break;
		default:        pooled[2 * tid] = xmax; pooled[2 * tid + 1] = xsum / cnt; break;
		}
	}
	__syncthreads();
	if (tid < np) pd[tid] = kept ? pooled[tid] : 0.f;                    // maskout: a dropped feature is exactly 0
	__syncthreads();

	// ---- dense head, forward
	if (tid < HC) {
		float s = 0.f;
		for (unsigned u = 0; u < np; ++u) s = fmaf(pd[u], w1s[u * WS + tid], s);
		s = s + b1v;
		h1[tid] = s;
		a1[tid] = s > 0.f ? s : 0.f;
	}
	__syncthreads();
	if (tid == 0) {
		float o;
		if (H) {
			float s = 0.f;
			for (unsigned c = 0; c < H; ++c) s = fmaf(a1[c], w2s[c], s);
			o = s + b2v;
		} else o = h1[0];
		s_z[strand] = a.loss_kind == 1 ? 1.f / (1.f + expf(-o)) : o;
	}
	__syncthreads();
	// loss and dout = (Z - Y) / B (loss.py:98-112); with strand pairs only the stronger strand of
	// a pair, the forward one on ties, carries loss and gradient (loss.py:113-117, maskout.cu:54-67).
	// Every thread works it out for itself: no hand-off.
	float dout, lossv;
	{
		const float z = s_z[strand];
		bool keep = true;
		if (a.strand_pairs) keep = (strand & 1u) ? !(s_z[strand ^ 1u] >= z) : (z >= s_z[strand ^ 1u]);
		float l;
		if (a.loss_kind == 1) l = logf(fmaxf(1e-15f, z)) * yv + logf(fmaxf(1e-15f, 1.f - z)) * (1.f - yv);
		else { const float e = z - yv; l = e * e; }
		dout = keep ? (z - yv) * (1.f / (float)a.B) : 0.f;
		lossv = keep ? l : 0.f;
	}
	// ---- dense head, backward
	if (tid < HC) dh[tid] = H ? (a1[tid] > 0.f ? dout * w2s[tid] : 0.f) : dout;
	__syncthreads();
	if (tid < np) {
		float s = 0.f;
		for (unsigned c = 0; c < HC; ++c) s = fmaf(dh[c], w1s[tid * WS + c], s);
		dpd[tid] = kept ? s : 0.f;
	}
	{   // the sample's record for the update kernel: pd | a1 | dh | dout | loss
		float* rec = d.rec + ((size_t)b * a.B + row_id) * d.RS;
		for (unsigned t = tid; t < d.RS; t += T) {
			float v;
			if (t < np) v = pd[t];
			else if (t < np + H) v = a1[t - np];
			else if (t < np + H + HC) v = dh[t - np - H];
			else v = t == np + H + HC ? dout : lossv;
			rec[t] = v;
		}
	}
	__syncthreads();

	// ---- pooling and rectifier backward: dZ in place of the activations
	float* davg = pooled, *dmax = pooled + F;
	if (tid < F) {
		const float cnt = (float)rows;
		float va = 0.f, vm = 0.f;
		switch (a.ptype) {
		case DB_PT_MAX: vm = dpd[tid]; break;
		case DB_PT_AVG: va = dpd[tid] / cnt; break;
		case DB_PT_SUM: va = dpd[tid]; break;
		default:        vm = dpd[2 * tid]; va = dpd[2 * tid + 1] / cnt; break;
		}
		if (a.ptype == DB_PT_MAX) vm = act[amax[tid] * AS + tid] > 0.f ? vm : 0.f;   // one nonzero row per filter: its delta
		davg[tid] = va; dmax[tid] = vm;
	}
	__syncthreads();
	const bool only_max = a.ptype == DB_PT_MAX;
	if (!only_max) {
		// a thread keeps its filter: its mean share, maximum delta and argmax row stay in registers
		const unsigned f = tid & (F - 1), rstep = T >> lf;
		const float va = davg[f], vm = a.ptype == DB_PT_ALL ? dmax[f] : 0.f;
		const unsigned am = a.ptype == DB_PT_ALL ? amax[f] : 0xffffffffu;
		float* col = act + f;
		#pragma unroll 4
		for (unsigned r = tid >> lf; r < rows; r += rstep) {
			float v = 0.f;
			if (col[r * AS] > 0.f) v = r == am ? va + vm : va;
			col[r * AS] = v;
		}
		__syncthreads();
	}

	// ---- the sample's filter and bias gradient: a thread per (four taps, filter) and row split,
	// rows ascending within a split, splits ascending after that
	float* part = d.partial + ((size_t)b * a.B + row_id) * (size_t)(4 * m + 1) * F;
	const unsigned nunit = ((m + 3) / 4) * F, U = nunit + F, RSP = ms_rsplit(m, F, T);
	const unsigned rchunk = ((rows + RSP - 1) / RSP + 3u) & ~3u;
	for (unsigned t0 = 0; t0 < U * RSP; t0 += T) {
		const unsigned t = t0 + tid;
		const unsigned split = t / U, unit = t % U;
		const bool on = t < U * RSP;
		const unsigned ra = min(rows, split * rchunk), rb = min(rows, ra + rchunk);
		float c[4][4];
		#pragma unroll
		for (int q = 0; q < 4; ++q)
			#pragma unroll
			for (int k = 0; k < 4; ++k) c[q][k] = 0.f;
		if (on && unit < nunit) {
			const unsigned j0 = 4 * (unit >> lf), fl = unit & (F - 1);
			const float4* ohj = oh + j0;
			if (only_max) {
				const unsigned r = amax[fl];
				if (r >= ra && r < rb && r < rows_w) {
					const float v = dmax[fl];
					bwd_fma4(c[0], v, ohj[r]); bwd_fma4(c[1], v, ohj[r + 1]); bwd_fma4(c[2], v, ohj[r + 2]); bwd_fma4(c[3], v, ohj[r + 3]);
				}
			} else {
				const unsigned re = min(rb, rows_w);
				const float* dzc = act + fl;
				unsigned r = ra;
				if (r + 4 <= re) {
					float4 w0 = ohj[r], w1 = ohj[r + 1], w2 = ohj[r + 2], w3 = ohj[r + 3];
					for (; r + 4 <= re; r += 4) {                           // the window of channel weights rotates through its registers
						float v = dzc[(r + 0) * AS];
						bwd_fma4(c[0], v, w0); bwd_fma4(c[1], v, w1); bwd_fma4(c[2], v, w2); bwd_fma4(c[3], v, w3);
						w0 = ohj[r + 4];
						v = dzc[(r + 1) * AS];
						bwd_fma4(c[0], v, w1); bwd_fma4(c[1], v, w2); bwd_fma4(c[2], v, w3); bwd_fma4(c[3], v, w0);
						w1 = ohj[r + 5];
						v = dzc[(r + 2) * AS];
						bwd_fma4(c[0], v, w2); bwd_fma4(c[1], v, w3); bwd_fma4(c[2], v, w0); bwd_fma4(c[3], v, w1);
						w2 = ohj[r + 6];
						v = dzc[(r + 3) * AS];
						bwd_fma4(c[0], v, w3); bwd_fma4(c[1], v, w0); bwd_fma4(c[2], v, w1); bwd_fma4(c[3], v, w2);
						w3 = ohj[r + 7];
					}
				}
				for (; r < re; ++r) {
					const float v = dzc[r * AS];
					bwd_fma4(c[0], v, ohj[r]); bwd_fma4(c[1], v, ohj[r + 1]); bwd_fma4(c[2], v, ohj[r + 2]); bwd_fma4(c[3], v, ohj[r + 3]);
				}
			}
		} else if (on) {
			const unsigned fl = unit - nunit;
			float s = 0.f;
			if (only_max) { if (ra == 0) s = dmax[fl]; }
			else for (unsigned r = ra; r < rb; ++r) s += act[r * AS + fl];
			c[0][0] = s;
		}
		if (RSP > 1) {
			if (on && split > 0) {
				float4* dst = reinterpret_cast<float4*>(accs + ((size_t)(split - 1) * U + unit) * 16);
				#pragma unroll
				for (int q = 0; q < 4; ++q) dst[q] = make_float4(c[q][0], c[q][1], c[q][2], c[q][3]);
			}
			__syncthreads();
			if (on && split == 0) {
				for (unsigned sp = 1; sp < RSP; ++sp) {
					const float4* src = reinterpret_cast<const float4*>(accs + ((size_t)(sp - 1) * U + unit) * 16);
					#pragma unroll
					for (int q = 0; q < 4; ++q) { const float4 v = src[q]; c[q][0] += v.x; c[q][1] += v.y; c[q][2] += v.z; c[q][3] += v.w; }
				}
			}
		}
		if (on && split == 0) {
			if (unit < nunit) {
				const unsigned j0 = 4 * (unit >> lf), fl = unit & (F - 1);
				#pragma unroll
				for (int q = 0; q < 4; ++q)
					if (j0 + q < m) {
						#pragma unroll
						for (int k = 0; k < 4; ++k) part[(size_t)(4 * (j0 + q) + k) * F + fl] = c[q][k];
					}
			} else part[(size_t)4 * m * F + (unit - nunit)] = c[0][0];
		}
	}
}

// A CTA per tile of US_E parameters of a model: warp w adds the shares of the w-th slice of the
// minibatch rows, ascending, all its loads in flight at once; warp 0 then adds the slices,
// ascending, adds the L1 decay term and applies the Nesterov update and the next look-ahead.
// The tile after the last parameter sums the loss; thread 0 of the launch advances the step
// counter.  The order of every sum is fixed.
__global__ void __launch_bounds__(US_E * US_S)
ministep_update_kernel(const ministep_dev d)
{
	const db_ministep_args& a = d.a;
	const unsigned m = a.m, F = a.nfilt, nf = F * a.nmodel, np = d.np, H = a.hidden, HC = d.HC, B = a.B, RS = d.RS;
	const unsigned b = blockIdx.y, lane = threadIdx.x % US_E, w = threadIdx.x / US_E;
	const unsigned e = blockIdx.x * US_E + lane;
	const unsigned NS = (4 * m + 1) * F, NH = np * HC + HC + (H ? H + 1 : 0);
	__shared__ float sums[US_S][US_E];
	const float* rec = d.rec + (size_t)b * B * RS;
	const unsigned per = (B + US_S - 1) / US_S, s0 = min(B, w * per), s1 = min(B, s0 + per);
	float g = 0.f;
	size_t pi = 0;
	// what this parameter's share of sample s is: one value (x1 = 1), or a product of two record entries
	const float* p0 = nullptr; const float* p1 = nullptr; size_t st = RS;
	if (e < NS) {
		const unsigned k = e / F, f = e % F;
		pi = k < 4 * m ? (size_t)a.off_Wscan + (size_t)k * nf + b * F + f : (size_t)a.off_bscan + b * F + f;
		p0 = d.partial + (size_t)b * B * NS + e; st = NS;
	} else if (e < NS + NH) {
		unsigned h = e - NS;
		if (h < np * HC) {                                                   // dW1 = sum_i pd_i (x) dh_i
			const unsigned u = h / HC, c = h % HC;
			pi = (size_t)a.off_W1 + ((size_t)b * np + u) * HC + c;
			p0 = rec + u; p1 = rec + np + H + c;
		} else if ((h -= np * HC) < HC) {                                    // db1 = sum_i dh_i
			pi = (size_t)a.off_b1 + b * HC + h; p0 = rec + np + H + h;
		} else if ((h -= HC) < H) {                                          // dW2 = sum_i a1_i * dout_i
			pi = (size_t)a.off_W2 + b * H + h; p0 = rec + np + h; p1 = rec + np + H + HC;
		} else {                                                             // db2 = sum_i dout_i
			pi = (size_t)a.off_b2 + b; p0 = rec + np + H + HC;
		}
	} else if (e == NS + NH) p0 = rec + np + H + HC + 1;                     // the loss terms
	// the parameter's state travels while the shares are added
	float pl = 0.f, mr = 0.f, dr = 0.f, mp0 = 0.f, dc = 0.f;
	if (w == 0 && p0 && e < NS + NH) {
		pl = a.PL[pi]; mr = a.mrate[pi]; dr = a.drate[pi]; mp0 = a.mP[pi];
		if (a.decay) dc = a.decay[pi];
	}
	// Launched as a programmatic dependent of the sample kernel, this grid may have started while
	// that one was still running: from here on everything depends on its results (and nothing
	// above was written by it or is still read by it).
	asm volatile("griddepcontrol.wait;" ::: "memory");
	if (b == 0 && blockIdx.x == 0 && threadIdx.x == 0 && a.counters) *a.counters = *a.counters + 1;
	if (p0) {
		for (unsigned s = s0; s < s1; s += 16) {
			float x0[16], x1[16];
			#pragma unroll
			for (int i = 0; i < 16; ++i) {
				const bool in = s + i < s1;
				x0[i] = in ? p0[(size_t)(s + i) * st] : 0.f;
				x1[i] = (in && p1) ? p1[(size_t)(s + i) * st] : 1.f;
			}
			#pragma unroll
			for (int i = 0; i < 16; ++i) g = fmaf(x0[i], x1[i], g);
		}
	}
	sums[w][lane] = g;
	__syncthreads();
	if (w != 0 || !p0) return;
	g = sums[0][lane];
	#pragma unroll
	for (int q = 1; q < US_S; ++q) g += sums[q][lane];
	if (e == NS + NH) {
		if (a.loss) a.loss[b] = (a.loss_kind == 0 ? 0.5f : -1.f) * (g * (1.f / (float)B));
		return;
	}
	if (a.decay) {
		const float sg = pl > 0.f ? 1.f : (pl < 0.f ? -1.f : 0.f);
		g = g + dc * sg;                                                     // corr1ord.py:112-126, full.py:102-119
	}
	if (a.dP) a.dP[pi] = g;
	// gradstep.cu:57-71 (second half of the Nesterov step), then gradstep.cu:46-50 for the next one
	const float delta = g * dr;
	const float mp = mp0 * mr - delta;
	const float p = pl - delta;
	a.mP[pi] = mp;
	a.P[pi] = p;
	a.PL[pi] = p + mr * mp;
}

__global__ void ministep_lookahead_kernel(float* __restrict__ PL, const float* __restrict__ P, const float* __restrict__ mP,
                                          const float* __restrict__ mrate, size_t n)
{
	for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
		PL[i] = P[i] + mrate[i] * mP[i];
}

static unsigned ms_npool(const db_ministep_args* a) { return a->ptype == DB_PT_ALL ? 2 * a->nfilt : a->nfilt; }

// Threads per sample: 256, or 128 where a region's rows fit one scan pass of 128 threads (the
// fixed work of the kernel's phases is per warp).
static unsigned ms_threads(const db_ministep_args* a) { return a->max_rows * (a->nfilt / 16u) <= 64u ? 128u : 256u; }

static size_t ms_smem(const db_ministep_args* a, unsigned spc)
{
	const unsigned HC = a->hidden ? a->hidden : 1u;
	return ms_common_bytes(a->m, a->nfilt, ms_npool(a), HC) +
	       (size_t)spc * ms_strand_layout(a->max_rows, a->m, a->nfilt, HC, ms_threads(a)).total;
}

// Samples per CTA: one, or the two strands of a pair.  Four samples sharing the staged lookup
// table and dense weights were measured slower where they could apply (12 models x 64 samples:
// 26.3 against 23.0 us per step): the barriers of a 1024-thread CTA cost more than the staging.
static unsigned ms_spc(const db_ministep_args* a) { return a->strand_pairs ? 2u : 1u; }

}  // namespace db

using namespace db;

DB_EXPORT int db_ministep_supported(const db_ministep_args* a)
{
	if (!a) return 0;
	if (a->nfilt != 16 && a->nfilt != 32) return 0;
	if (a->m < 1 || a->m > 64 || a->hidden > 128u || ms_npool(a) > 128u) return 0;
	if (a->ptype > (uint32_t)DB_PT_ALL) return 0;
	if (a->strand_pairs && (a->B & 1u)) return 0;
	if (!a->B || !a->nmodel || a->nmodel > 65535u || !a->max_rows) return 0;
	return ms_smem(a, a->strand_pairs ? 2u : 1u) <= 200 * 1024 ? 1 : 0;
}

DB_EXPORT size_t db_ministep_scratch_bytes(const db_ministep_args* a)
{
	if (!a) return 0;
	const unsigned HC = a->hidden ? a->hidden : 1u;
	const size_t RS = ms_npool(a) + a->hidden + HC + 2;
	return ((size_t)a->nmodel * a->B * ((size_t)(4 * a->m + 1) * a->nfilt + RS)) * sizeof(float) + 256;
}

DB_EXPORT void db_ministep_lookahead(float* PL, const float* P, const float* mP, const float* mrate, size_t n)
{
	DB_API_TRY
	if (!n) return;
	DB_REQUIRE(PL && P && mP && mrate, "ValueError: db_ministep_lookahead got a NULL pointer");
	ministep_lookahead_kernel<<<elemwise_grid(n), 256, 0, state().stream>>>(PL, P, mP, mrate, n);
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}

DB_EXPORT void db_ministep(const db_ministep_args* args)
{
	DB_API_TRY
	DB_REQUIRE(args != nullptr, "ValueError: db_ministep got NULL");
	DB_REQUIRE(db_ministep_supported(args), "ValueError: this model or minibatch shape is outside the two-launch step "
	           "(16 or 32 filters per model, at most %d pooled features and hidden units, regions that fit shared memory)", 128);
	const db_ministep_args& a = *args;
	DB_REQUIRE(a.X && a.R && a.Y && a.P && a.PL && a.mP && a.drate && a.mrate, "ValueError: db_ministep got a NULL pointer");
	DB_REQUIRE(!a.counters || a.nbatch, "ValueError: a step counter needs the number of minibatches");
	DB_REQUIRE(a.npos >= a.m, "ValueError: the ordinal buffer is shorter than the filters");
	ministep_dev d;
	d.a = a;
	if (!d.a.counters) d.a.nbatch = 1;
	d.np = ms_npool(args); d.HC = a.hidden ? a.hidden : 1u; d.RS = d.np + a.hidden + d.HC + 2;
	d.n = a.npos - a.m + 1;
	const size_t npart = (size_t)a.nmodel * a.B * (size_t)(4 * a.m + 1) * a.nfilt;
	float* sc = reinterpret_cast<float*>(scratch(db_ministep_scratch_bytes(args)));
	d.partial = sc; d.rec = sc + ((npart + 63) & ~(size_t)63);
	d.spc = ms_spc(args); d.T = ms_threads(args);
	const size_t smem = ms_smem(args, d.spc);
	dim3 grid(a.B / d.spc, a.nmodel), block(d.T * d.spc);
	auto launch = [&](auto kern) {
		DB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, (size_t)48 * 1024)));
		kern<<<grid, block, smem, state().stream>>>(d);
	};
	if (a.m == 24) launch(ministep_sample_kernel<24>);
	else if (a.m == 16) launch(ministep_sample_kernel<16>);
	else launch(ministep_sample_kernel<0>);
	DB_LAUNCH_CHECK();
	const unsigned nelem = (4 * a.m + 1) * a.nfilt + d.np * d.HC + d.HC + (a.hidden ? a.hidden + 1 : 0) + 1;
	{
		cudaLaunchConfig_t cfg = {};
		cfg.gridDim = dim3(divup(nelem, (unsigned)US_E), a.nmodel); cfg.blockDim = dim3(US_E * US_S);
		cfg.dynamicSmemBytes = 0; cfg.stream = state().stream;
		cudaLaunchAttribute attr[1];
		attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
		attr[0].val.programmaticStreamSerializationAllowed = 1;
		cfg.attrs = attr; cfg.numAttrs = 1;
		DB_CUDA(cudaLaunchKernelEx(&cfg, ministep_update_kernel, d));
	}
	DB_LAUNCH_CHECK();
	DB_API_CATCH
}
