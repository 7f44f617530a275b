/*
 * deepbind_b200 -- C ABI of libdeepbind_b200.so
 *
 * A from-scratch sm_100a implementation of DeepBind's data-parallel hot path
 * (motif scan over ordinal DNA/RNA, rectify + region pooling, the small dense
 * layers and the momentum update) behind the entry points the reference's
 * ctypes layer binds.  Citations name files of the reference tree
 * (jisraeli/DeepBind, paths relative to its root).
 *
 * Conventions kept from the reference (code/libs/smat/src/smat/smat.cpp:608-760,
 * code/libs/smat/py/smat/smat_dll.py:85-92,166-183):
 *   - every function is extern "C", returns void (or a plain value), never throws;
 *   - failures leave a message that api_get_last_error() returns until
 *     api_clear_last_error(); messages start with a Python exception name
 *     ("ValueError: ...", "TypeError: ...", "AssertionError: CUDA error ...");
 *   - arrays are 2-D, row-major; shape.x = columns, shape.y = rows;
 *   - calls are asynchronous on one CUDA stream; api_sync() waits for it;
 *   - accumulating operations (corr1ord's tail rows, corr1ord_bprop_W's dW,
 *     corr1ord_bprop_X's dX, poolrgn_bprop's unpooled) add into memory the
 *     caller has zeroed (code/libs/kangaroo/kangaroo/_ext/corr1ord.py:101,121,132;
 *     poolrgn.py:79,123,177).
 * There is no CPU fallback: without a CUDA device every compute call fails with
 * an error message.
 */
#ifndef DEEPBIND_B200_H
#define DEEPBIND_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype codes: code/libs/smat/src/smat/dtypes.h:67-80 */
enum db_dtype { DB_B8 = 0, DB_I8 = 1, DB_U8 = 2, DB_I16 = 3, DB_U16 = 4, DB_I32 = 5,
                DB_U32 = 6, DB_I64 = 7, DB_U64 = 8, DB_F32 = 9, DB_F64 = 10 };

/* value-type codes: code/libs/smat/src/smat/vm/argument.h:48-55 */
enum db_vtype { DB_VT_NONE = 0, DB_VT_HARRAY = 1, DB_VT_DARRAY = 2 };

typedef struct db_shape  { int32_t x, y, z; } db_shape;   /* smat/shape.h:62-74 */
typedef struct db_coord  { int32_t x, y, z; } db_coord;

/* Array handle.  The first four members are the prefix Python mirrors
 * (smat_dll.py:85-92); the rest is private to the library. */
typedef struct smat {
	int32_t  vtype;
	int32_t  dtype;
	db_shape shape;      /* x = columns, y = rows, z = 1 */
	db_coord strides;    /* in elements: x = 1, y = row stride */
	void*    data;       /* device address */
	int32_t  owns_data;  /* 1: api_delete frees data; 0: borrowed (api_wrap) */
	int32_t  device;
} smat;

/* option structs: kangaroo_smat.cpp:84-96, kangaroo_smat.h:38-47 */
typedef struct corr1ord_options_t { int32_t padmode; uint32_t nchannel; } corr1ord_options_t;
typedef struct poolrgn_options_t  { int32_t ptype; } poolrgn_options_t;
enum db_pooltype { DB_PT_MAX = 0, DB_PT_AVG = 1, DB_PT_SUM = 2, DB_PT_ALL = 3 };

/* ---- error channel, stream, handles (smat.cpp:612-613,622-660) ----------- */
const char* api_get_last_error(void);
void        api_clear_last_error(void);
void        api_sync(void);                         /* cuda_context.cpp:198-202 */
void        api_set_stream(void* cuda_stream);      /* no counterpart: lets the host share its stream */
void*       api_get_stream(void);
int         api_device_count(void);
void        api_set_device(int device);             /* "device=" backend option, cuda_context.cpp:184-188 */
smat*       api_empty(const db_shape* shape, int dtype);
smat*       api_zeros(const db_shape* shape, int dtype);
smat*       api_wrap(void* device_ptr, int rows, int cols, int dtype); /* borrowed memory; no counterpart */
void        api_delete(const smat* M);
int32_t     api_nrow(const smat* M);
int32_t     api_ncol(const smat* M);
size_t      api_size(const smat* M);
int         api_dtype(const smat* M);
void*       api_data(const smat* M);
void        api_copy_from(smat* M, const void* host_src, int32_t row_stride_bytes, int32_t col_stride_bytes);
void        api_copy_to(const smat* M, void* host_dst, int32_t row_stride_bytes, int32_t col_stride_bytes);
void        api_fill_zero(smat* M);
void        api_set_seed(uint64_t seed);            /* "seed=" backend option */
uint64_t    api_launch_count(void);                 /* kernels launched so far by this thread; no counterpart */
/* Scratch of the two-stage reductions (filter gradients, column sums).  It grows on
 * demand with cudaMalloc and is never freed while the process lives, because a CUDA
 * graph captured from a step keeps the address it saw.  It cannot grow while the
 * stream is being captured: run the step once first, or reserve the largest size
 * here.  No counterpart: the reference allocates per call from smat's heap. */
void        db_reserve_scratch(size_t bytes);
size_t      db_scratch_bytes(void);
void        register_ext(void);                     /* extension.cpp:159-169; nothing to register here */
void        api_autotune(void);                     /* kangaroo_smat.cpp (autotune.cu:91-113): no-op */

/* ---- kangaroo_smat (kangaroo_smat.cpp:333-418) ---------------------------- */
void api_corr1ord(const smat* W, const smat* X, smat* Z, const corr1ord_options_t* options);
void api_corr1ord_bprop_W(smat* dW, const smat* X, const smat* dZ, const corr1ord_options_t* options);
void api_corr1ord_bprop_X(smat* dX, const smat* W, const smat* dZ, const corr1ord_options_t* options);
void api_poolrgn(const smat* unpooledmaps, const smat* regions, smat* pooledmaps,
                 smat* pooledmaps_argmax /* nullable */, const poolrgn_options_t* options);
void api_poolrgn_bprop(smat* unpooledmaps, const smat* regions, const smat* pooledmaps,
                       const smat* pooledmaps_argmax /* nullable */, const poolrgn_options_t* options);
void api_dropoutord_fp_tr(const smat* X, smat* Z, smat* M, float rate);
/* same, with the uniform draws supplied (f32, one per element): reproducible masks */
void api_dropoutord_fp_tr_u(const smat* X, const smat* U, smat* Z, smat* M, float rate);

/* ---- deepity_smat (deepity_smat.cpp:497-607) ------------------------------ */
void api_gradstep(smat* P, const smat* dP, const smat* drate, smat* mP, const smat* mrate);
void api_gradstep_nesterov1(smat* P, const smat* mP, const smat* mrate);
void api_gradstep_nesterov2(smat* P, const smat* dP, const smat* drate, smat* mP, const smat* mrate);
void api_madd_bcast(const smat* A, const smat* b, uint32_t k, smat* dst);
void api_maskout(const smat* M, smat* A);
void api_calc_zmask(const smat* Z, smat* M);
void api_dropout_fp_tr(const smat* X, const smat* rate, smat* Z, smat* M, int matchrows);
void api_dropout_fp_tr_u(const smat* X, const smat* rate, const smat* U, smat* Z, smat* M, int matchrows);
void api_dropout_fp_te(const smat* X, const smat* rate, smat* Z);
void api_dropout_bp_tr(const smat* dZ, const smat* M, smat* dX);
void api_dropout_bp_te(const smat* dZ, const smat* rate, smat* dX);
void api_blockwise_dot(int nblock, const smat* X, const smat* W, smat* Z);
void api_blockwise_dot_nt(int nblock, const smat* dZ, const smat* W, smat* dX);
void api_blockwise_dot_tn(int nblock, const smat* X, const smat* dZ, smat* dW);
void api_blockwise_dot_combined(int nblock, int Xoffset, int Xbroadcast, const smat* X, const smat* W, smat* Z);
void api_blockwise_dot_nt_combined(int nblock, int Xoffset, int Xbroadcast, smat* dX, const smat* W, const smat* dZ);
void api_blockwise_dot_tn_combined(int nblock, int Xoffset, int Xbroadcast, const smat* X, smat* dW, const smat* dZ);

/* ---- layer arithmetic the reference runs through generic smat ops ---------
 * (code/libs/deepity/deepity/std/elemwise.py:71-82,162-180, softmax.py:50-77,
 * loss.py:52-155; smat_cuda/elemwise3.cuh, elemwise2.cuh, reduce_y.cuh:52-126).
 * Plain device pointers, f32, row-major. */
void db_bias_add(float* Z, const float* X, const float* b, uint32_t nrow, uint32_t ncol);        /* Z = X + b   */
void db_relu(float* Z, const float* X, size_t n);                                                /* max(0,X)    */
void db_relu_bprop(float* dX, const float* dZ, const float* Z, size_t n);                        /* dZ*sign(Z)  */
void db_colsum(float* out, const float* A, uint32_t nrow, uint32_t ncol);                        /* sum(A,axis=0), fixed order */
/* No counterpart in the reference.  Same result as db_colsum, for callers that
 * must not allocate device memory (a host that owns all GPU memory through its
 * own pool, or one that may not call cudaMalloc where it runs): the partial sums
 * go to a 1 MiB array built into the library, so no cudaMalloc/cudaFree happens
 * in this call.  Limit: ceil(nrow/256)*ncol <= 262144, else an error.  The
 * first call on a device looks the array's address up; make that call before
 * any stream capture.  All calls share the array: calls that overlap on the GPU
 * (different streams) race on it. */
void db_colsum_static(float* out, const float* A, uint32_t nrow, uint32_t ncol);
void db_logistic(float* Z, const float* X, size_t n);
/* Strand choice of scoring (kangaroo/predict.py:145-164): Z [2*npair, ncol] holds forward /
 * reverse-complement row pairs; out [npair, ncol] keeps the larger score, the forward one on ties. */
void db_strand_max(float* out, const float* Z, uint32_t npair, uint32_t ncol);
/* n standard normal draws (smat's randn, smat_cuda/rand.cu:66-88, which the trainer scales per
 * model with madd_bcast: sgd.py:331-340); the stream follows api_set_seed and advances per call. */
void db_randn(float* out, size_t n);
/* loss_node forward+backward (loss.py:52-112): kind 0 = mse, 1 = nll.  Z,Y [nrow,ncol];
 * Ymask/Zmask nullable bool [nrow,ncol]; loss_out [ncol] = scaled column means;
 * dZ (nullable) = maskout(Z-Y) / nrow. */
void db_loss(int kind, const float* Z, const float* Y, const uint8_t* Ymask, const uint8_t* Zmask,
             uint32_t nrow, uint32_t ncol, float* loss_out, float* dZ);

/* L1 weight decay (corr1ord.py:112-126, full.py:102-119): dP[i] += decay[i] * sign(P[i]);
 * `decay` is the per-model decay spread over the flat parameter vector, zero on biases. */
void db_l1_decay(float* dP, const float* P, const float* decay, size_t n);

/* Dropout keep-mask of one training step drawn on the device (dropout.cu:41-62: keep where
 * u >= rate[model]; matchrows: the two strands of a row pair share a mask row), for steps
 * replayed from a CUDA graph: the draw index is counters[0] (device uint32[2], zero before
 * the first call), advanced by the launch itself, so every replay draws a fresh mask.
 * M bool [nrow, ncol], ncol = features per model * nmodel; rate f32 [nmodel]. */
void db_dropout_mask(uint8_t* M, uint32_t nrow, uint32_t ncol, const float* rate, uint32_t nmodel,
                     int matchrows, uint32_t* counters);

/* Minibatch fetch on the device (the reference uploads every minibatch from the host:
 * deepity/data.py, kangaroo/data.py:274-354).  The dataset lies in HBM as `nbatch`
 * equally sized minibatches per array; one launch copies minibatch
 * order[counters[0] % nbatch] (or counters[0] % nbatch itself when order is NULL) of up
 * to three arrays (src_k + index * bytes_k -> dst_k; NULL pointers or 0 bytes skip an
 * array) and then advances counters[0].  counters is a device array of two uint32, both
 * zero before the first call.  Captured into a CUDA graph in front of a training step
 * it lets the graph be replayed with no host work between steps. */
void db_minibatch_fetch(uint32_t* counters, const uint32_t* order, uint32_t nbatch,
                        const void* src0, void* dst0, size_t bytes0,
                        const void* src1, void* dst1, size_t bytes1,
                        const void* src2, void* dst2, size_t bytes2);

/* Measurement aid, no counterpart in the reference: launches a register-only chain of
 * FP32 adds on every lane (2048 threads per SM, 128 * iters adds per thread) on the
 * library's stream and returns the number of adds launched (0 on error).  Timed with
 * events by the caller it gives the non-FMA FP32 issue rate the lookup-add kernels
 * are measured against.  `sink` (nullable, one float) is never written. */
uint64_t db_fadd_probe(float* sink, uint32_t iters);

/* The dense head of one training step in one launch (no counterpart as one call;
 * replaces dropout -> full -> bias -> rectify -> full -> bias -> logistic -> loss and
 * their backward passes: elemwise.py:128-150,171,74-78, full.py:78-89, softmax.py:50-61,
 * loss.py:52-112, deepity_smat.py:169-204).  One CTA per model holds that model's
 * minibatch in shared memory.  pooled/dpooled/dropmask [B, npool*nmodel]; Y [B, nmodel];
 * hidden = 0: linear head W1 [(npool*nmodel),1], b1 [nmodel]; hidden = H: W1
 * [(npool*nmodel),H], b1 [H*nmodel], W2 [(H*nmodel),1], b2 [nmodel].  loss_kind 0 = mse,
 * 1 = nll on logistic outputs.  strand_pairs != 0: rows 2k, 2k+1 are the two strands of
 * one sequence and only the row with the larger output (the first on ties) contributes
 * to loss and gradient, as calc_zmask + maskout do in loss.py:52-65,98-117; the mean
 * still divides by B.  Writes loss [nmodel], dpooled and the four parameter
 * gradients (overwritten).  B must not exceed db_head_max_batch(npool, hidden). */
uint32_t db_head_max_batch(uint32_t npool, uint32_t hidden);
void db_head_train(uint32_t nmodel, uint32_t npool, uint32_t hidden, int loss_kind, int strand_pairs, uint32_t B,
                   const float* pooled, const uint8_t* dropmask, const float* Y,
                   const float* W1, const float* b1, const float* W2, const float* b2,
                   float* loss, float* dpooled, float* dW1, float* db1, float* dW2, float* db2);

/* A whole minibatch step of a small model in two launches (what deepity.sgd runs per step,
 * sgd.py:121-147: look-ahead of gradstep.cu:46-50, forward and backward pass of the DeepBind
 * layer chain -- corr1ord.cuh:47-166, elemwise.py:71-82,116-180, poolrgn.cuh:44-160,
 * full.py:41-119, softmax.py:50-77, loss.py:40-155 and their gradients -- L1 decay, update of
 * gradstep.cu:57-71).  One CTA per (sample or strand pair, model) takes its sample through
 * the whole chain in shared memory and writes the sample's share of every gradient; a
 * second kernel adds the shares (sample ascending), updates P, mP and the look-ahead copy PL
 * = P + mrate*mP, and advances the step counter.  Gradients are taken at PL.
 *
 * The minibatch of a step is slot order[counters[0] % nbatch] (or the count itself without
 * order) of a device-resident dataset: X, R, Y, dropmask point at slot 0 and the strides (in
 * bytes) lead from slot to slot; counters = NULL: always slot 0.  All flat parameter vectors
 * hold the blocks Wscan [4m, nfilt*nmodel] (columns model-major), bscan, W1, b1, W2, b2 at the
 * given offsets (in elements); hidden = 0: a linear head, W1 [(npool*nmodel),1], b1 [nmodel],
 * off_W2/off_b2 unused.  npool = nfilt (max, avg, sum pooling) or 2*nfilt (all).  dropmask
 * (bool bytes [B, npool*nmodel], NULL: none), decay (NULL: none), dP (NULL: gradient not
 * kept), loss [nmodel] (NULL: not kept).  max_rows: the longest region of any minibatch, in
 * rows (L + m - 1); status (int32, may be NULL) is raised to 2 if a region is empty or longer.
 * Scratch comes from the library's buffer (db_ministep_scratch_bytes; reserve it before a
 * stream capture).  db_ministep_supported: nfilt 16 or 32, at most 128 pooled features and
 * hidden units, B even with strand pairs, regions that fit shared memory.
 * db_ministep_lookahead: PL = P + mrate*mP, to be called before the first step and whenever
 * the host changed P or mP. */
typedef struct db_ministep_args {
	uint32_t nmodel, nfilt, m, ptype, hidden, loss_kind, strand_pairs, B, max_rows, npos;
	const uint8_t* X; size_t X_stride;
	const uint32_t* R; size_t R_stride;
	const float* Y; size_t Y_stride;
	const uint8_t* dropmask; size_t mask_stride;
	uint32_t* counters; const uint32_t* order; uint32_t nbatch;
	float* P; float* PL; float* mP; float* dP;
	const float* drate; const float* mrate; const float* decay;
	uint32_t off_Wscan, off_bscan, off_W1, off_b1, off_W2, off_b2;
	float* loss;
	int32_t* status;
} db_ministep_args;
int db_ministep_supported(const db_ministep_args* args);
size_t db_ministep_scratch_bytes(const db_ministep_args* args);
void db_ministep_lookahead(float* PL, const float* P, const float* mP, const float* mrate, size_t n);
void db_ministep(const db_ministep_args* args);

/* ---- minibatch assembly on the device (replaces the host-side string joins of
 * kangaroo/data.py:309-334 with util.py:43-74 acgt2ord / revcomp, and the strand
 * doubling of data.py:274-283) -----------------------------------------------
 * text: the sequences' characters back to back; offsets [nseq+1]: where each starts
 * (a prefix sum of the lengths; offsets[0] need not be 0).  Writes
 *     X = pad | s0 | pad | s1 | ... | pad      (pad bytes of 255; A,C,G,T/U -> 0..3,
 *                                               either case; anything else -> 255)
 * of db_batch_bytes(...) bytes and regions [nrow,2] = (start of the row's leading
 * pad, end of its sequence).  reverse_complement != 0 doubles the rows: row 2b is
 * sequence b, row 2b+1 its reverse complement.  All pointers are device pointers. */
size_t db_batch_bytes(uint32_t nseq, size_t total_len, uint32_t pad, int reverse_complement);
void db_build_batch(const uint8_t* text, const uint32_t* offsets, uint32_t nseq, uint32_t pad,
                    int reverse_complement, uint8_t* X, uint32_t* regions);
/* Scan mode of kangaroo.predict (predict.py:270-285): each sequence, padded with
 * windowsize-1 'N' on both sides, is cut into windows of `windowsize` characters
 * every `stride` positions, and each window becomes a row of the batch (same layout
 * as db_build_batch; every row is pad + windowsize bytes).  Sequence b has
 * ceil(max(1, len_b + windowsize - 1) / stride) windows; window_offsets [nseq+1] is
 * the prefix sum of these counts and nwindow its last entry.  X needs
 * db_batch_bytes(nwindow, nwindow * windowsize, pad, reverse_complement) bytes. */
void db_build_windows(const uint8_t* text, const uint32_t* offsets, const uint32_t* window_offsets,
                      uint32_t nseq, uint32_t nwindow, uint32_t windowsize, uint32_t stride, uint32_t pad,
                      int reverse_complement, uint8_t* X, uint32_t* regions);

/* ---- fused hot path (no counterpart as one call; replaces the chain
 * api_corr1ord -> bias -> rectify -> api_poolrgn of corr1ord.py:97-102,
 * elemwise.py:171,74-78, poolrgn.py:59,153) --------------------------------
 * W [4m, nf] f32, bias [nf] (nullable), X [npos] u8, regions u32 [nregion,2],
 * pooled [nregion, nf] (max/avg/sum) or [nregion, 2nf] (all, interleaved),
 * argmax u32 [nregion, nf] (nullable; flat index row*nf+f as api_poolrgn),
 * actmask (nullable) u16 [npos, ceil(nf/16)]: bit f%16 of word f/16 of row i is
 * set iff the rectified activation is > 0 (what the backward pass needs instead
 * of Z).  Regions may lie anywhere in X; the backward pass needs them disjoint. */
void db_scanpool_fwd(const float* W, uint32_t m, uint32_t nf, const float* bias, int relu,
                     const uint8_t* X, uint32_t npos, const uint32_t* regions, uint32_t nregion,
                     int ptype, float* pooled, uint32_t* argmax, uint16_t* actmask);
/* Fused backward of the same chain: given dpooled (layout of pooled), argmax and
 * actmask from the forward call, accumulates dW [4m,nf] and dbias [nf] (both
 * overwritten, not accumulated) with a fixed summation order. */
void db_scanpool_bwd(uint32_t m, uint32_t nf, const uint8_t* X, uint32_t npos,
                     const uint32_t* regions, uint32_t nregion, int ptype,
                     const float* dpooled, const uint32_t* argmax, const uint16_t* actmask,
                     float* dW, float* dbias);

/* ---- many-model scan on tcgen05 tensor cores (no counterpart: replaces `nf/16`
 * passes of kangaroo.predict over the same sequences, predict.py:394-420, and
 * deepity's instance batching, hypertrain.py:576) ---------------------------
 * The scan is the dense contraction Z[f,p] = sum_k W[k,f] * onehot(X)[p,k], K = 4m.
 * Weights are prepared once per weight set into 16-bit operand tiles; `precision`
 * (enum db_tc_precision) picks the operand type and the pieces per weight, all
 * accumulated in FP32 (the one-hot operand is exact in either type):
 *   DB_TC_BF16 / _BF16X2 / _BF16X3: 1-3 bf16 pieces, 8/16/24 significant bits; max
 *       error about 2e-3 / 1e-5 / 1e-6 of the largest activation;
 *   DB_TC_F16 / _F16X2: 1-2 f16 pieces (11/22 bits) of the weights prescaled by a
 *       power of two (undone in the kernel, exactly): about 3e-4 / 1e-6, at the
 *       tensor-core cost of one / two bf16 pieces.
 * Pooled values follow
 * db_scanpool_fwd's layout; argmax is not produced (use the FP32 path to train).
 * If `scores` is given, each model's linear head (16 filters per model; headW
 * [(16|32)*nmodel] in the row order of full.W, headB [nmodel]) is applied in the
 * kernel and scores [nregion, nmodel] is written; `pooled` may then be NULL.
 * Regions (8-byte aligned table) must ascend without overlap (the batch layout of
 * data.py:329-334); rows between regions are scanned and discarded.  status: device
 * int the caller zeroes; 0 = ok, 1 = a device-side wait timed out, 3 = regions out
 * of order, 4 = the prepared filter bank held an Inf or NaN weight (nothing is written). */
enum db_tc_precision { DB_TC_BF16 = 1, DB_TC_BF16X2 = 2, DB_TC_BF16X3 = 3, DB_TC_F16X2 = 4, DB_TC_F16 = 5 };
size_t db_tc_weights_bytes(uint32_t m, uint32_t nf, int precision);
void db_tc_prepare(const float* W, uint32_t m, uint32_t nf, int precision, void* prepared);
void db_scanpool_tc(const void* prepared, uint32_t m, uint32_t nf, int precision, const float* bias, int relu,
                    const uint8_t* X, uint32_t npos, const uint32_t* regions, uint32_t nregion, int ptype,
                    float* pooled, const float* headW, const float* headB, uint32_t nmodel, float* scores,
                    int* status);
/* Multi-GPU scan (no counterpart: the reference gathers per-device results on the host,
 * kangaroo/predict.py:484-492).  For later db_scanpool_tc launches of the calling thread that
 * produce scores, every score is also stored into each of the `npeer` (<= 8) matrices
 * peer_scores[p] ([rows, nmodel] f32, device memory of this or of a peer GPU mapped into this
 * process), at row row_offset + region index: the all-gather of the ranks' score shards done
 * by the scan kernel itself with plain peer stores over NVLink.  The ranks must synchronise
 * (e.g. a barrier collective on the same stream) after their launches and before reading.
 * npeer = 0 switches it off. */
void db_scanpool_tc_peers(float* const* peer_scores, uint32_t npeer, uint32_t row_offset);
/* Test aid (no counterpart): for later db_scanpool_tc launches of the calling thread,
 * the deadline of the kernel's internal waits in clock cycles (0 = default, about 0.1 s)
 * and, with hold_operands != 0, operand encoders that never signal "stage ready", so
 * that the first wait of the MMA issuer runs out with nothing in flight.  The launch
 * then reports status 1 and returns; nothing faults.  Call with (0, 0) to restore. */
void db_scanpool_tc_debug(uint64_t timeout_clocks, int hold_operands);

#ifdef __cplusplus
}
#endif
#endif /* DEEPBIND_B200_H */
