/* tsa.h - C ABI of the B200 (sm_100a) quantized attention path.
 *
 * Drop-in boundary for TScale's attention kernels: each entry point enqueues work on a CUDA stream
 * and takes the same kind of arguments the reference passes to its own kernels through
 * CudaCall(...) (code/gpt/compute/gpt_cuda.cu:503-515,747-751,796-845): caller-owned 2-D device
 * buffers with a byte stride, per-head scale planes indexed [head][row], grouped span lists for
 * the mask, the ALiBi slope, and a sumWeightLog side output.  Nothing here allocates device
 * memory; scratch is passed in by the caller (tsa_*_workspace_bytes gives the size).
 *
 * Every function returns a tsa_status and never aborts.  Device-side problems (a bounded wait
 * that ran out) are reported through the optional int *statusWord in device memory: the kernels
 * OR a non-zero code into it and return normally.
 *
 * Naming follows the reference (code/gpt/model_params/model_params.h:8-12):
 *   qk = query vectors ("attention current token"), qv = key vectors ("attention remote"),
 *   v = value vectors, out = ValLookup, sumWeightLog = log2-sum-exp including the implicit sink.
 */
#ifndef TSA_H
#define TSA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *tsa_stream_t; /* == cudaStream_t */

enum tsa_status {
    TSA_OK = 0,
    TSA_BAD_ARG = 1,
    TSA_UNSUPPORTED = 2,
    TSA_CUDA_ERROR = 3,
    TSA_TIMEOUT = 4
};

enum tsa_dtype {
    TSA_I8 = 0,   /* int8 (reference type i8) */
    TSA_E4M3 = 1, /* fp8 e4m3 (reference type e4m3, code/util/fp8.h:122-139) */
    TSA_F16 = 2,
    TSA_BF16 = 3,
    TSA_F32 = 4
};

/* Mirrors TCuda2DPtr<T> (code/lib/cuda/cuda_arrays.h:203-237): row y starts at data + y * stride_bytes.
 * xsize / ysize are the extents in elements / rows and are used for argument validation and as the
 * bounds of TMA tensor maps; data == NULL means "argument not given" where the entry point allows it. */
typedef struct {
    void *data;
    int stride_bytes;
    int xsize;
    int ysize;
} tsa_ptr2d;

/* Mirrors TAttentionSpanGroup<64> (code/gpt/att/att.h:56-64): one record per 64-row query block and
 * round; Start/Finish are 128-aligned key-block bounds, SpanStart/SpanFinish the inclusive key span
 * of each of the 64 rows (unused rows: SpanStart = 1e9, SpanFinish = 1e9 - 1). */
#define TSA_ATT_GROUP 64
#define TSA_ATT_ALIGN 128
typedef struct {
    int Start;
    int Finish;
    int SpanStart[TSA_ATT_GROUP];
    int SpanFinish[TSA_ATT_GROUP];
} tsa_span_group;

/* Replaces the compile-time switches of code/gpt/compute/cfg_precision.h:9-12,46-58 (ATT_TYPE,
 * TAttVecFloat) and the constants of gpt_cuda.cu:40-45 (QK_VEC_SCALE, V_VEC_SCALE). */
typedef struct {
    int qk_dtype;       /* TSA_I8 or TSA_E4M3: type of qk and qv */
    int v_dtype;        /* TSA_I8 or TSA_E4M3 */
    int out_dtype;      /* TSA_F16, TSA_BF16 or TSA_F32: type of out (forward) */
    int grad_dtype;     /* TSA_F16, TSA_BF16 or TSA_F32: type of dOut, dQK, dQV, dV (backward) */
    int head_dim_qk;    /* Q_DIM */
    int head_dim_v;     /* TT_DIM */
    float qk_vec_scale; /* query scale used when qkScale is not given (QK_VEC_SCALE) */
    float v_vec_scale;  /* value scale used when vScale is not given; 1 returns "stored-V units" like Fp8Att */
    int flags;          /* TSA_FLAG_* */
} tsa_att_cfg;

#define TSA_FLAG_FORCE_GENERIC 1 /* use the SIMT kernels that accept any mask and head size */

const char *tsa_version(void);
/* text of the last error raised on the calling thread ("" if none) */
const char *tsa_last_error(void);

/* ---- forward ---------------------------------------------------------------------------------
 * Replaces Fp8Att (code/gpt/compute/gpt_att_fp8.cuh:43-46) and Fp16Att (gpt_att_fp16.cuh:121-127).
 *   qk, qv        [len][H*Dqk] 8-bit;   qkScale, qvScale  f32 [H][len] (qkScale may be absent)
 *   v             [len][H*Dv] 8-bit, NOT transposed;  vScale f32 [H][len] (may be absent)
 *   attSpans / attSpanPtr: grouped spans of lenAttTiles 64-row blocks, device memory (gpt_cuda.cu:362-363)
 *   out           [len][H*Dv] of cfg->out_dtype; sumWeightLog f32 [H][len] (may be absent)
 * logit(i,j) = dot(qk_i, qv_j) * qkScale_i * qvScale_j * sqrt(1/Dqk) * 0.5/0.693147 * (*qvGlobalScale)
 *              - alibiSlope * (i - j);  softmax base 2 with an extra logit-0 / value-0 sink;
 * rows without keys give 0.  qvGlobalScale: device scalar, NULL = 1.
 * Range of vScale on the tensor-core path: a weight is multiplied by vScale[key] / (the power of two at or above the head's
 * largest vScale over all key rows of the call) before it is rounded to e4m3, so the row's result keeps its precision while
 * the keys that carry its weight have value scales within a factor of 64 of that maximum (e4m3's normal range below 1), and
 * loses it gradually beyond (per-row abs-max scales of normalised vectors are within a small factor of each other; the
 * reference's kernel uses one constant value scale).  TSA_FLAG_FORCE_GENERIC keeps fp32 weights and has no such limit. */
int tsa_att_fwd(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, tsa_ptr2d sumWeightLog, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream);
/* workspace: tsa_att_fwd_workspace_bytes(...) bytes of 16-byte aligned device memory (per-head maxima of the vScale
 * plane and the work-item counter of the persistent kernel); the call clears what it uses. */
size_t tsa_att_fwd_workspace_bytes(const tsa_att_cfg *cfg, int headCount, int len);

/* Forward with the all-gather of its output fused in: the kernel stores every output row to outs[0] and to the outCount - 1
 * further matrices outs[1..] of the same shape, dtype and column offset, which may be the buffers of OTHER GPUs of the box
 * mapped into this process (CUDA peer access / IPC / symmetric memory over NVLink): each rank of a (fragment x head)-sharded
 * batch writes its block straight into every rank's copy of the whole output from the attention epilogue, so that no
 * separate collective has to move it afterwards (the reference gathers by copying device arrays between its per-device
 * contexts, code/gpt/compute/gpt_cuda.cu:1478-1738).  Plain 16- or 32-byte stores; no multicast.  One further destination
 * is stored by the thread that owns the row; two or more are served by a forwarding warp that re-reads finished rows from
 * L2 (e4m3 values only).  The callers order the
 * step themselves (a stream-ordered barrier across the ranks before anybody reads a gathered buffer).  Everything else as
 * tsa_att_fwd; outCount = 1 is tsa_att_fwd.  At most TSA_MAX_OUT_COPIES + 1 destinations; only the tensor-core path
 * takes more than one (TSA_UNSUPPORTED otherwise). */
#define TSA_MAX_OUT_COPIES 7
int tsa_att_fwd_to(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    const tsa_ptr2d *outs, int outCount, tsa_ptr2d sumWeightLog, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream);

/* One rank's part of an all-gather over peer memory, as a small kernel of the library: rows [0, rows) x rowBytes of src
 * (this rank's block) are copied to each of the dstCount destinations (the same block inside the other GPUs' buffers,
 * mapped into this process: peer access / IPC / symmetric memory).  Its CTAs (`ctas` of them, 0 = one per SM; 256 threads,
 * no shared memory) fit beside the attention kernel's, so that on a side stream the copy of one head slice runs under the
 * attention of the next; plain 32-byte loads and stores over NVLink, no multicast.  All rows 32-byte aligned. */
int tsa_peer_scatter(tsa_ptr2d src, const tsa_ptr2d *dsts, int dstCount, int rows, int rowBytes, int ctas, tsa_stream_t stream);

/* Forward for vectors that live in page-locked HOST memory.  Same arguments and results as tsa_att_fwd, except that qk,
 * qv, qkScale, qvScale, v, vScale, out and sumWeightLog point to host memory (cudaHostAlloc / cudaHostRegister; pageable
 * memory works but its copies do not overlap anything) while attSpans, attSpanPtr, qvGlobalScale and statusWord stay
 * device memory.  The heads are cut into `slices` groups of ceil(H / slices) heads; the head columns of slice s+1 are
 * copied in, slice s is computed and the output columns of slice s-1 are copied out at the same time, on three streams
 * the library keeps per device, ordered behind everything queued on `stream` before the call; `stream` continues when
 * the last output copy has landed, so the caller synchronises `stream` (or an event recorded on it) before reading out.
 * The reference moves whole arrays with TCuda2DArray::CopyToDevice / CopyToHost on its compute stream
 * (code/lib/cuda/cuda_arrays.h:353-369), copy - compute - copy in sequence; this entry overlaps the three.
 * outDevice (may be absent): device matrix [len][H*Dv] of cfg->out_dtype that also keeps the result, for a caller that
 * goes on with it on the GPU (an all-gather across ranks, the next layer); the host copy is made from it.
 * staging: tsa_att_fwd_host_staging_bytes(cfg, H, len, slices) bytes of 256-byte aligned device memory (two sets of one
 * slice's inputs, outputs and forward workspace).  One call at a time per device enqueues (the library serialises
 * callers); two calls on different streams that share a staging area are the caller's to order. */
int tsa_att_fwd_host(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, tsa_ptr2d sumWeightLog, tsa_ptr2d outDevice, int headCount, int lenAttTiles, int slices,
    void *staging, size_t stagingBytes, int *statusWord, tsa_stream_t stream);
size_t tsa_att_fwd_host_staging_bytes(const tsa_att_cfg *cfg, int headCount, int len, int slices);

/* ---- backward --------------------------------------------------------------------------------
 * Replaces Fp8AttGradQK + Fp8AttGradQV (gpt_att_fp8.cuh:277-284, 599-606) and Fp16AttGradQK/QV
 * (gpt_att_fp16.cuh:332, 459).  Additional inputs: dOut [len][H*Dv] of cfg->grad_dtype, out (forward
 * result, used when dScale is absent), dScale f32 [H][len] = sum_x dOut*out (absent: computed into the
 * workspace), sumWeightLog from the forward, revAttSpans / revAttSpanPtr = grouped spans of the
 * transposed mask (gpt_cuda.cu:812).  Outputs dQK, dQV [len][H*Dqk], dV [len][H*Dv] of
 * cfg->grad_dtype: gradients with respect to the true-scale (dequantised) vectors, times attGradMult
 * (the rope / normalise back-propagation of the reference epilogues is not part of this entry). */
int tsa_att_bwd(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    tsa_ptr2d dOut, tsa_ptr2d out, tsa_ptr2d dScale, tsa_ptr2d sumWeightLog,
    const tsa_span_group *attSpans, const int *attSpanPtr,
    const tsa_span_group *revAttSpans, const int *revAttSpanPtr,
    float alibiSlope, float attGradMult,
    tsa_ptr2d dQK, tsa_ptr2d dQV, tsa_ptr2d dV, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream);
size_t tsa_att_bwd_workspace_bytes(const tsa_att_cfg *cfg, int headCount, int len);

/* dScale[head][t] = sum_x out[t][head*Dv + x] * dOut[t][head*Dv + x].
 * Replaces CalcDScale (gpt_att_fp16.cuh:621-643) and the dScale part of KVProductBackpropE4fused
 * (gpt_combiner.cuh:184-217).  outDtype / gradDtype: TSA_F16, TSA_BF16 or TSA_F32. */
int tsa_calc_dscale(int outDtype, int gradDtype, tsa_ptr2d out, tsa_ptr2d dOut, tsa_ptr2d dScale,
    int headCount, int headDimV, int len, tsa_stream_t stream);

/* raw integer scores S[head][i][j] = sum_x qk[i][x] * qv[j][x] for i < lenQ, j < lenK, computed by the
 * same tcgen05 kind::i8 tile path the int8 forward uses (int32 [H][lenQ][lenK], dense).  Parity hook
 * for the exactness of the integer QK^T accumulators (s8 -> s32 tiles of gpt_att_fp16.cuh:76-101). */
int tsa_qk_scores_i32(tsa_ptr2d qk, tsa_ptr2d qv, int headCount, int headDim, int lenQ, int lenK,
    int32_t *scores, int *statusWord, tsa_stream_t stream);

/* Parity hook of the int8 forward itself: the next tsa_att_fwd calls with qk_dtype TSA_I8 on the tensor-core path
 * also store, for query tile `queryTile` (128 rows) of head `head`, the raw s32 accumulators of its `keyTile`-th
 * key tile exactly as the softmax threads read them from tensor memory, into dst (device memory, int32 [128][128],
 * row = query row inside the tile).  dst == NULL switches the dump off.  Process-wide setting, meant for tests; it
 * checks the bit-exactness of the s8 x s8 -> s32 products (gpt_att_fp16.cuh:76-101) inside the forward's own pipeline
 * (ring slots, barrier phases) rather than in tsa_qk_scores_i32's separate kernel. */
int tsa_att_fwd_set_score_dump(int32_t *dst, int head, int queryTile, int keyTile);

/* ---- status word and failure-path self-tests --------------------------------------------------------------------
 * The reference aborts the process on any CUDA error (code/lib/cuda/cuda_graph.cuh:147-150); here a kernel that gives up
 * ORs a code into the caller's status word and returns.  tsa_status_from_word maps a word read back from the device to a
 * tsa_status: 0 -> TSA_OK, a timed-out barrier wait (0x10 copy, 0x20 MMA) -> TSA_TIMEOUT, anything else -> TSA_BAD_ARG.
 * The two self-tests make a wait run out on purpose, without faulting or hanging anything:
 * tsa_selftest_bounded_wait launches one thread that waits, for at most limitCycles clock cycles, on a barrier nobody
 * arrives on, and must come back with 0x10 in *statusWord; tsa_selftest_fwd_withhold_copy makes the following
 * tsa_att_fwd calls (tensor-core path) wait at most waitCycles cycles per barrier and leave out the copy of every CTA's
 * withholdTile-th key tile, so the forward must notice, drain its other copies, free its tensor memory and return with
 * the time-out bits set (waitCycles = 0, withholdTile = -1 restores production behaviour).  Process-wide, for tests. */
int tsa_status_from_word(int statusWord);
int tsa_selftest_bounded_wait(long long limitCycles, int *statusWord, tsa_stream_t stream);
int tsa_selftest_fwd_withhold_copy(long long waitCycles, int withholdTile);

/* Bounds-check build (make -C tscale_b200/csrc bounds -> libtsa_b200_bounds.so, tests only): every row lookup the kernels make
 * through a tsa_ptr2d is checked against its ysize; a lookup outside is counted and redirected to row 0 instead of touching
 * memory outside the buffer (the reference has no counterpart: an index past a TCuda2DPtr goes unnoticed or ends in
 * cudaErrorIllegalAddress and the abort of code/lib/cuda/cuda_graph.cuh:147-150).  tsa_bounds_check_hits synchronises the
 * device and returns the count since the last reset (reset != 0 clears it), -1 in a production build.
 * tsa_selftest_bounds_check makes one out-of-range lookup on purpose on a one-row f32 plane (plane, sink: device memory,
 * one float each) and returns the number caught (1), -1 in a production build. */
int tsa_bounds_check_hits(int reset);
int tsa_selftest_bounds_check(float *plane, float *sink);

/* ---- per-row quantisers ----------------------------------------------------------------------
 * Replaces NormalizeVecsRowTile / NormalizeVecsRowTileMax (code/gpt/compute/row_tile_scale.cuh:11-34,
 * 59-82) and the stand-alone use of the TStoreRowTileNormalize epilogue (lib/cuda/cuda_matmul.cuh:147-204).
 * Per row and per tile of `tile` elements: TSA_QUANT_RMS: scale = sqrt(mean(x^2)) * vecScale;
 * TSA_QUANT_ABSMAX: scale = max|x| / 127 (i8) or / 256 (e4m3); dst = sat_rne(x / scale);
 * scale plane f32 [xsize/tile][len]; all-zero tiles give scale 0 and zeros.  Rows in [len, dst.ysize)
 * are written with zeros like the reference's padding rows.  srcDtype: TSA_F32, TSA_F16 or TSA_BF16. */
enum tsa_quant_kind { TSA_QUANT_RMS = 0, TSA_QUANT_ABSMAX = 1 };
int tsa_quant_rows(int kind, int srcDtype, int dstDtype, float vecScale, tsa_ptr2d src, tsa_ptr2d dst,
    tsa_ptr2d scale, int len, int tile, tsa_stream_t stream);

/* ---- producer of the attention inputs ("next" scope row: the step on the input side of the path) ------------
 * Replaces the TStoreRowTileNormalizeRope epilogue of the QKV projection used stand-alone (code/gpt/compute/
 * gpt_rope.cuh:4-66: normalise, rope, store, write the scale) and, with rope absent, TStoreRowTileNormalize
 * (lib/cuda/cuda_matmul.cuh:147-204).  Per row and head: scale = sqrt(mean(x^2)) * vecScale, y = x / scale, then
 * the rope rotation as the CPU model defines it (code/gpt/att/rope.cpp:28-46: inside every 64-element block elements
 * k and k + 32 rotate by the angle whose cosine is rope[row][block + k] and sine rope[row][block + k + 32] * ropeDir;
 * ropeDir = -1 rotates back), then dst = sat_rne(y) as i8 or e4m3 and scale plane f32 [H][len].  rope: table
 * [>= len][headDim] of f32 or f16 (the reference's TRopeFloat), absent = no rotation.  Rows in [len, dst.ysize) are
 * zeroed.  srcDtype: TSA_F32, TSA_F16 or TSA_BF16; headDim 64, 128, 256 or 512. */
int tsa_norm_rope_quant(int srcDtype, int dstDtype, float vecScale, tsa_ptr2d src, tsa_ptr2d rope, int ropeDtype,
    float ropeDir, tsa_ptr2d dst, tsa_ptr2d scale, int headCount, int headDim, int len, tsa_stream_t stream);

/* Back-propagation through tsa_norm_rope_quant's fp32 stage.  Replaces the inverse rope and the RMS-normalise
 * gradient folded into the epilogues of the reference's backward kernels (gpt_att_fp8.cuh:527-566, 917-981) and
 * ApplyRope(-1) + NormalizeStateBackward of the CPU model (gpt_cpu.cpp:329-360, 759-764).  grad [len][H*D]: gradient
 * with respect to the roped unit-RMS vector (what tsa_att_bwd returns, divided by the vector scale); src: the raw
 * projection the producer normalised; out (dtype of grad) = sqrt(D / sum2) * (g - src * dot(src, g) / sum2) per head,
 * g = grad rotated by -ropeDir; all-zero heads give zeros.  Supported (src, grad) dtypes: (f32, f32), (bf16, bf16),
 * (f16, f16), (f32, bf16), (bf16, f32). */
int tsa_rope_norm_bwd(int srcDtype, int gradDtype, tsa_ptr2d src, tsa_ptr2d grad, tsa_ptr2d rope, int ropeDtype,
    float ropeDir, tsa_ptr2d out, int headCount, int headDim, int len, tsa_stream_t stream);

/* ---- consumer of the attention output ("next" scope row: the step on the output side of the path) -------------
 * Replaces KVProduct and KVProductBackprop (code/gpt/compute/gpt_combiner.cuh:12-39, 85-217; CPU form
 * gpt_cpu.cpp:191-262): the input of the combiner matrix
 *   kv[t][head * 4 D + blk * D + z] = k[t][head * D + (z ^ blk)] * valLookup[t][head * D + z] * kvMult,  blk = 0 .. 3,
 * and its back-propagation dK[z] = sum_blk dkv[blk][z ^ blk] * val[z ^ blk], dValLookup[z] = sum_blk dkv[blk][z] *
 * k[z ^ blk], plus dScale[head][t] = sum_z dValLookup[z] * valLookup[z] (f32 plane [H][len], may be absent), which is
 * the dScale argument of tsa_att_bwd (the reference's KVProductBackpropE4fused computes it in the same pass).
 * Dtypes (in, out): (f32, f32), (bf16, bf16), (f16, f16), (bf16, f32), (f16, f32); backward (in, grad): the first
 * three and (bf16, f32).  Head size 64, 128 or 256; all buffers 16-byte aligned. */
int tsa_kv_product(int inDtype, int outDtype, tsa_ptr2d k, tsa_ptr2d valLookup, float kvMult, tsa_ptr2d kv,
    int headCount, int headDim, int len, tsa_stream_t stream);
int tsa_kv_product_bwd(int inDtype, int gradDtype, tsa_ptr2d k, tsa_ptr2d valLookup, tsa_ptr2d dkv, tsa_ptr2d dK,
    tsa_ptr2d dValLookup, tsa_ptr2d dScale, int headCount, int headDim, int len, tsa_stream_t stream);

/* tsa_att_fwd with the consumer fused into the kernel (the reference launches KVProduct right behind the attention,
 * code/gpt/compute/gpt_cuda.cu:520-523): besides out and sumWeightLog the call writes
 *   kv[t][head * 4 D + blk * D + z] = combinerK[t][head * D + (z ^ blk)] * out[t][head * D + z] * kvMult,  blk = 0 .. 3,
 * bit for bit what tsa_kv_product(bf16, bf16) gives on the stored output.  The thread that rounds a row of the output to
 * bf16 multiplies it with the row of combiner keys (prefetched into L2 while the block is computed) and stores the four
 * products with streaming 32-byte stores, so the stand-alone kernel's launch and its re-read of the output go away.
 * Measured on B200 the two calls it replaces are as fast or faster (the forward is bound by the instruction issue of
 * the threads that would do this work, the stand-alone product by memory bandwidth, which it reaches): prefer them
 * where speed decides.  combinerK bf16 [>= len][>= H*D], kv bf16 [>= len][>= 4*H*D],
 * both 16-byte aligned; out dtype bf16, e4m3 values, head size 64 or 128 (otherwise TSA_UNSUPPORTED: call tsa_att_fwd
 * and tsa_kv_product). */
int tsa_att_fwd_kv(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, tsa_ptr2d sumWeightLog, tsa_ptr2d combinerK, float kvMult, tsa_ptr2d kv, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream);

/* ---- KV-cache decode -------------------------------------------------------------------------
 * Replaces NCPUInfer::TAttentionVecHistory / ComputeValLookup (code/gpt/train/cpu_infer.cpp:397-460),
 * batched over sequences.  Per sequence the cache is caller-owned device memory:
 *   k, v    int8 [capacity][H*D] (row stride H*D bytes, base 16-byte aligned, H*D a multiple of 16);
 *   kScale, vScale scaleDtype [capacity][H].
 * tsa_kv_append writes each sequence's new token at row ctxLens[s] and then increments ctxLens[s]
 * (AddVectors, cpu_infer.cpp:403-408).  tsa_att_decode then attends, like the reference, to the keys
 * [cur - window, cur - 1] with cur = ctxLens[s] - 1 (window 0: the new token itself); logits use the exact
 * int32 dot, an extra logit-0 sink, and out = sum softmax * vScale * v. */
typedef struct {
    void *k;
    void *v;
    void *kScale;
    void *vScale;
} tsa_kv_seq;

typedef struct {
    int head_dim;       /* 64 or 128 */
    int scale_dtype;    /* TSA_F16 or TSA_F32: type of kScale / vScale planes */
    int out_dtype;      /* TSA_F32, TSA_F16 or TSA_BF16 */
    float qk_vec_scale; /* query scale when qScale is absent (VEC_SCALE of cpu_infer.cpp:16) */
} tsa_decode_cfg;

int tsa_kv_append(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, int *ctxLens, int nSeq, int capacity,
    tsa_ptr2d kNew, tsa_ptr2d kScaleNew, tsa_ptr2d vNew, tsa_ptr2d vScaleNew, int headCount,
    int *statusWord, tsa_stream_t stream);
/* q int8 [nSeq][H*D]; qScale f32 [nSeq][H] (may be absent); out [nSeq][H*D].  maxCtx: host-side upper
 * bound of ctxLens; it sizes the launch (short windows and contexts get a smaller grid), and a sequence that
 * turns out longer sets a bit in the status word instead of being attended in part.  seqs and ctxLens are
 * device arrays. */
int tsa_att_decode(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, const int *ctxLens, int nSeq, int maxCtx,
    tsa_ptr2d q, tsa_ptr2d qScale, int window, float alibiSlope, tsa_ptr2d out, int headCount,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream);
size_t tsa_att_decode_workspace_bytes(const tsa_decode_cfg *cfg, int nSeq, int headCount, int maxCtx);

/* Same decode step for callers that cannot give the library a scratch buffer.  It has no counterpart in the
 * reference.  Meant for hosts that fix all device memory when they start and never allocate again: a runtime
 * built like TScale's, which hands out buffers from pools sized at context creation and then only replays
 * kernel launches, or a server whose memory budget is fully committed to its caches, where a cudaMalloc in
 * the token loop would fail or stall the GPU.  The per-chunk partial results live in a fixed 32 MiB array in
 * the library image instead of a workspace argument; every GPU that loads the library holds that array until
 * the process ends.  The call allocates nothing and returns TSA_UNSUPPORTED, with a message, when
 * tsa_att_decode_workspace_bytes(cfg, nSeq, headCount, maxCtx) exceeds tsa_att_decode_static_capacity_bytes().
 * The first call on each device looks up the array's device address (a one-time set-up step on the host);
 * make that first call outside any stream capture.  All calls on a device share the one array and it keeps
 * whatever the previous call left there (each call overwrites every slot it later reads, so nothing has to be
 * cleared); two such calls that overlap in time on the same GPU, e.g. on different streams, race on it.  The
 * address found by the first call is kept for the life of the process, so do not call this entry point again on a
 * device after a cudaDeviceReset. */
int tsa_att_decode_static(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, const int *ctxLens, int nSeq, int maxCtx,
    tsa_ptr2d q, tsa_ptr2d qScale, int window, float alibiSlope, tsa_ptr2d out, int headCount,
    int *statusWord, tsa_stream_t stream);
size_t tsa_att_decode_static_capacity_bytes(void);

/* ---- host-side span preprocessing (CPU) ------------------------------------------------------
 * tsa_make_window_spans: causal window mask of AddAttSpans (code/gpt/att/sliding_window.cpp:80-87):
 *   row i of a fragment starting at f0 attends [max(f0, i - window), i - 1]; window <= 0: whole prefix.
 *   spans: (start, finish) int pairs, spanPtr: len + 1 offsets.  Returns the span count, or -(needed) if
 *   maxSpans is too small.
 * tsa_transpose_attention: TransposeAttention (code/gpt/att/att.cpp:26-56).
 * tsa_group_attention: GroupAttention<64,128> (code/gpt/att/att.h:95-181); groupPtr has ceil(len/64)+1 entries.
 * tsa_group_window_spans: closed form of the two above for window masks: writes grouped spans of the mask
 *   (transposed = 0) or of its transpose (transposed = 1) without enumerating pairs. */
int tsa_make_window_spans(int fragCount, const int *fragLens, int window, int maxSpans, int *spans, int *spanPtr);
int tsa_transpose_attention(int len, const int *spans, const int *spanPtr, int maxSpans, int *resSpans, int *resSpanPtr);
int tsa_group_attention(int len, const int *spans, const int *spanPtr, int maxGroups, tsa_span_group *groups, int *groupPtr);
int tsa_group_window_spans(int fragCount, const int *fragLens, int window, int transposed, int maxGroups,
    tsa_span_group *groups, int *groupPtr);

/* ---- partition over the GPUs of one box ---------------------------------------------------------------------
 * Replaces the per-device batch split of TMultiComputeContext (code/gpt/compute/gpt_cuda.cu:1478-1738; the split itself
 * code/gpt/train_ctx/backprop.cpp:10-23), at the granularity the attention path allows: one unit = one (fragment, head)
 * pair, unit = fragment * heads + head.  tsa_shard_range gives rank `rank` of `world` its contiguous, balanced block
 * [begin, end) of `units` (earlier ranks take the remainder).  tsa_shard_rects writes that block as at most three
 * rectangles of whole fragments x a head range; each rectangle is one tsa_att_fwd / tsa_att_bwd call on the
 * rectangle's rows, with qk / qv / v / out advanced by head_begin * D columns and the scale planes by head_begin rows.
 * No input crosses GPUs; the outputs are gathered with one NCCL all-gather per call (INTEGRATION.md shows the
 * per-rank call sequence).  Host functions; tsa_shard_rects returns the rectangle count or a negative tsa_status. */
typedef struct {
    int frag_begin, frag_end; /* fragments [frag_begin, frag_end) */
    int head_begin, head_end; /* heads [head_begin, head_end) */
} tsa_shard_rect;
int tsa_shard_range(int units, int world, int rank, int *begin, int *end);
int tsa_shard_rects(int begin, int end, int heads, tsa_shard_rect *rects);

/* ---- device-side span generation ("next" scope row: the mask preparation on the input side of the path) -------
 * The same records as tsa_group_window_spans, written by a kernel into device memory: no host work and no copy of the
 * mask per step (the reference prepares the spans on the CPU and uploads them, gpt_cuda.cu:1346-1353).
 * fragStarts: device array of fragCount + 1 ascending row offsets (fragStarts[0] = 0, fragStarts[fragCount] = len).
 * groups needs room for ceil(len / 64) records (maxGroups), groupPtr for ceil(len / 64) + 1 ints; the number of
 * groups ends up in groupPtr[ceil(len / 64)]. */
int tsa_group_window_spans_device(const int *fragStarts, int fragCount, int len, int window, int transposed,
    int maxGroups, tsa_span_group *groups, int *groupPtr, tsa_stream_t stream);

/* Device-side tsa_transpose_attention / tsa_group_attention for ARBITRARY span lists that already live in device memory
 * (TransposeAttention code/gpt/att/att.cpp:26-56, GroupAttention<64,128> code/gpt/att/att.h:95-181; the reference runs both on
 * the host for every batch, gpt_cuda.cu:1346-1353).  spans / spanPtr: device CSR of inclusive (start, finish) pairs per row,
 * every row's spans sorted by start and disjoint (what AddAttSpans produces).  Results are bit-identical to the host helpers.
 * The sizes are data: count (device, int[2]) receives the number of spans / groups and a flag that is set when the caller's
 * arrays (maxSpans / maxGroups entries) are too small, in which case only resSpanPtr / groupPtr are written.
 * maxInputSpans: upper bound of spanPtr[len] (sizes the workspace).  Typical use for the backward's transposed mask:
 * transpose, then group the result (the transposed CSR is sorted and disjoint by construction). */
int tsa_transpose_attention_device(int len, const int *spans, const int *spanPtr, int maxInputSpans,
    int maxSpans, int *resSpans, int *resSpanPtr, int *count, void *workspace, size_t workspaceBytes, tsa_stream_t stream);
size_t tsa_transpose_attention_device_workspace_bytes(int len, int maxInputSpans);
int tsa_group_attention_device(int len, const int *spans, const int *spanPtr, int maxGroups,
    tsa_span_group *groups, int *groupPtr, int *count, void *workspace, size_t workspaceBytes, tsa_stream_t stream);
size_t tsa_group_attention_device_workspace_bytes(int len);

/* ---- projection fused with the producer ("next" scope row: the GEMM epilogue in front of the path) ------------
 * Replaces MulForwardInt8 / MulForwardFp8 <TStoreRowTileNormalizeRope> and <TStoreRowTileNormalize>
 * (code/gpt/compute/gpt_cuda.cu:488-496; store ops code/lib/cuda/cuda_matmul.cuh:147-204; rope code/gpt/compute/gpt_rope.cuh:4-66):
 *   y[t][n] = (float)(int32 dot of x[t] and w[n]) * srcScale,   x int8 [len][dim], w int8 [H*D][dim] (dim % 64 == 0);
 *   srcDtype TSA_E4M3: x and w hold e4m3 bytes and the dot is accumulated in f32 by the tensor cores
 *   per head: discr = sqrt(sum y^2 / D) * vecScale; dst = quantise(rope(y / discr)); scale[head][t] = discr
 * i.e. tsa_norm_rope_quant applied to the projection without the projection ever going to memory.  rope: f32
 * [len][D] table or absent (the K and V projections are stored without rotation).  dst int8 or e4m3 [rows][H*D],
 * or f16 / bf16 (dstDtype TSA_F16 / TSA_BF16: the normalised, rotated values unquantised, the reference's K16),
 * rows in [len, dst.ysize) are zeroed with scale 0; scale f32 [H][rows] may be absent.  D = 64 or 128. */
int tsa_matmul_norm_rope_quant(int srcDtype, int dstDtype, float vecScale, float srcScale, tsa_ptr2d x, tsa_ptr2d w, tsa_ptr2d rope,
    float ropeDir, tsa_ptr2d dst, tsa_ptr2d scale, int headCount, int headDim, int len, int *statusWord,
    tsa_stream_t stream);

/* ---- one-token inference step with KV caches ("next" scope row: the caller of the decode kernel) ---------------
 * Replaces NCPUInfer::ComputePrediction / AddLookupProduct (code/gpt/train/cpu_infer.cpp:466-560), which steps one
 * sequence on the CPU, for a batch of up to 64 sequences on the GPU.  The model is in the reference's int8 form
 * (TCPUModelParams, cpu_infer.cpp:59-84, made by ConvertModel, cpu_infer.cpp:139-158): all matrices row-major int8
 * [rows][cols] in device memory, 16-byte aligned:
 *   qk, qv, k, v [head_count * head_dim][dim];  combiner [dim][4 * head_count * head_dim];
 *   expand [relu_dim][dim];  contract [dim][relu_dim];  label_embed [label_count][dim];  final_layer [vocab_size][dim]
 * bias f32 [vocab_size]; rope f32 [rope_len][head_dim] as FillRopeBuf writes it (code/gpt/att/rope.cpp:4-24).
 * Query and value heads have one size (QDim == TTDim == head_dim, 64 or 128); relu_dim = head_count * 128 * ReluMult
 * (TModelDims::GetReluDim, model_dim.h:66).  `layers` is a host array.
 * State per layer: one KV cache per sequence (tsa_kv_seq with f32 scale planes, capacity rows) and its token count;
 * layerSeqs[l] is a device array of nSeq tsa_kv_seq, ctxLens a device array [layer_count][nSeq] that the step
 * increments (all layers of a sequence hold the same count).  maxCtx: host-side upper bound of the counts before the
 * step.  labels: device int [nSeq][labelsPerSeq], the embedding rows summed for each sequence's new token.
 * prediction f32 [nSeq][vocab_size] (may be NULL) receives the distribution over the vocabulary, logits (may be NULL)
 * the exact int32 products of the final layer as floats.  Asynchronous on `stream`; allocates nothing. */
typedef struct {
    int dim;
    int head_dim;
    int head_count;
    int relu_dim;
    int vocab_size;
    int label_count;
    int layer_count;
} tsa_infer_dims;

typedef struct {
    const signed char *qk, *qv, *k, *v, *combiner, *expand, *contract;
    float qv_scale;       /* TAttentionMatrices::QVScale */
    float combiner_scale; /* CombinerScale */
    float contract_scale; /* ContractScale */
    int attention_width;  /* keys [cur - width, cur - 1]; 0: the new token itself (cpu_infer.cpp:424-432) */
    float alibi_slope;
} tsa_infer_layer;

typedef struct {
    tsa_infer_dims dims;
    const tsa_infer_layer *layers;
    const signed char *label_embed;
    float label_embed_scale;
    const signed char *final_layer;
    float final_layer_scale;
    const float *bias;
    const float *rope;
    int rope_len;
} tsa_infer_model;

size_t tsa_infer_workspace_bytes(const tsa_infer_model *model, int nSeq, int maxCtx);
int tsa_infer_step(const tsa_infer_model *model, const tsa_kv_seq *const *layerSeqs, int *ctxLens, int capacity,
    const int *labels, int labelsPerSeq, int nSeq, int maxCtx, float *prediction, float *logits,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
