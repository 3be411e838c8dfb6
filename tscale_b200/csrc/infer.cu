// One-token inference step of the int8 model over a batch of sequences with per-layer int8 KV caches: the caller of
// the decode attention kernel.  Replaces NCPUInfer::ComputePrediction / AddLookupProduct of the reference
// (code/gpt/train/cpu_infer.cpp:466-560), which runs one sequence on the CPU, by a batch of sequences on the GPU:
//
//   state = sum of label embeddings * scale                                    (cpu_infer.cpp:536-543)
//   per layer (cpu_infer.cpp:466-527):
//     norm   = NormalizeState(state, tiles of 128)            -> int8
//     qk, qv, k, v = int8 matrix * norm (exact int32), rope on qk and qv, NormalizeState per head -> int8
//     cache.append(qv, qvScale * QVScale * VEC_SCALE * dotScale(dim), v);  val = decode attention(qk, cache)
//     kv     = int8(k[z ^ blk] * val[z]), 4 blocks per head; state += Combiner * kv * scale
//     norm   = NormalizeState(state);  relu = max(0, NormalizeState(Expand * norm, per head));  state += Contract * relu * scale
//   prediction = softmax2(FinalLayer * NormalizeState(state) * scale + bias)    (cpu_infer.cpp:549-558)
//
// Everything but the attention weights and the last softmax is integer or single-rounded float arithmetic in the
// reference's order (sums of squares are accumulated sequentially like the scalar loops there), so those stages are
// bit-identical to the CPU code; the attention (tsa_att_decode) and the softmax use exp2 instead of the CPU's
// polynomial.  The matrix products read every int8 weight once per step for the whole batch (dp4a, the batch's
// vectors staged in shared memory, a lane per sequence); at realistic context lengths the step is dominated by the
// KV-cache stream of the decode kernel.
#include "tsa_common.cuh"

namespace tsa {

constexpr float INF_VEC_SCALE = 1.0f / 24; // VEC_SCALE, cpu_infer.cpp:16
constexpr int INF_NORM_TILE = 128;         // STATE_NORM_TILE, model_dim.h:23
constexpr int INF_GEMV_ROWS = 4;           // matrix rows per warp
constexpr int INF_GEMV_WARPS = 4;
constexpr int INF_MAX_SEQ = 64;            // sequences per step
constexpr int INF_TILE_BYTES = 200 * 1024; // shared memory of a matrix product block: 32 vectors and its matrix rows, a chunk of columns

// ConvertToInt8 (cpu_infer.cpp:88-92): round to nearest even, clamp to +-127
__device__ __forceinline__ int ToInt8Clamp127(float x)
{
    return max(-127, min(127, __float2int_rn(x)));
}

__global__ void __launch_bounds__(256) InferEmbedKernel(const int *labels, int labelsPerSeq, int labelCount, const signed char *embed, float embedScale, int dim,
    float *state, int *statusWord)
{
    const int b = blockIdx.x;
    for (int x = threadIdx.x; x < dim; x += blockDim.x) {
        float s = 0;
        for (int i = 0; i < labelsPerSeq; ++i) {
            const int label = labels[b * labelsPerSeq + i];
            if (label < 0 || label >= labelCount) {
                if (x == 0 && statusWord) {
                    atomicOr(statusWord, kDevBadSpan);
                }
                continue;
            }
            s = __fadd_rn(s, __fmul_rn((float)embed[(size_t)label * dim + x], embedScale));
        }
        state[(size_t)b * dim + x] = s;
    }
}

// Sum of squares of n floats in index order, one rounding per product and per sum (the scalar loop of NormalizeState,
// cpu_infer.cpp:369-372); every lane computes the same value from broadcast loads.
__device__ __forceinline__ float SequentialSum2(const float *v, int n)
{
    float sum2 = 0;
#pragma unroll 8
    for (int x = 0; x < n; ++x) {
        const float a = v[x];
        sum2 = __fadd_rn(sum2, __fmul_rn(a, a));
    }
    return sum2;
}

// discrScale and 1 / discrScale of NormalizeState (cpu_infer.cpp:381-383); both 0 for an all-zero group
__device__ __forceinline__ void NormScales(float sum2, int n, float *discr, float *mult)
{
    if (sum2 == 0) {
        *discr = 0;
        *mult = 0;
    } else {
        const float sko = __fsqrt_rn(__fdiv_rn(sum2, (float)n));
        *discr = __fmul_rn(sko, INF_VEC_SCALE);
        *mult = __fdiv_rn(1.0f, *discr);
    }
}

// NormalizeState over groups of groupSize elements: warp per (sequence, group); relu clamps negatives to 0 afterwards.
// The group is staged in shared memory (coalesced loads) when it fits, so that the sequential sum reads broadcasts.
constexpr int INF_NORM_STAGE = 512; // floats per warp
__global__ void __launch_bounds__(256) InferNormKernel(const float *src, int n, int groupSize, int nSeq, int8_t *dst, int relu)
{
    __shared__ float stage[8][INF_NORM_STAGE];
    const int groups = n / groupSize;
    const int task = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (task >= nSeq * groups) {
        return;
    }
    const int b = task / groups, g = task - b * groups;
    const float *s = src + (size_t)b * n + g * groupSize;
    if (groupSize <= INF_NORM_STAGE) {
        for (int x = lane; x < groupSize; x += 32) {
            stage[warp][x] = s[x];
        }
        __syncwarp();
        s = stage[warp];
    }
    float discr, mult;
    NormScales(SequentialSum2(s, groupSize), groupSize, &discr, &mult);
    int8_t *d = dst + (size_t)b * n + g * groupSize;
    for (int x = lane; x < groupSize; x += 32) {
        int q = ToInt8Clamp127(__fmul_rn(s[x], mult));
        d[x] = (int8_t)(relu ? max(q, 0) : q);
    }
}

// The four projections of a token: rope on qk and qv (ReferenceApplyRope, code/gpt/att/rope.cpp:28-46, position =
// tokens already in the cache), then NormalizeState per head.  proj f32 [nSeq][4 * hs] = qk | qv | k | v.
// Warp per (sequence, matrix, head).  qvScale = discrScale * qvMult (cpu_infer.cpp:503-505); vScale = VEC_SCALE.
template <int D>
__global__ void __launch_bounds__(128) InferRopeNormKernel(const float *proj, const float *rope, int ropeLen, const int *ctxLens, int nSeq, int headCount,
    float qvMult, int8_t *qk8, int8_t *qv8, int8_t *k8, int8_t *v8, float *qvScale, float *vScale, int *statusWord)
{
    __shared__ float buf[4][D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int task = blockIdx.x * 4 + warp;
    const int b = blockIdx.y;
    if (task >= 4 * headCount) {
        return;
    }
    const int m = task / headCount, head = task - m * headCount;
    const int hs = headCount * D;
    const float *s = proj + (size_t)b * 4 * hs + (size_t)m * hs + head * D;
    float *w = buf[warp];
    if (m < 2) {
        int pos = ctxLens[b];
        if (pos < 0 || pos >= ropeLen) {
            if (lane == 0 && statusWord) {
                atomicOr(statusWord, kDevBadSpan);
            }
            pos = 0;
        }
        const float *rp = rope + (size_t)pos * D;
#pragma unroll
        for (int blk = 0; blk < D; blk += 64) {
            const float v0 = s[blk + lane], v1 = s[blk + lane + 32];
            const float c = rp[blk + lane], sn = rp[blk + lane + 32];
            w[blk + lane] = __fsub_rn(__fmul_rn(v0, c), __fmul_rn(v1, sn));
            w[blk + lane + 32] = __fadd_rn(__fmul_rn(v0, sn), __fmul_rn(v1, c));
        }
    } else {
        for (int x = lane; x < D; x += 32) {
            w[x] = s[x];
        }
    }
    __syncwarp();
    float discr, mult;
    NormScales(SequentialSum2(w, D), D, &discr, &mult);
    int8_t *dst = (m == 0 ? qk8 : m == 1 ? qv8 : m == 2 ? k8 : v8) + (size_t)b * hs + head * D;
    for (int x = lane; x < D; x += 32) {
        dst[x] = (int8_t)ToInt8Clamp127(__fmul_rn(w[x], mult));
    }
    if (lane == 0) {
        if (m == 1) {
            qvScale[b * headCount + head] = __fmul_rn(discr, qvMult);
        } else if (m == 3) {
            vScale[b * headCount + head] = INF_VEC_SCALE;
        }
    }
}

// KVProduct of the inference path (cpu_infer.cpp:318-337): kv[head][blk][z] = int8(k[head][z ^ blk] * val[head][z])
__global__ void __launch_bounds__(256) InferKvProductKernel(const int8_t *k8, const float *val, int hs, int headDim, int nSeq, int8_t *kv)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nSeq * hs * 4) {
        return;
    }
    const int b = i / (hs * 4), r = i - b * hs * 4;
    const int head = r / (headDim * 4), r2 = r - head * headDim * 4;
    const int blk = r2 / headDim, z = r2 - blk * headDim;
    const float key = (float)k8[(size_t)b * hs + head * headDim + (z ^ blk)];
    kv[i] = (int8_t)ToInt8Clamp127(__fmul_rn(key, val[(size_t)b * hs + head * headDim + z]));
}

struct TGemvJob {
    const int8_t *W; // [Rows][cols] int8
    float *Out;      // element (b, r) at Out[b * OutStride + r]
    int Rows;
};
struct TGemvParams {
    TGemvJob Jobs[4]; // matrices that share the input vectors, blockIdx.y picks one
    const int8_t *Vec; // [nSeq][cols] int8
    int Cols, ChunkCols, NSeq, OutStride;
    float Scale;
};

__device__ __forceinline__ void InferCpAsync16(void *smemDst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smemDst)), "l"(src) : "memory");
}

// out[b][r] = (float)(int32 dot of vec[b] and W[r])            (MulForward, cpu_infer.cpp:282-293)
// ADD: out[b][r] += (float)dot * scale                          (AddScaled, cpu_infer.cpp:296-303)
// A block owns INF_GEMV_WARPS * INF_GEMV_ROWS matrix rows (blockIdx.x), one matrix (blockIdx.y) and 32 sequences
// (blockIdx.z).  Both operands go through shared memory a chunk of columns at a time, fetched with cp.async so that
// all of a block's loads are in flight at once: the matrix rows as they lie (every lane reads the same 16-byte word,
// a broadcast), the 32 vectors with a row pitch of an odd number of 16-byte words (the lanes' reads fall into
// different banks).  A lane owns one sequence, a warp INF_GEMV_ROWS rows.
template <bool ADD>
__global__ void __launch_bounds__(INF_GEMV_WARPS * 32) InferGemvKernel(TGemvParams p)
{
    extern __shared__ int4 gemvSmem[];
    constexpr int TILE_ROWS = INF_GEMV_WARPS * INF_GEMV_ROWS;
    const TGemvJob job = blockIdx.y == 0 ? p.Jobs[0] : blockIdx.y == 1 ? p.Jobs[1] : blockIdx.y == 2 ? p.Jobs[2] : p.Jobs[3];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rowBase = blockIdx.x * TILE_ROWS;
    if (rowBase >= job.Rows) {
        return; // whole block past this matrix
    }
    const int seqBase = blockIdx.z * 32;
    const int nb = min(32, p.NSeq - seqBase);
    const int c16 = p.Cols / 16, chunk16 = p.ChunkCols / 16;
    const int ld16 = chunk16 | 1; // odd pitch
    int4 *vecTile = gemvSmem;                  // [32][ld16]
    int4 *wTile = gemvSmem + 32 * ld16;        // [TILE_ROWS][chunk16]
    int acc[INF_GEMV_ROWS];
#pragma unroll
    for (int r = 0; r < INF_GEMV_ROWS; ++r) {
        acc[r] = 0;
    }
    const int b = min(lane, nb - 1);
    for (int x0 = 0; x0 < c16; x0 += chunk16) {
        const int n16 = min(chunk16, c16 - x0);
        __syncthreads(); // the previous chunk has been read
        for (int s = warp; s < nb; s += INF_GEMV_WARPS) {
            const int4 *src = reinterpret_cast<const int4 *>(p.Vec + (size_t)(seqBase + s) * p.Cols) + x0;
            for (int x = lane; x < n16; x += 32) {
                InferCpAsync16(vecTile + s * ld16 + x, src + x);
            }
        }
        for (int r = warp; r < TILE_ROWS; r += INF_GEMV_WARPS) {
            const int4 *src = reinterpret_cast<const int4 *>(job.W + (size_t)min(rowBase + r, job.Rows - 1) * p.Cols) + x0;
            for (int x = lane; x < n16; x += 32) {
                InferCpAsync16(wTile + r * chunk16 + x, src + x);
            }
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const int4 *vrow = vecTile + b * ld16;
        const int4 *wrow = wTile + warp * INF_GEMV_ROWS * chunk16;
#pragma unroll 4
        for (int x = 0; x < n16; ++x) {
            const int4 v = vrow[x];
#pragma unroll
            for (int r = 0; r < INF_GEMV_ROWS; ++r) {
                const int4 w = wrow[r * chunk16 + x];
                int a = acc[r];
                a = __dp4a(w.x, v.x, a);
                a = __dp4a(w.y, v.y, a);
                a = __dp4a(w.z, v.z, a);
                a = __dp4a(w.w, v.w, a);
                acc[r] = a;
            }
        }
    }
    if (lane < nb) {
#pragma unroll
        for (int r = 0; r < INF_GEMV_ROWS; ++r) {
            const int row = rowBase + warp * INF_GEMV_ROWS + r;
            if (row < job.Rows) {
                float *o = job.Out + (size_t)(seqBase + lane) * p.OutStride + row;
                if (ADD) {
                    *o = __fadd_rn(*o, __fmul_rn((float)acc[r], p.Scale));
                } else {
                    *o = (float)acc[r];
                }
            }
        }
    }
}

// SoftMax of the final layer (cpu_infer.cpp:340-354): base 2, the maximum starts at 0 (TSoftMaxBuf::Clear)
__global__ void __launch_bounds__(1024) InferSoftmaxKernel(const float *logits, const float *bias, float finalScale, int vocab, float *prediction)
{
    __shared__ float red[32];
    __shared__ float bcast;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *l = logits + (size_t)b * vocab;
    float *out = prediction + (size_t)b * vocab;
    float mx = 0;
    for (int x = tid; x < vocab; x += blockDim.x) {
        mx = fmaxf(mx, __fadd_rn(__fmul_rn(l[x], finalScale), bias[x]));
    }
    mx = WarpMax(mx);
    if (lane == 0) {
        red[warp] = mx;
    }
    __syncthreads();
    if (warp == 0) {
        float v = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.0f;
        v = WarpMax(v);
        if (lane == 0) {
            bcast = v;
        }
    }
    __syncthreads();
    mx = bcast;
    float sum = 0;
    for (int x = tid; x < vocab; x += blockDim.x) {
        const float e = exp2f(__fadd_rn(__fmul_rn(l[x], finalScale), bias[x]) - mx);
        out[x] = e;
        sum += e;
    }
    sum = WarpSum(sum);
    __syncthreads();
    if (lane == 0) {
        red[warp] = sum;
    }
    __syncthreads();
    if (warp == 0) {
        float v = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.0f;
        v = WarpSum(v);
        if (lane == 0) {
            bcast = 1.0f / v;
        }
    }
    __syncthreads();
    const float inv = bcast;
    for (int x = tid; x < vocab; x += blockDim.x) {
        out[x] *= inv;
    }
}

static int LaunchGemv(bool add, const TGemvJob *jobs, int jobCount, const int8_t *vec, int cols, int nSeq, int outStride, float scale, cudaStream_t stream)
{
    TGemvParams p;
    int maxRows = 0;
    for (int j = 0; j < 4; ++j) {
        p.Jobs[j] = jobs[j < jobCount ? j : 0];
        maxRows = p.Jobs[j].Rows > maxRows ? p.Jobs[j].Rows : maxRows;
    }
    p.Vec = vec;
    p.Cols = cols;
    p.NSeq = nSeq;
    p.OutStride = outStride;
    p.Scale = scale;
    // columns per shared-memory pass: all of them if 32 vectors and the block's matrix rows fit
    constexpr int TILE_ROWS = INF_GEMV_WARPS * INF_GEMV_ROWS;
    int chunk16 = (INF_TILE_BYTES / 16 - 32) / (32 + TILE_ROWS);
    chunk16 = chunk16 < cols / 16 ? chunk16 : cols / 16;
    p.ChunkCols = chunk16 * 16;
    const size_t smem = ((size_t)32 * (chunk16 | 1) + (size_t)TILE_ROWS * chunk16) * 16;
    const void *kern = add ? (const void *)InferGemvKernel<true> : (const void *)InferGemvKernel<false>;
    int rc = CheckCuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, INF_TILE_BYTES), "cudaFuncSetAttribute");
    if (rc != TSA_OK) {
        return rc;
    }
    dim3 grid((maxRows + TILE_ROWS - 1) / TILE_ROWS, jobCount, (nSeq + 31) / 32);
    void *args[] = {&p};
    return CheckCuda(cudaLaunchKernel(kern, grid, dim3(INF_GEMV_WARPS * 32), args, smem, stream), "inference matrix product launch");
}

static size_t Align256(size_t x)
{
    return (x + 255) / 256 * 256;
}

struct TInferBuffers {
    float *State, *Proj, *QvScale, *VScale, *Val, *Relu, *Logits;
    int8_t *Norm, *Qk8, *Qv8, *K8, *V8, *Kv8;
    void *DecodeWs;
    size_t DecodeWsBytes, Total;
};

static TInferBuffers CarveInferBuffers(const tsa_infer_model *m, int nSeq, int maxCtx, void *base)
{
    const tsa_infer_dims &d = m->dims;
    const size_t hs = (size_t)d.head_count * d.head_dim;
    const size_t widest = (size_t)(d.dim > d.relu_dim ? d.dim : d.relu_dim);
    tsa_decode_cfg cfg = {d.head_dim, TSA_F32, TSA_F32, INF_VEC_SCALE};
    TInferBuffers b;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        void *p = base ? (char *)base + off : nullptr;
        off += Align256(bytes);
        return p;
    };
    b.State = (float *)take(sizeof(float) * nSeq * d.dim);
    b.Proj = (float *)take(sizeof(float) * nSeq * 4 * hs);
    b.QvScale = (float *)take(sizeof(float) * nSeq * d.head_count);
    b.VScale = (float *)take(sizeof(float) * nSeq * d.head_count);
    b.Val = (float *)take(sizeof(float) * nSeq * hs);
    b.Relu = (float *)take(sizeof(float) * nSeq * d.relu_dim);
    b.Logits = (float *)take(sizeof(float) * nSeq * d.vocab_size);
    b.Norm = (int8_t *)take((size_t)nSeq * widest);
    b.Qk8 = (int8_t *)take((size_t)nSeq * hs);
    b.Qv8 = (int8_t *)take((size_t)nSeq * hs);
    b.K8 = (int8_t *)take((size_t)nSeq * hs);
    b.V8 = (int8_t *)take((size_t)nSeq * hs);
    b.Kv8 = (int8_t *)take((size_t)nSeq * hs * 4);
    b.DecodeWsBytes = tsa_att_decode_workspace_bytes(&cfg, nSeq, d.head_count, maxCtx + 1);
    b.DecodeWs = take(b.DecodeWsBytes);
    b.Total = off;
    return b;
}

static int CheckInferModel(const tsa_infer_model *m, int nSeq, const char *fn)
{
    TSA_REQUIRE(m != nullptr, "%s: null model", fn);
    const tsa_infer_dims &d = m->dims;
    TSA_REQUIRE(d.head_dim == 64 || d.head_dim == 128, "%s: head_dim %d must be 64 or 128 (query and value heads have one size here)", fn, d.head_dim);
    TSA_REQUIRE(d.dim > 0 && d.dim % INF_NORM_TILE == 0, "%s: dim %d must be a multiple of %d", fn, d.dim, INF_NORM_TILE);
    TSA_REQUIRE(d.head_count > 0 && d.relu_dim > 0 && d.relu_dim % d.head_count == 0 && d.relu_dim % 16 == 0,
        "%s: relu_dim %d must be a multiple of head_count %d and of 16", fn, d.relu_dim, d.head_count);
    TSA_REQUIRE(d.vocab_size > 0 && d.label_count > 0 && d.layer_count >= 0, "%s: vocab_size, label_count must be positive", fn);
    TSA_REQUIRE(nSeq >= 0 && nSeq <= INF_MAX_SEQ, "%s: %d sequences per step, at most %d", fn, nSeq, INF_MAX_SEQ);
    return TSA_OK;
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) size_t tsa_infer_workspace_bytes(const tsa_infer_model *model, int nSeq, int maxCtx)
{
    if (CheckInferModel(model, nSeq, "tsa_infer_workspace_bytes") != TSA_OK || nSeq == 0 || maxCtx < 0) {
        return 0;
    }
    return CarveInferBuffers(model, nSeq, maxCtx, nullptr).Total;
}

extern "C" __attribute__((visibility("default"))) int tsa_infer_step(const tsa_infer_model *model, const tsa_kv_seq *const *layerSeqs, int *ctxLens,
    int capacity, const int *labels, int labelsPerSeq, int nSeq, int maxCtx, float *prediction, float *logits, void *workspace,
    size_t workspaceBytes, int *statusWord, tsa_stream_t streamArg)
{
    int rc = CheckInferModel(model, nSeq, "tsa_infer_step");
    if (rc != TSA_OK) {
        return rc;
    }
    if (nSeq == 0) {
        return TSA_OK;
    }
    const tsa_infer_dims &d = model->dims;
    TSA_REQUIRE(labels && ctxLens && labelsPerSeq > 0 && maxCtx >= 0 && capacity > maxCtx, "tsa_infer_step: labels, ctxLens, capacity > maxCtx");
    TSA_REQUIRE(d.layer_count == 0 || (model->layers && layerSeqs), "tsa_infer_step: null layers");
    TSA_REQUIRE(model->label_embed && model->final_layer && model->bias && model->rope && model->rope_len > maxCtx,
        "tsa_infer_step: model tables (the rope table must cover position maxCtx = %d, it has %d rows)", maxCtx, model->rope_len);
    const TInferBuffers need = CarveInferBuffers(model, nSeq, maxCtx, nullptr);
    TSA_REQUIRE(workspace && workspaceBytes >= need.Total && (uintptr_t)workspace % 256 == 0, "tsa_infer_step: workspace of %zu bytes, 256-byte aligned, needed",
        need.Total);
    const TInferBuffers b = CarveInferBuffers(model, nSeq, maxCtx, workspace);
    cudaStream_t stream = (cudaStream_t)streamArg;
    const int H = d.head_count, D = d.head_dim, hs = H * D, dim = d.dim;
    tsa_decode_cfg cfg = {D, TSA_F32, TSA_F32, INF_VEC_SCALE};

    auto norm = [&](const float *src, int n, int groupSize, bool relu) {
        const int warps = nSeq * (n / groupSize);
        InferNormKernel<<<(warps * 32 + 255) / 256, 256, 0, stream>>>(src, n, groupSize, nSeq, b.Norm, relu ? 1 : 0);
        return CheckCuda(cudaGetLastError(), "inference normalise launch");
    };
    auto ptr2d = [](void *data, int strideBytes, int xs, int ys) {
        tsa_ptr2d p = {data, strideBytes, xs, ys};
        return p;
    };

    InferEmbedKernel<<<nSeq, 256, 0, stream>>>(labels, labelsPerSeq, d.label_count, model->label_embed, model->label_embed_scale, dim, b.State, statusWord);
    rc = CheckCuda(cudaGetLastError(), "inference embedding launch");
    for (int l = 0; l < d.layer_count && rc == TSA_OK; ++l) {
        const tsa_infer_layer &layer = model->layers[l];
        TSA_REQUIRE(layer.qk && layer.qv && layer.k && layer.v && layer.combiner && layer.expand && layer.contract && layerSeqs[l],
            "tsa_infer_step: layer %d has a null matrix or cache", l);
        int *lens = ctxLens + (size_t)l * nSeq;
        rc = norm(b.State, dim, INF_NORM_TILE, false);
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob proj[4] = {{layer.qk, b.Proj, hs}, {layer.qv, b.Proj + hs, hs}, {layer.k, b.Proj + 2 * hs, hs}, {layer.v, b.Proj + 3 * hs, hs}};
        rc = LaunchGemv(false, proj, 4, b.Norm, dim, nSeq, 4 * hs, 0.0f, stream);
        if (rc != TSA_OK) {
            break;
        }
        // same association as cpu_infer.cpp:504: qvScale *= (QVScale * VEC_SCALE) * dotScale(dim)
        const float qvMult = layer.qv_scale * INF_VEC_SCALE * sqrtf(1.0f / dim);
        dim3 gridR((4 * H + 3) / 4, nSeq);
        if (D == 64) {
            InferRopeNormKernel<64><<<gridR, 128, 0, stream>>>(b.Proj, model->rope, model->rope_len, lens, nSeq, H, qvMult, b.Qk8, b.Qv8, b.K8, b.V8, b.QvScale,
                b.VScale, statusWord);
        } else {
            InferRopeNormKernel<128><<<gridR, 128, 0, stream>>>(b.Proj, model->rope, model->rope_len, lens, nSeq, H, qvMult, b.Qk8, b.Qv8, b.K8, b.V8, b.QvScale,
                b.VScale, statusWord);
        }
        rc = CheckCuda(cudaGetLastError(), "inference rope launch");
        if (rc != TSA_OK) {
            break;
        }
        rc = tsa_kv_append(&cfg, layerSeqs[l], lens, nSeq, capacity, ptr2d(b.Qv8, hs, hs, nSeq), ptr2d(b.QvScale, H * 4, H, nSeq), ptr2d(b.V8, hs, hs, nSeq),
            ptr2d(b.VScale, H * 4, H, nSeq), H, statusWord, streamArg);
        if (rc != TSA_OK) {
            break;
        }
        tsa_ptr2d none = {nullptr, 0, 0, 0};
        rc = tsa_att_decode(&cfg, layerSeqs[l], lens, nSeq, maxCtx + 1, ptr2d(b.Qk8, hs, hs, nSeq), none, layer.attention_width, layer.alibi_slope,
            ptr2d(b.Val, hs * 4, hs, nSeq), H, b.DecodeWs, b.DecodeWsBytes, statusWord, streamArg);
        if (rc != TSA_OK) {
            break;
        }
        InferKvProductKernel<<<(nSeq * hs * 4 + 255) / 256, 256, 0, stream>>>(b.K8, b.Val, hs, D, nSeq, b.Kv8);
        rc = CheckCuda(cudaGetLastError(), "inference kv product launch");
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob comb[1] = {{layer.combiner, b.State, dim}};
        rc = LaunchGemv(true, comb, 1, b.Kv8, hs * 4, nSeq, dim, layer.combiner_scale * INF_VEC_SCALE * sqrtf(1.0f / (hs * 4)), stream);
        if (rc != TSA_OK) {
            break;
        }
        rc = norm(b.State, dim, INF_NORM_TILE, false);
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob expand[1] = {{layer.expand, b.Relu, d.relu_dim}};
        rc = LaunchGemv(false, expand, 1, b.Norm, dim, nSeq, d.relu_dim, 0.0f, stream);
        if (rc != TSA_OK) {
            break;
        }
        rc = norm(b.Relu, d.relu_dim, d.relu_dim / H, true);
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob contract[1] = {{layer.contract, b.State, dim}};
        rc = LaunchGemv(true, contract, 1, b.Norm, d.relu_dim, nSeq, dim, layer.contract_scale * INF_VEC_SCALE * sqrtf(1.0f / d.relu_dim), stream);
    }
    if (rc != TSA_OK) {
        return rc;
    }
    if (prediction || logits) {
        rc = norm(b.State, dim, INF_NORM_TILE, false);
        if (rc != TSA_OK) {
            return rc;
        }
        float *lg = logits ? logits : b.Logits;
        TGemvJob fin[1] = {{model->final_layer, lg, d.vocab_size}};
        rc = LaunchGemv(false, fin, 1, b.Norm, dim, nSeq, d.vocab_size, 0.0f, stream);
        if (rc != TSA_OK) {
            return rc;
        }
        if (prediction) {
            // CalcDotScale(dim) * CalcFinalLayerMult() * FinalLayerScale * VEC_SCALE (cpu_infer.cpp:555)
            const float finalScale = sqrtf(1.0f / dim) * (1.0f / 0.693147f) * model->final_layer_scale * INF_VEC_SCALE;
            InferSoftmaxKernel<<<nSeq, 1024, 0, stream>>>(lg, model->bias, finalScale, d.vocab_size, prediction);
            rc = CheckCuda(cudaGetLastError(), "inference softmax launch");
        }
    }
    return rc;
}
