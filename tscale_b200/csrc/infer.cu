// One-token inference step of the int8 model over a batch of sequences with per-layer int8 KV caches: the caller of
// the decode attention kernel.  Replaces NCPUInfer::ComputePrediction / AddLookupProduct of the reference
// (code/gpt/train/cpu_infer.cpp:466-560), which runs one sequence on the CPU, by a batch of sequences on the GPU:
//
//   state = sum of label embeddings * scale                                    (cpu_infer.cpp:536-543)
//   per layer (cpu_infer.cpp:466-527):
//     norm   = NormalizeState(state, tiles of 128)            -> int8
//     qk, qv, k, v = int8 matrix * norm (exact int32), rope on qk and qv, NormalizeState per head -> int8
//     cache.append(qv, qvScale * QVScale * VEC_SCALE * dotScale(dim), v)  (written by the rope kernel);  val = decode attention(qk, cache)
//     kv     = int8(k[z ^ blk] * val[z]), 4 blocks per head (written by the decode merge kernel); state += Combiner * kv * scale
//     norm   = NormalizeState(state);  relu = max(0, NormalizeState(Expand * norm, per head));  state += Contract * relu * scale
//   prediction = softmax2(FinalLayer * NormalizeState(state) * scale + bias)    (cpu_infer.cpp:549-558)
//
// Everything but the attention weights and the last softmax is integer or single-rounded float arithmetic in the
// reference's order (sums of squares are accumulated sequentially like the scalar loops there), so those stages are
// bit-identical to the CPU code; the attention (tsa_att_decode) and the softmax use exp2 instead of the CPU's
// polynomial.  The matrix products read every int8 weight once per step for the whole batch (tcgen05 kind::i8, exact
// int32 accumulators); at realistic context lengths the step is dominated by the KV-cache stream of the decode kernel.
#include "att_sm100_common.cuh"
#include <cooperative_groups.h>

namespace tsa {

// decode.cu: tsa_att_decode whose merge kernel also writes the combiner input
int DecodeWithKvProduct(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, const int *ctxLens, int nSeq, int maxCtx, tsa_ptr2d q, tsa_ptr2d qScale, int window,
    float alibiSlope, tsa_ptr2d out, int headCount, void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream, const int8_t *kvKey,
    int8_t *kvOut, int ctxBias);

constexpr float INF_VEC_SCALE = 1.0f / 24; // VEC_SCALE, cpu_infer.cpp:16
constexpr int INF_NORM_TILE = 128;         // STATE_NORM_TILE, model_dim.h:23
constexpr int INF_MAX_SEQ = 64;            // sequences per step

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
// Warp per (sequence, matrix, head).  qv and v go straight into the sequence's KV cache at row ctxLens[b]
// (AddVectors, cpu_infer.cpp:403-408) with the key scale discrScale * qvMult (cpu_infer.cpp:503-505) and the value
// scale VEC_SCALE; the token is counted by InferCountKernel at the end of the step, the attention in between is told
// to add one to every count.
template <int D>
__global__ void __launch_bounds__(128) InferRopeNormKernel(const float *proj, const float *rope, int ropeLen, const int *ctxLens, int nSeq, int headCount,
    float qvMult, int8_t *qk8, int8_t *k8, const tsa_kv_seq *seqs, int capacity, int *statusWord)
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
    int pos = ctxLens[b];
    if (pos < 0 || pos >= ropeLen || pos >= capacity) {
        if (lane == 0 && statusWord) {
            atomicOr(statusWord, kDevBadSpan); // the cache or the rope table is full
        }
        return;
    }
    if (m < 2) {
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
    int8_t *dst;
    if (m == 0 || m == 2) {
        dst = (m == 0 ? qk8 : k8) + (size_t)b * hs + head * D;
    } else {
        const tsa_kv_seq sq = seqs[b];
        dst = (int8_t *)(m == 1 ? sq.k : sq.v) + (size_t)pos * hs + head * D;
        if (lane == 0) {
            float *scale = (float *)(m == 1 ? sq.kScale : sq.vScale) + (size_t)pos * headCount + head;
            *scale = m == 1 ? __fmul_rn(discr, qvMult) : INF_VEC_SCALE;
        }
    }
    for (int x = lane; x < D; x += 32) {
        dst[x] = (int8_t)ToInt8Clamp127(__fmul_rn(w[x], mult));
    }
}

// counts the step's token in every layer's cache
__global__ void InferCountKernel(int *ctxLens, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        ctxLens[i] += 1;
    }
}

struct TGemvJob {
    const int8_t *W; // [Rows][cols] int8
    float *Out;      // element (b, r) at Out[b * OutStride + r]
    int Rows;
};

// ---- int8 matrix products on the tensor cores --------------------------------------------------------------------
// out[b][r] = (float)(int32 dot of vec[b] and W[r])            (MulForward, cpu_infer.cpp:282-293)
// ADD: out[b][r] += (float)dot * scale                          (AddScaled, cpu_infer.cpp:296-303)
// One CTA = 128 rows of one matrix (blockIdx.x, blockIdx.y) times all sequences (at most 64): tcgen05.mma kind::i8,
// M = 128 matrix rows, N = 64 sequences, exact int32 accumulators in 64 tensor-memory columns.  Thread 0 streams the
// row slab and the batch's vectors through a ring of GEMM_STAGES shared-memory stages of 128 columns (TMA, 128-byte
// swizzle; rows past the matrix and sequences past the batch read as zeros) and issues the MMAs; afterwards thread t
// holds row t of the tile and writes its 64 products, coalesced over the rows of a warp.  Every wait is bounded.
// A matrix with few rows and many columns (the combiner: 768 x 3072) would leave a handful of CTAs each waiting on
// two dozen dependent-latency chunk loads, so its columns are split over the KSplit CTAs of a thread-block cluster:
// every CTA accumulates its share, ranks above 0 park their int32 tile in their own shared memory and rank 0 adds
// them through distributed shared memory (exact, order does not matter) before the epilogue.
constexpr int GEMM_STAGES = 8;
constexpr int GEMM_M = 128, GEMM_N = 64, GEMM_KB = 128;
constexpr int GEMM_STAGE_BYTES = (GEMM_M + GEMM_N) * GEMM_KB;
constexpr int GEMM_SMEM_BYTES = GEMM_STAGES * GEMM_STAGE_BYTES + 1024 /* barriers */ + 1024 /* alignment */;

struct TGemmMisc {
    uint64_t Full[GEMM_STAGES], Empty[GEMM_STAGES], Done;
    uint32_t TmemBase;
};
struct TGemmArgs {
    float *Out[4];
    int Rows[4];
    int OutStride, NSeq, Chunks;
    float Scale;
    int8_t *NormOut; // may be null: NormalizeState of the tile's 128 result rows, [NSeq][OutStride] int8
    int NormRelu;    // clamp the normalised values at 0 (the relu block's input)
    int KSplit;      // CTAs of a cluster that share a row tile, each with Chunks / KSplit of the columns
};

// KS > 1: the matrix columns (the inner dimension) are split over a cluster of KS CTAs (wide matrices).
// NS > 1: the sequences are split over NS independent CTAs, each with its own MMA of GEMM_N / NS accumulator columns
// (matrices with few row tiles: more CTAs, and each runs a share of the epilogue).
template <bool ADD, int KS, int NS>
__global__ void __launch_bounds__(128, 1) InferGemmI8Kernel(const __grid_constant__ CUtensorMap tmW0, const __grid_constant__ CUtensorMap tmW1,
    const __grid_constant__ CUtensorMap tmW2, const __grid_constant__ CUtensorMap tmW3, const __grid_constant__ CUtensorMap tmVec, TGemmArgs a,
    int *status)
{
    constexpr int NT = GEMM_N / NS;                                       // accumulator columns (sequences) of this CTA's MMA
    constexpr int TMEM_COLS = NT < 32 ? 32 : NT;
    constexpr uint32_t STAGE_TX = (GEMM_M + NT) * GEMM_KB;                // bytes a stage receives
    constexpr uint32_t IDESC = MakeInstrDesc(2, 1, 1, 0, 0, GEMM_M, NT); // s32 accumulators, s8 x s8, both K-major
    extern __shared__ uint8_t gemmSmemRaw[];
    const int job = blockIdx.y;
    const int rows = job == 0 ? a.Rows[0] : job == 1 ? a.Rows[1] : job == 2 ? a.Rows[2] : a.Rows[3];
    float *out = job == 0 ? a.Out[0] : job == 1 ? a.Out[1] : job == 2 ? a.Out[2] : a.Out[3];
    const CUtensorMap *tmW = job == 0 ? &tmW0 : job == 1 ? &tmW1 : job == 2 ? &tmW2 : &tmW3;
    constexpr int kSplit = KS * NS;            // CTAs that share this row tile
    constexpr int CPR = GEMM_N / kSplit;       // sequences (accumulator columns) a CTA finishes
    const int kRank = blockIdx.x % KS;         // rank in the cluster (share of the inner dimension)
    const int nRank = (blockIdx.x / KS) % NS;  // share of the sequences
    const int rowBase = (blockIdx.x / kSplit) * GEMM_M;
    if (rowBase >= rows) {
        return; // the grid is sized for the tallest matrix of the launch; a cluster leaves as a whole
    }
    uint8_t *smem = (uint8_t *)(((uintptr_t)gemmSmemRaw + 1023) & ~(uintptr_t)1023);
    TGemmMisc &misc = *reinterpret_cast<TGemmMisc *>(smem + GEMM_STAGES * GEMM_STAGE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < GEMM_STAGES; ++s) {
            MbarInit(&misc.Full[s], 1);
            MbarInit(&misc.Empty[s], 1);
        }
        MbarInit(&misc.Done, 1);
        FenceBarrierInit();
    }
    if (warp == 0) {
        TmemAlloc(&misc.TmemBase, TMEM_COLS);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;
    bool failed = false;
    if (tid == 0) {
        PrefetchTensorMap(tmW);
        PrefetchTensorMap(&tmVec);
        auto load = [&](int chunk) {
            const int s = chunk % GEMM_STAGES;
            uint8_t *sA = smem + s * GEMM_STAGE_BYTES, *sB = sA + GEMM_M * GEMM_KB;
            MbarExpectTx(&misc.Full[s], STAGE_TX);
            const int col = ((KS > 1 ? kRank * (a.Chunks / KS) : 0) + chunk) * GEMM_KB;
            TmaLoad2D(sA, tmW, col, rowBase, &misc.Full[s]);
            TmaLoad2D(sB, &tmVec, col, nRank * NT, &misc.Full[s]);
        };
        // GEMM_AHEAD chunks are in flight; the stage a new load overwrites was read by the MMAs of two iterations ago,
        // whose completion has long arrived (waiting for the previous iteration's would stall every step on the
        // commit round trip)
        constexpr int GEMM_AHEAD = GEMM_STAGES - 2;
        const int chunks = a.Chunks / KS;
        int issued = 0, landed = 0; // chunks requested / chunks whose copies were seen to arrive
        for (int c = 0; c < GEMM_AHEAD && c < chunks; ++c) {
            load(c);
            ++issued;
        }
        for (int c = 0; c < chunks && !failed; ++c) {
            const int ahead = c + GEMM_AHEAD;
            if (ahead < chunks) {
                if (ahead >= GEMM_STAGES && !WaitBar(&misc.Empty[ahead % GEMM_STAGES], (uint32_t)((ahead / GEMM_STAGES - 1) & 1))) {
                    failed = true; // the MMAs that read this stage never finished
                    if (status) {
                        atomicOr(status, kDevTimeoutMma);
                    }
                    break;
                }
                load(ahead);
                ++issued;
            }
            const int s = c % GEMM_STAGES;
            if (!WaitBar(&misc.Full[s], (uint32_t)((c / GEMM_STAGES) & 1))) {
                failed = true;
                if (status) {
                    atomicOr(status, kDevTimeoutTma);
                }
                break;
            }
            ++landed;
            TcFenceAfter();
            const uint32_t sA = SmemAddr(smem + s * GEMM_STAGE_BYTES), sB = sA + GEMM_M * GEMM_KB;
#pragma unroll
            for (int ks = 0; ks < GEMM_KB / 32; ++ks) {
                const uint64_t aDesc = MakeSmemDesc(sA + ks * 32, 16, 8 * GEMM_KB, 128);
                const uint64_t bDesc = MakeSmemDesc(sB + ks * 32, 16, 8 * GEMM_KB, 128);
                MmaI8SS(tmem, aDesc, bDesc, IDESC, (c > 0 || ks > 0) ? 1u : 0u);
            }
            MmaCommit(&misc.Empty[s]);
        }
        if (failed) {
            // copies that were requested but never consumed must not land after the CTA is gone: wait (bounded) for them
            for (int t = landed; t < issued; ++t) {
                WaitBar(&misc.Full[t % GEMM_STAGES], (uint32_t)((t / GEMM_STAGES) & 1));
            }
        }
        MmaCommit(&misc.Done);
    }
    if (!WaitBar(&misc.Done, 0)) {
        failed = true;
        if (status) {
            atomicOr(status, kDevTimeoutMma);
        }
    }
    TcFenceAfter();
    failed = __syncthreads_or(failed ? 1 : 0) != 0;
    const int row = rowBase + tid;
    // With NormOut: the tile's 128 rows are one normalisation group (a STATE_NORM_TILE of the state, or a head of the
    // relu block when its heads are 128 wide), so the
    // int8 input of the next matrix product is made here, from the values just stored: they go through shared memory
    // (the ring is idle by now), one thread per sequence adds the squares in row order like the scalar loop of
    // NormalizeState, then every thread converts its row.
    float *normTile = reinterpret_cast<float *>(smem);            // [GEMM_N][GEMM_M + 1]
    float *normMult = normTile + GEMM_N * (GEMM_M + 1);           // [GEMM_N]
    const bool withNorm = a.NormOut != nullptr;
    uint32_t accum[NT];
    {
        const uint32_t tLane = tmem + ((uint32_t)(warp * 32) << 16);
        if (NT == 16) {
            TmemLd16(tLane, accum);
        } else {
            TmemLd32(tLane, accum);
            if (NT == 64) {
                TmemLd32(tLane + 32, accum + (NT == 64 ? 32 : 0));
            }
        }
        TmemWaitLd();
    }
    // Reduce-scatter over the cluster: every CTA parks its int32 tile in its own shared memory, then finishes CPR of the
    // 64 sequences: it adds the other CTAs' partial sums of those columns through distributed shared memory (exact, the
    // order does not matter) and runs the epilogue for them, so the epilogue's work is split as well.
    int sum[KS > 1 ? CPR : 1];
    if (KS > 1) {
        // both cluster barriers are passed by every CTA whatever happened before, so that none waits alone
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        int *part = reinterpret_cast<int *>(smem); // [NT][GEMM_M], the ring is idle by now
#pragma unroll
        for (int cc = 0; cc < NT; ++cc) {
            part[cc * GEMM_M + tid] = (int)accum[cc];
        }
        cluster.sync();
#pragma unroll
        for (int j = 0; j < CPR; ++j) {
            sum[j] = part[(kRank * CPR + j) * GEMM_M + tid];
        }
        for (int step = 1; step < KS; ++step) {
            const int *remote = cluster.map_shared_rank(part, (kRank + step) % KS);
#pragma unroll
            for (int j = 0; j < CPR; ++j) {
                sum[j] += remote[(kRank * CPR + j) * GEMM_M + tid];
            }
        }
        cluster.sync(); // every CTA's shared memory has been read: it may be reused and the CTA may leave
    }
    const int colBase = nRank * NT + kRank * CPR;
    if (!failed) {
        constexpr int BLK = CPR < 32 ? CPR : 32;
#pragma unroll
        for (int c0 = 0; c0 < CPR; c0 += BLK) {
            if (row < rows) {
                float *o = out + (size_t)(colBase + c0) * a.OutStride + row;
                float old[BLK];
                if (ADD) { // all loads before the first store: they are independent, a store in between would serialise them
#pragma unroll
                    for (int cc = 0; cc < BLK; ++cc) {
                        old[cc] = (colBase + c0 + cc < a.NSeq) ? o[(size_t)cc * a.OutStride] : 0.0f;
                    }
                }
#pragma unroll
                for (int cc = 0; cc < BLK; ++cc) {
                    if (colBase + c0 + cc < a.NSeq) {
                        const float v = (float)(KS > 1 ? sum[(c0 + cc) % (KS > 1 ? CPR : 1)] : (int)accum[(c0 + cc) % NT]);
                        const float res = ADD ? __fadd_rn(old[cc], __fmul_rn(v, a.Scale)) : v;
                        if (ADD || !withNorm) { // a product that is only normalised does not need its fp32 form in memory
                            o[(size_t)cc * a.OutStride] = res;
                        }
                        if (withNorm) {
                            normTile[(c0 + cc) * (GEMM_M + 1) + tid] = res;
                        }
                    }
                }
            }
        }
        if (withNorm) {
            __syncthreads();
            if (tid < CPR && colBase + tid < a.NSeq) {
                float discr, mult;
                NormScales(SequentialSum2(normTile + tid * (GEMM_M + 1), GEMM_M), GEMM_M, &discr, &mult);
                normMult[tid] = mult;
            }
            __syncthreads();
            if (row < rows) {
#pragma unroll 8
                for (int s = 0; s < CPR; ++s) {
                    if (colBase + s < a.NSeq) {
                        const int q = ToInt8Clamp127(__fmul_rn(normTile[s * (GEMM_M + 1) + tid], normMult[s]));
                        a.NormOut[(size_t)(colBase + s) * a.OutStride + row] = (int8_t)(a.NormRelu ? max(q, 0) : q);
                    }
                }
            }
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == 0) {
        TmemDealloc(tmem, TMEM_COLS);
    }
}

// SoftMax of the final layer (cpu_infer.cpp:340-354): base 2, the maximum starts at 0 (TSoftMaxBuf::Clear).
// Two kernels over (sequence, slice of the vocabulary) so that a batch of 64 sequences fills the GPU: the first leaves
// each slice's maximum and sum of 2^(w - max), the second merges the slices' pairs and writes the probabilities.
constexpr int INF_SOFTMAX_SLICES = 8;

__device__ __forceinline__ float BlockReduce(float v, bool isMax, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    v = isMax ? WarpMax(v) : WarpSum(v);
    __syncthreads(); // red may still be read from the previous reduction
    if (lane == 0) {
        red[warp] = v;
    }
    __syncthreads();
    float r = red[0];
    for (int w = 1; w < warps; ++w) {
        r = isMax ? fmaxf(r, red[w]) : r + red[w];
    }
    return r;
}

__global__ void __launch_bounds__(256) InferSoftmaxPartKernel(const float *logits, const float *bias, float finalScale, int vocab, float *part)
{
    __shared__ float red[8];
    const int b = blockIdx.y, slice = blockIdx.x;
    const int per = (vocab + INF_SOFTMAX_SLICES - 1) / INF_SOFTMAX_SLICES;
    const int x0 = slice * per, x1 = min(x0 + per, vocab);
    const float *l = logits + (size_t)b * vocab;
    float mx = 0;
    for (int x = x0 + threadIdx.x; x < x1; x += blockDim.x) {
        mx = fmaxf(mx, __fadd_rn(__fmul_rn(l[x], finalScale), bias[x]));
    }
    mx = BlockReduce(mx, true, red);
    float sum = 0;
    for (int x = x0 + threadIdx.x; x < x1; x += blockDim.x) {
        sum += exp2f(__fadd_rn(__fmul_rn(l[x], finalScale), bias[x]) - mx);
    }
    sum = BlockReduce(sum, false, red);
    if (threadIdx.x == 0) {
        part[(b * INF_SOFTMAX_SLICES + slice) * 2] = mx;
        part[(b * INF_SOFTMAX_SLICES + slice) * 2 + 1] = sum;
    }
}

__global__ void __launch_bounds__(256) InferSoftmaxKernel(const float *logits, const float *bias, float finalScale, int vocab, const float *part,
    float *prediction)
{
    const int b = blockIdx.y, slice = blockIdx.x;
    const int per = (vocab + INF_SOFTMAX_SLICES - 1) / INF_SOFTMAX_SLICES;
    const int x0 = slice * per, x1 = min(x0 + per, vocab);
    float mx = 0;
#pragma unroll
    for (int s = 0; s < INF_SOFTMAX_SLICES; ++s) {
        mx = fmaxf(mx, part[(b * INF_SOFTMAX_SLICES + s) * 2]);
    }
    float sum = 0;
#pragma unroll
    for (int s = 0; s < INF_SOFTMAX_SLICES; ++s) {
        sum += part[(b * INF_SOFTMAX_SLICES + s) * 2 + 1] * exp2f(part[(b * INF_SOFTMAX_SLICES + s) * 2] - mx);
    }
    const float inv = 1.0f / sum;
    const float *l = logits + (size_t)b * vocab;
    float *out = prediction + (size_t)b * vocab;
    for (int x = x0 + threadIdx.x; x < x1; x += blockDim.x) {
        out[x] = exp2f(__fadd_rn(__fmul_rn(l[x], finalScale), bias[x]) - mx) * inv;
    }
}

static int LaunchGemv(bool add, const TGemvJob *jobs, int jobCount, const int8_t *vec, int cols, int nSeq, int outStride, float scale, int8_t *normOut,
    int *statusWord, cudaStream_t stream, bool normRelu = false)
{
    CUtensorMap mw[4], mv;
    TGemmArgs a;
    int maxRows = 0;
    for (int j = 0; j < 4; ++j) {
        const TGemvJob &job = jobs[j < jobCount ? j : 0];
        tsa_ptr2d w = {(void *)job.W, cols, cols, job.Rows};
        int rc = MakeTileMapEx(&mw[j], w, 1, GEMM_KB, GEMM_M, "inference matrix");
        if (rc != TSA_OK) {
            return rc;
        }
        a.Out[j] = job.Out;
        a.Rows[j] = job.Rows;
        maxRows = job.Rows > maxRows ? job.Rows : maxRows;
    }
    const int rowTiles = (maxRows + GEMM_M - 1) / GEMM_M;
    const int chunkCount = cols / GEMM_KB;
    // about six 128-column chunks per CTA: a cluster of 2 or 4 CTAs shares a row tile of a wide matrix; a narrow matrix
    // with few row tiles spreads the sequences over 2 or 4 CTAs per row tile instead
    const int kSplit = (chunkCount >= 24 && chunkCount % 4 == 0) ? 4 : (chunkCount >= 12 && chunkCount % 2 == 0) ? 2 : 1;
    int nSplit = (rowTiles * jobCount * kSplit > 48 || nSeq <= 16) ? 1 : (nSeq <= 32 ? 2 : 4);
    if (kSplit * nSplit > 4) {
        nSplit = 4 / kSplit; // a CTA finishes at least 16 sequences
    }
    tsa_ptr2d v = {(void *)vec, cols, cols, nSeq};
    int rc = MakeTileMapEx(&mv, v, 1, GEMM_KB, GEMM_N / nSplit, "inference vectors");
    if (rc != TSA_OK) {
        return rc;
    }
    a.OutStride = outStride;
    a.NSeq = nSeq;
    a.Chunks = cols / GEMM_KB;
    a.Scale = scale;
    a.NormOut = normOut;
    a.NormRelu = normRelu ? 1 : 0;
    a.KSplit = kSplit;
    const void *kern = nullptr;
#define TSA_GEMM_CASE(KS, NS)                                                                                              \
    if (kSplit == KS && nSplit == NS) {                                                                                    \
        kern = add ? (const void *)InferGemmI8Kernel<true, KS, NS> : (const void *)InferGemmI8Kernel<false, KS, NS>;       \
    }
    TSA_GEMM_CASE(1, 1)
    TSA_GEMM_CASE(2, 1)
    TSA_GEMM_CASE(4, 1)
    TSA_GEMM_CASE(1, 2)
    TSA_GEMM_CASE(1, 4)
    TSA_GEMM_CASE(2, 2)
#undef TSA_GEMM_CASE
    rc = CheckCuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES), "cudaFuncSetAttribute");
    if (rc != TSA_OK) {
        return rc;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = a.KSplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(rowTiles * kSplit * nSplit, jobCount);
    lc.blockDim = dim3(128);
    lc.dynamicSmemBytes = GEMM_SMEM_BYTES;
    lc.stream = stream;
    lc.attrs = attr;
    lc.numAttrs = 1;
    void *args[] = {&mw[0], &mw[1], &mw[2], &mw[3], &mv, &a, &statusWord};
    return CheckCuda(cudaLaunchKernelExC(&lc, kern, args), "inference matrix product launch");
}

static size_t Align256(size_t x)
{
    return (x + 255) / 256 * 256;
}

struct TInferBuffers {
    float *State, *Proj, *Val, *Relu, *Logits, *SoftmaxPart;
    int8_t *NormState, *NormRelu, *Qk8, *K8, *Kv8;
    void *DecodeWs;
    size_t DecodeWsBytes, Total;
};

static TInferBuffers CarveInferBuffers(const tsa_infer_model *m, int nSeq, int maxCtx, void *base)
{
    const tsa_infer_dims &d = m->dims;
    const size_t hs = (size_t)d.head_count * d.head_dim;
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
    b.Val = (float *)take(sizeof(float) * nSeq * hs);
    b.Relu = (float *)take(sizeof(float) * nSeq * d.relu_dim);
    b.Logits = (float *)take(sizeof(float) * nSeq * d.vocab_size);
    b.SoftmaxPart = (float *)take(sizeof(float) * nSeq * INF_SOFTMAX_SLICES * 2);
    b.NormState = (int8_t *)take((size_t)nSeq * d.dim);
    b.NormRelu = (int8_t *)take((size_t)nSeq * d.relu_dim);
    b.Qk8 = (int8_t *)take((size_t)nSeq * hs);
    b.K8 = (int8_t *)take((size_t)nSeq * hs);
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
    TSA_REQUIRE(d.head_count > 0 && d.relu_dim > 0 && d.relu_dim % d.head_count == 0 && d.relu_dim % GEMM_KB == 0,
        "%s: relu_dim %d must be a multiple of head_count %d and of %d", fn, d.relu_dim, d.head_count, GEMM_KB);
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

    auto norm = [&](const float *src, int n, int groupSize, int8_t *dst, bool relu) {
        const int warps = nSeq * (n / groupSize);
        InferNormKernel<<<(warps * 32 + 255) / 256, 256, 0, stream>>>(src, n, groupSize, nSeq, dst, relu ? 1 : 0);
        return CheckCuda(cudaGetLastError(), "inference normalise launch");
    };
    auto ptr2d = [](void *data, int strideBytes, int xs, int ys) {
        tsa_ptr2d p = {data, strideBytes, xs, ys};
        return p;
    };

    InferEmbedKernel<<<nSeq, 256, 0, stream>>>(labels, labelsPerSeq, d.label_count, model->label_embed, model->label_embed_scale, dim, b.State, statusWord);
    rc = CheckCuda(cudaGetLastError(), "inference embedding launch");
    if (rc == TSA_OK) {
        // the state's int8 form; afterwards the matrix products that update the state renew it in their epilogues
        rc = norm(b.State, dim, INF_NORM_TILE, b.NormState, false);
    }
    for (int l = 0; l < d.layer_count && rc == TSA_OK; ++l) {
        const tsa_infer_layer &layer = model->layers[l];
        TSA_REQUIRE(layer.qk && layer.qv && layer.k && layer.v && layer.combiner && layer.expand && layer.contract && layerSeqs[l],
            "tsa_infer_step: layer %d has a null matrix or cache", l);
        int *lens = ctxLens + (size_t)l * nSeq;
        TGemvJob proj[4] = {{layer.qk, b.Proj, hs}, {layer.qv, b.Proj + hs, hs}, {layer.k, b.Proj + 2 * hs, hs}, {layer.v, b.Proj + 3 * hs, hs}};
        rc = LaunchGemv(false, proj, 4, b.NormState, dim, nSeq, 4 * hs, 0.0f, nullptr, statusWord, stream);
        if (rc != TSA_OK) {
            break;
        }
        // same association as cpu_infer.cpp:504: qvScale *= (QVScale * VEC_SCALE) * dotScale(dim)
        const float qvMult = layer.qv_scale * INF_VEC_SCALE * sqrtf(1.0f / dim);
        dim3 gridR((4 * H + 3) / 4, nSeq);
        if (D == 64) {
            InferRopeNormKernel<64><<<gridR, 128, 0, stream>>>(b.Proj, model->rope, model->rope_len, lens, nSeq, H, qvMult, b.Qk8, b.K8, layerSeqs[l], capacity,
                statusWord);
        } else {
            InferRopeNormKernel<128><<<gridR, 128, 0, stream>>>(b.Proj, model->rope, model->rope_len, lens, nSeq, H, qvMult, b.Qk8, b.K8, layerSeqs[l], capacity,
                statusWord);
        }
        rc = CheckCuda(cudaGetLastError(), "inference rope launch");
        if (rc != TSA_OK) {
            break;
        }
        tsa_ptr2d none = {nullptr, 0, 0, 0};
        // attention; its merge kernel also forms the combiner input kv = int8(k[z ^ blk] * val[z])
        rc = DecodeWithKvProduct(&cfg, layerSeqs[l], lens, nSeq, maxCtx + 1, ptr2d(b.Qk8, hs, hs, nSeq), none, layer.attention_width, layer.alibi_slope,
            ptr2d(b.Val, hs * 4, hs, nSeq), H, b.DecodeWs, b.DecodeWsBytes, statusWord, streamArg, b.K8, b.Kv8, 1);
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob comb[1] = {{layer.combiner, b.State, dim}};
        rc = LaunchGemv(true, comb, 1, b.Kv8, hs * 4, nSeq, dim, layer.combiner_scale * INF_VEC_SCALE * sqrtf(1.0f / (hs * 4)), b.NormState,
            statusWord, stream);
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob expand[1] = {{layer.expand, b.Relu, d.relu_dim}};
        if (d.relu_dim / H == GEMM_M) {
            // 128-wide relu heads coincide with the product's row tiles: normalise + relu in its epilogue
            rc = LaunchGemv(false, expand, 1, b.NormState, dim, nSeq, d.relu_dim, 0.0f, b.NormRelu, statusWord, stream, true);
        } else {
            rc = LaunchGemv(false, expand, 1, b.NormState, dim, nSeq, d.relu_dim, 0.0f, nullptr, statusWord, stream);
            if (rc == TSA_OK) {
                rc = norm(b.Relu, d.relu_dim, d.relu_dim / H, b.NormRelu, true);
            }
        }
        if (rc != TSA_OK) {
            break;
        }
        TGemvJob contract[1] = {{layer.contract, b.State, dim}};
        rc = LaunchGemv(true, contract, 1, b.NormRelu, d.relu_dim, nSeq, dim, layer.contract_scale * INF_VEC_SCALE * sqrtf(1.0f / d.relu_dim), b.NormState,
            statusWord, stream);
    }
    if (rc != TSA_OK) {
        return rc;
    }
    if (d.layer_count > 0) {
        InferCountKernel<<<(d.layer_count * nSeq + 255) / 256, 256, 0, stream>>>(ctxLens, d.layer_count * nSeq);
        rc = CheckCuda(cudaGetLastError(), "inference count launch");
        if (rc != TSA_OK) {
            return rc;
        }
    }
    if (prediction || logits) {
        float *lg = logits ? logits : b.Logits;
        TGemvJob fin[1] = {{model->final_layer, lg, d.vocab_size}};
        rc = LaunchGemv(false, fin, 1, b.NormState, dim, nSeq, d.vocab_size, 0.0f, nullptr, statusWord, stream);
        if (rc != TSA_OK) {
            return rc;
        }
        if (prediction) {
            // CalcDotScale(dim) * CalcFinalLayerMult() * FinalLayerScale * VEC_SCALE (cpu_infer.cpp:555)
            const float finalScale = sqrtf(1.0f / dim) * (1.0f / 0.693147f) * model->final_layer_scale * INF_VEC_SCALE;
            dim3 gridS(INF_SOFTMAX_SLICES, nSeq);
            InferSoftmaxPartKernel<<<gridS, 256, 0, stream>>>(lg, model->bias, finalScale, d.vocab_size, b.SoftmaxPart);
            InferSoftmaxKernel<<<gridS, 256, 0, stream>>>(lg, model->bias, finalScale, d.vocab_size, b.SoftmaxPart, prediction);
            rc = CheckCuda(cudaGetLastError(), "inference softmax launch");
        }
    }
    return rc;
}
