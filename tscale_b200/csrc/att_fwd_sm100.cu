// Quantized attention forward for sm_100a: persistent, warp-specialised CTAs around tcgen05 MMA with accumulators in
// tensor memory, a TMA loader warp that runs ahead across work items, and a one-thread-per-row base-2 softmax.
//
// Replaces Fp8Att (code/gpt/compute/gpt_att_fp8.cuh:43-248) and the int8 QK^T variant of Fp16Att
// (gpt_att_fp16.cuh:121-318) of the reference:
//   S = Q K^T          kind::f8f6f4 (e4m3 x e4m3 -> f32) or kind::i8 (s8 x s8 -> s32, exact), 128 x 128 x D
//   z = S * sq_i * sk_j * c - slope * (i - j), masked by the row's span            (gpt_att_fp8.cuh:137-147)
//   m = integer-valued running reference of the row maximum, so that rescale factors are powers of two
//                                                                                    (gpt_att_fp8.cuh:163-164)
//   P = e4m3(2^(z - m) * 128 * sv_j / svRef); O += P V   kind::f8f6f4, A = P from tensor memory,
//                                                         B = V tile as an MN-major operand (no transposed copy)
//   out = O * (svRef / 128) / (2^-m + sum 2^(z - m));  sumWeightLog = m + log2(...)   (gpt_att_fp8.cuh:225-245)
//
// Work item = one head x 128 query rows (two 64-row span blocks).  A CTA takes items from a counter (late rows
// first, as they are the long ones under a causal mask) until none is left; two CTAs share an SM (256 of the 512
// tensor-memory columns each), so one CTA's softmax runs under the other's MMAs.
//
// Warp roles (192 threads):
//   warps 0-3  softmax: thread t owns query row t of the item = tensor-memory lane t.  It reads the 128 scores of a
//              key tile 16 columns at a time (the next chunk's tcgen05.ld is in flight while the current one is being
//              worked on), scales them and exponentiates once against the reference m it already holds.  Only when
//              a score exceeds m by more than the e4m3 headroom (weights up to 2^8.75 < 448) does the warp take the
//              slow path: raise m and shrink O, the sum and the tile's weights written so far.
//              Tiles the span mask cuts through add a second e4m3 residual term (P split into
//              e4m3(P) + e4m3(P - e4m3(P)), two MMAs), which removes the 3-bit-mantissa rounding where it is not
//              averaged out over many keys (rows with few keys see only such tiles).
//   warp 4     lane 0 issues every MMA: S = Q K^T, then, once the softmax threads have written P over S, O += P V.
//   warp 5     loader: reads the item's span groups and query scales, publishes one "round" record per span round
//              in shared memory (per-row spans, tile range), and streams Q, K, V tiles (TMA) and the key / value scale
//              rows (bulk copies) through shared-memory rings, up to a full ring ahead of the consumers and across
//              item boundaries, so DRAM latency of short items (window layers) is hidden.
// Tensor memory: columns [0,128) S (f32 / s32); the e4m3 weights of each 32-key block overwrite the first 8 (16 with
// the residual) of the block's own 32 score columns;
// columns [128, 128 + D) O (f32).
// Every barrier wait is bounded; when one runs out the kernel records a code in *statusWord, all roles stop at their
// next wait, outstanding copies are drained, tensor memory is freed and the kernel returns.
#include "att_internal.cuh"
#include "att_sm100_common.cuh"

namespace tsa {

using namespace sm100;

constexpr int FW_SOFTMAX_THREADS = 128;
constexpr int FW_MMA_WARP = 4;
constexpr int FW_LOAD_WARP = 5;
constexpr int FW_COPY_WARP = 6; // forwards finished output rows to the further destinations (kernels built with FORWARD only)
constexpr int FW_THREADS = 192;
constexpr int FW_THREADS_FORWARD = 224;
constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t TMEM_O_COL = 128;
constexpr int ROUND_SLOTS = 4;
constexpr int Q_SLOTS = 2;
// a weight is 2^t with t = z - m + 7; e4m3 holds up to 448 = 2^8.8, so t may reach 8.75 before m has to move
constexpr float P_HEADROOM = 8.75f;

enum { RF_FIRST = 1, RF_LAST = 2, RF_END = 4 };

struct TFwdParams {
    int HeadCount;
    int HeadGroup;    // heads whose work items are handed out together (1 .. HeadCount)
    int OutRows;      // rows of out that may be written
    int KeyRows;      // rows of K / V
    int LenAttTiles;  // number of 64-row span blocks
    int QTiles;       // number of 128-row query tiles
    int TotalItems;   // QTiles * HeadCount
    int *Counter;     // work-item counter, zero at launch
    const tsa_span_group *Spans;
    const int *SpanPtr;
    P2D<float> QScale, KScale, VScale;
    const float *VRef; // per head max of VScale (workspace), null without VScale
    int ScaleBulk;     // key / value scale rows may be fetched with 16-byte bulk copies
    P2D<char> Out;
    P2D<char> OutCopy[TSA_MAX_OUT_COPIES]; // further destinations of the output rows (other GPUs' buffers among them)
    int OutCopies;
    int WideStores;   // every destination's rows are 32-byte aligned
    // the consumer of the output, formed in the epilogue of kernels built with KV (null KvOut: none):
    // kv[t][head * 4 D + blk * D + z] = KvK[t][head * D + (z ^ blk)] * out[t][head * D + z] * KvMult, all bf16
    P2D<char> KvK, KvOut;
    float KvMult;
    int KvWide;       // rows of kv are 32-byte aligned
    P2D<float> Lse;
    const float *GlobalScale;
    float C;
    float QkVecScale, VVecScale;
    float Slope;
    int OutDtype;
    int *Status;
    // parity hook: raw s32 scores of one tile as this kernel read them from tensor memory (null in production)
    int32_t *DumpScores;
    int DumpHead, DumpQTile, DumpTile;
    // self-test of the failure path: bound of every barrier wait in clock cycles (about a second in production) and the
    // index, in a CTA's own tile sequence, of a key tile whose copy the loader requests but never issues (-1: none)
    long long WaitCycles;
    int WithholdTile;
};

// one span round of a work item, published by the loader
struct TFwdRound {
    int SpanS[TILE_M];   // inclusive key span of each row in this round, clipped to the key range (empty: 1, 0)
    int SpanF[TILE_M];
    float Sq[TILE_M];    // query scale of each row (0 for rows past the end)
    int J0;              // first key tile of the round (multiple of 128)
    int NTiles;
    int Flags;           // RF_*
    int QTile, Head, QSlot;
    int FullLo, FullHi;  // key tiles inside [FullLo, FullHi] are attended in full by every row
};

struct TFwdAux {
    float Sk[TILE_N];    // key scale of each column of the tile
    float Sv[TILE_N];    // value scale times the head's power-of-two normaliser
};

struct TFwdMisc {
    uint64_t QFull[Q_SLOTS], QEmpty[Q_SLOTS];
    uint64_t KvFull[4], KvEmpty[4];
    uint64_t RFull[ROUND_SLOTS], REmpty[ROUND_SLOTS];
    // a key tile is handed back and forth in two halves of 64 keys, so that the MMAs of one half (O += P V, then the next
    // tile's S = Q K^T into the columns just freed) run while the softmax threads work on the other half
    uint64_t BarS[2];    // MMA -> softmax: this half of S is ready
    uint64_t BarP[2];    // softmax -> MMA: this half of P is written, 128 arrivals
    uint64_t BarOFull;   // MMA -> softmax: the item's last PV has retired, O is final (its own barrier: the S barrier
                         // could otherwise run two phases ahead of the softmax threads across an item boundary)
    uint32_t TmemBase;
    int Abort;           // a bounded wait ran out somewhere in the CTA
    float Al[TILE_N];    // ALiBi term slope * column
    // softmax threads -> forwarding warp: the rows of an item are in the local output (ring of COPY_SLOTS records)
    uint64_t CopyFull[4], CopyEmpty[4];
    int CopyRow0[4], CopyHead[4];
};
constexpr int COPY_SLOTS = 4;

template <int D, bool V_I8>
struct TFwdSmem {
    static constexpr int STAGES = (D == 64) ? (V_I8 ? 3 : 4) : 2;
    static constexpr int NV = V_I8 ? 2 : 1; // value tiles per stage (int8 values come as two e4m3 planes)
    static constexpr int TILE_BYTES = 128 * D;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_SLOTS * TILE_BYTES;
    static constexpr int V_OFF = K_OFF + STAGES * TILE_BYTES;
    static constexpr int AUX_OFF = V_OFF + STAGES * NV * TILE_BYTES;
    static constexpr int ROUND_OFF = AUX_OFF + STAGES * (int)sizeof(TFwdAux);
    static constexpr int MISC_OFF = ROUND_OFF + ROUND_SLOTS * (int)sizeof(TFwdRound);
    static constexpr int TOTAL = MISC_OFF + (int)sizeof(TFwdMisc) + 1024; // + alignment slack
};

// tcgen05.wait::ld that names the registers an earlier tcgen05.ld fills, so that no use of them moves above the wait
__device__ __forceinline__ void TmemWaitLdRegs(uint32_t *r)
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}

__device__ __forceinline__ void TmemWaitLdRegs16(uint32_t *r)
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
                 : "memory");
}

// 2^x for a pair on the FMA / ALU pipes instead of the special-function unit: x = n + r with n = round(x),
// |r| <= 0.5, 2^r by a cubic (relative error 7.5e-5, far below the e4m3 rounding of the weights), n added to the
// exponent field.  x is clamped at -120 so the exponent cannot wrap; such weights are zero after the e4m3 pack.
__device__ __forceinline__ float2 PolyExp2Pair(float2 x)
{
    const float kMagic = 12582912.0f; // 1.5 * 2^23: the sum's low mantissa bits hold round(x)
    x.x = fmaxf(x.x, -120.0f);
    x.y = fmaxf(x.y, -120.0f);
    const float2 magic2 = make_float2(kMagic, kMagic);
    float2 y = __fadd2_rn(x, magic2);
    float2 r = __fadd2_rn(x, __fadd2_rn(make_float2(kMagic, kMagic), make_float2(-y.x, -y.y)));
    float2 p = __ffma2_rn(r, make_float2(0.0551716685f, 0.0551716685f), make_float2(0.242611125f, 0.242611125f));
    p = __ffma2_rn(p, r, make_float2(0.693260968f, 0.693260968f));
    p = __ffma2_rn(p, r, make_float2(0.999928057f, 0.999928057f));
    // the low 9 bits of the magic constant's pattern are zero, so (bits(y) << 23) is round(x) << 23
    return make_float2(__uint_as_float(__float_as_uint(p.x) + (__float_as_uint(y.x) << 23)),
        __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(y.y) << 23)));
}

// Slow path of the softmax: the row's reference moves up by d whole units, so what has been accumulated shrinks by
// alpha = 2^-d: the O accumulator (D columns) and this tile's e4m3 weights that are already in tensor memory.  The
// weights of the 32-key block b sit in columns [32b, 32b + 8) and their residuals in [32b + 8, 32b + 16);
// quads [firstQuad, firstQuad + nQuads) are the 4-column (16-key) groups written and not yet handed to the MMA.  All lanes of the warp execute the
// tensor-memory accesses; a lane whose row needs no change passes alpha = 1.  Kept out of line and in small pieces:
// it is rare, and inlined it costs the common path registers.
template <int D>
__device__ __noinline__ void ShrinkAccumulated(uint32_t tLane, float alpha, int hasO, int firstQuad, int nQuads, int withResidual)
{
    TmemWaitSt(); // the weights stored so far have landed
    if (hasO) {
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 8) {
            uint32_t o[8];
            TmemLd8(tLane + TMEM_O_COL + c0, o);
            TmemWaitLd();
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            }
            TmemStN<8>(tLane + TMEM_O_COL + c0, o);
        }
    }
    const __half2 ah = __float2half2_rn(alpha);
    const uint32_t ah2 = *reinterpret_cast<const uint32_t *>(&ah);
#pragma unroll 1
    for (int q = firstQuad; q < firstQuad + nQuads; ++q) {
#pragma unroll 1
        for (int part = 0; part < (withResidual ? 2 : 1); ++part) {
            const uint32_t col = 32 * (q >> 1) + 4 * (q & 1) + 8 * part;
#pragma unroll 1
            for (int k = 0; k < 4; k += 2) {
                uint32_t w0, w1;
                TmemLd2(tLane + col + k, w0, w1);
                TmemWaitLd();
                w0 = ScaleE4M3x4(w0, ah2);
                w1 = ScaleE4M3x4(w1, ah2);
                TmemSt2(tLane + col + k, w0, w1);
            }
        }
    }
    TmemWaitSt();
}

// e with 2^(e-1) < x <= 2^e for a positive float (clamped below so that 2^-e stays finite)
__device__ __forceinline__ int ValueScaleExponent(float x)
{
    const int bits = __float_as_int(x);
    const int e = ((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffff) ? 1 : 0);
    return max(e, -100);
}

// pause between barrier polls, in nanoseconds, of the MMA-issuing thread and of the softmax threads
#ifndef TSA_FWD_SLEEP_MMA
#define TSA_FWD_SLEEP_MMA 20
#endif
#ifndef TSA_FWD_SLEEP_SOFTMAX
#define TSA_FWD_SLEEP_SOFTMAX 40
#endif

// number of register pairs out of every 8 whose exponentials go to the polynomial (0 = all on the SFU)
#ifndef TSA_FWD_POLY_PAIRS
#define TSA_FWD_POLY_PAIRS 0
#endif

// V_I8: the values are int8.  They reach the tensor cores exactly, as the sum of two e4m3 planes a pre-pass writes
// (v = 16 * floor(v / 16) + (v mod 16): multiples of 16 up to 128 in magnitude and integers 0..15 are all e4m3 numbers),
// so every O += P V becomes two MMAs on the same weights; every tile also carries the weights' e4m3 residual term, which
// brings the result within 1e-3 of the reference's fp32 accumulation (the reference's int8 mode keeps its weights in
// half precision, gpt_att_fp16.cuh:121-318).
// FORWARD: the kernel carries the warp that forwards output rows to two or more further destinations (a seventh warp;
// built as its own kernel so that the usual launch keeps its 192 threads and register allocation)
// KV: the epilogue also forms the consumer's input (the reference's KVProduct) from the row it has just rounded to bf16.
// Measured against the two launches it replaces (attention, then the stand-alone product, which streams at 0.94 of the copy
// bandwidth): equal on a full-causal layer of 16 x 4096 x 12 x 64 (0.941 against 0.938 ms), slower on the window-64 layer
// (0.231 against 0.219 ms) and on 32768 x 16 x 128 (3.95 against 3.86 ms).  A kernel that carries this code runs its hot
// loop 6-7 % slower even when none of the consumer's memory accesses execute, and the same holds for the two other forms
// that were built: the products as a pass of their own that reads the stored row back from L2 (same register count as the
// plain kernel; 0.290 / 0.949 / 3.99 ms) and a seventh warp that takes finished blocks from L2 (0.271 / 1.075 / 4.00 ms).
template <int D, bool QK_I8, bool HAS_VSCALE, bool HAS_ALIBI, bool V_I8, bool FORWARD = false, bool KV = false>
__global__ void __launch_bounds__(FORWARD ? FW_THREADS_FORWARD : FW_THREADS, 2) FwdSm100Kernel(const __grid_constant__ CUtensorMap tmQ,
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmV2,
    TFwdParams p)
{
    using SM = TFwdSmem<D, V_I8>;
    constexpr int NV = SM::NV;
    constexpr int STAGES = SM::STAGES;
    constexpr int SWZ = (D == 128) ? 128 : 64;
    constexpr uint32_t GROUP_BYTES = 8 * D; // 8 rows of a tile
    constexpr uint32_t IDESC_QK = QK_I8 ? MakeInstrDesc(2, 1, 1, 0, 0, TILE_M, TILE_N) : MakeInstrDesc(1, 0, 0, 0, 0, TILE_M, TILE_N);
    constexpr uint32_t IDESC_PV = MakeInstrDesc(1, 0, 0, 0, 1, TILE_M, D);

    extern __shared__ __align__(1024) uint8_t smem[]; // tiles need 1024-byte alignment for the 128 B swizzle
    uint8_t *sQ = smem + SM::Q_OFF;
    uint8_t *sK = smem + SM::K_OFF;
    uint8_t *sV = smem + SM::V_OFF;
    TFwdAux *aux = reinterpret_cast<TFwdAux *>(smem + SM::AUX_OFF);
    TFwdRound *rounds = reinterpret_cast<TFwdRound *>(smem + SM::ROUND_OFF);
    TFwdMisc &misc = *reinterpret_cast<TFwdMisc *>(smem + SM::MISC_OFF);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if ((SmemAddr(smem) & 1023u) != 0) {
        // the launch did not honour the alignment: report instead of computing on mis-swizzled tiles
        if (tid == 0 && p.Status) {
            atomicOr(p.Status, kDevBadSpan);
        }
        return;
    }
    if (tid == 0) {
        for (int s = 0; s < Q_SLOTS; ++s) {
            MbarInit(&misc.QFull[s], 1);
            MbarInit(&misc.QEmpty[s], 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            MbarInit(&misc.KvFull[s], 2); // the TMA issue (with the byte count) and the loader's own staging of the scales
            MbarInit(&misc.KvEmpty[s], 1);
        }
        for (int s = 0; s < ROUND_SLOTS; ++s) {
            MbarInit(&misc.RFull[s], 1);
            MbarInit(&misc.REmpty[s], FW_SOFTMAX_THREADS + 1);
        }
        for (int h = 0; h < 2; ++h) {
            MbarInit(&misc.BarS[h], 1);
            MbarInit(&misc.BarP[h], FW_SOFTMAX_THREADS);
        }
        MbarInit(&misc.BarOFull, 1);
        for (int s = 0; s < COPY_SLOTS; ++s) {
            MbarInit(&misc.CopyFull[s], FW_SOFTMAX_THREADS);
            MbarInit(&misc.CopyEmpty[s], 1);
        }
        misc.Abort = 0;
        FenceBarrierInit();
    }
    if (warp == FW_MMA_WARP) {
        TmemAlloc(&misc.TmemBase, TMEM_COLS);
        TmemRelinquish();
    }
    if (tid < TILE_N) {
        misc.Al[tid] = p.Slope * (float)tid;
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;
    const int *abortFlag = &misc.Abort;
    auto fail = [&](int code) {
        *(volatile int *)&misc.Abort = 1;
        if (p.Status) {
            atomicOr(p.Status, code);
        }
    };

    if (warp == FW_LOAD_WARP) {
        // ------------------------------------------------------------------------------------ loader warp
        if (lane == 0) {
            PrefetchTensorMap(&tmQ);
            PrefetchTensorMap(&tmK);
            PrefetchTensorMap(&tmV);
            if (V_I8) {
                PrefetchTensorMap(&tmV2);
            }
        }
        int kvCount = 0, qCount = 0, rCount = 0;
        bool failed = false;
        int item = 0;
        if (lane == 0) {
            item = atomicAdd(p.Counter, 1);
        }
        item = __shfl_sync(0xffffffffu, item, 0);
        // waits of the whole warp on one barrier: every lane polls, all get the same answer
        auto waitAll = [&](uint64_t *bar, uint32_t parity, int code) {
            bool ok = WaitBarSleep<200>(bar, parity, abortFlag, p.WaitCycles);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok && !failed) {
                failed = true;
                if (lane == 0) {
                    fail(code);
                }
            }
            return ok;
        };
        while (!failed) {
            const bool end = item >= p.TotalItems;
            int nextItem = 0;
            if (!end && lane == 0) {
                nextItem = atomicAdd(p.Counter, 1); // in flight while this item is set up
            }
            // Order of the work items: heads in groups of p.HeadGroup, inside a group late (long) rows first with the group's
            // heads side by side.  The CTAs that run at the same time then read the keys and values of that many heads; the
            // host sizes the group so that these stay L2-resident (with everything of every head in flight at once the
            // four-fragment long-context batch ran 3.5 % slower, with groups smaller than needed shorter batches 2-8 % slower).
            // The launch still ends on short items.
            const int groupItems = p.QTiles * p.HeadGroup;
            const int grp = item / groupItems, rem = item - grp * groupItems;
            const int groupHeads = min(p.HeadGroup, p.HeadCount - grp * p.HeadGroup);
            const int qTile = end ? 0 : p.QTiles - 1 - rem / groupHeads;
            const int head = end ? 0 : grp * p.HeadGroup + rem % groupHeads;
            const int b0 = 2 * qTile;
            int p0 = 0, n0 = 0, p1 = 0, n1 = 0, nRounds = 0;
            int qSlot = qCount % Q_SLOTS;
            float sqv[4] = {0, 0, 0, 0};
            float kMul = 0; // power of two that brings the head's largest value scale into (1/2, 1]
            if (!end) {
                if (HAS_VSCALE) {
                    const float vRef = p.VRef[head];
                    if (vRef > 0) {
                        kMul = __int_as_float((127 - ValueScaleExponent(vRef)) << 23);
                    }
                }
                int pv = 0;
                if (lane < 3 && b0 + lane <= p.LenAttTiles) {
                    pv = p.SpanPtr[b0 + lane];
                }
                const int a = __shfl_sync(0xffffffffu, pv, 0), b = __shfl_sync(0xffffffffu, pv, 1), c = __shfl_sync(0xffffffffu, pv, 2);
                if (b0 < p.LenAttTiles) {
                    p0 = a;
                    n0 = b - a;
                }
                if (b0 + 1 < p.LenAttTiles) {
                    p1 = b;
                    n1 = c - b;
                }
                nRounds = max(n0, n1);
                // the query tile goes out first
                if (!waitAll(&misc.QEmpty[qSlot], ((qCount / Q_SLOTS) & 1) ^ 1, kDevTimeoutTma)) {
                    break;
                }
                if (lane == 0) {
                    MbarExpectTx(&misc.QFull[qSlot], SM::TILE_BYTES);
                    TmaLoad2D(sQ + qSlot * SM::TILE_BYTES, &tmQ, head * D, qTile * TILE_M, &misc.QFull[qSlot]);
                }
                ++qCount;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int row = qTile * TILE_M + lane + 32 * k;
                    if (row < p.OutRows) {
                        sqv[k] = p.QScale.Valid() ? p.QScale.Row(head)[row] : p.QkVecScale;
                    }
                }
            }
            // tile range of a round from the two blocks' group headers
            auto roundRange = [&](int r, int &lo, int &hi) {
                lo = 0x7fffffff;
                hi = -1;
                if (r < n0) {
                    lo = min(lo, p.Spans[p0 + r].Start);
                    hi = max(hi, p.Spans[p0 + r].Finish);
                }
                if (r < n1) {
                    lo = min(lo, p.Spans[p1 + r].Start);
                    hi = max(hi, p.Spans[p1 + r].Finish);
                }
                lo = max(lo, 0) & ~(TILE_N - 1);
                hi = min(hi, p.KeyRows - 1) & ~(TILE_N - 1);
            };
            int firstRound = -1, lastRound = -1;
            for (int r = 0; r < nRounds; ++r) {
                int lo, hi;
                roundRange(r, lo, hi);
                if (lo <= hi) {
                    if (firstRound < 0) {
                        firstRound = r;
                    }
                    lastRound = r;
                }
            }
            // an item without key tiles (or the end marker) still gets one record
            const int rBegin = firstRound < 0 ? 0 : firstRound, rEnd = firstRound < 0 ? 0 : lastRound;
            for (int r = rBegin; r <= rEnd && !failed; ++r) {
                int lo = 0, hi = -1;
                if (firstRound >= 0) {
                    roundRange(r, lo, hi);
                    if (lo > hi) {
                        continue;
                    }
                }
                int ss[4], sf[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    ss[k] = 1;
                    sf[k] = 0;
                }
                if (firstRound >= 0) {
                    if (r < n0) {
                        const tsa_span_group *g = p.Spans + p0 + r;
                        ss[0] = g->SpanStart[lane];
                        sf[0] = g->SpanFinish[lane];
                        ss[1] = g->SpanStart[lane + 32];
                        sf[1] = g->SpanFinish[lane + 32];
                    }
                    if (r < n1) {
                        const tsa_span_group *g = p.Spans + p1 + r;
                        ss[2] = g->SpanStart[lane];
                        sf[2] = g->SpanFinish[lane];
                        ss[3] = g->SpanStart[lane + 32];
                        sf[3] = g->SpanFinish[lane + 32];
                    }
                }
                int mxS = -0x7fffffff, mnF = 0x7fffffff;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    ss[k] = max(ss[k], 0);
                    sf[k] = min(sf[k], p.KeyRows - 1);
                    if (ss[k] > sf[k]) {
                        ss[k] = 1;
                        sf[k] = 0;
                    }
                    mxS = max(mxS, ss[k]);
                    mnF = min(mnF, sf[k]);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    mxS = max(mxS, __shfl_xor_sync(0xffffffffu, mxS, o));
                    mnF = min(mnF, __shfl_xor_sync(0xffffffffu, mnF, o));
                }
                const int rSlot = rCount % ROUND_SLOTS;
                if (!waitAll(&misc.REmpty[rSlot], ((rCount / ROUND_SLOTS) & 1) ^ 1, kDevTimeoutMma)) {
                    break;
                }
                TFwdRound &rd = rounds[rSlot];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    rd.SpanS[lane + 32 * k] = ss[k];
                    rd.SpanF[lane + 32 * k] = sf[k];
                    rd.Sq[lane + 32 * k] = sqv[k];
                }
                const int nTiles = (lo <= hi) ? (hi - lo) / TILE_N + 1 : 0;
                if (lane == 0) {
                    rd.J0 = lo;
                    rd.NTiles = nTiles;
                    rd.Flags = end ? RF_END : ((r == rBegin ? RF_FIRST : 0) | (r == rEnd ? RF_LAST : 0));
                    rd.QTile = qTile;
                    rd.Head = head;
                    rd.QSlot = qSlot;
                    rd.FullLo = mxS;
                    rd.FullHi = mnF;
                }
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&misc.RFull[rSlot]);
                }
                ++rCount;
                // the round's key / value tiles
                for (int t = 0; t < nTiles; ++t) {
                    const int j0 = lo + t * TILE_N;
                    const int slot = kvCount % STAGES;
                    const bool bulk = p.ScaleBulk && j0 + TILE_N <= p.KeyRows;
                    // the scale rows this warp stages itself are requested before the wait for the slot: value scales
                    // (multiplied by kMul on the way) always, key scales when a bulk copy cannot fetch them
                    float skv[4] = {0, 0, 0, 0}, svv[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int j = j0 + lane + 32 * k;
                        if (j < p.KeyRows) {
                            if (!bulk) {
                                skv[k] = p.KScale.Row(head)[j];
                            }
                            if (HAS_VSCALE) {
                                svv[k] = p.VScale.Row(head)[j];
                            }
                        }
                    }
                    if (!waitAll(&misc.KvEmpty[slot], ((kvCount / STAGES) & 1) ^ 1, kDevTimeoutMma)) {
                        break;
                    }
                    if (lane == 0) {
                        MbarExpectTx(&misc.KvFull[slot], (1 + NV) * SM::TILE_BYTES + (bulk ? TILE_N * 4 : 0));
                        if (kvCount != p.WithholdTile) { // self-test: the bytes of a withheld copy never arrive
                            TmaLoad2D(sK + slot * SM::TILE_BYTES, &tmK, head * D, j0, &misc.KvFull[slot]);
                        }
                        TmaLoad2D(sV + slot * NV * SM::TILE_BYTES, &tmV, head * D, j0, &misc.KvFull[slot]);
                        if (V_I8) {
                            TmaLoad2D(sV + (slot * NV + 1) * SM::TILE_BYTES, &tmV2, head * D, j0, &misc.KvFull[slot]);
                        }
                        if (bulk) {
                            BulkLoad(aux[slot].Sk, p.KScale.Row(head) + j0, TILE_N * 4, &misc.KvFull[slot]);
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (!bulk) {
                            aux[slot].Sk[lane + 32 * k] = skv[k];
                        }
                        if (HAS_VSCALE) {
                            aux[slot].Sv[lane + 32 * k] = svv[k] * kMul;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        MbarArrive(&misc.KvFull[slot]);
                    }
                    ++kvCount;
                }
            }
            if (end) {
                break;
            }
            item = __shfl_sync(0xffffffffu, nextItem, 0);
        }
        if (failed || *(volatile int *)&misc.Abort) {
            // drain copies that were requested but may never be consumed, so none lands after the CTA is gone
            for (int k = max(0, kvCount - STAGES); k < kvCount; ++k) {
                WaitBar(&misc.KvFull[k % STAGES], (k / STAGES) & 1, p.WaitCycles);
            }
            for (int k = max(0, qCount - Q_SLOTS); k < qCount; ++k) {
                WaitBar(&misc.QFull[k % Q_SLOTS], (k / Q_SLOTS) & 1, p.WaitCycles);
            }
        }
        __syncwarp();
    } else if (warp == FW_MMA_WARP) {
        // ------------------------------------------------------------------------------------ MMA warp
        // Software pipeline over the CTA's whole tile sequence: S(t+1) = Q K^T is issued directly behind O += P(t) V(t),
        // and everything tile t+1 needs (its round record, Q, K/V stage) is waited for before the wait for P(t), so that
        // between the softmax threads' "P written" and their next "S ready" lie only the two groups of MMA instructions.
        // The whole warp runs the loop and the waits; one elected lane (always the same one) issues, so descriptors and
        // addresses stay in uniform registers instead of being moved there per instruction.
        {
            const uint32_t sQa = SmemAddr(sQ), sKa = SmemAddr(sK), sVa = SmemAddr(sV);
            // descriptors without the tile's address: the address field (bits 0-13, in 16-byte units) is added per use
            const uint64_t descBase = MakeSmemDesc(0, 16, GROUP_BYTES, SWZ);
            int kvCount = 0, pCount = 0, rCount = 0, itemCount = 0, tilesInItem = 0;
            bool failed = false;
            // the tile whose QK^T has been issued and whose PV is still to come
            bool pending = false, pendAccum = false, pendMasked = false, pendLast = false;
            int pendSlot = 0, pendQSlot = 0;
            auto wait = [&](uint64_t *bar, uint32_t parity, int code) {
                if (__all_sync(0xffffffffu, WaitBarSleep<TSA_FWD_SLEEP_MMA>(bar, parity, abortFlag, p.WaitCycles))) {
                    return true;
                }
                if (!failed) {
                    failed = true;
                    if (lane == 0) {
                        fail(code);
                    }
                }
                return false;
            };
            constexpr uint32_t IDESC_QK_HALF = QK_I8 ? MakeInstrDesc(2, 1, 1, 0, 0, TILE_M, TILE_N / 2) : MakeInstrDesc(1, 0, 0, 0, 0, TILE_M, TILE_N / 2);
            // S = Q K^T for the keys [64h, 64h + 64) of a tile (elected lane)
            auto issueQKHalf = [&](int h, uint64_t qDesc, uint64_t kDesc) {
                MmaGroupSSCommit<D / 32, QK_I8>(tmem + h * 64, qDesc, kDesc + ((h * 64 * D) >> 4), IDESC_QK_HALF, &misc.BarS[h]);
            };
            // O += P V for half h of the pending tile, item-end signals behind the last (elected lane)
            auto issuePVHalf = [&](int h) {
                const uint64_t vDesc = descBase + ((sVa + pendSlot * NV * SM::TILE_BYTES) >> 4);
                MmaPairF8TS(tmem + TMEM_O_COL, tmem + h * 64, vDesc + ((h * 64 * D) >> 4), (32 * D) >> 4, IDESC_PV,
                    (pendAccum || h > 0) ? 1u : 0u, pendMasked);
                if (V_I8) {
                    MmaPairF8TS(tmem + TMEM_O_COL, tmem + h * 64, vDesc + ((SM::TILE_BYTES + h * 64 * D) >> 4), (32 * D) >> 4, IDESC_PV,
                        1u, pendMasked);
                }
                if (h == 1) {
                    MmaCommit(&misc.KvEmpty[pendSlot]);
                    if (pendLast) {
                        MmaCommit(&misc.BarOFull);
                        MmaCommit(&misc.QEmpty[pendQSlot]);
                    }
                }
            };
            // waits for half h of the pending tile's weights (whole warp)
            auto waitWeights = [&](int h) {
                if (!wait(&misc.BarP[h], pCount & 1, kDevTimeoutMma)) {
                    return false;
                }
                TcFenceAfter();
                return true;
            };
            auto retireHalf = [&](int h) {
                if (h == 1) {
                    ++pCount;
                    pending = false;
                }
            };
            while (!failed) {
                const int rSlot = rCount % ROUND_SLOTS;
                if (!wait(&misc.RFull[rSlot], (rCount / ROUND_SLOTS) & 1, kDevTimeoutTma)) {
                    break;
                }
                const volatile TFwdRound &rd = rounds[rSlot];
                const int j0r = rd.J0, nTiles = rd.NTiles, flags = rd.Flags, qSlot = rd.QSlot, fullLo = rd.FullLo, fullHi = rd.FullHi;
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&misc.REmpty[rSlot]);
                }
                ++rCount;
                if (flags & RF_END) {
                    break;
                }
                if (flags & RF_FIRST) {
                    tilesInItem = 0;
                    if (!wait(&misc.QFull[qSlot], (itemCount / Q_SLOTS) & 1, kDevTimeoutTma)) {
                        break;
                    }
                }
                const uint64_t qDesc = descBase + ((sQa + qSlot * SM::TILE_BYTES) >> 4);
                for (int t = 0; t < nTiles; ++t) {
                    const int j0 = j0r + t * TILE_N;
                    const int slot = kvCount % STAGES;
                    if (!wait(&misc.KvFull[slot], (kvCount / STAGES) & 1, kDevTimeoutTma)) {
                        break;
                    }
                    const uint64_t kDesc = descBase + ((sKa + slot * SM::TILE_BYTES) >> 4);
                    // O += P V of the previous tile's half h, then this tile's S into the columns that frees
                    if (pending) {
                        if (!waitWeights(0)) {
                            break;
                        }
                        if (ElectOne()) {
                            issuePVHalf(0);
                            issueQKHalf(0, qDesc, kDesc);
                        }
                        __syncwarp();
                        if (!waitWeights(1)) {
                            break;
                        }
                        if (ElectOne()) {
                            issuePVHalf(1);
                            issueQKHalf(1, qDesc, kDesc);
                        }
                        __syncwarp();
                        retireHalf(1);
                    } else {
                        TcFenceAfter();
                        if (ElectOne()) {
                            issueQKHalf(0, qDesc, kDesc);
                            issueQKHalf(1, qDesc, kDesc);
                        }
                        __syncwarp();
                    }
                    pending = true;
                    pendSlot = slot;
                    pendQSlot = qSlot;
                    pendAccum = tilesInItem > 0;
                    pendMasked = V_I8 || !(fullLo <= j0 && j0 + TILE_N - 1 <= fullHi);
                    pendLast = (flags & RF_LAST) && t == nTiles - 1;
                    ++kvCount;
                    ++tilesInItem;
                }
                if (failed) {
                    break;
                }
                if (flags & RF_LAST) {
                    if (tilesInItem == 0 && lane == 0) {
                        MbarArrive(&misc.QEmpty[qSlot]); // an item without key tiles: nothing was issued for it
                    }
                    ++itemCount;
                }
            }
            if (pending && !failed) {
                // the last tile: the commits that would follow the next tile's S stand in for it (a rescale in this tile's
                // second half waits on them to know that the first half's PV has retired)
                if (waitWeights(0)) {
                    if (ElectOne()) {
                        issuePVHalf(0);
                        MmaCommit(&misc.BarS[0]);
                    }
                    __syncwarp();
                    if (waitWeights(1)) {
                        if (ElectOne()) {
                            issuePVHalf(1);
                            MmaCommit(&misc.BarS[1]);
                        }
                        __syncwarp();
                        retireHalf(1);
                    }
                }
            }
        }
        __syncwarp();
    } else if (FORWARD && warp == FW_COPY_WARP) {
        // ------------------------------------------------------------------------------------ forwarding warp
        // The all-gather fused into the kernel: every finished item's rows go from the local output (still in L2) to the
        // further destinations, the other GPUs' buffers, 1 KB per instruction (whole 256-byte rows side by side), while the
        // softmax threads are already on their next item.  Stored by the softmax threads themselves, one row per thread, every
        // peer multiplied their store instructions (measured: slower than a separate NCCL all-gather from three peers on).
        if (FORWARD && p.OutCopies > 1) {
            const int esz = (p.OutDtype == TSA_F32) ? 4 : 2;
            const int rowBytes = D * esz;
            for (int n = 0;; ++n) {
                const int cs = n % COPY_SLOTS;
                if (!__all_sync(0xffffffffu, WaitBarSleep<100>(&misc.CopyFull[cs], (n / COPY_SLOTS) & 1, abortFlag, p.WaitCycles))) {
                    if (lane == 0) {
                        fail(kDevTimeoutMma);
                    }
                    break;
                }
                const int row0 = *(volatile int *)&misc.CopyRow0[cs], headC = *(volatile int *)&misc.CopyHead[cs];
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&misc.CopyEmpty[cs]);
                }
                if (headC < 0) {
                    break;
                }
                const int nRows = min(TILE_M, p.OutRows - row0);
                const size_t colOff = (size_t)headC * rowBytes;
                if (p.WideStores) {
                    const int chunks = rowBytes >> 5;
                    for (int id = lane; id < nRows * chunks; id += 32) {
                        const int rr = id / chunks, cc = id - rr * chunks;
                        const char *src = p.Out.Row(row0 + rr) + colOff + cc * 32;
                        const uint4 a = __ldcg(reinterpret_cast<const uint4 *>(src)), b = __ldcg(reinterpret_cast<const uint4 *>(src) + 1);
                        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll 1
                        for (int k = 0; k < p.OutCopies; ++k) {
                            StGlobal256(p.OutCopy[k].Row(row0 + rr) + colOff + cc * 32, w);
                        }
                    }
                } else {
                    const int chunks = rowBytes >> 4;
                    for (int id = lane; id < nRows * chunks; id += 32) {
                        const int rr = id / chunks, cc = id - rr * chunks;
                        const uint4 a = __ldcg(reinterpret_cast<const uint4 *>(p.Out.Row(row0 + rr) + colOff + cc * 16));
#pragma unroll 1
                        for (int k = 0; k < p.OutCopies; ++k) {
                            *reinterpret_cast<uint4 *>(p.OutCopy[k].Row(row0 + rr) + colOff + cc * 16) = a;
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------------------------ softmax warps
        const int r = tid; // row of the item's query tile = tensor-memory lane
        const uint32_t tLane = tmem + ((uint32_t)(warp * 32) << 16);
        const float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
        int rCount = 0, sCount = 0, kvCount = 0, oCount = 0;
        int pvEnabled = 0; // halves handed to the MMA so far = PV groups that have been or will be issued
        int tilesInItem = 0, row = 0, head = 0, qTile = 0;
        int copyCount = 0; // items handed to the forwarding warp
        bool rowOk = false, failed = false;
        float m = 0, rowMult = 0, invK = 0;
        float2 lacc2 = make_float2(0.0f, 0.0f); // 128 * sum of this row's weights
        auto wait = [&](uint64_t *bar, uint32_t parity, int code) {
            if (WaitBarSleep<TSA_FWD_SLEEP_SOFTMAX>(bar, parity, abortFlag, p.WaitCycles)) {
                return true;
            }
            if (!failed) {
                failed = true;
                fail(code);
            }
            return false;
        };
        // hands an item (or, with a negative head, the end of the work) to the forwarding warp: the record, a device-wide
        // fence behind this thread's output stores, one arrival per softmax thread
        auto postCopy = [&](int row0, int headOrEnd) {
            const int cs = copyCount % COPY_SLOTS;
            if (copyCount >= COPY_SLOTS && !wait(&misc.CopyEmpty[cs], ((copyCount / COPY_SLOTS) - 1) & 1, kDevTimeoutMma)) {
                return false;
            }
            if (tid == 0) {
                misc.CopyRow0[cs] = row0;
                misc.CopyHead[cs] = headOrEnd;
            }
            __threadfence();
            MbarArrive(&misc.CopyFull[cs]);
            ++copyCount;
            return true;
        };
        while (true) {
            const int rSlot = rCount % ROUND_SLOTS;
            if (!wait(&misc.RFull[rSlot], (rCount / ROUND_SLOTS) & 1, kDevTimeoutTma)) {
                break;
            }
            const TFwdRound &rd = rounds[rSlot];
            const int spanS = rd.SpanS[r], spanF = rd.SpanF[r];
            const float sq = rd.Sq[r];
            const int j0r = rd.J0, nTiles = rd.NTiles, flags = rd.Flags, fullLo = rd.FullLo, fullHi = rd.FullHi;
            const int rdQTile = rd.QTile, rdHead = rd.Head;
            MbarArrive(&misc.REmpty[rSlot]);
            ++rCount;
            if (flags & RF_END) {
                break;
            }
            if (flags & RF_FIRST) {
                qTile = rdQTile;
                head = rdHead;
                row = qTile * TILE_M + r;
                rowOk = row < p.OutRows;
                // a zero query scale would turn masked (-inf) scores into NaN; a tiny positive one keeps every logit at ~0
                rowMult = fmaxf(sq * p.C * g, 1e-30f);
                m = 0;
                lacc2 = make_float2(0.0f, 0.0f);
                tilesInItem = 0;
                if (KV && rowOk) {
                    // the row of combiner keys the epilogue will multiply with: on its way into L2 while the item is computed
                    const char *kp = p.KvK.Row(row) + (size_t)head * D * 2;
#pragma unroll
                    for (int o = 0; o < D * 2; o += 128) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(kp + o));
                    }
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(kp + D * 2 - 16));
                }
                if (HAS_VSCALE) {
                    // the loader stages sv_j * K with 1 / K = the power of two at or above the head's largest value scale,
                    // so the weights' e4m3 range is used whatever the scales' magnitude; O is in units of 1 / K
                    const float vRef = p.VRef[head];
                    invK = vRef > 0 ? __int_as_float((127 + ValueScaleExponent(vRef)) << 23) : 0.0f;
                }
            }
            const float2 rowMult2 = make_float2(rowMult, rowMult);
            for (int t = 0; t < nTiles; ++t) {
                const int j0 = j0r + t * TILE_N;
                const int slot = kvCount % STAGES;
                const bool masked = V_I8 || !(fullLo <= j0 && j0 + TILE_N - 1 <= fullHi);
                if (!wait(&misc.BarS[0], sCount & 1, kDevTimeoutMma)) {
                    break;
                }
                // the tile's scale rows arrived with K and V; this wait makes them visible to this thread
                if (!wait(&misc.KvFull[slot], (kvCount / STAGES) & 1, kDevTimeoutTma)) {
                    break;
                }
                TcFenceAfter();
                const float *skBuf = aux[slot].Sk;
                const float *svBuf = aux[slot].Sv;
                const float rowOff = HAS_ALIBI ? -p.Slope * (float)(row - j0) : 0.0f;
                const float headroom = P_HEADROOM;
                const bool hasO = tilesInItem > 0;
                // second half of S: ready long before it is needed (its MMAs were issued before this tile's first half was
                // even handed over), the wait is for the memory model
                auto waitSecondHalf = [&]() {
                    const bool ok = wait(&misc.BarS[1], sCount & 1, kDevTimeoutMma);
                    TcFenceAfter();
                    return ok;
                };
                // hands the finished half h of P to the MMA thread
                auto handOver = [&](int h) {
                    TmemWaitSt();
                    TcFenceBefore();
                    MbarArrive(&misc.BarP[h]);
                    ++pvEnabled;
                };

                if (QK_I8 && p.DumpScores && head == p.DumpHead && qTile == p.DumpQTile && tilesInItem == p.DumpTile) {
                    waitSecondHalf();
#pragma unroll 1
                    for (int c0 = 0; c0 < TILE_N; c0 += 32) {
                        uint32_t s[32];
                        TmemLd32(tLane + c0, s);
                        TmemWaitLdRegs(s);
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            p.DumpScores[r * TILE_N + c0 + c] = (int32_t)s[c];
                        }
                    }
                }

                // scaled logit offsets of a pair of columns: t = S * sk * rowMult (+ alibi) + eoff, eoff = rowOff - m + 7
                auto scalePair = [&](uint32_t s0, uint32_t s1, int col, float2 eoff2) {
                    float2 a = QK_I8 ? IntPairToFloat(s0, s1) : make_float2(__uint_as_float(s0), __uint_as_float(s1));
                    float2 x = __fmul2_rn(a, *reinterpret_cast<const float2 *>(skBuf + col));
                    if (HAS_ALIBI) {
                        x = __ffma2_rn(x, rowMult2, *reinterpret_cast<const float2 *>(misc.Al + col));
                        return __fadd2_rn(x, eoff2);
                    }
                    return __ffma2_rn(x, rowMult2, eoff2);
                };
                float eoff = rowOff - m + 7.0f;

                // One key tile in chunks of W columns: logits in place of the scores and their maximum, a vote whether the
                // row's reference has to move, then the weights.  The packed weights of the 32-key block b go to columns
                // [32b, 32b + 8) and their residuals to [32b + 8, 32b + 16): inside the block's own score columns, which are
                // in registers by then, so no store can hit scores that are still to be read.
                // Unmasked tiles: W = 16, the next chunk's tcgen05.ld in flight while this one is worked on.
                // Tiles the mask cuts through: W = 32, one buffer, residual term, chunks no row of the warp attends skipped.
                auto processTile = [&](auto maskedTag) {
                    constexpr bool MASKED = decltype(maskedTag)::value;
                    constexpr int W = MASKED ? 32 : 16;
                    int lsC = 0;
                    unsigned spanW = TILE_N - 1;
                    bool rowEmpty = false;
                    unsigned act = 0xf; // 32-column chunks some row of the warp attends
                    if (MASKED) {
                        const int ls = spanS - j0, lf = spanF - j0; // span in tile-local columns
                        lsC = max(ls, 0);
                        const int lfC = min(lf, TILE_N - 1);
                        rowEmpty = lsC > lfC;
                        spanW = rowEmpty ? 0u : (unsigned)(lfC - lsC);
                        act = 0;
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            if (__any_sync(0xffffffffu, !rowEmpty && lsC <= ch * 32 + 31 && lfC >= ch * 32)) {
                                act |= 1u << ch;
                            }
                        }
                    }
                    // the reference moves up by d whole units: everything accumulated so far shrinks by 2^-d, and the
                    // chunk's logits in s drop by d
                    auto raise = [&](float mxc, int storedQuads, uint32_t *s) {
                        const float d = (mxc > headroom) ? floorf(mxc - 7.0f) : 0.0f;
                        const float alpha = exp2f(-d);
                        // the chunk voted on is the next one to be stored: it lies in half storedQuads / 4, whose earlier
                        // quads are still this thread's; O holds something once a PV group of this item has been enabled,
                        // and may be touched once the last enabled group has retired
                        const int firstQuad = storedQuads & ~3;
                        const bool oLive = hasO || firstQuad > 0;
                        if (oLive && pvEnabled > 0) {
                            // the last PV group enabled must have retired: the S = Q K^T group issued right behind it has
                            // when its commit arrived (first half: the second half of this tile's S; second half: the
                            // first half of the next tile's S)
                            if (firstQuad == 0) {
                                wait(&misc.BarS[1], sCount & 1, kDevTimeoutMma);
                            } else {
                                wait(&misc.BarS[0], (sCount + 1) & 1, kDevTimeoutMma);
                            }
                            TcFenceAfter();
                        }
                        ShrinkAccumulated<D>(tLane, alpha, oLive ? 1 : 0, firstQuad, storedQuads - firstQuad, MASKED ? 1 : 0);
                        lacc2.x *= alpha;
                        lacc2.y *= alpha;
                        m += d;
                        eoff -= d;
#pragma unroll
                        for (int c = 0; c < W; ++c) {
                            s[c] = __float_as_uint(__uint_as_float(s[c]) - d);
                        }
                    };
                    // s: W scores of the columns from cb on; other: the buffer a tcgen05.ld may be filling meanwhile
                    auto chunk = [&](uint32_t *s, uint32_t *other, int cb, uint32_t *pk, uint32_t *pl) {
                        float mxc = -INFINITY;
                        {
                            const float2 eoff2 = make_float2(eoff, eoff);
#pragma unroll
                            for (int c = 0; c < W; c += 2) {
                                float2 tt = scalePair(s[c], s[c + 1], cb + c, eoff2);
                                if (MASKED) {
                                    // unsigned compare folds both bounds: lsC <= col <= lfC
                                    tt.x = ((unsigned)(cb + c - lsC) <= spanW) ? tt.x : -INFINITY;
                                    tt.y = ((unsigned)(cb + c + 1 - lsC) <= spanW) ? tt.y : -INFINITY;
                                }
                                mxc = Max3(mxc, tt.x, tt.y);
                                s[c] = __float_as_uint(tt.x);
                                s[c + 1] = __float_as_uint(tt.y);
                            }
                        }
                        if (MASKED && rowEmpty) {
                            mxc = -INFINITY; // spanW = 0 would otherwise let column lsC through
                        }
                        if (__any_sync(0xffffffffu, mxc > headroom)) {
                            if (!MASKED) {
                                TmemWaitLdRegs16(other); // no load is in flight across the out-of-line call
                            }
                            raise(mxc, cb >> 4, s);
                        }
                        // an empty row gets -inf so that every weight is 0 whatever the compare let through
                        const float kill = (MASKED && rowEmpty) ? -INFINITY : 0.0f;
#pragma unroll
                        for (int c = 0; c < W; c += 4) {
                            float2 e[2];
#pragma unroll
                            for (int k = 0; k < 2; ++k) {
                                const int cc = c + 2 * k;
                                float2 tt = make_float2(__uint_as_float(s[cc]), __uint_as_float(s[cc + 1]));
                                if (MASKED) {
                                    tt.x += kill;
                                    tt.y += kill;
                                }
                                float2 w;
                                if (!MASKED && ((cc >> 1) & 7) < TSA_FWD_POLY_PAIRS) {
                                    w = PolyExp2Pair(tt);
                                } else {
                                    w = make_float2(FastExp2(tt.x), FastExp2(tt.y));
                                }
                                lacc2 = __fadd2_rn(lacc2, w);
                                if (HAS_VSCALE) {
                                    e[k] = __fmul2_rn(w, *reinterpret_cast<const float2 *>(svBuf + cb + cc));
                                } else {
                                    e[k] = w;
                                }
                            }
                            const uint32_t hi4 = PackE4M3x4(e[0].x, e[0].y, e[1].x, e[1].y);
                            pk[c >> 2] = hi4;
                            if (MASKED) {
                                pl[c >> 2] = ResidualE4M3x2(e[0].x, e[0].y, hi4 & 0xffff) | (ResidualE4M3x2(e[1].x, e[1].y, hi4 >> 16) << 16);
                            }
                        }
                    };
                    if (MASKED) {
#pragma unroll 1
                        for (int ch = 0; ch < 4; ++ch) {
                            uint32_t s[32], pk[8], pl[8];
                            if (act & (1u << ch)) {
                                TmemLd32(tLane + ch * 32, s);
                                TmemWaitLdRegs(s);
                                chunk(s, s, ch * 32, pk, pl);
                            } else {
#pragma unroll
                                for (int k = 0; k < 8; ++k) {
                                    pk[k] = 0;
                                    pl[k] = 0;
                                }
                            }
                            TmemStN<8>(tLane + ch * 32, pk);
                            TmemStN<8>(tLane + ch * 32 + 8, pl);
                            if (ch == 1) {
                                handOver(0);
                                waitSecondHalf();
                            }
                        }
                    } else {
                        // Software pipeline over the 8 chunks, interleaved at the source level: in step c the exponentials
                        // of chunk c (special-function pipe) alternate with the scaling of chunk c + 1 (FMA pipe) inside one
                        // loop body, while chunk c + 2 is on its way from tensor memory; the vote on chunk c + 1 closes
                        // the step.  Raw scores of chunk k live in rawBuf[k & 1], logits in tBuf[k & 1].
                        uint32_t tBuf[2][16], rawBuf[2][16], pk[4];
                        float mxN = -INFINITY;
                        // c: chunk that becomes weights (even: buffers 0, odd: buffers 1).  A loop over pairs of steps: fully
                        // unrolled, the eight copies no longer fit the instruction cache and every head size got slower.
                        // MODE 0: chunks c + 1 and c + 2 exist; 1: only c + 1; 2: neither (the last step); 3: decided at run
                        // time, and the last step scales whatever the raw registers hold and ignores the result.  Head size
                        // 128 runs the loop over steps 0-5 in mode 0 and steps 6, 7 in modes 1, 2 (four copies of the step),
                        // head size 64 all eight steps in mode 3 (two copies): measured, each is the faster one for its size.
                        auto step = [&](auto modeTag, auto oddTag, int c) {
                            constexpr int MODE = decltype(modeTag)::value;
                            constexpr int ODD = decltype(oddTag)::value;
                            constexpr bool HAS_NEXT = MODE != 2;
                            const bool LOAD = MODE == 0 || (MODE == 3 && c < 6);
                            uint32_t *cur = tBuf[ODD], *nxt = tBuf[ODD ^ 1];
                            uint32_t *rawCur = rawBuf[ODD ^ 1], *rawNxt = rawBuf[ODD];
                            if (HAS_NEXT) {
                                TmemWaitLdRegs16(rawCur);
                            }
                            if (LOAD) {
                                if (c == 2) {
                                    waitSecondHalf(); // chunk 4 is the first of the second half
                                }
                                TmemLd16(tLane + (c + 2) * 16, rawNxt);
                            }
                            const float2 eoff2 = make_float2(eoff, eoff);
                            mxN = -INFINITY;
#pragma unroll
                            for (int k = 0; k < 16; k += 4) {
                                float2 e[2];
#pragma unroll
                                for (int kk = 0; kk < 4; kk += 2) {
                                    const int cc = k + kk;
                                    if (HAS_NEXT) {
                                        float2 tt = scalePair(rawCur[cc], rawCur[cc + 1], (c + 1) * 16 + cc, eoff2);
                                        mxN = Max3(mxN, tt.x, tt.y);
                                        nxt[cc] = __float_as_uint(tt.x);
                                        nxt[cc + 1] = __float_as_uint(tt.y);
                                    }
                                    float2 x = make_float2(__uint_as_float(cur[cc]), __uint_as_float(cur[cc + 1]));
                                    float2 w;
                                    if (((cc >> 1) & 7) < TSA_FWD_POLY_PAIRS) {
                                        w = PolyExp2Pair(x);
                                    } else {
                                        w = make_float2(FastExp2(x.x), FastExp2(x.y));
                                    }
                                    lacc2 = __fadd2_rn(lacc2, w);
                                    if (HAS_VSCALE) {
                                        e[kk >> 1] = __fmul2_rn(w, *reinterpret_cast<const float2 *>(svBuf + c * 16 + cc));
                                    } else {
                                        e[kk >> 1] = w;
                                    }
                                }
                                pk[k >> 2] = PackE4M3x4(e[0].x, e[0].y, e[1].x, e[1].y);
                            }
                            TmemStN<4>(tLane + 32 * (c >> 1) + 4 * (c & 1), pk);
                            if (c == 3) {
                                handOver(0);
                            }
                            if (HAS_NEXT && __any_sync(0xffffffffu, (MODE != 3 || c < 7) && mxN > headroom)) {
                                TmemWaitLdRegs16(rawNxt); // no load is in flight across the out-of-line call
                                raise(mxN, c + 1, nxt);
                            }
                        };
                        TmemLd16(tLane, rawBuf[0]);
                        TmemWaitLdRegs16(rawBuf[0]);
                        TmemLd16(tLane + 16, rawBuf[1]);
                        {
                            const float2 eoff2 = make_float2(eoff, eoff);
#pragma unroll
                            for (int cc = 0; cc < 16; cc += 2) {
                                float2 tt = scalePair(rawBuf[0][cc], rawBuf[0][cc + 1], cc, eoff2);
                                mxN = Max3(mxN, tt.x, tt.y);
                                tBuf[0][cc] = __float_as_uint(tt.x);
                                tBuf[0][cc + 1] = __float_as_uint(tt.y);
                            }
                        }
                        if (__any_sync(0xffffffffu, mxN > headroom)) {
                            TmemWaitLdRegs16(rawBuf[1]);
                            raise(mxN, 0, tBuf[0]);
                        }
                        using TEven = std::integral_constant<int, 0>;
                        using TOdd = std::integral_constant<int, 1>;
                        if (D == 128) {
#pragma unroll 1
                            for (int c = 0; c < 6; c += 2) {
                                step(std::integral_constant<int, 0>(), TEven(), c);
                                step(std::integral_constant<int, 0>(), TOdd(), c + 1);
                            }
                            step(std::integral_constant<int, 1>(), TEven(), 6);
                            step(std::integral_constant<int, 2>(), TOdd(), 7);
                        } else {
#pragma unroll 1
                            for (int c = 0; c < 8; c += 2) {
                                step(std::integral_constant<int, 3>(), TEven(), c);
                                step(std::integral_constant<int, 3>(), TOdd(), c + 1);
                            }
                        }
                    }
                };
                if constexpr (V_I8) {
                    processTile(std::true_type());
                } else {
                    if (masked) {
                        processTile(std::true_type());
                    } else {
                        processTile(std::false_type());
                    }
                }
                handOver(1);
                ++sCount;
                ++kvCount;
                ++tilesInItem;
            }
            if (failed) {
                break;
            }
            if (flags & RF_LAST) {
                // ---- epilogue of the item
                // consumer fused into the epilogue: the combiner keys of 32 columns at a time, one step ahead of their use
                uint32_t kcur[16];
                const char *kRow = nullptr;
                char *kvRow = nullptr;
                auto loadKeys = [&](int col, uint32_t *dst) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(kRow + col * 2);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 x = __ldcs(src + i);
                        dst[4 * i] = x.x, dst[4 * i + 1] = x.y, dst[4 * i + 2] = x.z, dst[4 * i + 3] = x.w;
                    }
                };
                if (KV) {
                    kRow = p.KvK.Row(rowOk ? row : 0) + (size_t)head * D * 2;
                    kvRow = p.KvOut.Row(rowOk ? row : 0) + (size_t)head * 4 * D * 2;
                    if (rowOk) {
                        loadKeys(0, kcur);
                    }
                }
                if (tilesInItem > 0) {
                    if (!wait(&misc.BarOFull, oCount & 1, kDevTimeoutMma)) {
                        break;
                    }
                    ++oCount;
                    TcFenceAfter();
                }
                const float lTot = (lacc2.x + lacc2.y) * (1.0f / 128.0f) + exp2f(-m);
                const float outMult = (HAS_VSCALE ? invK : p.VVecScale) * (1.0f / 128.0f) / lTot;
                if (rowOk && p.Lse.Valid()) {
                    p.Lse.Row(head)[row] = m + log2f(lTot);
                }
                const int esz = (p.OutDtype == TSA_F32) ? 4 : 2;
                char *oRow = p.Out.Row(rowOk ? row : 0) + (size_t)head * D * esz;
                const bool wideStores = p.WideStores != 0;
                const size_t headOff = (size_t)head * D * esz;
                // 32 bytes of the row to the output and to every further destination (fused all-gather: peer GPUs' buffers)
                auto storeAll = [&](char *local, size_t rowOff, const uint32_t *w) {
                    auto put = [&](char *dstp) {
                        if (wideStores) {
                            StGlobal256(dstp, w);
                        } else {
                            uint4 *dst = reinterpret_cast<uint4 *>(dstp);
                            dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    };
                    put(local);
                    if (p.OutCopies == 1) {
                        // a single further destination: the row's own thread stores there too (measured faster than the hand-over
                        // to the forwarding warp, which takes over from two destinations on)
                        put(p.OutCopy[0].Row(row) + rowOff);
                    }
                };
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t o[32];
                    uint32_t knext[16];
                    if (KV && rowOk && c0 + 32 < D) {
                        loadKeys(c0 + 32, knext);
                    }
                    if (tilesInItem > 0) {
                        TmemLd32(tLane + TMEM_O_COL + c0, o);
                        TmemWaitLdRegs(o);
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            o[c] = 0;
                        }
                    }
                    if (rowOk) {
                        // 32-byte stores where the output rows allow them (whole sectors, half the store instructions)
                        if (p.OutDtype == TSA_F32) {
#pragma unroll
                            for (int c = 0; c < 32; c += 8) {
                                uint32_t w[8];
#pragma unroll
                                for (int k = 0; k < 8; ++k) {
                                    w[k] = __float_as_uint(__uint_as_float(o[c + k]) * outMult);
                                }
                                storeAll(oRow + (c0 + c) * 4, headOff + (c0 + c) * 4, w);
                            }
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; c += 16) {
                                uint32_t w[8];
#pragma unroll
                                for (int k = 0; k < 8; ++k) {
                                    float a = __uint_as_float(o[c + 2 * k]) * outMult, b = __uint_as_float(o[c + 2 * k + 1]) * outMult;
                                    if (p.OutDtype == TSA_BF16) {
                                        __nv_bfloat162 hh = __floats2bfloat162_rn(a, b);
                                        w[k] = *reinterpret_cast<uint32_t *>(&hh);
                                    } else {
                                        w[k] = PackHalf2(a, b);
                                    }
                                }
                                storeAll(oRow + (c0 + c) * 2, headOff + (c0 + c) * 2, w);
                                if (KV) {
                                    // kv[blk][z] = k[z ^ blk] * out[z] * kvMult for these 16 columns, out as it was just rounded to
                                    // bf16 (so the result is that of the stand-alone kernel on the stored output, bit for bit);
                                    // z ^ blk stays inside an aligned group of four columns
                                    const uint32_t *kw = &kcur[c / 2];
                                    float2 of[8], kf[8], ks[8];
#pragma unroll
                                    for (int k = 0; k < 8; ++k) {
                                        of[k] = make_float2(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xffff0000u));
                                        kf[k] = make_float2(__uint_as_float(kw[k] << 16), __uint_as_float(kw[k] & 0xffff0000u));
                                        ks[k] = make_float2(kf[k].y, kf[k].x);
                                    }
                                    const float2 mult2 = make_float2(p.KvMult, p.KvMult);
#pragma unroll
                                    for (int blk = 0; blk < 4; ++blk) {
                                        uint32_t rr[8];
#pragma unroll
                                        for (int k = 0; k < 8; ++k) {
                                            const float2 kk = (blk & 1) ? ks[k ^ (blk >> 1)] : kf[k ^ (blk >> 1)];
                                            const float2 pr = __fmul2_rn(__fmul2_rn(kk, of[k]), mult2);
                                            const __nv_bfloat162 hh = __floats2bfloat162_rn(pr.x, pr.y);
                                            rr[k] = *reinterpret_cast<const uint32_t *>(&hh);
                                        }
                                        char *dstp = kvRow + ((size_t)blk * D + c0 + c) * 2;
                                        if (p.KvWide) {
                                            StGlobal256Stream(dstp, rr);
                                        } else {
                                            __stcs(reinterpret_cast<uint4 *>(dstp), make_uint4(rr[0], rr[1], rr[2], rr[3]));
                                            __stcs(reinterpret_cast<uint4 *>(dstp) + 1, make_uint4(rr[4], rr[5], rr[6], rr[7]));
                                        }
                                    }
                                }
                            }
                        }
                    }
                    if (KV) {
#pragma unroll
                        for (int k = 0; k < 16; ++k) {
                            kcur[k] = knext[k];
                        }
                    }
                }
                // no "O has been read" signal is needed: these same threads arrive on BarP for the next item's first
                // tile only after this read-out, and the PV that overwrites O is issued after that arrival
                if (FORWARD && p.OutCopies > 1 && !postCopy(qTile * TILE_M, head)) {
                    break;
                }
            }
        }
        if (FORWARD && p.OutCopies > 1 && !failed) {
            postCopy(0, -1); // no more items: the forwarding warp leaves
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == FW_MMA_WARP) {
        TmemDealloc(tmem, TMEM_COLS);
    }
}

// int8 values as two e4m3 planes whose sum is the value: a = 16 * floor(v / 16), b = v - a in 0..15 (both exact in e4m3).
// One thread per 16 bytes of a row; rows are rowBytes wide (a multiple of 16), planes have the pitch `pitch`.
__global__ void __launch_bounds__(256) SplitI8ValuesKernel(P2D<uint8_t> v, int rows, int rowBytes, uint8_t *va, uint8_t *vb, int pitch)
{
    const int perRow = rowBytes / 16;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * perRow) {
        return;
    }
    const int row = (int)(idx / perRow), c16 = (int)(idx % perRow);
    const int4 src = *reinterpret_cast<const int4 *>(v.Row(row) + c16 * 16);
    const uint32_t w[4] = {(uint32_t)src.x, (uint32_t)src.y, (uint32_t)src.z, (uint32_t)src.w};
    uint32_t oa[4], ob[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float fa[4], fb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int x = (int)(int8_t)(w[k] >> (8 * j));
            const int a = (x >> 4) * 16;
            fa[j] = (float)a;
            fb[j] = (float)(x - a);
        }
        oa[k] = PackE4M3x4(fa[0], fa[1], fa[2], fa[3]);
        ob[k] = PackE4M3x4(fb[0], fb[1], fb[2], fb[3]);
    }
    *reinterpret_cast<int4 *>(va + (size_t)row * pitch + c16 * 16) = make_int4((int)oa[0], (int)oa[1], (int)oa[2], (int)oa[3]);
    *reinterpret_cast<int4 *>(vb + (size_t)row * pitch + c16 * 16) = make_int4((int)ob[0], (int)ob[1], (int)ob[2], (int)ob[3]);
}

// per head maximum of the V scale plane (normalises the weights' e4m3 range).  Scales are non-negative, so
// the float maximum is the maximum of the bit patterns; the workspace is zeroed before the launch.
constexpr int VREF_CHUNK = 2048;
__global__ void __launch_bounds__(256) VRefKernel(P2D<float> vScale, int keyRows, float *vRef)
{
    int head = blockIdx.y;
    const float *rowp = vScale.Row(head);
    int t0 = blockIdx.x * VREF_CHUNK;
    float mx = 0;
#pragma unroll
    for (int k = 0; k < VREF_CHUNK / 256; ++k) {
        int t = t0 + k * 256 + threadIdx.x;
        if (t < keyRows) {
            mx = fmaxf(mx, rowp[t]);
        }
    }
    mx = WarpMax(mx);
    if ((threadIdx.x & 31) == 0 && mx > 0) {
        atomicMax(reinterpret_cast<int *>(vRef + head), __float_as_int(mx));
    }
}

// The same maximum with one CTA per head and no atomics, so that nothing has to be cleared first; the CTA of head 0 also
// zeroes the forward's work-item counter: one launch in front of the attention kernel instead of a memset and a kernel.
// Taken while a head's scale row is short enough for one CTA (VREF_ONE_CTA_ROWS).
constexpr int VREF_ONE_CTA_ROWS = 1 << 18;
__global__ void __launch_bounds__(1024) VRefHeadKernel(P2D<float> vScale, int keyRows, float *vRef, int *counter)
{
    __shared__ float part[32];
    const int head = blockIdx.x, tid = threadIdx.x;
    const float *rowp = vScale.Row(head);
    float mx = 0;
    if (((uintptr_t)rowp & 15) == 0) {
        const float4 *row4 = reinterpret_cast<const float4 *>(rowp);
        const int n4 = keyRows >> 2;
#pragma unroll 4
        for (int i = tid; i < n4; i += 1024) {
            const float4 x = row4[i];
            mx = fmaxf(fmaxf(mx, fmaxf(x.x, x.y)), fmaxf(x.z, x.w));
        }
        for (int t = (n4 << 2) + tid; t < keyRows; t += 1024) {
            mx = fmaxf(mx, rowp[t]);
        }
    } else {
#pragma unroll 8
        for (int t = tid; t < keyRows; t += 1024) {
            mx = fmaxf(mx, rowp[t]);
        }
    }
    mx = WarpMax(mx);
    if ((tid & 31) == 0) {
        part[tid >> 5] = mx;
    }
    __syncthreads();
    if (tid < 32) {
        mx = WarpMax(part[tid]);
        if (tid == 0) {
            vRef[head] = mx;
            if (head == 0) {
                *counter = 0;
            }
        }
    }
}

// ---- raw int32 score tiles (parity hook for the kind::i8 accumulators) -------------------------
struct TScoresMisc {
    uint64_t BarQ, BarMma;
    uint32_t TmemBase;
};
constexpr int SCORE_THREADS = 128;

template <int D>
__global__ void __launch_bounds__(SCORE_THREADS) ScoresI8Kernel(const __grid_constant__ CUtensorMap tmQ,
    const __grid_constant__ CUtensorMap tmK, int lenQ, int lenK, int32_t *scores, int *status)
{
    constexpr int SWZ = (D == 128) ? 128 : 64;
    constexpr uint32_t GROUP_BYTES = 8 * D;
    constexpr uint32_t IDESC = MakeInstrDesc(2, 1, 1, 0, 0, TILE_M, TILE_N);
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem, *sK = smem + 128 * D;
    TScoresMisc &misc = *reinterpret_cast<TScoresMisc *>(smem + 2 * 128 * D);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int head = blockIdx.z, qTile = blockIdx.y, kTile = blockIdx.x;
    if (tid == 0) {
        MbarInit(&misc.BarQ, 1);
        MbarInit(&misc.BarMma, 1);
        FenceBarrierInit();
    }
    if (warp == 0) {
        TmemAlloc(&misc.TmemBase, 128);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;
    const uint32_t tLane = tmem + ((uint32_t)(warp * 32) << 16);
    bool failed = false;
    if (tid == 0) {
        MbarExpectTx(&misc.BarQ, 2 * 128 * D);
        TmaLoad2D(sQ, &tmQ, head * D, qTile * TILE_M, &misc.BarQ);
        TmaLoad2D(sK, &tmK, head * D, kTile * TILE_N, &misc.BarQ);
        if (WaitBar(&misc.BarQ, 0)) {
            TcFenceAfter();
#pragma unroll
            for (int ks = 0; ks < D / 32; ++ks) {
                uint64_t aDesc = MakeSmemDesc(SmemAddr(sQ) + ks * 32, 16, GROUP_BYTES, SWZ);
                uint64_t bDesc = MakeSmemDesc(SmemAddr(sK) + ks * 32, 16, GROUP_BYTES, SWZ);
                MmaI8SS(tmem, aDesc, bDesc, IDESC, ks > 0);
            }
        } else {
            failed = true;
            if (status) {
                atomicOr(status, kDevTimeoutTma);
            }
        }
        MmaCommit(&misc.BarMma);
    }
    if (!WaitBar(&misc.BarMma, 0)) {
        failed = true;
        if (status) {
            atomicOr(status, kDevTimeoutMma);
        }
    }
    TcFenceAfter();
    failed = __syncthreads_or(failed ? 1 : 0) != 0;
    int i = qTile * TILE_M + tid;
    if (!failed) {
#pragma unroll
        for (int c0 = 0; c0 < TILE_N; c0 += 32) {
            uint32_t r[32];
            TmemLd32(tLane + c0, r);
            TmemWaitLd();
            if (i < lenQ) {
                int32_t *dst = scores + ((size_t)head * lenQ + i) * lenK + kTile * TILE_N + c0;
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    if (kTile * TILE_N + c0 + c < lenK) {
                        dst[c] = (int32_t)r[c];
                    }
                }
            }
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == 0) {
        TmemDealloc(tmem, 128);
    }
}

// ---- self-test of a bounded wait ----------------------------------------------------------------
// One thread arms a barrier nobody will ever arrive on and waits for it with the given bound: the wait must give up,
// report through the status word and return, leaving the context usable.
__global__ void BoundedWaitSelfTestKernel(long long limitCycles, int *status)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        MbarInit(&bar, 1);
        FenceBarrierInit();
        if (!WaitBar(&bar, 0, limitCycles) && status) {
            atomicOr(status, kDevTimeoutTma);
        }
    }
}

int LaunchBoundedWaitSelfTest(long long limitCycles, int *statusWord, cudaStream_t stream)
{
    BoundedWaitSelfTestKernel<<<1, 32, 0, stream>>>(limitCycles, statusWord);
    return CheckCuda(cudaGetLastError(), "bounded-wait self-test launch");
}

// ---- host side ---------------------------------------------------------------------------------

static bool TmaCompatible(tsa_ptr2d a)
{
    return a.data && ((uintptr_t)a.data % 16 == 0) && (a.stride_bytes % 16 == 0) && a.xsize > 0 && a.ysize > 0;
}

bool Sm100FwdSupports(const tsa_att_cfg *cfg, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v)
{
    if (cfg->flags & TSA_FLAG_FORCE_GENERIC) {
        return false;
    }
    if (cfg->head_dim_qk != cfg->head_dim_v || (cfg->head_dim_qk != 64 && cfg->head_dim_qk != 128)) {
        return false;
    }
    if (cfg->v_dtype == TSA_I8 && cfg->qk_dtype != TSA_I8) {
        return false; // int8 values with e4m3 queries and keys: no counterpart in the reference, generic kernels
    }
    return TmaCompatible(qk) && TmaCompatible(qv) && TmaCompatible(v);
}

// workspace: per-head V-scale maxima, then the work-item counter
static size_t VRefBytes(int headCount)
{
    return (size_t)((headCount * sizeof(float) + 255) / 256 * 256);
}
static int ValuePlanePitch(int headCount, int headDim)
{
    return (headCount * headDim + 15) / 16 * 16;
}
size_t Sm100FwdWorkspaceBytes(const tsa_att_cfg *cfg, int headCount, int keyRows)
{
    size_t bytes = VRefBytes(headCount) + 256;
    if (cfg && cfg->v_dtype == TSA_I8) {
        bytes += 2 * (size_t)keyRows * ValuePlanePitch(headCount, cfg->head_dim_v); // the two e4m3 planes of the int8 values
    }
    return bytes;
}

static TFwdDump g_dump;
void SetFwdScoreDump(const TFwdDump &d)
{
    g_dump = d;
}

template <int D, bool QK_I8, bool HAS_VSCALE, bool HAS_ALIBI, bool V_I8, bool FORWARD, bool KV = false>
static int LaunchFwdT2(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const CUtensorMap &mv2, const TFwdParams &fp, cudaStream_t stream)
{
    auto kern = FwdSm100Kernel<D, QK_I8, HAS_VSCALE, HAS_ALIBI, V_I8, FORWARD, KV>;
    int smemBytes = TFwdSmem<D, V_I8>::TOTAL;
    int dev = 0, smCount = 0;
    int rc = CheckCuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc == TSA_OK) {
        rc = CheckCuda(cudaDeviceGetAttribute(&smCount, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
    }
    if (rc == TSA_OK) {
        rc = CheckCuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes), "cudaFuncSetAttribute(forward)");
    }
    if (rc != TSA_OK) {
        return rc;
    }
    int ctas = 2 * smCount;
    if (ctas > fp.TotalItems) {
        ctas = fp.TotalItems;
    }
    kern<<<ctas, FORWARD ? FW_THREADS_FORWARD : FW_THREADS, smemBytes, stream>>>(mq, mk, mv, mv2, fp);
    return CheckCuda(cudaGetLastError(), "tcgen05 forward launch");
}

template <int D, bool QK_I8, bool HAS_VSCALE, bool HAS_ALIBI, bool V_I8>
static int LaunchFwdT(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const CUtensorMap &mv2, const TFwdParams &fp, cudaStream_t stream)
{
    // two or more further destinations: the kernel with the forwarding warp (e4m3 values only: the all-gather is a prefill feature)
    if (fp.KvOut.Data != nullptr) {
        // the consumer in the epilogue: its own kernel, so that the plain forward keeps its register allocation
        if (V_I8 || fp.OutCopies > 1 || fp.OutDtype != TSA_BF16) {
            return Fail(TSA_UNSUPPORTED, "tsa_att_fwd_kv: e4m3 values, a bf16 output and at most one further destination");
        }
        return LaunchFwdT2<D, QK_I8, HAS_VSCALE, HAS_ALIBI, false, false, true>(mq, mk, mv, mv2, fp, stream);
    }
    if (fp.OutCopies > 1) {
        if (V_I8) {
            return Fail(TSA_UNSUPPORTED, "tsa_att_fwd_to: more than two destinations with int8 values");
        }
        return LaunchFwdT2<D, QK_I8, HAS_VSCALE, HAS_ALIBI, false, true>(mq, mk, mv, mv2, fp, stream);
    }
    return LaunchFwdT2<D, QK_I8, HAS_VSCALE, HAS_ALIBI, V_I8, false>(mq, mk, mv, mv2, fp, stream);
}

int LaunchSm100Fwd(const tsa_att_cfg *cfg, const TGenParams &p, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v,
    int lenAttTiles, int keyRows, void *workspace, int *statusWord, cudaStream_t stream)
{
    const int D = cfg->head_dim_qk;
    const bool vI8 = cfg->v_dtype == TSA_I8;
    const size_t headBytes = VRefBytes(p.HeadCount) + 256; // value-scale maxima and the counter
    CUtensorMap mq, mk, mv, mv2;
    int rc = MakeTileMap(&mq, qk, D, "qk");
    if (rc == TSA_OK) {
        rc = MakeTileMap(&mk, qv, D, "qv");
    }
    if (rc == TSA_OK && !vI8) {
        rc = MakeTileMap(&mv, v, D, "v");
        mv2 = mv;
    }
    if (rc == TSA_OK && vI8) {
        // the two e4m3 planes of the int8 values live behind the head of the workspace
        const int pitch = ValuePlanePitch(p.HeadCount, D);
        const int rowBytes = p.HeadCount * D / 16 * 16;
        if (rowBytes != p.HeadCount * D) {
            return Fail(TSA_UNSUPPORTED, "tcgen05 forward with int8 values: H * D must be a multiple of 16");
        }
        uint8_t *va = (uint8_t *)workspace + headBytes, *vb = va + (size_t)keyRows * pitch;
        tsa_ptr2d pa = {va, pitch, p.HeadCount * D, keyRows}, pb = {vb, pitch, p.HeadCount * D, keyRows};
        rc = MakeTileMap(&mv, pa, D, "v (upper e4m3 plane)");
        if (rc == TSA_OK) {
            rc = MakeTileMap(&mv2, pb, D, "v (lower e4m3 plane)");
        }
        if (rc == TSA_OK) {
            const long long items = (long long)keyRows * (rowBytes / 16);
            SplitI8ValuesKernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(p.V, keyRows, rowBytes, va, vb, pitch);
            rc = CheckCuda(cudaGetLastError(), "int8 value split launch");
        }
    }
    if (rc != TSA_OK) {
        return rc;
    }
    const bool hasVs = p.VScale.Data != nullptr;
    const size_t vrefBytes = VRefBytes(p.HeadCount);
    TFwdParams fp;
    fp.HeadCount = p.HeadCount;
    {
        // keys + values of one head (an upper bound of what the items of one head touch); groups of heads that keep about 128 MB
        // in flight, the size of L2, and never fewer than four heads
        const long long perHead = (long long)keyRows * D * (vI8 ? 3 : 2);
        long long g = perHead > 0 ? (128ll << 20) / perHead : p.HeadCount;
        g = g < 4 ? 4 : g;
        fp.HeadGroup = (int)(g < p.HeadCount ? g : p.HeadCount);
    }
    fp.OutRows = p.Len;
    fp.KeyRows = keyRows;
    fp.LenAttTiles = lenAttTiles;
    fp.QTiles = (lenAttTiles + 1) / 2;
    fp.TotalItems = fp.QTiles * p.HeadCount;
    fp.Counter = reinterpret_cast<int *>((char *)workspace + vrefBytes);
    fp.Spans = p.Spans;
    fp.SpanPtr = p.SpanPtr;
    fp.QScale = p.QScale;
    fp.KScale = p.KScale;
    fp.VScale = p.VScale;
    fp.VRef = hasVs ? (const float *)workspace : nullptr;
    fp.ScaleBulk = ((uintptr_t)p.KScale.Data % 16 == 0 && p.KScale.Stride % 16 == 0 &&
        (!hasVs || ((uintptr_t)p.VScale.Data % 16 == 0 && p.VScale.Stride % 16 == 0))) ? 1 : 0;
    fp.Out = p.Out;
    fp.OutCopies = p.OutCopies;
    fp.WideStores = ((((uintptr_t)p.Out.Data | (uintptr_t)p.Out.Stride) & 31) == 0) ? 1 : 0;
    for (int k = 0; k < TSA_MAX_OUT_COPIES; ++k) {
        fp.OutCopy[k] = k < p.OutCopies ? p.OutCopy[k] : P2D<char>();
        if (k < p.OutCopies && ((((uintptr_t)p.OutCopy[k].Data | (uintptr_t)p.OutCopy[k].Stride) & 31) != 0)) {
            fp.WideStores = 0;
        }
    }
    fp.KvK = p.KvK;
    fp.KvOut = p.KvOut;
    fp.KvMult = p.KvMult;
    fp.KvWide = ((((uintptr_t)p.KvOut.Data | (uintptr_t)p.KvOut.Stride) & 31) == 0) ? 1 : 0;
    fp.Lse = p.Lse;
    fp.GlobalScale = p.GlobalScale;
    fp.C = p.C;
    fp.QkVecScale = p.QkVecScale;
    fp.VVecScale = p.VVecScale;
    fp.Slope = p.Slope;
    fp.OutDtype = p.OutDtype;
    fp.Status = statusWord;
    fp.DumpScores = g_dump.Dst;
    fp.DumpHead = g_dump.Head;
    fp.DumpQTile = g_dump.QTile;
    fp.DumpTile = g_dump.Tile;
    fp.WaitCycles = g_dump.WaitCycles > 0 ? g_dump.WaitCycles : WAIT_CYCLES;
    fp.WithholdTile = g_dump.WithholdTile;
    if (hasVs && keyRows <= VREF_ONE_CTA_ROWS) {
        // one launch writes the per-head maxima and zeroes the counter
        VRefHeadKernel<<<p.HeadCount, 1024, 0, stream>>>(p.VScale, keyRows, (float *)workspace, fp.Counter);
        rc = CheckCuda(cudaGetLastError(), "value-scale maximum launch");
        if (rc != TSA_OK) {
            return rc;
        }
    } else {
        // one clear covers the V-scale maxima and the counter behind them
        rc = CheckCuda(cudaMemsetAsync(hasVs ? workspace : (void *)fp.Counter, 0, hasVs ? vrefBytes + 256 : 256, stream), "clearing the forward workspace");
        if (rc != TSA_OK) {
            return rc;
        }
        if (hasVs) {
            dim3 vgrid((keyRows + VREF_CHUNK - 1) / VREF_CHUNK, p.HeadCount);
            VRefKernel<<<vgrid, 256, 0, stream>>>(p.VScale, keyRows, (float *)workspace);
        }
    }
    const bool i8 = cfg->qk_dtype == TSA_I8;
    const bool alibi = p.Slope != 0.0f;
#define TSA_FWD_CASE(DD, I8, VS)                                                                         \
    if (D == DD && i8 == I8 && hasVs == VS && !vI8) {                                                    \
        return alibi ? LaunchFwdT<DD, I8, VS, true, false>(mq, mk, mv, mv2, fp, stream)                  \
                     : LaunchFwdT<DD, I8, VS, false, false>(mq, mk, mv, mv2, fp, stream);                \
    }                                                                                                    \
    if (D == DD && i8 == I8 && hasVs == VS && vI8 && I8) {                                               \
        return alibi ? LaunchFwdT<DD, I8, VS, true, I8>(mq, mk, mv, mv2, fp, stream)                     \
                     : LaunchFwdT<DD, I8, VS, false, I8>(mq, mk, mv, mv2, fp, stream);                   \
    }
    TSA_FWD_CASE(64, false, false)
    TSA_FWD_CASE(64, false, true)
    TSA_FWD_CASE(64, true, false)
    TSA_FWD_CASE(64, true, true)
    TSA_FWD_CASE(128, false, false)
    TSA_FWD_CASE(128, false, true)
    TSA_FWD_CASE(128, true, false)
    TSA_FWD_CASE(128, true, true)
#undef TSA_FWD_CASE
    return Fail(TSA_UNSUPPORTED, "tcgen05 forward: unsupported head size %d", D);
}

int LaunchScoresI8(tsa_ptr2d qk, tsa_ptr2d qv, int headCount, int headDim, int lenQ, int lenK, int32_t *scores, int *statusWord, cudaStream_t stream)
{
    CUtensorMap mq, mk;
    int rc = MakeTileMap(&mq, qk, headDim, "qk");
    if (rc == TSA_OK) {
        rc = MakeTileMap(&mk, qv, headDim, "qv");
    }
    if (rc != TSA_OK) {
        return rc;
    }
    dim3 grid((lenK + TILE_N - 1) / TILE_N, (lenQ + TILE_M - 1) / TILE_M, headCount);
    int smemBytes = 2 * 128 * headDim + 4096 + 1024;
    if (headDim == 128) {
        ScoresI8Kernel<128><<<grid, SCORE_THREADS, smemBytes, stream>>>(mq, mk, lenQ, lenK, scores, statusWord);
    } else {
        ScoresI8Kernel<64><<<grid, SCORE_THREADS, smemBytes, stream>>>(mq, mk, lenQ, lenK, scores, statusWord);
    }
    return CheckCuda(cudaGetLastError(), "int8 score launch");
}

} // namespace tsa
