// Quantized attention forward for sm_100a: tcgen05 MMA with accumulators in tensor memory, TMA-staged
// Q/K/V tiles, online base-2 softmax in registers.
//
// Replaces Fp8Att (code/gpt/compute/gpt_att_fp8.cuh:43-248) and the int8 QK^T variant of Fp16Att
// (gpt_att_fp16.cuh:121-318) of the reference:
//   S = Q K^T          kind::f8f6f4 (e4m3 x e4m3 -> f32) or kind::i8 (s8 x s8 -> s32, exact), 128 x 128 x D
//   z = S * sq_i * sk_j * c - slope * (i - j), masked by the row's span            (gpt_att_fp8.cuh:137-147)
//   m = running floor(max) so that rescale factors are powers of two                 (gpt_att_fp8.cuh:163-164)
//   P = e4m3(2^(z - m) * 128 * sv_j / svRef); O += P V   kind::f8f6f4, A = P from tensor memory,
//                                                         B = V tile as an MN-major operand (no transposed copy)
//   out = O * (svRef / 128) / (2^-m + sum 2^(z - m));  sumWeightLog = m + log2(...)   (gpt_att_fp8.cuh:225-245)
// On tiles where the span mask is active (the only tiles a row with few keys ever sees) P is split into
// e4m3(P) + e4m3(P - e4m3(P)) and multiplied in two MMAs, which removes the 3-bit-mantissa rounding of the
// weights where it is not averaged out over many keys.
//
// Work item = one head x 128 query rows (two 64-row span blocks).  CTAs are persistent: two per SM, each takes
// items from a counter in the workspace (late, long rows first) until none is left, so barrier set-up, tensor
// memory allocation and the pipeline fill are paid once per CTA and one item's output store overlaps the next
// item's first MMAs.  Twelve warps in three warpgroups:
//   warps 0-7  softmax, two threads per query row (a row is one tensor-memory lane; each thread owns 64 of the
//              128 score columns of a tile and keeps them in registers between the maximum and the weights);
//   warp  8    lane 0 issues every MMA;
//   warp  9    loader: takes the next item, stages its spans / query scales in shared memory, issues the TMA
//              copies of Q and of the K/V ring (which runs on across item boundaries) and stages the key scales;
//   warps 10-11 only take part in the register reallocation (setmaxnreg hands their registers to the softmax warps).
// Tensor memory (256 columns, so two CTAs share an SM): S [0,128) f32 / s32, O [128, 128 + D) f32.  For D = 64 the
// weights have their own columns [192, 256), so S is free again as soon as every thread has loaded its scores:
// QK^T of the next tile runs while the softmax of this one is still computing, and P V follows when P arrives.
// For D = 128 P is written back over the thread's own S columns and the next QK^T follows P V.
// Shared memory: 2 Q tiles, STAGES x (K tile, V tile, key scales) filled by TMA with the 128 B (D = 128) or 64 B
// (D = 64) swizzle the MMA descriptors expect.  Softmax arithmetic uses packed f32x2 multiply-adds and 3-input max.
// Key tiles follow the reference's grouped spans: for round r the tiles [Start, Finish] of the two blocks'
// r-th groups; 32-column chunks no row of a warp attends cost no exponentials (window layers).
// Every barrier wait is bounded; when one runs out the kernel records a code in *statusWord, every role leaves
// its loop, outstanding copies are drained, tensor memory is freed and the CTA returns.
#include "att_internal.cuh"
#include "att_sm100_common.cuh"

namespace tsa {

using namespace sm100;

constexpr int SOFTMAX_THREADS = 256;
constexpr int SOFTMAX_WARPS = SOFTMAX_THREADS / 32;
constexpr int MMA_WARP = 8;
constexpr int LOAD_WARP = 9;
constexpr int FWD_THREADS = 384;
constexpr int SOFTMAX_REGS = 104; // after setmaxnreg: (384 * 80 - 128 * 32) / 256 = 104
constexpr int CONTROL_REGS = 32;
constexpr int SCORE_THREADS = 128;
constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t TMEM_O_COL = 128;
constexpr uint32_t TMEM_P_COL = 192; // D = 64 only
constexpr int ITEM_RING = 4;
constexpr int MAX_STAGES = 4;

struct TFwdParams {
    int HeadCount;
    int OutRows;      // rows of out that may be written
    int KeyRows;      // rows of K / V
    int LenAttTiles;  // number of 64-row span blocks
    int QTiles;       // 128-row query tiles
    const tsa_span_group *Spans;
    const int *SpanPtr;
    P2D<float> QScale, KScale, VScale;
    const float *VRef; // per head max of VScale (workspace), null without VScale
    int *Counter;      // next work item (workspace, zeroed before the launch)
    P2D<char> Out;
    P2D<float> Lse;
    const float *GlobalScale;
    float C;
    float QkVecScale, VVecScale;
    float Slope;
    int OutDtype;
    int *Status;
};

// what the loader publishes about a work item: everything the other warps would otherwise fetch from global
// memory at the start of the item
struct TItemSlot {
    int QTile, Head;     // QTile < 0: no more work
    int N0, N1;          // number of span groups (rounds) of the two 64-row blocks
    int A0, A1;          // index of each block's first group
    int Round0, J0, Hi;  // first non-empty round and its key-tile range; Valid = 0: the item has no key tile
    int Valid;
    int MaxS, MinF;      // max span start / min span finish over the 128 rows in round Round0
    float VRef;
    int Pad[3];
    int SpanS[TILE_M], SpanF[TILE_M]; // the rows' spans in round Round0
    float SQ[TILE_M];                 // the rows' query scales (0 beyond the last row)
};

struct TFwdMisc {
    TItemSlot Item[ITEM_RING];
    float Sk[MAX_STAGES][TILE_N]; // key scale of each column of the staged tile
    float Sv[MAX_STAGES][TILE_N]; // value scale / per-head maximum
    float Al[TILE_N];             // ALiBi term slope * column (tile invariant)
    float RowX[2][2][TILE_M];     // exchange between the two threads of a row, double buffered by tile parity
    uint64_t BarItem[ITEM_RING];      // loader -> all: item slot written
    uint64_t BarItemEmpty[ITEM_RING]; // softmax warps + MMA lane -> loader: slot read
    uint64_t BarQFull[2], BarQEmpty[2];
    uint64_t BarFull[MAX_STAGES], BarEmpty[MAX_STAGES];
    uint64_t BarS;     // MMA -> softmax: S(t) complete
    uint64_t BarSRead; // softmax -> MMA: S(t) is in registers (D = 64)
    uint64_t BarP;     // softmax -> MMA: P(t) written
    uint64_t BarPV;    // MMA -> softmax: P V(t) retired: O current, P columns free
    uint32_t TmemBase;
    int Abort;         // a bounded wait ran out somewhere in the CTA
};

template <int D>
struct TFwdSmem {
    static constexpr int STAGES = (D == 64) ? 4 : 2;
    static constexpr int TILE_BYTES = 128 * D;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = 2 * TILE_BYTES;
    static constexpr int V_OFF = K_OFF + STAGES * TILE_BYTES;
    static constexpr int MISC_OFF = V_OFF + STAGES * TILE_BYTES;
    static constexpr int TOTAL = MISC_OFF + (int)((sizeof(TFwdMisc) + 1023) / 1024 * 1024);
};

__device__ __forceinline__ void IterFromSlot(TTileIter &it, const TItemSlot &s, const tsa_span_group *spans, int keyRows)
{
    it.G0 = spans + s.A0;
    it.G1 = spans + s.A1;
    it.N0 = s.N0;
    it.N1 = s.N1;
    it.KeyRows = keyRows;
    it.Round = s.Round0;
    it.J0 = s.J0;
    it.Hi = s.Hi;
    it.Valid = s.Valid != 0;
}

template <int D, bool QK_I8, bool HAS_VSCALE, bool HAS_ALIBI>
__global__ void __launch_bounds__(FWD_THREADS, 2) FwdSm100Kernel(const __grid_constant__ CUtensorMap tmQ,
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, TFwdParams p)
{
    using SM = TFwdSmem<D>;
    constexpr int STAGES = SM::STAGES;
    constexpr bool SEP_P = (D == 64); // P has its own tensor-memory columns
    constexpr int SWZ = (D == 128) ? 128 : 64;
    constexpr uint32_t GROUP_BYTES = 8 * D; // 8 rows of a tile
    constexpr uint32_t IDESC_QK = QK_I8 ? MakeInstrDesc(2, 1, 1, 0, 0, TILE_M, TILE_N) : MakeInstrDesc(1, 0, 0, 0, 0, TILE_M, TILE_N);
    constexpr uint32_t IDESC_PV = MakeInstrDesc(1, 0, 0, 0, 1, TILE_M, D);
    constexpr int BAR_PAIR0 = 1;     // + (warp & 3): the two warps that share 32 rows
    constexpr int HALF_N = TILE_N / 2;
    constexpr int HALF_D = D / 2;

    extern __shared__ __align__(1024) uint8_t smem[]; // tiles need 1024-byte alignment for the 128 B swizzle
    uint8_t *sQ = smem + SM::Q_OFF;
    uint8_t *sK = smem + SM::K_OFF;
    uint8_t *sV = smem + SM::V_OFF;
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
        for (int s = 0; s < ITEM_RING; ++s) {
            MbarInit(&misc.BarItem[s], 1);
            MbarInit(&misc.BarItemEmpty[s], SOFTMAX_WARPS + 1);
        }
        for (int s = 0; s < 2; ++s) {
            MbarInit(&misc.BarQFull[s], 1);
            MbarInit(&misc.BarQEmpty[s], 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            MbarInit(&misc.BarFull[s], 1);
            MbarInit(&misc.BarEmpty[s], 1);
        }
        MbarInit(&misc.BarS, 1);
        MbarInit(&misc.BarSRead, SOFTMAX_WARPS);
        MbarInit(&misc.BarP, SOFTMAX_WARPS);
        MbarInit(&misc.BarPV, 1);
        misc.Abort = 0;
        FenceBarrierInit();
    }
    if (warp == MMA_WARP) {
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
    const int totalItems = p.QTiles * p.HeadCount;
    const int *abortFlag = &misc.Abort;
    auto giveUp = [&](int code) {
        *(volatile int *)&misc.Abort = 1;
        if (p.Status) {
            atomicOr(p.Status, code);
        }
    };

    if (warp >= SOFTMAX_WARPS) {
        RegDealloc<CONTROL_REGS>();
        if (warp == LOAD_WARP) {
            // ------------------------------------------------------------ loader warp
            if (lane == 0) {
                PrefetchTensorMap(&tmQ);
                PrefetchTensorMap(&tmK);
                PrefetchTensorMap(&tmV);
            }
            int g = 0;          // tiles issued into the K/V ring
            int nq = 0;         // Q tiles requested (items that have key tiles)
            bool failed = false;
            for (int k = 0; !failed; ++k) {
                int item = 0;
                if (lane == 0) {
                    item = atomicAdd(p.Counter, 1);
                }
                item = __shfl_sync(0xffffffffu, item, 0);
                const bool last = item >= totalItems;
                const int qTile = last ? -1 : p.QTiles - 1 - item / p.HeadCount; // late (long) rows first
                const int head = last ? 0 : item % p.HeadCount;
                TTileIter iter;
                iter.Valid = false;
                int a0 = 0, a1 = 0;
                int ss[4], sf[4];
                float sqv[4];
                float vRef = 0;
                if (!last) {
                    iter.Init(p.Spans, p.SpanPtr, p.LenAttTiles, qTile, p.KeyRows);
                    a0 = iter.G0 ? (int)(iter.G0 - p.Spans) : 0;
                    a1 = iter.G1 ? (int)(iter.G1 - p.Spans) : 0;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int r = lane + 32 * q;
                        const tsa_span_group *gp = (r < 64) ? iter.G0 : iter.G1;
                        const int n = (r < 64) ? iter.N0 : iter.N1;
                        ss[q] = 1;
                        sf[q] = 0;
                        if (iter.Valid && iter.Round < n) {
                            ss[q] = gp[iter.Round].SpanStart[r & 63];
                            sf[q] = gp[iter.Round].SpanFinish[r & 63];
                        }
                        const int row = qTile * TILE_M + r;
                        sqv[q] = 0;
                        if (row < p.OutRows) {
                            sqv[q] = p.QScale.Valid() ? p.QScale.Row(head)[row] : p.QkVecScale;
                        }
                    }
                    if (HAS_VSCALE) {
                        vRef = p.VRef[head];
                    }
                }
                const float svMult = (HAS_VSCALE && vRef > 0) ? 1.0f / vRef : 0.0f; // sv_j / svRef <= 1; the factor 128 sits in the exponent
                const int slotIdx = k & (ITEM_RING - 1);
                if (lane == 0) {
                    if (k >= ITEM_RING && !WaitBarA(&misc.BarItemEmpty[slotIdx], ((k / ITEM_RING) - 1) & 1, abortFlag)) {
                        failed = true;
                        giveUp(kDevTimeoutMma);
                    }
                }
                failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
                if (failed) {
                    break;
                }
                TItemSlot &slot = misc.Item[slotIdx];
                if (!last) {
                    int maxS = max(max(ss[0], ss[1]), max(ss[2], ss[3]));
                    int minF = min(min(sf[0], sf[1]), min(sf[2], sf[3]));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        maxS = max(maxS, __shfl_xor_sync(0xffffffffu, maxS, o));
                        minF = min(minF, __shfl_xor_sync(0xffffffffu, minF, o));
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        slot.SpanS[lane + 32 * q] = ss[q];
                        slot.SpanF[lane + 32 * q] = sf[q];
                        slot.SQ[lane + 32 * q] = sqv[q];
                    }
                    if (lane == 0) {
                        slot.Head = head;
                        slot.N0 = iter.N0;
                        slot.N1 = iter.N1;
                        slot.A0 = a0;
                        slot.A1 = a1;
                        slot.Round0 = iter.Round;
                        slot.J0 = iter.J0;
                        slot.Hi = iter.Hi;
                        slot.Valid = iter.Valid ? 1 : 0;
                        slot.MaxS = maxS;
                        slot.MinF = minF;
                        slot.VRef = vRef;
                    }
                }
                if (lane == 0) {
                    slot.QTile = qTile;
                }
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&misc.BarItem[slotIdx]);
                }
                if (last) {
                    break;
                }
                if (iter.Valid) {
                    if (lane == 0) {
                        const int qb = nq & 1;
                        // the buffer was last read by the QK^T products of the item two Q tiles back
                        if (nq >= 2 && !WaitBarA(&misc.BarQEmpty[qb], ((nq >> 1) - 1) & 1, abortFlag)) {
                            failed = true;
                            giveUp(kDevTimeoutMma);
                        } else {
                            MbarExpectTx(&misc.BarQFull[qb], SM::TILE_BYTES);
                            TmaLoad2D(sQ + qb * SM::TILE_BYTES, &tmQ, head * D, qTile * TILE_M, &misc.BarQFull[qb]);
                        }
                    }
                    ++nq;
                    failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
                }
                while (iter.Valid && !failed) {
                    const int stage = g % STAGES;
                    if (lane == 0) {
                        if (g >= STAGES && !WaitBarA(&misc.BarEmpty[stage], ((g / STAGES) - 1) & 1, abortFlag)) {
                            failed = true;
                            giveUp(kDevTimeoutMma);
                        } else {
                            MbarExpectTxOnly(&misc.BarFull[stage], 2 * SM::TILE_BYTES);
                            TmaLoad2D(sK + stage * SM::TILE_BYTES, &tmK, head * D, iter.J0, &misc.BarFull[stage]);
                            TmaLoad2D(sV + stage * SM::TILE_BYTES, &tmV, head * D, iter.J0, &misc.BarFull[stage]);
                        }
                    }
                    failed = __shfl_sync(0xffffffffu, failed ? 1 : 0, 0) != 0;
                    if (failed) {
                        break;
                    }
                    {
                        const float *ksRow = p.KScale.Row(head);
                        const float *vsRow = HAS_VSCALE ? p.VScale.Row(head) : nullptr;
                        float kq[4], vq[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int j = iter.J0 + lane + 32 * q;
                            kq[q] = 0;
                            vq[q] = 0;
                            if (j < p.KeyRows) {
                                kq[q] = ksRow[j];
                                if (HAS_VSCALE) {
                                    vq[q] = vsRow[j];
                                }
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            misc.Sk[stage][lane + 32 * q] = kq[q];
                            if (HAS_VSCALE) {
                                misc.Sv[stage][lane + 32 * q] = vq[q] * svMult;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        MbarArrive(&misc.BarFull[stage]);
                    }
                    ++g;
                    iter.Advance();
                }
            }
            if (*(volatile int *)&misc.Abort) {
                // drain copies that were requested, so none lands after the CTA is gone
                if (lane == 0) {
                    for (int t = max(0, g - STAGES); t < g; ++t) {
                        WaitBar(&misc.BarFull[t % STAGES], (t / STAGES) & 1);
                    }
                    if (nq > 0) {
                        WaitBar(&misc.BarQFull[(nq - 1) & 1], ((nq - 1) >> 1) & 1);
                    }
                }
            }
            __syncwarp();
        } else if (warp == MMA_WARP) {
            // ------------------------------------------------------------ MMA warp
            if (lane == 0) {
                const uint32_t sQa = SmemAddr(sQ), sKa = SmemAddr(sK), sVa = SmemAddr(sV);
                auto issuePV = [&](int stage, bool accumulate, bool withResidual) {
                    const uint32_t vAddr = sVa + stage * SM::TILE_BYTES;
#pragma unroll
                    for (int ks = 0; ks < TILE_N / 32; ++ks) {
                        uint64_t bDesc = MakeSmemDesc(vAddr + ks * 32 * D, 16, GROUP_BYTES, SWZ);
                        // D = 64: P is one 32-column block; D = 128: P of chunk ks sits at S columns 32 ks .. 32 ks + 7
                        uint32_t aCol = SEP_P ? TMEM_P_COL + ks * 8 : (uint32_t)(ks * 32);
                        MmaF8TS(tmem + TMEM_O_COL, tmem + aCol, bDesc, IDESC_PV, (accumulate || ks > 0) ? 1u : 0u);
                    }
                    if (withResidual) {
#pragma unroll
                        for (int ks = 0; ks < TILE_N / 32; ++ks) {
                            uint64_t bDesc = MakeSmemDesc(vAddr + ks * 32 * D, 16, GROUP_BYTES, SWZ);
                            uint32_t aCol = SEP_P ? TMEM_P_COL + 32 + ks * 8 : (uint32_t)(ks * 32 + 8);
                            MmaF8TS(tmem + TMEM_O_COL, tmem + aCol, bDesc, IDESC_PV, 1u);
                        }
                    }
                };
                auto issueQK = [&](int qb, int stage) {
                    const uint32_t qAddr = sQa + qb * SM::TILE_BYTES;
                    const uint32_t kAddr = sKa + stage * SM::TILE_BYTES;
#pragma unroll
                    for (int ks = 0; ks < D / 32; ++ks) {
                        uint64_t aDesc = MakeSmemDesc(qAddr + ks * 32, 16, GROUP_BYTES, SWZ);
                        uint64_t bDesc = MakeSmemDesc(kAddr + ks * 32, 16, GROUP_BYTES, SWZ);
                        if (QK_I8) {
                            MmaI8SS(tmem, aDesc, bDesc, IDESC_QK, ks > 0);
                        } else {
                            MmaF8SS(tmem, aDesc, bDesc, IDESC_QK, ks > 0);
                        }
                    }
                };
                int t = 0;  // tiles issued so far (parity of BarS / BarSRead / BarP / BarPV and ring position)
                int nq = 0; // items with key tiles so far (Q buffer and its barriers' parity)
                bool pending = false, pendAccum = false, pendMasked = false;
                int pendStage = 0;
                bool failed = false;
                // P V of the previous tile: needs its weights; frees the ring stage and the P columns when it retires
                auto flushPV = [&]() {
                    if (!WaitBarA<true>(&misc.BarP, (t - 1) & 1, abortFlag)) {
                        failed = true;
                        giveUp(kDevTimeoutMma);
                        return;
                    }
                    TcFenceAfter();
                    issuePV(pendStage, pendAccum, pendMasked);
                    MmaCommit(&misc.BarPV);
                    MmaCommit(&misc.BarEmpty[pendStage]);
                    pending = false;
                };
                for (int k = 0; !failed; ++k) {
                    const int slotIdx = k & (ITEM_RING - 1);
                    if (!WaitBarA(&misc.BarItem[slotIdx], (k / ITEM_RING) & 1, abortFlag)) {
                        failed = true;
                        giveUp(kDevTimeoutTma);
                        break;
                    }
                    const TItemSlot &slot = misc.Item[slotIdx];
                    const int qTile = slot.QTile;
                    TTileIter iter;
                    iter.Valid = false;
                    int maxS = 0, minF = 0, round0 = 0;
                    if (qTile >= 0) {
                        IterFromSlot(iter, slot, p.Spans, p.KeyRows);
                        maxS = slot.MaxS;
                        minF = slot.MinF;
                        round0 = slot.Round0;
                    }
                    MbarArrive(&misc.BarItemEmpty[slotIdx]);
                    if (qTile < 0) {
                        break;
                    }
                    if (!iter.Valid) {
                        continue;
                    }
                    const int qb = nq & 1;
                    for (int it = 0; iter.Valid && !failed; ++it, iter.Advance()) {
                        const int stage = t % STAGES;
                        if (!WaitBarA(&misc.BarFull[stage], (t / STAGES) & 1, abortFlag) ||
                            (it == 0 && !WaitBarA(&misc.BarQFull[qb], (nq >> 1) & 1, abortFlag))) {
                            failed = true;
                            giveUp(kDevTimeoutTma);
                            break;
                        }
                        if (SEP_P) {
                            if (t > 0 && !WaitBarA<true>(&misc.BarSRead, (t - 1) & 1, abortFlag)) {
                                failed = true;
                                giveUp(kDevTimeoutMma);
                                break;
                            }
                            TcFenceAfter();
                            issueQK(qb, stage);
                            MmaCommit(&misc.BarS);
                            if (pending) {
                                flushPV();
                            }
                        } else {
                            if (pending) {
                                flushPV();
                                if (failed) {
                                    break;
                                }
                            }
                            TcFenceAfter();
                            issueQK(qb, stage);
                            MmaCommit(&misc.BarS);
                        }
                        pending = true;
                        pendStage = stage;
                        pendAccum = it > 0;
                        pendMasked = !(iter.Round == round0 && iter.J0 >= maxS && iter.J0 + TILE_N - 1 <= minF);
                        ++t;
                    }
                    // the Q buffer is free once this item's QK^T products have retired
                    MmaCommit(&misc.BarQEmpty[qb]);
                    ++nq;
                }
                if (pending && !failed) {
                    flushPV();
                }
            }
            __syncwarp();
        }
    } else {
        RegAlloc<SOFTMAX_REGS>();
        // ---------------------------------------------------------------- softmax warps
        const int half = tid >> 7;
        const int r = tid & (TILE_M - 1);
        const int colBase = half * HALF_N;
        const uint32_t tLane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int pairBar = BAR_PAIR0 + (warp & 3);
        // packed weights of chunk ch: 8 columns (plus 8 for the residual); D = 128: inside the chunk's own S columns
        auto PHiCol = [](int ch) { return SEP_P ? TMEM_P_COL + (uint32_t)ch * 8 : (uint32_t)ch * 32; };
        auto PLoCol = [](int ch) { return SEP_P ? TMEM_P_COL + 32 + (uint32_t)ch * 8 : (uint32_t)ch * 32 + 8; };
        const float g = p.GlobalScale ? *p.GlobalScale : 1.0f;

        int t = 0; // tiles processed by this CTA (barrier parities, ring position)
        bool failed = false;
        for (int k = 0; !failed; ++k) {
            const int slotIdx = k & (ITEM_RING - 1);
            if (!WaitBarA(&misc.BarItem[slotIdx], (k / ITEM_RING) & 1, abortFlag)) {
                failed = true;
                giveUp(kDevTimeoutTma);
                break;
            }
            const TItemSlot &slot = misc.Item[slotIdx];
            const int qTile = slot.QTile;
            TTileIter cur;
            cur.Valid = false;
            int head = 0, round0 = 0, maxS = 0, minF = 0, span0S = 1, span0F = 0;
            float sq = 0, vRef = 0;
            if (qTile >= 0) {
                IterFromSlot(cur, slot, p.Spans, p.KeyRows);
                head = slot.Head;
                round0 = slot.Round0;
                maxS = slot.MaxS;
                minF = slot.MinF;
                span0S = slot.SpanS[r];
                span0F = slot.SpanF[r];
                sq = slot.SQ[r];
                vRef = slot.VRef;
            }
            __syncwarp();
            if (lane == 0) {
                MbarArrive(&misc.BarItemEmpty[slotIdx]);
            }
            if (qTile < 0) {
                break;
            }
            const int row = qTile * TILE_M + r;
            const bool rowOk = row < p.OutRows;
            // a zero query scale would turn masked (-inf) scores into NaN; a tiny positive one keeps every logit at ~0
            const float rowMult = fmaxf(sq * p.C * g, 1e-30f);
            const float2 rowMult2 = make_float2(rowMult, rowMult);

            int spanS = span0S, spanF = span0F, spanRound = round0;
            float m = 0;
            float2 lacc2 = make_float2(0.0f, 0.0f); // 128 * sum of this thread's weights
            int it = 0;
            while (cur.Valid) {
                if (cur.Round != spanRound) {
                    spanS = 1;
                    spanF = 0;
                    const tsa_span_group *gp = (r < 64) ? cur.G0 : cur.G1;
                    const int n = (r < 64) ? cur.N0 : cur.N1;
                    if (cur.Round < n) {
                        spanS = gp[cur.Round].SpanStart[r & 63];
                        spanF = gp[cur.Round].SpanFinish[r & 63];
                    }
                    spanRound = cur.Round;
                }
                const int stage = t % STAGES;
                const int j0 = cur.J0;
                // P carries a residual part on every tile that is not interior to all 128 rows (same rule in the MMA warp)
                const bool tileMasked = !(cur.Round == round0 && j0 >= maxS && j0 + TILE_N - 1 <= minF);
                // The four 32-column chunks of the tile are shared between the two threads of a row.  On an interior tile
                // thread h takes chunks h and h + 2.  On a masked tile only the chunks some row of the warp attends are
                // computed (both warps of a pair hold the same rows, so they agree) and they are dealt out alternately,
                // which keeps the pair balanced on window layers where the attended band covers two or three chunks.
                int ls = 0, lf = TILE_N - 1; // the row's span in tile-local columns
                bool warpMasked = false;
                int chKeep = half, chAgain = half + 2; // chunk kept in registers / chunk read twice (-1: none)
                unsigned zeroMask = 0;                 // chunks this thread fills with zero weights
                if (tileMasked) {
                    ls = spanS - j0;
                    lf = spanF - j0;
                    warpMasked = !__all_sync(0xffffffffu, ls <= 0 && lf >= TILE_N - 1);
                    if (warpMasked) {
                        unsigned need = 0;
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            if (__any_sync(0xffffffffu, ls <= ch * 32 + 31 && lf >= ch * 32 && ls <= lf)) {
                                need |= 1u << ch;
                            }
                        }
                        chKeep = -1;
                        chAgain = -1;
                        int pos = 0;
#pragma unroll
                        for (int ch = 0; ch < 4; ++ch) {
                            if (need & (1u << ch)) {
                                if ((pos & 1) == half) {
                                    if (chKeep < 0) {
                                        chKeep = ch;
                                    } else {
                                        chAgain = ch;
                                    }
                                }
                                ++pos;
                            } else if ((ch & 1) == half) {
                                zeroMask |= 1u << ch;
                            }
                        }
                    }
                }

                // the staged key scales (the wait also makes the loader's shared-memory writes visible), then S(t)
                // A thread whose wait ran out does not leave alone: it carries `failed` to the next barrier of its
                // pair (a reduction), so both threads of a row leave together and no named barrier is left waiting.
                if (!failed && (!WaitBarA(&misc.BarFull[stage], (t / STAGES) & 1, abortFlag) || !WaitBarA(&misc.BarS, t & 1, abortFlag))) {
                    failed = true;
                    giveUp(kDevTimeoutMma);
                }
                TcFenceAfter();
                const float *skBuf = misc.Sk[stage];
                const float *svBuf = misc.Sv[stage];
                const float *alBuf = misc.Al;

                // Register budget: only 32 scores stay in registers.  Chunk chAgain is read for the maximum, dropped, and
                // read again for the weights; chunk chKeep is read once and kept.  S is released to the MMA warp after the
                // last read, about half-way through the tile.
                float2 s[16];
                // u = S * sk (+ ALiBi, then already multiplied by the row factor), masked, left in s[]; returns the maximum
                auto scaleChunk = [&](auto maskedTag, int ch) {
                    constexpr bool MASKED = decltype(maskedTag)::value;
                    // span in chunk-local columns, clipped so that (unsigned)(c - lsH) <= spanW  <=>  ls <= col <= lf
                    const int lsC = max(ls, ch * 32), lfC = min(lf, ch * 32 + 31);
                    const int lsH = lsC - ch * 32;
                    const unsigned spanW = (lsC <= lfC) ? (unsigned)(lfC - lsC) : 0u;
                    const float4 *sk4 = reinterpret_cast<const float4 *>(skBuf + ch * 32);
                    const float4 *al4 = reinterpret_cast<const float4 *>(alBuf + ch * 32);
                    float mx = -INFINITY;
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        const float4 k4 = sk4[c >> 2];
                        float2 x0 = s[c >> 1], x1 = s[(c >> 1) + 1];
                        if (QK_I8) {
                            x0 = IntPairToFloat(__float_as_uint(x0.x), __float_as_uint(x0.y));
                            x1 = IntPairToFloat(__float_as_uint(x1.x), __float_as_uint(x1.y));
                        }
                        x0 = __fmul2_rn(x0, make_float2(k4.x, k4.y));
                        x1 = __fmul2_rn(x1, make_float2(k4.z, k4.w));
                        if (HAS_ALIBI) {
                            const float4 a4 = al4[c >> 2];
                            x0 = __ffma2_rn(x0, rowMult2, make_float2(a4.x, a4.y));
                            x1 = __ffma2_rn(x1, rowMult2, make_float2(a4.z, a4.w));
                        }
                        if (MASKED) {
                            x0.x = ((unsigned)(c - lsH) <= spanW) ? x0.x : -INFINITY;
                            x0.y = ((unsigned)(c + 1 - lsH) <= spanW) ? x0.y : -INFINITY;
                            x1.x = ((unsigned)(c + 2 - lsH) <= spanW) ? x1.x : -INFINITY;
                            x1.y = ((unsigned)(c + 3 - lsH) <= spanW) ? x1.y : -INFINITY;
                        }
                        s[c >> 1] = x0;
                        s[(c >> 1) + 1] = x1;
                        mx = Max3(mx, x0.x, x0.y);
                        mx = Max3(mx, x1.x, x1.y);
                    }
                    if (MASKED && lsC > lfC) {
                        mx = -INFINITY; // spanW = 0 would otherwise let column lsH through
                    }
                    return mx;
                };
                auto loadChunk = [&](int ch) {
                    TmemLd32Pairs(tLane + ch * 32, s);
                    TmemWaitLd();
                };
                auto releaseS = [&]() {
                    if (SEP_P) {
                        TcFenceBefore();
                        __syncwarp();
                        if (lane == 0) {
                            MbarArrive(&misc.BarSRead);
                        }
                    }
                };
                float mx = -INFINITY;
                if (!failed) {
                    if (chAgain >= 0) {
                        loadChunk(chAgain);
                        mx = warpMasked ? scaleChunk(std::true_type(), chAgain) : scaleChunk(std::false_type(), chAgain);
                    }
                    if (chKeep >= 0) {
                        loadChunk(chKeep);
                        if (chAgain < 0) {
                            releaseS(); // nothing is read twice
                        }
                        mx = fmaxf(mx, warpMasked ? scaleChunk(std::true_type(), chKeep) : scaleChunk(std::false_type(), chKeep));
                    } else {
                        releaseS();
                    }
                }
                const float rowOff = HAS_ALIBI ? -p.Slope * (float)(row - j0) : 0.0f;
                float zmax = mx;
                if (!HAS_ALIBI) {
                    zmax = (mx == -INFINITY) ? mx : mx * rowMult;
                }
                misc.RowX[t & 1][half][r] = zmax + rowOff;
                if (BarRedOr(pairBar, 64, failed)) {
                    failed = true;
                    break;
                }
                const float tileMax = fmaxf(zmax + rowOff, misc.RowX[t & 1][half ^ 1][r]);
                const float newM = fmaxf(m, floorf(tileMax)); // -inf stays below m
                const float alpha = exp2f(m - newM);
                // P V(t-1) retired: O is current and the P columns may be overwritten
                if (t > 0) {
                    if (!WaitBarA(&misc.BarPV, (t - 1) & 1, abortFlag)) {
                        failed = true;
                        giveUp(kDevTimeoutMma);
                        cur.Advance();
                        ++it;
                        ++t;
                        continue; // to the next barrier of the pair
                    }
                    TcFenceAfter();
                }
                if (it > 0 && __any_sync(0xffffffffu, newM != m)) {
#pragma unroll
                    for (int c0 = 0; c0 < HALF_D; c0 += 32) {
                        uint32_t o[32];
                        TmemLd32(tLane + TMEM_O_COL + half * HALF_D + c0, o);
                        TmemWaitLd();
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                        }
                        TmemSt32(tLane + TMEM_O_COL + half * HALF_D + c0, o);
                    }
                }
                lacc2.x *= alpha;
                lacc2.y *= alpha;
                m = newM;
                // weights, packed e4m3.  A row that attends nothing in a chunk gets an offset of -inf there, so every
                // weight is 0 whatever the masking compare let through.
                const float eoff = rowOff - m + 7.0f;
                auto weightChunk = [&](auto residTag, int ch) {
                    constexpr bool RESID = decltype(residTag)::value;
                    const bool chunkEmpty = warpMasked && max(ls, ch * 32) > min(lf, ch * 32 + 31);
                    const float eo = chunkEmpty ? -INFINITY : eoff;
                    const float2 eoff2 = make_float2(eo, eo);
                    const float4 *sv4 = reinterpret_cast<const float4 *>(svBuf + ch * 32);
                    uint32_t pk[8], pl[8];
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {
                        float2 t0 = HAS_ALIBI ? __fadd2_rn(s[c >> 1], eoff2) : __ffma2_rn(s[c >> 1], rowMult2, eoff2);
                        float2 t1 = HAS_ALIBI ? __fadd2_rn(s[(c >> 1) + 1], eoff2) : __ffma2_rn(s[(c >> 1) + 1], rowMult2, eoff2);
                        float2 w0 = FastExp2Pair(t0), w1 = FastExp2Pair(t1);
                        lacc2 = __fadd2_rn(lacc2, w0);
                        lacc2 = __fadd2_rn(lacc2, w1);
                        if (HAS_VSCALE) {
                            const float4 v4 = sv4[c >> 2];
                            w0 = __fmul2_rn(w0, make_float2(v4.x, v4.y));
                            w1 = __fmul2_rn(w1, make_float2(v4.z, v4.w));
                        }
                        const uint32_t hi4 = PackE4M3x4(w0.x, w0.y, w1.x, w1.y);
                        pk[c >> 2] = hi4;
                        if (RESID) {
                            pl[c >> 2] = ResidualE4M3x2(w0.x, w0.y, hi4 & 0xffff) | (ResidualE4M3x2(w1.x, w1.y, hi4 >> 16) << 16);
                        }
                    }
                    TmemStN<8>(tLane + PHiCol(ch), pk);
                    if (RESID) {
                        TmemStN<8>(tLane + PLoCol(ch), pl);
                    }
                };
                if (chKeep >= 0) {
                    if (tileMasked) {
                        weightChunk(std::true_type(), chKeep);
                    } else {
                        weightChunk(std::false_type(), chKeep);
                    }
                }
                if (chAgain >= 0) {
                    // second read of this chunk's scores, after which S belongs to the next QK^T
                    loadChunk(chAgain);
                    releaseS();
                    if (warpMasked) {
                        scaleChunk(std::true_type(), chAgain);
                    } else {
                        scaleChunk(std::false_type(), chAgain);
                    }
                    if (tileMasked) {
                        weightChunk(std::true_type(), chAgain);
                    } else {
                        weightChunk(std::false_type(), chAgain);
                    }
                }
                if (zeroMask) {
                    uint32_t z[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        z[q] = 0;
                    }
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch) {
                        if (zeroMask & (1u << ch)) {
                            TmemStN<8>(tLane + PHiCol(ch), z);
                            TmemStN<8>(tLane + PLoCol(ch), z);
                        }
                    }
                }
                TmemWaitSt();
                TcFenceBefore();
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&misc.BarP);
                }
                cur.Advance();
                ++it;
                ++t;
            }
            const int tiles = it;
            if (!failed && tiles > 0) {
                if (!WaitBarA(&misc.BarPV, (t - 1) & 1, abortFlag)) {
                    failed = true;
                    giveUp(kDevTimeoutMma);
                }
                TcFenceAfter();
            }
            // total weight of the row: both halves (the exchange buffer of the parity no tile is using)
            misc.RowX[t & 1][half][r] = lacc2.x + lacc2.y;
            if (BarRedOr(pairBar, 64, failed)) {
                failed = true;
                break;
            }
            const float lTot = (lacc2.x + lacc2.y + misc.RowX[t & 1][half ^ 1][r]) * (1.0f / 128.0f) + exp2f(-m);
            BarSync(pairBar, 64); // the partner has read before the next item's first tile may write this buffer
            const float outMult = (HAS_VSCALE ? vRef : p.VVecScale) * (1.0f / 128.0f) / lTot;
            if (rowOk && half == 0 && p.Lse.Valid()) {
                p.Lse.Row(head)[row] = m + log2f(lTot);
            }
            const int esz = (p.OutDtype == TSA_F32) ? 4 : 2;
            char *oRow = p.Out.Row(rowOk ? row : 0) + ((size_t)head * D + half * HALF_D) * esz;
#pragma unroll
            for (int c0 = 0; c0 < HALF_D; c0 += 32) {
                uint32_t o[32];
                if (tiles > 0) {
                    TmemLd32(tLane + TMEM_O_COL + half * HALF_D + c0, o);
                    TmemWaitLd();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        o[c] = 0;
                    }
                }
                if (rowOk) {
                    if (p.OutDtype == TSA_F32) {
                        float4 *dst = reinterpret_cast<float4 *>(oRow + c0 * 4);
#pragma unroll
                        for (int c = 0; c < 32; c += 4) {
                            dst[c >> 2] = make_float4(__uint_as_float(o[c]) * outMult, __uint_as_float(o[c + 1]) * outMult,
                                __uint_as_float(o[c + 2]) * outMult, __uint_as_float(o[c + 3]) * outMult);
                        }
                    } else {
                        uint4 *dst = reinterpret_cast<uint4 *>(oRow + c0 * 2);
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                float a = __uint_as_float(o[c + 2 * q]) * outMult, b = __uint_as_float(o[c + 2 * q + 1]) * outMult;
                                if (p.OutDtype == TSA_BF16) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                                    w[q] = *reinterpret_cast<uint32_t *>(&h);
                                } else {
                                    w[q] = PackHalf2(a, b);
                                }
                            }
                            dst[c >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
            // the next item's first P V overwrites O: its P arrival (after these loads in program order) orders it
            TcFenceBefore();
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == MMA_WARP) {
        TmemDealloc(tmem, TMEM_COLS);
    }
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

// ---- raw int32 score tiles (parity hook for the kind::i8 accumulators) -------------------------
struct TScoreMisc {
    uint64_t BarQ, BarMma;
    uint32_t TmemBase;
};

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
    TScoreMisc &misc = *reinterpret_cast<TScoreMisc *>(smem + 2 * 128 * D);
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
    if (cfg->v_dtype != TSA_E4M3) {
        return false; // int8 values take the generic kernels (exact fp32 accumulation)
    }
    return TmaCompatible(qk) && TmaCompatible(qv) && TmaCompatible(v);
}

// per-head V-scale maxima, then the work-item counter
static size_t VRefBytes(int headCount)
{
    return (size_t)((headCount * sizeof(float) + 255) / 256 * 256);
}
size_t Sm100FwdWorkspaceBytes(int headCount)
{
    return VRefBytes(headCount) + 256;
}

static int SmCount()
{
    static int count[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        return 148;
    }
    if (count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            n = 148;
        }
        count[dev] = n;
    }
    return count[dev];
}

template <int D, bool QK_I8, bool HAS_VSCALE, bool HAS_ALIBI>
static int LaunchFwdT(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const TFwdParams &fp, int qTiles, cudaStream_t stream)
{
    auto kern = FwdSm100Kernel<D, QK_I8, HAS_VSCALE, HAS_ALIBI>;
    int smemBytes = TFwdSmem<D>::TOTAL;
    int rc = CheckCuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes), "cudaFuncSetAttribute(forward)");
    if (rc != TSA_OK) {
        return rc;
    }
    const int items = qTiles * fp.HeadCount;
    const int resident = 2 * SmCount();
    dim3 grid(items < resident ? items : resident);
    kern<<<grid, FWD_THREADS, smemBytes, stream>>>(mq, mk, mv, fp);
    return CheckCuda(cudaGetLastError(), "tcgen05 forward launch");
}

int LaunchSm100Fwd(const tsa_att_cfg *cfg, const TGenParams &p, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v,
    int lenAttTiles, int keyRows, void *workspace, int *statusWord, cudaStream_t stream)
{
    const int D = cfg->head_dim_qk;
    CUtensorMap mq, mk, mv;
    int rc = MakeTileMap(&mq, qk, D, "qk");
    if (rc == TSA_OK) {
        rc = MakeTileMap(&mk, qv, D, "qv");
    }
    if (rc == TSA_OK) {
        rc = MakeTileMap(&mv, v, D, "v");
    }
    if (rc != TSA_OK) {
        return rc;
    }
    TFwdParams fp;
    fp.HeadCount = p.HeadCount;
    fp.OutRows = p.Len;
    fp.KeyRows = keyRows;
    fp.LenAttTiles = lenAttTiles;
    fp.Spans = p.Spans;
    fp.SpanPtr = p.SpanPtr;
    fp.QScale = p.QScale;
    fp.KScale = p.KScale;
    fp.VScale = p.VScale;
    fp.VRef = nullptr;
    fp.Out = p.Out;
    fp.Lse = p.Lse;
    fp.GlobalScale = p.GlobalScale;
    fp.C = p.C;
    fp.QkVecScale = p.QkVecScale;
    fp.VVecScale = p.VVecScale;
    fp.Slope = p.Slope;
    fp.OutDtype = p.OutDtype;
    fp.Status = statusWord;
    const bool hasVs = p.VScale.Data != nullptr;
    const int qTiles = (lenAttTiles + 1) / 2;
    fp.QTiles = qTiles;
    fp.Counter = (int *)((char *)workspace + VRefBytes(p.HeadCount));
    rc = CheckCuda(cudaMemsetAsync(workspace, 0, Sm100FwdWorkspaceBytes(p.HeadCount), stream), "clearing the forward workspace");
    if (rc != TSA_OK) {
        return rc;
    }
    if (hasVs) {
        fp.VRef = (const float *)workspace;
        dim3 vgrid((keyRows + VREF_CHUNK - 1) / VREF_CHUNK, p.HeadCount);
        VRefKernel<<<vgrid, 256, 0, stream>>>(p.VScale, keyRows, (float *)workspace);
    }
    const bool i8 = cfg->qk_dtype == TSA_I8;
    const bool alibi = p.Slope != 0.0f;
#define TSA_FWD_CASE(DD, I8, VS)                                                                         \
    if (D == DD && i8 == I8 && hasVs == VS) {                                                            \
        return alibi ? LaunchFwdT<DD, I8, VS, true>(mq, mk, mv, fp, qTiles, stream)                      \
                     : LaunchFwdT<DD, I8, VS, false>(mq, mk, mv, fp, qTiles, stream);                    \
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
