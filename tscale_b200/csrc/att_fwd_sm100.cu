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
// One CTA = one head x 128 query rows (two 64-row span blocks).  Eight softmax warps, two threads per row
// (each owns 64 of the row's 128 score columns; a row is one tensor-memory lane), plus a control warp whose
// lane 0 issues every TMA copy and every MMA.  Tensor memory: columns [0,128) S (f32 / s32); each half writes its
// packed e4m3 weights (16 columns, plus 16 for the residual) back over its own S columns; columns [128, 128 + D)
// hold O (f32).  256 columns are allocated so two CTAs share an SM and one CTA's softmax overlaps the other's
// MMAs.  Shared memory: Q tile, STAGES x (K tile, V tile) filled by TMA with the 128 B (D = 128) or 64 B (D = 64)
// swizzle the MMA descriptors expect.  Softmax arithmetic uses packed f32x2 multiply-adds and 3-input max.
// Key tiles follow the reference's grouped spans: for round r the tiles [Start, Finish] of the two blocks'
// r-th groups; 32-column chunks no row of a warp attends cost no exponentials (window layers).
// Every barrier wait is bounded; when one runs out the kernel records a code in *statusWord, drains its
// outstanding copies, frees its tensor memory and returns.
#include "att_internal.cuh"
#include "att_sm100_common.cuh"

namespace tsa {

using namespace sm100;

constexpr int SOFTMAX_THREADS = 256;
constexpr int CTRL_WARP = SOFTMAX_THREADS / 32;
constexpr int FWD_THREADS = SOFTMAX_THREADS + 32;
constexpr int SCORE_THREADS = 128;
constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t TMEM_O_COL = 128;

// Phase trace for profiling builds (-DTSA_FWD_TRACE): thread 0 of a few CTAs records clock64() at the phases of
// a CTA's life; tsa_debug_trace copies the buffer out.
#ifdef TSA_FWD_TRACE
__device__ long long g_trace[4096];
#define TRC(e) do { if (traceOn) g_trace[traceSlot * 16 + (e)] = clock64(); } while (0)
#else
#define TRC(e) do { } while (0)
#endif

struct TFwdParams {
    int HeadCount;
    int OutRows;      // rows of out that may be written
    int KeyRows;      // rows of K / V
    int LenAttTiles;  // number of 64-row span blocks
    const tsa_span_group *Spans;
    const int *SpanPtr;
    P2D<float> QScale, KScale, VScale;
    const float *VRef; // per head max of VScale (workspace), null without VScale
    P2D<char> Out;
    P2D<float> Lse;
    const float *GlobalScale;
    float C;
    float QkVecScale, VVecScale;
    float Slope;
    int OutDtype;
    int *Status;
};

template <int D>
struct TFwdSmem {
    static constexpr int STAGES = (D == 64) ? 3 : 2;
    static constexpr int TILE_BYTES = 128 * D;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = TILE_BYTES;
    static constexpr int V_OFF = K_OFF + STAGES * TILE_BYTES;
    static constexpr int MISC_OFF = V_OFF + STAGES * TILE_BYTES;
    static constexpr int TOTAL = MISC_OFF + 4096 + 1024; // misc + alignment slack
};

struct TFwdMisc {
    float Sk[2][TILE_N];     // key scale of each column of the tile, double buffered by tile parity: fast warps
    float Sv[2][TILE_N];     // stage the next tile's scales while slower warps still read the current ones
    float Al[TILE_N];        // ALiBi term slope * column (tile invariant)
    float RowX[2][TILE_M];   // exchange between the two threads of a row (tile max, final sum)
    int TileMasked[2];       // softmax -> control warp: P has a residual part for this tile
    int Abort;               // a bounded wait ran out somewhere in the CTA
    uint64_t BarQ;
    uint64_t BarFull[4];
    uint64_t BarMma;         // control -> softmax: S(it) ready (and PV(it-1) retired)
    uint64_t BarP;           // softmax -> control: P(it) written, 256 arrivals
    uint32_t TmemBase;
};

// Thread layout: warps 0-7 are softmax warps, two threads per query row: thread (half, row) with half = tid / 128
// owns columns [64 * half, 64 * half + 64) of the row's scores and columns [half * D/2, (half + 1) * D/2) of its
// output.  Warp 8 is the control warp: lane 0 issues every TMA copy and every MMA.
template <int D, bool QK_I8, bool HAS_VSCALE, bool HAS_ALIBI>
__global__ void __launch_bounds__(FWD_THREADS, 2) FwdSm100Kernel(const __grid_constant__ CUtensorMap tmQ,
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, TFwdParams p)
{
    using SM = TFwdSmem<D>;
    constexpr int STAGES = SM::STAGES;
    constexpr int SWZ = (D == 128) ? 128 : 64;
    constexpr uint32_t GROUP_BYTES = 8 * D; // 8 rows of a tile
    constexpr uint32_t IDESC_QK = QK_I8 ? MakeInstrDesc(2, 1, 1, 0, 0, TILE_M, TILE_N) : MakeInstrDesc(1, 0, 0, 0, 0, TILE_M, TILE_N);
    constexpr uint32_t IDESC_PV = MakeInstrDesc(1, 0, 0, 0, 1, TILE_M, D);
    constexpr int BAR_STAGE = 1;     // named barrier of the 256 softmax threads
    constexpr int BAR_PAIR0 = 2;     // + (warp & 3): the two warps that share 32 rows
    constexpr int HALF_N = TILE_N / 2;
    constexpr int HALF_D = D / 2;

    extern __shared__ __align__(1024) uint8_t smem[]; // tiles need 1024-byte alignment for the 128 B swizzle
    uint8_t *sQ = smem + SM::Q_OFF;
    uint8_t *sK = smem + SM::K_OFF;
    uint8_t *sV = smem + SM::V_OFF;
    TFwdMisc &misc = *reinterpret_cast<TFwdMisc *>(smem + SM::MISC_OFF);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int head = blockIdx.y;
    const int qTile = gridDim.x - 1 - blockIdx.x; // late (long) rows first
#ifdef TSA_FWD_TRACE
    const bool traceOn = tid == 0 && blockIdx.y == 5 && (blockIdx.x % 37) == 3 && blockIdx.x / 37 < 12;
    const int traceSlot = blockIdx.x / 37;
#endif
    TRC(0);

    if ((SmemAddr(smem) & 1023u) != 0) {
        // the launch did not honour the alignment: report instead of computing on mis-swizzled tiles
        if (tid == 0 && p.Status) {
            atomicOr(p.Status, kDevBadSpan);
        }
        return;
    }
    // the span groups of the tile are fetched first: two dependent global loads that overlap with the set-up below
    TTileIter cur;
    cur.Init(p.Spans, p.SpanPtr, p.LenAttTiles, qTile, p.KeyRows);
    TRC(1);
    if (tid == 0) {
        MbarInit(&misc.BarQ, 1);
        for (int s = 0; s < STAGES; ++s) {
            MbarInit(&misc.BarFull[s], 1);
        }
        MbarInit(&misc.BarMma, 1);
        MbarInit(&misc.BarP, SOFTMAX_THREADS);
        misc.Abort = 0;
        FenceBarrierInit();
    }
    if (warp == CTRL_WARP) {
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

    TRC(2);

    if (warp == CTRL_WARP) {
        // ---------------------------------------------------------------- control warp
        if ((tid & 31) == 0 && cur.Valid) {
            PrefetchTensorMap(&tmQ);
            PrefetchTensorMap(&tmK);
            PrefetchTensorMap(&tmV);
            const uint32_t sQa = SmemAddr(sQ), sKa = SmemAddr(sK), sVa = SmemAddr(sV);
            TTileIter prod = cur;
            int issued = 0, landed = 0;
            bool failed = false;
            auto issueLoad = [&](int slot, int j0) {
                MbarExpectTx(&misc.BarFull[slot], 2 * SM::TILE_BYTES);
                TmaLoad2D(sK + slot * SM::TILE_BYTES, &tmK, head * D, j0, &misc.BarFull[slot]);
                TmaLoad2D(sV + slot * SM::TILE_BYTES, &tmV, head * D, j0, &misc.BarFull[slot]);
            };
            auto issuePV = [&](int slot, bool accumulate, bool withResidual) {
                const uint32_t vAddr = sVa + slot * SM::TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < TILE_N / 32; ++ks) {
                    uint64_t bDesc = MakeSmemDesc(vAddr + ks * 32 * D, 16, GROUP_BYTES, SWZ);
                    uint32_t aCol = (ks >> 1) * HALF_N + (ks & 1) * 8; // P of half h sits at columns 64h .. 64h+15
                    MmaF8TS(tmem + TMEM_O_COL, tmem + aCol, bDesc, IDESC_PV, (accumulate || ks > 0) ? 1u : 0u);
                }
                if (withResidual) {
#pragma unroll
                    for (int ks = 0; ks < TILE_N / 32; ++ks) {
                        uint64_t bDesc = MakeSmemDesc(vAddr + ks * 32 * D, 16, GROUP_BYTES, SWZ);
                        uint32_t aCol = (ks >> 1) * HALF_N + 16 + (ks & 1) * 8;
                        MmaF8TS(tmem + TMEM_O_COL, tmem + aCol, bDesc, IDESC_PV, 1u);
                    }
                }
            };
            auto issueQK = [&](int slot) {
                const uint32_t kAddr = sKa + slot * SM::TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < D / 32; ++ks) {
                    uint64_t aDesc = MakeSmemDesc(sQa + ks * 32, 16, GROUP_BYTES, SWZ);
                    uint64_t bDesc = MakeSmemDesc(kAddr + ks * 32, 16, GROUP_BYTES, SWZ);
                    if (QK_I8) {
                        MmaI8SS(tmem, aDesc, bDesc, IDESC_QK, ks > 0);
                    } else {
                        MmaF8SS(tmem, aDesc, bDesc, IDESC_QK, ks > 0);
                    }
                }
            };
            auto fail = [&](int code) {
                failed = true;
                *(volatile int *)&misc.Abort = 1;
                if (p.Status) {
                    atomicOr(p.Status, code);
                }
            };

            MbarExpectTx(&misc.BarQ, SM::TILE_BYTES);
            TmaLoad2D(sQ, &tmQ, head * D, qTile * TILE_M, &misc.BarQ);
            for (int s = 0; s < STAGES && prod.Valid; ++s) {
                issueLoad(s, prod.J0);
                prod.Advance();
                ++issued;
            }
            if (!WaitBar(&misc.BarQ, 0)) {
                fail(kDevTimeoutTma);
            }
            int it = 0;
            TTileIter ctl = cur;
            for (; ctl.Valid && !failed; ++it, ctl.Advance()) {
                const int slot = it % STAGES;
                if (!WaitBar(&misc.BarFull[slot], (it / STAGES) & 1)) {
                    fail(kDevTimeoutTma);
                    break;
                }
                ++landed;
                if (it > 0) {
                    // P(it-1) written by all softmax threads
                    if (!WaitBar(&misc.BarP, (it - 1) & 1)) {
                        fail(kDevTimeoutMma);
                        break;
                    }
                    TcFenceAfter();
                    issuePV((it - 1) % STAGES, it - 1 > 0, misc.TileMasked[(it - 1) & 1] != 0);
                }
                TcFenceAfter();
                issueQK(slot);
                MmaCommit(&misc.BarMma);
                if (it > 0 && prod.Valid) {
                    // the slot of tile it-1 is free once PV(it-1) has retired, i.e. when this commit completes
                    if (!WaitBar(&misc.BarMma, it & 1)) {
                        fail(kDevTimeoutMma);
                        break;
                    }
                    issueLoad((it - 1) % STAGES, prod.J0);
                    prod.Advance();
                    ++issued;
                }
                if (*(volatile int *)&misc.Abort) {
                    failed = true;
                }
            }
            if (!failed && it > 0) {
                if (WaitBar(&misc.BarP, (it - 1) & 1)) {
                    TcFenceAfter();
                    issuePV((it - 1) % STAGES, it - 1 > 0, misc.TileMasked[(it - 1) & 1] != 0);
                } else {
                    fail(kDevTimeoutMma);
                }
            }
            MmaCommit(&misc.BarMma); // final phase (also releases softmax threads waiting after a failure)
            if (failed) {
                // drain copies that were requested but never consumed, so none lands after the CTA is gone
                for (int t = landed; t < issued; ++t) {
                    WaitBar(&misc.BarFull[t % STAGES], (t / STAGES) & 1);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- softmax warps
        const int half = tid >> 7;
        const int r = tid & (TILE_M - 1);
        const int row = qTile * TILE_M + r;
        const int colBase = half * HALF_N;
        const uint32_t tLane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int pairBar = BAR_PAIR0 + (warp & 3);

        const bool rowOk = row < p.OutRows;
        const float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
        float sq = 0;
        if (rowOk) {
            sq = p.QScale.Valid() ? p.QScale.Row(head)[row] : p.QkVecScale;
        }
        // a zero query scale would turn masked (-inf) scores into NaN; a tiny positive one keeps every logit at ~0
        const float rowMult = fmaxf(sq * p.C * g, 1e-30f);
        const float2 rowMult2 = make_float2(rowMult, rowMult);
        const float vRef = HAS_VSCALE ? p.VRef[head] : 0.0f;
        const float svMult = (HAS_VSCALE && vRef > 0) ? 1.0f / vRef : 0.0f; // sv_j / svRef <= 1; the factor 128 sits in the exponent

        int spanS = 1, spanF = 0, spanRound = -1;
        float m = 0;
        float2 lacc2 = make_float2(0.0f, 0.0f); // 128 * sum of this thread's weights
        float pfSk = 0, pfSv = 0;
        auto fetchScales = [&](int j0) {
            pfSk = 0;
            pfSv = 0;
            int j = j0 + tid;
            if (tid < TILE_N && j < p.KeyRows) {
                pfSk = p.KScale.Row(head)[j];
                if (HAS_VSCALE) {
                    pfSv = p.VScale.Row(head)[j] * svMult;
                }
            }
        };
        if (cur.Valid) {
            fetchScales(cur.J0);
        }
        bool failed = false;
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
            const int buf = it & 1;
            if (tid < TILE_N) {
                misc.Sk[buf][tid] = pfSk;
                if (HAS_VSCALE) {
                    misc.Sv[buf][tid] = pfSv;
                }
            }
            const int j0 = cur.J0;
            const int ls = spanS - j0, lf = spanF - j0; // span in tile-local columns
            const bool rowFull = ls <= 0 && lf >= TILE_N - 1;
            const bool warpMasked = !__all_sync(0xffffffffu, rowFull);
            // 32-column chunks of this thread's half that some row of the warp attends
            const bool any0 = __any_sync(0xffffffffu, ls <= colBase + 31 && lf >= colBase && ls <= lf);
            const bool any1 = __any_sync(0xffffffffu, ls <= colBase + 63 && lf >= colBase + 32 && ls <= lf);
            if (failed) {
                *(volatile int *)&misc.Abort = 1;
            }
            const bool tileMasked = BarRedOr(BAR_STAGE, SOFTMAX_THREADS, warpMasked);
            if (*(volatile int *)&misc.Abort) {
                failed = true;
                break;
            }
            TTileIter nxt = cur;
            nxt.Advance();
            if (nxt.Valid) {
                fetchScales(nxt.J0);
            }
            if (!WaitBar(&misc.BarMma, it & 1)) {
                failed = true;
                if (p.Status) {
                    atomicOr(p.Status, kDevTimeoutMma);
                }
            }
            TcFenceAfter();
            if (it < 4) {
                TRC(3 + 2 * it);
            }

            // The scores are read from tensor memory twice, 32 columns at a time (first for the row maximum, then for
            // the weights), which keeps the live registers of a thread at one chunk instead of its whole half row.
            // Masked and unmasked tiles run separate copies of the code (warp-uniform branches), so the common
            // unmasked tile pays for no compare / select.
            // span in half-local columns, clipped so that (unsigned)(c - lsH) <= spanW  <=>  ls <= c <= lf
            const int lsC = max(ls, colBase), lfC = min(lf, colBase + HALF_N - 1);
            const int lsH = lsC - colBase;
            const unsigned spanW = (lsC <= lfC) ? (unsigned)(lfC - lsC) : 0u;
            const bool rowEmpty = lsC > lfC;
            const float *skBuf = misc.Sk[buf] + colBase;
            const float *svBuf = misc.Sv[buf] + colBase;
            const float *alBuf = misc.Al + colBase;
            auto loadScaled = [&](auto maskedTag, int ch, float2 *u) {
                constexpr bool MASKED = decltype(maskedTag)::value;
                uint32_t sreg[32];
                TmemLd32(tLane + colBase + ch * 32, sreg);
                TmemWaitLd();
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const int lc = ch * 32 + c; // column inside this thread's half
                    float2 a = QK_I8 ? IntPairToFloat(sreg[c], sreg[c + 1]) : make_float2(__uint_as_float(sreg[c]), __uint_as_float(sreg[c + 1]));
                    float2 x = __fmul2_rn(a, *reinterpret_cast<const float2 *>(skBuf + lc));
                    if (HAS_ALIBI) {
                        x = __ffma2_rn(x, rowMult2, *reinterpret_cast<const float2 *>(alBuf + lc));
                    }
                    if (MASKED) {
                        // lsH / lfH: span in columns of this half; unsigned compare folds both bounds
                        x.x = ((unsigned)(lc - lsH) <= spanW) ? x.x : -INFINITY;
                        x.y = ((unsigned)(lc + 1 - lsH) <= spanW) ? x.y : -INFINITY;
                    }
                    u[c >> 1] = x;
                }
            };
            auto chunkMax = [&](auto maskedTag, int ch, float mxIn) {
                float2 u[16];
                loadScaled(maskedTag, ch, u);
                float mx = mxIn;
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    mx = Max3(mx, u[k].x, u[k].y);
                }
                return mx;
            };
            float mx = -INFINITY;
            if (warpMasked) {
                if (any0) {
                    mx = chunkMax(std::true_type(), 0, mx);
                }
                if (any1) {
                    mx = chunkMax(std::true_type(), 1, mx);
                }
                if (rowEmpty) {
                    mx = -INFINITY; // spanW = 0 would otherwise let column lsH through
                }
            } else {
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    mx = chunkMax(std::false_type(), ch, mx);
                }
            }
            const float rowOff = HAS_ALIBI ? -p.Slope * (float)(row - j0) : 0.0f;
            float zmax = mx;
            if (!HAS_ALIBI) {
                zmax = (mx == -INFINITY) ? mx : mx * rowMult;
            }
            misc.RowX[half][r] = zmax + rowOff;
            BarSync(pairBar, 64);
            const float tileMax = fmaxf(zmax + rowOff, misc.RowX[half ^ 1][r]);
            const float newM = fmaxf(m, floorf(tileMax)); // -inf stays below m
            const float alpha = exp2f(m - newM);
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
            // weights, packed e4m3 into this half's own S columns (both chunks are re-read before the first store)
            // an empty row gets eoff = -inf so that every weight is 0 whatever the compare above let through
            const float eoff = rowEmpty && warpMasked ? -INFINITY : rowOff - m + 7.0f;
            const float2 eoff2 = make_float2(eoff, eoff);
            auto chunkWeights = [&](auto maskedTag, auto residTag, int ch) {
                constexpr bool RESID = decltype(residTag)::value;
                uint32_t pk[8], pl[8];
                float2 u[16];
                loadScaled(maskedTag, ch, u);
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                    float2 e[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        float2 t = HAS_ALIBI ? __fadd2_rn(u[c + k], eoff2) : __ffma2_rn(u[c + k], rowMult2, eoff2);
                        float2 w = make_float2(FastExp2(t.x), FastExp2(t.y));
                        lacc2 = __fadd2_rn(lacc2, w);
                        e[k] = HAS_VSCALE ? __fmul2_rn(w, *reinterpret_cast<const float2 *>(svBuf + ch * 32 + 2 * (c + k))) : w;
                    }
                    const uint32_t hi4 = PackE4M3x4(e[0].x, e[0].y, e[1].x, e[1].y);
                    pk[c >> 1] = hi4;
                    if (RESID) {
                        pl[c >> 1] = ResidualE4M3x2(e[0].x, e[0].y, hi4 & 0xffff) | (ResidualE4M3x2(e[1].x, e[1].y, hi4 >> 16) << 16);
                    }
                }
                // the packed weights of a chunk land in S columns of chunk 0 of this half, which has been read by then
                TmemStN<8>(tLane + colBase + ch * 8, pk);
                if (RESID) {
                    TmemStN<8>(tLane + colBase + 16 + ch * 8, pl);
                }
            };
            auto zeroChunk = [&](int ch) {
                uint32_t z[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    z[k] = 0;
                }
                TmemStN<8>(tLane + colBase + ch * 8, z);
                TmemStN<8>(tLane + colBase + 16 + ch * 8, z);
            };
            if (warpMasked) {
                // masked tiles always carry the residual (tileMasked is true whenever any warp is masked)
                if (any0) {
                    chunkWeights(std::true_type(), std::true_type(), 0);
                } else {
                    zeroChunk(0);
                }
                if (any1) {
                    chunkWeights(std::true_type(), std::true_type(), 1);
                } else {
                    zeroChunk(1);
                }
            } else if (tileMasked) {
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    chunkWeights(std::false_type(), std::true_type(), ch);
                }
            } else {
#pragma unroll 1
                for (int ch = 0; ch < 2; ++ch) {
                    chunkWeights(std::false_type(), std::false_type(), ch);
                }
            }
            TmemWaitSt();
            TcFenceBefore();
            if (tid == 0) {
                misc.TileMasked[it & 1] = tileMasked ? 1 : 0;
            }
            MbarArrive(&misc.BarP);
            if (it < 4) {
                TRC(4 + 2 * it);
            }
            cur = nxt;
            ++it;
        }

        const int tiles = it;
        TRC(11);
        if (tiles > 0 && !failed) {
            if (!WaitBar(&misc.BarMma, tiles & 1)) {
                failed = true;
                if (p.Status) {
                    atomicOr(p.Status, kDevTimeoutMma);
                }
            }
            TcFenceAfter();
        }
        if (failed) {
            *(volatile int *)&misc.Abort = 1;
        }
        TRC(14);
        // total weight of the row: both halves
        misc.RowX[half][r] = lacc2.x + lacc2.y;
        BarSync(BAR_STAGE, SOFTMAX_THREADS);
        TRC(15);
        failed = failed || (*(volatile int *)&misc.Abort != 0);
        if (!failed) {
            const float lTot = (lacc2.x + lacc2.y + misc.RowX[half ^ 1][r]) * (1.0f / 128.0f) + exp2f(-m);
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
                            for (int k = 0; k < 4; ++k) {
                                float a = __uint_as_float(o[c + 2 * k]) * outMult, b = __uint_as_float(o[c + 2 * k + 1]) * outMult;
                                if (p.OutDtype == TSA_BF16) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                                    w[k] = *reinterpret_cast<uint32_t *>(&h);
                                } else {
                                    w[k] = PackHalf2(a, b);
                                }
                            }
                            dst[c >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
    }
    TRC(12);
    TcFenceBefore();
    __syncthreads();
    if (warp == CTRL_WARP) {
        TmemDealloc(tmem, TMEM_COLS);
    }
    TRC(13);
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
    TFwdMisc &misc = *reinterpret_cast<TFwdMisc *>(smem + 2 * 128 * D);
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

size_t Sm100FwdWorkspaceBytes(int headCount)
{
    return (size_t)((headCount * sizeof(float) + 255) / 256 * 256);
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
    dim3 grid(qTiles, fp.HeadCount);
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
    if (hasVs) {
        fp.VRef = (const float *)workspace;
        rc = CheckCuda(cudaMemsetAsync(workspace, 0, p.HeadCount * sizeof(float), stream), "clearing the V-scale maxima");
        if (rc != TSA_OK) {
            return rc;
        }
        dim3 vgrid((keyRows + VREF_CHUNK - 1) / VREF_CHUNK, p.HeadCount);
        VRefKernel<<<vgrid, 256, 0, stream>>>(p.VScale, keyRows, (float *)workspace);
    }
    const int qTiles = (lenAttTiles + 1) / 2;
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

#ifdef TSA_FWD_TRACE
extern "C" __attribute__((visibility("default"))) int tsa_debug_trace(long long *dst, int n)
{
    return (int)cudaMemcpyFromSymbol(dst, tsa::g_trace, n * sizeof(long long));
}
#endif
