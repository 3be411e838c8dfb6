// Quantized attention backward for sm_100a on the tensor cores (tcgen05, bf16 operands, f32 accumulators in
// tensor memory).
//
// Replaces Fp8AttGradQK / Fp8AttGradQV (code/gpt/compute/gpt_att_fp8.cuh:277-983) and Fp16AttGradQK / QV
// (gpt_att_fp16.cuh:332-616).  Math (TAttentionComputer::CalcDDot / GradQK / GradQV, gpt_cpu.cpp:465-555):
//   z_ij = dot(q8_i, k8_j) sq_i sk_j c - slope (i - j);   p_ij = 2^(z_ij - lse_i)
//   dP_ij = dO_i . (sv_j v8_j);   dS_ij = p_ij (dP_ij - delta_i) c ln2
//   dq_i = sum_j dS_ij sk_j k8_j;   dk_j = sum_i dS_ij sq_i q8_i;   dv_j = sum_i p_ij dO_i
// The reference quantises dS to e4m3 with a two-pass row maximum (doc/precision.md:44); here the stored 8-bit
// vectors are first widened to bf16 (exact: every int8 and e4m3 value is a bf16 number) into scratch, dO is taken
// as bf16, and all GEMMs run as kind::f16 with dS and P handed to the tensor core as bf16: one pass, no row maximum.
//
// One kernel, two modes, the same tile engine:
//   mode dQ     : CTA = head x 128 query rows (R1 = Q, R2 = dO), loop over key tiles (C1 = K, C2 = V) of the row
//                 spans:  S = R1 C1^T, dP = R2 C2^T, A1 = dS * sk_j,                  dQ  += A1 C1
//   mode dK,dV  : CTA = head x 128 key rows  (R1 = K, R2 = V ), loop over query tiles (C1 = Q, C2 = dO) of the
//                 transposed spans:  S^T = R1 C1^T, dP^T = R2 C2^T, A1 = dS * sq_i, A2 = P,  dK += A1 C1, dV += A2 C2
// Tensor memory (512 columns): [0,128) S, [128,256) dP, [256,256+D) first output, [256+D,256+2D) second output.
// A1 / A2 (bf16, two per column) are written back over the S / dP columns the writing thread has already consumed.
//
// A tile is worked on as two 64-column halves with their own barriers, so the tensor pipe and the arithmetic
// overlap: while the 16 arithmetic warps turn S / dP of one half into A1 / A2 (four threads per tile row, 16 columns
// each; packed f32x2 arithmetic on per-column factors staged in shared memory one tile ahead), the MMAs of the other
// half (its output products, then its S / dP of the next tile) run.  Each half has its own MMA-issuing warp (an elected
// lane of a converged warp issues, in grouped asm blocks); the two take turns block by block, so one does its waits
// while the other issues and the accumulation order is fixed; one more warp issues the TMA copies.  Row tiles stay in shared memory; column tiles stream through a ring of
// half stages (64 rows of C1 and C2), freed per half.  All waits are bounded; a failed wait is carried to the
// arithmetic threads' next named barrier so they leave together.
#include "att_sm100_common.cuh"

namespace tsa {

constexpr int BWD_ARITH_THREADS = 512;
constexpr int BWD_CTRL_WARP = BWD_ARITH_THREADS / 32; // and the next one: control warp h issues the products of half h
constexpr int BWD_LOAD_WARP = BWD_CTRL_WARP + 2;
constexpr int BWD_THREADS = BWD_ARITH_THREADS + 96;
constexpr uint32_t BWD_TMEM_COLS = 512;
constexpr uint32_t BWD_S_COL = 0, BWD_DP_COL = 128, BWD_OUT_COL = 256;

// Phase trace for profiling builds (-DTSA_BWD_TRACE): clock64() per tile from lane 0 of the first warp of each half
// and of the control warp of one CTA; tsa_debug_trace_bwd copies the buffer out.
#ifdef TSA_BWD_TRACE
__device__ long long g_traceBwd[4096];
#define TRB(T, e) do { if (traceOn && (T) < 64) g_traceBwd[(T) * 16 + (e)] = clock64(); } while (0)
#else
#define TRB(T, e) do { } while (0)
#endif

struct TBwdParams {
    int HeadCount;
    int Rows;         // rows of every matrix
    int LenAttTiles;  // number of 64-row span blocks
    const tsa_span_group *Spans; // spans of the rows of this mode (forward spans for dQ, transposed for dK/dV)
    const int *SpanPtr;
    P2D<float> QScale, KScale, VScale;
    float QkVecScale, VVecScale;
    P2D<float> Lse, DScale;
    const float *GlobalScale;
    float C;
    float Slope;
    float GradMult;
    P2D<char> Out1, Out2;
    int GradDtype;
    int *Status;
};

template <int D>
struct TBwdSmem {
    static constexpr int STAGES = (D == 64) ? 3 : 2;
    static constexpr int TILE_BYTES = 128 * D * 2;
    // column tiles travel in halves of 64 rows: a ring of HSTAGES half stages, each [C1 half][C2 half]
    static constexpr int HSTAGES = 2 * STAGES;
    static constexpr int HALF_TILE_BYTES = TILE_BYTES / 2;
    static constexpr int R1_OFF = 0;
    static constexpr int R2_OFF = TILE_BYTES;
    static constexpr int C_OFF = 2 * TILE_BYTES;              // half stage s: C1 rows at C_OFF + s * TILE, C2 rows right after
    static constexpr int MISC_OFF = C_OFF + STAGES * 2 * TILE_BYTES;
    static constexpr int TOTAL = MISC_OFF + 8192;
};

struct TBwdMisc {
    // per column of the tile, double buffered by tile parity, written by the half that uses them:
    float ColA[2][TILE_ROWS]; // scale of the column vector (dQ: sk_j, dK/dV: sq_i)
    float ColT[2][TILE_ROWS]; // additive term of the exponent (dQ: ALiBi column part, dK/dV: -lse_i - ALiBi column part)
    float ColB[2][TILE_ROWS]; // dQ: sv_j c ln2;  dK/dV: -delta_i c ln2
    int Abort;
    int Turn;                 // issue blocks handed to the tensor pipe so far: control warp h issues the blocks with index = h (mod 2)
    uint64_t BarR;            // TMA: row tiles landed
    uint64_t BarFull[8];      // TMA: half stage (64 rows of C1 and C2) landed
    uint64_t BarEmpty[8];     // MMA warp -> loader: the half stage's output products have retired
    uint64_t BarS[2];         // control -> half h: S and dP columns of the half ready
    uint64_t BarP[2];         // half h -> control: A1 / A2 of the half written (8 warp arrivals)
    uint64_t BarDone;         // control -> all: every output product has retired
    uint32_t TmemBase;
};
static_assert(sizeof(TBwdMisc) <= 8192, "misc block");

__device__ __forceinline__ uint32_t PackBf16x2(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// MODE_DKV = false: dQ pass; true: dK/dV pass
template <int D, bool MODE_DKV>
__global__ void __launch_bounds__(BWD_THREADS, 1) BwdSm100Kernel(const __grid_constant__ CUtensorMap tmR1,
    const __grid_constant__ CUtensorMap tmR2, const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
    const __grid_constant__ TBwdParams p)
{
    using SM = TBwdSmem<D>;
    constexpr int HSTAGES = SM::HSTAGES;
    constexpr uint32_t HALF_BLOCK_BYTES = 64 * 128;     // one [64 rows][128 bytes] block of a half column tile
    constexpr int KBLOCKS = D / 64;                     // 64-element (128-byte) blocks along the head dimension
    constexpr uint32_t BLOCK_BYTES = 128 * 128;         // one [128 rows][128 bytes] block of a tile
    constexpr uint32_t IDESC_SS = MakeInstrDesc(1, 1, 1, 0, 0, TILE_ROWS, 64); // bf16 x bf16 -> f32, both K-major, 64 columns
    constexpr uint32_t IDESC_OUT = MakeInstrDesc(1, 1, 1, 0, 1, TILE_ROWS, D); // A from tensor memory, B MN-major
    constexpr int BAR_ARITH = 1;                        // named barrier of the 512 arithmetic threads
    constexpr int QUARTER_D = D / 4;
    constexpr int OUTPUTS = MODE_DKV ? 2 : 1;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sR1 = smem + SM::R1_OFF;
    uint8_t *sR2 = smem + SM::R2_OFF;
    uint8_t *sC = smem + SM::C_OFF;
    TBwdMisc &misc = *reinterpret_cast<TBwdMisc *>(smem + SM::MISC_OFF);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.y;
    const int rowTile = gridDim.x - 1 - blockIdx.x;

    if ((SmemAddr(smem) & 1023u) != 0) {
        if (tid == 0 && p.Status) {
            atomicOr(p.Status, kDevBadSpan);
        }
        return;
    }
    if (tid == 0) {
        MbarInit(&misc.BarR, 1);
        for (int s = 0; s < HSTAGES; ++s) {
            MbarInit(&misc.BarFull[s], 1);
            MbarInit(&misc.BarEmpty[s], 1);
        }
        for (int h = 0; h < 2; ++h) {
            MbarInit(&misc.BarS[h], 1);
            MbarInit(&misc.BarP[h], BWD_ARITH_THREADS / 32);
        }
        MbarInit(&misc.BarDone, 2);
        misc.Abort = 0;
        misc.Turn = 0;
        FenceBarrierInit();
    }
    if (warp == BWD_CTRL_WARP) {
        TmemAlloc(&misc.TmemBase, BWD_TMEM_COLS);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;
    const int *abortFlag = &misc.Abort;
#ifdef TSA_BWD_TRACE
    const bool traceOn = blockIdx.x == 40 && blockIdx.y == 3 && lane == 0 && (warp == 0 || warp == 8 || warp == BWD_CTRL_WARP || warp == BWD_CTRL_WARP + 1);
#endif

    // The row tiles depend only on the CTA's coordinates: their copies start before the span lookup (two dependent global
    // loads) instead of behind it.
    if (warp == BWD_LOAD_WARP && lane == 0) {
        PrefetchTensorMap(&tmR1);
        PrefetchTensorMap(&tmR2);
        // every tensor map has boxes of 64 rows x 64 elements (128 bytes): a row tile is two boxes per block
        auto loadTile = [&](uint8_t *dst, const CUtensorMap *tm, int rowBase, uint64_t *bar) {
#pragma unroll
            for (int kb = 0; kb < KBLOCKS; ++kb) {
                TmaLoad2D(dst + kb * BLOCK_BYTES, tm, head * D + kb * 64, rowBase, bar);
                TmaLoad2D(dst + kb * BLOCK_BYTES + HALF_BLOCK_BYTES, tm, head * D + kb * 64, rowBase + 64, bar);
            }
        };
        MbarExpectTx(&misc.BarR, 2 * SM::TILE_BYTES);
        loadTile(sR1, &tmR1, rowTile * TILE_ROWS, &misc.BarR);
        loadTile(sR2, &tmR2, rowTile * TILE_ROWS, &misc.BarR);
    }

    TTileIter cur;
    cur.Init(p.Spans, p.SpanPtr, p.LenAttTiles, rowTile, p.Rows);

    if (warp == BWD_LOAD_WARP) {
        // ---------------------------------------------------------------- loader warp: every TMA copy
        if (lane == 0 && !cur.Valid) {
            WaitBar(&misc.BarR, 0); // a CTA without column tiles: the row tiles must have landed before it ends
        }
        if (lane == 0 && cur.Valid) {
            PrefetchTensorMap(&tmC1);
            PrefetchTensorMap(&tmC2);
            auto loadHalf = [&](uint8_t *dst, const CUtensorMap *tm, int rowBase, uint64_t *bar) {
#pragma unroll
                for (int kb = 0; kb < KBLOCKS; ++kb) {
                    TmaLoad2D(dst + kb * HALF_BLOCK_BYTES, tm, head * D + kb * 64, rowBase, bar);
                }
            };
            int g = 0; // half stages requested
            bool failed = false;
            for (TTileIter prod = cur; prod.Valid && !failed; prod.Advance()) {
#pragma unroll 1
                for (int h = 0; h < 2; ++h, ++g) {
                    const int slot = g % HSTAGES;
                    if (g >= HSTAGES && !WaitBarA(&misc.BarEmpty[slot], ((g / HSTAGES) - 1) & 1, abortFlag)) {
                        failed = true;
                        *(volatile int *)&misc.Abort = 1;
                        if (p.Status) {
                            atomicOr(p.Status, kDevTimeoutMma);
                        }
                        break;
                    }
                    MbarExpectTx(&misc.BarFull[slot], 2 * SM::HALF_TILE_BYTES);
                    loadHalf(sC + slot * 2 * SM::HALF_TILE_BYTES, &tmC1, prod.J0 + 64 * h, &misc.BarFull[slot]);
                    loadHalf(sC + slot * 2 * SM::HALF_TILE_BYTES + SM::HALF_TILE_BYTES, &tmC2, prod.J0 + 64 * h, &misc.BarFull[slot]);
                }
            }
            if (*(volatile int *)&misc.Abort) {
                // drain copies that were requested, so none lands after the CTA is gone
                WaitBar(&misc.BarR, 0);
                for (int t = max(0, g - HSTAGES); t < g; ++t) {
                    WaitBar(&misc.BarFull[t % HSTAGES], (t / HSTAGES) & 1);
                }
            }
        }
        __syncwarp();
    } else if (warp == BWD_CTRL_WARP || warp == BWD_CTRL_WARP + 1) {
        // ---------------------------------------------------------------- two MMA warps, one per 64-column half of the
        // tiles: the whole warp runs the loop and the waits, one elected lane issues (descriptors stay in uniform
        // registers that way).  The halves share nothing but the output accumulators, which the arithmetic threads
        // clear before their first hand-over so that every output product accumulates, whichever warp comes first; while
        // one warp is between two issue blocks (waits, votes, loop code) the other keeps the tensor pipe fed.
        const int h = warp - BWD_CTRL_WARP;
        if (cur.Valid) {
            const uint32_t sR1a = SmemAddr(sR1), sR2a = SmemAddr(sR2), sCa = SmemAddr(sC);
            bool failed = false;
            // descriptors of a K-major tile and of an MN-major half column tile without the address (added per use, in
            // 16-byte units)
            const uint64_t kDescBase = MakeSmemDesc(0, 16, 1024, 128), mnDescBase = MakeSmemDesc(0, HALF_BLOCK_BYTES, 1024, 128);
            // columns [64h, 64h + 64) of S = R1 C1^T and dP = R2 C2^T from half stage `slot` (the 64 rows of C1 and C2 that
            // belong to the half): both operands K-major, D / 16 steps of 16 elements (32 bytes), the B blocks 8 KB apart
            auto issueScores = [&](int slot, int h) {
                const uint32_t c1 = sCa + slot * 2 * SM::HALF_TILE_BYTES, c2 = c1 + SM::HALF_TILE_BYTES;
                MmaGroupF16SS<D / 16>(tmem + BWD_S_COL + h * 64, kDescBase + (sR1a >> 4), kDescBase + (c1 >> 4), IDESC_SS, HALF_BLOCK_BYTES >> 4);
                MmaGroupF16SS<D / 16>(tmem + BWD_DP_COL + h * 64, kDescBase + (sR2a >> 4), kDescBase + (c2 >> 4), IDESC_SS, HALF_BLOCK_BYTES >> 4);
            };
            // out1 += A1 C1 (and out2 += A2 C2) over the half's 64 tile columns = 4 steps of 16: A from tensor memory
            // (the bf16 pairs of tile columns [16k, 16k + 16) sit in columns 16k .. 16k+7), B = the half column tile read
            // MN-major (16 rows of 128 bytes per step)
            auto issueOutputs = [&](int slot, int h) {
                const uint32_t c1 = sCa + slot * 2 * SM::HALF_TILE_BYTES, c2 = c1 + SM::HALF_TILE_BYTES;
                MmaQuadF16TS(tmem + BWD_OUT_COL, tmem + BWD_S_COL + h * 64, mnDescBase + (c1 >> 4), IDESC_OUT, 1u);
                if (MODE_DKV) {
                    MmaQuadF16TS(tmem + BWD_OUT_COL + D, tmem + BWD_DP_COL + h * 64, mnDescBase + (c2 >> 4), IDESC_OUT, 1u);
                }
            };
            auto fail = [&](int code) {
                failed = true;
                if (lane == 0) {
                    *(volatile int *)&misc.Abort = 1;
                    if (p.Status) {
                        atomicOr(p.Status, code);
                    }
                }
            };
            if (!__all_sync(0xffffffffu, WaitBarA(&misc.BarR, 0, abortFlag))) {
                fail(kDevTimeoutTma);
            }
            // Order inside a half: out(h, it-1) then scores(h, it): the outputs read the half's A columns before the next
            // scores overwrite them, and a thread's products run in order.  The warp never waits for its own MMAs; the
            // loader refills a half stage when the commit made after its output products completes.  Half (it, h) lives
            // in half stage (2 it + h) % HSTAGES.
            // The two warps take turns: issue blocks go to the pipe whole and in a fixed order, h0 h1 h0 h1 ..., so the
            // output accumulators, which both halves add to, receive their terms in the same order on every run (f32
            // addition does not commute with rounding: without the turns the results differed in the last bit from run
            // to run).  The waits of one warp still overlap the issue block of the other.
            auto takeTurn = [&](int index) {
                const volatile int *turn = &misc.Turn;
                if (*turn == index) {
                    return true;
                }
                const long long t0 = clock64();
                for (;;) {
                    for (int i = 0; i < 64; ++i) {
                        __nanosleep(20);
                        if (*turn == index) {
                            return true;
                        }
                    }
                    if (*(const volatile int *)abortFlag || clock64() - t0 > WAIT_CYCLES) {
                        return false;
                    }
                }
            };
            auto passTurn = [&](int index) {
                __syncwarp();
                if (lane == 0) {
                    *(volatile int *)&misc.Turn = index + 1;
                }
            };
            int it = 0;
            TTileIter ctl = cur;
            for (; ctl.Valid && !failed; ++it, ctl.Advance()) {
                const int g = 2 * it + h;
                const int slot = g % HSTAGES, prevSlot = (g - 2 + HSTAGES) % HSTAGES;
                TRB(it, 8 + 4 * h);
                if (!__all_sync(0xffffffffu, WaitBarA(&misc.BarFull[slot], (g / HSTAGES) & 1, abortFlag))) {
                    fail(kDevTimeoutTma);
                    break;
                }
                if (it > 0) {
                    if (!__all_sync(0xffffffffu, WaitBarSleep<20>(&misc.BarP[h], (it - 1) & 1, abortFlag))) {
                        fail(kDevTimeoutMma);
                        break;
                    }
                }
                if (!__all_sync(0xffffffffu, takeTurn(g))) {
                    fail(kDevTimeoutMma);
                    break;
                }
                TcFenceAfter();
                TRB(it, 9 + 4 * h);
                if (ElectOne()) {
                    if (it > 0) {
                        issueOutputs(prevSlot, h);
                        MmaCommit(&misc.BarEmpty[prevSlot]);
                    }
                    issueScores(slot, h);
                    MmaCommit(&misc.BarS[h]);
                }
                passTurn(g);
                TRB(it, 10 + 4 * h);
            }
            if (!failed && it > 0) {
                if (__all_sync(0xffffffffu, WaitBarSleep<20>(&misc.BarP[h], (it - 1) & 1, abortFlag) && takeTurn(2 * it + h))) {
                    TcFenceAfter();
                    if (ElectOne()) {
                        issueOutputs((2 * (it - 1) + h) % HSTAGES, h);
                    }
                    passTurn(2 * it + h);
                } else {
                    fail(kDevTimeoutMma);
                }
            }
            __syncwarp();
            if (ElectOne()) {
                MmaCommit(&misc.BarDone);
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- arithmetic warps
        const int quarter = tid >> 7;          // 16-column block of each 64-column half
        const int r = tid & (TILE_ROWS - 1);
        const int row = rowTile * TILE_ROWS + r;
        const uint32_t tLane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const bool rowOk = row < p.Rows;
        const float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
        const float cg = p.C * g;
        const float dsMult = cg * kLog2;
        // per-row constants.  dQ pass: the row is a query (scale sq, lse, delta); dK/dV pass: the row is a key (sk, sv)
        float rowScale = 0, rowLse = 0, rowDelta = 0, rowSv = 0;
        if (rowOk) {
            if (!MODE_DKV) {
                rowScale = p.QScale.Valid() ? p.QScale.Row(head)[row] : p.QkVecScale;
                rowLse = p.Lse.Row(head)[row];
                rowDelta = p.DScale.Row(head)[row];
            } else {
                rowScale = p.KScale.Row(head)[row];
                rowSv = p.VScale.Valid() ? p.VScale.Row(head)[row] : p.VVecScale;
            }
        }
        const float rowMult = rowScale * cg;
        const float2 rowMult2 = make_float2(rowMult, rowMult);
        const float2 rowSvM2 = make_float2(rowSv * dsMult, rowSv * dsMult);
        const float2 negDeltaM2 = make_float2(-rowDelta * dsMult, -rowDelta * dsMult);

        int spanS = 1, spanF = 0, spanRound = -1;
        // the tile's 128 column factors are staged by the first 128 threads, one tile ahead
        float pfA = 0, pfT = 0, pfB = 0;
        auto fetchCols = [&](int c0) {
            pfA = 0;
            pfT = 0;
            pfB = 0;
            const int c = c0 + tid;
            if (tid < TILE_ROWS && c < p.Rows) {
                if (!MODE_DKV) {
                    pfA = p.KScale.Row(head)[c];
                    pfT = p.Slope * (float)tid;
                    pfB = (p.VScale.Valid() ? p.VScale.Row(head)[c] : p.VVecScale) * dsMult;
                } else {
                    pfA = p.QScale.Valid() ? p.QScale.Row(head)[c] : p.QkVecScale;
                    pfT = -p.Lse.Row(head)[c] - p.Slope * (float)tid;
                    pfB = -p.DScale.Row(head)[c] * dsMult;
                }
            }
        };
        if (cur.Valid) {
            fetchCols(cur.J0);
            // clear this thread's quarter of the output accumulators: every output product accumulates
            uint32_t zero[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                zero[k] = 0;
            }
#pragma unroll
            for (int o = 0; o < OUTPUTS; ++o) {
#pragma unroll
                for (int c = 0; c < QUARTER_D; c += 8) {
                    TmemStN<8>(tLane + BWD_OUT_COL + o * D + quarter * QUARTER_D + c, zero);
                }
            }
            TmemWaitSt();
            TcFenceBefore();
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
            TRB(it, 0);
            const int buf = it & 1;
            if (tid < TILE_ROWS) {
                misc.ColA[buf][tid] = pfA;
                misc.ColT[buf][tid] = pfT;
                misc.ColB[buf][tid] = pfB;
            }
            const int c0 = cur.J0;
            const int ls = spanS - c0, lf = min(spanF, p.Rows - 1) - c0; // span in tile-local columns
            const bool rowFull = ls <= 0 && lf >= TILE_ROWS - 1;
            const bool warpMasked = !__all_sync(0xffffffffu, rowFull);
            // publishes the staged columns; a failed wait is carried here so the arithmetic threads leave together
            if (BarRedOr(BAR_ARITH, BWD_ARITH_THREADS, failed || (*(volatile int *)&misc.Abort != 0))) {
                failed = true;
                break;
            }
            TRB(it, 1);
            {
                TTileIter nxt = cur;
                nxt.Advance();
                if (nxt.Valid) {
                    fetchCols(nxt.J0);
                }
            }
            // exponent = u * rowMult + (ColT + rowConst):  dQ: ALiBi + rowOff - lse_i;  dK/dV: -lse_i - ALiBi with the sign of the
            // transposed tile
            const float rowOff = -p.Slope * (float)(row - c0);
            const float rowConst = MODE_DKV ? -rowOff : rowOff - rowLse;
            const float2 rowConst2 = make_float2(rowConst, rowConst);
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                if (!WaitBarA(&misc.BarS[h], it & 1, abortFlag)) {
                    failed = true;
                    *(volatile int *)&misc.Abort = 1;
                    if (p.Status) {
                        atomicOr(p.Status, kDevTimeoutMma);
                    }
                    break; // to the next barrier of the arithmetic threads
                }
                TcFenceAfter();
                TRB(it, 4 * h + 2);
                const int cb = h * 64 + quarter * 16; // first tile column of this thread's block in the half
                // span clipped to this block, block-local: (unsigned)(c - lsQ) <= spanW  <=>  inside the span
                const int lsC = max(ls, cb), lfC = min(lf, cb + 15);
                const bool rowEmpty = lsC > lfC;
                const int lsQ = lsC - cb;
                const unsigned spanW = rowEmpty ? 0u : (unsigned)(lfC - lsC);
                const bool anyCh = !warpMasked || __any_sync(0xffffffffu, !rowEmpty);
                uint32_t a1[8], a2[8];
                if (anyCh) {
                    float2 s[8], d[8];
                    TmemLd16x2Pairs(tLane + BWD_S_COL + cb, tLane + BWD_DP_COL + cb, s, d);
                    const float4 *A4 = reinterpret_cast<const float4 *>(misc.ColA[buf] + cb);
                    const float4 *T4 = reinterpret_cast<const float4 *>(misc.ColT[buf] + cb);
                    const float4 *B4 = reinterpret_cast<const float4 *>(misc.ColB[buf] + cb);
#pragma unroll
                    for (int c = 0; c < 16; c += 4) {
                        const float4 a4 = A4[c >> 2], t4 = T4[c >> 2], b4 = B4[c >> 2];
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const int i = (c >> 1) + k;
                            const float2 ca = k ? make_float2(a4.z, a4.w) : make_float2(a4.x, a4.y);
                            const float2 ct = k ? make_float2(t4.z, t4.w) : make_float2(t4.x, t4.y);
                            const float2 cbv = k ? make_float2(b4.z, b4.w) : make_float2(b4.x, b4.y);
                            const float2 u = __fmul2_rn(s[i], ca);
                            const float2 e = __ffma2_rn(u, rowMult2, __fadd2_rn(ct, rowConst2));
                            float2 pij = FastExp2Pair(e);
                            if (warpMasked) {
                                pij.x = (!rowEmpty && (unsigned)(c + 2 * k - lsQ) <= spanW) ? pij.x : 0.0f;
                                pij.y = (!rowEmpty && (unsigned)(c + 2 * k + 1 - lsQ) <= spanW) ? pij.y : 0.0f;
                            }
                            const float2 dpv = MODE_DKV ? __ffma2_rn(d[i], rowSvM2, cbv) : __ffma2_rn(d[i], cbv, negDeltaM2);
                            const float2 ds = __fmul2_rn(__fmul2_rn(pij, dpv), ca);
                            a1[i] = PackBf16x2(ds.x, ds.y);
                            a2[i] = PackBf16x2(pij.x, pij.y);
                        }
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        a1[k] = 0;
                        a2[k] = 0;
                    }
                }
                // 16 bf16 values = 8 columns, written over the first half of the 16 columns this thread has just read
                TmemStN<8>(tLane + BWD_S_COL + cb, a1);
                if (MODE_DKV) {
                    TmemStN<8>(tLane + BWD_DP_COL + cb, a2);
                }
                TmemWaitSt();
                TcFenceBefore();
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&misc.BarP[h]);
                }
                TRB(it, 4 * h + 3);
            }
            cur.Advance();
            ++it;
        }

        const int tiles = it;
        if (!failed && tiles > 0) {
            if (!WaitBarA(&misc.BarDone, 0, abortFlag)) {
                failed = true;
                if (p.Status) {
                    atomicOr(p.Status, kDevTimeoutMma);
                }
            }
            TcFenceAfter();
        }
        // Outputs: tensor memory -> registers -> shared memory -> global memory in whole rows.  A thread holds a quarter of
        // one row, so stores straight from the registers would put 32 different rows into every store instruction (32
        // sectors each, serialised in the load/store unit: 4 K clocks per CTA); staged through shared memory (the tile
        // buffers are idle by now; row pitch padded by 16 bytes against bank conflicts) a warp writes two whole rows per
        // instruction.  The vote makes the staging barrier safe when some thread has given up.
        if (!BarRedOr(BAR_ARITH, BWD_ARITH_THREADS, failed)) {
            const int esz = (p.GradDtype == TSA_F32) ? 4 : 2;
            const int rowBytes = D * esz, pitch = rowBytes + 16;
            constexpr int STAGE_BYTES = TILE_ROWS * (D * 4 + 16);
#pragma unroll
            for (int o = 0; o < OUTPUTS; ++o) {
                uint32_t v[QUARTER_D];
                if (tiles > 0) {
                    if (QUARTER_D == 32) {
                        TmemLd32(tLane + BWD_OUT_COL + o * D + quarter * QUARTER_D, v);
                    } else {
                        TmemLd16(tLane + BWD_OUT_COL + o * D + quarter * QUARTER_D, v);
                    }
                    TmemWaitLd();
                } else {
#pragma unroll
                    for (int c = 0; c < QUARTER_D; ++c) {
                        v[c] = 0;
                    }
                }
                uint8_t *dstS = smem + o * STAGE_BYTES + r * pitch + quarter * QUARTER_D * esz;
                if (p.GradDtype == TSA_F32) {
                    float4 *dst = reinterpret_cast<float4 *>(dstS);
#pragma unroll
                    for (int c = 0; c < QUARTER_D; c += 4) {
                        dst[c >> 2] = make_float4(__uint_as_float(v[c]) * p.GradMult, __uint_as_float(v[c + 1]) * p.GradMult,
                            __uint_as_float(v[c + 2]) * p.GradMult, __uint_as_float(v[c + 3]) * p.GradMult);
                    }
                } else {
                    uint4 *dst = reinterpret_cast<uint4 *>(dstS);
#pragma unroll
                    for (int c = 0; c < QUARTER_D; c += 8) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float a = __uint_as_float(v[c + 2 * k]) * p.GradMult, b = __uint_as_float(v[c + 2 * k + 1]) * p.GradMult;
                            w[k] = (p.GradDtype == TSA_BF16) ? PackBf16x2(a, b) : PackHalf2(a, b);
                        }
                        dst[c >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            BarRedOr(BAR_ARITH, BWD_ARITH_THREADS, false);
            const int chunksPerRow = rowBytes >> 4;
#pragma unroll
            for (int o = 0; o < OUTPUTS; ++o) {
                const P2D<char> &outp = (o == 0) ? p.Out1 : p.Out2;
                const uint8_t *stage = smem + o * STAGE_BYTES;
                for (int id = tid; id < TILE_ROWS * chunksPerRow; id += BWD_ARITH_THREADS) {
                    const int rr = id / chunksPerRow, cc = id - rr * chunksPerRow;
                    const int grow = rowTile * TILE_ROWS + rr;
                    if (grow < p.Rows) {
                        *reinterpret_cast<uint4 *>(outp.Row(grow) + (size_t)head * D * esz + cc * 16) =
                            *reinterpret_cast<const uint4 *>(stage + rr * pitch + cc * 16);
                    }
                }
            }
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == BWD_CTRL_WARP) {
        TmemDealloc(tmem, BWD_TMEM_COLS);
    }
}

// ---- widening of the stored vectors to bf16 ------------------------------------------------------------
// src: [rows][cols] of i8 / e4m3 / f16 / bf16 / f32 -> dst bf16 [rows][cols] (dense); 8 elements per thread
__global__ void __launch_bounds__(256) ToBf16Kernel(int srcDtype, P2D<char> src, int rows, int cols, __nv_bfloat16 *dst)
{
    const long long groups = (long long)rows * (cols / 8);
    for (long long gidx = blockIdx.x * (long long)blockDim.x + threadIdx.x; gidx < groups; gidx += (long long)gridDim.x * blockDim.x) {
        const int rowIdx = (int)(gidx / (cols / 8));
        const int c0 = (int)(gidx - (long long)rowIdx * (cols / 8)) * 8;
        const void *rowp = src.Row(rowIdx);
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            w[k] = PackBf16x2(LoadAsFloat(rowp, c0 + 2 * k, srcDtype), LoadAsFloat(rowp, c0 + 2 * k + 1, srcDtype));
        }
        *reinterpret_cast<uint4 *>(dst + (size_t)rowIdx * cols + c0) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Q, K and V in one launch when all three are 8-bit with 16-byte aligned rows: blockIdx.y picks the matrix, a thread
// widens 16 elements (one 16-byte load, two 16-byte stores)
struct TWiden3 {
    const char *Src[3];
    int Stride[3];
    int Dtype[3];
    __nv_bfloat16 *Dst[3];
};

__device__ __forceinline__ uint32_t Widen2(uint32_t w, int shift, int dtype)
{
    if (dtype == TSA_I8) {
        // int8 -> f32 without a conversion instruction: the byte, biased by 128, becomes the low mantissa bits of 2^23
        // (ulp 1), and 2^23 + 128 is subtracted again; exact
        const uint32_t biased = w ^ 0x80808080u;
        const float a = __uint_as_float(__byte_perm(biased, 0x4B000000u, shift == 0 ? 0x7440 : 0x7442)) - 8388736.0f;
        const float b = __uint_as_float(__byte_perm(biased, 0x4B000000u, shift == 0 ? 0x7441 : 0x7443)) - 8388736.0f;
        return PackBf16x2(a, b);
    }
    return PackBf16x2(E4M3ToFloat((uint8_t)(w >> shift)), E4M3ToFloat((uint8_t)(w >> (shift + 8))));
}

__global__ void __launch_bounds__(256) Widen8x3Kernel(TWiden3 t, int rows, int cols)
{
    const int m = blockIdx.y;
    const char *src = t.Src[m];
    const int stride = t.Stride[m], dtype = t.Dtype[m];
    __nv_bfloat16 *dst = t.Dst[m];
    const int perRow = cols / 16;
    const long long groups = (long long)rows * perRow;
    const long long step = (long long)gridDim.x * blockDim.x;
    // four independent 16-byte loads in flight per thread
    for (long long g0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; g0 < groups; g0 += 4 * step) {
        uint4 in[4];
        int rowIdx[4], c0[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long gidx = g0 + u * step;
            rowIdx[u] = (int)(gidx / perRow);
            c0[u] = (int)(gidx - (long long)rowIdx[u] * perRow) * 16;
            if (gidx < groups) {
                in[u] = __ldg(reinterpret_cast<const uint4 *>(src + (size_t)rowIdx[u] * stride + c0[u]));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (g0 + u * step < groups) {
                const uint32_t w[4] = {in[u].x, in[u].y, in[u].z, in[u].w};
                uint32_t o[8];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    o[2 * k] = Widen2(w[k], 0, dtype);
                    o[2 * k + 1] = Widen2(w[k], 16, dtype);
                }
                // one 32-byte store: a whole sector per thread (the workspace is 256-byte aligned, cols a multiple of 16)
                StGlobal256(dst + (size_t)rowIdx[u] * cols + c0[u], o);
            }
        }
    }
}

// ---- host side ------------------------------------------------------------------------------------------
bool Sm100BwdSupports(const tsa_att_cfg *cfg, int headCount)
{
    if (cfg->flags & TSA_FLAG_FORCE_GENERIC) {
        return false;
    }
    if (cfg->head_dim_qk != cfg->head_dim_v || (cfg->head_dim_qk != 64 && cfg->head_dim_qk != 128)) {
        return false;
    }
    return headCount > 0;
}

size_t Sm100BwdWorkspaceBytes(int headCount, int headDim, int rows)
{
    const size_t mat = ((size_t)rows * headCount * headDim * 2 + 255) / 256 * 256;
    return 4 * mat; // Q, K, V, dO as bf16
}

template <int D, bool MODE_DKV>
static int LaunchBwdT(const CUtensorMap &r1, const CUtensorMap &r2, const CUtensorMap &c1, const CUtensorMap &c2, const TBwdParams &bp,
    int rowTiles, cudaStream_t stream)
{
    auto kern = BwdSm100Kernel<D, MODE_DKV>;
    const int smemBytes = TBwdSmem<D>::TOTAL;
    int rc = CheckCuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes), "cudaFuncSetAttribute(backward)");
    if (rc != TSA_OK) {
        return rc;
    }
    dim3 grid(rowTiles, bp.HeadCount);
    kern<<<grid, BWD_THREADS, smemBytes, stream>>>(r1, r2, c1, c2, bp);
    return CheckCuda(cudaGetLastError(), "tcgen05 backward launch");
}

int LaunchSm100Bwd(const tsa_att_cfg *cfg, const TGenParams &p, tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d v, tsa_ptr2d dOut,
    int lenAttTiles, void *workspace, int *statusWord, cudaStream_t stream)
{
    const int D = cfg->head_dim_qk;
    const int rows = p.Len;
    const int cols = p.HeadCount * D;
    const size_t mat = ((size_t)rows * cols * 2 + 255) / 256 * 256;
    __nv_bfloat16 *qb = (__nv_bfloat16 *)workspace;
    __nv_bfloat16 *kb = (__nv_bfloat16 *)((char *)workspace + mat);
    __nv_bfloat16 *vb = (__nv_bfloat16 *)((char *)workspace + 2 * mat);
    __nv_bfloat16 *dob = (__nv_bfloat16 *)((char *)workspace + 3 * mat);
    const long long groups = (long long)rows * (cols / 8);
    const int blocks = (int)((groups + 255) / 256 < 148 * 16 ? (groups + 255) / 256 : 148 * 16);
    auto aligned16 = [](const tsa_ptr2d &a) { return (uintptr_t)a.data % 16 == 0 && a.stride_bytes % 16 == 0; };
    if (cols % 16 == 0 && aligned16(qk) && aligned16(qv) && aligned16(v)) {
        TWiden3 t;
        const tsa_ptr2d *srcs[3] = {&qk, &qv, &v};
        __nv_bfloat16 *dsts[3] = {qb, kb, vb};
        for (int m = 0; m < 3; ++m) {
            t.Src[m] = (const char *)srcs[m]->data;
            t.Stride[m] = srcs[m]->stride_bytes;
            t.Dtype[m] = (m < 2) ? cfg->qk_dtype : cfg->v_dtype;
            t.Dst[m] = dsts[m];
        }
        const long long g16 = (long long)rows * (cols / 16);
        const int b16 = (int)((g16 + 255) / 256 < 148 * 8 ? (g16 + 255) / 256 : 148 * 8);
        Widen8x3Kernel<<<dim3(b16, 3), 256, 0, stream>>>(t, rows, cols);
    } else {
        ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->qk_dtype, P2D<char>(qk), rows, cols, qb);
        ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->qk_dtype, P2D<char>(qv), rows, cols, kb);
        ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->v_dtype, P2D<char>(v), rows, cols, vb);
    }
    // dO that already is bf16 in a TMA-compatible layout is read where it lies
    const bool dOutInPlace = cfg->grad_dtype == TSA_BF16 && (uintptr_t)dOut.data % 16 == 0 && dOut.stride_bytes % 16 == 0 && dOut.xsize >= cols;
    if (!dOutInPlace) {
        ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->grad_dtype, P2D<char>(dOut), rows, cols, dob);
    }
    int rc = CheckCuda(cudaGetLastError(), "bf16 widening launch");
    if (rc != TSA_OK) {
        return rc;
    }
    auto mapOf = [&](CUtensorMap *m, __nv_bfloat16 *ptr, const char *what) {
        tsa_ptr2d a = {ptr, cols * 2, cols, rows};
        return MakeTileMapEx(m, a, 2, 64, 64, what);
    };
    CUtensorMap mq, mk, mv, mdo;
    rc = mapOf(&mq, qb, "q bf16");
    if (rc == TSA_OK) {
        rc = mapOf(&mk, kb, "k bf16");
    }
    if (rc == TSA_OK) {
        rc = mapOf(&mv, vb, "v bf16");
    }
    if (rc == TSA_OK) {
        if (dOutInPlace) {
            tsa_ptr2d a = {dOut.data, dOut.stride_bytes, cols, rows};
            rc = MakeTileMapEx(&mdo, a, 2, 64, 64, "dOut bf16 (in place)");
        } else {
            rc = mapOf(&mdo, dob, "dOut bf16");
        }
    }
    if (rc != TSA_OK) {
        return rc;
    }
    TBwdParams bp;
    bp.HeadCount = p.HeadCount;
    bp.Rows = rows;
    bp.LenAttTiles = lenAttTiles;
    bp.QScale = p.QScale;
    bp.KScale = p.KScale;
    bp.VScale = p.VScale;
    bp.QkVecScale = p.QkVecScale;
    bp.VVecScale = p.VVecScale;
    bp.Lse = p.Lse;
    bp.DScale = p.DScale;
    bp.GlobalScale = p.GlobalScale;
    bp.C = p.C;
    bp.Slope = p.Slope;
    bp.GradMult = p.GradMult;
    bp.GradDtype = p.GradDtype;
    bp.Status = statusWord;
    const int rowTiles = (lenAttTiles + 1) / 2;
    // dQ pass: rows = queries
    bp.Spans = p.Spans;
    bp.SpanPtr = p.SpanPtr;
    bp.Out1 = p.DQ;
    bp.Out2 = p.DQ;
    rc = (D == 128) ? LaunchBwdT<128, false>(mq, mdo, mk, mv, bp, rowTiles, stream) : LaunchBwdT<64, false>(mq, mdo, mk, mv, bp, rowTiles, stream);
    if (rc != TSA_OK) {
        return rc;
    }
    // dK / dV pass: rows = keys, columns from the transposed spans
    bp.Spans = p.RevSpans;
    bp.SpanPtr = p.RevSpanPtr;
    bp.Out1 = p.DK;
    bp.Out2 = p.DV;
    return (D == 128) ? LaunchBwdT<128, true>(mk, mv, mq, mdo, bp, rowTiles, stream) : LaunchBwdT<64, true>(mk, mv, mq, mdo, bp, rowTiles, stream);
}

} // namespace tsa

#ifdef TSA_BWD_TRACE
extern "C" __attribute__((visibility("default"))) int tsa_debug_trace_bwd(long long *dst, int n)
{
    return (int)cudaMemcpyFromSymbol(dst, tsa::g_traceBwd, n * sizeof(long long));
}
#endif
