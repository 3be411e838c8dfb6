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
// 256 arithmetic threads, two per tile row, 64 columns each in chunks of 32; a control warp issues TMA and MMA.
// Row tiles stay in shared memory, column tiles stream through a TMA ring.  All waits are bounded.
#include "att_sm100_common.cuh"

namespace tsa {

constexpr int BWD_ARITH_THREADS = 256;
constexpr int BWD_CTRL_WARP = BWD_ARITH_THREADS / 32;
constexpr int BWD_THREADS = BWD_ARITH_THREADS + 32;
constexpr uint32_t BWD_TMEM_COLS = 512;
constexpr uint32_t BWD_S_COL = 0, BWD_DP_COL = 128, BWD_OUT_COL = 256;

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
    static constexpr int R1_OFF = 0;
    static constexpr int R2_OFF = TILE_BYTES;
    static constexpr int C_OFF = 2 * TILE_BYTES;              // stage s: C1 at C_OFF + s * 2 * TILE, C2 right after
    static constexpr int MISC_OFF = C_OFF + STAGES * 2 * TILE_BYTES;
    static constexpr int TOTAL = MISC_OFF + 8192;
};

struct TBwdMisc {
    float ColA[2][TILE_ROWS]; // per column of the tile, double buffered by tile parity
    float ColB[2][TILE_ROWS];
    float ColC[2][TILE_ROWS];
    float Al[TILE_ROWS];      // slope * column
    int Abort;
    uint64_t BarR;            // TMA: row tiles landed
    uint64_t BarFull[4];      // TMA: column stage landed
    uint64_t BarMma;          // control -> arithmetic: S and dP of tile t ready (and the outputs of tile t-1 issued before)
    uint64_t BarP;            // arithmetic -> control: A1 / A2 of tile t written, 256 arrivals
    uint32_t TmemBase;
};

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
    constexpr int STAGES = SM::STAGES;
    constexpr int KBLOCKS = D / 64;                     // 64-element (128-byte) blocks along the head dimension
    constexpr uint32_t BLOCK_BYTES = 128 * 128;         // one [128 rows][128 bytes] block of a tile
    constexpr uint32_t IDESC_SS = MakeInstrDesc(1, 1, 1, 0, 0, TILE_ROWS, TILE_ROWS); // bf16 x bf16 -> f32, both K-major
    constexpr uint32_t IDESC_OUT = MakeInstrDesc(1, 1, 1, 0, 1, TILE_ROWS, D);         // A from tensor memory, B MN-major
    constexpr int BAR_STAGE = 1;
    constexpr int HALF_N = TILE_ROWS / 2;
    constexpr int HALF_D = D / 2;
    constexpr int OUTPUTS = MODE_DKV ? 2 : 1;

    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t *sR1 = smem + SM::R1_OFF;
    uint8_t *sR2 = smem + SM::R2_OFF;
    uint8_t *sC = smem + SM::C_OFF;
    TBwdMisc &misc = *reinterpret_cast<TBwdMisc *>(smem + SM::MISC_OFF);

    const int tid = threadIdx.x, warp = tid >> 5;
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
        for (int s = 0; s < STAGES; ++s) {
            MbarInit(&misc.BarFull[s], 1);
        }
        MbarInit(&misc.BarMma, 1);
        MbarInit(&misc.BarP, BWD_ARITH_THREADS);
        misc.Abort = 0;
        FenceBarrierInit();
    }
    if (warp == BWD_CTRL_WARP) {
        TmemAlloc(&misc.TmemBase, BWD_TMEM_COLS);
        TmemRelinquish();
    }
    if (tid < TILE_ROWS) {
        misc.Al[tid] = p.Slope * (float)tid;
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;

    TTileIter cur;
    cur.Init(p.Spans, p.SpanPtr, p.LenAttTiles, rowTile, p.Rows);

    if (warp == BWD_CTRL_WARP) {
        // ---------------------------------------------------------------- control warp
        if ((tid & 31) == 0 && cur.Valid) {
            PrefetchTensorMap(&tmR1);
            PrefetchTensorMap(&tmR2);
            PrefetchTensorMap(&tmC1);
            PrefetchTensorMap(&tmC2);
            const uint32_t sR1a = SmemAddr(sR1), sR2a = SmemAddr(sR2), sCa = SmemAddr(sC);
            TTileIter prod = cur;
            int issued = 0, landed = 0;
            bool failed = false;
            auto loadTile = [&](uint8_t *dst, const CUtensorMap *tm, int rowBase, uint64_t *bar) {
#pragma unroll
                for (int kb = 0; kb < KBLOCKS; ++kb) {
                    TmaLoad2D(dst + kb * BLOCK_BYTES, tm, head * D + kb * 64, rowBase, bar);
                }
            };
            auto issueLoad = [&](int slot, int c0) {
                MbarExpectTx(&misc.BarFull[slot], 2 * SM::TILE_BYTES);
                loadTile(sC + slot * 2 * SM::TILE_BYTES, &tmC1, c0, &misc.BarFull[slot]);
                loadTile(sC + slot * 2 * SM::TILE_BYTES + SM::TILE_BYTES, &tmC2, c0, &misc.BarFull[slot]);
            };
            // S = R1 C1^T and dP = R2 C2^T: both operands K-major, D / 16 steps of 16 elements (32 bytes)
            auto issueScores = [&](int slot) {
                const uint32_t c1 = sCa + slot * 2 * SM::TILE_BYTES, c2 = c1 + SM::TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * BLOCK_BYTES + (ks & 3) * 32;
                    MmaF16SS(tmem + BWD_S_COL, MakeSmemDesc(sR1a + off, 16, 1024, 128), MakeSmemDesc(c1 + off, 16, 1024, 128), IDESC_SS, ks > 0);
                }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks >> 2) * BLOCK_BYTES + (ks & 3) * 32;
                    MmaF16SS(tmem + BWD_DP_COL, MakeSmemDesc(sR2a + off, 16, 1024, 128), MakeSmemDesc(c2 + off, 16, 1024, 128), IDESC_SS, ks > 0);
                }
            };
            // out1 += A1 C1 (and out2 += A2 C2): A from tensor memory (bf16, 8 columns per 16 rows of the tile's
            // column dimension), B = the column tile read MN-major: 16 rows per step, D columns over KBLOCKS blocks
            auto issueOutputs = [&](int slot, bool accumulate) {
                const uint32_t c1 = sCa + slot * 2 * SM::TILE_BYTES, c2 = c1 + SM::TILE_BYTES;
#pragma unroll
                for (int ks = 0; ks < TILE_ROWS / 16; ++ks) {
                    const uint32_t aCol = (ks >> 2) * HALF_N + (ks & 3) * 8;
                    MmaF16TS(tmem + BWD_OUT_COL, tmem + BWD_S_COL + aCol, MakeSmemDesc(c1 + ks * 16 * 128, BLOCK_BYTES, 1024, 128), IDESC_OUT,
                        (accumulate || ks > 0) ? 1u : 0u);
                }
                if (MODE_DKV) {
#pragma unroll
                    for (int ks = 0; ks < TILE_ROWS / 16; ++ks) {
                        const uint32_t aCol = (ks >> 2) * HALF_N + (ks & 3) * 8;
                        MmaF16TS(tmem + BWD_OUT_COL + D, tmem + BWD_DP_COL + aCol, MakeSmemDesc(c2 + ks * 16 * 128, BLOCK_BYTES, 1024, 128), IDESC_OUT,
                            (accumulate || ks > 0) ? 1u : 0u);
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

            MbarExpectTx(&misc.BarR, 2 * SM::TILE_BYTES);
            loadTile(sR1, &tmR1, rowTile * TILE_ROWS, &misc.BarR);
            loadTile(sR2, &tmR2, rowTile * TILE_ROWS, &misc.BarR);
            for (int s = 0; s < STAGES && prod.Valid; ++s) {
                issueLoad(s, prod.J0);
                prod.Advance();
                ++issued;
            }
            if (!WaitBar(&misc.BarR, 0)) {
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
                    if (!WaitBar(&misc.BarP, (it - 1) & 1)) {
                        fail(kDevTimeoutMma);
                        break;
                    }
                    TcFenceAfter();
                    issueOutputs((it - 1) % STAGES, it - 1 > 0);
                }
                TcFenceAfter();
                issueScores(slot);
                MmaCommit(&misc.BarMma);
                if (it > 0 && prod.Valid) {
                    // the slot of tile it-1 is free once its output MMAs have retired, i.e. when this commit completes
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
                    issueOutputs((it - 1) % STAGES, it - 1 > 0);
                } else {
                    fail(kDevTimeoutMma);
                }
            }
            MmaCommit(&misc.BarMma); // final phase (also releases arithmetic threads waiting after a failure)
            if (failed) {
                for (int t = landed; t < issued; ++t) {
                    WaitBar(&misc.BarFull[t % STAGES], (t / STAGES) & 1);
                }
            }
        }
        __syncwarp();
    } else {
        // ---------------------------------------------------------------- arithmetic warps
        const int half = tid >> 7;
        const int r = tid & (TILE_ROWS - 1);
        const int row = rowTile * TILE_ROWS + r;
        const int colBase = half * HALF_N;
        const uint32_t tLane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const bool rowOk = row < p.Rows;
        const float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
        const float cg = p.C * g;
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
        const float dsMult = cg * kLog2;
        const float alSign = MODE_DKV ? -1.0f : 1.0f;

        int spanS = 1, spanF = 0, spanRound = -1;
        float pfA = 0, pfB = 0, pfC = 0;
        auto fetchCols = [&](int c0) {
            pfA = 0;
            pfB = 0;
            pfC = 0;
            const int c = c0 + tid;
            if (tid < TILE_ROWS && c < p.Rows) {
                if (!MODE_DKV) {
                    pfA = p.KScale.Row(head)[c];
                    pfB = p.VScale.Valid() ? p.VScale.Row(head)[c] : p.VVecScale;
                } else {
                    pfA = p.QScale.Valid() ? p.QScale.Row(head)[c] : p.QkVecScale;
                    pfB = p.Lse.Row(head)[c];
                    pfC = p.DScale.Row(head)[c];
                }
            }
        };
        if (cur.Valid) {
            fetchCols(cur.J0);
        }
        bool failed = false;
        bool aborted = false;
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
            if (tid < TILE_ROWS) {
                misc.ColA[buf][tid] = pfA;
                misc.ColB[buf][tid] = pfB;
                misc.ColC[buf][tid] = pfC;
            }
            const int c0 = cur.J0;
            const int ls = spanS - c0, lf = min(spanF, p.Rows - 1) - c0; // span in tile-local columns
            const bool rowFull = ls <= 0 && lf >= TILE_ROWS - 1;
            const bool warpMasked = !__all_sync(0xffffffffu, rowFull);
            aborted = BarRedOr(BAR_STAGE, BWD_ARITH_THREADS, failed || (*(volatile int *)&misc.Abort != 0));
            if (aborted) {
                break;
            }
            {
                TTileIter nxt = cur;
                nxt.Advance();
                if (nxt.Valid) {
                    fetchCols(nxt.J0);
                }
            }
            if (!WaitBar(&misc.BarMma, it & 1)) {
                failed = true;
                if (p.Status) {
                    atomicOr(p.Status, kDevTimeoutMma);
                }
            }
            TcFenceAfter();

            const float rowOff = -p.Slope * (float)(row - c0);
            const float *colA = misc.ColA[buf] + colBase;
            const float *colB = misc.ColB[buf] + colBase;
            const float *colC = misc.ColC[buf] + colBase;
            const float *alBuf = misc.Al + colBase;
#pragma unroll
            for (int ch = 0; ch < 2; ++ch) {
                // span clipped to this chunk, chunk-local: (unsigned)(c - lsQ) <= spanW  <=>  inside the span
                const int cb = colBase + ch * 32;
                const int lsC = max(ls, cb), lfC = min(lf, cb + 31);
                const bool rowEmpty = lsC > lfC;
                const int lsQ = lsC - cb;
                const unsigned spanW = rowEmpty ? 0u : (unsigned)(lfC - lsC);
                const bool anyCh = !warpMasked || __any_sync(0xffffffffu, !rowEmpty);
                uint32_t a1[16], a2[16];
                if (anyCh) {
                    uint32_t sreg[32], preg[32];
                    TmemLd32(tLane + BWD_S_COL + cb, sreg);
                    TmemLd32(tLane + BWD_DP_COL + cb, preg);
                    TmemWaitLd();
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const int lc = ch * 32 + c;
                        float pv[2], dsv[2];
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const float ca = colA[lc + k];
                            const float u = __uint_as_float(sreg[c + k]) * ca;
                            const float z = fmaf(u, rowMult, alSign * (alBuf[lc + k] + rowOff));
                            const float lse = MODE_DKV ? colB[lc + k] : rowLse;
                            const float delta = MODE_DKV ? colC[lc + k] : rowDelta;
                            const float sv = MODE_DKV ? rowSv : colB[lc + k];
                            float pij = FastExp2(z - lse);
                            if (warpMasked) {
                                pij = (!rowEmpty && (unsigned)(c + k - lsQ) <= spanW) ? pij : 0.0f;
                            }
                            const float dp = __uint_as_float(preg[c + k]) * sv;
                            const float ds = pij * (dp - delta) * dsMult;
                            pv[k] = pij;
                            dsv[k] = ds * (MODE_DKV ? ca : ca); // dQ: dS * sk_j; dK: dS * sq_i (both are the column scale)
                        }
                        a1[c >> 1] = PackBf16x2(dsv[0], dsv[1]);
                        a2[c >> 1] = PackBf16x2(pv[0], pv[1]);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        a1[k] = 0;
                        a2[k] = 0;
                    }
                }
                // 32 bf16 values = 16 columns, written over columns this thread has already read
                TmemSt16(tLane + BWD_S_COL + colBase + ch * 16, a1);
                if (MODE_DKV) {
                    TmemSt16(tLane + BWD_DP_COL + colBase + ch * 16, a2);
                }
            }
            TmemWaitSt();
            TcFenceBefore();
            MbarArrive(&misc.BarP);
            cur.Advance();
            ++it;
        }

        const int tiles = it;
        if (!aborted && tiles > 0 && !failed) {
            if (!WaitBar(&misc.BarMma, tiles & 1)) {
                failed = true;
                if (p.Status) {
                    atomicOr(p.Status, kDevTimeoutMma);
                }
            }
            TcFenceAfter();
        }
        if (!aborted && !failed) {
            const int esz = (p.GradDtype == TSA_F32) ? 4 : 2;
#pragma unroll
            for (int o = 0; o < OUTPUTS; ++o) {
                const P2D<char> &outp = (o == 0) ? p.Out1 : p.Out2;
                char *oRow = outp.Row(rowOk ? row : 0) + ((size_t)head * D + half * HALF_D) * esz;
#pragma unroll
                for (int c0 = 0; c0 < HALF_D; c0 += 32) {
                    uint32_t v[32];
                    if (tiles > 0) {
                        TmemLd32(tLane + BWD_OUT_COL + o * D + half * HALF_D + c0, v);
                        TmemWaitLd();
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            v[c] = 0;
                        }
                    }
                    if (rowOk) {
                        if (p.GradDtype == TSA_F32) {
                            float4 *dst = reinterpret_cast<float4 *>(oRow + c0 * 4);
#pragma unroll
                            for (int c = 0; c < 32; c += 4) {
                                dst[c >> 2] = make_float4(__uint_as_float(v[c]) * p.GradMult, __uint_as_float(v[c + 1]) * p.GradMult,
                                    __uint_as_float(v[c + 2]) * p.GradMult, __uint_as_float(v[c + 3]) * p.GradMult);
                            }
                        } else {
                            uint4 *dst = reinterpret_cast<uint4 *>(oRow + c0 * 2);
#pragma unroll
                            for (int c = 0; c < 32; c += 8) {
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
    ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->qk_dtype, P2D<char>(qk), rows, cols, qb);
    ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->qk_dtype, P2D<char>(qv), rows, cols, kb);
    ToBf16Kernel<<<blocks, 256, 0, stream>>>(cfg->v_dtype, P2D<char>(v), rows, cols, vb);
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
        return MakeTileMapEx(m, a, 2, 64, 128, what);
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
            rc = MakeTileMapEx(&mdo, a, 2, 64, 128, "dOut bf16 (in place)");
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
