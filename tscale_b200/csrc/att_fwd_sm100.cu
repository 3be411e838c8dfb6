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
// One CTA = one head x 128 query rows (two 64-row span blocks), 128 threads; thread t owns row t, which is
// tensor-memory lane t.  Tensor memory: columns [0,128) S (f32 / s32), reused for P (32 + 32 columns of
// packed e4m3); columns [128, 128 + D) O (f32).  256 columns are allocated so two CTAs share an SM and one
// CTA's softmax overlaps the other's MMAs.  Shared memory: Q tile, STAGES x (K tile, V tile) filled by TMA
// with the 128 B (D = 128) or 64 B (D = 64) swizzle the MMA descriptors expect.  Thread 0 issues TMA and MMA.
// Key tiles follow the reference's grouped spans: for round r the tiles [Start, Finish] of the two blocks'
// r-th groups; tiles no row of a warp attends are still multiplied but cost no exponentials.
// Every barrier wait is bounded; when one runs out the kernel records a code in *statusWord, drains its
// outstanding copies, frees its tensor memory and returns.
#include "att_internal.cuh"
#include "sm100_ptx.cuh"
#include <cuda.h>

namespace tsa {

using namespace sm100;

constexpr int FWD_THREADS = 128;
constexpr int TILE_M = 128;
constexpr int TILE_N = 128;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t TMEM_O_COL = 128;
constexpr long long WAIT_CYCLES = 1ll << 31; // about a second

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
    float2 ColTerm[TILE_N]; // (sk_j, slope * jl)
    float SvTerm[TILE_N];   // sv_j / svRef
    uint64_t BarQ;
    uint64_t BarFull[4];
    uint64_t BarMma;
    uint32_t TmemBase;
};

__device__ __forceinline__ bool WaitBar(uint64_t *bar, uint32_t parity)
{
    long long t0 = clock64();
    for (;;) {
        if (MbarWaitBounded(bar, parity, 64)) {
            return true;
        }
        if (clock64() - t0 > WAIT_CYCLES) {
            return false;
        }
    }
}

// iterator over the key tiles of a 128-row query tile: rounds of the two 64-row blocks' span groups
struct TTileIter {
    const tsa_span_group *G0, *G1; // first group of each block (null: block absent)
    int N0, N1;
    int KeyRows;
    int Round, J0, Hi;
    bool Valid;

    __device__ void LoadRound()
    {
        int rounds = max(N0, N1);
        for (; Round < rounds; ++Round) {
            int lo = 0x7fffffff, hi = -1;
            if (Round < N0) {
                lo = min(lo, G0[Round].Start);
                hi = max(hi, G0[Round].Finish);
            }
            if (Round < N1) {
                lo = min(lo, G1[Round].Start);
                hi = max(hi, G1[Round].Finish);
            }
            lo = max(lo, 0) & ~(TILE_N - 1);
            hi = min(hi, KeyRows - 1) & ~(TILE_N - 1);
            if (lo <= hi) {
                J0 = lo;
                Hi = hi;
                Valid = true;
                return;
            }
        }
        Valid = false;
    }
    __device__ void Init(const tsa_span_group *spans, const int *spanPtr, int lenAttTiles, int qTile, int keyRows)
    {
        int b0 = qTile * 2, b1 = qTile * 2 + 1;
        G0 = G1 = nullptr;
        N0 = N1 = 0;
        if (b0 < lenAttTiles) {
            int a = spanPtr[b0], b = spanPtr[b0 + 1];
            G0 = spans + a;
            N0 = b - a;
        }
        if (b1 < lenAttTiles) {
            int a = spanPtr[b1], b = spanPtr[b1 + 1];
            G1 = spans + a;
            N1 = b - a;
        }
        KeyRows = keyRows;
        Round = 0;
        Valid = false;
        LoadRound();
    }
    __device__ void Advance()
    {
        J0 += TILE_N;
        if (J0 > Hi) {
            ++Round;
            LoadRound();
        }
    }
};

template <int N>
__device__ __forceinline__ void TmemStN(uint32_t taddr, const uint32_t *r);
template <>
__device__ __forceinline__ void TmemStN<8>(uint32_t taddr, const uint32_t *r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ float FastExp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t PackHalf2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
// residual of a pair after e4m3 rounding, again as an e4m3 pair
__device__ __forceinline__ uint32_t ResidualE4M3x2(float a, float b, uint32_t hiPair)
{
    uint32_t hb, lo;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hb) : "h"((uint16_t)hiPair));
    uint32_t ef = PackHalf2(a, b);
    uint32_t diff;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(diff) : "r"(ef), "r"(hb));
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(diff));
    lo = r;
    return lo;
}

template <int D, bool QK_I8, bool HAS_VSCALE>
__global__ void __launch_bounds__(FWD_THREADS) FwdSm100Kernel(const __grid_constant__ CUtensorMap tmQ,
    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, TFwdParams p)
{
    using SM = TFwdSmem<D>;
    constexpr int STAGES = SM::STAGES;
    constexpr int SWZ = (D == 128) ? 128 : 64;
    constexpr uint32_t GROUP_BYTES = 8 * D; // 8 rows of a tile
    constexpr uint32_t IDESC_QK = QK_I8 ? MakeInstrDesc(2, 1, 1, 0, 0, TILE_M, TILE_N) : MakeInstrDesc(1, 0, 0, 0, 0, TILE_M, TILE_N);
    constexpr uint32_t IDESC_PV = MakeInstrDesc(1, 0, 0, 0, 1, TILE_M, D);

    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
    uint8_t *sQ = smem + SM::Q_OFF;
    uint8_t *sK = smem + SM::K_OFF;
    uint8_t *sV = smem + SM::V_OFF;
    TFwdMisc &misc = *reinterpret_cast<TFwdMisc *>(smem + SM::MISC_OFF);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int head = blockIdx.y;
    const int qTile = gridDim.x - 1 - blockIdx.x; // late (long) rows first
    const int row = qTile * TILE_M + tid;

    if (tid == 0) {
        MbarInit(&misc.BarQ, 1);
        for (int s = 0; s < STAGES; ++s) {
            MbarInit(&misc.BarFull[s], 1);
        }
        MbarInit(&misc.BarMma, 1);
        FenceBarrierInit();
        PrefetchTensorMap(&tmQ);
        PrefetchTensorMap(&tmK);
        PrefetchTensorMap(&tmV);
    }
    if (warp == 0) {
        TmemAlloc(&misc.TmemBase, TMEM_COLS);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;
    const uint32_t tLane = tmem + ((uint32_t)(warp * 32) << 16);

    TTileIter cur;
    cur.Init(p.Spans, p.SpanPtr, p.LenAttTiles, qTile, p.KeyRows);
    TTileIter prod = cur; // thread 0: next tile to request from TMA
    int issued = 0, landed = 0;

    // row constants
    const bool rowOk = row < p.OutRows;
    const float g = p.GlobalScale ? *p.GlobalScale : 1.0f;
    float sq = 0;
    if (rowOk) {
        sq = p.QScale.Valid() ? p.QScale.Row(head)[row] : p.QkVecScale;
    }
    const float rowMult = sq * p.C * g;
    const float vRef = HAS_VSCALE ? p.VRef[head] : 0.0f;
    const float svMult = (HAS_VSCALE && vRef > 0) ? 1.0f / vRef : 0.0f; // sv_j / svRef <= 1; the factor 128 sits in the exponent

    const uint32_t sQa = SmemAddr(sQ), sKa = SmemAddr(sK), sVa = SmemAddr(sV);
    bool failed = false;

    auto issueLoad = [&](int slot, int j0) {
        MbarExpectTx(&misc.BarFull[slot], 2 * SM::TILE_BYTES);
        TmaLoad2D(sK + slot * SM::TILE_BYTES, &tmK, head * D, j0, &misc.BarFull[slot]);
        TmaLoad2D(sV + slot * SM::TILE_BYTES, &tmV, head * D, j0, &misc.BarFull[slot]);
    };
    auto issueQK = [&](int slot) {
        uint32_t kAddr = sKa + slot * SM::TILE_BYTES;
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

    if (tid == 0 && cur.Valid) {
        MbarExpectTx(&misc.BarQ, SM::TILE_BYTES);
        TmaLoad2D(sQ, &tmQ, head * D, qTile * TILE_M, &misc.BarQ);
        for (int s = 0; s < STAGES && prod.Valid; ++s) {
            issueLoad(s, prod.J0);
            prod.Advance();
            ++issued;
        }
        bool ok = WaitBar(&misc.BarQ, 0) && WaitBar(&misc.BarFull[0], 0);
        if (ok) {
            ++landed;
            TcFenceAfter();
            issueQK(0);
        } else {
            failed = true;
            if (p.Status) {
                atomicOr(p.Status, kDevTimeoutTma);
            }
        }
        MmaCommit(&misc.BarMma);
    }

    // per-row span of the current round
    int spanS = 1, spanF = 0, spanRound = -1;
    auto loadSpan = [&](int round) {
        spanS = 1;
        spanF = 0;
        const tsa_span_group *gp = (tid < 64) ? cur.G0 : cur.G1;
        int n = (tid < 64) ? cur.N0 : cur.N1;
        if (round < n) {
            spanS = gp[round].SpanStart[tid & 63];
            spanF = gp[round].SpanFinish[tid & 63];
        }
        spanRound = round;
    };

    float m = 0, lacc = 0; // lacc = 128 * sum of weights
    float pfSk = 0, pfSv = 0;
    auto fetchScales = [&](int j0) {
        int j = j0 + tid;
        pfSk = 0;
        pfSv = 0;
        if (j < p.KeyRows) {
            pfSk = p.KScale.Row(head)[j];
            if (HAS_VSCALE) {
                pfSv = p.VScale.Row(head)[j] * svMult;
            }
        }
    };
    if (cur.Valid) {
        fetchScales(cur.J0);
    }

    int it = 0;
    while (cur.Valid) {
        const int slot = it % STAGES;
        if (cur.Round != spanRound) {
            loadSpan(cur.Round);
        }
        misc.ColTerm[tid] = make_float2(pfSk, p.Slope * (float)tid);
        if (HAS_VSCALE) {
            misc.SvTerm[tid] = pfSv;
        }
        const int j0 = cur.J0;
        const bool rowFull = spanS <= j0 && spanF >= j0 + TILE_N - 1;
        const bool rowAny = spanS <= j0 + TILE_N - 1 && spanF >= j0 && spanS <= spanF;
        const bool warpMasked = !__all_sync(0xffffffffu, rowFull);
        const bool warpAny = __any_sync(0xffffffffu, rowAny);
        const int flags = __syncthreads_or((warpMasked ? 1 : 0) | (failed ? 2 : 0));
        if (flags & 2) {
            failed = true;
            break;
        }
        const bool tileMasked = (flags & 1) != 0;

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
        // S(it) complete implies PV(it-1) complete: its K/V slot is free again
        if (tid == 0 && it >= 1 && prod.Valid && !failed) {
            issueLoad((it - 1) % STAGES, prod.J0);
            prod.Advance();
            ++issued;
        }

        uint32_t sreg[TILE_N];
        if (warpAny) {
            TmemLd32(tLane + 0, sreg);
            TmemLd32(tLane + 32, sreg + 32);
            TmemLd32(tLane + 64, sreg + 64);
            TmemLd32(tLane + 96, sreg + 96);
            TmemWaitLd();
            // pass 1: logits relative to the tile (rowOff is added after the max)
            float mx = -INFINITY;
            if (warpMasked) {
                const int ls = spanS - j0, lf = spanF - j0;
#pragma unroll
                for (int c = 0; c < TILE_N; ++c) {
                    float a = QK_I8 ? (float)(int)sreg[c] : __uint_as_float(sreg[c]);
                    float2 ct = misc.ColTerm[c];
                    float z = fmaf(a * ct.x, rowMult, ct.y);
                    z = (c >= ls && c <= lf) ? z : -INFINITY;
                    sreg[c] = __float_as_uint(z);
                    mx = fmaxf(mx, z);
                }
            } else {
#pragma unroll
                for (int c = 0; c < TILE_N; ++c) {
                    float a = QK_I8 ? (float)(int)sreg[c] : __uint_as_float(sreg[c]);
                    float2 ct = misc.ColTerm[c];
                    float z = fmaf(a * ct.x, rowMult, ct.y);
                    sreg[c] = __float_as_uint(z);
                    mx = fmaxf(mx, z);
                }
            }
            const float rowOff = -p.Slope * (float)(row - j0);
            const float newM = fmaxf(m, floorf(mx + rowOff)); // -inf stays below m
            const float alpha = exp2f(m - newM);
            if (it > 0 && __any_sync(0xffffffffu, newM != m)) {
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t o[32];
                    TmemLd32(tLane + TMEM_O_COL + c0, o);
                    TmemWaitLd();
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                    }
                    TmemSt32(tLane + TMEM_O_COL + c0, o);
                }
            }
            lacc *= alpha;
            m = newM;
            // pass 2: weights, packed e4m3 into the S columns
            const float eoff = rowOff - m + 7.0f;
#pragma unroll
            for (int c0 = 0; c0 < TILE_N; c0 += 32) {
                uint32_t pk[8], pl[8];
#pragma unroll
                for (int c = 0; c < 32; c += 4) {
                    float e[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float w = FastExp2(__uint_as_float(sreg[c0 + c + k]) + eoff);
                        lacc += w;
                        e[k] = HAS_VSCALE ? w * misc.SvTerm[c0 + c + k] : w;
                    }
                    uint32_t lo2 = PackE4M3x2(e[0], e[1]), hi2 = PackE4M3x2(e[2], e[3]);
                    pk[c >> 2] = lo2 | (hi2 << 16);
                    if (tileMasked) {
                        pl[c >> 2] = ResidualE4M3x2(e[0], e[1], lo2) | (ResidualE4M3x2(e[2], e[3], hi2) << 16);
                    }
                }
                TmemStN<8>(tLane + (c0 >> 2), pk);
                if (tileMasked) {
                    TmemStN<8>(tLane + 32 + (c0 >> 2), pl);
                }
            }
        } else {
            // no row of this warp attends this tile: zero weights, no exponentials
            uint32_t zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int c0 = 0; c0 < 32; c0 += 8) {
                TmemStN<8>(tLane + c0, zero);
                if (tileMasked) {
                    TmemStN<8>(tLane + 32 + c0, zero);
                }
            }
        }
        TmemWaitSt();
        TcFenceBefore();
        __syncthreads();
        if (tid == 0 && !failed) {
            TcFenceAfter();
            uint32_t vAddr = sVa + slot * SM::TILE_BYTES;
#pragma unroll
            for (int ks = 0; ks < TILE_N / 32; ++ks) {
                uint64_t bDesc = MakeSmemDesc(vAddr + ks * 32 * D, 16, GROUP_BYTES, SWZ);
                MmaF8TS(tmem + TMEM_O_COL, tmem + ks * 8, bDesc, IDESC_PV, (it > 0 || ks > 0) ? 1u : 0u);
            }
            if (tileMasked) {
#pragma unroll
                for (int ks = 0; ks < TILE_N / 32; ++ks) {
                    uint64_t bDesc = MakeSmemDesc(vAddr + ks * 32 * D, 16, GROUP_BYTES, SWZ);
                    MmaF8TS(tmem + TMEM_O_COL, tmem + 32 + ks * 8, bDesc, IDESC_PV, 1u);
                }
            }
            if (nxt.Valid) {
                int ns = (it + 1) % STAGES;
                if (WaitBar(&misc.BarFull[ns], ((it + 1) / STAGES) & 1)) {
                    ++landed;
                    TcFenceAfter();
                    issueQK(ns);
                } else {
                    failed = true;
                    if (p.Status) {
                        atomicOr(p.Status, kDevTimeoutTma);
                    }
                }
            }
            MmaCommit(&misc.BarMma);
        } else if (tid == 0) {
            MmaCommit(&misc.BarMma);
        }
        cur = nxt;
        ++it;
    }

    const int tiles = it;
    if (tiles > 0 && !failed) {
        if (!WaitBar(&misc.BarMma, tiles & 1)) {
            failed = true;
            if (p.Status) {
                atomicOr(p.Status, kDevTimeoutMma);
            }
        }
        TcFenceAfter();
    }
    failed = __syncthreads_or(failed ? 1 : 0) != 0;

    if (!failed) {
        const float lTot = lacc * (1.0f / 128.0f) + exp2f(-m);
        const float outMult = (HAS_VSCALE ? vRef : p.VVecScale) * (1.0f / 128.0f) / lTot;
        if (rowOk && p.Lse.Valid()) {
            p.Lse.Row(head)[row] = m + log2f(lTot);
        }
        const int esz = (p.OutDtype == TSA_F32) ? 4 : 2;
        char *oRow = p.Out.Row(rowOk ? row : 0) + (size_t)head * D * esz;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t o[32];
            if (tiles > 0) {
                TmemLd32(tLane + TMEM_O_COL + c0, o);
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
    } else if (tid == 0) {
        // drain copies that were requested but never consumed, so none lands after the CTA is gone
        for (int t = landed; t < issued; ++t) {
            WaitBar(&misc.BarFull[t % STAGES], (t / STAGES) & 1);
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == 0) {
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
template <int D>
__global__ void __launch_bounds__(FWD_THREADS) ScoresI8Kernel(const __grid_constant__ CUtensorMap tmQ,
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
typedef CUresult (*TEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static TEncodeTiled GetEncodeTiled()
{
    static TEncodeTiled fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
            fn = (TEncodeTiled)ptr;
        }
    }
    return fn;
}

// rows x (xsize bytes) matrix of bytes, box = 128 rows x headDim bytes, swizzle = headDim bytes
static int MakeTileMap(CUtensorMap *map, tsa_ptr2d a, int headDim, const char *what)
{
    TEncodeTiled enc = GetEncodeTiled();
    if (!enc) {
        return Fail(TSA_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    }
    cuuint64_t dims[2] = {(cuuint64_t)a.xsize, (cuuint64_t)a.ysize};
    cuuint64_t strides[1] = {(cuuint64_t)a.stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)headDim, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.data, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        headDim == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return Fail(TSA_CUDA_ERROR, "cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
    }
    return TSA_OK;
}

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

template <int D, bool QK_I8, bool HAS_VSCALE>
static int LaunchFwdT(const CUtensorMap &mq, const CUtensorMap &mk, const CUtensorMap &mv, const TFwdParams &fp, int qTiles, cudaStream_t stream)
{
    auto kern = FwdSm100Kernel<D, QK_I8, HAS_VSCALE>;
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
#define TSA_FWD_CASE(DD, I8, VS) \
    if (D == DD && i8 == I8 && hasVs == VS) return LaunchFwdT<DD, I8, VS>(mq, mk, mv, fp, qTiles, stream);
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
        ScoresI8Kernel<128><<<grid, FWD_THREADS, smemBytes, stream>>>(mq, mk, lenQ, lenK, scores, statusWord);
    } else {
        ScoresI8Kernel<64><<<grid, FWD_THREADS, smemBytes, stream>>>(mq, mk, lenQ, lenK, scores, statusWord);
    }
    return CheckCuda(cudaGetLastError(), "int8 score launch");
}

} // namespace tsa
