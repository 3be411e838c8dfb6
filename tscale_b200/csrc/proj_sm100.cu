// The projection that feeds the attention fused with its store op: int8 activations x int8 matrix on the tensor cores,
// then per-head RMS normalise, rope and quantise in the epilogue, straight from the accumulators.
// Replaces MulForwardInt8 / MulForwardFp8 <TStoreRowTileNormalizeRope> / <TStoreRowTileNormalize> of the reference
// (code/gpt/compute/gpt_cuda.cu:488-496; store ops code/lib/cuda/cuda_matmul.cuh:147-204, rope
// code/gpt/compute/gpt_rope.cuh:4-66): the fp32 projection never goes to memory.
//
//   y[t][n]  = (float)(int32 dot of x[t] and w[n]) * srcScale      (e4m3 operands: f32 dot on the tensor cores)
//   per head: discr = sqrt(sum y^2 / D) * vecScale;  z = y / discr;  rope (elements k and k + 32 of a 64-block);
//             dst = quantise(z) (int8 or e4m3);  scale[head][t] = discr
//
// One CTA = 128 rows of x times 256 output columns (4 heads of 64 or 2 of 128): tcgen05.mma kind::i8, M = 128, N = 256,
// exact int32 accumulators in 256 tensor-memory columns; thread 0 streams both operands through a TMA ring of 64-column
// chunks and issues the MMAs.  In the epilogue a row belongs to two threads (256 per CTA), each with half of the tile's
// heads, so a head's sum of squares, the rotation partners
// and the 64 output bytes of a block are all in one thread: no exchange between threads, sums in the scalar loop's
// order (bit-identical to the stand-alone normalise + rope + quantise of the CPU code on the same projection).
#include "att_sm100_common.cuh"

namespace tsa {

// 64-column chunks (64-byte swizzle) keep a CTA's ring at 96 KB, so two CTAs share an SM (2 x 256 tensor-memory
// columns) and one's epilogue overlaps the other's loads and MMAs
constexpr int PROJ_STAGES = 4;
constexpr int PROJ_M = 128, PROJ_N = 256, PROJ_KB = 64;
constexpr int PROJ_STAGE_BYTES = (PROJ_M + PROJ_N) * PROJ_KB;
constexpr int PROJ_SMEM_BYTES = PROJ_STAGES * PROJ_STAGE_BYTES + 1024 /* barriers */ + 1024 /* alignment */;

// bounded barrier wait of this kernel: about 20 ms, then the caller records which wait gave up
__device__ __forceinline__ bool ProjWait(uint64_t *bar, uint32_t parity)
{
    const long long t0 = clock64();
    for (;;) {
        if (MbarWaitBounded(bar, parity, 16)) {
            return true;
        }
        if (clock64() - t0 > (1ll << 25)) {
            return false;
        }
    }
}
constexpr int kProjEmptyTimeout = 0x100, kProjFullTimeout = 0x200, kProjDoneTimeout = 0x400;

struct TProjMisc {
    uint64_t Full[PROJ_STAGES], Empty[PROJ_STAGES], Done;
    uint32_t TmemBase;
};

struct TProjArgs {
    P2D<float> Rope;  // [len][D] f32, may be absent
    P2D<uint8_t> Dst; // [rows][H * D]
    P2D<float> Scale; // [H][rows], may be absent
    float VecScale, SrcScale, RopeDir;
    int Len, Rows, HeadCount, Chunks;
};

// X_E4M3: both operands are e4m3 bytes (MulForwardFp8, gpt_cuda.cu:488-491), products accumulate in f32 on the tensor
// cores (kind::f8f6f4); otherwise int8 x int8 with exact int32 accumulators (kind::i8).
// DST: TSA_I8, TSA_E4M3 (quantised) or TSA_F16 / TSA_BF16 (the normalised, rotated values themselves: the reference's K16).
template <int D, int DST, bool X_E4M3>
__global__ void __launch_bounds__(256, 2) ProjNormRopeKernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, TProjArgs a, int *status)
{
    // s32 accumulators, s8 x s8 -- or f32 accumulators, e4m3 x e4m3; both operands K-major
    constexpr uint32_t IDESC = X_E4M3 ? MakeInstrDesc(1, 0, 0, 0, 0, PROJ_M, PROJ_N) : MakeInstrDesc(2, 1, 1, 0, 0, PROJ_M, PROJ_N);
    auto accValue = [](uint32_t bits) { return X_E4M3 ? __uint_as_float(bits) : (float)(int32_t)bits; };
    constexpr int HPC = PROJ_N / D;                                          // heads per CTA
    extern __shared__ uint8_t projSmemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)projSmemRaw + 1023) & ~(uintptr_t)1023);
    TProjMisc &misc = *reinterpret_cast<TProjMisc *>(smem + PROJ_STAGES * PROJ_STAGE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5;
    const int rowBase = blockIdx.x * PROJ_M, colBase = blockIdx.y * PROJ_N;
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < PROJ_STAGES; ++s) {
            MbarInit(&misc.Full[s], 1);
            MbarInit(&misc.Empty[s], 1);
        }
        MbarInit(&misc.Done, 1);
        FenceBarrierInit();
    }
    if (warp == 0) {
        TmemAlloc(&misc.TmemBase, PROJ_N);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmem = misc.TmemBase;
    bool failed = false;
    if (tid == 0) {
        PrefetchTensorMap(&tmX);
        PrefetchTensorMap(&tmW);
        auto load = [&](int chunk) {
            const int s = chunk % PROJ_STAGES;
            uint8_t *sA = smem + s * PROJ_STAGE_BYTES, *sB = sA + PROJ_M * PROJ_KB;
            MbarExpectTx(&misc.Full[s], PROJ_STAGE_BYTES);
            TmaLoad2D(sA, &tmX, chunk * PROJ_KB, rowBase, &misc.Full[s]);
            TmaLoad2D(sB, &tmW, chunk * PROJ_KB, colBase, &misc.Full[s]);
        };
        // PROJ_AHEAD chunks in flight; a stage is refilled once the MMAs of two iterations ago have released it
        constexpr int PROJ_AHEAD = PROJ_STAGES - 2;
        const int chunks = a.Chunks;
        int issued = 0, landed = 0; // chunks requested / chunks whose copies were seen to arrive
        for (int c = 0; c < PROJ_AHEAD && c < chunks; ++c) {
            load(c);
            ++issued;
        }
        for (int c = 0; c < chunks; ++c) {
            const int ahead = c + PROJ_AHEAD;
            if (ahead < chunks) {
                if (ahead >= PROJ_STAGES && !ProjWait(&misc.Empty[ahead % PROJ_STAGES], (uint32_t)((ahead / PROJ_STAGES - 1) & 1))) {
                    failed = true;
                    if (status) {
                        atomicOr(status, kDevTimeoutMma | kProjEmptyTimeout);
                    }
                    break;
                }
                load(ahead);
                ++issued;
            }
            const int s = c % PROJ_STAGES;
            if (!ProjWait(&misc.Full[s], (uint32_t)((c / PROJ_STAGES) & 1))) {
                failed = true;
                if (status) {
                    atomicOr(status, kDevTimeoutTma | kProjFullTimeout);
                }
                break;
            }
            ++landed;
            TcFenceAfter();
            const uint32_t sA = SmemAddr(smem + s * PROJ_STAGE_BYTES), sB = sA + PROJ_M * PROJ_KB;
#pragma unroll
            for (int ks = 0; ks < PROJ_KB / 32; ++ks) {
                const uint64_t aDesc = MakeSmemDesc(sA + ks * 32, 16, 8 * PROJ_KB, PROJ_KB);
                const uint64_t bDesc = MakeSmemDesc(sB + ks * 32, 16, 8 * PROJ_KB, PROJ_KB);
                if (X_E4M3) {
                    MmaF8SS(tmem, aDesc, bDesc, IDESC, (c > 0 || ks > 0) ? 1u : 0u);
                } else {
                    MmaI8SS(tmem, aDesc, bDesc, IDESC, (c > 0 || ks > 0) ? 1u : 0u);
                }
            }
            MmaCommit(&misc.Empty[s]);
        }
        if (failed) {
            // copies that were requested but never consumed must not land after the CTA is gone: wait (bounded) for them
            for (int t = landed; t < issued; ++t) {
                ProjWait(&misc.Full[t % PROJ_STAGES], (uint32_t)((t / PROJ_STAGES) & 1));
            }
        }
        MmaCommit(&misc.Done);
    }
    if (!ProjWait(&misc.Done, 0)) {
        failed = true;
        if (status) {
            atomicOr(status, kDevTimeoutMma | kProjDoneTimeout);
        }
    }
    TcFenceAfter();
    failed = __syncthreads_or(failed ? 1 : 0) != 0;

    // every thread of a warp takes part in the tensor-memory loads (they are warp-wide instructions): rows past the
    // buffer only skip their global loads and stores
    const int rowInTile = tid & (PROJ_M - 1), colHalf = tid >> 7; // two threads per row: each takes half of the tile's heads
    const int t = rowBase + rowInTile;
    const bool inBuf = t < a.Rows;
    // the tile's rows of the rope table through shared memory (the ring is idle now): coalesced loads, and a row pitch
    // of D + 1 words lets every thread walk its own row without bank conflicts
    float *ropeTile = reinterpret_cast<float *>(smem);
    const bool withRope = a.Rope.Valid();
    if (!failed && withRope) {
        for (int idx = tid; idx < PROJ_M * (D / 4); idx += 256) {
            const int row = idx / (D / 4), c4 = idx - row * (D / 4);
            float4 v = make_float4(0, 0, 0, 0);
            if (rowBase + row < a.Len) {
                v = *reinterpret_cast<const float4 *>(a.Rope.Row(rowBase + row) + c4 * 4);
            }
            float *dstRope = ropeTile + row * (D + 1) + c4 * 4;
            dstRope[0] = v.x, dstRope[1] = v.y, dstRope[2] = v.z, dstRope[3] = v.w;
        }
        __syncthreads();
    }
    if (!failed) {
        const uint32_t tLane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const bool live = t < a.Len;
#pragma unroll 1
        for (int hh = colHalf * (HPC / 2); hh < (colHalf + 1) * (HPC / 2); ++hh) {
            const int head = blockIdx.y * HPC + hh;
            if (head >= a.HeadCount) {
                break;
            }
            // sum of squares of the head in column order, one rounding per product and per sum
            float sum2 = 0;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t r[32];
                TmemLd32(tLane + hh * D + c0, r);
                TmemWaitLd();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const float y = __fmul_rn(accValue(r[i]), a.SrcScale);
                    sum2 = __fadd_rn(sum2, __fmul_rn(y, y));
                }
            }
            float discr = 0;
            if (sum2 > 0 && live) {
                discr = __fmul_rn(__fsqrt_rn(__fdiv_rn(sum2, (float)D)), a.VecScale);
            }
            const float mult = discr > 0 ? __fdiv_rn(1.0f, discr) : 0.0f;
            constexpr int ES = (DST == TSA_F16 || DST == TSA_BF16) ? 2 : 1; // bytes per output element
            uint8_t *dstRow = a.Dst.Row(inBuf ? t : 0) + head * D * ES;
#pragma unroll 1
            for (int blk = 0; blk < D; blk += 64) {
                uint32_t lo[32], hi[32];
                TmemLd32(tLane + hh * D + blk, lo);
                TmemLd32(tLane + hh * D + blk + 32, hi);
                TmemWaitLd();
                uint32_t outLo[8], outHi[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float z0[4], z1[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int k = q * 4 + i;
                        float y0 = __fmul_rn(__fmul_rn(accValue(lo[k]), a.SrcScale), mult);
                        float y1 = __fmul_rn(__fmul_rn(accValue(hi[k]), a.SrcScale), mult);
                        if (withRope && live) {
                            const float cs = ropeTile[rowInTile * (D + 1) + blk + k];
                            const float sn = __fmul_rn(ropeTile[rowInTile * (D + 1) + blk + k + 32], a.RopeDir);
                            const float r0 = __fsub_rn(__fmul_rn(y0, cs), __fmul_rn(y1, sn));
                            const float r1 = __fadd_rn(__fmul_rn(y0, sn), __fmul_rn(y1, cs));
                            y0 = r0;
                            y1 = r1;
                        }
                        z0[i] = y0;
                        z1[i] = y1;
                    }
                    if (ES == 2) {
                        uint2 w0, w1;
                        if (DST == TSA_F16) {
                            const __half2 a0 = __floats2half2_rn(z0[0], z0[1]), a1 = __floats2half2_rn(z0[2], z0[3]);
                            const __half2 b0 = __floats2half2_rn(z1[0], z1[1]), b1 = __floats2half2_rn(z1[2], z1[3]);
                            w0 = make_uint2(*reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1));
                            w1 = make_uint2(*reinterpret_cast<const uint32_t *>(&b0), *reinterpret_cast<const uint32_t *>(&b1));
                        } else {
                            const __nv_bfloat162 a0 = __floats2bfloat162_rn(z0[0], z0[1]), a1 = __floats2bfloat162_rn(z0[2], z0[3]);
                            const __nv_bfloat162 b0 = __floats2bfloat162_rn(z1[0], z1[1]), b1 = __floats2bfloat162_rn(z1[2], z1[3]);
                            w0 = make_uint2(*reinterpret_cast<const uint32_t *>(&a0), *reinterpret_cast<const uint32_t *>(&a1));
                            w1 = make_uint2(*reinterpret_cast<const uint32_t *>(&b0), *reinterpret_cast<const uint32_t *>(&b1));
                        }
                        if (inBuf) {
                            *reinterpret_cast<uint2 *>(dstRow + (blk + q * 4) * 2) = w0;
                            *reinterpret_cast<uint2 *>(dstRow + (blk + 32 + q * 4) * 2) = w1;
                        }
                    } else if (DST == TSA_E4M3) {
                        outLo[q] = PackE4M3x4(z0[0], z0[1], z0[2], z0[3]);
                        outHi[q] = PackE4M3x4(z1[0], z1[1], z1[2], z1[3]);
                    } else {
                        outLo[q] = 0;
                        outHi[q] = 0;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            outLo[q] |= (uint32_t)(FloatToI8Sat(z0[i]) & 0xff) << (8 * i);
                            outHi[q] |= (uint32_t)(FloatToI8Sat(z1[i]) & 0xff) << (8 * i);
                        }
                    }
                }
                if (inBuf && ES == 1) {
                    if ((((uintptr_t)a.Dst.Data | (uintptr_t)a.Dst.Stride) & 31) == 0) {
                        // two 32-byte stores: whole sectors from a thread that owns the row
                        StGlobal256(dstRow + blk, outLo);
                        StGlobal256(dstRow + blk + 32, outHi);
                    } else {
                        uint4 *d4 = reinterpret_cast<uint4 *>(dstRow + blk);
                        d4[0] = make_uint4(outLo[0], outLo[1], outLo[2], outLo[3]);
                        d4[1] = make_uint4(outLo[4], outLo[5], outLo[6], outLo[7]);
                        d4[2] = make_uint4(outHi[0], outHi[1], outHi[2], outHi[3]);
                        d4[3] = make_uint4(outHi[4], outHi[5], outHi[6], outHi[7]);
                    }
                }
            }
            if (a.Scale.Valid() && inBuf) {
                a.Scale.Row(head)[t] = discr;
            }
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == 0) {
        TmemDealloc(tmem, PROJ_N);
    }
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) int tsa_matmul_norm_rope_quant(int srcDtype, int dstDtype, float vecScale, float srcScale, tsa_ptr2d x, tsa_ptr2d w,
    tsa_ptr2d rope, float ropeDir, tsa_ptr2d dst, tsa_ptr2d scale, int headCount, int headDim, int len, int *statusWord, tsa_stream_t stream)
{
    TSA_REQUIRE(srcDtype == TSA_I8 || srcDtype == TSA_E4M3, "tsa_matmul_norm_rope_quant: x and w must both be i8 or both e4m3");
    TSA_REQUIRE(dstDtype == TSA_I8 || dstDtype == TSA_E4M3 || dstDtype == TSA_F16 || dstDtype == TSA_BF16,
        "tsa_matmul_norm_rope_quant: dst dtype must be i8, e4m3, f16 or bf16");
    TSA_REQUIRE(x.data && w.data && dst.data, "tsa_matmul_norm_rope_quant: null x / w / dst");
    TSA_REQUIRE(headCount > 0 && (headDim == 64 || headDim == 128), "tsa_matmul_norm_rope_quant: head size %d must be 64 or 128", headDim);
    const int dim = x.xsize, outCols = headCount * headDim;
    TSA_REQUIRE(dim > 0 && dim % PROJ_KB == 0 && w.xsize == dim, "tsa_matmul_norm_rope_quant: inner size %d (x) / %d (w) must be equal multiples of %d", dim,
        w.xsize, PROJ_KB);
    TSA_REQUIRE(w.ysize >= outCols && dst.xsize >= outCols, "tsa_matmul_norm_rope_quant: w has %d rows, dst %d columns, H*D = %d", w.ysize, dst.xsize, outCols);
    TSA_REQUIRE(len >= 0 && len <= x.ysize && len <= dst.ysize, "tsa_matmul_norm_rope_quant: len %d exceeds buffers (%d, %d rows)", len, x.ysize, dst.ysize);
    TSA_REQUIRE((uintptr_t)x.data % 16 == 0 && x.stride_bytes % 16 == 0 && (uintptr_t)w.data % 16 == 0 && w.stride_bytes % 16 == 0 &&
            (uintptr_t)dst.data % 16 == 0 && dst.stride_bytes % 16 == 0,
        "tsa_matmul_norm_rope_quant: x, w and dst must be 16-byte aligned with 16-byte multiples as row strides");
    if (scale.data) {
        TSA_REQUIRE(scale.ysize >= headCount && scale.xsize >= dst.ysize, "tsa_matmul_norm_rope_quant: scale plane too small");
    }
    if (rope.data) {
        TSA_REQUIRE(rope.xsize >= headDim && rope.ysize >= len, "tsa_matmul_norm_rope_quant: rope table smaller than [len][headDim]");
        TSA_REQUIRE((uintptr_t)rope.data % 16 == 0 && rope.stride_bytes % 16 == 0, "tsa_matmul_norm_rope_quant: rope table must be 16-byte aligned");
    }
    if (dst.ysize == 0) {
        return TSA_OK;
    }
    CUtensorMap mx, mw;
    tsa_ptr2d xv = x;
    xv.ysize = len; // rows past len read as zeros
    int rc = len > 0 ? MakeTileMapEx(&mx, xv, 1, PROJ_KB, PROJ_M, "x") : MakeTileMapEx(&mx, x, 1, PROJ_KB, PROJ_M, "x");
    if (rc == TSA_OK) {
        tsa_ptr2d wv = w;
        wv.ysize = outCols;
        rc = MakeTileMapEx(&mw, wv, 1, PROJ_KB, PROJ_N, "w");
    }
    if (rc != TSA_OK) {
        return rc;
    }
    TProjArgs a;
    a.Rope = P2D<float>(rope);
    a.Dst = P2D<uint8_t>(dst);
    a.Scale = P2D<float>(scale);
    a.VecScale = vecScale;
    a.SrcScale = srcScale;
    a.RopeDir = ropeDir;
    a.Len = len;
    a.Rows = dst.ysize;
    a.HeadCount = headCount;
    a.Chunks = dim / PROJ_KB;
    dim3 grid((dst.ysize + PROJ_M - 1) / PROJ_M, (outCols + PROJ_N - 1) / PROJ_N);
    const bool x8 = srcDtype == TSA_E4M3;
    const void *kern = nullptr;
#define TSA_PROJ_CASE(DD, DT, X8)                                       \
    if (headDim == DD && dstDtype == DT && x8 == X8) {                  \
        kern = (const void *)ProjNormRopeKernel<DD, DT, X8>;            \
    }
#define TSA_PROJ_CASES(DD, X8) TSA_PROJ_CASE(DD, TSA_I8, X8) TSA_PROJ_CASE(DD, TSA_E4M3, X8) TSA_PROJ_CASE(DD, TSA_F16, X8) TSA_PROJ_CASE(DD, TSA_BF16, X8)
    TSA_PROJ_CASES(64, false)
    TSA_PROJ_CASES(64, true)
    TSA_PROJ_CASES(128, false)
    TSA_PROJ_CASES(128, true)
#undef TSA_PROJ_CASES
#undef TSA_PROJ_CASE
    rc = CheckCuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PROJ_SMEM_BYTES), "cudaFuncSetAttribute");
    if (rc != TSA_OK) {
        return rc;
    }
    void *args[] = {&mx, &mw, &a, &statusWord};
    return CheckCuda(cudaLaunchKernel(kern, grid, dim3(256), args, PROJ_SMEM_BYTES, (cudaStream_t)stream), "tsa_matmul_norm_rope_quant launch");
}
