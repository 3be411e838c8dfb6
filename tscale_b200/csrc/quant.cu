// Per-row, per-tile quantisers and the dScale reduction: HBM-bound streaming kernels.
// One warp owns one (row, tile); lanes read VEC consecutive elements so a warp request covers a
// contiguous 32*VEC*sizeof(src) bytes and writes 32*VEC bytes.
// Reference behaviour: NormalizeVecsRowTile / NormalizeVecsRowTileMax
// (code/gpt/compute/row_tile_scale.cuh:11-34, 59-82), CalcDScale (gpt_att_fp16.cuh:621-643).
#include "tsa_common.cuh"
#include <type_traits>

namespace tsa {

template <class TSrc, int VEC>
__device__ __forceinline__ void LoadVec(const typename TSrc::T *p, float *dst)
{
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        dst[i] = TSrc::Load(p + i);
    }
}
template <>
__device__ __forceinline__ void LoadVec<TagF32, 4>(const float *p, float *dst)
{
    float4 v = *reinterpret_cast<const float4 *>(p);
    dst[0] = v.x, dst[1] = v.y, dst[2] = v.z, dst[3] = v.w;
}
template <>
__device__ __forceinline__ void LoadVec<TagF32, 2>(const float *p, float *dst)
{
    float2 v = *reinterpret_cast<const float2 *>(p);
    dst[0] = v.x, dst[1] = v.y;
}
template <>
__device__ __forceinline__ void LoadVec<TagF16, 4>(const __half *p, float *dst)
{
    uint2 raw = *reinterpret_cast<const uint2 *>(p);
    float2 a = __half22float2(*reinterpret_cast<__half2 *>(&raw.x));
    float2 b = __half22float2(*reinterpret_cast<__half2 *>(&raw.y));
    dst[0] = a.x, dst[1] = a.y, dst[2] = b.x, dst[3] = b.y;
}
template <>
__device__ __forceinline__ void LoadVec<TagBF16, 4>(const __nv_bfloat16 *p, float *dst)
{
    uint2 raw = *reinterpret_cast<const uint2 *>(p);
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&raw.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&raw.y));
    dst[0] = a.x, dst[1] = a.y, dst[2] = b.x, dst[3] = b.y;
}

// grid: x = ceil(rows * tiles / warpsPerBlock); rows = dst rows (>= len, padding rows are zeroed)
template <class TSrc, bool DST_E4M3, int VEC>
__global__ void __launch_bounds__(256) QuantRowsKernel(int kind, float vecScale, int len, int rows, int tileCount, int tile,
    P2D<typename TSrc::T> src, P2D<uint8_t> dst, P2D<float> scale)
{
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= rows * tileCount) {
        return;
    }
    int t = warp / tileCount;
    int tl = warp - t * tileCount;
    int base = tl * tile;
    constexpr int MAX_ITER = 8; // tile <= 32 * VEC * MAX_ITER
    float vals[MAX_ITER][VEC];
    int iters = tile / (32 * VEC);
    float sum2 = 0, mx = 0;
    if (t < len) {
#pragma unroll
        for (int it = 0; it < MAX_ITER; ++it) {
            if (it < iters) {
                LoadVec<TSrc, VEC>(src.Row(t) + base + (it * 32 + lane) * VEC, vals[it]);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    sum2 += vals[it][i] * vals[it][i];
                    mx = fmaxf(mx, fabsf(vals[it][i]));
                }
            }
        }
    }
    float discr = 0;
    if (kind == TSA_QUANT_ABSMAX) {
        mx = WarpMax(mx);
        if (mx > 0) {
            discr = DST_E4M3 ? __fdiv_rn(mx, 256.0f) : __fdiv_rn(mx, 127.0f);
        }
    } else {
        sum2 = WarpSum(sum2);
        if (sum2 > 0) {
            discr = __fmul_rn(__fsqrt_rn(__fdiv_rn(sum2, (float)tile)), vecScale);
        }
    }
    float mult = (discr > 0) ? __fdiv_rn(1.0f, discr) : 0.0f;
#pragma unroll
    for (int it = 0; it < MAX_ITER; ++it) {
        if (it < iters) {
            uint8_t *d = dst.Row(t) + base + (it * 32 + lane) * VEC;
            uint32_t packed = 0;
            if (t < len) {
                if (DST_E4M3) {
                    if (VEC == 4) {
                        packed = PackE4M3x4(vals[it][0] * mult, vals[it][1] * mult, vals[it][2] * mult, vals[it][3] * mult);
                    } else if (VEC == 2) {
                        packed = PackE4M3x2(vals[it][0] * mult, vals[it][1] * mult);
                    } else {
                        packed = PackE4M3x2(vals[it][0] * mult, 0.0f) & 0xff;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        packed |= (uint32_t)(FloatToI8Sat(vals[it][i] * mult) & 0xff) << (8 * i);
                    }
                }
            }
            if (VEC == 4) {
                *reinterpret_cast<uint32_t *>(d) = packed;
            } else if (VEC == 2) {
                *reinterpret_cast<uint16_t *>(d) = (uint16_t)packed;
            } else {
                *d = (uint8_t)packed;
            }
        }
    }
    if (lane == 0 && scale.Valid()) {
        scale.Row(tl)[t] = discr;
    }
}

template <class TSrc, bool DST_E4M3>
static int LaunchQuant(int kind, float vecScale, tsa_ptr2d src, tsa_ptr2d dst, tsa_ptr2d scale, int len, int tile, cudaStream_t stream)
{
    int rows = dst.ysize;
    int tileCount = dst.xsize / tile;
    long long warps = (long long)rows * tileCount;
    if (warps == 0) {
        return TSA_OK;
    }
    int blocks = (int)((warps * 32 + 255) / 256);
    P2D<typename TSrc::T> s(src);
    P2D<uint8_t> d(dst);
    P2D<float> sc(scale);
    bool aligned = ((uintptr_t)src.data % 16 == 0) && (src.stride_bytes % 16 == 0) && ((uintptr_t)dst.data % 4 == 0) && (dst.stride_bytes % 4 == 0);
    if (tile % 128 == 0 && aligned) {
        QuantRowsKernel<TSrc, DST_E4M3, 4><<<blocks, 256, 0, stream>>>(kind, vecScale, len, rows, tileCount, tile, s, d, sc);
    } else {
        QuantRowsKernel<TSrc, DST_E4M3, 1><<<blocks, 256, 0, stream>>>(kind, vecScale, len, rows, tileCount, tile, s, d, sc);
    }
    return CheckCuda(cudaGetLastError(), "tsa_quant_rows launch");
}

// dScale: one warp per (row, head)
__global__ void __launch_bounds__(256) DScaleKernel(int outDt, int gradDt, int len, int headCount, int headDim,
    P2D<char> out, P2D<char> dOut, P2D<float> dScale)
{
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= len * headCount) {
        return;
    }
    int t = warp / headCount;
    int head = warp - t * headCount;
    const void *o = out.Row(t);
    const void *g = dOut.Row(t);
    float sum = 0;
    for (int x = lane; x < headDim; x += 32) {
        int idx = head * headDim + x;
        sum += LoadAsFloat(o, idx, outDt) * LoadAsFloat(g, idx, gradDt);
    }
    sum = WarpSum(sum);
    if (lane == 0) {
        dScale.Row(head)[t] = sum;
    }
}

// dScale for 16-bit out / dOut: every thread takes 8 consecutive elements of both (one 16-byte load each), the
// headDim / 8 lanes of a head add up by shuffles.  A warp covers 256 consecutive elements of one row.
template <class T16>
__global__ void __launch_bounds__(256) DScaleVecKernel(int len, int headCount, int headDim, int chunksPerRow,
    P2D<char> out, P2D<char> dOut, P2D<float> dScale)
{
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)len * chunksPerRow) {
        return;
    }
    const int t = (int)(warp / chunksPerRow);
    const int x = ((int)(warp - (long long)t * chunksPerRow) * 32 + lane) * 8; // first element of this thread
    const int width = headCount * headDim;
    float sum = 0;
    if (x < width) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(out.Row(t) + (size_t)x * 2));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(dOut.Row(t) + (size_t)x * 2));
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 fa, fb;
            if (std::is_same<T16, __half>::value) {
                fa = __half22float2(*reinterpret_cast<const __half2 *>(&aw[k]));
                fb = __half22float2(*reinterpret_cast<const __half2 *>(&bw[k]));
            } else {
                fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&aw[k]));
                fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&bw[k]));
            }
            sum = fmaf(fa.x, fb.x, sum);
            sum = fmaf(fa.y, fb.y, sum);
        }
    }
    const int lanesPerHead = headDim / 8; // 2, 4, 8, 16 or 32
    for (int o = lanesPerHead >> 1; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    if (x < width && (lane & (lanesPerHead - 1)) == 0) {
        dScale.Row(x / headDim)[t] = sum;
    }
}

int LaunchDScale(int outDtype, int gradDtype, tsa_ptr2d out, tsa_ptr2d dOut, tsa_ptr2d dScale,
    int headCount, int headDimV, int len, cudaStream_t stream)
{
    long long warps = (long long)len * headCount;
    if (warps == 0) {
        return TSA_OK;
    }
    const bool pow2 = (headDimV & (headDimV - 1)) == 0 && headDimV >= 16 && headDimV <= 256;
    const bool aligned = (uintptr_t)out.data % 16 == 0 && out.stride_bytes % 16 == 0 && (uintptr_t)dOut.data % 16 == 0 && dOut.stride_bytes % 16 == 0;
    if (outDtype == gradDtype && (outDtype == TSA_F16 || outDtype == TSA_BF16) && pow2 && aligned) {
        const int chunksPerRow = (headCount * headDimV + 255) / 256;
        const long long vecWarps = (long long)len * chunksPerRow;
        const int vblocks = (int)((vecWarps * 32 + 255) / 256);
        if (outDtype == TSA_F16) {
            DScaleVecKernel<__half><<<vblocks, 256, 0, stream>>>(len, headCount, headDimV, chunksPerRow, P2D<char>(out), P2D<char>(dOut), P2D<float>(dScale));
        } else {
            DScaleVecKernel<__nv_bfloat16><<<vblocks, 256, 0, stream>>>(len, headCount, headDimV, chunksPerRow, P2D<char>(out), P2D<char>(dOut), P2D<float>(dScale));
        }
        return CheckCuda(cudaGetLastError(), "tsa_calc_dscale launch");
    }
    int blocks = (int)((warps * 32 + 255) / 256);
    DScaleKernel<<<blocks, 256, 0, stream>>>(outDtype, gradDtype, len, headCount, headDimV, P2D<char>(out), P2D<char>(dOut), P2D<float>(dScale));
    return CheckCuda(cudaGetLastError(), "tsa_calc_dscale launch");
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) int tsa_quant_rows(int kind, int srcDtype, int dstDtype, float vecScale, tsa_ptr2d src, tsa_ptr2d dst,
    tsa_ptr2d scale, int len, int tile, tsa_stream_t stream)
{
    TSA_REQUIRE(kind == TSA_QUANT_RMS || kind == TSA_QUANT_ABSMAX, "tsa_quant_rows: unknown kind %d", kind);
    TSA_REQUIRE(dstDtype == TSA_I8 || dstDtype == TSA_E4M3, "tsa_quant_rows: dst dtype must be i8 or e4m3");
    TSA_REQUIRE(src.data && dst.data, "tsa_quant_rows: null src/dst");
    TSA_REQUIRE(tile > 0 && tile % 32 == 0 && tile <= 1024, "tsa_quant_rows: tile %d must be a multiple of 32, at most 1024", tile);
    TSA_REQUIRE(dst.xsize % tile == 0 && src.xsize >= dst.xsize, "tsa_quant_rows: xsize %d is not a multiple of tile %d", dst.xsize, tile);
    TSA_REQUIRE(len >= 0 && len <= src.ysize && len <= dst.ysize, "tsa_quant_rows: len %d exceeds buffers (%d, %d rows)", len, src.ysize, dst.ysize);
    if (scale.data) {
        TSA_REQUIRE(scale.ysize >= dst.xsize / tile && scale.xsize >= dst.ysize, "tsa_quant_rows: scale plane too small");
    }
    cudaStream_t s = (cudaStream_t)stream;
    bool e4 = dstDtype == TSA_E4M3;
    switch (srcDtype) {
    case TSA_F32:
        return e4 ? LaunchQuant<TagF32, true>(kind, vecScale, src, dst, scale, len, tile, s) : LaunchQuant<TagF32, false>(kind, vecScale, src, dst, scale, len, tile, s);
    case TSA_F16:
        return e4 ? LaunchQuant<TagF16, true>(kind, vecScale, src, dst, scale, len, tile, s) : LaunchQuant<TagF16, false>(kind, vecScale, src, dst, scale, len, tile, s);
    case TSA_BF16:
        return e4 ? LaunchQuant<TagBF16, true>(kind, vecScale, src, dst, scale, len, tile, s) : LaunchQuant<TagBF16, false>(kind, vecScale, src, dst, scale, len, tile, s);
    }
    return Fail(TSA_BAD_ARG, "tsa_quant_rows: src dtype must be f32, f16 or bf16");
}

extern "C" __attribute__((visibility("default"))) int tsa_calc_dscale(int outDtype, int gradDtype, tsa_ptr2d out, tsa_ptr2d dOut, tsa_ptr2d dScale,
    int headCount, int headDimV, int len, tsa_stream_t stream)
{
    TSA_REQUIRE(out.data && dOut.data && dScale.data, "tsa_calc_dscale: null buffer");
    TSA_REQUIRE(outDtype >= TSA_F16 && outDtype <= TSA_F32 && gradDtype >= TSA_F16 && gradDtype <= TSA_F32, "tsa_calc_dscale: dtypes must be f16, bf16 or f32");
    TSA_REQUIRE(len <= out.ysize && len <= dOut.ysize && len <= dScale.xsize && headCount <= dScale.ysize, "tsa_calc_dscale: extents");
    TSA_REQUIRE(headCount * headDimV <= out.xsize && headCount * headDimV <= dOut.xsize, "tsa_calc_dscale: row width");
    return LaunchDScale(outDtype, gradDtype, out, dOut, dScale, headCount, headDimV, len, (cudaStream_t)stream);
}
