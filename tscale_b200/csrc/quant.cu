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

template <>
__device__ __forceinline__ void LoadVec<TagF32, 8>(const float *p, float *dst)
{
    LoadVec<TagF32, 4>(p, dst);
    LoadVec<TagF32, 4>(p + 4, dst + 4);
}
template <>
__device__ __forceinline__ void LoadVec<TagF16, 8>(const __half *p, float *dst)
{
    uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        dst[2 * i] = a.x, dst[2 * i + 1] = a.y;
    }
}
template <>
__device__ __forceinline__ void LoadVec<TagBF16, 8>(const __nv_bfloat16 *p, float *dst)
{
    uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
        dst[2 * i] = a.x, dst[2 * i + 1] = a.y;
    }
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

// ---- producer of the attention inputs: per-head RMS normalise, rope, quantise ---------------------------------
// A lane holds both rope partners: EPL consecutive elements from k and EPL from k + 32 of one 64-element block
// (code/gpt/att/rope.cpp:28-46 rotates k with k + 32), so the rotation needs no exchange between lanes.  EPL = 4 for
// f32 sources, 8 for 16-bit ones (16-byte loads either way): 32 / EPL lanes cover a block, a warp item = 64 * EPL
// consecutive elements of a row; heads wider than an item take several steps.  A warp works on ITEMS items at once
// (all their loads are issued before the first reduction) so that enough bytes are in flight per SM.
template <class TSrc, class TRope, bool DST_E4M3, int EPL, int ITEMS, int STEPS>
__global__ void __launch_bounds__(256) NormRopeQuantKernel(float vecScale, float ropeDir, int len, int rows, int headCount, int headShift,
    P2D<typename TSrc::T> src, P2D<typename TRope::T> rope, P2D<uint8_t> dst, P2D<float> scale)
{
    constexpr int LPB = 32 / EPL;                                   // lanes per 64-element block
    constexpr int STEP_ELEMS = 64 * EPL;                            // elements of a warp step
    const int headDim = 1 << headShift;
    const int span = STEP_ELEMS * STEPS;                            // elements of one item
    const int width = headCount << headShift;
    const int groups = (width + span - 1) / span;                   // items per row
    const unsigned items = (unsigned)rows * (unsigned)groups;      // the launcher checks that this fits 31 bits
    const unsigned first = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * ITEMS;
    const int lane = threadIdx.x & 31;
    if (first >= items) {
        return;
    }
    const int firstRow = (int)(first / (unsigned)groups), firstGroup = (int)(first - (unsigned)firstRow * (unsigned)groups);
    const float invHeadDim = 1.0f / (float)headDim;                 // a power of two: multiplying by it is the exact division
    const int laneOff = (lane / LPB) * 64 + (lane % LPB) * EPL;     // first element of the lane inside a step
    float lo[ITEMS][STEPS][EPL], hi[ITEMS][STEPS][EPL];
    int row[ITEMS], base[ITEMS];
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        // item first + j: ITEMS <= groups or groups == 1, so one wrap at most
        int g = firstGroup + j, r = firstRow;
        if (g >= groups) {
            r += g / groups;
            g = g % groups;
        }
        row[j] = first + j < items ? r : rows;                       // rows: nothing to do
        base[j] = first + j < items ? g * span : 0;
#pragma unroll
        for (int st = 0; st < STEPS; ++st) {
            const int e = base[j] + st * STEP_ELEMS + laneOff;
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                lo[j][st][i] = 0;
                hi[j][st][i] = 0;
            }
            if (row[j] < len && e < width) {
                LoadVec<TSrc, EPL>(src.Row(row[j]) + e, lo[j][st]);
                LoadVec<TSrc, EPL>(src.Row(row[j]) + e + 32, hi[j][st]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
        const int t = row[j];
        float sum2 = 0;
#pragma unroll
        for (int st = 0; st < STEPS; ++st) {
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                sum2 += lo[j][st][i] * lo[j][st][i] + hi[j][st][i] * hi[j][st][i];
            }
        }
        // sum over the head: LPB lanes per 64 elements
        const int headLanes = min(32, (headDim / 64) * LPB);
        for (int o = 1; o < headLanes; o <<= 1) {
            sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
        }
        float discr = 0;
        if (sum2 > 0) {
            discr = __fmul_rn(__fsqrt_rn(__fmul_rn(sum2, invHeadDim)), vecScale);
        }
        const float mult = (discr > 0) ? __fdiv_rn(1.0f, discr) : 0.0f;
#pragma unroll
        for (int st = 0; st < STEPS; ++st) {
            const int e = base[j] + st * STEP_ELEMS + laneOff;
            const bool live = t < len && e < width;
            // packed f32x2 arithmetic (two elements per instruction, each product and sum rounded on its own like the
            // scalar form: no fused multiply-add)
            float y0[EPL], y1[EPL];
            const float2 mult2 = make_float2(mult, mult);
#pragma unroll
            for (int i = 0; i < EPL; i += 2) {
                const float2 a = __fmul2_rn(make_float2(lo[j][st][i], lo[j][st][i + 1]), mult2);
                const float2 b = __fmul2_rn(make_float2(hi[j][st][i], hi[j][st][i + 1]), mult2);
                y0[i] = a.x, y0[i + 1] = a.y, y1[i] = b.x, y1[i + 1] = b.y;
            }
            if (rope.Valid() && live) {
                float cs[EPL], sn[EPL];
                const int k = e & (headDim - 1);
                LoadVec<TRope, EPL>(rope.Row(t) + k, cs);
                LoadVec<TRope, EPL>(rope.Row(t) + k + 32, sn);
                const float2 dir2 = make_float2(ropeDir, ropeDir), ndir2 = make_float2(-ropeDir, -ropeDir);
#pragma unroll
                for (int i = 0; i < EPL; i += 2) {
                    const float2 c2 = make_float2(cs[i], cs[i + 1]), s2 = make_float2(sn[i], sn[i + 1]);
                    const float2 sp = __fmul2_rn(s2, dir2), sm = __fmul2_rn(s2, ndir2); // sin * dir and its negative (exact)
                    const float2 v0 = make_float2(y0[i], y0[i + 1]), v1 = make_float2(y1[i], y1[i + 1]);
                    // r0 = v0 cos - v1 sin,  r1 = v0 sin + v1 cos
                    const float2 r0 = __fadd2_rn(__fmul2_rn(v0, c2), __fmul2_rn(v1, sm));
                    const float2 r1 = __fadd2_rn(__fmul2_rn(v0, sp), __fmul2_rn(v1, c2));
                    y0[i] = r0.x, y0[i + 1] = r0.y, y1[i] = r1.x, y1[i + 1] = r1.y;
                }
            }
            if (t < rows && e < width) {
                uint32_t p0[EPL / 4], p1[EPL / 4];
#pragma unroll
                for (int q = 0; q < EPL / 4; ++q) {
                    p0[q] = 0;
                    p1[q] = 0;
                    if (live) {
                        if (DST_E4M3) {
                            p0[q] = PackE4M3x4(y0[4 * q], y0[4 * q + 1], y0[4 * q + 2], y0[4 * q + 3]);
                            p1[q] = PackE4M3x4(y1[4 * q], y1[4 * q + 1], y1[4 * q + 2], y1[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                p0[q] |= (uint32_t)(FloatToI8Sat(y0[4 * q + i]) & 0xff) << (8 * i);
                                p1[q] |= (uint32_t)(FloatToI8Sat(y1[4 * q + i]) & 0xff) << (8 * i);
                            }
                        }
                    }
                }
                if (EPL == 8) {
                    *reinterpret_cast<uint2 *>(dst.Row(t) + e) = make_uint2(p0[0], p0[EPL / 4 - 1]);
                    *reinterpret_cast<uint2 *>(dst.Row(t) + e + 32) = make_uint2(p1[0], p1[EPL / 4 - 1]);
                } else {
                    *reinterpret_cast<uint32_t *>(dst.Row(t) + e) = p0[0];
                    *reinterpret_cast<uint32_t *>(dst.Row(t) + e + 32) = p1[0];
                }
                // one lane per head writes the scale: the lane that holds the head's first element
                if (scale.Valid() && st == 0 && (e & (headDim - 1)) == 0) {
                    scale.Row(e >> headShift)[t] = (t < len) ? discr : 0.0f;
                }
            }
        }
    }
}

template <class TSrc, class TRope>
static int LaunchNormRope(bool e4, float vecScale, float ropeDir, tsa_ptr2d src, tsa_ptr2d rope, tsa_ptr2d dst, tsa_ptr2d scale,
    int headCount, int headDim, int len, cudaStream_t stream)
{
    constexpr int EPL = sizeof(typename TSrc::T) == 4 ? 4 : 8;
    const int rows = dst.ysize;
    const int stepElems = 64 * EPL;
    const int steps = headDim > stepElems ? headDim / stepElems : 1;
    int headShift = 6;
    while ((1 << headShift) < headDim) {
        ++headShift;
    }
    const long long items = (long long)rows * ((headCount * headDim + stepElems * steps - 1) / (stepElems * steps));
    if (items == 0) {
        return TSA_OK;
    }
    TSA_REQUIRE(items < (1ll << 31) - 64, "tsa_norm_rope_quant: %lld warp items, fewer than 2^31 supported", items);
    P2D<typename TSrc::T> s(src);
    P2D<typename TRope::T> r(rope);
    P2D<uint8_t> d(dst);
    P2D<float> sc(scale);
#define TSA_NRQ_LAUNCH(E4, ITEMS, STEPS)                                                                                         \
    {                                                                                                                           \
        const long long warps = (items + ITEMS - 1) / ITEMS;                                                                    \
        const int blocks = (int)((warps * 32 + 255) / 256);                                                                     \
        NormRopeQuantKernel<TSrc, TRope, E4, EPL, ITEMS, STEPS><<<blocks, 256, 0, stream>>>(vecScale, ropeDir, len, rows, headCount, headShift, s, r, d, sc); \
    }
    if (steps == 1) {
        if (e4) TSA_NRQ_LAUNCH(true, 2, 1) else TSA_NRQ_LAUNCH(false, 2, 1)
    } else {
        if (e4) TSA_NRQ_LAUNCH(true, 1, 2) else TSA_NRQ_LAUNCH(false, 1, 2)
    }
#undef TSA_NRQ_LAUNCH
    return CheckCuda(cudaGetLastError(), "tsa_norm_rope_quant launch");
}

// N (4 or 8) consecutive results as one or two 8 / 16-byte stores
template <class TDst, int N>
__device__ __forceinline__ void StoreVec(typename TDst::T *p, const float *v)
{
    if (sizeof(typename TDst::T) == 4) {
#pragma unroll
        for (int i = 0; i < N; i += 4) {
            *reinterpret_cast<float4 *>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
    } else {
        uint32_t w[N / 2];
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            if (std::is_same<TDst, TagF16>::value) {
                __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&h);
            } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&h);
            }
        }
        if (N == 8) {
            *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[N / 2 - 2], w[N / 2 - 1]);
        } else {
            *reinterpret_cast<uint2 *>(p) = make_uint2(w[0], w[1]);
        }
    }
}

// ---- back-propagation through the producer: inverse rope, then the RMS-normalise gradient ----------------------
// Same lane layout as NormRopeQuantKernel.  grad (gradient with respect to the roped unit-RMS vector) and src (the raw
// projection) are read once; out = sqrt(D / sum2) * (g - src * dot(src, g) / sum2) with g = grad rotated back
// (code/gpt/compute/gpt_cpu.cpp:329-360, 759-764).
template <class TSrc, class TGrad, class TRope, int EPL, int STEPS>
__global__ void __launch_bounds__(256) RopeNormBwdKernel(float ropeDir, int len, int headCount, int headShift,
    P2D<typename TSrc::T> src, P2D<typename TGrad::T> grad, P2D<typename TRope::T> rope, P2D<typename TGrad::T> out)
{
    constexpr int LPB = 32 / EPL;
    constexpr int STEP_ELEMS = 64 * EPL;
    const int headDim = 1 << headShift;
    const int span = STEP_ELEMS * STEPS;
    const int width = headCount << headShift;
    const int groups = (width + span - 1) / span;
    const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (item >= (long long)len * groups) {
        return;
    }
    const int t = (int)(item / groups);
    const int base = (int)(item - (long long)t * groups) * span;
    const int laneOff = (lane / LPB) * 64 + (lane % LPB) * EPL;
    float s0[STEPS][EPL], s1[STEPS][EPL], g0[STEPS][EPL], g1[STEPS][EPL];
    float sum2 = 0, dp = 0;
#pragma unroll
    for (int st = 0; st < STEPS; ++st) {
        const int e = base + st * STEP_ELEMS + laneOff;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            s0[st][i] = s1[st][i] = g0[st][i] = g1[st][i] = 0;
        }
        if (e < width) {
            LoadVec<TSrc, EPL>(src.Row(t) + e, s0[st]);
            LoadVec<TSrc, EPL>(src.Row(t) + e + 32, s1[st]);
            LoadVec<TGrad, EPL>(grad.Row(t) + e, g0[st]);
            LoadVec<TGrad, EPL>(grad.Row(t) + e + 32, g1[st]);
            if (rope.Valid()) {
                float cs[EPL], sn[EPL];
                const int k = e & (headDim - 1);
                LoadVec<TRope, EPL>(rope.Row(t) + k, cs);
                LoadVec<TRope, EPL>(rope.Row(t) + k + 32, sn);
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    const float sinValue = __fmul_rn(sn[i], -ropeDir); // rotate back
                    const float r0 = __fsub_rn(__fmul_rn(g0[st][i], cs[i]), __fmul_rn(g1[st][i], sinValue));
                    const float r1 = __fadd_rn(__fmul_rn(g0[st][i], sinValue), __fmul_rn(g1[st][i], cs[i]));
                    g0[st][i] = r0;
                    g1[st][i] = r1;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
            sum2 += s0[st][i] * s0[st][i] + s1[st][i] * s1[st][i];
            dp += s0[st][i] * g0[st][i] + s1[st][i] * g1[st][i];
        }
    }
    const int headLanes = min(32, (headDim / 64) * LPB);
    for (int o = 1; o < headLanes; o <<= 1) {
        sum2 += __shfl_xor_sync(0xffffffffu, sum2, o);
        dp += __shfl_xor_sync(0xffffffffu, dp, o);
    }
    float sigma = 0, scale = 0;
    if (sum2 > 0) {
        sigma = __fdiv_rn(dp, sum2);
        scale = __fsqrt_rn(__fdiv_rn((float)headDim, sum2));
    }
#pragma unroll
    for (int st = 0; st < STEPS; ++st) {
        const int e = base + st * STEP_ELEMS + laneOff;
        if (e < width) {
            float r0[EPL], r1[EPL];
#pragma unroll
            for (int i = 0; i < EPL; ++i) {
                r0[i] = __fmul_rn(scale, __fsub_rn(g0[st][i], __fmul_rn(s0[st][i], sigma)));
                r1[i] = __fmul_rn(scale, __fsub_rn(g1[st][i], __fmul_rn(s1[st][i], sigma)));
            }
            StoreVec<TGrad, EPL>(out.Row(t) + e, r0);
            StoreVec<TGrad, EPL>(out.Row(t) + e + 32, r1);
        }
    }
}

template <class TSrc, class TGrad, class TRope>
static int LaunchRopeNormBwd(float ropeDir, tsa_ptr2d src, tsa_ptr2d grad, tsa_ptr2d rope, tsa_ptr2d out, int headCount, int headDim, int len,
    cudaStream_t stream)
{
    constexpr int EPL = (sizeof(typename TSrc::T) == 4 || sizeof(typename TGrad::T) == 4) ? 4 : 8;
    const int stepElems = 64 * EPL;
    const int steps = headDim > stepElems ? headDim / stepElems : 1;
    int headShift = 6;
    while ((1 << headShift) < headDim) {
        ++headShift;
    }
    const long long items = (long long)len * ((headCount * headDim + stepElems * steps - 1) / (stepElems * steps));
    if (items == 0) {
        return TSA_OK;
    }
    const int blocks = (int)((items * 32 + 255) / 256);
    P2D<typename TSrc::T> s(src);
    P2D<typename TGrad::T> g(grad), o(out);
    P2D<typename TRope::T> r(rope);
    if (steps == 1) {
        RopeNormBwdKernel<TSrc, TGrad, TRope, EPL, 1><<<blocks, 256, 0, stream>>>(ropeDir, len, headCount, headShift, s, g, r, o);
    } else {
        RopeNormBwdKernel<TSrc, TGrad, TRope, EPL, 2><<<blocks, 256, 0, stream>>>(ropeDir, len, headCount, headShift, s, g, r, o);
    }
    return CheckCuda(cudaGetLastError(), "tsa_rope_norm_bwd launch");
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

extern "C" __attribute__((visibility("default"))) int tsa_norm_rope_quant(int srcDtype, int dstDtype, float vecScale, tsa_ptr2d src,
    tsa_ptr2d rope, int ropeDtype, float ropeDir, tsa_ptr2d dst, tsa_ptr2d scale, int headCount, int headDim, int len, tsa_stream_t stream)
{
    TSA_REQUIRE(dstDtype == TSA_I8 || dstDtype == TSA_E4M3, "tsa_norm_rope_quant: dst dtype must be i8 or e4m3");
    TSA_REQUIRE(src.data && dst.data, "tsa_norm_rope_quant: null src/dst");
    TSA_REQUIRE(headCount > 0 && (headDim == 64 || headDim == 128 || headDim == 256 || headDim == 512), "tsa_norm_rope_quant: head size %d must be 64, 128, 256 or 512", headDim);
    TSA_REQUIRE(dst.xsize >= headCount * headDim && src.xsize >= headCount * headDim, "tsa_norm_rope_quant: rows narrower than H*D");
    TSA_REQUIRE(len >= 0 && len <= src.ysize && len <= dst.ysize, "tsa_norm_rope_quant: len %d exceeds buffers (%d, %d rows)", len, src.ysize, dst.ysize);
    TSA_REQUIRE((uintptr_t)src.data % 16 == 0 && src.stride_bytes % 16 == 0 && (uintptr_t)dst.data % 8 == 0 && dst.stride_bytes % 8 == 0,
        "tsa_norm_rope_quant: src must be 16-byte aligned, dst 8-byte aligned");
    if (scale.data) {
        TSA_REQUIRE(scale.ysize >= headCount && scale.xsize >= dst.ysize, "tsa_norm_rope_quant: scale plane too small");
    }
    if (rope.data) {
        TSA_REQUIRE(ropeDtype == TSA_F32 || ropeDtype == TSA_F16, "tsa_norm_rope_quant: rope dtype must be f32 or f16");
        TSA_REQUIRE(rope.xsize >= headDim && rope.ysize >= len, "tsa_norm_rope_quant: rope table smaller than [len][headDim]");
        TSA_REQUIRE((uintptr_t)rope.data % 16 == 0 && rope.stride_bytes % 16 == 0, "tsa_norm_rope_quant: rope table must be 16-byte aligned");
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool e4 = dstDtype == TSA_E4M3;
    const bool ropeF16 = rope.data && ropeDtype == TSA_F16;
#define TSA_NRQ(TS)                                                                                                            \
    return ropeF16 ? LaunchNormRope<TS, TagF16>(e4, vecScale, ropeDir, src, rope, dst, scale, headCount, headDim, len, s)     \
                   : LaunchNormRope<TS, TagF32>(e4, vecScale, ropeDir, src, rope, dst, scale, headCount, headDim, len, s);
    switch (srcDtype) {
    case TSA_F32:
        TSA_NRQ(TagF32)
    case TSA_F16:
        TSA_NRQ(TagF16)
    case TSA_BF16:
        TSA_NRQ(TagBF16)
    }
#undef TSA_NRQ
    return Fail(TSA_BAD_ARG, "tsa_norm_rope_quant: src dtype must be f32, f16 or bf16");
}

extern "C" __attribute__((visibility("default"))) int tsa_rope_norm_bwd(int srcDtype, int gradDtype, tsa_ptr2d src, tsa_ptr2d grad,
    tsa_ptr2d rope, int ropeDtype, float ropeDir, tsa_ptr2d out, int headCount, int headDim, int len, tsa_stream_t stream)
{
    TSA_REQUIRE(src.data && grad.data && out.data, "tsa_rope_norm_bwd: null buffer");
    TSA_REQUIRE(headCount > 0 && (headDim == 64 || headDim == 128 || headDim == 256 || headDim == 512), "tsa_rope_norm_bwd: head size %d must be 64, 128, 256 or 512", headDim);
    const int width = headCount * headDim;
    TSA_REQUIRE(src.xsize >= width && grad.xsize >= width && out.xsize >= width, "tsa_rope_norm_bwd: rows narrower than H*D");
    TSA_REQUIRE(len >= 0 && len <= src.ysize && len <= grad.ysize && len <= out.ysize, "tsa_rope_norm_bwd: len %d exceeds buffers", len);
    TSA_REQUIRE((uintptr_t)src.data % 16 == 0 && src.stride_bytes % 16 == 0 && (uintptr_t)grad.data % 16 == 0 && grad.stride_bytes % 16 == 0 &&
                    (uintptr_t)out.data % 16 == 0 && out.stride_bytes % 16 == 0, "tsa_rope_norm_bwd: buffers must be 16-byte aligned");
    if (rope.data) {
        TSA_REQUIRE(ropeDtype == TSA_F32 || ropeDtype == TSA_F16, "tsa_rope_norm_bwd: rope dtype must be f32 or f16");
        TSA_REQUIRE(rope.xsize >= headDim && rope.ysize >= len, "tsa_rope_norm_bwd: rope table smaller than [len][headDim]");
        TSA_REQUIRE((uintptr_t)rope.data % 16 == 0 && rope.stride_bytes % 16 == 0, "tsa_rope_norm_bwd: rope table must be 16-byte aligned");
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool ropeF16 = rope.data && ropeDtype == TSA_F16;
#define TSA_RNB(TS, TG)                                                                                                   \
    return ropeF16 ? LaunchRopeNormBwd<TS, TG, TagF16>(ropeDir, src, grad, rope, out, headCount, headDim, len, s)        \
                   : LaunchRopeNormBwd<TS, TG, TagF32>(ropeDir, src, grad, rope, out, headCount, headDim, len, s);
    if (srcDtype == TSA_F32 && gradDtype == TSA_F32) {
        TSA_RNB(TagF32, TagF32)
    }
    if (srcDtype == TSA_BF16 && gradDtype == TSA_BF16) {
        TSA_RNB(TagBF16, TagBF16)
    }
    if (srcDtype == TSA_F16 && gradDtype == TSA_F16) {
        TSA_RNB(TagF16, TagF16)
    }
    if (srcDtype == TSA_F32 && gradDtype == TSA_BF16) {
        TSA_RNB(TagF32, TagBF16)
    }
    if (srcDtype == TSA_BF16 && gradDtype == TSA_F32) {
        TSA_RNB(TagBF16, TagF32)
    }
#undef TSA_RNB
    return Fail(TSA_UNSUPPORTED, "tsa_rope_norm_bwd: src / grad dtypes must be (f32, f32), (bf16, bf16), (f16, f16), (f32, bf16) or (bf16, f32)");
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
