// The consumer of the attention output: the combiner input kv = shuffled(k) * valLookup (4 blocks per head) and its
// back-propagation, which also yields dScale for the attention backward.
// Replaces KVProduct and KVProductBackprop of the reference (code/gpt/compute/gpt_combiner.cuh:12-39, 85-217;
// CPU form code/gpt/compute/gpt_cpu.cpp:191-262):
//   kv[t][head * 4 D + blk * D + z] = k[t][head * D + (z ^ blk)] * val[t][head * D + z] * kvMult,  blk = 0 .. 3
//   dK[z]   = sum_blk dkv[blk][z ^ blk] * val[z ^ blk]
//   dVal[z] = sum_blk dkv[blk][z] * k[z ^ blk]
//   dScale[head][t] = sum_z dVal[z] * val[z]
// z ^ blk with blk < 4 stays inside an aligned group of 4 elements, so a thread that holds 8 consecutive elements of
// k and val (one 16-byte load each for 16-bit types) has every operand it needs: pure streaming, HBM-bound.
#include "tsa_common.cuh"
#include <type_traits>

namespace tsa {

constexpr int KV_REP = 4;

template <class T>
__device__ __forceinline__ void Load8(const typename T::T *p, float *dst)
{
    if (sizeof(typename T::T) == 4) {
        const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
        dst[0] = a.x, dst[1] = a.y, dst[2] = a.z, dst[3] = a.w, dst[4] = b.x, dst[5] = b.y, dst[6] = b.z, dst[7] = b.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 a;
            if (std::is_same<T, TagF16>::value) {
                a = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            } else {
                a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
            }
            dst[2 * i] = a.x, dst[2 * i + 1] = a.y;
        }
    }
}

template <class T>
__device__ __forceinline__ void Store8(typename T::T *p, const float *v)
{
    if (sizeof(typename T::T) == 4) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (std::is_same<T, TagF16>::value) {
                __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&h);
            } else {
                __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t *>(&h);
            }
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// one thread = 8 consecutive elements of one row; grid-stride over (row, group of 8)
template <class TIn, class TOut>
__global__ void __launch_bounds__(256) KvProductKernel(int len, int headCount, int headDim, float kvMult, P2D<typename TIn::T> k,
    P2D<typename TIn::T> val, P2D<typename TOut::T> kv)
{
    const int width = headCount * headDim;
    const int groups = width / 8;
    const long long total = (long long)len * groups;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / groups);
        const int e = (int)(idx - (long long)t * groups) * 8;
        const int head = e / headDim, z = e - head * headDim;
        float kk[8], vv[8];
        Load8<TIn>(k.Row(t) + e, kk);
        Load8<TIn>(val.Row(t) + e, vv);
        typename TOut::T *dst = kv.Row(t) + (size_t)head * headDim * KV_REP + z;
#pragma unroll
        for (int blk = 0; blk < KV_REP; ++blk) {
            float r[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                r[i] = __fmul_rn(__fmul_rn(kk[i ^ blk], vv[i]), kvMult);
            }
            Store8<TOut>(dst + blk * headDim, r);
        }
    }
}

// one thread = 8 consecutive elements of one (row, head); the headDim / 8 threads of a head are neighbours in a warp
template <class TIn, class TGrad>
__global__ void __launch_bounds__(256) KvProductBwdKernel(int len, int headCount, int headDim, P2D<typename TIn::T> k, P2D<typename TIn::T> val,
    P2D<typename TGrad::T> dkv, P2D<typename TGrad::T> dK, P2D<typename TGrad::T> dVal, P2D<float> dScale)
{
    const int width = headCount * headDim;
    const int groups = width / 8;
    const long long total = (long long)len * groups;
    const long long padded = (total + 31) / 32 * 32; // whole warps take part in the shuffles
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < padded; idx += (long long)gridDim.x * blockDim.x) {
        const bool live = idx < total;
        const long long id = live ? idx : total - 1;
        const int t = (int)(id / groups);
        const int e = (int)(id - (long long)t * groups) * 8;
        const int head = e / headDim, z = e - head * headDim;
        float kk[8], vv[8], dk[8], dv[8];
        Load8<TIn>(k.Row(t) + e, kk);
        Load8<TIn>(val.Row(t) + e, vv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            dk[i] = 0;
            dv[i] = 0;
        }
        const typename TGrad::T *src = dkv.Row(t) + (size_t)head * headDim * KV_REP + z;
#pragma unroll
        for (int blk = 0; blk < KV_REP; ++blk) {
            float g[8];
            Load8<TGrad>(src + blk * headDim, g);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                dk[i] = __fadd_rn(dk[i], __fmul_rn(g[i ^ blk], vv[i ^ blk]));
                dv[i] = __fadd_rn(dv[i], __fmul_rn(g[i], kk[i ^ blk]));
            }
        }
        float ds = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ds += dv[i] * vv[i];
        }
        // the head's headDim / 8 threads (8, 16 or 32 lanes of a warp; groups is a multiple of that, so heads do not
        // straddle warps) add up their parts
        for (int o = 1; o < headDim / 8; o <<= 1) {
            ds += __shfl_xor_sync(0xffffffffu, ds, o);
        }
        if (live) {
            Store8<TGrad>(dK.Row(t) + e, dk);
            Store8<TGrad>(dVal.Row(t) + e, dv);
            if (z == 0 && dScale.Valid()) {
                dScale.Row(head)[t] = ds;
            }
        }
    }
}

static int CombinerGrid(long long threads)
{
    long long blocks = (threads + 255) / 256;
    const long long cap = 148 * 32;
    return (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

static bool Aligned16(tsa_ptr2d a)
{
    return a.data && (uintptr_t)a.data % 16 == 0 && a.stride_bytes % 16 == 0;
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) int tsa_kv_product(int inDtype, int outDtype, tsa_ptr2d k, tsa_ptr2d valLookup, float kvMult,
    tsa_ptr2d kv, int headCount, int headDim, int len, tsa_stream_t stream)
{
    TSA_REQUIRE(headCount > 0 && (headDim == 64 || headDim == 128 || headDim == 256), "tsa_kv_product: head size %d must be 64, 128 or 256", headDim);
    const int width = headCount * headDim;
    TSA_REQUIRE(Aligned16(k) && Aligned16(valLookup) && Aligned16(kv), "tsa_kv_product: buffers must be present and 16-byte aligned");
    TSA_REQUIRE(k.xsize >= width && valLookup.xsize >= width && kv.xsize >= width * KV_REP, "tsa_kv_product: rows narrower than H*D (kv: 4*H*D)");
    TSA_REQUIRE(len >= 0 && len <= k.ysize && len <= valLookup.ysize && len <= kv.ysize, "tsa_kv_product: len %d exceeds buffers", len);
    if (len == 0) {
        return TSA_OK;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = CombinerGrid((long long)len * (width / 8));
#define TSA_KVP(TI, TO) KvProductKernel<TI, TO><<<grid, 256, 0, s>>>(len, headCount, headDim, kvMult, P2D<typename TI::T>(k), P2D<typename TI::T>(valLookup), P2D<typename TO::T>(kv))
    if (inDtype == TSA_F32 && outDtype == TSA_F32) {
        TSA_KVP(TagF32, TagF32);
    } else if (inDtype == TSA_BF16 && outDtype == TSA_BF16) {
        TSA_KVP(TagBF16, TagBF16);
    } else if (inDtype == TSA_F16 && outDtype == TSA_F16) {
        TSA_KVP(TagF16, TagF16);
    } else if (inDtype == TSA_BF16 && outDtype == TSA_F32) {
        TSA_KVP(TagBF16, TagF32);
    } else if (inDtype == TSA_F16 && outDtype == TSA_F32) {
        TSA_KVP(TagF16, TagF32);
    } else {
        return Fail(TSA_UNSUPPORTED, "tsa_kv_product: (in, out) dtypes must be (f32, f32), (bf16, bf16), (f16, f16), (bf16, f32) or (f16, f32)");
    }
#undef TSA_KVP
    return CheckCuda(cudaGetLastError(), "tsa_kv_product launch");
}

extern "C" __attribute__((visibility("default"))) int tsa_kv_product_bwd(int inDtype, int gradDtype, tsa_ptr2d k, tsa_ptr2d valLookup, tsa_ptr2d dkv,
    tsa_ptr2d dK, tsa_ptr2d dValLookup, tsa_ptr2d dScale, int headCount, int headDim, int len, tsa_stream_t stream)
{
    TSA_REQUIRE(headCount > 0 && (headDim == 64 || headDim == 128 || headDim == 256), "tsa_kv_product_bwd: head size %d must be 64, 128 or 256", headDim);
    const int width = headCount * headDim;
    TSA_REQUIRE(Aligned16(k) && Aligned16(valLookup) && Aligned16(dkv) && Aligned16(dK) && Aligned16(dValLookup),
        "tsa_kv_product_bwd: buffers must be present and 16-byte aligned");
    TSA_REQUIRE(k.xsize >= width && valLookup.xsize >= width && dK.xsize >= width && dValLookup.xsize >= width && dkv.xsize >= width * KV_REP,
        "tsa_kv_product_bwd: rows narrower than H*D (dkv: 4*H*D)");
    TSA_REQUIRE(len >= 0 && len <= k.ysize && len <= valLookup.ysize && len <= dkv.ysize && len <= dK.ysize && len <= dValLookup.ysize,
        "tsa_kv_product_bwd: len %d exceeds buffers", len);
    if (dScale.data) {
        TSA_REQUIRE(dScale.ysize >= headCount && dScale.xsize >= len, "tsa_kv_product_bwd: dScale plane too small");
    }
    if (len == 0) {
        return TSA_OK;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = CombinerGrid((long long)len * (width / 8));
#define TSA_KVB(TI, TG) KvProductBwdKernel<TI, TG><<<grid, 256, 0, s>>>(len, headCount, headDim, P2D<typename TI::T>(k), P2D<typename TI::T>(valLookup), \
    P2D<typename TG::T>(dkv), P2D<typename TG::T>(dK), P2D<typename TG::T>(dValLookup), P2D<float>(dScale))
    if (inDtype == TSA_F32 && gradDtype == TSA_F32) {
        TSA_KVB(TagF32, TagF32);
    } else if (inDtype == TSA_BF16 && gradDtype == TSA_BF16) {
        TSA_KVB(TagBF16, TagBF16);
    } else if (inDtype == TSA_F16 && gradDtype == TSA_F16) {
        TSA_KVB(TagF16, TagF16);
    } else if (inDtype == TSA_BF16 && gradDtype == TSA_F32) {
        TSA_KVB(TagBF16, TagF32);
    } else {
        return Fail(TSA_UNSUPPORTED, "tsa_kv_product_bwd: (in, grad) dtypes must be (f32, f32), (bf16, bf16), (f16, f16) or (bf16, f32)");
    }
#undef TSA_KVB
    return CheckCuda(cudaGetLastError(), "tsa_kv_product_bwd launch");
}
