// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's int8 KV-cache CPU inference attention
// (NCPUInfer::TAttentionVecHistory / ComputeValLookup / NormalizeState,
// code/gpt/train/cpu_infer.cpp:357-460).  The history struct is local to that source
// file, so this translation unit includes it where it lies in the reference checkout.
#include <gpt/train/stdafx.h>
#include <gpt/train/cpu_infer.cpp>
#include <cstring>
#include <cstdlib>
#include <new>

// DotInt8 (cpu_infer.cpp:199-210) dereferences __m256i pointers, i.e. issues aligned 32-byte loads
// on vector storage; the reference gets that alignment from its own allocator (hu_alloc), which is
// not linked here.  Give every allocation made inside this library 64-byte alignment instead
// (all symbols of the library are local, so this does not leak into the host process).
void *operator new(size_t sz)
{
    void *p = aligned_alloc(64, (sz + 63) / 64 * 64);
    if (!p) {
        throw std::bad_alloc();
    }
    return p;
}
void *operator new[](size_t sz) { return operator new(sz); }
void operator delete(void *p) noexcept { free(p); }
void operator delete[](void *p) noexcept { free(p); }
void operator delete(void *p, size_t) noexcept { free(p); }
void operator delete[](void *p, size_t) noexcept { free(p); }

extern "C" {

// One decode step for one sequence.  The cache holds ctxLen tokens INCLUDING the one just
// appended (the reference appends before it attends, cpu_infer.cpp:506-509).
//   kCache, vCache : int8 [ctxLen][H*D]; kScale : f32 [ctxLen][H]; q : int8 [H*D]
// Logit = int32dot * kScale * attDotScale * VEC_SCALE - slope * (cur - to), VEC_SCALE = 1/24;
// result = sum softmax * VEC_SCALE * v   (f32 [H*D]).
void ref_decode_step(int ctxLen, int headCount, int headDim, int width, float alibiSlope,
    const signed char *kCache, const float *kScale, const signed char *vCache, const signed char *q,
    float *out)
{
    using namespace NCPUInfer;
    TModelDims dims;
    dims.QDim = headDim;
    dims.TTDim = headDim;
    dims.HeadCount = headCount;
    int rowSize = headCount * headDim;
    TAttentionVecHistory hist;
    hist.QVState.resize(ctxLen);
    hist.QVStateScaleArr.resize(ctxLen);
    hist.VState.resize(ctxLen);
    for (int t = 0; t < ctxLen; ++t) {
        hist.QVState[t].resize(rowSize);
        hist.VState[t].resize(rowSize);
        hist.QVStateScaleArr[t].resize(headCount);
        memcpy(hist.QVState[t].data(), kCache + (size_t)t * rowSize, rowSize);
        memcpy(hist.VState[t].data(), vCache + (size_t)t * rowSize, rowSize);
        memcpy(hist.QVStateScaleArr[t].data(), kScale + (size_t)t * headCount, sizeof(float) * headCount);
    }
    TVector<i8> qk;
    qk.resize(rowSize);
    memcpy(qk.data(), q, rowSize);
    TVector<float> res;
    ComputeValLookup(width, alibiSlope, dims, hist, qk, &res);
    memcpy(out, res.data(), sizeof(float) * rowSize);
}

// NormalizeState (cpu_infer.cpp:357-391): per-head RMS normalise to int8 with clamp +-127;
// headScale (may be null) receives sqrt(sum2/headDim) * VEC_SCALE
void ref_normalize_state(int dim, int headCount, const float *state, signed char *res, float *headScale)
{
    using namespace NCPUInfer;
    TVector<float> src;
    src.resize(dim);
    memcpy(src.data(), state, sizeof(float) * dim);
    TVector<i8> dst;
    TVector<float> scale;
    NormalizeState(&dst, src, headCount, headScale ? &scale : nullptr);
    memcpy(res, dst.data(), dim);
    if (headScale) {
        memcpy(headScale, scale.data(), sizeof(float) * headCount);
    }
}

float ref_vec_scale()
{
    return VEC_SCALE;
}

// ConvertE4toFloat (code/util/fp8.h:4-21)
float ref_e4m3_to_float(int x)
{
    return ConvertE4toFloat((i8)x);
}

}
