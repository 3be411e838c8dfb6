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

// ---- the whole one-token inference step (NCPUInfer::ComputePrediction, cpu_infer.cpp:530-560) ------------------
// The model is handed over already in the reference's int8 form (TCPUModelParams, cpu_infer.cpp:59-84):
//   layerMats  : 7 matrices per layer, row-major int8: QK, QV [H*D][dim], K, V [H*D][dim], Combiner [dim][4*H*D],
//                Expand [reluDim][dim], Contract [dim][reluDim]
//   layerScalars : 5 floats per layer: QVScale, CombinerScale, ContractScale, attention width, ALiBi slope
// ropeLen is the number of positions the context can take (the reference sizes its rope table by the widest window).
struct TRefInfer
{
    NCPUInfer::TCPUModelParams Params;
    NCPUInfer::TCPUInferContext Ctx;
};

static void FillMatrix(TArray2D<i8> *p, const signed char *src, yint xSize, yint ySize)
{
    p->SetSizes(xSize, ySize);
    for (yint y = 0; y < ySize; ++y) {
        memcpy(&(*p)[y][0], src + y * xSize, xSize);
    }
}

void *ref_infer_create(int dim, int headDim, int headCount, int reluMult, int vocab, int labelCount, int layerCount, int ropeLen,
    const signed char *const *layerMats, const float *layerScalars, const signed char *labelEmbed, float labelEmbedScale,
    const signed char *finalLayer, float finalLayerScale, const float *bias)
{
    using namespace NCPUInfer;
    TRefInfer *h = new TRefInfer;
    TCPUModelParams &p = h->Params;
    p.ModelDescr.Dims.Dim = dim;
    p.ModelDescr.Dims.QDim = headDim;
    p.ModelDescr.Dims.TTDim = headDim;
    p.ModelDescr.Dims.HeadCount = headCount;
    p.ModelDescr.Dims.ReluMult = reluMult;
    p.ModelDescr.VocabSize = vocab;
    p.ModelDescr.LabelCount = labelCount;
    p.ModelDescr.AttentionWidthArr.push_back(ropeLen);
    yint hs = (yint)headDim * headCount;
    yint reluDim = p.ModelDescr.Dims.GetReluDim();
    p.LayerArr.resize(layerCount);
    for (int d = 0; d < layerCount; ++d) {
        TCPUModelParams::TAttentionMatrices &att = p.LayerArr[d];
        const signed char *const *m = layerMats + d * 7;
        FillMatrix(&att.QK, m[0], dim, hs);
        FillMatrix(&att.QV, m[1], dim, hs);
        FillMatrix(&att.K, m[2], dim, hs);
        FillMatrix(&att.V, m[3], dim, hs);
        FillMatrix(&att.Combiner, m[4], hs * COMBINER_REP, dim);
        FillMatrix(&att.Expand, m[5], dim, reluDim);
        FillMatrix(&att.Contract, m[6], reluDim, dim);
        const float *s = layerScalars + d * 5;
        att.QVScale = s[0];
        att.CombinerScale = s[1];
        att.ContractScale = s[2];
        att.AttentionWidth = (int)s[3];
        att.AlibiSlope = s[4];
        p.ModelDescr.Layers.push_back(TModelDescr::TAttentionPosParams(s[4], 0));
    }
    FillMatrix(&p.LabelEmbed, labelEmbed, dim, labelCount);
    p.LabelEmbedScale = labelEmbedScale;
    FillMatrix(&p.FinalLayer, finalLayer, dim, vocab);
    p.FinalLayerScale = finalLayerScale;
    p.Bias.resize(vocab);
    memcpy(p.Bias.data(), bias, sizeof(float) * vocab);
    h->Ctx.Init(p);
    return h;
}

// one step: the labels of the new token in, the distribution over the vocabulary out (prediction may be null)
void ref_infer_step(void *handle, const int *labels, int labelCount, float *prediction)
{
    using namespace NCPUInfer;
    TRefInfer *h = (TRefInfer *)handle;
    TVector<TLabelIndex> labelArr;
    for (int i = 0; i < labelCount; ++i) {
        labelArr.push_back(labels[i]);
    }
    TVector<float> distr;
    ComputePrediction(h->Params, labelArr, &h->Ctx, prediction ? &distr : nullptr);
    if (prediction) {
        memcpy(prediction, distr.data(), sizeof(float) * YSize(distr));
    }
}

void ref_infer_free(void *handle)
{
    delete (TRefInfer *)handle;
}

}
