// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// C entry points around the reference's own fp32 CPU attention
// (NCPU_GPT::TAttentionComputer, code/gpt/compute/gpt_cpu.cpp:367-556) and its span
// preprocessing (GroupAttention / TransposeAttention, code/gpt/att/att.h:95-181,
// code/gpt/att/att.cpp:26-56).  TAttentionComputer is local to gpt_cpu.cpp, so this
// translation unit includes that source file where it lies in the reference checkout;
// nothing of the reference is copied into this repository.  The result is
// oracle/_ref/libtsa_ref.so, used only to validate the restated oracle and as the
// timed CPU baseline.
#include <gpt/compute/stdafx.h>
#include <gpt/compute/gpt_cpu.cpp>
#include <gpt/att/att.h>
#include <cstring>

using namespace NCPU_GPT;

namespace {

static void FillArr(TArray2D<float> *p, const float *src, int xSize, int ySize)
{
    p->SetSizes(xSize, ySize);
    for (int y = 0; y < ySize; ++y) {
        memcpy((*p)[y], src + (size_t)y * xSize, sizeof(float) * xSize);
    }
}

static void StoreArr(const TArray2D<float> &a, float *dst)
{
    for (yint y = 0; y < a.GetYSize(); ++y) {
        memcpy(dst + (size_t)y * a.GetXSize(), a[y], sizeof(float) * a.GetXSize());
    }
}

static void FillAtt(TAttentionInfo *p, int len, const int *spans, const int *spanPtr)
{
    p->Init();
    for (int t = 0; t < len; ++t) {
        for (int k = spanPtr[t]; k < spanPtr[t + 1]; ++k) {
            p->AddSpan(TAttentionSpan(spans[k * 2], spans[k * 2 + 1]));
        }
        p->AddSample();
    }
}

static TModelDims MakeDims(int headCount, int qDim, int ttDim)
{
    TModelDims dims;
    dims.QDim = qDim;
    dims.TTDim = ttDim;
    dims.HeadCount = headCount;
    dims.Dim = 256;
    return dims;
}

} // namespace


extern "C" {

// forward: q,k are [len][H*qDim], v is [len][H*ttDim], spans are (start,finish) pairs in CSR form.
// out [len][H*ttDim]; sumWeight and maxDP are [H][len].
void ref_att_fwd(int len, int headCount, int qDim, int ttDim, float alibiSlope,
    const float *q, const float *k, const float *v, const int *spans, const int *spanPtr,
    float *out, float *sumWeight, float *maxDP)
{
    TModelDims dims = MakeDims(headCount, qDim, ttDim);
    TArray2D<float> qa, ka, va, res;
    FillArr(&qa, q, headCount * qDim, len);
    FillArr(&ka, k, headCount * qDim, len);
    FillArr(&va, v, headCount * ttDim, len);
    TAttentionInfo att;
    FillAtt(&att, len, spans, spanPtr);
    TAttentionComputer comp(dims, alibiSlope);
    comp.ComputeValLookup(len, dims, qa, ka, va, att, &res);
    StoreArr(res, out);
    if (sumWeight) {
        StoreArr(comp.SumWeight, sumWeight);
    }
    if (maxDP) {
        StoreArr(comp.MaxDP, maxDP);
    }
}

// backward: dOut [len][H*ttDim], dScale [H][len] (= sum_x dOut*out per head, gpt_cpu.cpp:255-263).
// revSpans describe the transposed mask.  Outputs dq, dk [len][H*qDim], dv [len][H*ttDim].
void ref_att_bwd(int len, int headCount, int qDim, int ttDim, float alibiSlope,
    const float *q, const float *k, const float *v, const float *dOut, const float *dScale,
    const int *spans, const int *spanPtr, const int *revSpans, const int *revSpanPtr,
    float *dq, float *dk, float *dv)
{
    TModelDims dims = MakeDims(headCount, qDim, ttDim);
    TArray2D<float> qa, ka, va, doa, dsa, res;
    FillArr(&qa, q, headCount * qDim, len);
    FillArr(&ka, k, headCount * qDim, len);
    FillArr(&va, v, headCount * ttDim, len);
    FillArr(&doa, dOut, headCount * ttDim, len);
    FillArr(&dsa, dScale, len, headCount);
    TAttentionInfo att, revAtt;
    FillAtt(&att, len, spans, spanPtr);
    FillAtt(&revAtt, len, revSpans, revSpanPtr);
    TAttentionComputer comp(dims, alibiSlope);
    comp.ComputeValLookup(len, dims, qa, ka, va, att, &res); // fills SumWeight / MaxDP
    TAttentionComputer::TGradData data(dims, qa, ka, va, doa, dsa);
    TArray2D<float> dqa, dka, dva;
    comp.GradQK(len, dims, data, att, &dqa);
    comp.GradQV(len, dims, data, revAtt, &dka, &dva);
    StoreArr(dqa, dq);
    StoreArr(dka, dk);
    StoreArr(dva, dv);
}

// TransposeAttention; returns span count, fills up to maxSpans pairs
int ref_transpose_attention(int len, const int *spans, const int *spanPtr, int maxSpans, int *resSpans, int *resSpanPtr)
{
    TAttentionInfo att;
    FillAtt(&att, len, spans, spanPtr);
    TAttentionInfo rev = TransposeAttention(att);
    int n = (int)YSize(rev.Spans);
    if (n > maxSpans) {
        return -n;
    }
    for (int i = 0; i < n; ++i) {
        resSpans[i * 2] = rev.Spans[i].Start;
        resSpans[i * 2 + 1] = rev.Spans[i].Finish;
    }
    for (int t = 0; t <= len; ++t) {
        resSpanPtr[t] = rev.SpanPtr[t];
    }
    return n;
}

// GroupAttention<64,128>; group record = {Start, Finish, SpanStart[64], SpanFinish[64]} = 130 ints.
// returns group count (negative needed count if maxGroups is too small); groupPtr has ceil(len/64)+1 entries
int ref_group_attention_64_128(int len, const int *spans, const int *spanPtr, int maxGroups, int *groups, int *groupPtr)
{
    TAttentionInfo att;
    FillAtt(&att, len, spans, spanPtr);
    TAttentionInfoGrouped<64> gg;
    GroupAttention<64, 128>(att, &gg);
    int n = (int)YSize(gg.SpanGroups);
    if (n > maxGroups) {
        return -n;
    }
    static_assert(sizeof(TAttentionSpanGroup<64>) == 130 * sizeof(int), "span group layout");
    if (n > 0) {
        memcpy(groups, gg.SpanGroups.data(), sizeof(TAttentionSpanGroup<64>) * n);
    }
    for (yint i = 0; i < YSize(gg.SpanGroupPtr); ++i) {
        groupPtr[i] = gg.SpanGroupPtr[i];
    }
    return n;
}

// FillRopeBuf / ApplyRope (code/gpt/att/rope.cpp:4-61) and NormalizeState (gpt_cpu.cpp:297-324): the producer of the
// attention inputs on the CPU path (gpt_cpu.cpp:625-630: normalise per head, then rope on the query / key vectors)
void ref_fill_rope(int width, int maxLen, float *rope)
{
    TArray2D<float> buf;
    FillRopeBuf(&buf, width, maxLen);
    StoreArr(buf, rope);
}

// data [len][dim] in place; rope [len][width]
void ref_apply_rope(int width, int len, int dim, float dir, const float *rope, float *data)
{
    TArray2D<float> buf, arr;
    FillArr(&buf, rope, width, len);
    FillArr(&arr, data, dim, len);
    ApplyRope(buf, dir, &arr);
    StoreArr(arr, data);
}

void ref_normalize_state_f32(int len, int dim, int headCount, const float *src, float *dst)
{
    TArray2D<float> arr;
    FillArr(&arr, src, dim, len);
    TArray2D<float> res = NormalizeState(arr, headCount);
    StoreArr(res, dst);
}

void ref_normalize_state_backward_f32(int len, int dim, int headCount, const float *src, const float *dNorm, float *grad)
{
    TArray2D<float> arr, dn, res;
    FillArr(&arr, src, dim, len);
    FillArr(&dn, dNorm, dim, len);
    NormalizeStateBackward(arr, headCount, dn, &res);
    StoreArr(res, grad);
}

// KVProduct / KVProductBackprop (gpt_cpu.cpp:191-262): the consumer of the attention output on the CPU path
static TModelDims CombinerDims(int headCount, int ttDim)
{
    TModelDims dims;
    dims.TTDim = ttDim;
    dims.HeadCount = headCount;
    return dims;
}

void ref_kv_product(int len, int headCount, int ttDim, const float *k, const float *valLookup, float *kv)
{
    TArray2D<float> ka, va, res;
    FillArr(&ka, k, headCount * ttDim, len);
    FillArr(&va, valLookup, headCount * ttDim, len);
    KVProduct(CombinerDims(headCount, ttDim), ka, va, &res);
    StoreArr(res, kv);
}

// dScale [headCount][len]
void ref_kv_product_backprop(int len, int headCount, int ttDim, const float *k, const float *valLookup, const float *dkv,
    float *dK, float *dValLookup, float *dScale)
{
    TArray2D<float> ka, va, da, dk, dv, ds;
    FillArr(&ka, k, headCount * ttDim, len);
    FillArr(&va, valLookup, headCount * ttDim, len);
    FillArr(&da, dkv, headCount * ttDim * COMBINER_REP, len);
    KVProductBackprop(CombinerDims(headCount, ttDim), ka, va, da, &dk, &dv, &ds);
    StoreArr(dk, dK);
    StoreArr(dv, dValLookup);
    StoreArr(ds, dScale);
}

int ref_float2i8(float x)
{
    return Float2I8(x);
}

}
