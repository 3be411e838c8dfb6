// C-ABI entry points of the attention path: argument validation and dispatch to the kernels.
// Nothing here falls back to the CPU; a configuration no kernel covers returns TSA_UNSUPPORTED.
#include "att_internal.cuh"
#include <cstdarg>
#include <cstdio>
#include <cstring>

namespace tsa {

static thread_local char g_err[512] = "";

int Fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int CheckCuda(cudaError_t err, const char *what)
{
    if (err == cudaSuccess) {
        return TSA_OK;
    }
    return Fail(TSA_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(err));
}

int LaunchScoresI8(tsa_ptr2d qk, tsa_ptr2d qv, int headCount, int headDim, int lenQ, int lenK, int32_t *scores, int *statusWord, cudaStream_t stream);

static bool Is8Bit(int dt)
{
    return dt == TSA_I8 || dt == TSA_E4M3;
}
static bool IsFloatType(int dt)
{
    return dt == TSA_F16 || dt == TSA_BF16 || dt == TSA_F32;
}

// checks shared by forward and backward; fills the parameter block
static int FillCommon(const char *fn, const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale, tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope, int headCount, int lenAttTiles, TGenParams *pp)
{
    TSA_REQUIRE(cfg != nullptr, "%s: null cfg", fn);
    TSA_REQUIRE(Is8Bit(cfg->qk_dtype) && Is8Bit(cfg->v_dtype), "%s: qk/v dtype must be i8 or e4m3", fn);
    TSA_REQUIRE(cfg->head_dim_qk > 0 && cfg->head_dim_qk <= GEN_MAX_DIM && cfg->head_dim_qk % 4 == 0, "%s: head_dim_qk %d must be a multiple of 4, at most %d", fn, cfg->head_dim_qk, GEN_MAX_DIM);
    TSA_REQUIRE(cfg->head_dim_v > 0 && cfg->head_dim_v <= GEN_MAX_DIM && cfg->head_dim_v % 4 == 0, "%s: head_dim_v %d must be a multiple of 4, at most %d", fn, cfg->head_dim_v, GEN_MAX_DIM);
    TSA_REQUIRE(headCount > 0 && lenAttTiles >= 0, "%s: headCount %d / lenAttTiles %d", fn, headCount, lenAttTiles);
    TSA_REQUIRE(qk.data && qv.data && v.data && qvScale.data, "%s: null qk/qv/v/qvScale", fn);
    TSA_REQUIRE(lenAttTiles == 0 || (attSpans && attSpanPtr), "%s: null span arrays", fn);
    TSA_REQUIRE(qk.xsize >= headCount * cfg->head_dim_qk && qv.xsize >= headCount * cfg->head_dim_qk, "%s: qk/qv rows narrower than H*Dqk", fn);
    TSA_REQUIRE(v.xsize >= headCount * cfg->head_dim_v, "%s: v rows narrower than H*Dv", fn);
    TSA_REQUIRE(qv.ysize == v.ysize, "%s: qv and v row counts differ (%d, %d)", fn, qv.ysize, v.ysize);
    TSA_REQUIRE(qvScale.ysize >= headCount && qvScale.xsize >= qv.ysize, "%s: qvScale plane smaller than [H][rows]", fn);
    TSA_REQUIRE((uintptr_t)qk.data % 4 == 0 && qk.stride_bytes % 4 == 0 && (uintptr_t)qv.data % 4 == 0 && qv.stride_bytes % 4 == 0 &&
        (uintptr_t)v.data % 4 == 0 && v.stride_bytes % 4 == 0, "%s: 8-bit buffers must be 4-byte aligned", fn);
    if (qkScale.data) {
        TSA_REQUIRE(qkScale.ysize >= headCount && qkScale.xsize >= qk.ysize, "%s: qkScale plane smaller than [H][rows]", fn);
    }
    if (vScale.data) {
        TSA_REQUIRE(vScale.ysize >= headCount && vScale.xsize >= v.ysize, "%s: vScale plane smaller than [H][rows]", fn);
    }
    TGenParams &p = *pp;
    memset(&p, 0, sizeof(p));
    p.Len = lenAttTiles * TSA_ATT_GROUP < qk.ysize ? lenAttTiles * TSA_ATT_GROUP : qk.ysize;
    p.KeyRows = qv.ysize;
    p.HeadCount = headCount;
    p.Dq = cfg->head_dim_qk;
    p.Dv = cfg->head_dim_v;
    p.QkDtype = cfg->qk_dtype;
    p.VDtype = cfg->v_dtype;
    p.OutDtype = cfg->out_dtype;
    p.GradDtype = cfg->grad_dtype;
    p.C = HostAttDotScale(cfg->head_dim_qk);
    p.GlobalScale = qvGlobalScale;
    p.QkVecScale = cfg->qk_vec_scale;
    p.VVecScale = cfg->v_vec_scale;
    p.Slope = alibiSlope;
    p.GradMult = 1;
    p.Q = P2D<uint8_t>(qk);
    p.K = P2D<uint8_t>(qv);
    p.V = P2D<uint8_t>(v);
    p.QScale = P2D<float>(qkScale);
    p.KScale = P2D<float>(qvScale);
    p.VScale = P2D<float>(vScale);
    p.Spans = attSpans;
    p.SpanPtr = attSpanPtr;
    return TSA_OK;
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) const char *tsa_version(void)
{
    return "tsa-b200 0.1 (sm_100a)";
}

#ifdef TSA_BOUNDS_CHECK
namespace tsa {
static int (*g_boundsReaders[64])(int);
static int g_boundsReaderCount = 0;
int RegisterBoundsReader(int (*reader)(int reset))
{
    if (g_boundsReaderCount < 64) {
        g_boundsReaders[g_boundsReaderCount++] = reader;
    }
    return g_boundsReaderCount;
}
__global__ void BoundsSelfTestKernel(P2D<float> plane, int row, float *sink)
{
    *sink = plane.Row(row)[0];
}
} // namespace tsa
#endif

// number of out-of-range row lookups the kernels of a bounds-check build have caught (and redirected) since the last
// reset; -1 in a production build, which carries no checks
extern "C" __attribute__((visibility("default"))) int tsa_bounds_check_hits(int reset)
{
#ifdef TSA_BOUNDS_CHECK
    if (cudaDeviceSynchronize() != cudaSuccess) {
        return -2;
    }
    int total = 0;
    for (int i = 0; i < tsa::g_boundsReaderCount; ++i) {
        total += tsa::g_boundsReaders[i](reset);
    }
    return total;
#else
    (void)reset;
    return -1;
#endif
}

// bounds-check build: looks up row `rows` of a one-row plane on purpose (device memory plane[0..0], sink) and returns the
// number of lookups caught (1 when the check works); the lookup is redirected to row 0, so no memory outside the plane
// is read.  -1 in a production build.
extern "C" __attribute__((visibility("default"))) int tsa_selftest_bounds_check(float *plane, float *sink)
{
#ifdef TSA_BOUNDS_CHECK
    tsa_bounds_check_hits(1);
    tsa_ptr2d a = {plane, 4, 1, 1};
    tsa::BoundsSelfTestKernel<<<1, 1>>>(tsa::P2D<float>(a), 1, sink);
    return tsa_bounds_check_hits(1);
#else
    (void)plane;
    (void)sink;
    return -1;
#endif
}

extern "C" __attribute__((visibility("default"))) const char *tsa_last_error(void)
{
    return g_err;
}

extern "C" __attribute__((visibility("default"))) size_t tsa_att_fwd_workspace_bytes(const tsa_att_cfg *cfg, int headCount, int len)
{
    return headCount > 0 ? Sm100FwdWorkspaceBytes(cfg, headCount, len > 0 ? len : 0) : 0;
}

static int AttFwdImpl(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, const tsa_ptr2d *copies, int copyCount, tsa_ptr2d sumWeightLog, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream,
    const tsa_ptr2d *combinerK = nullptr, float kvMult = 1.0f, const tsa_ptr2d *kv = nullptr)
{
    TGenParams p;
    int rc = FillCommon("tsa_att_fwd", cfg, qvGlobalScale, qk, qv, qkScale, qvScale, v, vScale, attSpans, attSpanPtr, alibiSlope, headCount, lenAttTiles, &p);
    if (rc != TSA_OK) {
        return rc;
    }
    TSA_REQUIRE(IsFloatType(cfg->out_dtype), "tsa_att_fwd: out dtype must be f16, bf16 or f32");
    TSA_REQUIRE(out.data && out.xsize >= headCount * cfg->head_dim_v, "tsa_att_fwd: out missing or narrower than H*Dv");
    TSA_REQUIRE((uintptr_t)out.data % 16 == 0 && out.stride_bytes % 16 == 0, "tsa_att_fwd: out must be 16-byte aligned");
    if (sumWeightLog.data) {
        TSA_REQUIRE(sumWeightLog.ysize >= headCount, "tsa_att_fwd: sumWeightLog needs H rows");
    }
    if (p.Len > out.ysize) {
        p.Len = out.ysize;
    }
    if (sumWeightLog.data && p.Len > sumWeightLog.xsize) {
        p.Len = sumWeightLog.xsize;
    }
    p.Out = P2D<char>(out);
    p.Lse = P2D<float>(sumWeightLog);
    if (p.Len == 0) {
        return TSA_OK;
    }
    cudaStream_t s = (cudaStream_t)stream;
    TSA_REQUIRE(copyCount >= 0 && copyCount <= TSA_MAX_OUT_COPIES && (copyCount == 0 || copies), "tsa_att_fwd_to: %d destinations", copyCount + 1);
    for (int k = 0; k < copyCount; ++k) {
        TSA_REQUIRE(copies[k].data && copies[k].xsize >= headCount * cfg->head_dim_v && copies[k].ysize >= p.Len &&
            (uintptr_t)copies[k].data % 16 == 0 && copies[k].stride_bytes % 16 == 0, "tsa_att_fwd_to: destination %d missing, too small or not 16-byte aligned", k + 1);
        p.OutCopy[k] = P2D<char>(copies[k]);
    }
    p.OutCopies = copyCount;
    if (kv) {
        const int D = cfg->head_dim_v;
        TSA_REQUIRE(combinerK != nullptr, "tsa_att_fwd_kv: null combiner key argument");
        if (!Sm100FwdSupports(cfg, qk, qv, v) || cfg->out_dtype != TSA_BF16 || cfg->v_dtype == TSA_I8) {
            return Fail(TSA_UNSUPPORTED, "tsa_att_fwd_kv needs the tensor-core forward (head size 64 or 128, aligned buffers), e4m3 values and a bf16 output");
        }
        TSA_REQUIRE(combinerK->data && combinerK->xsize >= headCount * D && combinerK->ysize >= p.Len &&
            (uintptr_t)combinerK->data % 16 == 0 && combinerK->stride_bytes % 16 == 0, "tsa_att_fwd_kv: combiner keys missing, too small or not 16-byte aligned");
        TSA_REQUIRE(kv->data && kv->xsize >= headCount * 4 * D && kv->ysize >= p.Len &&
            (uintptr_t)kv->data % 16 == 0 && kv->stride_bytes % 16 == 0, "tsa_att_fwd_kv: kv missing, too small or not 16-byte aligned");
        p.KvK = P2D<char>(*combinerK);
        p.KvOut = P2D<char>(*kv);
        p.KvMult = kvMult;
    }
    if (copyCount > 0 && !Sm100FwdSupports(cfg, qk, qv, v)) {
        return Fail(TSA_UNSUPPORTED, "tsa_att_fwd_to: more than one destination needs the tensor-core forward (head size 64 or 128, aligned buffers)");
    }
    if (Sm100FwdSupports(cfg, qk, qv, v)) {
        size_t need = Sm100FwdWorkspaceBytes(cfg, headCount, qv.ysize); // per-head V-scale maxima, the work-item counter, e4m3 planes of int8 values
        TSA_REQUIRE(workspace && workspaceBytes >= need, "tsa_att_fwd: workspace of %zu bytes needed, %zu given", need, workspaceBytes);
        TSA_REQUIRE((uintptr_t)workspace % 16 == 0, "tsa_att_fwd: workspace must be 16-byte aligned");
        return LaunchSm100Fwd(cfg, p, qk, qv, v, lenAttTiles, qv.ysize, workspace, statusWord, s);
    }
    return LaunchGenericFwd(p, s);
}

extern "C" __attribute__((visibility("default"))) int tsa_att_fwd(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, tsa_ptr2d sumWeightLog, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream)
{
    return AttFwdImpl(cfg, qvGlobalScale, qk, qv, qkScale, qvScale, v, vScale, attSpans, attSpanPtr, alibiSlope, out, nullptr, 0, sumWeightLog,
        headCount, lenAttTiles, workspace, workspaceBytes, statusWord, stream);
}

extern "C" __attribute__((visibility("default"))) int tsa_att_fwd_to(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    const tsa_ptr2d *outs, int outCount, tsa_ptr2d sumWeightLog, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream)
{
    TSA_REQUIRE(outs != nullptr && outCount >= 1 && outCount <= TSA_MAX_OUT_COPIES + 1, "tsa_att_fwd_to: between 1 and %d destinations", TSA_MAX_OUT_COPIES + 1);
    return AttFwdImpl(cfg, qvGlobalScale, qk, qv, qkScale, qvScale, v, vScale, attSpans, attSpanPtr, alibiSlope, outs[0], outs + 1, outCount - 1,
        sumWeightLog, headCount, lenAttTiles, workspace, workspaceBytes, statusWord, stream);
}

extern "C" __attribute__((visibility("default"))) int tsa_att_fwd_kv(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, tsa_ptr2d sumWeightLog, tsa_ptr2d combinerK, float kvMult, tsa_ptr2d kv, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream)
{
    return AttFwdImpl(cfg, qvGlobalScale, qk, qv, qkScale, qvScale, v, vScale, attSpans, attSpanPtr, alibiSlope, out, nullptr, 0, sumWeightLog,
        headCount, lenAttTiles, workspace, workspaceBytes, statusWord, stream, &combinerK, kvMult, &kv);
}

static TFwdDump g_hooks; // process-wide test hooks of the forward (score dump, failure-path self-test)

extern "C" __attribute__((visibility("default"))) int tsa_att_fwd_set_score_dump(int32_t *dst, int head, int queryTile, int keyTile)
{
    TSA_REQUIRE(dst == nullptr || (head >= 0 && queryTile >= 0 && keyTile >= 0), "tsa_att_fwd_set_score_dump: negative index");
    g_hooks.Dst = dst;
    g_hooks.Head = head;
    g_hooks.QTile = queryTile;
    g_hooks.Tile = keyTile;
    SetFwdScoreDump(g_hooks);
    return TSA_OK;
}

extern "C" __attribute__((visibility("default"))) int tsa_selftest_fwd_withhold_copy(long long waitCycles, int withholdTile)
{
    TSA_REQUIRE(waitCycles >= 0, "tsa_selftest_fwd_withhold_copy: negative bound");
    g_hooks.WaitCycles = waitCycles;
    g_hooks.WithholdTile = withholdTile;
    SetFwdScoreDump(g_hooks);
    return TSA_OK;
}

extern "C" __attribute__((visibility("default"))) int tsa_selftest_bounded_wait(long long limitCycles, int *statusWord, tsa_stream_t stream)
{
    TSA_REQUIRE(statusWord != nullptr && limitCycles > 0 && limitCycles <= (1ll << 31), "tsa_selftest_bounded_wait: status word and a bound of at most 2^31 cycles");
    return LaunchBoundedWaitSelfTest(limitCycles, statusWord, (cudaStream_t)stream);
}

extern "C" __attribute__((visibility("default"))) int tsa_status_from_word(int statusWord)
{
    if (statusWord == 0) {
        return TSA_OK;
    }
    if (statusWord & (kDevTimeoutTma | kDevTimeoutMma)) {
        return Fail(TSA_TIMEOUT, "a bounded device wait ran out (status word %#x)", statusWord);
    }
    return Fail(TSA_BAD_ARG, "the device rejected its inputs (status word %#x)", statusWord);
}

extern "C" __attribute__((visibility("default"))) size_t tsa_att_bwd_workspace_bytes(const tsa_att_cfg *cfg, int headCount, int len)
{
    (void)cfg;
    if (headCount <= 0 || len <= 0) {
        return 0;
    }
    size_t rowBytes = ((size_t)len * sizeof(float) + 255) / 256 * 256;
    size_t bytes = rowBytes * headCount; // dScale plane when the caller does not supply one
    if (cfg && Sm100BwdSupports(cfg, headCount)) {
        int rows = (len + TSA_ATT_GROUP - 1) / TSA_ATT_GROUP * TSA_ATT_GROUP;
        bytes += Sm100BwdWorkspaceBytes(headCount, cfg->head_dim_qk, rows); // bf16 copies of Q, K, V, dOut
    }
    return bytes;
}

extern "C" __attribute__((visibility("default"))) int tsa_att_bwd(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale,
    tsa_ptr2d v, tsa_ptr2d vScale,
    tsa_ptr2d dOut, tsa_ptr2d out, tsa_ptr2d dScale, tsa_ptr2d sumWeightLog,
    const tsa_span_group *attSpans, const int *attSpanPtr,
    const tsa_span_group *revAttSpans, const int *revAttSpanPtr,
    float alibiSlope, float attGradMult,
    tsa_ptr2d dQK, tsa_ptr2d dQV, tsa_ptr2d dV, int headCount, int lenAttTiles,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream)
{
    TGenParams p;
    int rc = FillCommon("tsa_att_bwd", cfg, qvGlobalScale, qk, qv, qkScale, qvScale, v, vScale, attSpans, attSpanPtr, alibiSlope, headCount, lenAttTiles, &p);
    if (rc != TSA_OK) {
        return rc;
    }
    TSA_REQUIRE(IsFloatType(cfg->grad_dtype), "tsa_att_bwd: grad dtype must be f16, bf16 or f32");
    TSA_REQUIRE(lenAttTiles == 0 || (revAttSpans && revAttSpanPtr), "tsa_att_bwd: null transposed span arrays");
    TSA_REQUIRE(dOut.data && sumWeightLog.data && dQK.data && dQV.data && dV.data, "tsa_att_bwd: null dOut/sumWeightLog/dQK/dQV/dV");
    TSA_REQUIRE(dOut.xsize >= headCount * cfg->head_dim_v && dV.xsize >= headCount * cfg->head_dim_v, "tsa_att_bwd: dOut/dV narrower than H*Dv");
    TSA_REQUIRE(dQK.xsize >= headCount * cfg->head_dim_qk && dQV.xsize >= headCount * cfg->head_dim_qk, "tsa_att_bwd: dQK/dQV narrower than H*Dqk");
    TSA_REQUIRE(qk.ysize == qv.ysize, "tsa_att_bwd: qk and qv row counts differ");
    int len = p.Len;
    TSA_REQUIRE(dOut.ysize >= len && dQK.ysize >= len && dQV.ysize >= len && dV.ysize >= len && sumWeightLog.xsize >= len && sumWeightLog.ysize >= headCount,
        "tsa_att_bwd: a buffer has fewer than %d rows", len);
    if (len == 0) {
        return TSA_OK;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool tensorPath = Sm100BwdSupports(cfg, headCount) && (uintptr_t)dQK.data % 16 == 0 && dQK.stride_bytes % 16 == 0 &&
        (uintptr_t)dQV.data % 16 == 0 && dQV.stride_bytes % 16 == 0 && (uintptr_t)dV.data % 16 == 0 && dV.stride_bytes % 16 == 0;
    const size_t dsRowBytes = ((size_t)len * sizeof(float) + 255) / 256 * 256;
    const size_t dsBytes = dsRowBytes * headCount;
    const size_t need = dsBytes + (tensorPath ? Sm100BwdWorkspaceBytes(headCount, cfg->head_dim_qk, len) : 0);
    if (tensorPath || !dScale.data) {
        TSA_REQUIRE(workspace && workspaceBytes >= need, "tsa_att_bwd: workspace of %zu bytes needed, %zu given", need, workspaceBytes);
        TSA_REQUIRE((uintptr_t)workspace % 256 == 0, "tsa_att_bwd: workspace must be 256-byte aligned");
    }
    tsa_ptr2d ds = dScale;
    if (!ds.data) {
        TSA_REQUIRE(out.data && IsFloatType(cfg->out_dtype) && out.ysize >= len && out.xsize >= headCount * cfg->head_dim_v,
            "tsa_att_bwd: without dScale the forward result `out` is required");
        ds.data = workspace;
        ds.stride_bytes = (int)dsRowBytes;
        ds.xsize = len;
        ds.ysize = headCount;
        rc = LaunchDScale(cfg->out_dtype, cfg->grad_dtype, out, dOut, ds, headCount, cfg->head_dim_v, len, s);
        if (rc != TSA_OK) {
            return rc;
        }
    } else {
        TSA_REQUIRE(ds.xsize >= len && ds.ysize >= headCount, "tsa_att_bwd: dScale plane smaller than [H][len]");
    }
    p.GradMult = attGradMult;
    p.Lse = P2D<float>(sumWeightLog);
    p.DOut = P2D<char>(dOut);
    p.DScale = P2D<float>(ds);
    p.DQ = P2D<char>(dQK);
    p.DK = P2D<char>(dQV);
    p.DV = P2D<char>(dV);
    p.RevSpans = revAttSpans;
    p.RevSpanPtr = revAttSpanPtr;
    if (tensorPath) {
        return LaunchSm100Bwd(cfg, p, qk, qv, v, dOut, lenAttTiles, (char *)workspace + dsBytes, statusWord, s);
    }
    return LaunchGenericBwd(p, s);
}

extern "C" __attribute__((visibility("default"))) int tsa_qk_scores_i32(tsa_ptr2d qk, tsa_ptr2d qv, int headCount, int headDim, int lenQ, int lenK,
    int32_t *scores, int *statusWord, tsa_stream_t stream)
{
    TSA_REQUIRE(qk.data && qv.data && scores, "tsa_qk_scores_i32: null buffer");
    TSA_REQUIRE(headDim == 64 || headDim == 128, "tsa_qk_scores_i32: head size must be 64 or 128");
    TSA_REQUIRE(headCount > 0 && lenQ > 0 && lenK > 0 && lenQ <= qk.ysize && lenK <= qv.ysize, "tsa_qk_scores_i32: extents");
    TSA_REQUIRE(qk.xsize >= headCount * headDim && qv.xsize >= headCount * headDim, "tsa_qk_scores_i32: rows narrower than H*D");
    TSA_REQUIRE((uintptr_t)qk.data % 16 == 0 && qk.stride_bytes % 16 == 0 && (uintptr_t)qv.data % 16 == 0 && qv.stride_bytes % 16 == 0,
        "tsa_qk_scores_i32: buffers must be 16-byte aligned");
    return LaunchScoresI8(qk, qv, headCount, headDim, lenQ, lenK, scores, statusWord, (cudaStream_t)stream);
}
