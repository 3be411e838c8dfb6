// Forward attention on vectors that live in page-locked HOST memory: the heads are cut into slices and the copy-in of
// slice s+1, the attention kernel of slice s and the copy-out of slice s-1 run at the same time on three streams.
// The reference keeps every array in TCuda2DArray objects that own a host and a device copy and moves them whole with
// CopyToDevice / CopyToHost on the compute stream (code/lib/cuda/cuda_arrays.h:353-369), i.e. copy, compute, copy in
// sequence; this entry is what a host-resident caller (a test harness, a CPU-side producer of the quantised vectors)
// calls instead of doing those three steps itself.
#include "att_internal.cuh"
#include <mutex>

namespace tsa {

namespace {

constexpr int HOST_PIPE_DEPTH = 2;   // staging sets: slice s lives in set s % 2
constexpr int HOST_PIPE_MAX_DEVICES = 64;

struct THostPipe {
    bool Ready = false;
    cudaStream_t In = nullptr, Compute = nullptr, Out = nullptr;
    cudaEvent_t Start = nullptr;
    cudaEvent_t InDone[HOST_PIPE_DEPTH] = {}, KernelDone[HOST_PIPE_DEPTH] = {}, OutDone[HOST_PIPE_DEPTH] = {};
};

std::mutex g_pipeLock;
THostPipe g_pipes[HOST_PIPE_MAX_DEVICES];

size_t RoundUp256(size_t x)
{
    return (x + 255) & ~(size_t)255;
}

int ElemBytes(int dt)
{
    return dt == TSA_F32 ? 4 : ((dt == TSA_F16 || dt == TSA_BF16) ? 2 : 1);
}

// layout of one staging set for slices of at most hs heads
struct TStageLayout {
    size_t Qk, Qv, V, QkScale, QvScale, VScale, Out, Lse, Work, Total;
    int PitchQk, PitchV, PitchOut, PitchScale;
    size_t WorkBytes;
};

TStageLayout MakeLayout(const tsa_att_cfg *cfg, int hs, int len)
{
    TStageLayout l;
    l.PitchQk = (int)RoundUp256((size_t)hs * cfg->head_dim_qk);
    l.PitchV = (int)RoundUp256((size_t)hs * cfg->head_dim_v);
    l.PitchOut = (int)RoundUp256((size_t)hs * cfg->head_dim_v * ElemBytes(cfg->out_dtype));
    l.PitchScale = (int)RoundUp256((size_t)len * 4);
    l.WorkBytes = Sm100FwdWorkspaceBytes(cfg, hs, len);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t at = off;
        off += RoundUp256(bytes);
        return at;
    };
    l.Qk = take((size_t)len * l.PitchQk);
    l.Qv = take((size_t)len * l.PitchQk);
    l.V = take((size_t)len * l.PitchV);
    l.QkScale = take((size_t)hs * l.PitchScale);
    l.QvScale = take((size_t)hs * l.PitchScale);
    l.VScale = take((size_t)hs * l.PitchScale);
    l.Out = take((size_t)len * l.PitchOut);
    l.Lse = take((size_t)hs * l.PitchScale);
    l.Work = take(l.WorkBytes);
    l.Total = off;
    return l;
}

int GetPipe(THostPipe **res)
{
    int dev = 0;
    int rc = CheckCuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc != TSA_OK) {
        return rc;
    }
    TSA_REQUIRE(dev >= 0 && dev < HOST_PIPE_MAX_DEVICES, "tsa_att_fwd_host: device index %d", dev);
    THostPipe &p = g_pipes[dev];
    if (!p.Ready) {
#define TSA_PIPE_TRY(x) do { int rc_ = CheckCuda((x), #x); if (rc_ != TSA_OK) return rc_; } while (0)
        TSA_PIPE_TRY(cudaStreamCreateWithFlags(&p.In, cudaStreamNonBlocking));
        TSA_PIPE_TRY(cudaStreamCreateWithFlags(&p.Compute, cudaStreamNonBlocking));
        TSA_PIPE_TRY(cudaStreamCreateWithFlags(&p.Out, cudaStreamNonBlocking));
        TSA_PIPE_TRY(cudaEventCreateWithFlags(&p.Start, cudaEventDisableTiming));
        for (int b = 0; b < HOST_PIPE_DEPTH; ++b) {
            TSA_PIPE_TRY(cudaEventCreateWithFlags(&p.InDone[b], cudaEventDisableTiming));
            TSA_PIPE_TRY(cudaEventCreateWithFlags(&p.KernelDone[b], cudaEventDisableTiming));
            TSA_PIPE_TRY(cudaEventCreateWithFlags(&p.OutDone[b], cudaEventDisableTiming));
        }
#undef TSA_PIPE_TRY
        p.Ready = true;
    }
    *res = &p;
    return TSA_OK;
}

} // namespace

} // namespace tsa

namespace tsa {

// One rank's part of an all-gather over peer memory: the rows of src go to every destination (the same block inside the
// other GPUs' buffers).  No shared memory and few registers, so its CTAs fit beside the attention CTAs of the next head
// slice and the copy runs under that kernel (a library collective's kernels waited for the attention CTAs to leave).
// A thread moves 32 bytes at a time: one load, one store per destination.
struct TPeerDsts {
    char *Data[TSA_MAX_OUT_COPIES];
    long long Stride[TSA_MAX_OUT_COPIES];
    int Count;
};

__global__ void __launch_bounds__(256) PeerScatterKernel(const char *src, long long srcStride, TPeerDsts dsts, int rows, int rowBytes)
{
    const int chunksPerRow = rowBytes >> 5;
    const long long total = (long long)rows * chunksPerRow;
    for (long long id = blockIdx.x * (long long)blockDim.x + threadIdx.x; id < total; id += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(id / chunksPerRow), c = (int)(id - (long long)r * chunksPerRow);
        uint32_t v[8];
        asm volatile("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                     : "l"(src + r * srcStride + c * 32));
        for (int k = 0; k < dsts.Count; ++k) {
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dsts.Data[k] + r * dsts.Stride[k] + c * 32), "r"(v[0]), "r"(v[1]),
                         "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                         : "memory");
        }
    }
}

} // namespace tsa

using namespace tsa;

extern "C" __attribute__((visibility("default"))) size_t tsa_att_fwd_host_staging_bytes(const tsa_att_cfg *cfg, int headCount, int len, int slices)
{
    if (!cfg || headCount <= 0 || len <= 0 || slices <= 0) {
        return 0;
    }
    const int hs = (headCount + slices - 1) / slices;
    return MakeLayout(cfg, hs, len).Total * HOST_PIPE_DEPTH;
}

extern "C" __attribute__((visibility("default"))) int tsa_att_fwd_host(const tsa_att_cfg *cfg, const float *qvGlobalScale,
    tsa_ptr2d qk, tsa_ptr2d qv, tsa_ptr2d qkScale, tsa_ptr2d qvScale, tsa_ptr2d v, tsa_ptr2d vScale,
    const tsa_span_group *attSpans, const int *attSpanPtr, float alibiSlope,
    tsa_ptr2d out, tsa_ptr2d sumWeightLog, tsa_ptr2d outDevice, int headCount, int lenAttTiles, int slices,
    void *staging, size_t stagingBytes, int *statusWord, tsa_stream_t stream)
{
    TSA_REQUIRE(cfg != nullptr, "tsa_att_fwd_host: null cfg");
    TSA_REQUIRE(headCount > 0 && slices > 0 && slices <= headCount, "tsa_att_fwd_host: %d slices of %d heads", slices, headCount);
    TSA_REQUIRE(qk.data && qv.data && v.data && qvScale.data && out.data, "tsa_att_fwd_host: null qk/qv/v/qvScale/out");
    const int dq = cfg->head_dim_qk, dv = cfg->head_dim_v, esz = ElemBytes(cfg->out_dtype);
    const int len = qv.ysize;
    TSA_REQUIRE(len > 0 && qk.ysize == len && v.ysize == len && out.ysize >= len, "tsa_att_fwd_host: qk, qv, v and out need the same %d rows", len);
    TSA_REQUIRE(qk.xsize >= headCount * dq && qv.xsize >= headCount * dq && v.xsize >= headCount * dv && out.xsize >= headCount * dv,
        "tsa_att_fwd_host: rows narrower than H*D");
    TSA_REQUIRE(qvScale.ysize >= headCount && qvScale.xsize >= len, "tsa_att_fwd_host: qvScale plane smaller than [H][rows]");
    TSA_REQUIRE(!qkScale.data || (qkScale.ysize >= headCount && qkScale.xsize >= len), "tsa_att_fwd_host: qkScale plane smaller than [H][rows]");
    TSA_REQUIRE(!vScale.data || (vScale.ysize >= headCount && vScale.xsize >= len), "tsa_att_fwd_host: vScale plane smaller than [H][rows]");
    TSA_REQUIRE(!outDevice.data || (outDevice.ysize >= len && outDevice.xsize >= headCount * dv && (uintptr_t)outDevice.data % 16 == 0 &&
        outDevice.stride_bytes % 16 == 0 && ((size_t)dv * esz) % 16 == 0), "tsa_att_fwd_host: outDevice smaller than [rows][H*Dv] or not 16-byte aligned");
    TSA_REQUIRE(!sumWeightLog.data || (sumWeightLog.ysize >= headCount && sumWeightLog.xsize >= len), "tsa_att_fwd_host: sumWeightLog plane smaller than [H][rows]");
    const int hs = (headCount + slices - 1) / slices;
    const TStageLayout lay = MakeLayout(cfg, hs, len);
    TSA_REQUIRE(staging && stagingBytes >= lay.Total * HOST_PIPE_DEPTH, "tsa_att_fwd_host: staging of %zu bytes needed, %zu given",
        lay.Total * HOST_PIPE_DEPTH, stagingBytes);
    TSA_REQUIRE((uintptr_t)staging % 256 == 0, "tsa_att_fwd_host: staging must be 256-byte aligned");

    std::lock_guard<std::mutex> guard(g_pipeLock);
    THostPipe *pp = nullptr;
    int rc = GetPipe(&pp);
    if (rc != TSA_OK) {
        return rc;
    }
    THostPipe &pipe = *pp;
    cudaStream_t user = (cudaStream_t)stream;
#define TSA_TRY(x) do { int rc_ = CheckCuda((x), #x); if (rc_ != TSA_OK) return rc_; } while (0)
    // everything queued on the caller's stream so far (previous users of the staging area among it) comes first
    TSA_TRY(cudaEventRecord(pipe.Start, user));
    TSA_TRY(cudaStreamWaitEvent(pipe.In, pipe.Start, 0));
    TSA_TRY(cudaStreamWaitEvent(pipe.Compute, pipe.Start, 0));
    TSA_TRY(cudaStreamWaitEvent(pipe.Out, pipe.Start, 0));

    char *base = (char *)staging;
    int nDone = 0;
    for (int s = 0, h0 = 0; h0 < headCount; ++s, h0 += hs) {
        const int b = s % HOST_PIPE_DEPTH;
        const int hn = (headCount - h0 < hs) ? headCount - h0 : hs;
        char *set = base + (size_t)b * lay.Total;
        // ---- copy in: this slice's head columns of the three matrices, its rows of the scale planes
        if (s >= HOST_PIPE_DEPTH) {
            TSA_TRY(cudaStreamWaitEvent(pipe.In, pipe.KernelDone[b], 0)); // the kernel that read this set two slices ago
        }
        auto copyIn = [&](size_t dstOff, int dstPitch, const tsa_ptr2d &src, size_t srcColBytes, size_t widthBytes, int rows, size_t srcRow0) {
            return cudaMemcpy2DAsync(set + dstOff, dstPitch, (const char *)src.data + srcRow0 * src.stride_bytes + srcColBytes, src.stride_bytes,
                widthBytes, rows, cudaMemcpyHostToDevice, pipe.In);
        };
        TSA_TRY(copyIn(lay.Qk, lay.PitchQk, qk, (size_t)h0 * dq, (size_t)hn * dq, len, 0));
        TSA_TRY(copyIn(lay.Qv, lay.PitchQk, qv, (size_t)h0 * dq, (size_t)hn * dq, len, 0));
        TSA_TRY(copyIn(lay.V, lay.PitchV, v, (size_t)h0 * dv, (size_t)hn * dv, len, 0));
        TSA_TRY(copyIn(lay.QvScale, lay.PitchScale, qvScale, 0, (size_t)len * 4, hn, h0));
        if (qkScale.data) {
            TSA_TRY(copyIn(lay.QkScale, lay.PitchScale, qkScale, 0, (size_t)len * 4, hn, h0));
        }
        if (vScale.data) {
            TSA_TRY(copyIn(lay.VScale, lay.PitchScale, vScale, 0, (size_t)len * 4, hn, h0));
        }
        TSA_TRY(cudaEventRecord(pipe.InDone[b], pipe.In));

        // ---- attention of the slice
        TSA_TRY(cudaStreamWaitEvent(pipe.Compute, pipe.InDone[b], 0));
        if (s >= HOST_PIPE_DEPTH) {
            TSA_TRY(cudaStreamWaitEvent(pipe.Compute, pipe.OutDone[b], 0)); // the copy-out that read this set's output
        }
        auto dev2d = [&](size_t off, int pitch, int xsize, int ysize) {
            tsa_ptr2d r;
            r.data = set + off;
            r.stride_bytes = pitch;
            r.xsize = xsize;
            r.ysize = ysize;
            return r;
        };
        tsa_ptr2d none = {nullptr, 0, 0, 0};
        // the slice's output: its columns of the caller's device matrix when there is one, else the staging set
        tsa_ptr2d devOut = dev2d(lay.Out, lay.PitchOut, hn * dv, len);
        if (outDevice.data) {
            devOut.data = (char *)outDevice.data + (size_t)h0 * dv * esz;
            devOut.stride_bytes = outDevice.stride_bytes;
        }
        rc = tsa_att_fwd(cfg, qvGlobalScale, dev2d(lay.Qk, lay.PitchQk, hn * dq, len), dev2d(lay.Qv, lay.PitchQk, hn * dq, len),
            qkScale.data ? dev2d(lay.QkScale, lay.PitchScale, len, hn) : none, dev2d(lay.QvScale, lay.PitchScale, len, hn),
            dev2d(lay.V, lay.PitchV, hn * dv, len), vScale.data ? dev2d(lay.VScale, lay.PitchScale, len, hn) : none,
            attSpans, attSpanPtr, alibiSlope, devOut,
            sumWeightLog.data ? dev2d(lay.Lse, lay.PitchScale, len, hn) : none, hn, lenAttTiles,
            set + lay.Work, lay.WorkBytes, statusWord, (tsa_stream_t)pipe.Compute);
        if (rc != TSA_OK) {
            break;
        }
        TSA_TRY(cudaEventRecord(pipe.KernelDone[b], pipe.Compute));

        // ---- copy out
        TSA_TRY(cudaStreamWaitEvent(pipe.Out, pipe.KernelDone[b], 0));
        TSA_TRY(cudaMemcpy2DAsync((char *)out.data + (size_t)h0 * dv * esz, out.stride_bytes, devOut.data, devOut.stride_bytes, (size_t)hn * dv * esz, len,
            cudaMemcpyDeviceToHost, pipe.Out));
        if (sumWeightLog.data) {
            TSA_TRY(cudaMemcpy2DAsync((char *)sumWeightLog.data + (size_t)h0 * sumWeightLog.stride_bytes, sumWeightLog.stride_bytes, set + lay.Lse,
                lay.PitchScale, (size_t)len * 4, hn, cudaMemcpyDeviceToHost, pipe.Out));
        }
        TSA_TRY(cudaEventRecord(pipe.OutDone[b], pipe.Out));
        ++nDone;
    }
    // the caller's stream continues when the last copies are home (and the kernels with them)
    for (int b = 0; b < HOST_PIPE_DEPTH && b < nDone; ++b) {
        TSA_TRY(cudaStreamWaitEvent(user, pipe.OutDone[b], 0));
    }
    if (rc != TSA_OK) {
        // a slice was refused: what was queued before it still completes; join the streams so the staging area is quiescent
        TSA_TRY(cudaEventRecord(pipe.Start, pipe.In));
        TSA_TRY(cudaStreamWaitEvent(user, pipe.Start, 0));
    }
#undef TSA_TRY
    return rc;
}

extern "C" __attribute__((visibility("default"))) int tsa_peer_scatter(tsa_ptr2d src, const tsa_ptr2d *dsts, int dstCount, int rows, int rowBytes,
    int ctas, tsa_stream_t stream)
{
    TSA_REQUIRE(src.data && dsts && dstCount >= 1 && dstCount <= TSA_MAX_OUT_COPIES, "tsa_peer_scatter: between 1 and %d destinations", TSA_MAX_OUT_COPIES);
    TSA_REQUIRE(rows >= 0 && rowBytes > 0 && rowBytes % 32 == 0, "tsa_peer_scatter: rowBytes %d must be a multiple of 32", rowBytes);
    TSA_REQUIRE(((uintptr_t)src.data | (uintptr_t)src.stride_bytes) % 32 == 0 && src.ysize >= rows, "tsa_peer_scatter: source rows must be 32-byte aligned");
    TPeerDsts d;
    d.Count = dstCount;
    for (int k = 0; k < TSA_MAX_OUT_COPIES; ++k) {
        d.Data[k] = nullptr;
        d.Stride[k] = 0;
    }
    for (int k = 0; k < dstCount; ++k) {
        TSA_REQUIRE(dsts[k].data && ((uintptr_t)dsts[k].data | (uintptr_t)dsts[k].stride_bytes) % 32 == 0 && dsts[k].ysize >= rows,
            "tsa_peer_scatter: destination %d missing, too small or not 32-byte aligned", k);
        d.Data[k] = (char *)dsts[k].data;
        d.Stride[k] = dsts[k].stride_bytes;
    }
    if (rows == 0) {
        return TSA_OK;
    }
    const long long total = (long long)rows * (rowBytes / 32);
    long long want = (total + 255) / 256;
    int grid = (int)(want < (ctas > 0 ? ctas : 148) ? want : (ctas > 0 ? ctas : 148));
    PeerScatterKernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const char *)src.data, src.stride_bytes, d, rows, rowBytes);
    return CheckCuda(cudaGetLastError(), "tsa_peer_scatter launch");
}
