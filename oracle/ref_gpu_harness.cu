// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
// Finite harness around the reference's own GPU attention kernel Fp8Att (code/gpt/compute/gpt_att_fp8.cuh:43-248),
// compiled for sm_100a from the sources where they lie in the reference checkout (oracle/Makefile, target ref_gpu) into
// oracle/_ref/libtsa_ref_gpu.so.  It fills the kernel's TCuda2DPtr / TCuda1DPtr arguments from raw device pointers and
// launches it a given number of times, so that bench.py can time the reference's mma.sync kernel beside this
// library's on the same GPU and inputs, and a test can compare the two outputs.  Nothing of the reference is copied
// here; its shipped test loops (TestAttFp8, TestAttGradQVfp8) never return and are not used.
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <util/eden_core.h>
#define KERNEL_UNIT "tsa_ref_gpu_harness/"
#include <gpt/att/att.h>
#include <gpt/att/rope.h>
#include <gpt/model_params/model_dim.h>
#include <lib/cuda/cuda_arrays.h>
#include <lib/cuda/cuda_util.cuh>
#include <lib/cuda/cuda_mma.cuh>
#include <lib/cuda/cuda_i8.cuh>
#include <lib/cuda/cuda_fp8.cuh>
#include <lib/cuda/vec_util.cuh>

using namespace NCuda;

// the kernels' block sizes are registered for the reference's graph runtime, which the harness does not use
#undef KERNEL_BLOCK_SIZE
#define KERNEL_BLOCK_SIZE(...)

namespace NRefGpuHarness
{
// the constants of the reference's kernel test harness (code/gpt/compute/gpt_att.cu:21-25)
constexpr float QK_VEC_SCALE = 1 / 32.0f;
constexpr float V_VEC_SCALE = 1 / 32.0f;
constexpr int Q_DIM = 128;
constexpr int ATT_GROUP = 64;
constexpr int ATT_ALIGN = 128;
#include <gpt/compute/gpt_rope.cuh>
#include <gpt/compute/gpt_att_fp8.cuh>
}

// Launches Fp8Att `reps` times on `stream` and returns the mean milliseconds per launch in *msOut (CUDA events).
// qk, qv e4m3 [len][H*128]; qvScale f32 [H][len]; vT e4m3 [H*128][len] (V transposed); spans / spanPtr: grouped spans
// (TAttentionSpanGroup<64>); out half [len][H*128]; sumWeightLog f32 [H][len]; strides in bytes.  Returns the CUDA
// error code of the last call.
extern "C" __attribute__((visibility("default"))) int ref_gpu_fp8_att(float *qvGlobalScale, void *qk, int qkStride, void *qv, int qvStride,
    float *qvScale, int qvScaleStride, void *vT, int vTStride, void *spans, int spanCount, int *spanPtr, float alibiSlope,
    void *out, int outStride, float *sumWeightLog, int swlStride, int headCount, int len, int reps, float *msOut, cudaStream_t stream)
{
    using namespace NRefGpuHarness;
    const int lenAttTiles = len / ATT_GROUP;
    TCuda2DPtr<e4m3> pQk(qk, qkStride, headCount * Q_DIM, len), pQv(qv, qvStride, headCount * Q_DIM, len);
    TCuda2DPtr<float> pQvScale(qvScale, qvScaleStride, len, headCount);
    TCuda2DPtr<e4m3> pVT(vT, vTStride, len, headCount * Q_DIM);
    TCuda1DPtr<TAttentionSpanGroup<ATT_GROUP>> pSpans(spans, spanCount);
    TCuda1DPtr<int> pSpanPtr(spanPtr, lenAttTiles + 1);
    TCuda2DPtr<half> pOut(out, outStride, headCount * Q_DIM, len);
    TCuda2DPtr<float> pSwl(sumWeightLog, swlStride, len, headCount);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, stream);
    for (int i = 0; i < reps; ++i) {
        Fp8Att<<<dim3(headCount, lenAttTiles), dim3(32, 4), 0, stream>>>(qvGlobalScale, pQk, pQv, pQvScale, pVT, pSpans, pSpanPtr, alibiSlope, pOut, pSwl);
    }
    cudaEventRecord(e1, stream);
    cudaError_t err = cudaEventSynchronize(e1);
    float ms = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    if (msOut) {
        *msOut = reps > 0 ? ms / reps : 0;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaError_t last = cudaGetLastError();
    return (int)(err != cudaSuccess ? err : last);
}
