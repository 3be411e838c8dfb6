// Shared device/host helpers of the attention library: 2-D pointer views, 8-bit conversions,
// error reporting.  Constants follow code/gpt/model_params/model_dim.h:19-33 of the reference.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "tsa.h"

namespace tsa {

constexpr float kLog2 = 0.693147f;           // LOG2
constexpr float kAttDotProductScale = 0.5f;  // ATT_DOTPRODUCT_SCALE
constexpr int kFarRight = 1000000000;        // GroupAttention's FAR_RIGHT (att/att.h:98)

// sqrt(1/dim) * 0.5 / LOG2  (CalcDotScale * CalcAttentionMult)
inline float HostAttDotScale(int qDim)
{
    return sqrtf(1.0f / qDim) * (kAttDotProductScale / kLog2);
}

// device status codes OR-ed into *statusWord
constexpr int kDevTimeoutTma = 0x10;  // bounded wait on a TMA barrier ran out
constexpr int kDevTimeoutMma = 0x20;  // bounded wait on an MMA-completion barrier ran out
constexpr int kDevBadSpan = 0x40;     // span record outside the key range

// host-side error text (thread local), returns code
int Fail(int code, const char *fmt, ...);
int CheckCuda(cudaError_t err, const char *what);

#define TSA_REQUIRE(cond, ...)                       \
    do {                                             \
        if (!(cond)) {                               \
            return ::tsa::Fail(TSA_BAD_ARG, __VA_ARGS__); \
        }                                            \
    } while (0)

#ifdef TSA_BOUNDS_CHECK
// Bounds-check build (make -C tscale_b200/csrc bounds): every row lookup through P2D is checked against the row count of
// the caller's tsa_ptr2d.  A row outside it is counted in a device word of the translation unit and redirected to row 0,
// so nothing outside the buffer is touched and nothing traps; tsa_bounds_check_hits() adds the words up.
static __device__ int g_tsaBoundsHits;
int RegisterBoundsReader(int (*reader)(int reset));
static int ReadBoundsHitsOfThisFile(int reset)
{
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tsaBoundsHits, sizeof(int)) != cudaSuccess) {
        return 0;
    }
    if (reset) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tsaBoundsHits, &zero, sizeof(int));
    }
    return v;
}
static const int g_tsaBoundsRegistered = RegisterBoundsReader(ReadBoundsHitsOfThisFile);
#endif

template <class T>
struct P2D {
    char *Data;
    int Stride;
#ifdef TSA_BOUNDS_CHECK
    int YSize;
    __host__ __device__ P2D() : Data(nullptr), Stride(0), YSize(0) {}
    __host__ __device__ explicit P2D(const tsa_ptr2d &p) : Data((char *)p.data), Stride(p.stride_bytes), YSize(p.ysize) {}
    __device__ __forceinline__ T *Row(int y) const
    {
        if ((unsigned)y >= (unsigned)YSize) {
            atomicAdd(&g_tsaBoundsHits, 1);
            y = 0;
        }
        return (T *)(Data + (size_t)y * Stride);
    }
#else
    __host__ __device__ P2D() : Data(nullptr), Stride(0) {}
    __host__ __device__ explicit P2D(const tsa_ptr2d &p) : Data((char *)p.data), Stride(p.stride_bytes) {}
    __device__ __forceinline__ T *Row(int y) const { return (T *)(Data + (size_t)y * Stride); }
#endif
    __device__ __forceinline__ bool Valid() const { return Data != nullptr; }
};

inline int DtypeSize(int dt)
{
    switch (dt) {
    case TSA_I8:
    case TSA_E4M3:
        return 1;
    case TSA_F16:
    case TSA_BF16:
        return 2;
    case TSA_F32:
        return 4;
    }
    return 0;
}

// ---- 8-bit conversions (cvt.rn.satfinite.e4m3x2.f32 / cvt.rni.sat.s8.f32, as the reference's
// CvtToE4 util/fp8.h:48-60 and CvtToI8 lib/cuda/cuda_util.cuh:33-38)
__device__ __forceinline__ uint32_t PackE4M3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint32_t PackE4M3x4(float a, float b, float c, float d)
{
    uint32_t r;
    asm("{\n\t"
        ".reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t"
        "}"
        : "=r"(r)
        : "f"(a), "f"(b), "f"(c), "f"(d));
    return r;
}
__device__ __forceinline__ float2 UnpackE4M3x2(uint32_t pair)
{
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)pair));
    __half2 h = *reinterpret_cast<__half2 *>(&h2);
    return __half22float2(h);
}
__device__ __forceinline__ float E4M3ToFloat(uint8_t x)
{
    return UnpackE4M3x2(x).x;
}
__device__ __forceinline__ int FloatToI8Sat(float x)
{
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

// element loads as float, by storage type tag
struct TagI8 {
    typedef int8_t T;
    static __device__ __forceinline__ float Load(const T *p) { return (float)*p; }
};
struct TagE4M3 {
    typedef uint8_t T;
    static __device__ __forceinline__ float Load(const T *p) { return E4M3ToFloat(*p); }
};
struct TagF16 {
    typedef __half T;
    static __device__ __forceinline__ float Load(const T *p) { return __half2float(*p); }
    static __device__ __forceinline__ void Store(T *p, float x) { *p = __float2half_rn(x); }
};
struct TagBF16 {
    typedef __nv_bfloat16 T;
    static __device__ __forceinline__ float Load(const T *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void Store(T *p, float x) { *p = __float2bfloat16_rn(x); }
};
struct TagF32 {
    typedef float T;
    static __device__ __forceinline__ float Load(const T *p) { return *p; }
    static __device__ __forceinline__ void Store(T *p, float x) { *p = x; }
};

__device__ __forceinline__ float LoadAsFloat(const void *base, int idx, int dt)
{
    switch (dt) {
    case TSA_I8:
        return (float)((const int8_t *)base)[idx];
    case TSA_E4M3:
        return E4M3ToFloat(((const uint8_t *)base)[idx]);
    case TSA_F16:
        return __half2float(((const __half *)base)[idx]);
    case TSA_BF16:
        return __bfloat162float(((const __nv_bfloat16 *)base)[idx]);
    default:
        return ((const float *)base)[idx];
    }
}

__device__ __forceinline__ void StoreFromFloat(void *base, int idx, int dt, float x)
{
    switch (dt) {
    case TSA_F16:
        ((__half *)base)[idx] = __float2half_rn(x);
        break;
    case TSA_BF16:
        ((__nv_bfloat16 *)base)[idx] = __float2bfloat16_rn(x);
        break;
    default:
        ((float *)base)[idx] = x;
        break;
    }
}

__device__ __forceinline__ float WarpMax(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    }
    return x;
}
__device__ __forceinline__ float WarpSum(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        x += __shfl_xor_sync(0xffffffffu, x, o);
    }
    return x;
}

} // namespace tsa
