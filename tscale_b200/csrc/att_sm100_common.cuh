// Device and host helpers shared by the tcgen05 attention kernels (forward and backward): bounded barrier waits,
// named barriers, the key-tile iterator over grouped spans, small arithmetic wrappers, TMA tensor-map creation.
#pragma once
#include "att_internal.cuh"
#include "sm100_ptx.cuh"
#include <cuda.h>
#include <type_traits>

namespace tsa {

using namespace sm100;

constexpr long long WAIT_CYCLES = 1ll << 31; // about a second
constexpr int TILE_ROWS = 128;               // rows / columns of a score tile

__device__ __forceinline__ bool WaitBar(uint64_t *bar, uint32_t parity, long long limit = WAIT_CYCLES)
{
    long long t0 = clock64();
    for (;;) {
        if (MbarWaitBounded(bar, parity, 64)) {
            return true;
        }
        if (clock64() - t0 > limit) {
            return false;
        }
    }
}

// the same with an abort flag of the CTA: returns false as soon as another thread has given up.
// FAST polls without a suspend hint (the waiting thread's wake-up latency is on the critical path).
template <bool FAST = false>
__device__ __forceinline__ bool WaitBarA(uint64_t *bar, uint32_t parity, const int *abortFlag)
{
    if (FAST ? MbarTryWaitFast(bar, parity) : MbarTryWait(bar, parity)) {
        return true;
    }
    long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 32; ++i) {
            if (FAST ? MbarTryWaitFast(bar, parity) : MbarTryWait(bar, parity)) {
                return true;
            }
        }
        if (*(const volatile int *)abortFlag) {
            return false;
        }
        if (clock64() - t0 > WAIT_CYCLES) {
            return false;
        }
    }
}

// Polling wait with a pause between polls: a waiting warp issues a handful of instructions every SLEEP_NS instead of
// spinning, so it does not take issue slots from the warps that share its scheduler (a tight try_wait loop of the
// MMA-issuing warp cost the softmax warp next to it a third of its issue rate).  Returns false when the CTA's abort
// flag is set or after about a second.
template <int SLEEP_NS>
__device__ __forceinline__ bool WaitBarSleep(uint64_t *bar, uint32_t parity, const int *abortFlag, long long limit = WAIT_CYCLES)
{
    if (MbarTryWaitFast(bar, parity)) {
        return true;
    }
    long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; ++i) {
            __nanosleep(SLEEP_NS);
            if (MbarTryWaitFast(bar, parity)) {
                return true;
            }
        }
        if (*(const volatile int *)abortFlag) {
            return false;
        }
        if (clock64() - t0 > limit) {
            return false;
        }
    }
}

__device__ __forceinline__ void MbarArrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

// named barrier over `count` threads with an OR reduction of a predicate
__device__ __forceinline__ bool BarRedOr(int id, int count, bool flag)
{
    uint32_t res;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(res)
        : "r"(id), "r"(count), "r"((uint32_t)flag)
        : "memory");
    return res != 0;
}
__device__ __forceinline__ void BarSync(int id, int count)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// iterator over the key tiles of a 128-row query tile: rounds of the two 64-row blocks' span groups
struct TTileIter {
    const tsa_span_group *G0, *G1; // first group of each block (null: block absent)
    int N0, N1;
    int KeyRows;
    int Round, J0, Hi;
    bool Valid;

    __device__ void LoadRound()
    {
        int rounds = max(N0, N1);
        for (; Round < rounds; ++Round) {
            int lo = 0x7fffffff, hi = -1;
            if (Round < N0) {
                lo = min(lo, G0[Round].Start);
                hi = max(hi, G0[Round].Finish);
            }
            if (Round < N1) {
                lo = min(lo, G1[Round].Start);
                hi = max(hi, G1[Round].Finish);
            }
            lo = max(lo, 0) & ~(TILE_ROWS - 1);
            hi = min(hi, KeyRows - 1) & ~(TILE_ROWS - 1);
            if (lo <= hi) {
                J0 = lo;
                Hi = hi;
                Valid = true;
                return;
            }
        }
        Valid = false;
    }
    __device__ void Init(const tsa_span_group *spans, const int *spanPtr, int lenAttTiles, int qTile, int keyRows)
    {
        int b0 = qTile * 2, b1 = qTile * 2 + 1;
        G0 = G1 = nullptr;
        N0 = N1 = 0;
        if (b0 < lenAttTiles) {
            int a = spanPtr[b0], b = spanPtr[b0 + 1];
            G0 = spans + a;
            N0 = b - a;
        }
        if (b1 < lenAttTiles) {
            int a = spanPtr[b1], b = spanPtr[b1 + 1];
            G1 = spans + a;
            N1 = b - a;
        }
        KeyRows = keyRows;
        Round = 0;
        Valid = false;
        LoadRound();
    }
    __device__ void Advance()
    {
        J0 += TILE_ROWS;
        if (J0 > Hi) {
            ++Round;
            LoadRound();
        }
    }
};

// one 32-byte store (the address must be 32-byte aligned): a thread that writes its own row fills whole 32-byte sectors
// with half as many store instructions as with 16-byte stores
__device__ __forceinline__ void StGlobal256(void *p, const uint32_t *v)
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]),
                 "r"(v[6]), "r"(v[7])
                 : "memory");
}

// the same store with the streaming hint: data that is written once and read by a later kernel should not displace the
// tiles this kernel keeps re-reading from L2
__device__ __forceinline__ void StGlobal256Stream(void *p, const uint32_t *v)
{
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]),
                 "r"(v[6]), "r"(v[7])
                 : "memory");
}

template <int N>
__device__ __forceinline__ void TmemStN(uint32_t taddr, const uint32_t *r);
template <>
__device__ __forceinline__ void TmemStN<4>(uint32_t taddr, const uint32_t *r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
template <>
__device__ __forceinline__ void TmemStN<8>(uint32_t taddr, const uint32_t *r)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 :
                 : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void TmemLd2(uint32_t taddr, uint32_t &a, uint32_t &b)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void TmemSt2(uint32_t taddr, uint32_t a, uint32_t b)
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void TmemLd8(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void TmemSt16(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// 32 consecutive columns of this thread's lane as 16 register pairs (for packed f32x2 arithmetic without
// re-pairing moves); includes the wait for the load.
__device__ __forceinline__ void TmemLd32Pairs(uint32_t taddr, float2 *s)
{
    uint64_t v[16];
    asm volatile(
        "{\n\t"
        ".reg .b32 t<32>;\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, t16, t17, t18, t19, t20, t21, t22, t23, t24, t25, t26, t27, t28, t29, t30, t31}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n\t"
        "mov.b64 %0, {t0, t1};\n\t"
        "mov.b64 %1, {t2, t3};\n\t"
        "mov.b64 %2, {t4, t5};\n\t"
        "mov.b64 %3, {t6, t7};\n\t"
        "mov.b64 %4, {t8, t9};\n\t"
        "mov.b64 %5, {t10, t11};\n\t"
        "mov.b64 %6, {t12, t13};\n\t"
        "mov.b64 %7, {t14, t15};\n\t"
        "mov.b64 %8, {t16, t17};\n\t"
        "mov.b64 %9, {t18, t19};\n\t"
        "mov.b64 %10, {t20, t21};\n\t"
        "mov.b64 %11, {t22, t23};\n\t"
        "mov.b64 %12, {t24, t25};\n\t"
        "mov.b64 %13, {t26, t27};\n\t"
        "mov.b64 %14, {t28, t29};\n\t"
        "mov.b64 %15, {t30, t31};\n\t"
        "}"
        : "=l"(v[0]), "=l"(v[1]), "=l"(v[2]), "=l"(v[3]), "=l"(v[4]), "=l"(v[5]), "=l"(v[6]), "=l"(v[7]), "=l"(v[8]), "=l"(v[9]), "=l"(v[10]), "=l"(v[11]), "=l"(v[12]), "=l"(v[13]), "=l"(v[14]), "=l"(v[15])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        s[i] = make_float2(__uint_as_float((uint32_t)v[i]), __uint_as_float((uint32_t)(v[i] >> 32)));
    }
}

// 64 consecutive columns of this thread's lane as 32 register pairs, one wait for both loads
__device__ __forceinline__ void TmemLd64Pairs(uint32_t taddr, float2 *s)
{
    uint64_t v[32];
    asm volatile(
        "{\n\t"
        ".reg .b32 t<32>;\n\t"
        ".reg .b32 u<32>;\n\t"
        ".reg .b32 a2;\n\t"
        "add.u32 a2, %32, 32;\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {t0, t1, t2, t3, t4, t5, t6, t7, t8, t9, t10, t11, t12, t13, t14, t15, t16, t17, t18, t19, t20, t21, t22, t23, t24, t25, t26, t27, t28, t29, t30, t31}, [%32];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {u0, u1, u2, u3, u4, u5, u6, u7, u8, u9, u10, u11, u12, u13, u14, u15, u16, u17, u18, u19, u20, u21, u22, u23, u24, u25, u26, u27, u28, u29, u30, u31}, [a2];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n\t"
        "mov.b64 %0, {t0, t1};\n\t"
        "mov.b64 %1, {t2, t3};\n\t"
        "mov.b64 %2, {t4, t5};\n\t"
        "mov.b64 %3, {t6, t7};\n\t"
        "mov.b64 %4, {t8, t9};\n\t"
        "mov.b64 %5, {t10, t11};\n\t"
        "mov.b64 %6, {t12, t13};\n\t"
        "mov.b64 %7, {t14, t15};\n\t"
        "mov.b64 %8, {t16, t17};\n\t"
        "mov.b64 %9, {t18, t19};\n\t"
        "mov.b64 %10, {t20, t21};\n\t"
        "mov.b64 %11, {t22, t23};\n\t"
        "mov.b64 %12, {t24, t25};\n\t"
        "mov.b64 %13, {t26, t27};\n\t"
        "mov.b64 %14, {t28, t29};\n\t"
        "mov.b64 %15, {t30, t31};\n\t"
        "mov.b64 %16, {u0, u1};\n\t"
        "mov.b64 %17, {u2, u3};\n\t"
        "mov.b64 %18, {u4, u5};\n\t"
        "mov.b64 %19, {u6, u7};\n\t"
        "mov.b64 %20, {u8, u9};\n\t"
        "mov.b64 %21, {u10, u11};\n\t"
        "mov.b64 %22, {u12, u13};\n\t"
        "mov.b64 %23, {u14, u15};\n\t"
        "mov.b64 %24, {u16, u17};\n\t"
        "mov.b64 %25, {u18, u19};\n\t"
        "mov.b64 %26, {u20, u21};\n\t"
        "mov.b64 %27, {u22, u23};\n\t"
        "mov.b64 %28, {u24, u25};\n\t"
        "mov.b64 %29, {u26, u27};\n\t"
        "mov.b64 %30, {u28, u29};\n\t"
        "mov.b64 %31, {u30, u31};\n\t"
        "}"
        : "=l"(v[0]), "=l"(v[1]), "=l"(v[2]), "=l"(v[3]), "=l"(v[4]), "=l"(v[5]), "=l"(v[6]), "=l"(v[7]), "=l"(v[8]), "=l"(v[9]), "=l"(v[10]), "=l"(v[11]), "=l"(v[12]), "=l"(v[13]), "=l"(v[14]), "=l"(v[15]), "=l"(v[16]), "=l"(v[17]), "=l"(v[18]), "=l"(v[19]), "=l"(v[20]), "=l"(v[21]), "=l"(v[22]), "=l"(v[23]), "=l"(v[24]), "=l"(v[25]), "=l"(v[26]), "=l"(v[27]), "=l"(v[28]), "=l"(v[29]), "=l"(v[30]), "=l"(v[31])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        s[i] = make_float2(__uint_as_float((uint32_t)v[i]), __uint_as_float((uint32_t)(v[i] >> 32)));
    }
}

// 16 consecutive columns from each of two tensor-memory addresses (same lane) as register pairs, one wait for both
__device__ __forceinline__ void TmemLd16x2Pairs(uint32_t taddrA, uint32_t taddrB, float2 *a, float2 *b)
{
    uint64_t v[16];
    asm volatile(
        "{\n\t"
        ".reg .b32 s<16>;\n\t"
        ".reg .b32 d<16>;\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {s0, s1, s2, s3, s4, s5, s6, s7, s8, s9, s10, s11, s12, s13, s14, s15}, [%16];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {d0, d1, d2, d3, d4, d5, d6, d7, d8, d9, d10, d11, d12, d13, d14, d15}, [%17];\n\t"
        "tcgen05.wait::ld.sync.aligned;\n\t"
        "mov.b64 %0, {s0, s1};\n\t"
        "mov.b64 %1, {s2, s3};\n\t"
        "mov.b64 %2, {s4, s5};\n\t"
        "mov.b64 %3, {s6, s7};\n\t"
        "mov.b64 %4, {s8, s9};\n\t"
        "mov.b64 %5, {s10, s11};\n\t"
        "mov.b64 %6, {s12, s13};\n\t"
        "mov.b64 %7, {s14, s15};\n\t"
        "mov.b64 %8, {d0, d1};\n\t"
        "mov.b64 %9, {d2, d3};\n\t"
        "mov.b64 %10, {d4, d5};\n\t"
        "mov.b64 %11, {d6, d7};\n\t"
        "mov.b64 %12, {d8, d9};\n\t"
        "mov.b64 %13, {d10, d11};\n\t"
        "mov.b64 %14, {d12, d13};\n\t"
        "mov.b64 %15, {d14, d15};\n\t"
        "}"
        : "=l"(v[0]), "=l"(v[1]), "=l"(v[2]), "=l"(v[3]), "=l"(v[4]), "=l"(v[5]), "=l"(v[6]), "=l"(v[7]), "=l"(v[8]), "=l"(v[9]), "=l"(v[10]), "=l"(v[11]), "=l"(v[12]), "=l"(v[13]), "=l"(v[14]), "=l"(v[15])
        : "r"(taddrA), "r"(taddrB)
        : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a[i] = make_float2(__uint_as_float((uint32_t)v[i]), __uint_as_float((uint32_t)(v[i] >> 32)));
        b[i] = make_float2(__uint_as_float((uint32_t)v[8 + i]), __uint_as_float((uint32_t)(v[8 + i] >> 32)));
    }
}

// 2^x of a register pair, result again a pair
__device__ __forceinline__ float2 FastExp2Pair(float2 x)
{
    uint64_t in = (uint64_t)__float_as_uint(x.x) | ((uint64_t)__float_as_uint(x.y) << 32), out;
    asm("{\n\t"
        ".reg .f32 a, b;\n\t"
        "mov.b64 {a, b}, %1;\n\t"
        "ex2.approx.ftz.f32 a, a;\n\t"
        "ex2.approx.ftz.f32 b, b;\n\t"
        "mov.b64 %0, {a, b};\n\t"
        "}"
        : "=l"(out)
        : "l"(in));
    return make_float2(__uint_as_float((uint32_t)out), __uint_as_float((uint32_t)(out >> 32)));
}

__device__ __forceinline__ float FastExp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float Max3(float a, float b, float c)
{
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ uint32_t PackHalf2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
// residual of a pair after e4m3 rounding, again as an e4m3 pair
__device__ __forceinline__ uint32_t ResidualE4M3x2(float a, float b, uint32_t hiPair)
{
    uint32_t hb;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hb) : "h"((uint16_t)hiPair));
    uint32_t ef = PackHalf2(a, b);
    uint32_t diff;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(diff) : "r"(ef), "r"(hb));
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(r) : "r"(diff));
    return r;
}

// four packed e4m3 values times a power of two given as an f16 pair (exact unless the result leaves the e4m3 range)
__device__ __forceinline__ uint32_t ScaleE4M3x4(uint32_t w, uint32_t alphaH2)
{
    uint32_t lo, hi;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"((uint16_t)(w & 0xffff)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"((uint16_t)(w >> 16)));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(lo) : "r"(alphaH2));
    asm("mul.rn.f16x2 %0, %0, %1;" : "+r"(hi) : "r"(alphaH2));
    uint16_t a, b;
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(a) : "r"(lo));
    asm("cvt.rn.satfinite.e4m3x2.f16x2 %0, %1;" : "=h"(b) : "r"(hi));
    return (uint32_t)a | ((uint32_t)b << 16);
}

// exact int32 -> float for |x| < 2^22 without the conversion pipe: bits(1.5 * 2^23 + x) - 1.5 * 2^23
__device__ __forceinline__ float2 IntPairToFloat(uint32_t a, uint32_t b)
{
    float2 t = make_float2(__uint_as_float(a + 0x4B400000u), __uint_as_float(b + 0x4B400000u));
    return __fadd2_rn(t, make_float2(-12582912.0f, -12582912.0f));
}


// ---- host side: TMA tensor maps ------------------------------------------------------------------
typedef CUresult (*TEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline TEncodeTiled GetEncodeTiled()
{
    static TEncodeTiled fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess) {
            fn = (TEncodeTiled)ptr;
        }
    }
    return fn;
}

// 2-D tensor map of a row-major matrix with `elemBytes`-byte elements: box = boxRows rows x boxCols elements,
// swizzle span = boxCols * elemBytes (64 or 128 bytes)
static inline int MakeTileMapEx(CUtensorMap *map, tsa_ptr2d a, int elemBytes, int boxCols, int boxRows, const char *what)
{
    TEncodeTiled enc = GetEncodeTiled();
    if (!enc) {
        return Fail(TSA_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    }
    cuuint64_t dims[2] = {(cuuint64_t)a.xsize, (cuuint64_t)a.ysize};
    cuuint64_t strides[1] = {(cuuint64_t)a.stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)boxCols, (cuuint32_t)boxRows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, elemBytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.data, dims, strides, box, estr,
        CU_TENSOR_MAP_INTERLEAVE_NONE, boxCols * elemBytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return Fail(TSA_CUDA_ERROR, "cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
    }
    return TSA_OK;
}

// rows x (xsize bytes) matrix of bytes, box = 128 rows x headDim bytes, swizzle = headDim bytes
static inline int MakeTileMap(CUtensorMap *map, tsa_ptr2d a, int headDim, const char *what)
{
    TEncodeTiled enc = GetEncodeTiled();
    if (!enc) {
        return Fail(TSA_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    }
    cuuint64_t dims[2] = {(cuuint64_t)a.xsize, (cuuint64_t)a.ysize};
    cuuint64_t strides[1] = {(cuuint64_t)a.stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)headDim, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a.data, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
        headDim == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return Fail(TSA_CUDA_ERROR, "cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
    }
    return TSA_OK;
}


} // namespace tsa
