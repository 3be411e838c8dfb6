// Thin inline-PTX wrappers for the sm_100a features the attention kernels use: mbarrier with
// bounded waits, TMA tile loads, tensor-memory allocation / load / store, tcgen05 MMA issue,
// and the shared-memory / instruction descriptors that go with it.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100 {

__device__ __forceinline__ uint32_t SmemAddr(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void MbarInit(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void FenceBarrierInit()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void FenceProxyAsync()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
// adds to the transaction count of the current phase without arriving (the arrival follows separately)
__device__ __forceinline__ void MbarExpectTxOnly(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
// one poll with the default (short) suspend time: for the thread whose wake-up latency is on the critical path
__device__ __forceinline__ bool MbarTryWaitFast(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// register reallocation between the warpgroups of a CTA (all four warps of the warpgroup execute it)
template <int N>
__device__ __forceinline__ void RegDealloc()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void RegAlloc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
// upper bound, in nanoseconds, for which one try_wait may keep the thread suspended before it returns false
constexpr uint32_t kTryWaitHintNs = 200000;
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity), "r"(kTryWaitHintNs)
        : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity; gives up after maxSpins polls and returns false.
// Every wait in this library is bounded so that a lost signal ends in an error code, not a hang.
__device__ __forceinline__ bool MbarWaitBounded(uint64_t *bar, uint32_t parity, uint32_t maxSpins)
{
    for (uint32_t i = 0; i < maxSpins; ++i) {
        if (MbarTryWait(bar, parity)) {
            return true;
        }
    }
    return false;
}

// ---- TMA -------------------------------------------------------------------------------------
// 2-D tile load global -> shared, completion counted in bytes on the mbarrier.
// x is the innermost coordinate; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void TmaLoad2D(void *smemDst, const void *tensorMap, int x, int y, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        :
        : "r"(SmemAddr(smemDst)), "l"(tensorMap), "r"(x), "r"(y), "r"(SmemAddr(bar))
        : "memory");
}
// untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void BulkLoad(void *smemDst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :
                 : "r"(SmemAddr(smemDst)), "l"(gsrc), "r"(bytes), "r"(SmemAddr(bar))
                 : "memory");
}
__device__ __forceinline__ void PrefetchTensorMap(const void *tensorMap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tensorMap) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------
// whole warp; writes the base address (lane 0, first column) to *smemSlot
__device__ __forceinline__ void TmemAlloc(uint32_t *smemSlot, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemSlot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void TcFenceAfter()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void TmemWaitLd()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemWaitSt()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread l of the warp gets lane (laneBase + l)
__device__ __forceinline__ void TmemLd32(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemLd16(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemSt32(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// ---- descriptors -----------------------------------------------------------------------------
enum TmaSwizzleBytes { SW64 = 64, SW128 = 128 };

// Shared-memory matrix descriptor (tcgen05): start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1, swizzle mode in bits 61-63 (2 = 128 B, 4 = 64 B).
// The tile base must be aligned to 8 rows of the swizzle span (1024 B / 512 B).
__device__ __forceinline__ uint64_t MakeSmemDesc(uint32_t smemAddr, uint32_t leadingBytes, uint32_t strideBytes, int swizzleBytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smemAddr & 0x3ffff) >> 4);
    d |= (uint64_t)((leadingBytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)((strideBytes >> 4) & 0x3fff) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(swizzleBytes == 128 ? 2 : 4) << 61;
    return d;
}

// Instruction descriptor (32 bit): c format bits 4-5 (1 = f32, 2 = s32), a/b format bits 7-9 / 10-12
// (f8f6f4: 0 = e4m3; i8: 1 = signed), a/b major bits 15 / 16 (1 = MN-major), N>>3 bits 17-22, M>>4 bits 24-28.
__host__ __device__ constexpr uint32_t MakeInstrDesc(int cFormat, int aFormat, int bFormat, int aMnMajor, int bMnMajor, int m, int n)
{
    return ((uint32_t)cFormat << 4) | ((uint32_t)aFormat << 7) | ((uint32_t)bFormat << 10) | ((uint32_t)aMnMajor << 15) |
        ((uint32_t)bMnMajor << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// One lane of a converged warp, chosen by the hardware.  Code that issues tcgen05.mma runs warp-uniform up to the
// instruction itself and wraps only the issue in `if (ElectOne())`: descriptors and addresses then stay in uniform
// registers.  Issued from a divergent `if (lane == 0)` region instead, every operand is moved per instruction, and under
// busy arithmetic warps the issuing thread was measured three times slower (216 against 70 clocks per MMA).
__device__ __forceinline__ uint32_t ElectOne()
{
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}"
        : "=r"(pred));
    return pred;
}

// ---- MMA issue (one thread) ------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void MmaF8SS(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void MmaI8SS(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void MmaF8TS(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// bf16 operands, f32 accumulation
__device__ __forceinline__ void MmaF16SS(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void MmaF16TS(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// ---- grouped issue -----------------------------------------------------------------------------
// One asm block per group of MMAs on the same accumulator: the descriptor increments happen inside the block, so the
// compiler moves the base values to the uniform datapath once per group instead of once per instruction, and the
// issuing thread (a single thread whose instruction stream sits on the critical path between the softmax warps'
// "weights written" and "scores ready") gets through a group in a fraction of the time.
//
// D[tmem] = A[smem] * B[smem] over KSTEPS steps of 32 bytes along K (both operands K-major, descriptor address field in
// 16-byte units), then a commit on `bar`.  I8: kind::i8, else kind::f8f6f4.
template <int KSTEPS, bool I8>
__device__ __forceinline__ void MmaGroupSSCommit(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint64_t *bar)
{
    static_assert(KSTEPS == 2 || KSTEPS == 4, "two or four K steps");
    if (KSTEPS == 2) {
        if (I8) {
            asm volatile(
                "{\n\t"
                ".reg .pred pf, pt;\n\t"
                ".reg .b64 a1, b1;\n\t"
                "setp.ne.u32 pf, 0, 0;\n\t"
                "setp.eq.u32 pt, 0, 0;\n\t"
                "add.u64 a1, %1, 2;\n\t"
                "add.u64 b1, %2, 2;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, pf;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %3, pt;\n\t"
                "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t"
                "}"
                :
                : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(SmemAddr(bar))
                : "memory");
        } else {
            asm volatile(
                "{\n\t"
                ".reg .pred pf, pt;\n\t"
                ".reg .b64 a1, b1;\n\t"
                "setp.ne.u32 pf, 0, 0;\n\t"
                "setp.eq.u32 pt, 0, 0;\n\t"
                "add.u64 a1, %1, 2;\n\t"
                "add.u64 b1, %2, 2;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, pf;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a1, b1, %3, pt;\n\t"
                "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t"
                "}"
                :
                : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(SmemAddr(bar))
                : "memory");
        }
    } else {
        if (I8) {
            asm volatile(
                "{\n\t"
                ".reg .pred pf, pt;\n\t"
                ".reg .b64 a1, b1, a2, b2, a3, b3;\n\t"
                "setp.ne.u32 pf, 0, 0;\n\t"
                "setp.eq.u32 pt, 0, 0;\n\t"
                "add.u64 a1, %1, 2;\n\t"
                "add.u64 b1, %2, 2;\n\t"
                "add.u64 a2, %1, 4;\n\t"
                "add.u64 b2, %2, 4;\n\t"
                "add.u64 a3, %1, 6;\n\t"
                "add.u64 b3, %2, 6;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, pf;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], a1, b1, %3, pt;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], a2, b2, %3, pt;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], a3, b3, %3, pt;\n\t"
                "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t"
                "}"
                :
                : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(SmemAddr(bar))
                : "memory");
        } else {
            asm volatile(
                "{\n\t"
                ".reg .pred pf, pt;\n\t"
                ".reg .b64 a1, b1, a2, b2, a3, b3;\n\t"
                "setp.ne.u32 pf, 0, 0;\n\t"
                "setp.eq.u32 pt, 0, 0;\n\t"
                "add.u64 a1, %1, 2;\n\t"
                "add.u64 b1, %2, 2;\n\t"
                "add.u64 a2, %1, 4;\n\t"
                "add.u64 b2, %2, 4;\n\t"
                "add.u64 a3, %1, 6;\n\t"
                "add.u64 b3, %2, 6;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, pf;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a1, b1, %3, pt;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a2, b2, %3, pt;\n\t"
                "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a3, b3, %3, pt;\n\t"
                "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%4];\n\t"
                "}"
                :
                : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(SmemAddr(bar))
                : "memory");
        }
    }
}

// D[tmem] (+)= A[tmem] * B[smem], kind::f8f6f4, two K steps of 32: A at aTmem and aTmem + 32 columns, B descriptors
// bDesc and bDesc + bStep (16-byte units); `accumulate` applies to the first step.  With residual: two more steps with A
// 8 columns further on and the same B.
__device__ __forceinline__ void MmaPairF8TS(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t bStep, uint32_t idesc,
    uint32_t accumulate, bool withResidual)
{
    if (!withResidual) {
        asm volatile(
            "{\n\t"
            ".reg .pred p0, pt;\n\t"
            ".reg .b64 b1, st;\n\t"
            ".reg .b32 a1;\n\t"
            "setp.ne.b32 p0, %4, 0;\n\t"
            "setp.eq.u32 pt, 0, 0;\n\t"
            "cvt.u64.u32 st, %5;\n\t"
            "add.u64 b1, %2, st;\n\t"
            "add.u32 a1, %1, 32;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a1], b1, %3, pt;\n\t"
            "}"
            :
            : "r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(bStep)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p0, pt;\n\t"
            ".reg .b64 b1, st;\n\t"
            ".reg .b32 a1, a2, a3;\n\t"
            "setp.ne.b32 p0, %4, 0;\n\t"
            "setp.eq.u32 pt, 0, 0;\n\t"
            "cvt.u64.u32 st, %5;\n\t"
            "add.u64 b1, %2, st;\n\t"
            "add.u32 a1, %1, 32;\n\t"
            "add.u32 a2, %1, 8;\n\t"
            "add.u32 a3, %1, 40;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a1], b1, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a2], %2, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [a3], b1, %3, pt;\n\t"
            "}"
            :
            : "r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(bStep)
            : "memory");
    }
}


// bf16: D[tmem] = A[smem] * B[smem] over KSTEPS steps of 16 elements along K, both operands K-major tiles made of
// [128 rows][128 bytes] blocks (16 KB each) with the 128-byte swizzle: four steps per block, then the next block.
// One asm block per group for the reason given above.
template <int KSTEPS>
__device__ __forceinline__ void MmaGroupF16SS(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t bBlockUnits = 1024)
{
    static_assert(KSTEPS == 4 || KSTEPS == 8, "four or eight K steps");
    // A: [128 rows][128 bytes] blocks, 1024 descriptor units (16 KB) apart; B: blocks bBlockUnits apart (a B tile of 64 rows
    // has 8 KB blocks = 512 units)
    const uint64_t bDesc2 = bDesc + bBlockUnits;
    if (KSTEPS == 4) {
        asm volatile(
            "{\n\t"
            ".reg .pred pf, pt;\n\t"
            ".reg .b64 a<4>, b<4>;\n\t"
            "setp.ne.u32 pf, 0, 0;\n\t"
            "setp.eq.u32 pt, 0, 0;\n\t"
            "add.u64 a1, %1, 2;\n\t"
            "add.u64 b1, %2, 2;\n\t"
            "add.u64 a2, %1, 4;\n\t"
            "add.u64 b2, %2, 4;\n\t"
            "add.u64 a3, %1, 6;\n\t"
            "add.u64 b3, %2, 6;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, pt;\n\t"
            "}"
            :
            : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "l"(bDesc2)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred pf, pt;\n\t"
            ".reg .b64 a<8>, b<8>;\n\t"
            "setp.ne.u32 pf, 0, 0;\n\t"
            "setp.eq.u32 pt, 0, 0;\n\t"
            "add.u64 a1, %1, 2;\n\t"
            "add.u64 b1, %2, 2;\n\t"
            "add.u64 a2, %1, 4;\n\t"
            "add.u64 b2, %2, 4;\n\t"
            "add.u64 a3, %1, 6;\n\t"
            "add.u64 b3, %2, 6;\n\t"
            "add.u64 a4, %1, 1024;\n\t"
            "add.u64 b4, %4, 0;\n\t"
            "add.u64 a5, %1, 1026;\n\t"
            "add.u64 b5, %4, 2;\n\t"
            "add.u64 a6, %1, 1028;\n\t"
            "add.u64 b6, %4, 4;\n\t"
            "add.u64 a7, %1, 1030;\n\t"
            "add.u64 b7, %4, 6;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a4, b4, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a5, b5, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a6, b6, %3, pt;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], a7, b7, %3, pt;\n\t"
            "}"
            :
            : "r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "l"(bDesc2)
            : "memory");
    }
}

// bf16: D[tmem] (+)= A[tmem] * B[smem] over four K steps of 16: A at aTmem + 0, 16, 32, 48 columns (each block of 16
// keys keeps its packed pairs in the first 8 of its own 16 columns), B descriptors bDesc + 0, 128, 256, 384 (16 rows of 128 bytes per
// step, MN-major); `accumulate` applies to the first step.
__device__ __forceinline__ void MmaQuadF16TS(uint32_t dTmem, uint32_t aTmem, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p0, pt;\n\t"
        ".reg .b64 b1, b2, b3;\n\t"
        ".reg .b32 a1, a2, a3;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\t"
        "setp.eq.u32 pt, 0, 0;\n\t"
        "add.u64 b1, %2, 128;\n\t"
        "add.u64 b2, %2, 256;\n\t"
        "add.u64 b3, %2, 384;\n\t"
        "add.u32 a1, %1, 16;\n\t"
        "add.u32 a2, %1, 32;\n\t"
        "add.u32 a3, %1, 48;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %3, pt;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %3, pt;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %3, pt;\n\t"
        "}"
        :
        : "r"(dTmem), "r"(aTmem), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// arrive on the mbarrier when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void MmaCommit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

} // namespace sm100
