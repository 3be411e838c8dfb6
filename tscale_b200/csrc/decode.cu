// KV-cache decode step: a bandwidth-bound stream over the int8 K and V rows of each sequence.
//
// Reference behaviour: NCPUInfer::ComputeValLookup (code/gpt/train/cpu_infer.cpp:413-460): for the
// newest token cur of a sequence, keys to = cur - dt, dt = 1..min(cur, width) (width 0: to = cur),
// logit = int32dot(q, k[to]) * kScale[to][h] * attDotScale * qScale - slope * (cur - to), a sink with
// logit 0, softmax in base 2, out = sum softmax * vScale[to][h] * v[to].
//
// Layout: per sequence K and V are [capacity][H*D] int8 with the heads of one token contiguous, so a
// token range of a sequence is one contiguous byte range.  A CTA owns (sequence, chunk of DEC_CHUNK
// tokens) and all heads: a 128-bit load per lane covers 512 contiguous bytes per warp = 32/LPH heads
// of one token (LPH = D/16 lanes per head).  The int8 dot uses dp4a (exact int32), partial sums are
// reduced over the LPH lanes of a head with shuffles.  Each CTA keeps an online (max, sum, acc[D])
// per head and writes it to the scratch buffer; a second kernel merges the chunks of a sequence and
// adds the sink.  Algorithmic traffic per key: 2*D bytes + 2 scales per head.
#include "tsa_common.cuh"
#include <mutex>

namespace tsa {

constexpr int DEC_WARPS = 4;

struct TDecodeParams {
    const tsa_kv_seq *Seqs;
    const int *CtxLens;
    int NSeq;
    int HeadCount;
    int Window;
    int ScaleDtype;
    int OutDtype;
    float Slope;
    float DotScale;  // attDotScale
    float QVecScale; // constant query scale when QScale is absent
    P2D<int8_t> Q;
    P2D<float> QScale;
    P2D<char> Out;
    float *Partial;  // [chunk slot][H][D + 4]
    int *Plan;       // workspace header: Plan[0] = tokens per chunk, Plan[1 + s] = first chunk slot of sequence s
    int TargetCtas;  // chunk slots the keys of all sequences are spread over
    int *Status;     // device status word (may be null)
    int MaxSlots;    // TargetCtas + nSeq
    int MaxCtx;      // the caller's upper bound of CtxLens: sizes the grid, checked on the device
    // inference step only (null otherwise): the merge kernel also writes the combiner input
    // kv[seq][head][blk][z] = int8(KvKey[seq][head][z ^ blk] * out[seq][head][z]), blk = 0..3 (KVProduct, cpu_infer.cpp:318-337)
    const int8_t *KvKey;
    int8_t *KvOut;
    int CtxBias;     // added to every CtxLens entry: 1 when the caller has written the new token but not yet counted it
};

__device__ __forceinline__ int CtxLenOf(const TDecodeParams &p, int s)
{
    return p.CtxLens[s] + p.CtxBias;
}

__device__ __forceinline__ float LoadScale(const void *base, size_t idx, int dt)
{
    return dt == TSA_F16 ? __half2float(((const __half *)base)[idx]) : ((const float *)base)[idx];
}

__device__ __forceinline__ void KeyRange(int ctxLen, int window, int *j0, int *j1)
{
    int cur = ctxLen - 1;
    if (window == 0) {
        *j0 = cur;
        *j1 = cur + 1;
    } else {
        *j0 = max(0, cur - window);
        *j1 = cur;
    }
}

constexpr int DEC_MIN_CHUNK = 16; // keys: short windows are spread over several CTAs of two batches rather than one CTA of eight

__device__ __forceinline__ int SeqKeys(const int *ctxLens, int ctxBias, int s, int window)
{
    int ctxLen = ctxLens[s] + ctxBias;
    if (ctxLen <= 0) {
        return 0;
    }
    int j0, j1;
    KeyRange(ctxLen, window, &j0, &j1);
    return j1 - j0;
}

// Balanced plan: all keys of all sequences are cut into chunks of (nearly) the same size C = total / TargetCtas, so
// that every CTA streams the same number of bytes whatever the mix of context lengths.  Chunk slots are numbered
// sequence by sequence.  Every CTA derives the plan from ctxLens itself (a block-wide sum and scan); CTA 0 also
// writes it to the workspace header for the merge kernel.  Returns false if this CTA has no chunk.
// barrier of the DEC_WARPS * 32 planning threads (the producer warp does not take part)
__device__ __forceinline__ void PlanSync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_WARPS * 32) : "memory");
}

__device__ bool DecodePlan(const TDecodeParams &p, int slot, int *pSeq, int *pBeg, int *pEnd)
{
    __shared__ int red[DEC_WARPS];
    __shared__ int sliceBase[DEC_WARPS * 32 + 1];
    __shared__ int found[3];
    const int tid = threadIdx.x, nThreads = DEC_WARPS * 32;
    // total number of keys
    int sum = 0;
    for (int s = tid; s < p.NSeq; s += nThreads) {
        sum += SeqKeys(p.CtxLens, p.CtxBias, s, p.Window);
        if (CtxLenOf(p, s) > p.MaxCtx && blockIdx.x == 0 && p.Status) {
            atomicOr(p.Status, kDevBadSpan); // the grid was sized for shorter sequences
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    if ((tid & 31) == 0) {
        red[tid >> 5] = sum;
    }
    PlanSync();
    int total = 0;
    for (int w = 0; w < DEC_WARPS; ++w) {
        total += red[w];
    }
    int chunk = (total + p.TargetCtas - 1) / p.TargetCtas;
    chunk = max((chunk + 7) & ~7, DEC_MIN_CHUNK);
    // A sequence's last chunk is a partial one, so that chunk size can give up to NSeq chunks more than CTAs are
    // resident, and those would run as a second, nearly empty wave.  Take the smallest chunk size (a multiple of 8)
    // whose chunks all fit the one wave instead: the count of chunks falls as the size grows, and
    // total / (TargetCtas - NSeq) is always enough, so a bisection between the two finds it.
    if (p.NSeq < p.TargetCtas) {
        int lo = chunk / 8;
        int hi = max(((total + (p.TargetCtas - p.NSeq) - 1) / (p.TargetCtas - p.NSeq) + 7) / 8, lo);
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            int cnt = 0;
            for (int s = tid; s < p.NSeq; s += nThreads) {
                cnt += (SeqKeys(p.CtxLens, p.CtxBias, s, p.Window) + mid * 8 - 1) / (mid * 8);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
            }
            PlanSync(); // the previous round's sums have been read
            if ((tid & 31) == 0) {
                red[tid >> 5] = cnt;
            }
            PlanSync();
            cnt = 0;
            for (int w = 0; w < DEC_WARPS; ++w) {
                cnt += red[w];
            }
            if (cnt <= p.TargetCtas) {
                hi = mid;
            } else {
                lo = mid + 1;
            }
        }
        chunk = lo * 8;
    }
    // chunk slots per contiguous slice of sequences, then an exclusive scan over the slices
    const int per = (p.NSeq + nThreads - 1) / nThreads;
    const int s0 = tid * per, s1 = min(s0 + per, p.NSeq);
    int mine = 0;
    for (int s = s0; s < s1; ++s) {
        mine += (SeqKeys(p.CtxLens, p.CtxBias, s, p.Window) + chunk - 1) / chunk;
    }
    sliceBase[tid + 1] = mine;
    if (tid == 0) {
        sliceBase[0] = 0;
        found[0] = -1;
    }
    PlanSync();
    if (tid == 0) {
        for (int i = 1; i <= nThreads; ++i) {
            sliceBase[i] += sliceBase[i - 1];
        }
    }
    PlanSync();
    int base = sliceBase[tid];
    const bool writePlan = blockIdx.x == 0;
    if (writePlan && tid == 0) {
        p.Plan[0] = chunk;
    }
    for (int s = s0; s < s1; ++s) {
        int keys = SeqKeys(p.CtxLens, p.CtxBias, s, p.Window);
        int n = (keys + chunk - 1) / chunk;
        if (writePlan) {
            p.Plan[1 + s] = base;
        }
        if (slot >= base && slot < base + n) {
            int ctxLen = CtxLenOf(p, s);
            int j0, j1;
            KeyRange(ctxLen, p.Window, &j0, &j1);
            found[0] = s;
            found[1] = j0 + (slot - base) * chunk;
            found[2] = min(found[1] + chunk, j1);
        }
        base += n;
    }
    if (writePlan && tid == nThreads - 1) {
        p.Plan[1 + p.NSeq] = sliceBase[nThreads];
    }
    PlanSync();
    *pSeq = found[0];
    *pBeg = found[1];
    *pEnd = found[2];
    return found[0] >= 0;
}

template <bool F16>
struct TScaleOf {
    typedef __half T;
};
template <>
struct TScaleOf<false> {
    typedef float T;
};
__device__ __forceinline__ float LoadScaleT(const __half *p) { return __half2float(__ldg(p)); }
__device__ __forceinline__ float LoadScaleT(const float *p) { return __ldg(p); }
// sum of four (unsigned byte of a) x (signed byte of b) products, plus c
__device__ __forceinline__ int Dp4aUS(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// two 16-bit x 8-bit products added to c: a = (w0 | w1 << 16) unsigned, b bytes signed; lo takes bytes 0 and 1 of b, hi bytes 2 and 3
__device__ __forceinline__ int Dp2aLoUS(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp2a.lo.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int Dp2aHiUS(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp2a.hi.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One CTA = one chunk slot of the balanced plan, four warps, all heads.  Each lane keeps DEC_UNROLL tokens of K and
// V (16 bytes each) in flight; four such CTAs are resident per SM.
// FINAL: every sequence attends so few keys (a short window or short contexts, decided on the host from its bound) that
// one CTA takes a whole sequence: no plan, no partials and no merge kernel -- the CTA adds the sink and writes the
// result (and the inference step's combiner input) itself.
template <int D, int DEC_UNROLL, bool SCALE_F16, bool FINAL>
__global__ void __launch_bounds__(DEC_WARPS * 32, 4) DecodePartialKernel(TDecodeParams p)
{
    constexpr int LPH = D / 16;       // lanes per head
    constexpr int HPW = 32 / LPH;     // heads per warp-wide load
    const int chunk = blockIdx.x;     // chunk slot (FINAL: the sequence)
    int seq, cBeg, cEnd;
    if (FINAL) {
        seq = blockIdx.x;
        const int len = CtxLenOf(p, seq);
        if (len > p.MaxCtx && threadIdx.x == 0 && p.Status) {
            atomicOr(p.Status, kDevBadSpan); // the launch was sized for shorter sequences
        }
        if (len > 0) {
            KeyRange(len, p.Window, &cBeg, &cEnd);
        } else {
            cBeg = cEnd = 0; // no token yet: zeros
        }
    } else if (!DecodePlan(p, chunk, &seq, &cBeg, &cEnd)) {
        return;
    }
    const int ctxLen = CtxLenOf(p, seq);
    const int cur = ctxLen - 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPH;             // 16-byte slice inside the head
    const int H = p.HeadCount;
    const int rowInt4 = H * D / 16;          // int4 words per token row
    const tsa_kv_seq sq = p.Seqs[seq];
    typedef typename TScaleOf<SCALE_F16>::T TScale;

    const int headGroups = (H + HPW - 1) / HPW;
    // With fewer head groups than warps (12 heads x 64: two groups) the spare warps would idle: the warps that share a
    // head group split the chunk's tokens between them instead and merge their partial sums through shared memory.
    __shared__ float mergeBuf[DEC_WARPS][32][18];
    const int split = headGroups == 1 ? 4 : headGroups == 2 ? 2 : 1;
    const int tokenPart = split > 1 ? warp / headGroups : 0;
    const int perPart = (((cEnd - cBeg) + split - 1) / split + 7) & ~7;
    const int tBeg = cBeg + tokenPart * perPart, tEnd = min(tBeg + perPart, cEnd);
    for (int hg = split > 1 ? warp % headGroups : warp; hg < headGroups; hg += DEC_WARPS) {
        const int head = hg * HPW + lane / LPH;
        const bool headOk = head < H;
        const int headC = headOk ? head : H - 1;
        const int colOff = headC * D + sub * 16;
        const int4 qv = *reinterpret_cast<const int4 *>(p.Q.Row(seq) + colOff);
        const float qs = p.QScale.Valid() ? p.QScale.Row(seq)[headC] : p.QVecScale;
        const float logitMult = p.DotScale * qs;
        // running pointers: one add per token instead of a 64-bit multiply
        const int4 *kp = reinterpret_cast<const int4 *>((const int8_t *)sq.k + (size_t)tBeg * H * D + colOff);
        const int4 *vp = reinterpret_cast<const int4 *>((const int8_t *)sq.v + (size_t)tBeg * H * D + colOff);
        const TScale *ksp = (const TScale *)sq.kScale + (size_t)tBeg * H + headC;
        const TScale *vsp = (const TScale *)sq.vScale + (size_t)tBeg * H + headC;

        float m = -1e30f, l = 0;
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            acc[i] = 0;
        }
        for (int tBase = tBeg; tBase < tEnd; tBase += DEC_UNROLL) {
            int4 kv[DEC_UNROLL], vv[DEC_UNROLL];
            float ks[DEC_UNROLL], vs[DEC_UNROLL];
            const int cnt = tEnd - tBase; // tokens left, >= 1
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                const int tt = u < cnt ? u : cnt - 1;
                kv[u] = __ldg(kp + tt * rowInt4);
                vv[u] = __ldg(vp + tt * rowInt4);
                ks[u] = LoadScaleT(ksp + tt * H);
                vs[u] = LoadScaleT(vsp + tt * H);
            }
            kp += DEC_UNROLL * rowInt4;
            vp += DEC_UNROLL * rowInt4;
            ksp += DEC_UNROLL * H;
            vsp += DEC_UNROLL * H;
            float z[DEC_UNROLL];
            float cm = m;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                int dot = __dp4a(qv.x, kv[u].x, 0);
                dot = __dp4a(qv.y, kv[u].y, dot);
                dot = __dp4a(qv.z, kv[u].z, dot);
                dot = __dp4a(qv.w, kv[u].w, dot);
#pragma unroll
                for (int o = LPH / 2; o > 0; o >>= 1) {
                    dot += __shfl_xor_sync(0xffffffffu, dot, o);
                }
                // same association as the reference: ((dot * kScale) * attDotScale) * qScale - slope * dist
                const float zz = (float)dot * ks[u] * logitMult - p.Slope * (float)(cur - (tBase + u));
                z[u] = (u < cnt) ? zz : -1e30f;
                cm = fmaxf(cm, z[u]);
            }
            if (cm != m) {
                const float corr = exp2f(m - cm);
                m = cm;
                l *= corr;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    acc[i] *= corr;
                }
            }
            // weights times value scales of the batch as 16-bit integers relative to the batch maximum (relative error of a
            // weight at most 2^-17 of the largest one), so that the 8 x 16 byte products run as two-token integer dot
            // products (dp2a) instead of a convert and a multiply-add per byte; one float update per batch
            float wv[DEC_UNROLL];
            float bmax = 0;
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; ++u) {
                const float w = exp2f(z[u] - m);
                l += w;
                wv[u] = w * vs[u];
                bmax = fmaxf(bmax, wv[u]);
            }
            const float qScale = bmax > 0 ? 65535.0f / bmax : 0.0f;
            int iacc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                iacc[i] = 0;
            }
#pragma unroll
            for (int u = 0; u < DEC_UNROLL; u += 2) {
                const uint32_t wp = __float2uint_rn(wv[u] * qScale) | (__float2uint_rn(wv[u + 1] * qScale) << 16);
                const uint32_t w0[4] = {(uint32_t)vv[u].x, (uint32_t)vv[u].y, (uint32_t)vv[u].z, (uint32_t)vv[u].w};
                const uint32_t w1[4] = {(uint32_t)vv[u + 1].x, (uint32_t)vv[u + 1].y, (uint32_t)vv[u + 1].z, (uint32_t)vv[u + 1].w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    // bytes (t0 b0, t1 b0, t0 b1, t1 b1) and (t0 b2, t1 b2, t0 b3, t1 b3)
                    const uint32_t lo = __byte_perm(w0[wi], w1[wi], 0x5140);
                    const uint32_t hi = __byte_perm(w0[wi], w1[wi], 0x7362);
                    iacc[wi * 4 + 0] = Dp2aLoUS(wp, lo, iacc[wi * 4 + 0]);
                    iacc[wi * 4 + 1] = Dp2aHiUS(wp, lo, iacc[wi * 4 + 1]);
                    iacc[wi * 4 + 2] = Dp2aLoUS(wp, hi, iacc[wi * 4 + 2]);
                    iacc[wi * 4 + 3] = Dp2aHiUS(wp, hi, iacc[wi * 4 + 3]);
                }
            }
            const float deq = bmax * (1.0f / 65535.0f);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                acc[i] = fmaf((float)iacc[i], deq, acc[i]);
            }
        }
        if (split > 1) {
            float *mine = mergeBuf[warp][lane];
            mine[0] = m;
            mine[1] = l;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                mine[2 + i] = acc[i];
            }
            PlanSync(); // every warp passes here exactly once when the tokens are split
            if (tokenPart == 0) {
                for (int s = 1; s < split; ++s) {
                    const float *other = mergeBuf[warp + s * headGroups][lane];
                    const float mAll = fmaxf(m, other[0]);
                    const float c1 = exp2f(m - mAll), c2 = exp2f(other[0] - mAll);
                    l = l * c1 + other[1] * c2;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        acc[i] = acc[i] * c1 + other[2 + i] * c2;
                    }
                    m = mAll;
                }
            }
        }
        if (FINAL) {
            if (headOk && tokenPart == 0) {
                // the sink has logit 0 (softMax.Add(0), cpu_infer.cpp:444); same arithmetic as the merge kernel with one chunk
                const float mAll = fmaxf(m, 0.0f);
                const float f = exp2f(m - mAll);
                const float lAll = exp2f(-mAll) + f * l;
                const size_t rowSize = (size_t)H * D;
                int4 keyWords = make_int4(0, 0, 0, 0);
                if (p.KvOut) {
                    keyWords = *reinterpret_cast<const int4 *>(p.KvKey + seq * rowSize + head * D + sub * 16);
                }
                const int8_t *key = reinterpret_cast<const int8_t *>(&keyWords);
                int8_t *kv = p.KvOut ? p.KvOut + (seq * rowSize + head * D) * 4 : nullptr;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float res = ctxLen > 0 ? (f * acc[i]) / lAll : 0.0f;
                    const int x = sub * 16 + i;
                    StoreFromFloat(p.Out.Row(seq), head * D + x, p.OutDtype, res);
                    if (kv) {
#pragma unroll
                        for (int blk = 0; blk < 4; ++blk) {
                            // ConvertToInt8 (cpu_infer.cpp:88-92): round to nearest even, clamp to +-127
                            kv[blk * D + x] = (int8_t)max(-127, min(127, __float2int_rn(__fmul_rn((float)key[i ^ blk], res))));
                        }
                    }
                }
            }
        } else if (headOk && tokenPart == 0) {
            float *dst = p.Partial + ((size_t)chunk * H + head) * (D + 4);
            if (sub == 0) {
                dst[D] = m;
                dst[D + 1] = l;
            }
            float4 *d4 = reinterpret_cast<float4 *>(dst + sub * 16);
            d4[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            d4[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
            d4[2] = make_float4(acc[8], acc[9], acc[10], acc[11]);
            d4[3] = make_float4(acc[12], acc[13], acc[14], acc[15]);
        }
    }
}

// merge chunk partials of one (sequence, head): block = D threads
template <int D>
__global__ void __launch_bounds__(D) DecodeCombineKernel(TDecodeParams p)
{
    int seq = blockIdx.y, head = blockIdx.x, x = threadIdx.x;
    int ctxLen = CtxLenOf(p, seq);
    float res = 0;
    if (ctxLen > 0) {
        const int first = p.Plan[1 + seq];
        const int chunks = p.Plan[2 + seq] - first;
        const float *base = p.Partial + ((size_t)first * p.HeadCount + head) * (D + 4);
        size_t cstride = (size_t)p.HeadCount * (D + 4);
        float m = 0; // the sink has logit 0 (softMax.Add(0), cpu_infer.cpp:444)
        for (int c = 0; c < chunks; ++c) {
            m = fmaxf(m, base[c * cstride + D]);
        }
        float l = exp2f(-m);
        float acc = 0;
        for (int c = 0; c < chunks; ++c) {
            float f = exp2f(base[c * cstride + D] - m);
            l += f * base[c * cstride + D + 1];
            acc += f * base[c * cstride + x];
        }
        res = acc / l;
    }
    StoreFromFloat(p.Out.Row(seq), head * D + x, p.OutDtype, res);
    if (p.KvOut) {
        const size_t rowSize = (size_t)p.HeadCount * D;
        const int8_t *key = p.KvKey + seq * rowSize + head * D;
        int8_t *kv = p.KvOut + (seq * rowSize + head * D) * 4;
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
            // ConvertToInt8 (cpu_infer.cpp:88-92): round to nearest even, clamp to +-127
            kv[blk * D + x] = (int8_t)max(-127, min(127, __float2int_rn(__fmul_rn((float)key[x ^ blk], res))));
        }
    }
}

__global__ void KvAppendKernel(const tsa_kv_seq *seqs, int *ctxLens, int nSeq, int capacity, int rowBytes, int headCount, int scaleBytes,
    P2D<int8_t> kNew, P2D<char> kScaleNew, P2D<int8_t> vNew, P2D<char> vScaleNew, int *statusWord)
{
    int seq = blockIdx.x;
    int pos = ctxLens[seq];
    if (pos >= capacity || pos < 0) {
        if (threadIdx.x == 0 && statusWord) {
            atomicOr(statusWord, kDevBadSpan);
        }
        return;
    }
    tsa_kv_seq sq = seqs[seq];
    if ((((uintptr_t)sq.k | (uintptr_t)sq.v) & 15) != 0) {
        // the cache blocks are written 16 bytes at a time: a misaligned base is reported, not stored through
        if (threadIdx.x == 0 && statusWord) {
            atomicOr(statusWord, kDevBadSpan);
        }
        return;
    }
    for (int i = threadIdx.x * 16; i < rowBytes; i += blockDim.x * 16) {
        *reinterpret_cast<int4 *>((int8_t *)sq.k + (size_t)pos * rowBytes + i) = *reinterpret_cast<const int4 *>(kNew.Row(seq) + i);
        *reinterpret_cast<int4 *>((int8_t *)sq.v + (size_t)pos * rowBytes + i) = *reinterpret_cast<const int4 *>(vNew.Row(seq) + i);
    }
    int sb = headCount * scaleBytes;
    for (int i = threadIdx.x; i < sb; i += blockDim.x) {
        ((char *)sq.kScale)[(size_t)pos * sb + i] = kScaleNew.Row(seq)[i];
        ((char *)sq.vScale)[(size_t)pos * sb + i] = vScaleNew.Row(seq)[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        ctxLens[seq] = pos + 1;
    }
}

constexpr int DEC_SINGLE_KEYS = 16;       // up to this many keys per sequence (one batch per warp) one CTA takes the whole sequence; with 64 keys four CTAs and the merge kernel are faster (0.80 against 0.81 ms per inference step)
constexpr int DEC_MAX_TARGET_CTAS = 1024; // workspace is sized for this many chunk slots plus one per sequence

static size_t DecodeHeaderBytes(int nSeq)
{
    return ((size_t)(nSeq + 2) * sizeof(int) + 255) / 256 * 256;
}

size_t DecodeWorkspaceBytes(int headDim, int nSeq, int headCount, int maxCtx)
{
    (void)maxCtx;
    return DecodeHeaderBytes(nSeq) + (size_t)(DEC_MAX_TARGET_CTAS + nSeq) * headCount * (headDim + 4) * sizeof(float);
}

int LaunchDecode(const tsa_decode_cfg *cfg, TDecodeParams p, int maxCtx, cudaStream_t stream, const int8_t *kvKey = nullptr, int8_t *kvOut = nullptr,
    int ctxBias = 0)
{
    p.KvKey = kvKey;
    p.KvOut = kvOut;
    p.CtxBias = ctxBias;
    int dev = 0, sms = 0;
    int rc = CheckCuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc == TSA_OK) {
        rc = CheckCuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
    }
    if (rc != TSA_OK) {
        return rc;
    }
    const bool f16 = cfg->scale_dtype == TSA_F16;
    // at most DEC_SINGLE_KEYS keys per sequence: one CTA per sequence finishes it, no merge kernel
    const long long keysBound = p.Window > 0 ? (p.Window < maxCtx ? p.Window : maxCtx) : 1;
    const bool single = keysBound <= DEC_SINGLE_KEYS;
    const void *kern = nullptr;
    if (cfg->head_dim == 128) {
        kern = single ? (f16 ? (const void *)DecodePartialKernel<128, 8, true, true> : (const void *)DecodePartialKernel<128, 8, false, true>)
                      : (f16 ? (const void *)DecodePartialKernel<128, 8, true, false> : (const void *)DecodePartialKernel<128, 8, false, false>);
    } else {
        kern = single ? (f16 ? (const void *)DecodePartialKernel<64, 8, true, true> : (const void *)DecodePartialKernel<64, 8, false, true>)
                      : (f16 ? (const void *)DecodePartialKernel<64, 8, true, false> : (const void *)DecodePartialKernel<64, 8, false, false>);
    }
    // one full wave of equal chunks: as many chunk slots as CTAs are resident at once
    int perSm = 0;
    rc = CheckCuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kern, DEC_WARPS * 32, 0), "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
    if (rc != TSA_OK) {
        return rc;
    }
    perSm = perSm < 1 ? 1 : perSm;
    p.TargetCtas = sms * perSm < DEC_MAX_TARGET_CTAS ? sms * perSm : DEC_MAX_TARGET_CTAS;
    p.MaxSlots = p.TargetCtas + p.NSeq;
    p.MaxCtx = maxCtx;
    p.Plan = (int *)p.Partial;
    p.Partial = (float *)((char *)p.Partial + DecodeHeaderBytes(p.NSeq));
    // chunks hold at least DEC_MIN_CHUNK keys, so short windows or contexts need fewer CTAs than the full wave
    const long long keysMax = p.Window > 0 ? (p.Window < maxCtx ? p.Window : maxCtx) : 1;
    const long long slotBound = (long long)p.NSeq * (keysMax / DEC_MIN_CHUNK + 1);
    dim3 grid(single ? (unsigned)p.NSeq : (unsigned)(slotBound < p.MaxSlots ? slotBound : p.MaxSlots));
    dim3 gridC(p.HeadCount, p.NSeq);
    void *args[] = {&p};
    rc = CheckCuda(cudaLaunchKernel(kern, grid, dim3(DEC_WARPS * 32), args, 0, stream), "decode launch");
    if (rc != TSA_OK || single) {
        return rc;
    }
    if (cfg->head_dim == 128) {
        DecodeCombineKernel<128><<<gridC, 128, 0, stream>>>(p);
    } else {
        DecodeCombineKernel<64><<<gridC, 64, 0, stream>>>(p);
    }
    return CheckCuda(cudaGetLastError(), "tsa_att_decode launch");
}

} // namespace tsa

using namespace tsa;

static int CheckDecodeCfg(const tsa_decode_cfg *cfg, const char *fn)
{
    TSA_REQUIRE(cfg != nullptr, "%s: null cfg", fn);
    TSA_REQUIRE(cfg->head_dim == 64 || cfg->head_dim == 128, "%s: head_dim %d must be 64 or 128", fn, cfg->head_dim);
    TSA_REQUIRE(cfg->scale_dtype == TSA_F16 || cfg->scale_dtype == TSA_F32, "%s: scale dtype must be f16 or f32", fn);
    TSA_REQUIRE(cfg->out_dtype >= TSA_F16 && cfg->out_dtype <= TSA_F32, "%s: out dtype must be f16, bf16 or f32", fn);
    return TSA_OK;
}

extern "C" __attribute__((visibility("default"))) size_t tsa_att_decode_workspace_bytes(const tsa_decode_cfg *cfg, int nSeq, int headCount, int maxCtx)
{
    if (!cfg || nSeq <= 0 || headCount <= 0 || maxCtx < 0) {
        return 0;
    }
    return DecodeWorkspaceBytes(cfg->head_dim, nSeq, headCount, maxCtx);
}

namespace tsa {
// tsa_att_decode plus the inference step's combiner input written by the merge kernel (kvKey int8 [nSeq][H*D] packed,
// kvOut int8 [nSeq][4*H*D] packed; both null for the plain entry point); ctxBias is added to every ctxLens entry
int DecodeWithKvProduct(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, const int *ctxLens, int nSeq, int maxCtx,
    tsa_ptr2d q, tsa_ptr2d qScale, int window, float alibiSlope, tsa_ptr2d out, int headCount,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream, const int8_t *kvKey, int8_t *kvOut, int ctxBias)
{
    int rc = CheckDecodeCfg(cfg, "tsa_att_decode");
    if (rc != TSA_OK) {
        return rc;
    }
    TSA_REQUIRE(seqs && ctxLens && q.data && out.data, "tsa_att_decode: null buffer");
    TSA_REQUIRE(nSeq >= 0 && headCount > 0 && maxCtx >= 0 && window >= 0, "tsa_att_decode: negative size");
    if (nSeq == 0) {
        return TSA_OK;
    }
    int rowSize = headCount * cfg->head_dim;
    TSA_REQUIRE(q.xsize >= rowSize && q.ysize >= nSeq && out.xsize >= rowSize && out.ysize >= nSeq, "tsa_att_decode: q/out extents");
    TSA_REQUIRE((uintptr_t)q.data % 16 == 0 && q.stride_bytes % 16 == 0, "tsa_att_decode: q must be 16-byte aligned");
    TSA_REQUIRE((uintptr_t)out.data % 16 == 0 && out.stride_bytes % 16 == 0, "tsa_att_decode: out must be 16-byte aligned");
    if (qScale.data) {
        TSA_REQUIRE(qScale.xsize >= headCount && qScale.ysize >= nSeq, "tsa_att_decode: qScale extents");
    }
    size_t need = DecodeWorkspaceBytes(cfg->head_dim, nSeq, headCount, maxCtx);
    TSA_REQUIRE(workspace && workspaceBytes >= need, "tsa_att_decode: workspace of %zu bytes needed, %zu given", need, workspaceBytes);
    TSA_REQUIRE((uintptr_t)workspace % 16 == 0, "tsa_att_decode: workspace must be 16-byte aligned");
    TDecodeParams p;
    p.Status = statusWord;
    p.Seqs = seqs;
    p.CtxLens = ctxLens;
    p.NSeq = nSeq;
    p.HeadCount = headCount;
    p.Window = window;
    p.ScaleDtype = cfg->scale_dtype;
    p.OutDtype = cfg->out_dtype;
    p.Slope = alibiSlope;
    p.DotScale = HostAttDotScale(cfg->head_dim);
    p.QVecScale = cfg->qk_vec_scale;
    p.Q = P2D<int8_t>(q);
    p.QScale = P2D<float>(qScale);
    p.Out = P2D<char>(out);
    p.Partial = (float *)workspace;
    return LaunchDecode(cfg, p, maxCtx, (cudaStream_t)stream, kvKey, kvOut, ctxBias);
}
} // namespace tsa

extern "C" __attribute__((visibility("default"))) int tsa_att_decode(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, const int *ctxLens, int nSeq, int maxCtx,
    tsa_ptr2d q, tsa_ptr2d qScale, int window, float alibiSlope, tsa_ptr2d out, int headCount,
    void *workspace, size_t workspaceBytes, int *statusWord, tsa_stream_t stream)
{
    return DecodeWithKvProduct(cfg, seqs, ctxLens, nSeq, maxCtx, q, qScale, window, alibiSlope, out, headCount, workspace, workspaceBytes, statusWord, stream,
        nullptr, nullptr, 0);
}

extern "C" __attribute__((visibility("default"))) int tsa_kv_append(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, int *ctxLens, int nSeq, int capacity,
    tsa_ptr2d kNew, tsa_ptr2d kScaleNew, tsa_ptr2d vNew, tsa_ptr2d vScaleNew, int headCount,
    int *statusWord, tsa_stream_t stream)
{
    int rc = CheckDecodeCfg(cfg, "tsa_kv_append");
    if (rc != TSA_OK) {
        return rc;
    }
    TSA_REQUIRE(seqs && ctxLens && kNew.data && vNew.data && kScaleNew.data && vScaleNew.data, "tsa_kv_append: null buffer");
    if (nSeq <= 0) {
        return nSeq == 0 ? TSA_OK : Fail(TSA_BAD_ARG, "tsa_kv_append: negative nSeq");
    }
    TSA_REQUIRE(headCount > 0 && capacity > 0, "tsa_kv_append: headCount %d / capacity %d must be positive", headCount, capacity);
    int rowBytes = headCount * cfg->head_dim;
    TSA_REQUIRE(rowBytes % 16 == 0, "tsa_kv_append: H * D = %d must be a multiple of 16 (rows are copied 16 bytes at a time)", rowBytes);
    TSA_REQUIRE(kNew.xsize >= rowBytes && vNew.xsize >= rowBytes && kNew.ysize >= nSeq && vNew.ysize >= nSeq, "tsa_kv_append: kNew/vNew extents");
    TSA_REQUIRE(kScaleNew.xsize >= headCount && vScaleNew.xsize >= headCount && kScaleNew.ysize >= nSeq && vScaleNew.ysize >= nSeq,
        "tsa_kv_append: kScaleNew/vScaleNew must be [nSeq][H]");
    TSA_REQUIRE((uintptr_t)kNew.data % 16 == 0 && kNew.stride_bytes % 16 == 0 && (uintptr_t)vNew.data % 16 == 0 && vNew.stride_bytes % 16 == 0,
        "tsa_kv_append: kNew/vNew must be 16-byte aligned");
    KvAppendKernel<<<nSeq, 128, 0, (cudaStream_t)stream>>>(seqs, ctxLens, nSeq, capacity, rowBytes, headCount, DtypeSize(cfg->scale_dtype),
        P2D<int8_t>(kNew), P2D<char>(kScaleNew), P2D<int8_t>(vNew), P2D<char>(vScaleNew), statusWord);
    return CheckCuda(cudaGetLastError(), "tsa_kv_append launch");
}

// ---- decode without any allocation -------------------------------------------------------------------
// Some hosts cannot hand this library a scratch buffer at call time: TScale's own runtime carves all device
// memory out of pools when a context is created and afterwards only replays a fixed list of kernel launches
// (code/lib/cuda/cuda_graph.cuh:131-349, cuda_memory.h), and a serving loop that already owns the whole
// memory budget has nothing left to ask cudaMalloc for (which would also stall the device while it runs).
// For them the chunk partials of the decode live in this fixed array inside the library image; every GPU
// that loads the library keeps these 32 MiB until the process exits.
constexpr size_t kStaticScratchBytes = (size_t)32 << 20;
static __device__ __align__(256) unsigned char g_decodeScratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratchLock;
void *g_scratchAddr[kMaxDevices]; // device address of g_decodeScratch, per device, filled on first use

// The array's name is only a host-side handle; the address a kernel can use has to be asked for, on the
// device that is current, once per device.  The answer is kept for the life of the process: after a cudaDeviceReset
// the module is loaded afresh and the kept address is stale, so a process that resets a device must not call
// tsa_att_decode_static on it again.
int StaticScratchAddress(void **out)
{
    int dev = -1;
    int rc = tsa::CheckCuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc != TSA_OK) {
        return rc;
    }
    if (dev < 0 || dev >= kMaxDevices) {
        return tsa::Fail(TSA_UNSUPPORTED, "tsa_att_decode_static: device index %d not supported", dev);
    }
    std::lock_guard<std::mutex> guard(g_scratchLock);
    if (!g_scratchAddr[dev]) {
        void *ptr = nullptr;
        rc = tsa::CheckCuda(cudaGetSymbolAddress((void **)&ptr, g_decodeScratch), "cudaGetSymbolAddress(decode scratch)");
        if (rc != TSA_OK) {
            return rc;
        }
        g_scratchAddr[dev] = ptr;
    }
    *out = g_scratchAddr[dev];
    return TSA_OK;
}
} // namespace

extern "C" __attribute__((visibility("default"))) size_t tsa_att_decode_static_capacity_bytes(void)
{
    return kStaticScratchBytes;
}

extern "C" __attribute__((visibility("default"))) int tsa_att_decode_static(const tsa_decode_cfg *cfg, const tsa_kv_seq *seqs, const int *ctxLens, int nSeq, int maxCtx,
    tsa_ptr2d q, tsa_ptr2d qScale, int window, float alibiSlope, tsa_ptr2d out, int headCount,
    int *statusWord, tsa_stream_t stream)
{
    // only the size check and the address look-up are this entry point's own; validation and launch are tsa_att_decode's
    TSA_REQUIRE(cfg != nullptr && (cfg->head_dim == 64 || cfg->head_dim == 128), "tsa_att_decode_static: head_dim must be 64 or 128");
    TSA_REQUIRE(nSeq >= 0 && headCount > 0 && maxCtx >= 0, "tsa_att_decode_static: negative size");
    if (nSeq == 0) {
        return TSA_OK;
    }
    size_t need = DecodeWorkspaceBytes(cfg->head_dim, nSeq, headCount, maxCtx);
    if (need > kStaticScratchBytes) {
        return Fail(TSA_UNSUPPORTED,
            "tsa_att_decode_static: nSeq %d x maxCtx %d x %d heads needs %zu bytes of chunk partials, the built-in scratch holds %zu; "
            "use tsa_att_decode with a caller workspace",
            nSeq, maxCtx, headCount, need, kStaticScratchBytes);
    }
    void *scratch = nullptr;
    int rc = StaticScratchAddress(&scratch);
    if (rc != TSA_OK) {
        return rc;
    }
    return DecodeWithKvProduct(cfg, seqs, ctxLens, nSeq, maxCtx, q, qScale, window, alibiSlope, out, headCount, scratch, kStaticScratchBytes,
        statusWord, stream, nullptr, nullptr, 0);
}
